"""Command-line flags of the LM benchmark: the reference's names and defaults (benchmarks/config.py:6-35) plus the
execution mode, dtype and model family."""
import argparse


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="rtp_b200 language-model benchmark")
    p.add_argument("--max_batch", type=int, default=4, help="Max number of batches")
    p.add_argument("--use_synthetic_data", action="store_true", default=True)
    p.add_argument("--dry_run", action="store_true")
    p.add_argument("--model_name", default="lm")
    p.add_argument("--debug", action="store_true")
    p.add_argument("--enable_auto_wrap", action="store_true")
    p.add_argument("--benchmark_eval", action="store_true")
    p.add_argument("--full_fp16", action="store_true", help="bf16 parameters and activations")
    p.add_argument("--vocab_size", type=int, default=10240)
    p.add_argument("--ninp", type=int, default=2048)
    p.add_argument("--nhid", type=int, default=2048)
    p.add_argument("--nhead", type=int, default=32)
    p.add_argument("--dropout", type=float, default=0)
    p.add_argument("--initrange", type=float, default=0.1)
    p.add_argument("--clip_value", type=float, default=0.05)
    p.add_argument("--num_decoder_layers", type=int, default=5)
    p.add_argument("--seq_len", type=int, default=128)
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--lr", type=float, default=0.001)
    p.add_argument("--batch_size", type=int, default=1)
    # additions
    p.add_argument("--mode", default="rtp", choices=["rtp", "rtp_inplace", "nccl_rtp", "dp", "fsdp", "tp"],
                   help="rtp: fused sm_100a rotation; rtp_inplace: in-place modules; nccl_rtp: functional ring "
                        "(torch.distributed send/recv); dp/fsdp/tp: baselines")
    p.add_argument("--dtype", default=None, choices=[None, "fp32", "bf16"])
    p.add_argument("--model", default="lm", choices=["lm", "gpt", "llama", "moe"])
    p.add_argument("--is_moe", action="store_true")
    p.add_argument("--num_local_experts", type=int, default=1)
    p.add_argument("--gpus", type=int, default=None, help="ranks to spawn (default: all visible GPUs, or 1 on CPU)")
    p.add_argument("--backend", default=None, choices=[None, "nccl", "gloo"])
    p.add_argument("--metrics_jsonl", default=None)
    p.add_argument("--checkpoint_dir", default=None, help="write a sharded checkpoint at the end")
    p.add_argument("--resume", default=None, help="resume from a sharded checkpoint directory")
    return p.parse_args(argv)
