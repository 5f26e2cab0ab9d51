"""Language-model training benchmark with the reference's flags (benchmarks/rtp_benchmark.py, dp_/fsdp_/tp_
variants are ``--mode``).  Prints ``| batch | wps | loss | ppl`` lines, throughput (tokens/s per rank and per box,
device-timed, max over ranks) and peak allocated GiB per rank.

    python -m rtp_b200.bench.lm_benchmark --full_fp16 --num_decoder_layers 10 --seq_len 32 --batch_size 32 \\
        --dropout 0.1 --max_batch 20 --mode rtp
"""
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from .config import parse_args
from ..utils.data import SyntheticLM
from ..utils.metrics import MetricsLogger, peak_memory_gib
from ..utils.timing import max_over_ranks


def build_model(args, rank, world, device, dtype):
    kw = dict(ntokens=args.vocab_size, ninp=args.ninp, nhead=args.nhead, nhid=args.nhid, dropout=args.dropout,
              initrange=args.initrange, ndecoder=args.num_decoder_layers)
    if args.mode in ("rtp", "nccl_rtp"):
        from ..models.transformer_lm_rtp import TransformerLM
        model = TransformerLM(**kw, world_size=world, rank=rank, is_moe=args.is_moe,
                              num_local_experts=args.num_local_experts)
    elif args.mode == "rtp_inplace":
        from ..inplace.models.transformer_lm_rtp_inplace import TransformerLM
        model = TransformerLM(**kw, world_size=world, rank=rank, is_moe=args.is_moe,
                              num_local_experts=args.num_local_experts)
    elif args.mode == "tp":
        from ..models.transformer_lm_tp import TransformerLM
        model = TransformerLM(**kw, world_size=world, rank=rank)
    else:
        from ..models.transformer_lm_fsdp import TransformerLM
        model = TransformerLM(**kw, is_moe=args.is_moe, num_local_experts=args.num_local_experts)
    model = model.to(device=device, dtype=dtype)
    if args.mode == "dp" and world > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[device.index] if device.type == "cuda" else None)
    elif args.mode == "fsdp" and world > 1:
        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
        model = FSDP(model)
    return model


def train(args, rank, world, device, dtype):
    from ..optim import ShardedAdam
    from ..parallel.context import set_backend
    log = MetricsLogger(args.metrics_jsonl, rank)
    model = build_model(args, rank, world, device, dtype)
    fused = args.mode == "rtp" and device.type == "cuda" and dtype == torch.bfloat16 and not args.is_moe \
        and args.ninp // args.nhead == 64 and args.seq_len <= 96
    if args.mode == "nccl_rtp":
        set_backend("functional")
    sum_grads = args.mode in ("rtp", "rtp_inplace", "nccl_rtp")    # rotated layers sum gradients over the ring
    data = SyntheticLM(args.vocab_size, args.seq_len, args.batch_size, n_batches=args.max_batch + 1,
                       rank=0 if args.mode == "tp" else rank, pin=device.type == "cuda")
    if fused:
        from ..models.fused_lm import FusedLMTrainer
        trainer = FusedLMTrainer(model, lr=args.lr, clip_value=args.clip_value)
    else:
        if sum_grads:
            opt = ShardedAdam(model.parameters(), lr=args.lr, clip_value=args.clip_value)
        else:
            opt = torch.optim.Adam(model.parameters(), lr=args.lr)
    start_step = 0
    if args.resume:
        from ..checkpoint import load_sharded
        # the fused trainer plays the optimizer's part: its state_dict carries the Adam moments and the step counters
        start_step = load_sharded(args.resume, model, trainer if fused else opt)
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    tokens, t_ms, e0 = 0, 0.0, None
    loss_val = float("nan")
    for i, (x, y) in enumerate(data):
        if i > args.max_batch:
            break
        if i == 1 and device.type == "cuda":          # batch 0 is warm-up, as in the reference
            torch.cuda.synchronize()
            e0 = torch.cuda.Event(enable_timing=True)
            e0.record()
            t_host = time.time()
        if i == 1 and device.type != "cuda":
            t_host = time.time()
        if fused:
            loss = trainer.step(x, y)
        else:
            x, y = x.to(device, non_blocking=True), y.to(device, non_blocking=True)
            model.train()
            opt.zero_grad()
            out = model(x)
            loss = F.cross_entropy(out.reshape(-1, args.vocab_size).float(), y.reshape(-1))
            (loss / world if sum_grads else loss).backward()
            if not sum_grads:
                torch.nn.utils.clip_grad_value_(model.parameters(), args.clip_value)
            opt.step()
        if i >= 1:
            tokens += x.numel()
        loss_val = float(loss.item())
        if i >= 1:
            el = (time.time() - t_host)
            log.batch(i, tokens / max(el, 1e-9), loss_val)
    if device.type == "cuda":
        e1 = torch.cuda.Event(enable_timing=True)
        e1.record()
        torch.cuda.synchronize()
        t_ms = e0.elapsed_time(e1) if e0 is not None else 0.0
    else:
        t_ms = (time.time() - t_host) * 1e3
    t_ms = max_over_ranks(t_ms)
    if fused:
        trainer.check()
    wps_rank = tokens / (t_ms / 1e3) if t_ms > 0 else 0.0
    peak = peak_memory_gib(device) if device.type == "cuda" else 0.0
    if args.checkpoint_dir:
        from ..checkpoint import save_sharded
        save_sharded(args.checkpoint_dir, model, trainer if fused else opt, step=start_step + args.max_batch)
    log.summary(mode=args.mode, world=world, tokens_per_s_per_rank=wps_rank, tokens_per_s_box=wps_rank * world,
                ms_per_step=t_ms / max(args.max_batch, 1), peak_allocated_gib=peak, final_loss=loss_val)
    if rank == 0:
        print("Throughput(wps) is {:.2f} per rank, {:.2f} per box.".format(wps_rank, wps_rank * world))
    print("Peak allocated bytes on cuda:{}: {:1f}GiB".format(rank, peak))
    return wps_rank


def worker(rank, world, args, port):
    use_cuda = torch.cuda.is_available()
    backend = args.backend or ("nccl" if use_cuda else "gloo")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = str(port)
    if use_cuda:
        torch.cuda.set_device(rank)
    dist.init_process_group(backend, rank=rank, world_size=world)
    torch.manual_seed(0)
    device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, None: torch.bfloat16 if args.full_fp16 else torch.float32}[args.dtype]
    try:
        train(args, rank, world, device, dtype)
    finally:
        dist.barrier()
        dist.destroy_process_group()


def main(argv=None):
    args = parse_args(argv)
    world = args.gpus or (torch.cuda.device_count() if torch.cuda.is_available() else 1)
    if args.dry_run:
        print(vars(args))
        return
    port = 29501 + os.getpid() % 1000
    if world == 1:
        worker(0, 1, args, port)
    else:
        mp.spawn(worker, args=(world, args, port), nprocs=world, join=True)


if __name__ == "__main__":
    main(sys.argv[1:])
