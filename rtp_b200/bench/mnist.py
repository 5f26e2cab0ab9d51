"""MNIST-style CNN example with the automatic wrapper (reference: rtp_mnist.py, benchmarks/rtp_mnist.py, and the
DDP / FSDP twins).  ``--mode rtp`` wraps the net with ``RotatedTensorParallel``; ``--mode rtp_modules`` builds it
from rotated layers by hand; ``dp`` / ``fsdp`` are the stock PyTorch baselines.  Without the dataset on disk
(``--data``), synthetic 28x28 images with learnable labels are used.

    python -m rtp_b200.bench.mnist --gpus 2 --epochs 1 --mode rtp
"""
import argparse
import os
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
import torch.nn.functional as F


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 32, 3, 1)
        self.conv2 = nn.Conv2d(32, 64, 3, 1)
        self.dropout1 = nn.Dropout(0.25)
        self.dropout2 = nn.Dropout(0.5)
        self.fc1 = nn.Linear(9216, 128)
        self.fc2 = nn.Linear(128, 10)

    def forward(self, x):
        x = F.relu(self.conv1(x))
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        x = torch.flatten(self.dropout1(x), 1)
        x = self.dropout2(F.relu(self.fc1(x)))
        return F.log_softmax(self.fc2(x), dim=1)


class RotatedNet(Net):
    """The same network assembled from rotated layers (reference: benchmarks/rtp_mnist.py:42-66)."""

    def __init__(self):
        nn.Module.__init__(self)
        from ..module.conv import ColumnParallelConv2d
        from ..module.linear import ColumnParallelLinear, RowParallelLinear
        world = dist.get_world_size() if dist.is_initialized() else 1
        self.conv1 = ColumnParallelConv2d(1, 32, 3, 1)
        self.conv2 = ColumnParallelConv2d(32, 64, 3, 1)
        self.dropout1 = nn.Dropout(0.25)
        self.dropout2 = nn.Dropout(0.5)
        self.fc1 = ColumnParallelLinear(9216, 128)
        self.fc2 = ColumnParallelLinear(128, 10) if 10 % world == 0 else RowParallelLinear(128, 10)


def synthetic_mnist(n, seed):
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, 10, (n,), generator=g)
    x = torch.randn(n, 1, 28, 28, generator=g) * 0.3
    for c in range(10):                      # a class-dependent blob so that the task is learnable
        x[y == c, 0, 2 * c:2 * c + 6, 2 * c:2 * c + 6] += 1.5
    return x, y


def load_data(args, rank, world):
    n_train, n_test = args.train_samples, args.test_samples
    if args.data and os.path.isdir(args.data):
        try:
            from torchvision import datasets, transforms
            tf = transforms.Compose([transforms.ToTensor(), transforms.Normalize((0.1307,), (0.3081,))])
            tr = datasets.MNIST(args.data, train=True, download=False, transform=tf)
            te = datasets.MNIST(args.data, train=False, download=False, transform=tf)
            xtr = torch.stack([tr[i][0] for i in range(min(n_train, len(tr)))])
            ytr = torch.tensor([tr[i][1] for i in range(min(n_train, len(tr)))])
            xte = torch.stack([te[i][0] for i in range(min(n_test, len(te)))])
            yte = torch.tensor([te[i][1] for i in range(min(n_test, len(te)))])
            return (xtr, ytr), (xte, yte)
        except Exception:
            pass
    return synthetic_mnist(n_train, 0), synthetic_mnist(n_test, 1)


def worker(rank, world, args, port):
    from ..optim import ShardedAdam
    from ..rotated_tensor_parallel import RotatedTensorParallel
    use_cuda = torch.cuda.is_available()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = str(port)
    if use_cuda:
        torch.cuda.set_device(rank)
    dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world)
    device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    torch.manual_seed(args.seed)
    (xtr, ytr), (xte, yte) = load_data(args, rank, world)
    rotated = args.mode in ("rtp", "rtp_inplace", "rtp_modules")
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    if args.mode == "rtp_modules":
        model = RotatedNet().to(device, dtype)
    else:
        model = Net().to(device, dtype)
        if args.mode in ("rtp", "rtp_inplace"):
            model = RotatedTensorParallel(model, inplace=args.mode == "rtp_inplace")
        elif args.mode == "dp" and world > 1:
            model = nn.parallel.DistributedDataParallel(model, device_ids=[rank] if use_cuda else None)
        elif args.mode == "fsdp" and world > 1:
            from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
            model = FSDP(model)
    opt = ShardedAdam(model.parameters(), lr=args.lr) if rotated else torch.optim.Adam(model.parameters(), lr=args.lr)
    per = args.batch_size
    t0 = time.time()
    for epoch in range(1, args.epochs + 1):
        model.train()
        perm = torch.randperm(xtr.size(0), generator=torch.Generator().manual_seed(epoch))
        tot = torch.zeros(2, device=device)
        for i in range(0, xtr.size(0) - per * world + 1, per * world):
            idx = perm[i + rank * per:i + (rank + 1) * per]
            x, y = xtr[idx].to(device, dtype), ytr[idx].to(device)
            opt.zero_grad()
            loss = F.nll_loss(model(x).float(), y, reduction="sum")
            # rotated layers SUM gradients over the ring: scale the loss like the reference (rtp_mnist.py:78)
            (loss / (per * world) if rotated else loss / per).backward()
            opt.step()
            tot += torch.tensor([loss.item(), float(per)], device=device)
        dist.all_reduce(tot)
        model.eval()
        correct = torch.zeros(2, device=device)
        with torch.no_grad():
            for i in range(rank * per, xte.size(0) - per + 1, per * world):
                x, y = xte[i:i + per].to(device, dtype), yte[i:i + per].to(device)
                correct += torch.tensor([(model(x).argmax(1) == y).sum().item(), float(per)], device=device)
        dist.all_reduce(correct)
        if rank == 0:
            print("Train Epoch: {} \tLoss: {:.6f} \tTest accuracy: {:.2f}%".format(
                epoch, (tot[0] / tot[1]).item(), 100.0 * (correct[0] / correct[1]).item()), flush=True)
    if use_cuda:
        torch.cuda.synchronize()
    if rank == 0:
        print(f"elapsed {time.time() - t0:.2f}s; peak allocated "
              f"{(torch.cuda.max_memory_allocated() / 2**20 if use_cuda else 0):.1f} MB")
    if args.save_model:
        from ..checkpoint import save_sharded
        save_sharded(args.save_model, model, opt, step=args.epochs)       # every rank writes its shard
    dist.barrier()
    dist.destroy_process_group()


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--batch-size", dest="batch_size", type=int, default=64)
    p.add_argument("--epochs", type=int, default=2)
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--seed", type=int, default=1)
    p.add_argument("--mode", default="rtp", choices=["rtp", "rtp_inplace", "rtp_modules", "dp", "fsdp"])
    p.add_argument("--gpus", type=int, default=None)
    p.add_argument("--data", default=None)
    p.add_argument("--train-samples", dest="train_samples", type=int, default=2048)
    p.add_argument("--test-samples", dest="test_samples", type=int, default=512)
    p.add_argument("--save-model", dest="save_model", default=None)
    p.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"],
                   help="bf16 on CUDA puts the rotated layers on the fused sm_100a kernels (fp32 uses the functional engine)")
    args = p.parse_args(argv)
    world = args.gpus or (torch.cuda.device_count() if torch.cuda.is_available() else 1)
    port = 12355 + os.getpid() % 1000
    if world == 1:
        worker(0, 1, args, port)
    else:
        mp.spawn(worker, args=(world, args, port), nprocs=world, join=True)


if __name__ == "__main__":
    main()
