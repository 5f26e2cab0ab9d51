"""Sharding helpers with the reference's names and semantics (rtp/module/utils.py:19-103)."""
from typing import List, Optional, Sequence

import torch


def ensure_divisibility(numerator: int, denominator: int) -> None:
    if numerator % denominator != 0:
        raise AssertionError(f"{numerator} is not divisible by {denominator}")


def divide_and_check_no_remainder(numerator: int, denominator: int) -> int:
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


divide = divide_and_check_no_remainder


def split_tensor_along_last_dim(tensor: torch.Tensor, num_partitions: int,
                                contiguous_split_chunks: bool = False):
    size = divide(tensor.size(-1), num_partitions)
    parts = torch.split(tensor, size, dim=tensor.dim() - 1)
    if contiguous_split_chunks:
        return tuple(p.contiguous() for p in parts)
    return parts


def affine_weight(weight: torch.Tensor, master_weight: torch.Tensor, per_partition_size: int,
                  partition_dim: int, world_size: int, rank: int, stride: int = 1) -> Optional[torch.Tensor]:
    """Copy rank ``rank``'s block of ``master_weight`` (split along ``partition_dim``) into ``weight``."""
    size = divide_and_check_no_remainder(per_partition_size, stride)
    blocks = torch.split(master_weight, size, dim=partition_dim)
    with torch.no_grad():
        weight.copy_(blocks[rank])
    return None


def affine_weight_attention(weight: torch.Tensor, master_weight: torch.Tensor, index: Sequence[int],
                            per_partition_size: int, partition_dim: int, world_size: int, rank: int,
                            stride: int = 1) -> Optional[torch.Tensor]:
    """Copy the concatenation of blocks ``index`` (e.g. ``[r, r+N, r+2N]`` = this rank's q, k and v rows
    of a packed in-projection) into ``weight``."""
    size = divide_and_check_no_remainder(per_partition_size, stride)
    blocks = torch.split(master_weight, size, dim=partition_dim)
    with torch.no_grad():
        weight.copy_(torch.cat([blocks[i] for i in index], dim=partition_dim))
    return None


def qkv_block_index(rank: int, world_size: int) -> List[int]:
    """Blocks of a 3N-way row split of a packed in-projection that belong to ``rank``."""
    return [rank, rank + world_size, rank + 2 * world_size]
