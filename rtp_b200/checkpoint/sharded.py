"""Sharded checkpoints.

The per-rank ``state_dict`` of a rotated model has the reference's keys and shapes (only the local shard
is a registered parameter).  The reference saves rank 0's shard only (rtp_mnist.py:161-166) and cannot
resume; here every rank writes ``rank{r}-of-{N}.pt`` (model shard, optimizer shard state, step, RNG) next
to a JSON manifest, and the shards can be consolidated into full tensors or re-sharded for another ring
size offline.
"""
import json
import os
import re
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from ..parallel.context import get_context
from ..parallel.flat import RotatedModule


def sharding_plan(model: torch.nn.Module) -> Dict[str, Tuple]:
    """Map state_dict key -> rule for every tensor that is sharded: ("split", dim), ("qkv", dim),
    ("sum",) for biases stored as b/N, ("expert", L) for whole local experts. Other keys are replicated."""
    plan = {}
    for path, mod in model.named_modules(remove_duplicate=False):
        if isinstance(mod, RotatedModule):
            for k, rule in mod.shard_spec().items():
                plan[f"{path}.{k}" if path else k] = tuple(rule)
    return plan


def _shard_tensor(full: torch.Tensor, rule: Tuple, rank: int, world: int) -> torch.Tensor:
    kind = rule[0]
    if kind == "split":
        return torch.chunk(full, world, dim=rule[1])[rank].clone()
    if kind in ("qkv", "packed"):
        parts = 3 if kind == "qkv" else rule[2]
        blocks = torch.chunk(full, parts * world, dim=rule[1])
        return torch.cat([blocks[rank + k * world] for k in range(parts)], dim=rule[1])
    if kind == "sum":
        return full / world
    raise ValueError(kind)


def _unshard_tensors(shards: List[torch.Tensor], rule: Tuple) -> torch.Tensor:
    kind, world = rule[0], len(shards)
    if kind == "split":
        return torch.cat(shards, dim=rule[1])
    if kind in ("qkv", "packed"):
        n = 3 if kind == "qkv" else rule[2]
        parts = [torch.chunk(s, n, dim=rule[1]) for s in shards]
        return torch.cat([parts[r][k] for k in range(n) for r in range(world)], dim=rule[1])
    if kind == "sum":
        return shards[0] * world
    raise ValueError(kind)


_EXPERT_RE = re.compile(r"^(.*\.experts\.)(\d+)(\..*)$")


def consolidate(rank_state_dicts: List[Dict[str, torch.Tensor]], plan: Dict[str, Tuple]) -> Dict[str, torch.Tensor]:
    """Full (unsharded) tensors under the same keys; local expert ``e`` of rank ``r`` becomes global expert
    ``r*L + e``."""
    world = len(rank_state_dicts)
    out = {}
    for k, v in rank_state_dicts[0].items():
        rule = plan.get(k)
        if rule is None:
            out[k] = v.clone()
        elif rule[0] == "expert":
            L = rule[1]
            m = _EXPERT_RE.match(k)
            for r in range(world):
                out[f"{m.group(1)}{r * L + int(m.group(2))}{m.group(3)}"] = rank_state_dicts[r][k].clone()
        else:
            out[k] = _unshard_tensors([sd[k] for sd in rank_state_dicts], rule)
    return out


def shard_full(full_sd: Dict[str, torch.Tensor], plan: Dict[str, Tuple], rank: int, world: int
               ) -> Dict[str, torch.Tensor]:
    """Rank ``rank``'s state_dict of a ``world``-rank ring from consolidated tensors. ``plan`` must come from a
    model built for ``world`` ranks (expert rules carry the number of local experts)."""
    out = {}
    expert_rules = {k: r for k, r in plan.items() if r[0] == "expert"}
    for k, v in full_sd.items():
        m = _EXPERT_RE.match(k)
        if m and any(p.startswith(m.group(1)) for p in expert_rules):
            L = next(r[1] for p, r in expert_rules.items() if p.startswith(m.group(1)))
            g = int(m.group(2))
            if g // L == rank:
                out[f"{m.group(1)}{g % L}{m.group(3)}"] = v.clone()
            continue
        rule = plan.get(k)
        out[k] = v.clone() if rule is None else _shard_tensor(v, rule, rank, world)
    return out


def reshard(rank_state_dicts: List[Dict[str, torch.Tensor]], old_plan, new_plan, new_world: int):
    """N -> N' re-sharding: consolidate, then shard again."""
    full = consolidate(rank_state_dicts, old_plan)
    return [shard_full(full, new_plan, r, new_world) for r in range(new_world)]


def plain_lm_to_rtp_keys(plain_sd: Dict[str, torch.Tensor], n_layers_total: int) -> Dict[str, torch.Tensor]:
    """Rename the keys of the unsharded ``transformer_lm_fsdp.TransformerLM`` to those of the rotated LM."""
    out = {}
    last = n_layers_total - 1
    for k, v in plain_sd.items():
        idx, rest = k.split(".", 1)
        i = int(idx)
        if i == 0 and rest == "weight":
            nk = "0.embedding.embedding.weight"
        elif i == last and rest in ("weight", "bias"):
            nk = f"{i}.linear.linear.{rest}"
        elif rest.startswith("self_attn."):
            nk = f"{i}.self_attn.MultiheadAttention.{rest[len('self_attn.'):]}"
        elif rest.startswith("ff_block.linear"):
            a, b, c = rest.split(".")
            nk = f"{i}.ff_block.{b}.linear.{c}"
        else:
            nk = k
        out[nk] = v
    # the MoE gate is registered twice in the rotated model (layer.gate and layer.moe_layer.gate)
    for k in list(out):
        if ".moe_layer.gate." in k:
            out[k.replace(".moe_layer.gate.", ".gate.")] = out[k]
        elif re.search(r"^\d+\.gate\.", k):
            out[k.replace(".gate.", ".moe_layer.gate.", 1)] = out[k]
    return out


def shard_state_dict(plain_sd, rtp_model, rank: int, world: int):
    """state_dict for ``rtp_model`` (a rotated TransformerLM) from the unsharded plain LM's state_dict."""
    full = plain_lm_to_rtp_keys(plain_sd, len(rtp_model))
    sd = shard_full(full, sharding_plan(rtp_model), rank, world)
    return {k: v for k, v in sd.items() if k in rtp_model.state_dict()}


def save_sharded(directory: str, model, optimizer=None, step: int = 0, extra=None, group=None):
    """Every rank writes its shard; rank 0 also writes ``manifest.json``."""
    ctx = get_context(group)
    os.makedirs(directory, exist_ok=True)
    for m in model.modules():
        if isinstance(m, RotatedModule):
            m.assert_home()
    payload = {"model": model.state_dict(), "step": step, "extra": extra,
               "rng_cpu": torch.get_rng_state(),
               "rng_cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None}
    if optimizer is not None:
        # a FusedLMTrainer plays the optimizer's part too: its state_dict holds the Adam moments and both step counters
        payload["optimizer"] = optimizer.state_dict()
        payload["optimizer_step"] = getattr(optimizer, "_step", None)
    path = os.path.join(directory, f"rank{ctx.rank}-of-{ctx.world}.pt")
    torch.save(payload, path + ".tmp")
    os.replace(path + ".tmp", path)
    if ctx.rank == 0:
        plan = sharding_plan(model)
        manifest = {"world_size": ctx.world, "step": step, "format": "rtp-sharded-v1",
                    "plan": {k: list(v) for k, v in plan.items()},
                    "dtype": str(next(model.parameters()).dtype)}
        with open(os.path.join(directory, "manifest.json"), "w") as f:
            json.dump(manifest, f, indent=1)
    if ctx.world > 1:
        dist.barrier(group=ctx.group)
    return path


def load_sharded(directory: str, model, optimizer=None, group=None, restore_rng: bool = True) -> int:
    """Load this rank's shard (re-sharding on the fly when the checkpoint was written by another ring size).
    Returns the saved step."""
    ctx = get_context(group)
    with open(os.path.join(directory, "manifest.json")) as f:
        manifest = json.load(f)
    old_world = manifest["world_size"]
    if old_world == ctx.world:
        payload = torch.load(os.path.join(directory, f"rank{ctx.rank}-of-{ctx.world}.pt"), map_location="cpu",
                             weights_only=False)
        model.load_state_dict(payload["model"])
        if optimizer is not None and "optimizer" in payload:
            optimizer.load_state_dict(payload["optimizer"])
            if payload.get("optimizer_step") is not None and hasattr(optimizer, "_step"):
                optimizer._step = payload["optimizer_step"]
                optimizer._step_dev = None
        if restore_rng:
            torch.set_rng_state(payload["rng_cpu"])
            if payload.get("rng_cuda") is not None and torch.cuda.is_available():
                states = payload["rng_cuda"]
                if len(states) != torch.cuda.device_count():
                    # saved on a machine with another number of visible devices: restore this process's device only
                    dev = torch.cuda.current_device()
                    torch.cuda.set_rng_state(states[min(dev, len(states) - 1)], dev)
                else:
                    torch.cuda.set_rng_state_all(states)
        return payload["step"]
    # different ring size: weights only (optimizer state restarts)
    sds = [torch.load(os.path.join(directory, f"rank{r}-of-{old_world}.pt"), map_location="cpu",
                      weights_only=False)["model"] for r in range(old_world)]
    old_plan = {k: tuple(v) for k, v in manifest["plan"].items()}
    full = consolidate(sds, old_plan)
    model.load_state_dict(shard_full(full, sharding_plan(model), ctx.rank, ctx.world))
    return manifest["step"]
