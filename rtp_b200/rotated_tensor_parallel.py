"""Automatic wrapper: ``RotatedTensorParallel(model)`` shards and rotates every ``nn.Linear``, ``nn.Conv2d``,
``nn.Embedding`` and ``nn.MultiheadAttention`` of an arbitrary model; everything else stays replicated
(reference: rtp/rotated_tensor_parallel.py:296-571).

``FlyweightWarpper`` (the reference's spelling) rotates the parameters of one already-sharded module:
its ``.module`` is the local shard, so state_dict keys are ``<path>.module.weight`` / ``.bias`` as in the
reference.  Unlike the reference, the rotating attention wrapper is really installed in the parent module,
and ``inplace=True`` produces correct gradients.
"""
from typing import Any, List, Optional

import torch
import torch.nn as nn

from .attention import ParallelMultiheadAttention
from .parallel.context import get_context
from .parallel.flat import RotatedModule
from .parallel.rotated import rotated_apply


def split_tensor(tensor: torch.Tensor, num_partitions: int, partition_dim: int = 0) -> List[torch.Tensor]:
    """Equal split of ``tensor`` along ``partition_dim`` (must divide)."""
    size = tensor.size(partition_dim)
    if size % num_partitions != 0:
        raise ValueError(f"dimension {partition_dim} of size {size} is not divisible by {num_partitions}")
    return list(torch.split(tensor, size // num_partitions, dim=partition_dim))


class FlyweightWarpper(RotatedModule):
    """Rotates all parameters of ``module`` (the local shard) around the ring.

    Modes (as in the reference's forward, lines 360-417):
      * default: outputs of the N visiting shards are concatenated along ``output_partition_dim``;
      * ``row_partition=True``: the input is split along ``input_partition_dim``, shard j sees block j, outputs are summed;
      * ``cat_output=False``: every shard sees the whole input, outputs are summed (attention heads).
    """

    def __init__(self, module: nn.Module, group: Optional[Any] = None, param_list=None, flat_param_names=None,
                 partition_dim=None, output_partition_dim=None, row_partition=False, input_partition_dim=None,
                 cat_output=True, inplace=False):
        super().__init__()
        self._setup_ring(group)
        self.module = module
        self.inplace = inplace
        self.partition_dim = partition_dim
        self.output_partition_dim = -1 if output_partition_dim is None else output_partition_dim
        self.input_partition_dim = -1 if input_partition_dim is None else input_partition_dim
        self.row_partition = row_partition
        self.cat_output = cat_output
        self._pnames = [n for n, _ in module.named_parameters()]
        self._shard_rules = {}
        self._flatten()

    def shard_parameters(self):
        return [p for _, p in self.module.named_parameters()]

    def shard_names(self):
        return list(self._pnames)

    def shard_spec(self):
        return {f"module.{k}": v for k, v in self._shard_rules.items()}

    @property
    def flat_param(self):
        return self._full_param

    @property
    def module_list(self):
        return [self.module] * self.world_size

    def _forward_fused(self, args, kwargs):
        """The wrapped shard on the fused sm_100a kernels (bf16 CUDA tensors, shapes the kernels can take); returns
        NotImplemented when the functional engine has to run it."""
        from .parallel import fused
        mod, N = self.module, self.world_size
        flat = self._full_param
        if not flat.is_cuda:
            return NotImplemented
        from .parallel import engine as E
        if isinstance(mod, nn.Linear):
            if len(args) != 1 or kwargs or not isinstance(args[0], torch.Tensor) or not fused.use_fused(args[0], flat):
                return NotImplemented
            row = self.row_partition
            in_f = mod.in_features * N if row else mod.in_features
            out_f = mod.out_features if row else mod.out_features * N
            if not E.fused_linear_ok(row, in_f, out_f, N):
                return NotImplemented
            spec = E.linear_spec(self, row, in_f, out_f, mod.weight, mod.bias)
            params = [p for p in (mod.weight, mod.bias) if p is not None]
            spec.recompute = getattr(args[0], "_rtp_recompute", None)
            return E._FusedSubLinearFn.apply(spec, args[0], *params)
        if isinstance(mod, nn.Embedding):
            if len(args) != 1 or kwargs or not fused.use_fused(flat, flat):
                return NotImplemented
            if mod.padding_idx is not None or mod.max_norm is not None or mod.scale_grad_by_freq or mod.sparse \
                    or mod.embedding_dim % 8:
                return NotImplemented
            return E.fused_embedding(self, args[0], mod.weight, mod.embedding_dim * N)
        if isinstance(mod, nn.Conv2d):
            if len(args) != 1 or kwargs or not isinstance(args[0], torch.Tensor) or not fused.use_fused(args[0], flat):
                return NotImplemented
            if (self.inplace and N > 1) or not E.fused_conv_ok(mod, args[0]):
                return NotImplemented
            return E.fused_conv(self, mod, args[0])
        if isinstance(mod, ParallelMultiheadAttention):
            if len(args) < 3:
                return NotImplemented
            query, key, value = args[:3]
            names = ("key_padding_mask", "need_weights", "attn_mask", "average_attn_weights", "is_causal")
            kw = dict(zip(names, args[3:]))
            kw.update(kwargs)
            if set(kw) - set(names):
                return NotImplemented
            need_w = kw.get("need_weights", True)
            if not E.mha_fused_ok(self, mod, query, key, value, kw.get("key_padding_mask"), need_w, kw.get("attn_mask"),
                                  self.training):
                return NotImplemented
            return E.fused_mha(self, mod, query, is_causal=kw.get("is_causal", False), attn_mask=kw.get("attn_mask"),
                               key_padding_mask=kw.get("key_padding_mask"), need_weights=need_w,
                               average_attn_weights=kw.get("average_attn_weights", True), training=self.training)
        return NotImplemented

    def forward(self, *args, **kwargs):
        out = self._forward_fused(args, kwargs)
        if out is not NotImplemented:
            return out
        names, mod = self._pnames, self.module
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        tpos = [i for i, a in enumerate(args) if isinstance(a, torch.Tensor)]
        ipd, row = self.input_partition_dim, self.row_partition
        N = self.world_size

        def fn(j, views, *tens):
            call_args = list(args)
            for pos, t in zip(tpos, tens):
                call_args[pos] = t
            if row:
                x = call_args[0]
                size = x.size(ipd) // N
                call_args[0] = x.narrow(ipd, j * size, size)
            return torch.func.functional_call(mod, dict(zip(names, views)), tuple(call_args), kwargs)

        combine = "sum" if (row or not self.cat_output) else "cat"
        stochastic = self.training and any(isinstance(m, nn.Dropout) and m.p > 0 for m in mod.modules()) \
            or (self.training and getattr(mod, "dropout", 0) and isinstance(getattr(mod, "dropout"), float))
        return rotated_apply(self.ring, fn, self.shard_parameters(), self._full_param, self._layout, tensors,
                             combine=combine, cat_dim=self.output_partition_dim, inplace=self.inplace,
                             stochastic=bool(stochastic), owner=self)


class RotatedTensorParallel(nn.Module):
    """Wrap ``module`` so that all its weight matrices are sharded 1/N and rotated.

    Sharding rules (reference lines 454-529): Linear by output rows when ``out % N == 0``, else by input
    columns when ``in % N == 0`` (bias stored as ``b/N``), else ``ValueError``; Conv2d by output channels;
    Embedding by embedding dim; MultiheadAttention by heads.  The wrapped model must hold identical weights on
    every rank before wrapping (each rank keeps its own slice).
    """

    def __init__(self, module: nn.Module, group: Optional[Any] = None, inplace: bool = False):
        super().__init__()
        ctx = get_context(group)
        self.ring, self.rank, self.world_size = ctx, ctx.rank, ctx.world
        self.inplace = inplace
        self.FlyweightModule_list: List[FlyweightWarpper] = []
        self.module = self._visit(module)

    @property
    def group(self):
        return self.ring.group

    # -- recursive replacement ---------------------------------------------------------------
    def _wrap(self, shard, rules, **kw):
        fw = FlyweightWarpper(shard, group=self.ring.group, inplace=self.inplace, **kw)
        fw._shard_rules = rules
        self.FlyweightModule_list.append(fw)
        return fw

    def _visit(self, m: nn.Module) -> nn.Module:
        N, r = self.world_size, self.rank
        if isinstance(m, nn.MultiheadAttention):
            return self._convert_mha(m)
        if isinstance(m, nn.Linear):
            has_b = m.bias is not None
            if m.out_features % N == 0:
                s = nn.Linear(m.in_features, m.out_features // N, bias=has_b, device=m.weight.device, dtype=m.weight.dtype)
                with torch.no_grad():
                    s.weight.copy_(split_tensor(m.weight, N, 0)[r])
                    if has_b:
                        s.bias.copy_(split_tensor(m.bias, N, 0)[r])
                rules = {"weight": ("split", 0), **({"bias": ("split", 0)} if has_b else {})}
                return self._wrap(s, rules, partition_dim=0)
            if m.in_features % N == 0:
                s = nn.Linear(m.in_features // N, m.out_features, bias=has_b, device=m.weight.device, dtype=m.weight.dtype)
                with torch.no_grad():
                    s.weight.copy_(split_tensor(m.weight, N, 1)[r])
                    if has_b:
                        s.bias.copy_(m.bias / N)
                if has_b:
                    s.bias.rtp_sum_replicated = N
                rules = {"weight": ("split", 1), **({"bias": ("sum",)} if has_b else {})}
                return self._wrap(s, rules, partition_dim=1, row_partition=True, input_partition_dim=-1)
            raise ValueError(f"nn.Linear({m.in_features}, {m.out_features}) cannot be split over {N} ranks")
        if isinstance(m, nn.Conv2d):
            if m.out_channels % N != 0:
                raise ValueError(f"nn.Conv2d with {m.out_channels} output channels cannot be split over {N} ranks")
            has_b = m.bias is not None
            s = nn.Conv2d(m.in_channels, m.out_channels // N, m.kernel_size, m.stride, m.padding, m.dilation,
                          m.groups, has_b, m.padding_mode, device=m.weight.device, dtype=m.weight.dtype)
            with torch.no_grad():
                s.weight.copy_(split_tensor(m.weight, N, 0)[r])
                if has_b:
                    s.bias.copy_(split_tensor(m.bias, N, 0)[r])
            rules = {"weight": ("split", 0), **({"bias": ("split", 0)} if has_b else {})}
            return self._wrap(s, rules, partition_dim=0, output_partition_dim=1)
        if isinstance(m, nn.Embedding):
            if m.embedding_dim % N != 0:
                raise ValueError(f"nn.Embedding with dim {m.embedding_dim} cannot be split over {N} ranks")
            s = nn.Embedding(m.num_embeddings, m.embedding_dim // N, padding_idx=m.padding_idx, max_norm=m.max_norm,
                             norm_type=m.norm_type, scale_grad_by_freq=m.scale_grad_by_freq,
                             device=m.weight.device, dtype=m.weight.dtype)
            with torch.no_grad():
                s.weight.copy_(split_tensor(m.weight, N, 1)[r])
            return self._wrap(s, {"weight": ("split", 1)}, partition_dim=1)
        for name, child in list(m.named_children()):
            new = self._visit(child)
            if new is not child:
                setattr(m, name, new)
        return m

    def _convert_mha(self, m: nn.MultiheadAttention) -> nn.Module:
        s = ParallelMultiheadAttention(m.embed_dim, m.num_heads, dropout=m.dropout, bias=m.in_proj_bias is not None,
                                       add_bias_kv=m.bias_k is not None, add_zero_attn=m.add_zero_attn, kdim=m.kdim,
                                       vdim=m.vdim, batch_first=m.batch_first, device=m.out_proj.weight.device,
                                       dtype=m.out_proj.weight.dtype, group=self.ring.group)
        s.affine_weight(m)
        kinds = {"in_proj_weight": ("qkv", 0), "in_proj_bias": ("qkv", 0), "q_proj_weight": ("split", 0),
                 "k_proj_weight": ("split", 0), "v_proj_weight": ("split", 0), "out_proj.weight": ("split", 1),
                 "out_proj.bias": ("sum",), "bias_k": ("split", 2), "bias_v": ("split", 2)}
        rules = {n: kinds[n] for n, _ in s.named_parameters()}
        return self._wrap(s, rules, cat_output=False)

    # -- nn.Module API -----------------------------------------------------------------------
    def forward(self, *args: Any, **kwargs: Any) -> Any:
        return self.module(*args, **kwargs)

    def cuda(self, device=None):
        return super().cuda(device)   # flat buffers are rebuilt by each FlyweightWarpper._apply
