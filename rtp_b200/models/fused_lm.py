"""Fused training step of the rotated ``TransformerLM`` on sm_100a.

``FusedLMTrainer`` drives one full step (forward, loss, backward, gradient sync of the replicated
LayerNorm parameters, Adam) of a ``rtp_b200.models.transformer_lm_rtp.TransformerLM`` whose parameters
are bf16 CUDA tensors, entirely with the library's own kernels:

* every linear (QKV, out-projection, both FFN matrices, LM head) is one launch of the rotation GEMM
  kernel per direction: tcgen05 tiles, bias/ReLU/dropout in the epilogue, shards pushed to the peers
  over NVLink from inside the kernel, weight gradients reduced around the ring in the wgrad epilogue;
* embedding (+ sqrt(D) scale, positional encoding, dropout), dropout+residual+LayerNorm, causal
  attention, softmax cross-entropy and the multi-tensor Adam update are the memory-bound kernels of
  ``csrc/kernels.cu``;
* dropout masks are regenerated from (seed, per-op offset, device step counter), never stored;
* the whole step is captured once in a CUDA graph and replayed.

The math is the model's: post-LN decoder layers ``x = LN1(x + drop(MHA(x)))``, ``x = LN2(x + FF(x))``,
``FF = drop(lin2(drop(relu(lin1(x)))))`` (reference: rtp/models/transformer_lm_rtp.py:77-89,171-179).
"""
import math
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops import _lib
from ..parallel import engine as E
from ..parallel.context import get_context
from ..utils.timing import nvtx_range


class _Lin:
    """Launch descriptor of one rotated linear: flat shard, layout info and persistent gradient buffer."""

    def __init__(self, module, row, in_f, out_f, flat=None, layout_info=None, params=None):
        self.module, self.row, self.in_f, self.out_f = module, row, in_f, out_f
        self.flat = flat
        self.info = layout_info
        self.gflat = None     # set by the trainer: a buffer of its own, or a window of the shared gradient scratch
        self.plan = None      # Adam plan of this layer alone (optimizer-in-backward mode)
        self.params = params  # [(param, offset, numel, lr_mult)]


class FusedLMTrainer:
    def __init__(self, model, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adamw=False,
                 clip_value: Optional[float] = None, loss_scale: Optional[float] = None, use_graph: bool = True,
                 seed: int = 1234, group=None, state_dtype=None, keep_grads: Optional[bool] = True):
        """``state_dtype``: Adam moment policy, ``None`` / ``"fp32"`` (default), ``"mixed"`` or ``"bf16"``
        (see ``rtp_b200.ops.kernels.adam_state_dtypes``).

        ``keep_grads=True``: every parameter's ``.grad`` holds its gradient after ``step`` and Adam runs once at the end.
        ``keep_grads=False`` (optimizer in backward): the gradients of one decoder layer (or of the head, or of the
        embedding) land in ONE shared scratch buffer and that group's Adam update runs right after its last backward
        launch, so only one group's gradient is alive at a time (the gradients are 1/4 to 1/6 of the per-rank model
        state); ``.grad`` is not meaningful afterwards.
        Both modes apply the same updates.  ``keep_grads=None`` picks by size: a model whose per-rank share is under half a
        billion parameters keeps its gradients (one Adam launch per step instead of one per layer: such a step is bound by
        launches, not memory), a larger one updates in backward."""
        self.model = model
        if keep_grads is None:
            keep_grads = sum(p.numel() for p in model.parameters()) < 500_000_000
        self.keep_grads = keep_grads
        self.state_dtypes = K.adam_state_dtypes(state_dtype)
        self.ring = get_context(group)
        self.N = self.ring.world
        cfg = model.config
        self.V, self.D, self.H, self.heads, self.L = cfg["ntokens"], cfg["ninp"], cfg["nhid"], cfg["nhead"], cfg["ndecoder"]
        if cfg["is_moe"]:
            raise NotImplementedError("the fused trainer covers the dense LM; MoE layers run through the module path")
        if self.D // self.heads != 64:
            raise NotImplementedError("fused attention kernel needs head_dim 64")
        self.p_drop = float(cfg["dropout"])
        self.lr, self.betas, self.eps, self.wd, self.adamw = lr, betas, eps, weight_decay, adamw
        self.clip = clip_value or 0.0
        self.loss_scale = loss_scale if loss_scale is not None else 1.0 / self.N
        self.use_graph = use_graph
        self.seed = seed
        p0 = next(model.parameters())
        if not (p0.is_cuda and p0.dtype == torch.bfloat16):
            raise ValueError("FusedLMTrainer needs a bf16 CUDA model")
        self.dev = p0.device
        self.eng = E.get_engine(self.ring)
        self._build_descriptors()
        # weight shards of the next rotated linear travel while the current one computes (RTP_PREFETCH=0: every launch
        # pushes its own shards at its start)
        self.prefetch = self.N > 1 and os.environ.get("RTP_PREFETCH", "1") != "0"
        self._build_chain()
        self._ci = 0
        self._graph = None
        self._static = None
        self.step_dev = torch.zeros(1, dtype=torch.int64, device=self.dev)       # Adam step
        self.rng_step = torch.zeros(1, dtype=torch.int64, device=self.dev)       # dropout step counter
        self.launches_per_step = 0
        self._counting = False
        self._calls = 0

    # ------------------------------------------------------------------------------------------
    def _lin_desc(self, rot_module, row):
        lay = rot_module._layout
        has_bias = "bias" in lay.names
        info = (has_bias, lay.offset_of("bias") if has_bias else -1, E._round_up(lay.numel * 2, 16))
        params = []
        for n, p in zip(lay.names, rot_module.shard_parameters()):
            mult = 1.0 / getattr(p, "rtp_sum_replicated") if getattr(p, "rtp_sum_replicated", None) else 1.0
            params.append((p, lay.offset_of(n), p.numel(), mult))
        return _Lin(rot_module, row, rot_module.in_features, rot_module.out_features, rot_module._full_param, info,
                    params)

    def _build_descriptors(self):
        m, N, D = self.model, self.N, self.D
        self.emb = m[0].embedding            # ParallelEmbedding
        self.pe = m[1].pe.view(-1, D).to(torch.bfloat16).contiguous()
        self.layers = []
        for li in range(self.L):
            layer = m[2 + li]
            mha = layer.self_attn
            lay = mha._layout
            Es = D // N
            # the MHA shard [in_proj_weight, in_proj_bias, out_proj.weight, out_proj.bias] is rotated as two
            # linears: a column-rotated packed QKV projection and a row-rotated output projection
            names = lay.names
            assert names == ["in_proj_weight", "in_proj_bias", "out_proj.weight", "out_proj.bias"], names
            flat = mha._full_param
            o_inw, o_inb = lay.offset_of("in_proj_weight"), lay.offset_of("in_proj_bias")
            o_ow, o_ob = lay.offset_of("out_proj.weight"), lay.offset_of("out_proj.bias")
            qkv_flat = flat[o_inw:o_ow]
            out_flat = flat[o_ow:]
            sub = mha.MultiheadAttention
            qkv = _Lin(mha, False, D, 3 * D, qkv_flat, (True, o_inb - o_inw, E._round_up(qkv_flat.numel() * 2, 16)),
                       [(sub.in_proj_weight, 0, sub.in_proj_weight.numel(), 1.0),
                        (sub.in_proj_bias, o_inb - o_inw, sub.in_proj_bias.numel(), 1.0)])
            outp = _Lin(mha, True, D, D, out_flat, (True, o_ob - o_ow, E._round_up(out_flat.numel() * 2, 16)),
                        [(sub.out_proj.weight, 0, sub.out_proj.weight.numel(), 1.0),
                         (sub.out_proj.bias, o_ob - o_ow, sub.out_proj.bias.numel(), 1.0 / N)])
            ff1 = self._lin_desc(layer.ff_block.linear1, False)
            ff2 = self._lin_desc(layer.ff_block.linear2, False)
            self.layers.append(dict(qkv=qkv, out=outp, ff1=ff1, ff2=ff2, n1=layer.norm1, n2=layer.norm2,
                                    eps=layer.norm1.eps))
        self.head = self._lin_desc(m[2 + self.L].linear, False)
        E.reserve_shard_bytes(max(x.info[2] for l in self.layers for x in (l["qkv"], l["out"], l["ff1"], l["ff2"])))
        # replicated LayerNorm parameters: fp32 gradient bucket (all-reduced over the ring) + bf16 copy for Adam
        self.ln_params = []
        for l in self.layers:
            self.ln_params += [l["n1"].weight, l["n1"].bias, l["n2"].weight, l["n2"].bias]
        self.ln_grad32 = torch.zeros(len(self.ln_params) * D, dtype=torch.float32, device=self.dev)
        self.ln_grad16 = torch.zeros(len(self.ln_params) * D, dtype=torch.bfloat16, device=self.dev)
        # gradient buffers: one per layer, or windows of one scratch as large as the largest shard
        lins = [l[k] for l in self.layers for k in ("qkv", "out", "ff1", "ff2")] + [self.head]
        if self.keep_grads:
            for d in lins:
                d.gflat = torch.zeros_like(d.flat)
            self.emb_gflat = torch.zeros_like(self.emb._full_param)
        else:
            # update groups in backward order: the head, then each decoder layer (its four linears side by side in the
            # scratch, one Adam launch after the layer's last backward), then the embedding
            groups = [[self.head]] + [[l[k] for k in ("ff2", "ff1", "out", "qkv")] for l in reversed(self.layers)]
            offs, nmax = {}, self.emb._full_param.numel()
            for grp in groups:
                o = 0
                for d in grp:
                    offs[id(d)] = o
                    o += E._round_up(d.flat.numel(), 64)
                nmax = max(nmax, o)
            self.gscratch = torch.zeros(nmax, dtype=torch.bfloat16, device=self.dev)
            for d in lins:
                d.gflat = self.gscratch[offs[id(d)]:offs[id(d)] + d.flat.numel()]
            self.emb_gflat = self.gscratch[:self.emb._full_param.numel()]
        # Adam plans over views of the flat buffers: one for everything, or one per layer
        entries = []

        def entry(p, g):
            m1 = torch.zeros_like(p, dtype=self.state_dtypes[0])
            m2 = torch.zeros_like(p, dtype=self.state_dtypes[1])
            mult = 1.0 / getattr(p, "rtp_sum_replicated") if getattr(p, "rtp_sum_replicated", None) else 1.0
            e = (p.data, g, m1, m2, mult)
            entries.append(e)
            if self.keep_grads:
                p.grad = g
            return e

        emb_e = [entry(self.emb.embedding.weight, self.emb._layout.views(self.emb_gflat)[0])]
        per_lin = []
        for d in lins:
            per_lin.append([entry(p, d.gflat[off:off + n].view(p.shape)) for p, off, n, mult in d.params])
        ln_e = [entry(p, self.ln_grad16[k * D:(k + 1) * D]) for k, p in enumerate(self.ln_params)]
        self.adam_entries = entries
        by_ptr = {p.data_ptr(): n for n, p in self.model.named_parameters()}
        self._entry_names = {e[0].data_ptr(): by_ptr[e[0].data_ptr()] for e in entries}
        if self.keep_grads:
            self.plan = K.AdamPlan(entries, self.dev)
        else:
            self.plan = None
            self.emb_plan = K.AdamPlan(emb_e, self.dev)
            self.ln_plan = K.AdamPlan(ln_e, self.dev)
            by_lin = {id(d): es for d, es in zip(lins, per_lin)}
            for grp in groups:
                for d in grp:
                    d.plan = None
                grp[-1].plan = K.AdamPlan([e for d in grp for e in by_lin[id(d)]], self.dev)

    def _adam(self, plan):
        plan.step(self.step_dev, self.lr, self.betas[0], self.betas[1], self.eps, self.wd, self.adamw, self.clip)
        self._count(1)

    # ------------------------------------------------------------------------------------------
    def _alloc_static(self, S, B):
        M, D, H, V, dev = S * B, self.D, self.H, self.V, self.dev
        bf = torch.bfloat16
        st = dict(S=S, B=B, M=M)
        st["ids"] = torch.zeros(S, B, dtype=torch.int64, device=dev)
        st["tgt"] = torch.zeros(S, B, dtype=torch.int64, device=dev)
        st["x0"] = torch.empty(M, D, dtype=bf, device=dev)
        acts = []
        # all bf16 activations come out of one arena, so that memory of layers whose backward has run can be lent out
        sizes = dict(qkv=3 * D, ctx=D, h1=D, x1=D, a1=H, h2=D, x2=D)
        per_layer = M * sum(sizes.values())
        arena = torch.empty(self.L * per_layer, dtype=bf, device=dev)
        for li in range(self.L):
            slab = arena[li * per_layer:(li + 1) * per_layer]
            a, off = {}, 0
            for name, w in sizes.items():
                a[name] = slab[off:off + M * w].view(M, w)
                off += M * w
            for name in ("mean1", "rstd1", "mean2", "rstd2"):
                a[name] = torch.empty(M, dtype=torch.float32, device=dev)
            acts.append(a)
        st["acts"] = acts
        # outputs of the out-projection and of the second FFN linear are consumed by the residual + norm kernel at once
        # and never read in backward: one buffer each serves every layer
        st["sa"] = torch.empty(M, D, dtype=bf, device=dev)
        st["f"] = torch.empty(M, D, dtype=bf, device=dev)
        st["logits"] = torch.empty(M, V, dtype=bf, device=dev)
        st["loss_rows"] = torch.empty(M, dtype=torch.float32, device=dev)
        st["loss"] = torch.zeros(1, dtype=torch.float32, device=dev)
        # backward scratch (reused by every layer)
        st["dxa"] = torch.empty(M, D, dtype=bf, device=dev)
        st["dxb"] = torch.empty(M, D, dtype=bf, device=dev)
        st["dsub"] = torch.empty(M, D, dtype=bf, device=dev)
        st["dz1"] = torch.empty(M, H, dtype=bf, device=dev)
        st["dctx"] = torch.empty(M, D, dtype=bf, device=dev)
        st["dqkv"] = torch.empty(M, 3 * D, dtype=bf, device=dev)
        st["dbias"] = torch.empty(max(3 * D, V, H), dtype=torch.float32, device=dev)
        if self.N > 1:
            # Block-major scatter buffer of the embedding gradient ([N, V, D/N]).  It is only alive after the backward of
            # every layer, so it lives on top of the (by then dead) activations.
            need = V * D
            buf = arena[:need] if arena.numel() >= need else torch.empty(need, dtype=bf, device=dev)
            st["emb_dense"] = buf.view(self.N, V, D // self.N)
        return st

    # ------------------------------------------------------------------------------------------
    def _embed_fwd(self, st):
        N, D = self.N, self.D
        Ds = D // N
        tab = self.emb.embedding.weight
        if N == 1:
            K.embed_fwd(tab, st["ids"].view(-1), st["x0"], 0, D=D, scale=math.sqrt(D), pe=self.pe,
                        tokens_per_pos=st["B"], drop_p=self.p_drop, seed=self.seed, offset=1, step=self.rng_step)
            self._count(1)
        else:
            E.embed_fwd_rot(self.eng, self.emb._full_param, tab.shape[0], Ds, st["ids"].view(-1), st["x0"], D,
                            math.sqrt(D), self.pe, st["B"], self.p_drop, self.seed, 1, self.rng_step)
            self._count(1)

    def _embed_bwd(self, st, dx0):
        N, D = self.N, self.D
        tab_g = self.emb._layout.views(self.emb_gflat)[0]
        if N == 1:
            self.emb_gflat.zero_()
            K.embed_bwd(tab_g, st["ids"].view(-1), dx0, 0, D=D, scale=math.sqrt(D), drop_p=self.p_drop,
                        seed=self.seed, offset=1, step=self.rng_step)
            self._count(2)
        else:
            E.embed_bwd_rot(self.eng, self, st, dx0)
            self._count(3)
        if not self.keep_grads:
            self._adam(self.emb_plan)

    def _count(self, n):
        if self._counting:
            self.launches_per_step += n

    def _chain_args(self, d, kind):
        """Cross-launch prefetch: the rotated linears of a step form one chain (forward order, then backward order).  Each
        launch reads its visiting shards from one weight-slot bank, where the previous launch of the chain pushed them,
        and pushes the shards of the next launch into the other bank while it computes."""
        if not self.prefetch:
            return {}
        k = self._ci
        self._ci += 1
        assert self._chain[k] == (id(d), kind), "the chain of rotated linears changed between steps"
        nxt = self._chain_desc[k + 1] if k + 1 < len(self._chain_desc) else None
        return dict(bank=k & 1, pushed=k > 0, next_flat=nxt[0].flat if nxt else None, next_kind=nxt[1] if nxt else 0)

    def _build_chain(self):
        fwd = [l[n] for l in self.layers for n in ("qkv", "out", "ff1", "ff2")] + [self.head]
        bwd = [self.head] + [l[n] for l in reversed(self.layers) for n in ("ff2", "ff1", "out", "qkv")]
        self._chain_desc = [(d, 0) for d in fwd] + [(d, 1) for d in bwd]
        self._chain = [(id(d), k) for d, k in self._chain_desc]

    def _lin_fwd(self, d, x, out, act=0, drop_p=0.0, offset=0):
        E.linear_fwd_raw(self.eng, d.flat, d.info, x, d.row, d.in_f, d.out_f, act=act, drop_p=drop_p, seed=self.seed,
                         offset=offset, out=out, step=self.rng_step, **self._chain_args(d, 0))
        self._count(1)

    def _lin_bwd(self, d, x, dy, st, dx_out=None, need_dx=True, mask=None, mask_scale=1.0, dx_accumulate=False):
        dbuf = st["dbias"][: d.out_f]
        n0 = _lib.launches
        E.linear_bwd_raw(self.eng, d.flat, d.info, x, dy, d.row, d.in_f, d.out_f, need_dx=need_dx, mask=mask,
                         mask_scale=mask_scale, grad_out=d.gflat, dx_out=dx_out, dx_accumulate=dx_accumulate,
                         dbias_buf=dbuf, **self._chain_args(d, 1))
        self._count(_lib.launches - n0)  # fused dgrad/wgrad program (+ column sums of dy where they are a kernel of their own)
        if not self.keep_grads and d.plan is not None:
            # The shards of a decoder layer (or the head) are updated as soon as the group's last gradient is complete.
            # Their home buffers are no longer read by anyone in this step: the pushes of them (by their own launches or
            # the ones before) precede the update in stream order.
            self._adam(d.plan)

    def _step_impl(self, st):
        S, B, M, D, L = st["S"], st["B"], st["M"], self.D, self.L
        p = self.p_drop
        rs = self.rng_step
        self._ci = 0
        # ---------------- forward
        self._embed_fwd(st)
        x = st["x0"]
        for li, (l, a) in enumerate(zip(self.layers, st["acts"])):
            with nvtx_range(f"forward layer {li}"):
                o = 16 * (li + 1)
                self._lin_fwd(l["qkv"], x, a["qkv"])
                K.attn_small_fwd(a["qkv"], S, B, self.heads, nshard=self.N, causal=True, drop_p=p, seed=self.seed,
                                 offset=o + 1, step=rs, out=a["ctx"])
                self._lin_fwd(l["out"], a["ctx"], st["sa"])
                K.norm_fwd(x, st["sa"], l["n1"].weight, l["n1"].bias, eps=l["eps"], drop_p=p, seed=self.seed, offset=o + 2,
                           step=rs, out=a["x1"], h_out=a["h1"], mean_out=a["mean1"], rstd_out=a["rstd1"])
                self._lin_fwd(l["ff1"], a["x1"], a["a1"], act=1, drop_p=p, offset=o + 3)
                self._lin_fwd(l["ff2"], a["a1"], st["f"])
                K.norm_fwd(a["x1"], st["f"], l["n2"].weight, l["n2"].bias, eps=l["eps"], drop_p=p, seed=self.seed,
                           offset=o + 4, step=rs, out=a["x2"], h_out=a["h2"], mean_out=a["mean2"], rstd_out=a["rstd2"])
                self._count(3)
                x = a["x2"]
        with nvtx_range("head + cross-entropy"):
            self._lin_fwd(self.head, x, st["logits"])
            K_scale = self.loss_scale / M
            rows = K.cross_entropy_into(st["logits"], st["tgt"].view(-1), st["loss_rows"], grad_scale=K_scale)
            K.sum_f32(rows, st["loss"], scale=1.0 / M)
            self._count(2)
        # ---------------- backward
        self.ln_grad32.zero_()
        self.step_dev.add_(1)          # the Adam step of this iteration (the updates may run inside backward)
        self._count(1)
        dx = st["dxa"]
        self._lin_bwd(self.head, x, st["logits"], st, dx_out=dx)
        scale_keep = 1.0 / (1.0 - p) if p > 0 else 1.0
        for li in reversed(range(L)):
            with nvtx_range(f"backward layer {li}"):
                l, a = self.layers[li], st["acts"][li]
                o = 16 * (li + 1)
                xin = st["acts"][li - 1]["x2"] if li > 0 else st["x0"]
                g = self.ln_grad32
                k0 = 4 * li * D
                # LN2: dx (grad of x2) -> dh2 (= grad of x1 via the residual) and df (through dropout)
                dx1 = st["dxb"]
                K.norm_bwd(dx, a["h2"], l["n2"].weight, a["mean2"], a["rstd2"], drop_p=p, seed=self.seed, offset=o + 4,
                           step=rs, dgamma=g[k0 + 2 * D:k0 + 3 * D], dbeta=g[k0 + 3 * D:k0 + 4 * D], dx=dx1, dsub=st["dsub"])
                # FFN2 backward; the ReLU+dropout backward of the hidden activation rides in its dgrad epilogue
                self._lin_bwd(l["ff2"], a["a1"], st["dsub"], st, dx_out=st["dz1"], mask=a["a1"], mask_scale=scale_keep)
                # FFN1 backward accumulates onto the residual gradient
                self._lin_bwd(l["ff1"], a["x1"], st["dz1"], st, dx_out=dx1, dx_accumulate=True)
                # LN1
                dxin = dx  # reuse: dx is dead after LN2 backward
                K.norm_bwd(dx1, a["h1"], l["n1"].weight, a["mean1"], a["rstd1"], drop_p=p, seed=self.seed, offset=o + 2,
                           step=rs, dgamma=g[k0:k0 + D], dbeta=g[k0 + D:k0 + 2 * D], dx=dxin, dsub=st["dsub"])
                self._lin_bwd(l["out"], a["ctx"], st["dsub"], st, dx_out=st["dctx"])
                K.attn_small_bwd(a["qkv"], st["dctx"], S, B, self.heads, nshard=self.N, causal=True, drop_p=p,
                                 seed=self.seed, offset=o + 1, step=rs, out=st["dqkv"])
                self._lin_bwd(l["qkv"], xin, st["dqkv"], st, dx_out=dxin, dx_accumulate=True)
                self._count(3)
                dx = dxin
        self._embed_bwd(st, dx)
        # ---------------- replicated-parameter gradients and optimizer
        if self.N > 1:
            dist.all_reduce(self.ln_grad32, group=self.ring.group)
            self._count(1)
        K.cast_f32_bf16(self.ln_grad32, self.ln_grad16)
        with nvtx_range("optimizer"):
            self._adam(self.plan if self.keep_grads else self.ln_plan)
        self.rng_step.add_(1)
        self._count(3)

    # ------------------------------------------------------------------------------------------
    def step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One training step on ``ids``/``targets`` of shape [seq, batch] (CUDA int64, or pinned host
        tensors which are copied asynchronously). Returns the mean token loss as a 1-element CUDA tensor."""
        S, B = ids.shape
        if self._static is None or (self._static["S"], self._static["B"]) != (S, B):
            self._static = self._alloc_static(S, B)
            self._graph = None
            self._calls = 0
        st = self._static
        st["ids"].copy_(ids, non_blocking=True)
        st["tgt"].copy_(targets, non_blocking=True)
        if not self.use_graph:
            self._counting = self.launches_per_step == 0
            self._step_impl(st)
            self._counting = False
            return st["loss"]
        self._calls += 1
        if self._calls == 1:
            # first call runs eagerly: sets kernel attributes, sizes the workspace, warms NCCL up
            self._counting = self.launches_per_step == 0
            self._step_impl(st)
            self._counting = False
            torch.cuda.synchronize()
            self.check()
            return st["loss"]
        if self._graph is None:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._step_impl(st)
            self._graph = g
        self._graph.replay()
        return st["loss"]

    # ------------------------------------------------------------------------------------------
    def state_dict(self):
        """Optimizer side of a checkpoint: Adam moments of every parameter (keyed by parameter name), the Adam step and
        the dropout step counter.  Together with ``model.state_dict()`` a run resumes bit-exactly."""
        names = {id(p): n for n, p in self.model.named_parameters()}
        moments = {}
        for (p_data, g, m1, m2, mult) in self.adam_entries:
            moments[self._entry_names[p_data.data_ptr()]] = (m1.detach().cpu().clone(), m2.detach().cpu().clone())
        del names
        return {"moments": moments, "adam_step": int(self.step_dev.item()), "rng_step": int(self.rng_step.item()),
                "state_dtypes": [str(d) for d in self.state_dtypes]}

    def load_state_dict(self, sd):
        if [str(d) for d in self.state_dtypes] != list(sd["state_dtypes"]):
            raise ValueError(f"checkpoint holds Adam moments as {sd['state_dtypes']}, this trainer as "
                             f"{[str(d) for d in self.state_dtypes]}")
        for (p_data, g, m1, m2, mult) in self.adam_entries:
            a, b = sd["moments"][self._entry_names[p_data.data_ptr()]]
            m1.copy_(a)
            m2.copy_(b)
        self.step_dev.fill_(sd["adam_step"])
        self.rng_step.fill_(sd["rng_step"])

    def check(self):
        """Raise if any kernel of the previous steps reported an expired wait (synchronises)."""
        self.eng.check()
        _lib.check_status(self.dev)
