"""Rotated embedding: the table is sharded along the *embedding* dimension (``[V, D/N]``) and the N
column blocks of the lookup are concatenated (reference: rtp/module/embedding.py:33-164)."""
from typing import Callable, Optional

import torch
import torch.nn.functional as F
from torch import nn
from torch.nn import init

from ..parallel.flat import RotatedModule
from ..parallel.rotated import rotated_apply
from .utils import affine_weight, divide_and_check_no_remainder


class ModelParallelEmbedding(nn.Embedding):
    """Embedding-dim shard ``[V, D/N]`` (reference: rtp/module/embedding.py:33-71)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, world_size: int = 1, rank: int = 0, **kw):
        self.world_size, self.rank = world_size, rank
        self.full_embedding_dim = embedding_dim
        self.embedding_dim_per_partition = divide_and_check_no_remainder(embedding_dim, world_size)
        super().__init__(num_embeddings, self.embedding_dim_per_partition, **kw)

    def affine_weight(self, Embedding_layer: Optional[nn.Embedding]):
        if Embedding_layer is not None:
            affine_weight(self.weight, Embedding_layer.weight, self.embedding_dim_per_partition, 1,
                          self.world_size, self.rank)


class ParallelEmbedding(RotatedModule):
    def __init__(self, num_embeddings: int, embedding_dim: int, world_size: Optional[int] = None,
                 rank: Optional[int] = None, padding_idx: Optional[int] = None, max_norm: Optional[float] = None,
                 norm_type: float = 2.0, scale_grad_by_freq: bool = False, sparse: bool = False,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = init.xavier_normal_,
                 keep_master_weight_for_test: bool = False, Embedding_layer: Optional[nn.Embedding] = None,
                 device=None, dtype=None, group=None):
        super().__init__()
        self._setup_ring(group, world_size, rank)
        if sparse:
            raise ValueError("sparse gradients cannot travel in a flat shard buffer")
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padding_idx, self.max_norm, self.norm_type = padding_idx, max_norm, norm_type
        self.scale_grad_by_freq = scale_grad_by_freq
        self.embedding = ModelParallelEmbedding(num_embeddings, embedding_dim, self.world_size, self.rank,
                                                padding_idx=padding_idx, max_norm=max_norm, norm_type=norm_type,
                                                scale_grad_by_freq=scale_grad_by_freq, device=device, dtype=dtype)
        self.embedding_dim_per_partition = self.embedding.embedding_dim_per_partition
        self.embedding.affine_weight(Embedding_layer)
        self._flatten()

    def shard_parameters(self):
        return [self.embedding.weight]

    def shard_names(self):
        return ["weight"]

    def shard_spec(self):
        return {"embedding.weight": ("split", 1)}

    @property
    def embeddings(self):
        return [self.embedding] * self.world_size

    def forward(self, input_: torch.Tensor) -> torch.Tensor:  # type: ignore
        pad, mx, nt, sg = self.padding_idx, self.max_norm, self.norm_type, self.scale_grad_by_freq
        from ..parallel import fused
        if pad is None and mx is None and not sg and self._full_param.is_cuda and \
                fused.use_fused(self._full_param, self._full_param) and self.embedding_dim_per_partition % 8 == 0:
            from ..parallel.engine import fused_embedding
            return fused_embedding(self, input_, self.embedding.weight, self.embedding_dim)

        def fn(j, views, ids):
            return F.embedding(ids, views[0], pad, mx, nt, sg, False)
        return rotated_apply(self.ring, fn, self.shard_parameters(), self._full_param, self._layout, (input_,),
                             combine="cat", cat_dim=-1, inplace=self.inplace, owner=self)
