"""LayerNorm / RMSNorm modules (replicated parameters) that run the library's sm_100a kernels on bf16 CUDA tensors
and plain PyTorch elsewhere.  State_dict keys are ``weight`` / ``bias`` like ``torch.nn.LayerNorm``."""
import torch
from torch import nn

from ..ops import functional as FO


class LayerNorm(nn.LayerNorm):
    def forward(self, x):
        if self.elementwise_affine and self.bias is not None and len(self.normalized_shape) == 1:
            return FO.layer_norm(x, self.weight, self.bias, self.eps)
        return super().forward(x)


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-5, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x):
        return FO.rms_norm(x, self.weight, self.eps)
