"""Rotation runtime: process-group context, ring transport (torch.distributed) and the autograd
machinery that rotates weight shards and carries their gradients home."""
from .context import RingContext, get_context, set_backend, get_backend  # noqa: F401
from .rotated import rotated_apply, ShardLayout  # noqa: F401
