from .sharded_adam import ShardedAdam, ShardedAdamW, sync_replicated_grads, clip_grad_value_  # noqa: F401
