from .sharded import (sharding_plan, shard_full, consolidate, reshard, save_sharded, load_sharded,  # noqa: F401
                      shard_state_dict, plain_lm_to_rtp_keys)
