"""rtp_b200: rotated tensor parallelism for B200 (sm_100a).

Import paths mirror the reference package below the root: ``rtp_b200.module.linear``,
``rtp_b200.inplace.module.linear``, ``rtp_b200.models.transformer_lm_rtp``,
``rtp_b200.rotated_tensor_parallel`` and so on.
"""
from .version import __version__  # noqa: F401
