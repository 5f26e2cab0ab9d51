"""Same helpers as rtp_b200.module.utils (the reference keeps an identical copy under rtp/inplace/module)."""
from ...module.utils import *  # noqa: F401,F403
