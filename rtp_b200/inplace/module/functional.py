"""Same helpers as rtp_b200.module.functional (the reference keeps an identical copy under rtp/inplace/module)."""
from ...module.functional import *  # noqa: F401,F403
