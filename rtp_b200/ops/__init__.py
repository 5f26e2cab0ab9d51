"""Hand-written sm_100a kernels (ctypes front-ends). Nothing here falls back to PyTorch ops."""
