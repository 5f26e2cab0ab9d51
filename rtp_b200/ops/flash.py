"""Long-sequence attention entry point (tcgen05 flash kernel)."""


def flash_attention_available(seq_len: int, head_dim: int) -> bool:
    return False


def flash_attention(q, k, v, causal=True):
    raise NotImplementedError
