"""Synthetic data with the reference's shapes (benchmarks/datasets/wikitext2_data.py:25-33,61-107): one long token
stream batchified to ``[seq_len, batch]`` blocks; targets are the inputs shifted by one token.  Unlike the
reference the vocabulary size is honoured and every rank may draw its own stream."""
import torch


def synthetic_stream(vocab_size: int, n_tokens: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab_size, (n_tokens,), generator=g, dtype=torch.int64)


def batchify(stream: torch.Tensor, batch_size: int) -> torch.Tensor:
    n = stream.numel() // batch_size
    return stream[: n * batch_size].view(batch_size, n).t().contiguous()


def get_batch(source: torch.Tensor, i: int, seq_len: int):
    """``source`` is ``[n, batch]``; returns inputs ``[seq_len, batch]`` and next-token targets of the same shape."""
    seq_len = min(seq_len, source.size(0) - 1 - i)
    return source[i:i + seq_len], source[i + 1:i + 1 + seq_len]


class SyntheticLM:
    def __init__(self, vocab_size, seq_len, batch_size, n_batches=64, seed=0, rank=0, pin=False):
        stream = synthetic_stream(vocab_size, (seq_len * n_batches + 1) * batch_size, seed + rank)
        self.source = batchify(stream, batch_size)
        self.seq_len, self.n = seq_len, n_batches
        self.pin = pin

    def __len__(self):
        return self.n

    def __iter__(self):
        for b in range(self.n):
            x, y = get_batch(self.source, b * self.seq_len, self.seq_len)
            x, y = x.contiguous(), y.contiguous()
            if self.pin:
                x, y = x.pin_memory(), y.pin_memory()
            yield x, y
