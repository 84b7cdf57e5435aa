"""Helpers around ``PackedSequence`` (``opacus/utils/packed_sequences.py:22-117``)."""
from typing import List, Optional

import torch
from torch.nn.utils.rnn import PackedSequence, pack_padded_sequence, pad_sequence


def _gen_packed_data(minibatch_size: int, max_seq_length: int, input_dim: int, batch_first: bool,
                     sorted_: Optional[bool] = False) -> PackedSequence:
    """Random packed batch with lengths uniform in ``[1, max_seq_length]``."""
    lengths = torch.randint(1, max_seq_length + 1, (minibatch_size,)).tolist()
    if sorted_:
        lengths.sort(reverse=True)
    seqs = [torch.randn(n, input_dim) for n in lengths]
    if batch_first:
        padded = pad_sequence(seqs, batch_first=True)
    else:
        padded = torch.zeros(max_seq_length, minibatch_size, input_dim)
        for b, s in enumerate(seqs):
            padded[: len(s), b] = s
    return pack_padded_sequence(padded, lengths, batch_first=batch_first, enforce_sorted=bool(sorted_))


def compute_seq_lengths(batch_sizes: torch.Tensor) -> List[int]:
    """Sequence lengths (descending) from ``PackedSequence.batch_sizes``:
    sequence ``b`` is as long as the number of time steps whose batch size exceeds ``b``."""
    sizes = batch_sizes.tolist()
    if not sizes:
        return []
    return [sum(1 for s in sizes if s > b) for b in range(sizes[0])]
