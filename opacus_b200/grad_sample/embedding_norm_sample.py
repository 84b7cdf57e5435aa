"""Kept as a module for import compatibility; the implementation lives in
:mod:`.embedding` (``opacus/grad_sample/embedding_norm_sample.py:27``)."""
from .embedding import compute_embedding_norm_sample  # noqa: F401
