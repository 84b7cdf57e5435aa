"""Per-sample gradient of an embedding table kept in compact form.

The dense per-sample gradient of ``nn.Embedding`` is ``[B, V, D]`` with at most
``T`` non-zero rows per sample -- 3.9 GB of zeros for a 30000 x 512 table at
batch 64, which is what ``opacus/grad_sample/embedding.py:53-61`` materialises.
:class:`LazyEmbeddingGradSample` *is* a tensor of that shape as far as ``shape``,
``dtype``, ``device`` and ``isinstance`` go, but only holds the token ids
``[B, T]`` and the output gradient ``[B, T, D]``.  The two things DP-SGD does with
a per-sample gradient have direct forms on the compact pair -- the squared norm
is the masked Gram product ``<[id_t == id_s], g g^T>`` and the clip-weighted sum
is a scatter-add -- and :func:`opacus_b200.ops.grad_sample_norm_sq` /
:func:`opacus_b200.ops.weighted_sum` take them.  Any other torch operation on
the object first builds the dense tensor (once) and then runs on it, so code that
reads ``p.grad_sample`` keeps working.
"""
import torch
from torch.utils._pytree import tree_map

from . import _ref


class LazyEmbeddingGradSample(torch.Tensor):
    @staticmethod
    def __new__(cls, ids: torch.Tensor, g: torch.Tensor, num_embeddings: int, padding_idx=None):
        B, D = ids.shape[0], g.shape[-1]
        out = torch.Tensor._make_wrapper_subclass(cls, (B, num_embeddings, D), dtype=g.dtype, device=g.device,
                                                  requires_grad=False)
        out._ids = ids.reshape(B, -1)
        out._g = g.reshape(B, -1, D)
        out._num_embeddings = num_embeddings
        out._padding_idx = padding_idx
        out._dense = None
        return out

    def dense(self) -> torch.Tensor:
        """The ``[B, V, D]`` tensor (built on first use, then kept)."""
        if self._dense is None:
            self._dense = _ref.embedding_grad_sample(self._ids, self._g, self._num_embeddings)
        return self._dense

    @property
    def is_materialized(self) -> bool:
        return self._dense is not None

    def __repr__(self):
        return (f"LazyEmbeddingGradSample(shape={tuple(self.shape)}, tokens={tuple(self._ids.shape)}, "
                f"materialized={self.is_materialized})")

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        unwrap = lambda t: t.dense() if isinstance(t, cls) else t
        return func(*tree_map(unwrap, args), **tree_map(unwrap, kwargs or {}))
