"""GEMMs fused with the collective next to them, over NVLink peer memory
(``csrc/tp_gemm.cu``): one kernel per rank pulls the peers' shards while the
tensor cores already work on the rows that have arrived, or pushes finished
output tiles to their owners while the remaining tiles are computed.

* :class:`AllGatherGemm` -- ``y = gather_rows(x) @ w.T`` (sequence-sharded
  activations into a column-parallel layer) or ``y = x @ gather_rows(w).T``
  (row-sharded weights, ZeRO-3 / FSDP style, into their first use).  The
  gathered operand stays in ``self.full`` for the backward pass (per-sample
  gradient norms need the whole sequence).
* :class:`GemmReduceScatter` -- ``y_rows_of_this_rank = sum_ranks (x_r @ w_r.T)``
  (row-parallel layer producing sequence-sharded output).

Each object owns its symmetric buffers; constructing one is a collective call.
The reference reaches the same dataflow through DTensor redistributions, i.e.
separate NCCL all-gather / reduce-scatter kernels around cuBLAS
(``examples/tensor_parallelism_llama.py:104-152``, ``opacus/utils/fsdp_utils.py:52-60``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import symm


def _kernels():
    from ..ops import _cuda

    return _cuda.load()


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """``a @ b.T`` for bf16 ``a [M, K]``, ``b [N, K]`` with this package's tcgen05 kernel."""
    if out is None:
        out = torch.empty(a.shape[0], b.shape[0], dtype=torch.bfloat16, device=a.device)
    _kernels().tp_gemm(a, b, out, 0, [], [], [], None, 0, 1, 0, 0)
    return out


class AllGatherGemm:
    """``gather="a"``: ``__call__(w)`` returns ``full_x @ w.T`` where rank ``r``'s rows of
    ``full_x`` are what rank ``r`` wrote into its ``shard`` (``[rows_per_rank, K]``).
    ``gather="b"``: ``__call__(x)`` returns ``x @ full_w.T`` likewise for weight rows.
    ``rows_per_rank`` must be a multiple of 128 (``"a"``) or 256 (``"b"``), ``K`` of 32 / 16."""

    def __init__(self, rows_per_rank: int, K: int, device, group=None, gather: str = "a"):
        if gather not in ("a", "b"):
            raise ValueError("gather must be 'a' or 'b'")
        self.group = group
        self.rank, self.world = symm.world_info(group)
        self.gather = gather
        self.unit = 128 if gather == "a" else 256
        if rows_per_rank % self.unit or (self.unit * K * 2) % 8192:
            raise ValueError(f"rows_per_rank must be a multiple of {self.unit} and K of {8192 // (2 * self.unit)}")
        self.rows_per_rank, self.K = rows_per_rank, K
        self.device = torch.device(device)
        self._shard = symm.alloc(rows_per_rank * K, torch.bfloat16, self.device, group)
        self._flags = symm.alloc(64, torch.int32, self.device, group)
        self.shard = self._shard.tensor.view(rows_per_rank, K)
        self.full = torch.zeros(rows_per_rank * self.world, K, dtype=torch.bfloat16, device=self.device)
        self._ready = torch.zeros(rows_per_rank * self.world // self.unit, dtype=torch.int32, device=self.device)
        self._epoch = 0
        if self.world > 1:
            dist.barrier(group=group)

    def __call__(self, other: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        rows = self.rows_per_rank * self.world
        M, N = (rows, other.shape[0]) if self.gather == "a" else (other.shape[0], rows)
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)
        self._epoch += 1
        a, b = (self.full, other) if self.gather == "a" else (other, self.full)
        _kernels().tp_gemm(a, b, out, 1 if self.gather == "a" else 2, self._shard.ptrs, [], self._flags.ptrs,
                           self._ready, self.rank, self.world, self._epoch, 0)
        return out


class GemmReduceScatter:
    """``__call__(x_local [M, K_local], w_local [N, K_local])`` returns this rank's
    ``M / world`` rows of ``sum_ranks x_r @ w_r.T`` (bf16 partials, fp32 summation in
    rank order).  ``M`` must be a multiple of ``128 * world``."""

    def __init__(self, M: int, N: int, device, group=None):
        self.group = group
        self.rank, self.world = symm.world_info(group)
        if M % (128 * self.world) or N % 8:
            raise ValueError("M must be a multiple of 128 * world and N of 8")
        self.M, self.N = M, N
        self.device = torch.device(device)
        self._slots = symm.alloc(2 * M * N, torch.bfloat16, self.device, group, zero=False)
        self._flags = symm.alloc(64, torch.int32, self.device, group)
        self._epoch = 0
        if self.world > 1:
            dist.barrier(group=group)

    def __call__(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        if x.shape[0] != self.M or w.shape[0] != self.N:
            raise ValueError("operand shapes do not match the buffers of this object")
        if out is None:
            out = torch.empty(self.M // self.world, self.N, dtype=torch.bfloat16, device=self.device)
        self._epoch += 1
        _kernels().tp_gemm(x, w, out, 3, [], self._slots.ptrs, self._flags.ptrs, None, self.rank, self.world,
                           self._epoch, 0)
        return out
