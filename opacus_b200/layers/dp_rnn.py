"""Recurrent layers (Elman RNN, GRU, LSTM) built from two linear maps per cell
so that per-sample gradients are ordinary Linear per-sample gradients.

Layout differs from a naive time loop in one important way: the input
projection ``ih`` does not depend on the recurrence, so it is applied **once to
the whole (padded) sequence** as a single ``[B, T, in] -> [B, T, k*H]`` GEMM.
Only the hidden projection ``hh`` runs per time step.  The per-sample gradient
of ``ih`` is then a single contraction over ``K = T`` instead of ``T`` rank-one
updates, and the per-step ``hh`` calls are stacked by the gradient engine into
one ``K = T`` contraction as well.

Packed (variable-length) input is handled by padding to ``[T, B, *]`` and
freezing the state rows of sequences that have ended (or not yet started, for
the reverse direction).

Semantics and ``state_dict`` layout follow ``torch.nn.RNN/GRU/LSTM``
(behavioural parity: ``opacus/layers/dp_rnn.py:39-737``).  ``proj_size > 0`` is
not supported.
"""
import math
import numbers
import warnings
from typing import List, Optional, Type, Union

import torch
import torch.nn as nn
from torch import Tensor
from torch.nn.utils.rnn import PackedSequence

from ..utils.packed_sequences import compute_seq_lengths  # noqa: F401  (re-exported as in the reference)
from .param_rename import RenameParamsMixin


def apply_permutation(tensor: Tensor, dim: int, permutation: Optional[Tensor]) -> Tensor:
    """``tensor`` reordered along ``dim`` by ``permutation`` (unchanged when the permutation is None); the helper
    that ``opacus/layers/dp_rnn.py:30-36`` exports for the sorted / unsorted indices of a ``PackedSequence``."""
    return tensor if permutation is None else tensor.index_select(dim, permutation)


class RNNLinear(nn.Linear):
    """``nn.Linear`` used inside the recurrent cells.  A distinct type so the
    gradient engine knows that the batch is always axis 0 and that repeated
    calls within one forward pass are time steps of the same samples."""

    max_batch_len: int


class DPRNNCellBase(nn.Module):
    has_cell_state: bool = False
    num_chunks: int = 1

    def __init__(self, input_size: int, hidden_size: int, bias: bool, num_chunks: Optional[int] = None) -> None:
        super().__init__()
        if num_chunks is not None:
            self.num_chunks = num_chunks
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.bias = bias
        self.ih = RNNLinear(input_size, self.num_chunks * hidden_size, bias)
        self.hh = RNNLinear(hidden_size, self.num_chunks * hidden_size, bias)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        bound = 1.0 / math.sqrt(self.hidden_size)
        for w in self.parameters():
            nn.init.uniform_(w, -bound, bound)

    def set_max_batch_length(self, max_batch_length: int) -> None:
        self.ih.max_batch_len = max_batch_length
        self.hh.max_batch_len = max_batch_length

    # --- the two halves of a step -------------------------------------------------
    def project_input(self, x: Tensor) -> Tensor:
        """``ih`` applied to any ``[..., input_size]`` tensor."""
        return self.ih(x)

    def recur(self, gx: Tensor, state):
        """One step given the pre-computed input projection ``gx`` ``[b, k*H]``
        and the previous state restricted to the same ``b`` rows."""
        raise NotImplementedError

    def forward(self, input: Tensor, hx=None, batch_size_t: Optional[int] = None):
        """Single-step interface compatible with ``nn.RNNCell``-style use."""
        b = input.shape[0]
        if hx is None:
            z = torch.zeros(b, self.hidden_size, dtype=input.dtype, device=input.device)
            hx = (z, z) if self.has_cell_state else z
        if batch_size_t is not None:
            hx = tuple(s[:batch_size_t] for s in hx) if self.has_cell_state else hx[:batch_size_t]
        return self.recur(self.project_input(input), hx)


class DPRNNCell(DPRNNCellBase):
    """h' = act(W_ih x + b_ih + W_hh h + b_hh)."""

    def __init__(self, input_size: int, hidden_size: int, bias: bool, nonlinearity: str = "tanh") -> None:
        super().__init__(input_size, hidden_size, bias, num_chunks=1)
        if nonlinearity not in ("tanh", "relu"):
            raise ValueError(f"Unsupported nonlinearity: {nonlinearity}")
        self.nonlinearity = nonlinearity

    def recur(self, gx, h):
        pre = gx + self.hh(h)
        return torch.tanh(pre) if self.nonlinearity == "tanh" else torch.relu(pre)


class DPGRUCell(DPRNNCellBase):
    """r, z gates then candidate n = tanh(x_n + r * h_n); h' = (1-z) n + z h."""

    def __init__(self, input_size: int, hidden_size: int, bias: bool) -> None:
        super().__init__(input_size, hidden_size, bias, num_chunks=3)

    def recur(self, gx, h):
        xr, xz, xn = gx.chunk(3, dim=1)
        hr, hz, hn = self.hh(h).chunk(3, dim=1)
        r = torch.sigmoid(xr + hr)
        z = torch.sigmoid(xz + hz)
        n = torch.tanh(xn + r * hn)
        return n + z * (h - n)


class DPLSTMCell(DPRNNCellBase):
    """Gate order i, f, g, o as in ``nn.LSTM``."""

    has_cell_state = True

    def __init__(self, input_size: int, hidden_size: int, bias: bool) -> None:
        super().__init__(input_size, hidden_size, bias, num_chunks=4)

    def recur(self, gx, state):
        h, c = state
        i, f, g, o = (gx + self.hh(h)).chunk(4, dim=1)
        c_new = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        return torch.sigmoid(o) * torch.tanh(c_new), c_new


RNN_CELL_TYPES = {
    "RNN_TANH": (DPRNNCell, {"nonlinearity": "tanh"}),
    "RNN_RELU": (DPRNNCell, {"nonlinearity": "relu"}),
    "GRU": (DPGRUCell, {}),
    "LSTM": (DPLSTMCell, {}),
}


def _pad_packed(data: Tensor, batch_sizes: List[int]) -> Tensor:
    """``PackedSequence.data`` -> zero padded ``[T, B, F]`` (rows in packed order)."""
    T, B = len(batch_sizes), batch_sizes[0]
    out = data.new_zeros(T, B, data.shape[-1])
    ofs = 0
    for t, b in enumerate(batch_sizes):
        out[t, :b] = data[ofs: ofs + b]
        ofs += b
    return out


class DPRNNBase(RenameParamsMixin, nn.Module):
    """Multi-layer, optionally bidirectional recurrent network over any cell type."""

    def __init__(
        self,
        mode: Union[str, Type[DPRNNCellBase]],
        input_size: int,
        hidden_size: int,
        num_layers: int = 1,
        bias: bool = True,
        batch_first: bool = False,
        dropout: float = 0.0,
        bidirectional: bool = False,
        proj_size: int = 0,
        cell_params: Optional[dict] = None,
    ) -> None:
        super().__init__()
        self.cell_params = {}
        if isinstance(mode, str):
            if mode not in RNN_CELL_TYPES:
                raise ValueError(f"Invalid RNN mode '{mode}', available options: {list(RNN_CELL_TYPES.keys())}")
            self.cell_type, defaults = RNN_CELL_TYPES[mode]
            self.cell_params.update(defaults)
        else:
            self.cell_type = mode
        self.cell_params.update(cell_params or {})

        if not isinstance(dropout, numbers.Number) or isinstance(dropout, bool) or not 0 <= dropout <= 1:
            raise ValueError(
                "dropout should be a number in range [0, 1] representing the probability of an element being zeroed"
            )
        if dropout > 0 and num_layers == 1:
            warnings.warn(
                "dropout option adds dropout after all but last recurrent layer, so non-zero dropout expects "
                f"num_layers greater than 1, but got dropout={dropout} and num_layers={num_layers}"
            )
        if proj_size > 0:
            raise NotImplementedError("proj_size > 0 is not supported")
        if proj_size < 0:
            raise ValueError("proj_size should be a positive integer or zero to disable projections")

        self.has_cell_state = self.cell_type.has_cell_state
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.num_layers = num_layers
        self.bias = bias
        self.batch_first = batch_first
        self.dropout = float(dropout)
        self.bidirectional = bidirectional
        self.proj_size = proj_size
        self.num_directions = 2 if bidirectional else 1
        self.dropout_layer = nn.Dropout(dropout) if dropout > 0 else None
        self.cells = self.initialize_cells()

    # ---------------------------------------------------------------- construction
    def initialize_cells(self) -> List[DPRNNCellBase]:
        cells, names = [], {}
        for layer in range(self.num_layers):
            width_in = self.input_size if layer == 0 else self.hidden_size * self.num_directions
            for direction in range(self.num_directions):
                tag = f"l{layer}" + ("_reverse" if direction else "")
                cell = self.cell_type(width_in, self.hidden_size, bias=self.bias, **self.cell_params)
                setattr(self, tag, cell)
                cells.append(cell)
                for part in ("weight", "bias") if self.bias else ("weight",):
                    for mat in ("ih", "hh"):
                        names[f"{tag}.{mat}.{part}"] = f"{part}_{mat}_{tag}"
        self.set_rename_map(names)
        return cells

    def iterate_layers(self, *args):
        """Yield ``(layer, [(direction, tuple(arg[idx] ...)), ...])`` in ``nn.LSTM`` order."""
        for layer in range(self.num_layers):
            yield layer, [
                (d, tuple(a[self.num_directions * layer + d] for a in args)) for d in range(self.num_directions)
            ]

    # --------------------------------------------------------------------- forward
    def forward(self, input: Union[Tensor, PackedSequence], state_init=None):
        packed = isinstance(input, PackedSequence)
        if packed:
            data, batch_sizes_t, sorted_idx, unsorted_idx = input
            batch_sizes = [int(b) for b in batch_sizes_t]
            x = _pad_packed(data, batch_sizes)
        else:
            batch_sizes_t = sorted_idx = unsorted_idx = None
            x = input.transpose(0, 1) if self.batch_first else input
            batch_sizes = None
        T, B = x.shape[0], x.shape[1]
        for cell in self.cells:
            cell.set_max_batch_length(B)

        n_states = self.num_layers * self.num_directions

        def _init(s):
            if s is None:
                return x.new_zeros(n_states, B, self.hidden_size)
            return s if sorted_idx is None else s.index_select(1, sorted_idx)

        if self.has_cell_state:
            h0s, c0s = state_init if state_init is not None else (None, None)
            h0s, c0s = _init(h0s), _init(c0s)
        else:
            h0s, c0s = _init(state_init), [None] * n_states

        last_h, last_c = [], []
        seq = x
        for layer, directions in self.iterate_layers(self.cells, h0s, c0s):
            outs = []
            for direction, (cell, h0, c0) in directions:
                y, h, c = self.forward_layer(seq, h0, c0, batch_sizes, cell, reverse=direction == 1)
                outs.append(y)
                last_h.append(h)
                last_c.append(c)
            seq = outs[0] if len(outs) == 1 else torch.cat(outs, dim=2)
            if self.dropout_layer is not None and layer < self.num_layers - 1:
                seq = self.dropout_layer(seq)

        if packed:
            flat = torch.cat([seq[t, :b] for t, b in enumerate(batch_sizes)], dim=0)
            output = PackedSequence(flat, batch_sizes_t, sorted_idx, unsorted_idx)
        else:
            output = seq.transpose(0, 1) if self.batch_first else seq

        def _final(states):
            s = torch.stack(states, dim=0)
            return s if unsorted_idx is None else s.index_select(1, unsorted_idx)

        hidden = (_final(last_h), _final(last_c)) if self.has_cell_state else _final(last_h)
        return output, hidden

    def forward_layer(self, x: Tensor, h0: Tensor, c0: Optional[Tensor], batch_sizes: Optional[List[int]],
                      cell: DPRNNCellBase, reverse: bool):
        """Run one direction of one layer over padded time-major ``x`` ``[T, B, F]``.

        Returns ``(y [T, B, H], h_last [B, H], c_last or None)``.
        """
        T, B = x.shape[0], x.shape[1]
        # One GEMM for every time step's input projection; batch is axis 0 for RNNLinear.
        gx = cell.project_input(x.transpose(0, 1))  # [B, T, k*H]
        h, c = h0, c0
        ys: List[Optional[Tensor]] = [None] * T
        steps = range(T - 1, -1, -1) if reverse else range(T)
        for t in steps:
            b = B if batch_sizes is None else batch_sizes[t]
            g_t = gx[:b, t]
            if self.has_cell_state:
                h_new, c_new = cell.recur(g_t, (h[:b], c[:b]))
                c = c_new if b == B else torch.cat([c_new, c[b:]], dim=0)
            else:
                h_new = cell.recur(g_t, h[:b])
            h = h_new if b == B else torch.cat([h_new, h[b:]], dim=0)
            ys[t] = h_new if b == B else torch.cat([h_new, h_new.new_zeros(B - b, h_new.shape[1])], dim=0)
        y = torch.stack(ys, dim=0) if T > 0 else x.new_zeros(0, B, self.hidden_size)
        return y, h, c


class DPRNN(DPRNNBase):
    """Drop-in for ``nn.RNN`` with per-sample-gradient friendly parameters."""

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True,
                 batch_first: bool = False, dropout: float = 0, bidirectional: bool = False, proj_size: int = 0,
                 nonlinearity: str = "tanh") -> None:
        super().__init__(DPRNNCell, input_size, hidden_size, num_layers=num_layers, bias=bias,
                         batch_first=batch_first, dropout=dropout, bidirectional=bidirectional,
                         proj_size=proj_size, cell_params={"nonlinearity": nonlinearity})


class DPGRU(DPRNNBase):
    """Drop-in for ``nn.GRU``."""

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True,
                 batch_first: bool = False, dropout: float = 0, bidirectional: bool = False, proj_size: int = 0) -> None:
        super().__init__(DPGRUCell, input_size, hidden_size, num_layers=num_layers, bias=bias,
                         batch_first=batch_first, dropout=dropout, bidirectional=bidirectional, proj_size=proj_size)


class DPLSTM(DPRNNBase):
    """Drop-in for ``nn.LSTM``."""

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True,
                 batch_first: bool = False, dropout: float = 0, bidirectional: bool = False, proj_size: int = 0) -> None:
        super().__init__(DPLSTMCell, input_size, hidden_size, num_layers=num_layers, bias=bias,
                         batch_first=batch_first, dropout=dropout, bidirectional=bidirectional, proj_size=proj_size)
