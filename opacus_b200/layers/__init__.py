"""Layers whose parameters live in plain ``nn.Linear``-like children so that
per-sample gradients can be taken: recurrent nets and multi-head attention."""
from .cross_entropy import FusedCrossEntropyLoss, fused_cross_entropy
from .dp_multihead_attention import DPMultiheadAttention, SequenceBias
from .dp_rnn import DPGRU, DPLSTM, DPRNN, DPGRUCell, DPLSTMCell, DPRNNCell, RNNLinear
from .param_rename import RenameParamsMixin

__all__ = [
    "DPRNN", "DPGRU", "DPLSTM", "DPRNNCell", "DPGRUCell", "DPLSTMCell", "RNNLinear",
    "DPMultiheadAttention", "SequenceBias", "RenameParamsMixin", "FusedCrossEntropyLoss", "fused_cross_entropy",
]
