"""Recurrent layers (nn/rnn.go:20-863, nn/sequtil.go:15-268, nn/seq2seq.go:23-88).

Cells: ``RNNCell`` (tanh / ReLU), ``LSTMCell`` (gate order i, f, g, o; optional projection
``whr``), ``GRUCell`` (r, z, n).  Children are named ``wih`` / ``whh`` (/ ``whr``).  Stacks
``RNN`` / ``LSTM`` / ``GRU``: batch-first input (B, T, F); options layers, bidirectional,
dropout between layers, ReLU (RNN), proj_size (LSTM); children ``cells.N``, ``backcells.N``,
``dropout.N``.  State layout for stacks: (L * D, B, H).  Gates are computed by the fused
Linear kernels and one fused gate kernel per cell and direction (``ops/rnn.py``); the time
loop stays on the autograd tape.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from ..ops import elementwise as _ew
from ..ops import rnn as _rnn_ops
from .dropout import Dropout
from .embedding import Embedding
from .linear import Linear
from .module import Module, ModuleList


def _sig(x):
    return _ew.unary("sigmoid", x.contiguous())


def _tanh(x):
    return _ew.unary("tanh", x.contiguous())


class RNNCell(Module):
    def __init__(self, input_size: int, hidden_size: int, relu: bool = False, *, dtype=torch.float32, device=None):
        super().__init__()
        self.input_size, self.hidden_size, self.relu = input_size, hidden_size, relu
        self.wih = Linear(input_size, hidden_size, True, dtype=dtype, device=device)
        self.whh = Linear(hidden_size, hidden_size, False, dtype=dtype, device=device)

    def forward(self, x, h=None):
        if h is None:
            h = x.new_zeros(x.shape[0], self.hidden_size)
        pre = self.wih(x) + self.whh(h)
        return _ew.unary("relu", pre) if self.relu else _tanh(pre)


class LSTMCell(Module):
    def __init__(self, input_size: int, hidden_size: int, proj_size: int = 0, *, dtype=torch.float32, device=None):
        super().__init__()
        if proj_size < 0 or proj_size >= hidden_size > 0 and proj_size >= hidden_size:
            raise ValueError("LSTMCell: proj_size must be in [0, hidden_size)")
        self.input_size, self.hidden_size, self.proj_size = input_size, hidden_size, proj_size
        h_out = proj_size if proj_size > 0 else hidden_size
        self.wih = Linear(input_size, 4 * hidden_size, True, dtype=dtype, device=device)
        self.whh = Linear(h_out, 4 * hidden_size, False, dtype=dtype, device=device)
        if proj_size > 0:
            self.whr = Linear(hidden_size, proj_size, False, dtype=dtype, device=device)
        else:
            self.whr = None

    def hidden_out(self):
        return self.proj_size if self.proj_size > 0 else self.hidden_size

    def forward(self, x, state: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        B, H = x.shape[0], self.hidden_size
        if state is None:
            state = (x.new_zeros(B, self.hidden_out()), x.new_zeros(B, H))
        h, c = state
        # the second projection adds onto the first in its GEMM epilogue; the gate arithmetic is
        # one fused kernel per direction (ops/rnn.py)
        gates = self.whh(h, residual=self.wih(x))
        h_new, c_new = _rnn_ops.lstm_gates(gates, c)
        if self.whr is not None:
            h_new = self.whr(h_new)
        return h_new, c_new


class GRUCell(Module):
    def __init__(self, input_size: int, hidden_size: int, *, dtype=torch.float32, device=None):
        super().__init__()
        self.input_size, self.hidden_size = input_size, hidden_size
        self.wih = Linear(input_size, 3 * hidden_size, True, dtype=dtype, device=device)
        self.whh = Linear(hidden_size, 3 * hidden_size, True, dtype=dtype, device=device)

    def forward(self, x, h=None):
        H = self.hidden_size
        if h is None:
            h = x.new_zeros(x.shape[0], H)
        return _rnn_ops.gru_gates(self.wih(x), self.whh(h), h)


# ---------------------------------------------------------------------------------------
# sequence utilities
# ---------------------------------------------------------------------------------------
class PackedSequence:
    """Padded storage (B, T, F) plus per-sequence lengths (the reference keeps padded storage)."""

    def __init__(self, data: torch.Tensor, lengths: Sequence[int]):
        self.data, self.lengths = data, [int(l) for l in lengths]


def PadSequence(seqs: Sequence[torch.Tensor], padding_value: float = 0.0) -> torch.Tensor:
    T = max(s.shape[0] for s in seqs)
    out = seqs[0].new_full((len(seqs), T) + tuple(seqs[0].shape[1:]), padding_value)
    for i, s in enumerate(seqs):
        out[i, :s.shape[0]] = s
    return out


def UnpadSequence(padded: torch.Tensor, lengths: Sequence[int]) -> List[torch.Tensor]:
    return [padded[i, :int(l)] for i, l in enumerate(lengths)]


def PackPaddedSequence(padded: torch.Tensor, lengths: Sequence[int]) -> PackedSequence:
    if len(lengths) != padded.shape[0] or any(int(l) < 0 or int(l) > padded.shape[1] for l in lengths):
        raise ValueError("PackPaddedSequence: bad lengths")
    return PackedSequence(padded, lengths)


def PackSequence(seqs: Sequence[torch.Tensor]) -> PackedSequence:
    return PackedSequence(PadSequence(seqs), [s.shape[0] for s in seqs])


def PadPackedSequence(packed: PackedSequence, padding_value: float = 0.0):
    T = max(packed.lengths) if packed.lengths else 0
    data = packed.data[:, :T].clone()
    for i, l in enumerate(packed.lengths):
        data[i, l:] = padding_value
    return data, list(packed.lengths)


def _reverse_valid_prefix(x: torch.Tensor, lengths: Sequence[int]) -> torch.Tensor:
    """Reverses the first ``lengths[b]`` steps of every sequence, leaves the padding in place."""
    B, T = x.shape[:2]
    idx = torch.arange(T, device=x.device)[None].repeat(B, 1)
    for b, l in enumerate(lengths):
        idx[b, :l] = torch.arange(l - 1, -1, -1, device=x.device)
    return x.gather(1, idx.reshape(B, T, *([1] * (x.dim() - 2))).expand_as(x))


def _gather_last_steps(out: torch.Tensor, lengths: Sequence[int]) -> torch.Tensor:
    idx = torch.as_tensor([max(int(l) - 1, 0) for l in lengths], device=out.device)
    return out[torch.arange(out.shape[0], device=out.device), idx]


# ---------------------------------------------------------------------------------------
# stacks
# ---------------------------------------------------------------------------------------
class _RNNStack(Module):
    kind = "rnn"

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bidirectional: bool = False,
                 dropout: float = 0.0, relu: bool = False, proj_size: int = 0, *, dtype=torch.float32, device=None):
        super().__init__()
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.bidirectional, self.proj_size = bidirectional, proj_size
        D = 2 if bidirectional else 1
        h_out = proj_size if (proj_size > 0 and self.kind == "lstm") else hidden_size
        kw = dict(dtype=dtype, device=device)

        def cell(i):
            n_in = input_size if i == 0 else h_out * D
            if self.kind == "lstm":
                return LSTMCell(n_in, hidden_size, proj_size, **kw)
            if self.kind == "gru":
                return GRUCell(n_in, hidden_size, **kw)
            return RNNCell(n_in, hidden_size, relu, **kw)

        self.cells = ModuleList([cell(i) for i in range(num_layers)])
        self.backcells = ModuleList([cell(i) for i in range(num_layers)]) if bidirectional else None
        self.dropout = ModuleList([Dropout(dropout) for _ in range(max(num_layers - 1, 0))]) if dropout > 0 else None

    def _run_dir(self, cell, x, lengths, reverse, st0):
        B, T = x.shape[:2]
        if reverse:
            x = _reverse_valid_prefix(x, lengths) if lengths is not None else x.flip(1)
        st = st0
        outs = []
        for t in range(T):
            new = cell(x[:, t], st)
            if lengths is not None:
                alive = torch.as_tensor([1.0 if t < l else 0.0 for l in lengths], device=x.device, dtype=x.dtype)[:, None]
                if self.kind == "lstm":
                    h0 = st[0] if st is not None else torch.zeros_like(new[0])
                    c0 = st[1] if st is not None else torch.zeros_like(new[1])
                    new = (alive * new[0] + (1 - alive) * h0, alive * new[1] + (1 - alive) * c0)
                    outs.append(new[0] * alive)
                else:
                    h0 = st if st is not None else torch.zeros_like(new)
                    new = alive * new + (1 - alive) * h0
                    outs.append(new * alive)
            else:
                outs.append(new[0] if self.kind == "lstm" else new)
            st = new
        out = torch.stack(outs, 1)
        if reverse:
            out = _reverse_valid_prefix(out, lengths) if lengths is not None else out.flip(1)
        return out, st

    def ForwardWithState(self, x, state=None, lengths=None):
        """Returns (output (B, T, D*H_out), final state); state tensors are (L*D, B, H)."""
        D = 2 if self.bidirectional else 1
        hs, cs = [], []
        inp = x
        for l in range(self.num_layers):
            outs = []
            for d in range(D):
                cell = self.cells[l] if d == 0 else self.backcells[l]
                st0 = None
                if state is not None:
                    k = l * D + d
                    st0 = (state[0][k], state[1][k]) if self.kind == "lstm" else state[k]
                o, st = self._run_dir(cell, inp, lengths, d == 1, st0)
                outs.append(o)
                if self.kind == "lstm":
                    hs.append(st[0]); cs.append(st[1])
                else:
                    hs.append(st)
            inp = outs[0] if D == 1 else torch.cat(outs, -1)
            if self.dropout is not None and l < self.num_layers - 1:
                inp = self.dropout[l](inp)
        h = torch.stack(hs)
        return inp, ((h, torch.stack(cs)) if self.kind == "lstm" else h)

    def forward(self, x):
        return self.ForwardWithState(x)[0]

    def ForwardPacked(self, packed: PackedSequence, state=None):
        """Runs over a packed batch: padding steps neither update the state nor produce output."""
        out, st = self.ForwardWithState(packed.data, state, packed.lengths)
        return PackedSequence(out, packed.lengths), st


class RNN(_RNNStack):
    kind = "rnn"


class LSTM(_RNNStack):
    kind = "lstm"


class GRU(_RNNStack):
    kind = "gru"


class Seq2Seq(Module):
    """LSTM encoder / decoder with teacher forcing; children ``embsrc, embtgt, encoder, decoder,
    outproj``."""

    def __init__(self, src_vocab: int, tgt_vocab: int, embed_dim: int, hidden_size: int, *, dtype=torch.float32,
                 device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.embsrc = Embedding(src_vocab, embed_dim, **kw)
        self.embtgt = Embedding(tgt_vocab, embed_dim, **kw)
        self.encoder = LSTM(embed_dim, hidden_size, **kw)
        self.decoder = LSTM(embed_dim, hidden_size, **kw)
        self.outproj = Linear(hidden_size, tgt_vocab, **kw)

    def forward(self, src, tgt_in):
        """src (B, Ts), tgt_in (B, Tt) token ids -> logits (B, Tt, tgt_vocab)."""
        _, st = self.encoder.ForwardWithState(self.embsrc(src))
        out, _ = self.decoder.ForwardWithState(self.embtgt(tgt_in), st)
        return self.outproj(out)
