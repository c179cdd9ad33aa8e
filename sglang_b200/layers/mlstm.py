"""Matrix memory with exponential gates and a running maximum (the mLSTM cell of xLSTM).  Per head, on the projections of the layer input h:

    q = W_q h / sqrt(dim),  k = W_k h,  v = W_v h
    i = cap tanh((W_i h + b_i) / cap)                       log input gate
    f = logsigmoid(cap tanh((W_f h + b_f) / cap))           log forget gate
    m_t = max(f + m_(t-1), i)                               m = 0, S = 0, n = 0 at the start of a sequence
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T            S: [dim, vdim]
    n_t = exp(f + m_(t-1) - m_t) n_(t-1) + exp(i - m_t) k
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

then every head's o is divided by its root mean square, the heads together times a weight, times ``sigmoid(W_g h)``, and the output projection.

How it runs: m depends on the gates alone, so ``ops.mlstm_prepare`` walks it first (fp32, one lane per request and head) and leaves every
token's decay ``exp(f + m_(t-1) - m_t)`` and input scale ``exp(i - m_t)``; with those the memory is the Mamba-2 recurrence with a per-token
decay and step, and n is one more column of it (a value that is always 1), so S and n run on the framework's ragged scan kernel
(``ops.mamba2_scan(gates=...)``, csrc/kernels/mamba.cu: v -> x with the ones column, k -> B, q -> C): one launch for prompt portions,
decode tokens and mixed batches, state read and written once per call, token order fixed.  ``ops.mlstm_readout`` divides, norms and gates.
Gate pre-activations are a true fp32 product (they enter the recurrence); q / k / v / g come from one GEMM in the model dtype.  The state
lives in a ``LayeredStatePool`` entry per request slot: fp32 ``[heads, dim, vdim + 1]`` (S | n) and ``aux`` ``[heads]`` (m).
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..model_executor.forward_batch import ForwardBatch


class MLSTMMixer(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float, dtype):
        super().__init__()
        self.H, self.D, self.Dv, self.eps, self.cap = heads, dim, vdim, eps, float(gate_cap or 0.0)
        self.n_k, self.n_v = heads * dim, heads * vdim
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype), requires_grad=False)
        self.in_weight = mk(2 * self.n_k + 2 * self.n_v, width)                  # rows [q | k | v | g]: one GEMM
        self.gate_weight = nn.Parameter(torch.zeros(2 * heads, width, dtype=torch.float32), requires_grad=False)      # rows [i | f], fp32
        self.gate_bias = nn.Parameter(torch.zeros(2 * heads, dtype=torch.float32), requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(self.n_v, dtype=dtype), requires_grad=False)
        self.o_weight = mk(width, self.n_v)

    # ---- geometry for the recurrent-state pool: (conv channels, taps, heads, state rows, state columns, aux numbers)
    def state_geometry(self):
        return (0, 1, self.H, self.D, self.Dv + 1, self.H)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        a, b, c = self.n_k, 2 * self.n_k, 2 * self.n_k + self.n_v
        rows = {"q": (0, a), "k": (a, b), "v": (b, c), "g": (c, c + self.n_v)}
        H = self.H
        if leaf in rows:
            self.in_weight.data[rows[leaf][0]:rows[leaf][1]].copy_(w)
        elif leaf in ("i", "f"):
            self.gate_weight.data[(0 if leaf == "i" else H):(H if leaf == "i" else 2 * H)].copy_(w.float())
        elif leaf in ("i.b", "f.b"):
            self.gate_bias.data[(0 if leaf == "i.b" else H):(H if leaf == "i.b" else 2 * H)].copy_(w.float())
        elif leaf == "norm":
            self.norm_weight.data.copy_(w)
        elif leaf == "o":
            self.o_weight.data.copy_(w)
        else:
            return False
        return True

    def forward(self, h: torch.Tensor, fb: ForwardBatch, state_idx: int) -> torch.Tensor:
        proj = ops.linear(h, self.in_weight)
        raw = torch.nn.functional.linear(h.float(), self.gate_weight, self.gate_bias)          # fp32 product on the (possibly bf16-rounded) input
        pool = fb.kv_pool.mamba
        u, gates = ops.mlstm_prepare(proj, raw, self.H, self.D, self.Dv, self.cap, pool.aux[state_idx], fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens)
        y = ops.mamba2_scan(u, None, None, None, None, None, pool.ssm[state_idx], fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens,
                            self.H, self.Dv + 1, self.D, self.H, gates=gates)
        n = 2 * self.n_k + self.n_v
        o = ops.mlstm_readout(y, gates, self.H, self.Dv, self.norm_weight, self.eps, proj[:, n:n + self.n_v], proj.dtype)
        return ops.linear(o, self.o_weight)
