"""Linear attention with a constant decay per head ("lightning attention"): on SiLU-activated projections,

    S_t = decay_h S_(t-1) + k_t v_t^T            S: [dim, vdim] per head, fp32, zero at the start of a sequence
    o_t = S_t^T q_t                               (no other scale)

then the heads' outputs together pass one RMS norm with a weight, times ``sigmoid(g_t)``, and the output projection.

The recurrence is the Mamba-2 one with step size 1 and a constant decay, so it runs on the same ragged kernel (``ops.mamba2_scan(decay=...)``,
csrc/kernels/mamba.cu) with v in the place of x, k of B and q of C: one launch for prompt portions, decode tokens and mixed batches, state read
and written once per call, token order fixed (a position's result does not depend on how its prompt was cut).  The state lives in a
``LayeredStatePool`` entry (``state_idx``) per request slot; there is no convolution.  The projection is one GEMM with rows
``[v | k | q | g]``, so that one activation pass over its first columns yields the scan's input; the gated norm is one kernel
(``ops.grouped_rmsnorm(gate=...)``).

The projection may belong to a parent that feeds several mixers from one GEMM (``in_rows`` / ``load_in`` / ``forward_projected``).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
from torch import nn

from .. import ops
from ..model_executor.forward_batch import ForwardBatch


class DecayLinearAttention(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float, dtype, own_projection: bool = True):
        super().__init__()
        assert len(decay) == heads, "one decay per head"
        self.H, self.D, self.Dv, self.eps = heads, dim, vdim, eps
        self.n_v, self.n_k = heads * vdim, heads * dim
        self.rows = 2 * self.n_v + 2 * self.n_k
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype), requires_grad=False)
        self.in_weight = mk(self.rows, width) if own_projection else None
        self.norm_weight = nn.Parameter(torch.ones(self.n_v, dtype=dtype), requires_grad=False)
        self.o_weight = mk(width, self.n_v)
        self.decay = nn.Parameter(torch.tensor([float(d) for d in decay], dtype=torch.float64).float(), requires_grad=False)
        self.out_scale = 1.0         # folded into the gated norm (a parent that sums several mixers sets it)

    # ---- geometry for the recurrent-state pool: (conv channels, taps, heads, state rows, head_dim): no convolution
    def state_geometry(self):
        return (0, 1, self.H, self.D, self.Dv)

    def in_rows(self) -> dict:
        a, b, c = self.n_v, self.n_v + self.n_k, self.n_v + 2 * self.n_k
        return {"v": (0, a), "k": (a, b), "q": (b, c), "g": (c, self.rows)}

    def load_in(self, leaf: str, w: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], offset: int = 0) -> bool:
        rows = self.in_rows()
        if leaf not in rows:
            return False
        a, b = rows[leaf]
        weight.data[offset + a:offset + b].copy_(w)
        return True

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if self.in_weight is not None and self.load_in(leaf, w, self.in_weight, None):
            return True
        name = {"o": "o_weight", "norm": "norm_weight"}.get(leaf)
        if name is None:
            return False
        getattr(self, name).data.copy_(w)
        return True

    def forward(self, h: torch.Tensor, fb: ForwardBatch, state_idx: int) -> torch.Tensor:
        return self.forward_projected(ops.linear(h, self.in_weight), fb, state_idx)

    def attend(self, proj: torch.Tensor, fb: ForwardBatch, state_idx: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """projection rows [v | k | q | g] -> normed, gated heads [T, H * vdim] (times ``out_scale``), before the output projection"""
        n = self.n_v + 2 * self.n_k
        u = ops.activation(proj[:, :n], "silu", torch.float32)                   # [silu(v) | silu(k) | silu(q)] fp32: the scan's [x | B | C]
        o = ops.mamba2_scan(u, None, None, None, None, None, fb.kv_pool.mamba.ssm[state_idx], fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens,
                            self.H, self.Dv, self.D, self.H, decay=self.decay)
        return ops.grouped_rmsnorm(o, self.norm_weight, 1, self.eps, proj.dtype, proj[:, n:n + self.n_v], self.out_scale, out)

    def forward_projected(self, proj: torch.Tensor, fb: ForwardBatch, state_idx: int) -> torch.Tensor:
        return ops.linear(self.attend(proj, fb, state_idx), self.o_weight)
