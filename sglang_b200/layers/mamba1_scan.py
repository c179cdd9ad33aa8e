"""Mamba-1 mixer (selective scan) on the ragged recurrent kernels: one projection ``[x | z]``, a short causal convolution (+ bias, SiLU) over
x, a low-rank projection ``[dt | B | C]`` of the result, the step size ``dt = softplus(W_dt dt + b)`` per channel, and per channel c and
state n the recurrence

    S_t[c, n] = exp(dt_t[c] A[c, n]) S_(t-1)[c, n] + dt_t[c] x_t[c] B_t[n]          A = -exp(A_log), S fp32
    y_t[c]    = sum_n S_t[c, n] C_t[n] + D[c] x_t[c]

then ``y * silu(z)`` and the output projection.

The framework's other Mamba-1 path (``models/mamba.py`` ``Mamba1Mixer``) scans prompts with a chunked PyTorch formulation and updates decode
tokens with tensor expressions.  This mixer serves prompt portions, single decode tokens and mixed batches with the same two kernels
(``ops.causal_conv1d`` and ``ops.mamba1_scan``, csrc/kernels/mamba.cu) and takes the convolution history and the state from a
``LayeredStatePool`` entry per request slot, addressed by ``state_idx``.  Step size, decay, state, skip and gate are fp32 (the step-size
projection returns fp32); the other projections and the convolution inputs are in the model dtype.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..model_executor.forward_batch import ForwardBatch


class Mamba1ScanMixer(nn.Module):
    def __init__(self, width: int, inner: int, state: int, dt_rank: int, taps: int, dtype, conv_bias: bool = True):
        super().__init__()
        self.inner, self.N, self.R, self.taps = inner, state, dt_rank, taps
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.float32), requires_grad=False)
        self.in_weight = mk(2 * inner, width)                       # rows [x | z]
        self.conv_weight = mk(inner, taps)
        self.conv_bias = mk(inner) if conv_bias else None
        self.x_weight = mk(dt_rank + 2 * state, inner)              # rows [dt | B | C]
        self.dt_weight = mk(inner, dt_rank)
        self.dt_bias, self.A_log, self.D = f32(inner), f32(inner, state), f32(inner)
        self.o_weight = mk(width, inner)
        self._dt32 = None

    # ---- geometry for the recurrent-state pool: (conv channels, taps, heads, state rows, head_dim) -> state [slots, 1, inner, state]
    def state_geometry(self):
        return (self.inner, self.taps, 1, self.inner, self.N)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        name = {"in": "in_weight", "conv": "conv_weight", "conv.b": "conv_bias", "x": "x_weight", "dt": "dt_weight", "dt.b": "dt_bias", "A_log": "A_log",
                "D": "D", "o": "o_weight"}.get(leaf)
        if name is None or getattr(self, name) is None:
            return False
        p = getattr(self, name)
        p.data.copy_(w.to(p.dtype).reshape(p.shape))
        self._dt32 = None
        return True

    def forward(self, h: torch.Tensor, fb: ForwardBatch, state_idx: int) -> torch.Tensor:
        pool = fb.kv_pool.mamba
        inner, R, N = self.inner, self.R, self.N
        proj = ops.linear(h, self.in_weight)                                     # [T, x | z]
        xin = proj[:, :inner]
        if self.taps > 1:
            u = ops.causal_conv1d(xin, self.conv_weight, self.conv_bias, pool.conv[state_idx], fb.cu_q, fb.req_slots, fb.seq_lens, fb.max_q_len, silu=True)
        else:
            a = xin.float() * self.conv_weight[:, 0].float()
            u = torch.nn.functional.silu(a + self.conv_bias.float() if self.conv_bias is not None else a).contiguous()
        low = ops.linear(u.to(h.dtype) if h.dtype != torch.float32 else u, self.x_weight)          # [T, dt | B | C]
        # the step size enters the recurrence: its (rank-R) projection accumulates and returns fp32
        if self._dt32 is None or self._dt32.device != h.device:
            self._dt32 = self.dt_weight.detach().float()
        dt_raw = torch.nn.functional.linear(low[:, :R].float(), self._dt32)
        y = ops.mamba1_scan(u, dt_raw, self.dt_bias, self.A_log, low[:, R:R + N], low[:, R + N:R + 2 * N], self.D, proj[:, inner:], pool.ssm[state_idx],
                            fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens, h.dtype)
        return ops.linear(y, self.o_weight)
