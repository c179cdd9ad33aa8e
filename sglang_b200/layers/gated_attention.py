"""Grouped-query attention with an output gate, whose other parts are switched on by its arguments:

    q, k, v, g = W h (+ b)                        one GEMM, rows [q | k | v | g]
    q, k       <- rms(q) * w_q, rms(k) * w_k      ``qk_norm``: over the WHOLE projection (all heads at once), plain weights
    q, k       <- rotation by position            ``rotary = (dims, inv_freq)``: the first ``dims`` coordinates of every head, coordinate i paired
                                                  with i + dims/2, angle = position * inv_freq[i] (fp32)
    v          <- (1 - lam) v + lam v_first       ``value_mix``: v_first = the values of the first such layer for the same token; the blend is cached
    s_ij       = q_i . k_j * scale - r1_h ln(1 + r2_h (i - j))            ``log_bias``
    visible    j <= i and (i - j < window or j < keep_first)               (no window: every j <= i)
    o_i        = soft-max(s_i) v  *  sigmoid(g_i)                           ``gate = "head"``: one number per head; ``"element"``: one per coordinate
    y          = W_o o (+ b_o)

``ops.attention_prepare`` does the second to fourth line and the cache write in one kernel; ``ops.window_attention`` the scores, mask,
soft-max, value product and the gate (csrc/kernels/window_attention.cu), for prompt portions and decode tokens alike.  Scores, bias,
soft-max, norms, angles and the gate are fp32; q and the cache are in the model dtype.  bf16 models with key / value heads at most 128
wide and a group size that divides 128 run the framework's tcgen05 attention kernels (``ops.paged_attention``: window, kept first tokens
and the logarithmic bias are arguments of those kernels) on heads laid out 128 columns wide (``pad``; see ``layers/window_attention.py``),
followed by the gate.

The paged pool holds one flat row per token and plane (``FlatCacheSpec`` of ``layers/window_attention.py``); ``cache_idx`` selects the pool
layer.  The window only masks: pages behind it stay with the request until it ends.

The projection may belong to a parent that feeds several mixers from one GEMM: ``in_rows`` / ``load_in`` describe and fill this mixer's rows
of any weight tensor, and ``forward_projected`` starts from the GEMM's output.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..model_executor.forward_batch import ForwardBatch


def scaled_inv_freq(dims: int, base: float, scaling: Optional[dict] = None) -> torch.Tensor:
    """rotary frequencies ``base^(-2i/dims)``, i < dims/2, fp32.  ``scaling = {factor, low, high, original}``: by wavelength ``l = 2 pi / f``,
    short waves (``l < original / high``) keep f, long waves (``l > original / low``) use ``f / factor``, and between the two the blend
    ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``"""
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        factor, low, high, orig = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"]), float(scaling["original"])
        out = []
        for fi in f:
            wl = 2.0 * math.pi / fi
            if wl < orig / high:
                out.append(fi)
            elif wl > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wl - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=torch.float64).float()


class GatedAttention(nn.Module):
    tc_route = True            # class-wide switch of the tcgen05 route (tests compare it with the general kernel)

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: Optional[float], eps: float, dtype, *, bias: bool = False,
                 qk_norm: bool = False, rotary: Optional[Tuple[int, torch.Tensor]] = None, window: int = -1, keep_first: int = 0,
                 log_bias: bool = False, gate: str = "head", value_mix: bool = False, own_projection: bool = True):
        super().__init__()
        assert heads % kv_heads == 0 and gate in ("head", "element")
        self.H, self.G, self.D, self.Dv, self.eps = heads, kv_heads, dim, vdim, eps
        self.scale = float(scale) if scale is not None else dim ** -0.5
        self.window, self.keep_first = int(window or -1), int(keep_first or 0)
        self.gate_kind, self.value_mix = gate, value_mix
        self.n_q, self.n_k, self.n_v = heads * dim, kv_heads * dim, kv_heads * vdim
        self.n_g = heads if gate == "head" else heads * vdim
        self.rows = self.n_q + self.n_k + self.n_v + self.n_g
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.float32), requires_grad=False)
        self.has_bias = bias
        self.in_weight = mk(self.rows, width) if own_projection else None
        self.in_bias = mk(self.rows) if own_projection and bias else None
        self.o_weight = mk(width, heads * vdim)
        self.o_bias = mk(width) if bias else None
        self.q_norm = mk(self.n_q) if qk_norm else None
        self.k_norm = mk(self.n_k) if qk_norm else None
        self.r1, self.r2 = (f32(heads), f32(heads)) if log_bias else (None, None)
        self.rot_dims = int(rotary[0]) if rotary else 0
        assert self.rot_dims % 2 == 0 and self.rot_dims <= dim
        self.inv_freq = nn.Parameter(rotary[1].float().clone(), requires_grad=False) if rotary else None
        self.vmix = 0.0              # lam (read when this layer is not the first value-mixing one)
        self.pad = 0                 # 128: heads laid out 128 columns wide for the tcgen05 kernels (the model decides, see ``wants_padding``)
        self.out_scale = 1.0         # folded into the gate epilogue (a parent that sums several mixers sets it)

    # ---- cache geometry
    def wants_padding(self, dtype) -> bool:
        """whether this layer would run the tcgen05 kernels if its pool rows are ``kv_heads * 128`` wide"""
        return bool(self.tc_route and dtype == torch.bfloat16 and self.D <= 128 and self.Dv <= 128 and 128 % (self.H // self.G) == 0)

    @property
    def cache_width(self) -> int:
        return self.G * (self.pad if self.pad else max(self.D, self.Dv))

    # ---- weights
    def in_rows(self) -> dict:
        a, b, c = self.n_q, self.n_q + self.n_k, self.n_q + self.n_k + self.n_v
        return {"q": (0, a), "k": (a, b), "v": (b, c), "g": (c, self.rows)}

    def load_in(self, leaf: str, w: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], offset: int = 0) -> bool:
        """a projection's tensor (``q``, ``k.b`` ...) into this mixer's rows of ``weight`` / ``bias``, which start at ``offset``"""
        rows = self.in_rows()
        if leaf in rows:
            a, b = rows[leaf]
            weight.data[offset + a:offset + b].copy_(w)
            return True
        if leaf.endswith(".b") and leaf[:-2] in rows and bias is not None:
            a, b = rows[leaf[:-2]]
            bias.data[offset + a:offset + b].copy_(w)
            return True
        return False

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if self.in_weight is not None and self.load_in(leaf, w, self.in_weight, self.in_bias):
            return True
        name = {"o": "o_weight", "o.b": "o_bias", "q.norm": "q_norm", "k.norm": "k_norm", "r1": "r1", "r2": "r2"}.get(leaf)
        if leaf == "vmix" and self.value_mix:
            self.vmix = float(w.float().reshape(()))
            return True
        if name is None or getattr(self, name) is None:
            return False
        p = getattr(self, name)
        p.data.copy_(w.to(p.dtype).reshape(p.shape))
        return True

    # ---- forward
    def forward(self, h: torch.Tensor, fb: ForwardBatch, cache_idx: int, v_first: Optional[torch.Tensor] = None):
        return self.forward_projected(ops.linear(h, self.in_weight, self.in_bias), fb, cache_idx, v_first)

    def values_of(self, proj: torch.Tensor) -> torch.Tensor:
        """the v columns of this mixer's projection (what a later value-mixing layer blends with)"""
        a = self.n_q + self.n_k
        return proj[:, a:a + self.n_v]

    def attend(self, proj: torch.Tensor, fb: ForwardBatch, cache_idx: int, v_first: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """projection rows [q | k | v | g] -> gated heads [T, H * Dv] (times ``out_scale``), before the output projection"""
        T = proj.shape[0]
        H, G, D, Dv = self.H, self.G, self.D, self.Dv
        kc, vc = fb.kv_pool.k(cache_idx), fb.kv_pool.v(cache_idx)                  # [slots, 1, cache_width] each
        pad = self.pad
        q = ops.attention_prepare(proj, H, G, D, Dv, fb.positions, kc, vc, fb.out_cache_loc, self.q_norm, self.k_norm, self.eps, self.inv_freq,
                                  v_first if self.value_mix else None, self.vmix, pad)
        gate = proj[:, self.rows - self.n_g:self.rows]
        if self.tc_route and pad == 128 and kc.shape[-1] >= G * 128:
            k4, v4 = kc[:, 0, :G * 128].unflatten(-1, (G, 128)), vc[:, 0, :G * 128].unflatten(-1, (G, 128))      # the leading columns of the pool's rows
            if ops.tc_attention_ok(q, k4, v4, fb.page_size):
                dec = fb.cu_q is None
                o = ops.paged_attention(q, k4, v4, fb.page_table, fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens, fb.max_q_len, fb.page_size, self.scale,
                                        causal=True, window=self.window, num_splits=fb.num_splits if dec else 1, workspace=fb.attn_workspace if dec else None,
                                        slopes=self.r1, log_rates=self.r2, keep_first=self.keep_first)
                return ops.sigmoid_gate(o, gate, Dv, self.out_scale, out)
        return ops.window_attention(q, kc, vc, G, Dv, fb.page_table, fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens, fb.max_q_len, fb.page_size,
                                    self.scale, 0.0, self.window, self.r1, None, D, pad, self.keep_first, self.r2, gate, self.out_scale,
                                    out).reshape(T, H * Dv)

    def forward_projected(self, proj: torch.Tensor, fb: ForwardBatch, cache_idx: int, v_first: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.linear(self.attend(proj, fb, cache_idx, v_first), self.o_weight, self.o_bias)
