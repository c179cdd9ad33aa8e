"""Grouped-query attention with an output gate, whose other parts are switched on by its arguments:

    q, k, v, g = W h (+ b)                        one GEMM, rows [q | k | v | g]
    q, k       <- rms(q) * w_q, rms(k) * w_k      ``qk_norm``: over the WHOLE projection (all heads at once), plain weights
    q, k       <- rotation by position            ``rotary = (dims, inv_freq)``: the first ``dims`` coordinates of every head, coordinate i paired
                                                  with i + dims/2, angle = position * inv_freq[i] (fp32)
    v          <- (1 - lam) v + lam v_first       ``value_mix``: v_first = the values of the first such layer for the same token; the blend is cached
    v_j        <- v_j turned by position j        ``value_rotary = (inv_freq, interleaved)``: over the whole head, cached so; o_i is turned back by
                                                  position i behind the soft-max, so that a value enters by its distance to the query
    s_ij       = q_i . k_j * scale - r1_h ln(1 + r2_h (i - j))            ``log_bias``
    s_ij       <- cap tanh(s_ij / cap)                                      ``softcap``
    visible    j <= i and (i - j < window or j < keep_first)               (no window: every j <= i)
    p_ij       = exp(s_ij) / (sum_j' exp(s_ij') + exp(sink_h))             ``sinks``: a key without a value per head (stored zero: one more in the denominator)
    o_i        = p_i v  *  sigmoid(g_i)                                     ``gate = "head"``: one number per head; ``"element"``: one per coordinate; None: no gate
    y          = W_o o (+ b_o)

``ops.attention_prepare`` does the second to fourth line and the cache write in one kernel; ``ops.window_attention`` the scores, mask,
soft-max, value product and the gate (csrc/kernels/window_attention.cu), for prompt portions and decode tokens alike.  Scores, bias,
soft-max, norms, angles and the gate are fp32; q and the cache are in the model dtype.  bf16 models with key / value heads at most 128
wide and a group size that divides 128 run the framework's tcgen05 attention kernels (``ops.paged_attention``: window, kept first tokens
the logarithmic bias and the score cap are arguments of those kernels; a sink enters through their log-sum-exp) on heads laid out 128
columns wide (``pad``; see ``layers/window_attention.py``), followed by one pass for the sink, the back-rotation and the gate.

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
                 log_bias: bool = False, gate: Optional[str] = "head", value_mix: bool = False, own_projection: bool = True, softcap: float = 0.0,
                 sinks: bool = False, value_rotary: Optional[Tuple[torch.Tensor, bool]] = None):
        super().__init__()
        assert heads % kv_heads == 0 and gate in ("head", "element", None)
        self.H, self.G, self.D, self.Dv, self.eps = heads, kv_heads, dim, vdim, eps
        f32z = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.float32), requires_grad=False)
        self.scale = float(scale) if scale is not None else dim ** -0.5
        self.window, self.keep_first = int(window or -1), int(keep_first or 0)
        self.gate_kind, self.value_mix = gate, value_mix
        self.n_q, self.n_k, self.n_v = heads * dim, kv_heads * dim, kv_heads * vdim
        self.n_g = 0 if gate is None else heads if gate == "head" else heads * vdim
        self.softcap = float(softcap or 0.0)
        self.sinks = f32z(heads) if sinks else None
        if value_rotary is not None:
            assert vdim % 2 == 0 and value_rotary[0].numel() == vdim // 2, "values rotate over their whole (even) width"
        self.v_inv_freq = nn.Parameter(value_rotary[0].float().clone(), requires_grad=False) if value_rotary is not None else None
        self.v_interleaved = bool(value_rotary[1]) if value_rotary is not None else False
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
        rows = {"q": (0, a), "k": (a, b), "v": (b, c)}
        if self.n_g:
            rows["g"] = (c, self.rows)
        return rows

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
        name = {"o": "o_weight", "o.b": "o_bias", "q.norm": "q_norm", "k.norm": "k_norm", "r1": "r1", "r2": "r2", "sink": "sinks"}.get(leaf)
        if leaf == "vmix" and self.value_mix:
            self.vmix = float(w.float().reshape(()))
            return True
        if name is None or getattr(self, name) is None:
            return False
        p = getattr(self, name)
        p.data.copy_(w.to(p.dtype).reshape(p.shape))
        return True

    # ---- forward
    def forward(self, h: torch.Tensor, fb: ForwardBatch, cache_idx: int, v_first: Optional[torch.Tensor] = None, planes=None):
        return self.forward_projected(ops.linear(h, self.in_weight, self.in_bias), fb, cache_idx, v_first, planes)

    def values_of(self, proj: torch.Tensor) -> torch.Tensor:
        """the v columns of this mixer's projection (what a later value-mixing layer blends with)"""
        a = self.n_q + self.n_k
        return proj[:, a:a + self.n_v]

    def attend(self, proj: torch.Tensor, fb: ForwardBatch, cache_idx: int, v_first: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None, planes=None) -> torch.Tensor:
        """projection rows [q | k | v | g] -> gated heads [T, H * Dv] (times ``out_scale``), before the output projection"""
        T = proj.shape[0]
        H, G, D, Dv = self.H, self.G, self.D, self.Dv
        kc, vc = planes if planes is not None else (fb.kv_pool.k(cache_idx), fb.kv_pool.v(cache_idx))      # [slots, 1, cache_width] each
        pad = self.pad
        q = ops.attention_prepare(proj, H, G, D, Dv, fb.positions, kc, vc, fb.out_cache_loc, self.q_norm, self.k_norm, self.eps, self.inv_freq,
                                  v_first if self.value_mix else None, self.vmix, pad, self.v_inv_freq, self.v_interleaved)
        gate = proj[:, self.rows - self.n_g:self.rows] if self.n_g else None
        turn = self.v_inv_freq is not None
        # where the back-rotation may write the caller's buffer directly: nothing follows it
        direct = out if turn and gate is None and self.out_scale == 1.0 and out is not None and out.is_contiguous() else None
        if self.tc_route and pad == 128 and kc.shape[-1] >= G * 128:
            k4, v4 = kc[:, 0, :G * 128].unflatten(-1, (G, 128)), vc[:, 0, :G * 128].unflatten(-1, (G, 128))      # the leading columns of the pool's rows
            if ops.tc_attention_ok(q, k4, v4, fb.page_size):
                dec = fb.cu_q is None
                lse = torch.empty(T, H, dtype=torch.float32, device=q.device) if self.sinks is not None else None
                o = ops.paged_attention(q, k4, v4, fb.page_table, fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens, fb.max_q_len, fb.page_size, self.scale,
                                        causal=True, window=self.window, logit_cap=self.softcap, num_splits=fb.num_splits if dec else 1,
                                        workspace=fb.attn_workspace if dec else None, lse=lse, slopes=self.r1, log_rates=self.r2, keep_first=self.keep_first)
                if turn:             # the sink's share, the back-rotation and the end of the head padding in one pass
                    o = ops.rotate_heads(o, fb.positions, self.v_inv_freq, Dv, self.v_interleaved, True, lse, self.sinks, direct)
                    if direct is not None:
                        return o
                    o = o.view(T, H, Dv)
                elif lse is not None:
                    o = ops.attention_sink_gate(o, lse, self.sinks, Dv)
                if gate is None:
                    return self._plain(o, Dv, out)
                return ops.sigmoid_gate(o, gate, Dv, self.out_scale, out)
        o = ops.window_attention(q, kc, vc, G, Dv, fb.page_table, fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens, fb.max_q_len, fb.page_size,
                                 self.scale, self.softcap, self.window, self.r1, self.sinks, D, pad, self.keep_first, self.r2, None if turn else gate,
                                 1.0 if turn else self.out_scale, None if turn else out)
        if not turn:
            return o.reshape(T, H * Dv)
        o = ops.rotate_heads(o.reshape(T, H, Dv), fb.positions, self.v_inv_freq, Dv, self.v_interleaved, True, None, None, direct)
        if direct is not None:
            return o
        if gate is None:
            return self._plain(o.view(T, H, Dv), Dv, out)
        return ops.sigmoid_gate(o.view(T, H, Dv), gate, Dv, self.out_scale, out)

    def _plain(self, o: torch.Tensor, Dv: int, out: Optional[torch.Tensor]) -> torch.Tensor:
        """ungated heads [T, H, >= Dv] -> [T, H * Dv] (times ``out_scale``), into ``out`` when given"""
        T, H = o.shape[0], o.shape[1]
        y = o[:, :, :Dv].reshape(T, H * Dv)
        if self.out_scale != 1.0:
            y = (y.float() * self.out_scale).to(o.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def forward_projected(self, proj: torch.Tensor, fb: ForwardBatch, cache_idx: int, v_first: Optional[torch.Tensor] = None, planes=None) -> torch.Tensor:
        return ops.linear(self.attend(proj, fb, cache_idx, v_first, planes=planes), self.o_weight, self.o_bias)
