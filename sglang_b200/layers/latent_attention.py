"""Latent (low-rank KV) attention without positional rotation, with a sliding window and per-head soft-max sinks.

Every token caches ONE latent row ``c = rmsnorm(W_dkv h)`` of ``kv_rank`` numbers; keys and values of all heads are linear maps of it
(``k_h = W_uk,h c``, ``v_h = W_uv,h c``).  Attention runs in the absorbed form, like the framework's other latent-attention family
(``models/deepseek.py``): the key up-projection moves to the query side and the value up-projection behind the soft-max,

    q~_h = W_uk,h^T q_h                      [kv_rank]
    p_hij = softmax_j(scale * q~_hi . c_j)   over the window  0 <= i - j < window, with exp(sink_h) added to the denominator
    o_hi  = W_uv,h (sum_j p_hij c_j)

so the paged cache holds ``kv_rank`` values per token and layer and the kernel is multi-query attention over the latent rows
(``ops.latent_attention``, csrc/kernels/latent_attention.cu: one kernel for prompt portions and single decode tokens).  The soft-max, the
latent norm and both absorbed products are fp32; the cache is in the model dtype.

Prompt portions of bf16 models whose key and value heads are both 128 wide take the expanded route instead: the latent rows a portion can
see (its own tokens and the window before them) are gathered once per forward, up-projected to per-head keys and values by one GEMM each
into a scratch paged buffer, and the framework's tcgen05 flash-attention kernel runs over them with the same window; the sink enters
through the log-sum-exp (``o * sigmoid(lse - sink)``).  Per (query, key, head) that costs ``dim + vdim`` multiply-adds on tensor cores
instead of ``2 * kv_rank`` on CUDA cores.  Decode, fp32 serving and every other head size stay on the absorbed kernel.

The window only masks: pages of tokens that left the window are still held until the request ends (the pool is sized by live tokens).

``RotaryLatentAttention`` is the positional form: queries pass a normed latent of their own, every head has ``dim`` unrotated and
``rot_dim`` rotary query / key coordinates, and ONE rotary key part per token is shared by all heads.  The cache row is
``[c (kv_rank) | rotary key (rot_dim)]``; in the absorbed form the query is ``[W_uk,h^T q_h | rotary part]`` and the same kernel scores over
the whole row while only its first ``kv_rank`` columns are values (``ops.latent_attention(v_rank=...)``).  Large prompt portions take the
expanded form over up-projected rows: on the general attention kernel (keys up to 256 wide, fp32 and bf16), or, for long bf16 portions, as
Q K^T and P V on the tensor cores (vendor batched GEMMs, fp32 scores) around ``ops.causal_softmax``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch
from torch import nn

from .. import ops
from ..model_executor.forward_batch import ForwardBatch


class LatentCacheSpec:
    """what the model runner reads to size the paged pool: one "KV head" of ``cache_width`` per token, a single plane (values are a view)"""

    def __init__(self, num_heads: int, cache_width: int, layer_id: int, scale: float, window: int):
        self.num_heads, self.num_kv_heads, self.head_dim, self.kv_head_dim = num_heads, 1, cache_width, cache_width
        self.latent_v_dim = cache_width
        self.layer_id, self.scale, self.window, self.logit_cap, self.rope, self.sinks = layer_id, scale, window, 0.0, None, None


def expand_plan(fb: ForwardBatch, window: int, page: int):
    """which cached rows this forward's prompt portions can see, laid out as a scratch paged buffer of ``page``-token pages (built once per
    forward and window on the host from the lengths the scheduler already holds; shared by all layers with that window)"""
    plans = fb.__dict__.setdefault("_latent_expand", {})
    W = window
    if (W, page) in plans:
        return plans[(W, page)]
    ps, P = fb.page_size, page
    sl, ql, slots = np.asarray(fb.seq_lens_cpu, dtype=np.int64), np.asarray(fb.q_lens_cpu, dtype=np.int64), fb.req_slots
    lo = np.maximum(0, sl - ql - W + 1) if W > 0 else np.zeros_like(sl)
    n = sl - lo
    pages = (n + P - 1) // P
    first = np.concatenate([[0], np.cumsum(pages)[:-1]]) + 1                      # (page 0 stays unused, like in the real pool)
    B = len(sl)
    pt = np.zeros((B, int(pages.max())), dtype=np.int32)
    req = np.repeat(np.arange(B), n)
    rel = np.concatenate([np.arange(k) for k in n])
    for b in range(B):
        pt[b, : pages[b]] = first[b] + np.arange(pages[b])
    dev = fb.seq_lens.device
    to = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(dev, non_blocking=True).to(dt)
    pos = to(lo[req] + rel, torch.int64)
    reqd = to(req, torch.int64)
    src = fb.page_table[slots.long()[reqd], pos // ps].long() * ps + pos % ps           # rows of the latent cache
    dst = to((first[req] * P + rel), torch.int64)                                       # rows of the scratch buffer
    plan = {"src": src, "dst": dst, "rows": int((first[-1] + pages[-1]) * P), "pt": to(pt, torch.int32), "n": to(n, torch.int32),
            "slots": torch.arange(B, dtype=torch.int32, device=dev), "max_n": int(n.max()), "total": int(n.sum()), "first_rows": first * P, "n_cpu": n,
            "lo_cpu": lo}
    plans[(W, page)] = plan
    return plan


class WindowedLatentAttention(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, vdim: int, kv_rank: int, scale: Optional[float], window: int, eps: float, layer_id: int,
                 dtype, cache_width: Optional[int] = None, sinks: bool = True):
        super().__init__()
        self.H, self.D, self.Dv, self.R = heads, dim, vdim, kv_rank
        self.eps = eps
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype), requires_grad=False)
        self.qc_weight = mk(heads * dim + kv_rank, width)          # rows [q (heads x dim) | latent down-projection (kv_rank)]: one GEMM
        self.latent_norm = nn.Parameter(torch.ones(kv_rank, dtype=dtype), requires_grad=False)
        self.uk = mk(heads * dim, kv_rank)
        self.uv = mk(heads * vdim, kv_rank)
        self.o_weight = mk(width, heads * vdim)
        self.sinks = nn.Parameter(torch.zeros(heads, dtype=torch.float32), requires_grad=False) if sinks else None
        self.attn = LatentCacheSpec(heads, cache_width or kv_rank, layer_id, float(scale) if scale is not None else dim ** -0.5, int(window or -1))
        self._uk32 = self._uv32 = None

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        hd = self.H * self.D
        if leaf == "q":
            self.qc_weight.data[:hd].copy_(w)
        elif leaf == "dkv":
            self.qc_weight.data[hd:].copy_(w)
        elif leaf == "dkv.norm":
            self.latent_norm.data.copy_(w)
        elif leaf in ("uk", "uv"):
            getattr(self, leaf).data.copy_(w)
            self._uk32 = self._uv32 = None
        elif leaf == "sink":
            self.sinks.data.copy_(w.float())
        elif leaf == "o":
            self.o_weight.data.copy_(w)
        else:
            return False
        return True

    def _absorbed(self):
        if self._uk32 is None or self._uk32.device != self.uk.device:
            self._uk32 = self.uk.detach().float().view(self.H, self.D, self.R).contiguous()                   # [H, D, R]
            self._uv32 = self.uv.detach().float().view(self.H, self.Dv, self.R).transpose(1, 2).contiguous()  # [H, R, Dv]
        return self._uk32, self._uv32

    EXPAND_PAGE = 64
    expand_prefill = True            # class-wide switch of the expanded prompt route (tests compare it with the absorbed kernel)

    def _expand_plan(self, fb: ForwardBatch):
        return expand_plan(fb, self.attn.window, self.EXPAND_PAGE)

    def _forward_expanded(self, q: torch.Tensor, cache: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        T, H, D = q.shape[0], self.H, self.D
        pl = self._expand_plan(fb)
        c = cache[pl["src"], 0, : self.R]                                                   # [N, R] visible latent rows
        kbuf = torch.zeros(pl["rows"], H, D, dtype=q.dtype, device=q.device)
        vbuf = torch.zeros(pl["rows"], H, self.Dv, dtype=q.dtype, device=q.device)
        kbuf[pl["dst"]] = ops.linear(c, self.uk).view(-1, H, D)
        vbuf[pl["dst"]] = ops.linear(c, self.uv).view(-1, H, self.Dv)
        lse = torch.empty(T, H, dtype=torch.float32, device=q.device) if self.sinks is not None else None
        o = ops.paged_attention(q.view(T, H, D), kbuf, vbuf, pl["pt"], pl["slots"], pl["n"], fb.cu_q, fb.q_lens, fb.max_q_len, self.EXPAND_PAGE,
                                self.attn.scale, causal=True, window=self.attn.window, lse=lse)
        if lse is not None:
            o = (o.float() * torch.sigmoid(lse - self.sinks[None, :]).unsqueeze(-1)).to(o.dtype)
        return o.reshape(T, H * self.Dv)

    def forward(self, h: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        T = h.shape[0]
        hd = self.H * self.D
        qc = ops.linear(h, self.qc_weight)
        c = ops.rmsnorm(qc[:, hd:].contiguous(), self.latent_norm, self.eps)
        cache = fb.kv_pool.k(self.attn.layer_id)                          # [slots, 1, cache_width]
        cache[fb.out_cache_loc.long(), 0, : self.R] = c.to(cache.dtype)
        if (self.expand_prefill and fb.cu_q is not None and fb.max_q_len > 1 and h.is_cuda and h.dtype == torch.bfloat16 and self.D == 128 and self.Dv == 128
                and fb.q_lens_cpu is not None and ops.native_available() and ops.attn_impl() == 0):
            return ops.linear(self._forward_expanded(qc[:, :hd].contiguous(), cache, fb), self.o_weight)
        uk, uv = self._absorbed()
        q_lat = torch.bmm(qc[:, :hd].float().view(T, self.H, self.D).transpose(0, 1), uk).transpose(0, 1).contiguous()      # [T, H, R]
        o_lat = ops.latent_attention(q_lat, cache, self.R, fb.page_table, fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens, fb.max_q_len, fb.page_size,
                                     self.attn.scale, self.attn.window, self.sinks, fb.max_kv_len)
        o = torch.bmm(o_lat.transpose(0, 1), uv).transpose(0, 1).reshape(T, self.H * self.Dv)
        return ops.linear(o.to(h.dtype), self.o_weight)


def yarn_inv_freq(dims: int, base: float, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, float]:
    """rotary frequencies ``f_i = base^(-2i/dims)``, i < dims/2, with YaRN's blend, and the factor on sine and cosine.

    ``scaling = {factor, original, fast, slow}``: with ``dim(t) = dims ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(dim(fast)), 0)``,
    ``hi = min(ceil(dim(slow)), dims - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency is
    ``f_i / factor * ramp_i + f_i (1 - ramp_i)``, and sine and cosine are multiplied by ``0.1 ln(factor) + 1``.  Without ``scaling``:
    the plain frequencies and 1."""
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    mult = 1.0
    if scaling:
        factor, orig, fast, slow = float(scaling["factor"]), float(scaling["original"]), float(scaling["fast"]), float(scaling["slow"])
        dim_of = lambda t: dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(float(base)))
        lo, hi = max(math.floor(dim_of(fast)), 0), min(math.ceil(dim_of(slow)), dims - 1)
        ramp = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(dims // 2)]
        f = [fi / factor * r + fi * (1.0 - r) for fi, r in zip(f, ramp)]
        mult = 0.1 * math.log(factor) + 1.0
    return torch.tensor(f, dtype=torch.float64).float(), mult


class RotaryLatentAttention(nn.Module):
    """latent attention with a query latent and a decoupled rotary part (neighbouring coordinates paired), causal, ordinary soft-max:

        c_q = rmsnorm(W_dq h) * w_q,   q_h = W_uq,h c_q = [q_h^0 (dim) | q_h^r (rot_dim)]
        [c' | k^r] = W_dkv h,          c = rmsnorm(c') * w_kv  (kv_rank),   k^r (rot_dim) shared by all heads
        s_hij = scale * (q_hi^0 . W_uk,h c_j + rot_i(q_hi^r) . rot_j(k_j^r)),   o_hi = W_uv,h sum_j softmax_j(s_hij) c_j

    ``cache`` is a [slots, 1, >= kv_rank + rot_dim] plane of the paged pool that the model hands in (a latent layer needs one plane)."""

    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int, scale: Optional[float], eps: float, dtype,
                 rotary: Optional[Tuple[torch.Tensor, float]] = None, window: int = -1):
        super().__init__()
        self.H, self.D, self.Dr, self.Dv, self.R, self.Rq = heads, dim, rot_dim, vdim, kv_rank, q_rank
        self.eps, self.window = eps, int(window or -1)
        self.scale = float(scale) if scale is not None else (dim + rot_dim) ** -0.5
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype), requires_grad=False)
        self.down_weight = mk(q_rank + kv_rank + rot_dim, width)       # rows [query latent | key/value latent | rotary key]: one GEMM
        self.q_norm = nn.Parameter(torch.ones(q_rank, dtype=dtype), requires_grad=False)
        self.kv_norm = nn.Parameter(torch.ones(kv_rank, dtype=dtype), requires_grad=False)
        self.uq = mk(heads * (dim + rot_dim), q_rank)
        self.uk = mk(heads * dim, kv_rank)
        self.uv = mk(heads * vdim, kv_rank)
        self.o_weight = mk(width, heads * vdim)
        assert rot_dim % 2 == 0 and (rotary is None or rotary[0].numel() == rot_dim // 2)
        self.inv_freq = nn.Parameter(rotary[0].float().clone(), requires_grad=False) if rotary is not None and rot_dim else None
        self.rot_mult = float(rotary[1]) if rotary is not None else 1.0
        self._uk32 = self._uv32 = None

    @property
    def cache_width(self) -> int:
        return self.R + self.Dr

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "dq":
            self.down_weight.data[:self.Rq].copy_(w)
        elif leaf == "dkv":
            self.down_weight.data[self.Rq:].copy_(w)
        elif leaf == "dq.norm":
            self.q_norm.data.copy_(w)
        elif leaf == "dkv.norm":
            self.kv_norm.data.copy_(w)
        elif leaf in ("uq", "uk", "uv"):
            getattr(self, leaf).data.copy_(w)
            self._uk32 = self._uv32 = None
        elif leaf == "o":
            self.o_weight.data.copy_(w)
        else:
            return False
        return True

    def _absorbed(self):
        if self._uk32 is None or self._uk32.device != self.uk.device:
            self._uk32 = self.uk.detach().float().view(self.H, self.D, self.R).contiguous()                   # [H, D, R]
            self._uv32 = self.uv.detach().float().view(self.H, self.Dv, self.R).transpose(1, 2).contiguous()  # [H, R, Dv]
        return self._uk32, self._uv32

    EXPAND_PAGE = 64
    expand_prefill = True            # class-wide switch of the expanded prompt route (tests compare it with the absorbed kernel)

    def _wants_expanded(self, fb: ForwardBatch, T: int) -> bool:
        """prompt portions that make up a fair share of what they see: per (query, key, head) the expanded form costs ``dim + rot_dim + vdim``
        multiply-adds, the absorbed one ``2 kv_rank + rot_dim``, but it up-projects every visible row first"""
        if not (self.expand_prefill and fb.cu_q is not None and fb.max_q_len > 1 and T >= 64 and fb.q_lens_cpu is not None and fb.seq_lens_cpu is not None
                and self.D + self.Dr <= 256 and self.Dv <= 256 and self.D + self.Dr + self.Dv < 2 * self.R + self.Dr):
            return False
        return int(np.sum(np.asarray(fb.seq_lens_cpu, dtype=np.int64))) <= 16 * T

    def _forward_expanded(self, q: torch.Tensor, cache: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        """the visible cache rows are gathered once, up-projected to per-head keys ``[W_uk,h c | rotary key]`` and values ``W_uv,h c`` in a
        scratch paged buffer (the queries' rotary part turned in place); over them runs the framework's general attention kernel or, for long
        bf16 portions, two batched matrix products around a soft-max kernel (``_attend_by_gemms``)"""
        T, H, D, Dr, R, Dv = q.shape[0], self.H, self.D, self.Dr, self.R, self.Dv
        pl = expand_plan(fb, self.window, self.EXPAND_PAGE)
        rows = cache[pl["src"], 0, : R + Dr]                                                # [N, R + Dr] visible rows
        c = rows[:, :R].contiguous()
        nk, nv = H * (D + Dr), H * Dv
        buf = torch.zeros(pl["rows"], nk + nv, dtype=q.dtype, device=q.device)              # one row = [keys of all heads | values of all heads]
        k = torch.empty(rows.shape[0], H, D + Dr, dtype=q.dtype, device=q.device)
        k[:, :, :D] = ops.linear(c, self.uk).view(-1, H, D)
        k[:, :, D:] = rows[:, None, R:]
        buf[pl["dst"], :nk] = k.view(-1, nk)
        buf[pl["dst"], nk:] = ops.linear(c, self.uv)
        if Dr:
            qr = ops.latent_query(q, torch.empty(H, T, 0, dtype=torch.float32, device=q.device), D, Dr, fb.positions, self.inv_freq, self.rot_mult)
            q = torch.cat([q[:, :, :D], qr.to(q.dtype)], -1)
        q = q.contiguous()
        if self.gemm_prefill and q.is_cuda and q.dtype == torch.bfloat16 and fb.max_q_len >= self.GEMM_MIN_Q and self.window <= 0 and ops.native_available():
            return self._attend_by_gemms(q, buf, nk, pl, fb).reshape(T, H * Dv)
        o = ops.window_attention(q, buf[:, None, :nk], buf[:, None, nk:], H, Dv, pl["pt"], pl["slots"], pl["n"], fb.cu_q, fb.q_lens, fb.max_q_len,
                                 self.EXPAND_PAGE, self.scale, 0.0, self.window, None, None, D + Dr, 0)
        return o.reshape(T, H * Dv)

    GEMM_MIN_Q = 256
    GEMM_SCORE_BYTES = 1 << 28
    gemm_prefill = True              # class-wide switch of the two-product form of the expanded route (tests compare it with the attention kernel)

    def _attend_by_gemms(self, q: torch.Tensor, buf: torch.Tensor, nk: int, pl: dict, fb: ForwardBatch) -> torch.Tensor:
        """long bf16 prompt portions over the up-projected rows as two batched matrix products on the tensor cores around ``ops.causal_softmax``:
        scores = Q K^T with fp32 results, soft-max weights in fp32 rounded to bf16 for the second product, out = P V.  The framework's tcgen05
        attention kernels take 128-wide heads and these keys are ``dim + rot_dim`` wide; the score matrix goes through memory instead, in query
        chunks of at most ``GEMM_SCORE_BYTES``.  Requests are walked on the host (their lengths are the scheduler's)."""
        T, H, Dk = q.shape
        Dv = self.Dv
        out = torch.empty(T, H, Dv, dtype=q.dtype, device=q.device)
        qs = 0
        for b in range(len(pl["n_cpu"])):
            tq, L, r0, n = int(fb.q_lens_cpu[b]), int(fb.seq_lens_cpu[b]), int(pl["first_rows"][b]), int(pl["n_cpu"][b])
            if tq <= 0:
                continue
            rows = buf[r0:r0 + n]
            kb = rows[:, :nk].unflatten(1, (H, Dk)).permute(1, 2, 0)                        # [H, Dk, n] (a view)
            vb = rows[:, nk:].unflatten(1, (H, Dv)).permute(1, 0, 2)                        # [H, n, Dv]
            qb = q[qs:qs + tq].transpose(0, 1)                                              # [H, tq, Dk]
            step = max(16, min(tq, self.GEMM_SCORE_BYTES // (4 * H * max(1, L))))
            for c0 in range(0, tq, step):
                c1 = min(tq, c0 + step)
                kmax = L - tq + c1                                                          # keys the chunk's last query sees
                sc = torch.bmm(qb[:, c0:c1], kb[:, :, :kmax], out_dtype=torch.float32)      # [H, c, kmax] fp32
                pw = ops.causal_softmax(sc.view(H * (c1 - c0), kmax), c1 - c0, L - tq + c0, self.scale, q.dtype)
                out[qs + c0:qs + c1] = torch.bmm(pw.view(H, c1 - c0, kmax), vb[:, :kmax]).transpose(0, 1)
            qs += tq
        return out

    def forward(self, h: torch.Tensor, fb: ForwardBatch, cache: torch.Tensor) -> torch.Tensor:
        T, H, D, Dr, R = h.shape[0], self.H, self.D, self.Dr, self.R
        down = ops.linear(h, self.down_weight)
        cq = ops.latent_prepare(down, self.Rq, self.q_norm, R, Dr, self.kv_norm, self.eps, fb.positions, self.inv_freq, self.rot_mult, cache,
                                fb.out_cache_loc)
        q = ops.linear(cq, self.uq).view(T, H, D + Dr)
        if self._wants_expanded(fb, T):
            return ops.linear(self._forward_expanded(q, cache, fb), self.o_weight)
        uk, uv = self._absorbed()
        q_abs = torch.bmm(q[:, :, :D].float().transpose(0, 1), uk)                                            # [H, T, R] fp32
        q_lat = ops.latent_query(q, q_abs, D, Dr, fb.positions, self.inv_freq, self.rot_mult)                 # [T, H, R + Dr] fp32
        o_lat = ops.latent_attention(q_lat, cache, R + Dr, fb.page_table, fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens, fb.max_q_len, fb.page_size,
                                     self.scale, self.window, None, fb.max_kv_len, v_rank=R)
        o = torch.bmm(o_lat.transpose(0, 1), uv).transpose(0, 1).reshape(T, H * self.Dv)
        return ops.linear(o.to(h.dtype), self.o_weight)
