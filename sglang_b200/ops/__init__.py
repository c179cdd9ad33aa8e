"""Op front door.  CUDA tensors -> our sm_100a kernels (``torch.ops.sglb.*`` from ``_C.so``); CPU tensors ->
the fp32 torch reference (``torch_ref``) so the scheduler/model stack is testable without a GPU.

There is no multi-backend dispatch on the GPU: if the extension is missing on a CUDA box the ops raise
(``SGLB_REQUIRE_NATIVE``), they never fall back silently (the driver records which .so files were loaded).
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Optional, Tuple

import torch

from ..environ import envs
from . import torch_ref

_SO = Path(__file__).resolve().parent.parent / "_C.so"
_loaded = False
_load_error: Optional[str] = None


def load_native(build_if_missing: bool = False) -> bool:
    global _loaded, _load_error
    if _loaded:
        return True
    if not _SO.exists() and build_if_missing:
        from .. import build as _b

        _b.build_all()
    try:
        torch.ops.load_library(str(_SO))
        _loaded = True
    except Exception as e:  # pragma: no cover - depends on the box
        _load_error = f"{type(e).__name__}: {e}"
    return _loaded


def native_available() -> bool:
    return load_native()


def _use_native(t: torch.Tensor) -> bool:
    if not t.is_cuda or envs.SGLB_FORCE_TORCH_OPS.get():
        return False
    if not load_native():
        if envs.SGLB_REQUIRE_NATIVE.get():
            raise RuntimeError(f"sglang_b200 CUDA extension not loaded ({_load_error}); run `python -m sglang_b200.build`")
        return False
    return True


def launch_count() -> int:
    return int(torch.ops.sglb.launch_count()) if _loaded else 0


def reset_launch_count() -> None:
    if _loaded:
        torch.ops.sglb.reset_launch_count()


# ------------------------------------------------------------------ norms / activations
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None, gemma: bool = False) -> torch.Tensor:
    if _use_native(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:      # (16-byte vector lanes)
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        out = torch.empty_like(x2) if out is None else out.view(-1, shp[-1])
        torch.ops.sglb.rmsnorm(x2, None, weight, out, eps, gemma)
        return out.view(shp)
    r = torch_ref.gemma_rmsnorm(x, weight, eps) if gemma else torch_ref.rmsnorm(x, weight, eps)
    if out is not None:
        out.copy_(r)
        return out
    return r


def fused_add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float, gemma: bool = False) -> None:
    """residual += x ; x = rmsnorm(residual) * w   (in place)"""
    if _use_native(x) and x.dtype == torch.bfloat16:
        torch.ops.sglb.rmsnorm(x, residual, weight, x, eps, gemma)
        return
    if gemma:
        s = x.float() + residual.float()
        residual.copy_(s.to(residual.dtype))
        x.copy_(torch_ref.gemma_rmsnorm(residual, weight, eps))
    else:
        torch_ref.fused_add_rmsnorm(x, residual, weight, eps)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    if _use_native(x) and x.dtype == torch.bfloat16 and x.shape[1] % 16 == 0:      # (16-byte vector lanes)
        out = torch.empty(x.shape[0], x.shape[1] // 2, dtype=x.dtype, device=x.device)
        torch.ops.sglb.act_and_mul(x, out, 0)
        return out
    return torch_ref.silu_and_mul(x)


def gelu_and_mul(x: torch.Tensor, approximate: str = "none") -> torch.Tensor:
    if _use_native(x) and x.dtype == torch.bfloat16:
        out = torch.empty(x.shape[0], x.shape[1] // 2, dtype=x.dtype, device=x.device)
        torch.ops.sglb.act_and_mul(x, out, 2 if approximate == "tanh" else 1)
        return out
    return torch_ref.gelu_and_mul(x, approximate)


# ------------------------------------------------------------------ rope + KV write
def rope_kv_write(q, k, v, positions, cos_sin, k_cache, v_cache, out_cache_loc, is_neox: bool = True,
                  k_scale: float = 1.0, v_scale: float = 1.0, nslabs: int = 1, slab_stride: int = 0) -> None:
    """``nslabs > 1``: q/k/v are slab 0 of a split-K QKV GEMM; the kernel sums the slabs while it rotates (q is written back
    into slab 0, k/v go to the cache)."""
    if _use_native(q) and q.dtype == torch.bfloat16:
        torch.ops.sglb.rope_kv_write(q, k, v, positions, cos_sin, k_cache, v_cache, out_cache_loc, is_neox, k_scale, v_scale,
                                     nslabs, slab_stride)
        return
    assert nslabs == 1
    torch_ref.rope_kv_write(q, k, v, positions, cos_sin, k_cache, v_cache, out_cache_loc, is_neox, k_scale, v_scale)


# ------------------------------------------------------------------ attention
def attn_impl() -> int:
    v = envs.SGLB_ATTN_IMPL.get()
    return 1 if v == "simt" else 0


def paged_attention(q, k_cache, v_cache, page_table, req_slots, seq_lens, cu_q, q_lens, max_q_len: int, page_size: int,
                    scale: float, causal: bool = True, window: int = -1, logit_cap: float = 0.0, k_scale: float = 1.0,
                    v_scale: float = 1.0, num_splits: int = 1, workspace=None, tok2req=None, out=None, lse=None,
                    impl: Optional[int] = None, custom_mask=None, tree_anc=None, slopes=None, log_rates=None, keep_first: int = 0):
    """q [T,Hq,D]; caches [slots,Hkv,D]; cu_q None => decode (q_len 1).  ``slopes`` fp32 [Hq]: a distance bias ``- slopes[h] * (i - j)`` added to
    the (capped) scores, or ``- slopes[h] * ln(1 + log_rates[h] * (i - j))`` when ``log_rates`` fp32 [Hq] is given; ``keep_first``: with a window,
    keys at positions below it stay visible to every later query; all three on the tcgen05 kernels only (``tc_attention_ok`` says whether a call takes them).  ``tree_anc`` int32 [T]: speculative token-tree verification on the
    tcgen05 kernel (bit k = draft node k is an ancestor-or-self of this query node); ``custom_mask`` = the general (reference-path) form."""
    tree_ok = (tree_anc is not None and _use_native(q) and q.dtype == torch.bfloat16 and attn_impl() == 0 and q.shape[-1] == 128
               and k_cache.dtype == torch.bfloat16 and 128 % (q.shape[1] // k_cache.shape[1]) == 0 and int(max_q_len) <= 32 and window <= 0)
    if _use_native(q) and q.dtype == torch.bfloat16 and (tree_ok or (custom_mask is None and tree_anc is None)):
        if out is None:
            out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        impl = attn_impl() if impl is None else impl
        D = q.shape[-1]
        Hq, Hkv = q.shape[1], k_cache.shape[1]
        G = Hq // Hkv
        if impl == 0 and (D != 128 or k_cache.dtype != torch.bfloat16 or 128 % G != 0 or page_size < 8 or page_size > 128):
            impl = 1
        if slopes is not None or keep_first > 0:
            assert impl == 0 and tree_anc is None, "distance bias / kept first tokens: tcgen05 attention kernels only"
        part_o = part_lse = None
        if impl in (0, 2) and num_splits > 1:
            if workspace is None:
                T = q.shape[0]
                part_o = torch.empty(num_splits, T, Hq, D, dtype=torch.float32, device=q.device)
                part_lse = torch.empty(num_splits, T, Hq, dtype=torch.float32, device=q.device)
            else:
                part_o, part_lse = workspace
        else:
            num_splits = 1
        if impl == 1 and cu_q is not None and tok2req is None:
            ql = cu_q[1:] - cu_q[:-1]
            tok2req = torch.repeat_interleave(torch.arange(ql.numel(), device=q.device, dtype=torch.int32), ql.long()).to(torch.int32)
        if tree_ok:
            impl, num_splits, part_o, part_lse = 0, 1, None, None
        if impl == 0 and envs.SGLB_ATTN_PERSIST.get():
            impl = 2        # same kernel family, persistent CTAs with an atomic work queue (falls back to the classic launch when small)
        torch.ops.sglb.attn_fwd(q, k_cache, v_cache, out, lse, part_o, part_lse, page_table, req_slots, seq_lens, cu_q, tok2req,
                                int(max_q_len), int(page_size), int(num_splits), float(scale), bool(causal), int(window),
                                float(logit_cap), float(k_scale), float(v_scale), int(impl), tree_anc if tree_ok else None, slopes,
                                log_rates if slopes is not None else None, int(keep_first) if window > 0 else 0)
        return out
    assert slopes is None and keep_first <= 0, "distance bias / kept first tokens: tcgen05 attention kernels only"
    if custom_mask is None and tree_anc is not None:
        custom_mask = torch_ref.tree_anc_to_mask(tree_anc, q_lens, seq_lens)
    r = torch_ref.paged_attention(q, k_cache, v_cache, page_table, req_slots, seq_lens, q_lens, page_size, scale, causal,
                                  window, logit_cap, k_scale, v_scale, custom_mask=custom_mask, return_lse=lse is not None)
    if lse is not None:
        o, l = r
        lse.copy_(l)
        r = o
    if out is not None:
        out.copy_(r)
        return out
    return r


def tc_attention_ok(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int) -> bool:
    """whether ``paged_attention`` runs this call on the tcgen05 kernels: bf16, 128-wide heads, a group size that divides 128, caches whose rows are
    contiguous (or the leading columns of wider rows that are multiples of 16 bytes)"""
    if not (_use_native(q) and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and attn_impl() == 0 and q.dim() == 3 and k_cache.dim() == 3):
        return False
    Hq, Hkv = q.shape[1], k_cache.shape[1]
    return (q.shape[-1] == 128 and k_cache.shape[-1] == 128 and v_cache.shape == k_cache.shape and Hq % Hkv == 0 and 128 % (Hq // Hkv) == 0
            and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0 and q.is_contiguous() and k_cache.stride() == v_cache.stride()
            and k_cache.stride(2) == 1 and k_cache.stride(1) == 128 and k_cache.stride(0) >= Hkv * 128 and k_cache.stride(0) % 8 == 0
            and k_cache.data_ptr() % 16 == 0 and v_cache.data_ptr() % 16 == 0)


# ------------------------------------------------------------------ GEMM
EPI_NONE, EPI_BIAS, EPI_SILU_MUL, EPI_PUSH, EPI_SILU_SPLIT, EPI_ROWSCALE = 0, 1, 2, 3, 4, 5


def gemm_impl() -> str:
    return envs.SGLB_GEMM_IMPL.get()


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, impl: Optional[str] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T,K] @ w[N,K]^T.  impl: 'tc' = our tcgen05 GEMM, 'lib' = cuBLASLt (plain library GEMM)."""
    impl = impl or gemm_impl()
    if impl != "lib" and streamk_ok(x, w) and (out is None or (out.dim() == 2 and out.stride(1) == 1 and out.stride(0) % 8 == 0
                                                                 and out.data_ptr() % 16 == 0)):
        # decode shapes: persistent stream-K weight streaming (gemm_streamk.cu) — also writes straight into an NVL arena slot (``out``)
        return gemm_streamk(x, w, bias, out=out)
    if impl in ("tc", "auto") and _use_native(x) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 \
            and x.dim() == 2 and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1 \
            and impl == "tc":
        if out is None:
            out = torch.empty(x.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
        torch.ops.sglb.gemm(x, w, out, bias, EPI_BIAS if bias is not None else EPI_NONE, 0)
        return out
    if out is not None and bias is None and x.dim() == 2 and out.is_contiguous():
        return torch.mm(x, w.t(), out=out)       # cuBLAS writes straight into the caller's buffer (e.g. an NVL arena slot)
    r = torch.nn.functional.linear(x, w, bias)
    if out is not None:
        out.copy_(r)
        return out
    return r


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, epilogue: int = EPI_NONE, bn: int = 0,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    n_out = w.shape[0] // 2 if epilogue in (EPI_SILU_MUL, EPI_SILU_SPLIT) else w.shape[0]
    if out is None:
        out = torch.empty(x.shape[0], n_out, dtype=x.dtype, device=x.device)
    torch.ops.sglb.gemm(x, w, out, bias, epilogue, bn)
    return out


# ------------------------------------------------------------------ decode-shape ("skinny") GEMM: swap-AB + split-K slabs
SKINNY_MAX_M = 256


def skinny_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """decode-shape policy: tokens <= 256, bf16, 16-byte aligned rows (``SGLB_SKINNY=0`` disables, ``1`` forces the check only)"""
    return (x.is_cuda and x.dim() == 2 and 0 < x.shape[0] <= SKINNY_MAX_M and x.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and w.dim() == 2 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] % 8 == 0
            and w.shape[0] % 8 == 0 and _use_native(x))


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, silu_split: bool = False,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[T<=256,K] @ w[N,K]^T in one pass (no K split).  ``silu_split``: w = [gate; up] -> silu(x@gate^T) * (x@up^T)"""
    n_out = w.shape[0] // 2 if silu_split else w.shape[0]
    if out is None:
        out = torch.empty(x.shape[0], n_out, dtype=x.dtype, device=x.device)
    torch.ops.sglb.gemm_skinny(x, w, out, bias, EPI_SILU_SPLIT if silu_split else (EPI_BIAS if bias is not None else EPI_NONE), 1)
    return out


def streamk_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """shape / layout policy of the stream-K decode GEMM (``SGLB_STREAMK_MAX_M`` tokens at most, bf16, TMA-compatible strides)"""
    mx = envs.SGLB_STREAMK_MAX_M.get()
    return (mx > 0 and x.is_cuda and x.dim() == 2 and 0 < x.shape[0] <= min(mx, 256) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.dim() == 2 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.shape[1] % 8 == 0
            and w.shape[0] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and _use_native(x))


def gemm_streamk(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, silu_split: bool = False,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[T<=256,K] @ w[N,K]^T on the persistent stream-K tcgen05 kernel (csrc/kernels/gemm_streamk.cu): every SM streams an equal share of
    the weights, split tiles are reduced in-kernel (deterministic), TMA-store epilogue.  ``silu_split``: w = [gate; up] -> silu(g) * u."""
    n_out = w.shape[0] // 2 if silu_split else w.shape[0]
    if out is None:
        out = torch.empty(x.shape[0], n_out, dtype=x.dtype, device=x.device)
    torch.ops.sglb.gemm_streamk(x, w, out, bias, EPI_SILU_SPLIT if silu_split else (EPI_BIAS if bias is not None else EPI_NONE))
    return out


def gemm_skinny_slabs(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, max_splits: int = 8) -> torch.Tensor:
    """split-K partials [splits, T, N] (bf16); the consumer sums the slabs (``slab_reduce_add_rmsnorm``, ``rope_kv_write``)"""
    T, K = x.shape
    N = w.shape[0]
    s = int(torch.ops.sglb.gemm_skinny_splits(T, N, K, max_splits))
    slabs = torch.empty(s, T, N, dtype=x.dtype, device=x.device)
    if s == 1:
        torch.ops.sglb.gemm_skinny(x, w, slabs[0], bias, EPI_BIAS if bias is not None else EPI_NONE, 1)
    else:
        torch.ops.sglb.gemm_skinny(x, w, slabs, bias, EPI_BIAS if bias is not None else EPI_NONE, s)
    return slabs


def slab_reduce_add_rmsnorm(slabs: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                            gemma: bool = False) -> torch.Tensor:
    """out = rmsnorm(residual += sum_s slabs[s]) * w    (residual updated in place when given)"""
    out = torch.empty(slabs.shape[1], slabs.shape[2], dtype=slabs.dtype, device=slabs.device)
    torch.ops.sglb.slab_reduce_add_rmsnorm(slabs, residual, weight, out, eps, gemma)
    return out


# ------------------------------------------------------------------ misc index ops
def apply_pt_delta(page_table: torch.Tensor, rows: torch.Tensor, cols: torch.Tensor, vals: torch.Tensor, n: Optional[torch.Tensor] = None,
                   n_max: Optional[int] = None) -> None:
    n_max = rows.numel() if n_max is None else n_max
    if n_max == 0:
        return
    if _use_native(page_table):
        torch.ops.sglb.apply_pt_delta(page_table, rows, cols, vals, n, n_max)
        return
    page_table[rows.long(), cols.long()] = vals


def embedding(weight: torch.Tensor, ids: torch.Tensor, gather_idx: Optional[torch.Tensor] = None, vocab_start: int = 0) -> torch.Tensor:
    T = ids.shape[0] if gather_idx is None else gather_idx.shape[0]
    if _use_native(weight) and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0:      # (16-byte vector lanes)
        out = torch.empty(T, weight.shape[1], dtype=weight.dtype, device=weight.device)
        torch.ops.sglb.embedding(weight, ids, gather_idx, out, vocab_start)
        return out
    if gather_idx is not None:
        ids = ids[gather_idx.long()]
    idl = ids.long() - vocab_start
    ok = (idl >= 0) & (idl < weight.shape[0])
    out = torch.nn.functional.embedding(idl.clamp(0, weight.shape[0] - 1), weight)
    return out * ok[:, None].to(out.dtype)


def gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    if _use_native(x) and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0:      # (16-byte vector lanes)
        out = torch.empty(idx.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
        torch.ops.sglb.gather_rows(x, idx, out)
        return out
    return x[idx.long()]


# ------------------------------------------------------------------ sampling
def sample(logits, temperature, top_k, top_p, min_p, seeds=None, out_slots=None, next_token_buf=None, out_logprobs=None,
           global_seed: int = 0, step_ptr=None, step: int = 0, generator=None) -> torch.Tensor:
    B = logits.shape[0]
    if _use_native(logits):
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
        torch.ops.sglb.sample(logits, temperature, top_k, top_p, min_p, seeds, out_slots, next_token_buf, out, out_logprobs,
                              int(global_seed) & 0x7FFFFFFFFFFFFFFF, step_ptr, int(step))
        return out
    g = generator
    if g is None:
        g = torch.Generator(device="cpu")
        g.manual_seed((int(global_seed) * 1000003 + int(step)) & 0x7FFFFFFF)
    u = torch.rand(B, generator=g)
    if seeds is not None:      # seeded rows: one uniform from (seed, own output position) — same contract as the kernel
        for j, (sd, pos) in enumerate(seeds.tolist()):
            if pos >= 0:
                gj = torch.Generator(device="cpu")
                gj.manual_seed(((int(sd) * 0x9E3779B1) ^ (int(pos) * 0x85EBCA6B + 0x5bd1e995)) & 0x7FFFFFFFFFFFFFFF)
                u[j] = torch.rand(1, generator=gj)[0]
    u = u.to(logits.device)
    tok = torch_ref.sample(logits, temperature, top_k, top_p, min_p, u).to(torch.int32)
    if out_logprobs is not None:
        lp = torch.log_softmax(logits.float() / temperature.clamp(min=1e-6)[:, None], dim=-1)
        out_logprobs.copy_(lp.gather(1, tok.long()[:, None]).squeeze(1))
    if next_token_buf is not None and out_slots is not None:
        next_token_buf[out_slots.long()] = tok
    return tok


def causal_conv1d(x: torch.Tensor, w: torch.Tensor, bias, conv_state: torch.Tensor, cu_q, req_slots: torch.Tensor, seq_lens: torch.Tensor,
                  max_q_len: int = 1, silu: bool = True) -> torch.Tensor:
    """Mamba causal depthwise conv1d over a ragged batch, rolling state updated in place (csrc/kernels/mamba.cu); fp32 [T, C] out"""
    if _use_native(x) and x.dtype in (torch.bfloat16, torch.float32) and x.stride(1) == 1 and 2 <= w.shape[1] <= 8:
        u = torch.empty(x.shape[0], x.shape[1], dtype=torch.float32, device=x.device)
        torch.ops.sglb.causal_conv1d(x, w.contiguous(), bias, conv_state, cu_q, req_slots, seq_lens, int(max_q_len), bool(silu), u)
        return u
    return torch_ref.causal_conv1d(x, w, bias, conv_state, cu_q, req_slots, seq_lens, silu)


def selective_state_update(state: torch.Tensor, req_slots: torch.Tensor, x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, Bm: torch.Tensor,
                           Cm: torch.Tensor, D=None) -> torch.Tensor:
    """Mamba-2 single-token state update + read-out, ONE pass over the fp32 state (csrc/kernels/mamba.cu); y fp32 [B, H, P]"""
    if (_use_native(state) and state.dtype == torch.float32 and state.shape[3] % 4 == 0 and all(t.dtype == torch.float32 for t in (x, dt, A, Bm, Cm))
            and Bm.stride(0) % 4 == 0 and Bm.stride(0) == Cm.stride(0) and Bm.data_ptr() % 16 == 0 and Cm.data_ptr() % 16 == 0 and x.stride(1) == 1):
        B, (H, P) = req_slots.numel(), state.shape[1:3]
        y = torch.empty(B, H, P, dtype=torch.float32, device=state.device)
        torch.ops.sglb.selective_state_update(state, req_slots, x, dt.contiguous(), A.contiguous(), Bm, Cm, D, y)
        return y
    return torch_ref.selective_state_update(state, req_slots, x, dt, A, Bm, Cm, D)


def gated_delta_update(state: torch.Tensor, req_slots: torch.Tensor, u: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, Hk: int) -> Optional[torch.Tensor]:
    """gated delta rule, one token per request: u fp32 [B, 2*Hk*Dk + Hv*Dv] = conv output rows [q | k | v] (q, k un-normalised), state fp32
    [slots, Hv, Dk, Dv] updated in place -> o fp32 [B, Hv, Dv]; None when the native kernel does not cover the shape (caller falls back)"""
    if (_use_native(state) and state.dtype == torch.float32 and u.dtype == torch.float32 and u.stride(1) == 1 and state.shape[2] in (64, 128)
            and state.shape[3] <= (256 if state.shape[2] == 64 else 128)):
        B, Hv, Dv = req_slots.numel(), state.shape[1], state.shape[3]
        out = torch.empty(B, Hv, Dv, dtype=torch.float32, device=state.device)
        torch.ops.sglb.gated_delta_update(state, req_slots, u, g.float().contiguous(), beta.float().contiguous(), int(Hk), out)
        return out
    return None


def greedy_shard(logits: torch.Tensor, v_valid: int, v_offset: int, rank: int, tp: int, buf: torch.Tensor) -> None:
    """argmax of this rank's vocabulary shard -> buf[rank, row] = (max logit, idx byte 0, 1, 2) as bf16; the other ranks' planes are zeroed so
    that an all-reduce (sum) of ``buf`` is an exact all-gather (sampling.cu greedy_shard_kernel)"""
    B = logits.shape[0]
    if _use_native(logits):
        torch.ops.sglb.greedy_shard(logits, int(v_valid), int(v_offset), int(rank), int(tp), buf)
        return
    buf[:, :B].zero_()
    if v_valid > 0:
        val, idx = logits[:, :v_valid].float().max(dim=1)
        g = idx + int(v_offset)
    else:
        val = torch.full((B,), -3.3e38, dtype=torch.float32, device=logits.device)
        g = torch.zeros(B, dtype=torch.long, device=logits.device)
    buf[rank, :B, 0] = val.clamp(min=-3.3e38).to(buf.dtype)
    buf[rank, :B, 1] = (g & 255).to(buf.dtype)
    buf[rank, :B, 2] = ((g >> 8) & 255).to(buf.dtype)
    buf[rank, :B, 3] = ((g >> 16) & 255).to(buf.dtype)


def greedy_merge(buf: torch.Tensor, B: int, out_slots=None, next_token_buf=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """winner over the gathered per-rank (max, index) pairs; equal maxima keep the lowest global index"""
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=buf.device)
    if _use_native(buf):
        torch.ops.sglb.greedy_merge(buf, int(B), out_slots, next_token_buf, out)
        return out
    v = buf[:, :B, 0].float()                              # [tp, B]
    r = v.argmax(dim=0)                                    # first maximum = lowest rank
    w = buf[:, :B, 1:].float().long()                      # [tp, B, 3]
    sel = w.gather(0, r.view(1, B, 1).expand(1, B, 3)).squeeze(0)
    tok = (sel[:, 0] | (sel[:, 1] << 8) | (sel[:, 2] << 16)).to(torch.int32)
    out[:B] = tok
    if next_token_buf is not None and out_slots is not None:
        next_token_buf[out_slots[:B].long()] = tok
    return out


def apply_token_bitmask(logits: torch.Tensor, bitmask: torch.Tensor, row_idx: Optional[torch.Tensor] = None) -> None:
    if _use_native(logits):
        torch.ops.sglb.apply_token_bitmask(logits, bitmask, row_idx)
        return
    if row_idx is None:
        torch_ref.apply_token_bitmask(logits, bitmask)
    else:
        sub = logits[row_idx.long()]
        torch_ref.apply_token_bitmask(sub, bitmask)
        logits[row_idx.long()] = sub


def apply_penalties(logits, counts, prompt_mask, freq, pres, rep) -> None:
    if _use_native(logits) and logits.dtype == torch.float32:
        torch.ops.sglb.apply_penalties(logits, counts, prompt_mask, freq, pres, rep)
        return
    pm = prompt_mask.bool() if prompt_mask is not None else torch.zeros_like(counts, dtype=torch.bool)
    torch_ref.apply_penalties(logits, counts, pm, freq, pres, rep)


def merge_attn_states(o1, lse1, o2, lse2):
    return torch_ref.merge_attn_states(o1, lse1, o2, lse2)


# ------------------------------------------------------------------ fp32 residual stream / latent attention / gated delta rule / clamped GLU
def add_rmsnorm_f32(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, zero_centred: bool = False,
                    out_dtype: torch.dtype = torch.bfloat16, post_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 residual stream: ``residual += delta`` (in place, fp32 sum) and the RMS norm of the new residual in ``out_dtype``, one kernel
    (csrc/kernels/residual_f32.cu).  ``zero_centred``: the weight is stored around zero and applied as ``1 + w``.  ``post_weight``: the branch
    output is itself RMS-normed, times ``1 + post_weight`` (``post_weight`` when not ``zero_centred``), before it joins the residual
    (sandwich-norm blocks), in the same kernel.  A weight of one element is one gain for all coordinates."""
    if post_weight is not None and delta is not None:
        if _use_native(residual) and residual.dtype == torch.float32 and residual.is_contiguous() and out_dtype in (torch.bfloat16, torch.float32) \
                and delta.dtype in (torch.bfloat16, torch.float32) and delta.is_contiguous() and weight.dtype == out_dtype and post_weight.dtype == out_dtype:
            out = torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
            torch.ops.sglb.postnorm_add_rmsnorm_f32(residual, delta, post_weight, weight, out, float(eps), bool(zero_centred))
            return out
        return torch_ref.postnorm_add_rmsnorm_f32(residual, delta, post_weight, weight, eps, out_dtype, zero_centred)
    if _use_native(residual) and residual.dtype == torch.float32 and residual.is_contiguous() and out_dtype in (torch.bfloat16, torch.float32) \
            and weight.dtype == out_dtype and (delta is None or (delta.dtype in (torch.bfloat16, torch.float32) and delta.is_contiguous())):
        out = torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
        torch.ops.sglb.add_rmsnorm_f32(residual, delta, weight, out, float(eps), bool(zero_centred))
        return out
    return torch_ref.add_rmsnorm_f32(residual, delta, weight, eps, zero_centred, out_dtype)


def clamped_glu(gu: torch.Tensor, limit: float, alpha: float = 1.702) -> torch.Tensor:
    """[gate | up] halves -> min(g, limit) * sigmoid(alpha g) * (clamp(u, +-limit) + 1), fp32 math (csrc/kernels/residual_f32.cu)"""
    if _use_native(gu) and gu.dtype in (torch.bfloat16, torch.float32) and gu.dim() == 2 and gu.is_contiguous():
        out = torch.empty(gu.shape[0], gu.shape[1] // 2, dtype=gu.dtype, device=gu.device)
        torch.ops.sglb.clamped_glu(gu, out, float(limit), float(alpha))
        return out
    return torch_ref.clamped_glu(gu, limit, alpha)


def latent_attention(q_lat: torch.Tensor, cache: torch.Tensor, rank: int, page_table: torch.Tensor, req_slots: torch.Tensor, seq_lens: torch.Tensor,
                     cu_q: Optional[torch.Tensor], q_lens: Optional[torch.Tensor], max_q_len: int, page_size: int, scale: float, window: int = -1,
                     sinks: Optional[torch.Tensor] = None, max_kv_len: int = 0, v_rank: Optional[int] = None) -> torch.Tensor:
    """absorbed multi-query attention over a paged cache of latent rows with a sliding window and per-head sinks
    (csrc/kernels/latent_attention.cu; contract in ``torch_ref.latent_attention``).  ``cu_q`` None = one query per request.
    ``max_kv_len`` (host-side longest sequence; 0 = unknown) only steers how decode splits the keys over CTAs.  ``v_rank``: how many leading
    columns of a cached row are its value (default: all ``rank``; the others, e.g. a rotary key part, take part in the scores only)."""
    v_rank = int(rank if v_rank is None else v_rank)
    if (_use_native(q_lat) and q_lat.dtype == torch.float32 and cache.dtype in (torch.bfloat16, torch.float32) and q_lat.is_contiguous()
            and rank <= 1024 and req_slots.numel() <= 65535):          # (a key tile and one head's accumulators have to fit shared memory)
        out = torch.empty(q_lat.shape[0], q_lat.shape[1], v_rank, dtype=torch.float32, device=q_lat.device)
        torch.ops.sglb.latent_attention(q_lat, cache, int(rank), page_table, req_slots, seq_lens, cu_q, int(max_q_len),
                                        int(max_kv_len) if max_kv_len else (int(window) if window > 0 else 4096), int(page_size), float(scale),
                                        int(window), sinks, out, v_rank)
        return out
    return torch_ref.latent_attention(q_lat, cache, rank, page_table, req_slots, seq_lens, q_lens, page_size, scale, window, sinks, v_rank)


def _delta_shape_ok(Dk: int, Dv: int) -> bool:
    """the kernel keeps a column of the state in 1..16 lanes of 16, 32 or 64 rows each, one CTA (<= 512 or 1024 threads) per head"""
    for rows, max_threads in ((32, 512), (16, 1024), (64, 512)):
        ks = 1
        while ks * rows < Dk and ks < 16:
            ks <<= 1
        if ks * rows >= Dk and Dv * ks <= max_threads:
            return True
    return False


def gated_delta_rule(u: torch.Tensor, Hk: int, Dk: int, H: int, Dv: int, a_raw: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor,
                     b_raw: torch.Tensor, state: torch.Tensor, req_slots: torch.Tensor, seq_lens: torch.Tensor, cu_q: Optional[torch.Tensor],
                     q_lens: Optional[torch.Tensor], gate_raw: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                     eps: float = 1e-6, gate_act: str = "silu", per_channel: Optional[bool] = None) -> torch.Tensor:
    """gated delta rule over a ragged batch (prefill portions and single decode tokens alike): unit-norm q/k, decay and beta from their raw
    projections, the fp32 state update and read-out, and the gated per-head RMS norm of the output, in one kernel
    (csrc/kernels/delta_rule.cu; contract in ``torch_ref.gated_delta_rule``)."""
    if per_channel is None:
        per_channel = a_raw.shape[1] != H
    if (_use_native(u) and u.dtype == torch.float32 and state.dtype == torch.float32 and u.is_contiguous() and _delta_shape_ok(Dk, Dv)
            and req_slots.numel() <= 65535):
        T = u.shape[0]
        out = torch.empty(T, H, Dv, dtype=torch.float32, device=u.device)
        f = lambda t: None if t is None else t.float().contiguous()
        torch.ops.sglb.gated_delta_rule(u, int(Hk), int(Dk), int(H), int(Dv), f(a_raw), f(A_log), f(dt_bias), f(b_raw), state, req_slots, seq_lens,
                                        cu_q, f(gate_raw), f(norm_w), float(eps), gate_act == "silu", bool(per_channel), out)
        return out
    return torch_ref.gated_delta_rule(u, Hk, Dk, H, Dv, a_raw, A_log, dt_bias, b_raw, state, req_slots, seq_lens, q_lens, gate_raw, norm_w, eps,
                                      gate_act, per_channel)


# ------------------------------------------------------------------ bigram embedding / Mamba-2 scan / biased window attention / soft-max router with identity experts
def bigram_embedding(embed: torch.Tensor, bigram: Optional[torch.Tensor], ids: torch.Tensor, prev_tokens: Optional[torch.Tensor], cu_q,
                     req_slots: torch.Tensor, seq_lens: torch.Tensor, max_q_len: int, scale: float, mul_prev: int = 0, mul_cur: int = 0,
                     buckets: int = 0) -> torch.Tensor:
    """token embedding times ``scale`` plus a hashed (previous token, token) row, straight into the fp32 residual stream
    (csrc/kernels/elementwise.cu; semantics in ``torch_ref.bigram_embedding``).  ``prev_tokens`` int32 [slots] carries every request's last
    token from call to call."""
    if _use_native(embed) and embed.dtype in (torch.bfloat16, torch.float32) and embed.is_contiguous() and ids.dtype == torch.int32 \
            and req_slots.numel() <= 65535 and (bigram is None or (bigram.dtype == embed.dtype and bigram.is_contiguous())):
        out = torch.empty(ids.shape[0], embed.shape[1], dtype=torch.float32, device=embed.device)
        torch.ops.sglb.bigram_embedding(embed, bigram, ids.contiguous(), prev_tokens if bigram is not None else None, cu_q, req_slots, seq_lens,
                                        int(max_q_len), float(scale), int(mul_prev), int(mul_cur), int(buckets), out)
        return out
    return torch_ref.bigram_embedding(embed, bigram, ids, prev_tokens, cu_q, req_slots, seq_lens, scale, mul_prev, mul_cur, buckets)


def grouped_rmsnorm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, out_dtype: torch.dtype, gate: Optional[torch.Tensor] = None,
                    out_scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 [T, C] in ``groups`` equal parts, each divided by its own root mean square, times weight; with ``gate`` [T, C] (a column view is
    fine) also times ``sigmoid(gate)``, then times ``out_scale`` (csrc/kernels/residual_f32.cu).  ``out``: a [T, C] view with unit column
    stride to write into (e.g. columns of a wider buffer)."""
    if _use_native(x) and x.dtype == torch.float32 and x.is_contiguous() and out_dtype in (torch.bfloat16, torch.float32) and weight.dtype == out_dtype \
            and x.shape[1] % groups == 0 and (gate is None or (gate.dtype == out_dtype and gate.stride(1) == 1)):
        if out is None:
            out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        assert out.dtype == out_dtype and out.stride(1) == 1
        torch.ops.sglb.grouped_rmsnorm(x, weight, int(groups), float(eps), out, gate, float(out_scale))
        return out
    y = torch_ref.grouped_rmsnorm(x, weight, groups, eps, out_dtype, gate, out_scale)
    if out is not None:
        out.copy_(y)
        return out
    return y


def mamba2_scan(u: torch.Tensor, z: Optional[torch.Tensor], dt_raw: Optional[torch.Tensor], dt_bias: Optional[torch.Tensor],
                A_log: Optional[torch.Tensor], D: Optional[torch.Tensor], state: torch.Tensor, req_slots: torch.Tensor, seq_lens: torch.Tensor,
                cu_q: Optional[torch.Tensor], q_lens: Optional[torch.Tensor], H: int, P: int, N: int, G: int,
                decay: Optional[torch.Tensor] = None, gates: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Mamba-2 recurrence over a ragged batch (prompt portions and single decode tokens alike): softplus step size, decay, the fp32 state update
    and read-out, the skip term and the silu(z) gate in one kernel (csrc/kernels/mamba.cu; semantics in ``torch_ref.mamba2_scan``).  ``z`` and
    ``dt_raw`` may be column views of the projection's output.  ``decay`` fp32 [H] replaces the input-dependent step: step size 1, the
    head's state times its constant every token (``dt_raw``, ``dt_bias``, ``A_log`` unused).  ``gates`` fp32 [T, H, n >= 2] contiguous: every
    token brings its decay ``gates[t, h, 0]`` and its step ``gates[t, h, 1]`` (exponentially gated memories such as ``layers/mlstm.py``)."""
    fixed = decay is not None or gates is not None
    if (_use_native(u) and u.dtype == torch.float32 and u.is_contiguous() and state.dtype == torch.float32 and N <= 1024 and req_slots.numel() <= 65535
            and (fixed or (dt_raw.stride(1) == 1 and dt_raw.dtype in (torch.bfloat16, torch.float32)))
            and (gates is None or (gates.dtype == torch.float32 and gates.is_contiguous()))
            and (z is None or (z.stride(1) == 1 and z.dtype in (torch.bfloat16, torch.float32) and (fixed or z.dtype == dt_raw.dtype)))):
        out = torch.empty(u.shape[0], H * P, dtype=torch.float32, device=u.device)
        f = lambda t: None if t is None else t.float().contiguous()
        if gates is not None:
            torch.ops.sglb.mamba2_scan(u, z, None, None, None, f(D), state, req_slots, seq_lens, cu_q, int(H), int(P), int(N), int(G), out, None, gates)
        elif decay is not None:
            torch.ops.sglb.mamba2_scan(u, z, None, None, None, f(D), state, req_slots, seq_lens, cu_q, int(H), int(P), int(N), int(G), out, f(decay), None)
        else:
            torch.ops.sglb.mamba2_scan(u, z, dt_raw, f(dt_bias), f(A_log), f(D), state, req_slots, seq_lens, cu_q, int(H), int(P), int(N), int(G), out, None, None)
        return out
    return torch_ref.mamba2_scan(u, z, dt_raw, dt_bias, A_log, D, state, req_slots, seq_lens, q_lens, H, P, N, G, decay, gates)


def attention_sink_gate(o: torch.Tensor, lse: torch.Tensor, sinks: torch.Tensor, Dv: Optional[int] = None) -> torch.Tensor:
    """``o[:, :, :Dv] * sigmoid(lse - sink_h)``: adds a per-head sink to the soft-max denominator of an attention that returned the log-sum-exp
    of its scores, and drops zero padding behind ``Dv`` (csrc/kernels/window_attention.cu); o [T, H, D] -> [T, H, Dv]"""
    Dv = o.shape[2] if Dv is None else Dv
    if _use_native(o) and o.dtype == torch.bfloat16 and o.is_contiguous() and lse.dtype == torch.float32 and lse.is_contiguous():
        out = torch.empty(o.shape[0], o.shape[1], Dv, dtype=o.dtype, device=o.device)
        torch.ops.sglb.attention_sink_gate(o, lse, sinks.float().contiguous(), int(Dv), out)
        return out
    return (o[:, :, :Dv].float() * torch.sigmoid(lse - sinks[None, :]).unsqueeze(-1)).to(o.dtype)


def sigmoid_gate(o: torch.Tensor, gate: torch.Tensor, Dv: Optional[int] = None, out_scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``o[:, :, :Dv] * sigmoid(gate) * out_scale`` -> [T, H * Dv]: the output gate of an attention whose kernel has no gate epilogue, one number
    per head (``gate`` [T, H]) or per element ([T, H*Dv]; a column view is fine); also drops zero padding behind ``Dv``
    (csrc/kernels/window_attention.cu).  ``out``: a [T, H*Dv] view with unit column stride to write into."""
    T, H = o.shape[0], o.shape[1]
    Dv = o.shape[2] if Dv is None else Dv
    if _use_native(o) and o.dtype in (torch.bfloat16, torch.float32) and o.is_contiguous() and gate.dtype == o.dtype and gate.stride(1) == 1 \
            and gate.shape[1] in (H, H * Dv):
        if out is None:
            out = torch.empty(T, H * Dv, dtype=o.dtype, device=o.device)
        assert out.dtype == o.dtype and out.stride(1) == 1
        torch.ops.sglb.sigmoid_gate(o, gate, int(Dv), float(out_scale), out)
        return out
    g = torch.sigmoid(gate.float())
    y = (o[:, :, :Dv].float() * (g[:, :, None] if g.shape[1] == H else g.view(T, H, Dv)) * out_scale).to(o.dtype).reshape(T, H * Dv)
    if out is not None:
        out.copy_(y)
        return out
    return y


def qk_norm_cache_write(qkv: torch.Tensor, H: int, G: int, D: int, Dv: int, positions: torch.Tensor, eps: float, temp_coef: float, temp_every: int,
                        k_cache: torch.Tensor, v_cache: torch.Tensor, out_cache_loc: torch.Tensor, normalise: bool = True, pad: int = 0) -> torch.Tensor:
    """per-head unit-RMS q and k, position-dependent query temperature, and the write of k / v rows into the paged cache, one kernel
    (csrc/kernels/window_attention.cu; semantics in ``torch_ref.qk_norm_cache_write``).  Returns q [T, H, D] in the cache dtype.
    ``pad > 0``: every head of q, k and v is laid out ``pad`` columns wide with zeros behind its values (the tcgen05 kernels' head size)."""
    if (_use_native(qkv) and qkv.dtype in (torch.bfloat16, torch.float32) and qkv.is_contiguous() and k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
            and k_cache.stride(-1) == 1 and v_cache.stride(-1) == 1 and k_cache.stride(0) == v_cache.stride(0)):
        q = torch.empty(qkv.shape[0], H, pad if pad > 0 else D, dtype=qkv.dtype, device=qkv.device)
        torch.ops.sglb.qk_norm_cache_write(qkv, int(H), int(G), int(D), int(Dv), positions, float(eps), float(temp_coef), int(max(1, temp_every)), k_cache,
                                           v_cache, out_cache_loc, bool(normalise), q, int(pad))
        return q
    return torch_ref.qk_norm_cache_write(qkv, H, G, D, Dv, positions, eps, temp_coef, max(1, temp_every), k_cache, v_cache, out_cache_loc, normalise, pad)


def window_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, G: int, Dv: int, page_table: torch.Tensor, req_slots: torch.Tensor,
                     seq_lens: torch.Tensor, cu_q: Optional[torch.Tensor], q_lens: Optional[torch.Tensor], max_q_len: int, page_size: int, scale: float,
                     softcap: float = 0.0, window: int = -1, slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None,
                     dim: int = 0, pad: int = 0, keep_first: int = 0, log_rates: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                     out_scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """paged grouped-query attention with a tanh score cap, a per-head distance bias, a sliding window and soft-max sinks, for prompt portions
    and decode tokens (csrc/kernels/window_attention.cu; semantics in ``torch_ref.window_attention``).  Returns [T, H, Dv] in q's dtype.
    ``pad > 0``: heads are laid out ``pad`` columns wide in q and in the cache rows; ``dim`` is the key size that counts.
    ``keep_first``: the sequence's first positions stay visible behind the window.  ``log_rates``: the bias is ``slopes_h ln(1 + log_rates_h
    (i - j))``.  ``gate`` [T, H] or [T, H*Dv] (q's dtype, a column view is fine): the output times ``sigmoid(gate)``, per head or per element,
    then times ``out_scale``, in the kernel's epilogue.  ``out``: a [T, H*Dv] view with unit column stride to write into."""
    T, H, D = q.shape
    if pad > 0:
        D = dim
    if (_use_native(q) and q.dtype in (torch.bfloat16, torch.float32) and q.is_contiguous() and k_cache.dtype == q.dtype and v_cache.dtype == q.dtype
            and D <= 256 and Dv <= 256 and req_slots.numel() <= 65535 and k_cache.stride(0) == v_cache.stride(0)
            and (gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1 and gate.shape[1] in (H, H * Dv)))):
        if out is None:
            out = torch.empty(T, H * Dv, dtype=q.dtype, device=q.device)
        assert out.dtype == q.dtype and out.stride(1) == 1 and out.shape == (T, H * Dv)
        f = lambda t: None if t is None else t.float().contiguous()
        torch.ops.sglb.window_attention(q, k_cache, v_cache, int(G), int(Dv), page_table, req_slots, seq_lens, cu_q, int(max_q_len), int(page_size),
                                        float(scale), float(softcap), int(window), f(slopes), f(sinks), out, int(D), int(pad), int(keep_first),
                                        f(log_rates), gate, float(out_scale))
        return out.view(T, H, Dv) if out.is_contiguous() else out
    y = torch_ref.window_attention(q, k_cache, v_cache, G, Dv, page_table, req_slots, seq_lens, q_lens, page_size, scale, softcap, window, slopes,
                                   sinks, dim, pad, keep_first, log_rates, gate, out_scale).to(q.dtype)
    if out is not None:
        out.copy_(y.view(T, H * Dv))
        return out
    return y


# ------------------------------------------------------------------ attention preparation / selective scan / element-wise activations
def attention_prepare(qkv: torch.Tensor, H: int, G: int, D: int, Dv: int, positions: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      out_cache_loc: torch.Tensor, q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
                      inv_freq: Optional[torch.Tensor] = None, v_first: Optional[torch.Tensor] = None, v_lambda: float = 0.0, pad: int = 0,
                      v_inv_freq: Optional[torch.Tensor] = None, v_interleaved: bool = False) -> torch.Tensor:
    """what lies between the q / k / v projection and the attention kernel, in one pass per token: an RMS norm of q and of k over their whole
    projection with a weight, a rotation of the first coordinates of every head by position (pairs half a rotary width apart, angles in
    fp32 from ``inv_freq``), a blend of v with another layer's values of the same token, and the write of k / v rows into the paged cache
    (csrc/kernels/window_attention.cu; semantics in ``torch_ref.attention_prepare``).  ``qkv`` may be the first columns of a wider
    projection; ``v_first`` may be a column view.  ``v_inv_freq`` fp32 [Dv/2]: every value head is also turned over its whole width by
    ``position * v_inv_freq[m]`` before it is cached (pairs half a head apart, or neighbours with ``v_interleaved``).  Returns q [T, H, D | pad]
    in the cache dtype."""
    if (_use_native(qkv) and qkv.dtype in (torch.bfloat16, torch.float32) and qkv.stride(1) == 1 and k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
            and k_cache.stride(-1) == 1 and v_cache.stride(-1) == 1 and k_cache.stride(0) == v_cache.stride(0)
            and (v_first is None or (v_first.dtype == qkv.dtype and v_first.stride(1) == 1))
            and (q_norm_w is None or (q_norm_w.dtype == qkv.dtype and k_norm_w.dtype == qkv.dtype))):
        q = torch.empty(qkv.shape[0], H, pad if pad > 0 else D, dtype=qkv.dtype, device=qkv.device)
        torch.ops.sglb.attention_prepare(qkv, int(H), int(G), int(D), int(Dv), positions, k_cache, v_cache, out_cache_loc, q_norm_w, k_norm_w, float(eps),
                                         inv_freq, v_first, float(v_lambda), q, int(pad), v_inv_freq, bool(v_interleaved))
        return q
    return torch_ref.attention_prepare(qkv, H, G, D, Dv, positions, k_cache, v_cache, out_cache_loc, q_norm_w, k_norm_w, eps, inv_freq, v_first, v_lambda, pad,
                                       v_inv_freq, v_interleaved)


def mamba1_scan(u: torch.Tensor, dt_raw: torch.Tensor, dt_bias: Optional[torch.Tensor], A_log: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
                D: Optional[torch.Tensor], z: Optional[torch.Tensor], state: torch.Tensor, req_slots: torch.Tensor, seq_lens: torch.Tensor,
                cu_q: Optional[torch.Tensor], q_lens: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """selective scan (Mamba-1) over a ragged batch (prompt portions and single decode tokens alike): softplus step size, per-channel and
    per-state decay ``exp(-dt exp(A_log))``, the fp32 state update and read-out, the skip term and the silu(z) gate in one kernel
    (csrc/kernels/mamba.cu; semantics in ``torch_ref.mamba1_scan``).  ``dt_raw`` fp32 [T, C]; ``Bm`` / ``Cm`` / ``z`` may be column views of
    their projections' outputs (bf16 or fp32)."""
    ok = lambda t: t.stride(1) == 1 and t.dtype in (torch.bfloat16, torch.float32)
    if (_use_native(u) and u.dtype == torch.float32 and u.is_contiguous() and state.dtype == torch.float32 and state.is_contiguous() and A_log.shape[1] <= 256
            and req_slots.numel() <= 65535 and dt_raw.dtype == torch.float32 and dt_raw.stride(1) == 1 and ok(Bm) and ok(Cm) and Bm.dtype == Cm.dtype
            and Bm.stride(0) == Cm.stride(0) and (z is None or ok(z)) and out_dtype in (torch.bfloat16, torch.float32)):
        out = torch.empty(u.shape, dtype=out_dtype, device=u.device)
        f = lambda t: None if t is None else t.float().contiguous()
        torch.ops.sglb.mamba1_scan(u, dt_raw, f(dt_bias), f(A_log), Bm, Cm, f(D), z, state, req_slots, seq_lens, cu_q, out)
        return out
    return torch_ref.mamba1_scan(u, dt_raw, dt_bias, A_log, Bm, Cm, D, z, state, req_slots, seq_lens, q_lens, out_dtype)


def activation(x: torch.Tensor, kind: str, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """element-wise ``silu`` or ``gelu_tanh`` (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))) of a [T, n] tensor or column view, fp32 math,
    into a contiguous tensor of ``out_dtype`` (csrc/kernels/elementwise.cu)"""
    out_dtype = out_dtype or x.dtype
    if _use_native(x) and x.dim() == 2 and x.stride(1) == 1 and x.dtype in (torch.bfloat16, torch.float32) and out_dtype in (torch.bfloat16, torch.float32):
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        torch.ops.sglb.activation(x, {"silu": 0, "gelu_tanh": 2}[kind], out)
        return out
    xf = x.float()
    y = torch.nn.functional.silu(xf) if kind == "silu" else torch.nn.functional.gelu(xf, approximate="tanh")
    return y.to(out_dtype)


# ------------------------------------------------------------------ rotated values / parallel blocks / rotary latent attention / exponentially gated matrix memory
def rotate_heads(o: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, Dv: int, interleaved: bool = False, inverse: bool = True,
                 lse: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """o [T, H, >= Dv] -> [T, H * Dv]: the heads of an attention output turned over their whole width by ``-+ position * inv_freq[m]`` (fp32
    angle, sine and cosine; pairs half a head apart or, ``interleaved``, neighbours), after ``o * sigmoid(lse - sink_h)`` when the attention
    returned the log-sum-exp of its scores; drops zero padding behind ``Dv`` (csrc/kernels/window_attention.cu).  Values cached with the
    rotation of their own position (``attention_prepare(v_inv_freq=...)``) come out relative to the query's."""
    T, H = o.shape[0], o.shape[1]
    if (_use_native(o) and o.dtype in (torch.bfloat16, torch.float32) and o.is_contiguous() and Dv % 2 == 0
            and (lse is None or (lse.dtype == torch.float32 and lse.is_contiguous()))):
        if out is None:
            out = torch.empty(T, H * Dv, dtype=o.dtype, device=o.device)
        assert out.dtype == o.dtype and out.is_contiguous()
        torch.ops.sglb.rotate_heads(o, positions, inv_freq, int(Dv), bool(interleaved), bool(inverse), lse,
                                    None if lse is None else sinks.float().contiguous(), out)
        return out
    y = torch_ref.rotate_heads(o, positions, inv_freq, Dv, interleaved, inverse, lse, sinks)
    if out is not None:
        out.copy_(y)
        return out
    return y


def causal_softmax(scores: torch.Tensor, tq: int, first: int, scale: float, out_dtype: torch.dtype) -> torch.Tensor:
    """soft-max weights of raw scores under a causal limit, for attention that runs as two matrix products around it: ``scores`` fp32 [R, n]
    contiguous, row ``r = h * tq + i`` sees keys ``j <= first + i``; scale, maximum, exponential and sum in fp32, weights out in ``out_dtype``
    (csrc/kernels/window_attention.cu)"""
    if _use_native(scores) and scores.dtype == torch.float32 and scores.dim() == 2 and scores.is_contiguous() and out_dtype in (torch.bfloat16, torch.float32):
        out = torch.empty(scores.shape, dtype=out_dtype, device=scores.device)
        torch.ops.sglb.causal_softmax(scores, int(tq), int(first), float(scale), out)
        return out
    return torch_ref.causal_softmax(scores, tq, first, scale, out_dtype)


def parallel_add_rmsnorm_f32(residual: torch.Tensor, deltas, w1: torch.Tensor, w2: Optional[torch.Tensor], eps: float, zero_centred: bool = False,
                             out_dtype: torch.dtype = torch.bfloat16, extra: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """fp32 residual stream of blocks whose branches read the same input: ``residual += sum(deltas) + extra`` (in place; ``deltas``: up to two
    branch outputs in the model dtype, ``extra``: one fp32 tensor, e.g. an embedding added again) and the RMS norm of the new residual under
    TWO weights (the second may be None), one kernel (csrc/kernels/residual_f32.cu).  Returns (norm * g(w1), norm * g(w2) | None) in
    ``out_dtype``."""
    deltas = [d for d in deltas if d is not None]
    if (_use_native(residual) and residual.dtype == torch.float32 and residual.is_contiguous() and out_dtype in (torch.bfloat16, torch.float32)
            and len(deltas) <= 2 and all(d.dtype == out_dtype and d.is_contiguous() for d in deltas)
            and (extra is None or (extra.dtype == torch.float32 and extra.is_contiguous())) and w1.dtype == out_dtype
            and (w2 is None or w2.dtype == out_dtype)):
        o1 = torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
        o2 = torch.empty_like(o1) if w2 is not None else None
        torch.ops.sglb.parallel_add_rmsnorm_f32(residual, deltas[0] if deltas else None, deltas[1] if len(deltas) > 1 else None, extra, w1, w2, o1, o2,
                                                float(eps), bool(zero_centred))
        return o1, o2
    return torch_ref.parallel_add_rmsnorm_f32(residual, deltas + ([extra] if extra is not None else []), w1, w2, eps, zero_centred, out_dtype)


def glu_activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    """[gate | up] halves -> act(gate) * up with ``silu`` or ``gelu_tanh``, fp32 math, bf16 or fp32 tensors (csrc/kernels/elementwise.cu)"""
    if _use_native(x) and x.dim() == 2 and x.is_contiguous() and x.dtype in (torch.bfloat16, torch.float32) and x.shape[1] % 2 == 0:
        out = torch.empty(x.shape[0], x.shape[1] // 2, dtype=x.dtype, device=x.device)
        F_ = x.shape[1] // 2
        torch.ops.sglb.activation(x[:, :F_], {"silu": 0, "gelu_tanh": 2}[kind], out, x[:, F_:])
        return out
    return torch_ref.glu_activation(x, kind)


def latent_prepare(x: torch.Tensor, q_rank: int, q_norm_w: Optional[torch.Tensor], rank: int, rot_dim: int, kv_norm_w: torch.Tensor, eps: float,
                   positions: torch.Tensor, inv_freq: Optional[torch.Tensor], mult: float, cache: torch.Tensor,
                   out_cache_loc: torch.Tensor) -> Optional[torch.Tensor]:
    """what lies behind the down-projections of latent attention, one pass per token: RMS norm of the query latent (returned) and of the
    key / value latent (into the first ``rank`` columns of the token's cache row), and the shared rotary key turned by position into the
    next ``rot_dim`` columns (csrc/kernels/latent_attention.cu; semantics in ``torch_ref.latent_prepare``).  ``x`` may be a column view."""
    if (_use_native(x) and x.dtype in (torch.bfloat16, torch.float32) and x.stride(1) == 1 and cache.dtype == x.dtype and cache.stride(-1) == 1
            and kv_norm_w.dtype == x.dtype and (q_norm_w is None or q_norm_w.dtype == x.dtype) and rot_dim % 2 == 0):
        cq = torch.empty(x.shape[0], q_rank, dtype=x.dtype, device=x.device) if q_rank > 0 else None
        torch.ops.sglb.latent_prepare(x, int(q_rank), q_norm_w, int(rank), int(rot_dim), kv_norm_w, float(eps), positions, inv_freq, float(mult), cache,
                                      out_cache_loc, cq)
        return cq
    return torch_ref.latent_prepare(x, q_rank, q_norm_w, rank, rot_dim, kv_norm_w, eps, positions, inv_freq, mult, cache, out_cache_loc)


def latent_query(q: torch.Tensor, q_abs: torch.Tensor, dim: int, rot_dim: int, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                 mult: float = 1.0) -> torch.Tensor:
    """assembles the query of absorbed latent attention with a rotary part: [q_abs (fp32 [H, T, rank]) | rotary columns of q turned by
    position] -> fp32 [T, H, rank + rot_dim] (csrc/kernels/latent_attention.cu; semantics in ``torch_ref.latent_query``)"""
    if (_use_native(q) and q.dtype in (torch.bfloat16, torch.float32) and q.is_contiguous() and q_abs.dtype == torch.float32 and q_abs.is_contiguous()
            and rot_dim % 2 == 0):
        T, H = q.shape[0], q.shape[1]
        out = torch.empty(T, H, q_abs.shape[2] + rot_dim, dtype=torch.float32, device=q.device)
        torch.ops.sglb.latent_query(q, q_abs, int(dim), int(rot_dim), positions, inv_freq, float(mult), out)
        return out
    return torch_ref.latent_query(q, q_abs, dim, rot_dim, positions, inv_freq, mult)


def mlstm_prepare(proj: torch.Tensor, gates_raw: torch.Tensor, H: int, D: int, Dv: int, cap: float, mstate: torch.Tensor, req_slots: torch.Tensor,
                  seq_lens: torch.Tensor, cu_q: Optional[torch.Tensor], q_lens: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """inputs of the exponentially gated matrix memory (mLSTM) for ``mamba2_scan(gates=...)``: the scan's [x | B | C] rows in fp32 (values with
    a column of ones per head, keys, scaled queries) and, from the capped gate pre-activations and the running maximum carried in ``mstate``,
    every token's (decay, input scale, denominator floor) (csrc/kernels/mamba.cu; semantics in ``torch_ref.mlstm_prepare``).  ``proj`` may be
    a column view of a wider projection."""
    if (_use_native(proj) and proj.dtype in (torch.bfloat16, torch.float32) and proj.stride(1) == 1 and gates_raw.dtype == torch.float32
            and gates_raw.is_contiguous() and mstate.dtype == torch.float32 and mstate.is_contiguous() and req_slots.numel() <= 65535):
        T = proj.shape[0]
        u = torch.empty(T, H * (Dv + 1) + 2 * H * D, dtype=torch.float32, device=proj.device)
        gates = torch.empty(T, H, 3, dtype=torch.float32, device=proj.device)
        torch.ops.sglb.mlstm_prepare(proj, gates_raw, int(H), int(D), int(Dv), float(cap), mstate, req_slots, seq_lens, cu_q, u, gates)
        return u, gates
    return torch_ref.mlstm_prepare(proj, gates_raw, H, D, Dv, cap, mstate, req_slots, seq_lens, q_lens)


def mlstm_readout(y: torch.Tensor, gates: torch.Tensor, H: int, Dv: int, norm_w: torch.Tensor, eps: float, gate: Optional[torch.Tensor],
                  out_dtype: torch.dtype) -> torch.Tensor:
    """read-out of the exponentially gated matrix memory: division by the floored normaliser, per-head unit RMS, weight, sigmoid gate, cast
    (csrc/kernels/mamba.cu; semantics in ``torch_ref.mlstm_readout``).  ``gate`` may be a column view."""
    if (_use_native(y) and y.dtype == torch.float32 and y.is_contiguous() and gates.dtype == torch.float32 and gates.is_contiguous()
            and out_dtype in (torch.bfloat16, torch.float32) and norm_w.dtype == out_dtype and (gate is None or (gate.dtype == out_dtype and gate.stride(1) == 1))):
        out = torch.empty(y.shape[0], H * Dv, dtype=out_dtype, device=y.device)
        torch.ops.sglb.mlstm_readout(y, gates, int(H), int(Dv), norm_w, float(eps), gate, out)
        return out
    return torch_ref.mlstm_readout(y, gates, H, Dv, norm_w, eps, gate, out_dtype)
