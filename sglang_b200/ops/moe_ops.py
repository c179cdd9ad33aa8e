"""MoE ops: routing (top-k softmax), token alignment by expert, grouped expert MLP.

GPU path: ``topk_softmax`` / ``moe_align`` / ``grouped_gemm`` from ``csrc/kernels/moe.cu`` when built (own kernels:
warp-per-token routing, counting-sort alignment to 128-row tiles, tcgen05 grouped GEMM that walks a tile->expert
map); otherwise a sort + per-expert GEMM loop.  CPU: ``torch_ref.fused_moe``.
Reference: ``moe_topk_softmax_kernels.cu:628-715``, ``moe_align_kernel.cu:350-386``, ``fused_moe_triton_kernels.py:324``.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import silu_and_mul, linear, torch_ref


def _has(op: str) -> bool:
    return hasattr(torch.ops, "sglb") and hasattr(torch.ops.sglb, op)


def topk_softmax(router_logits: torch.Tensor, top_k: int, renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    if router_logits.is_cuda and _has("moe_topk_softmax") and router_logits.shape[1] <= 512 and top_k <= 32:
        T = router_logits.shape[0]
        w = torch.empty(T, top_k, dtype=torch.float32, device=router_logits.device)
        ids = torch.empty(T, top_k, dtype=torch.int32, device=router_logits.device)
        torch.ops.sglb.moe_topk_softmax(router_logits, w, ids, renormalize)
        return w, ids
    return torch_ref.moe_topk_softmax(router_logits, top_k, renormalize)


def fused_moe(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor,
              expert_offset: int = 0, act=None) -> torch.Tensor:
    """``act``: None = silu(gate) * up; ``("clamped_glu", limit, alpha)`` = min(g, limit) * sigmoid(alpha g) * (clamp(u, +-limit) + 1)"""
    fn = None
    if act is not None:
        kind, limit, alpha = act
        assert kind == "clamped_glu", kind
        from . import clamped_glu

        fn = lambda gu: clamped_glu(gu.contiguous(), limit, alpha)
    if not x.is_cuda:
        return torch_ref.fused_moe(x, w13, w2, topk_w, topk_ids, expert_offset, fn)
    H, I = x.shape[1], w2.shape[2]
    if (act is not None and x.dtype == torch.bfloat16 and _has("moe_grouped_mlp_glu") and H % 32 == 0 and I % 16 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0):
        # expert-sorted rows through the tcgen05 grouped GEMMs, no host sync: align -> gather -> gate|up GEMM -> clamped GLU -> down GEMM -> combine
        out = torch.empty_like(x)
        torch.ops.sglb.moe_grouped_mlp_glu(x, w13, w2, topk_w, topk_ids, out, expert_offset, float(limit), float(alpha))
        return out
    if act is None and x.dtype == torch.bfloat16 and _has("moe_grouped_mlp") and H % 32 == 0 and I % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0:
        out = torch.empty_like(x)
        torch.ops.sglb.moe_grouped_mlp(x, w13, w2, topk_w, topk_ids, out, expert_offset)
        return out
    return _fused_moe_sorted(x, w13, w2, topk_w, topk_ids, expert_offset, fn)


def _fused_moe_sorted(x, w13, w2, topk_w, topk_ids, expert_offset, act=None):
    """sort (token, k) pairs by expert, run one GEMM pair per local expert on its contiguous slice, scatter-add."""
    T, H = x.shape
    E = w13.shape[0]
    K = topk_ids.shape[1]
    flat = topk_ids.reshape(-1).long() - expert_offset
    local = (flat >= 0) & (flat < E)
    key = torch.where(local, flat, torch.full_like(flat, E))
    order = torch.argsort(key, stable=True)
    counts = torch.bincount(key, minlength=E + 1)[:E].tolist()   # host sync: acceptable off the graph path
    tok = (order // K)
    xs = x.index_select(0, tok[: sum(counts)])
    ws = topk_w.reshape(-1)[order[: sum(counts)]].to(torch.float32)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    off = 0
    for e, c in enumerate(counts):
        if c == 0:
            continue
        h = linear(xs[off:off + c], w13[e])
        h = silu_and_mul(h) if act is None else act(h)
        y = linear(h, w2[e]).float() * ws[off:off + c, None]
        out.index_add_(0, tok[off:off + c], y)
        off += c
    return out.to(x.dtype)


def softmax_bias_route(logits: torch.Tensor, correction, top_k: int, n_real: int):
    """soft-max scores over real and identity experts, choice by ``score + correction``, weights = the chosen plain scores (warp-per-token
    kernel in csrc/kernels/moe.cu; semantics in ``torch_ref.softmax_bias_route``) -> (weights, ids, summed weight of the identity picks)"""
    T, E = logits.shape
    if logits.is_cuda and _has("moe_softmax_bias_route") and logits.dtype == torch.float32 and logits.stride(1) == 1 and E <= 1024 and top_k <= 32:
        w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
        ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
        ident = torch.empty(T, dtype=torch.float32, device=logits.device)
        torch.ops.sglb.moe_softmax_bias_route(logits, None if correction is None else correction.float().contiguous(), int(n_real), w, ids, ident)
        return w, ids, ident
    return torch_ref.softmax_bias_route(logits, correction, top_k, n_real)


def moe_identity_shared_combine(y: torch.Tensor, h: torch.Tensor, ident_w, shared, shared_logit) -> torch.Tensor:
    """y + ident_w * h + sigmoid(shared_logit) * shared, rows of [T, width] (identity experts return their input; the always-on expert is gated
    by one number per token, or joins ungated when ``shared_logit`` is None); fp32 sums (csrc/kernels/moe.cu)"""
    if ident_w is None and shared is None:
        return y
    if y.is_cuda and _has("moe_identity_shared_combine") and y.dtype in (torch.bfloat16, torch.float32) and y.is_contiguous() and h.is_contiguous() \
            and h.dtype == y.dtype and (shared is None or (shared.is_contiguous() and shared.dtype == y.dtype)):
        torch.ops.sglb.moe_identity_shared_combine(y, h, None if ident_w is None else ident_w.float().contiguous(), shared,
                                                   None if shared is None or shared_logit is None else shared_logit.float().contiguous())
        return y
    out = y.float()
    if ident_w is not None:
        out = out + ident_w.float()[:, None] * h.float()
    if shared is not None:
        out = out + (torch.sigmoid(shared_logit.float()).reshape(-1, 1) * shared.float() if shared_logit is not None else shared.float())
    return out.to(y.dtype)
