"""Plain-PyTorch fp32 reference of every hot op.

Two jobs: (1) the numerics oracle every CUDA kernel test compares against (tests/test_kernels_gpu.py),
(2) the CPU execution path for the no-GPU test tier (reference analogue:
``python/sglang/srt/layers/attention/torch_native_backend.py`` and the ``forward_native`` methods).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps) * weight.float()).to(x.dtype)


def fused_add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """residual <- x + residual ; x <- rmsnorm(residual) * w   (both in place)"""
    s = x.float() + residual.float()
    residual.copy_(s.to(residual.dtype))
    sf = residual.float()
    var = sf.pow(2).mean(-1, keepdim=True)
    x.copy_((sf * torch.rsqrt(var + eps) * weight.float()).to(x.dtype))


def gemma_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps) * (1.0 + weight.float())).to(x.dtype)


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps).to(x.dtype)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    return (F.silu(x[..., :d].float()) * x[..., d:].float()).to(x.dtype)


def gelu_and_mul(x: torch.Tensor, approximate: str = "none") -> torch.Tensor:
    d = x.shape[-1] // 2
    return (F.gelu(x[..., :d].float(), approximate=approximate) * x[..., d:].float()).to(x.dtype)


def build_cos_sin_cache(head_dim: int, max_pos: int, base: float = 10000.0, rope_scaling: Optional[dict] = None,
                        rotary_dim: Optional[int] = None) -> torch.Tensor:
    """[max_pos, rotary_dim] fp32: cos | sin halves (reference rotary_embedding/base.py; llama3 scaling
    ``rotary_embedding/*`` llama3 variant)"""
    rd = rotary_dim or head_dim
    inv_freq = 1.0 / (base ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
    if rope_scaling and rope_scaling.get("rope_type", rope_scaling.get("type")) == "llama3":
        factor = rope_scaling.get("factor", 8.0)
        lo = rope_scaling.get("low_freq_factor", 1.0)
        hi = rope_scaling.get("high_freq_factor", 4.0)
        old = rope_scaling.get("original_max_position_embeddings", 8192)
        wavelen = 2 * math.pi / inv_freq
        smooth = (old / wavelen - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv_freq / factor,
                             torch.where(wavelen < old / hi, inv_freq, (1 - smooth) * inv_freq / factor + smooth * inv_freq))
        inv_freq = scaled
    elif rope_scaling and rope_scaling.get("rope_type", rope_scaling.get("type")) == "linear":
        inv_freq = inv_freq / rope_scaling.get("factor", 1.0)
    mscale = 1.0
    kind = (rope_scaling or {}).get("rope_type", (rope_scaling or {}).get("type"))
    if kind in ("yarn", "deepseek_yarn"):
        # YaRN (reference rotary_embedding yarn / deepseek_yarn): interpolate the low frequencies by ``factor``, keep the high ones, blend
        # linearly between the two correction dims; cos / sin carry the attention temperature ("mscale")
        rs = rope_scaling
        factor = float(rs.get("factor", 1.0))
        old = rs.get("original_max_position_embeddings", max_pos)
        fast, slow = rs.get("beta_fast", 32), rs.get("beta_slow", 1)
        corr = lambda rot: (rd * math.log(old / (rot * 2 * math.pi))) / (2 * math.log(base))
        lo, hi = corr(fast), corr(slow)
        if rs.get("truncate", True):
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, rd - 1)
        if lo == hi:
            hi += 0.001
        ramp = ((torch.arange(rd // 2, dtype=torch.float32) - lo) / (hi - lo)).clamp(0, 1)
        extrap_mask = 1 - ramp
        inv_freq = inv_freq / factor * (1 - extrap_mask) + inv_freq * extrap_mask
        get_ms = lambda sc, m=1.0: 1.0 if sc <= 1 else 0.1 * m * math.log(sc) + 1.0
        if rs.get("attention_factor") is not None:
            mscale = float(rs["attention_factor"])
        elif rs.get("mscale") and rs.get("mscale_all_dim"):
            mscale = get_ms(factor, rs["mscale"]) / get_ms(factor, rs["mscale_all_dim"])
        else:
            mscale = get_ms(factor)
    elif kind in ("longrope", "su"):
        # Phi-3 LongRoPE: per-dimension rescale factors (short / long table chosen by the served context length)
        rs = rope_scaling
        old = rs.get("original_max_position_embeddings", max_pos)
        ext = torch.tensor(rs["long_factor"] if max_pos > old else rs["short_factor"], dtype=torch.float32)
        inv_freq = inv_freq / ext
        sc = max_pos / old
        mscale = 1.0 if sc <= 1.0 else math.sqrt(1 + math.log(sc) / math.log(old))
    elif kind == "dynamic":
        # dynamic NTK evaluated at the served context length (static table: one base for all positions)
        rs = rope_scaling
        factor = float(rs.get("factor", 1.0))
        old = rs.get("original_max_position_embeddings", max_pos)
        if max_pos > old:
            nb = base * ((factor * max_pos / old) - (factor - 1)) ** (rd / (rd - 2))
            inv_freq = 1.0 / (nb ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
    t = torch.arange(max_pos, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq)
    return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor, is_neox: bool = True) -> torch.Tensor:
    """x [T, H, D]; rotary over the first rotary_dim = cos_sin.shape[1] dims"""
    rd = cos_sin.shape[1]
    cs = cos_sin.to(x.device)[positions.long()]
    cos, sin = cs[:, : rd // 2].unsqueeze(1).float(), cs[:, rd // 2:].unsqueeze(1).float()
    xr, xp = x[..., :rd].float(), x[..., rd:]
    if is_neox:
        x1, x2 = xr[..., : rd // 2], xr[..., rd // 2:]
        o = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
    else:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        o = torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).flatten(-2)
    return torch.cat([o.to(x.dtype), xp], dim=-1)


def rope_kv_write(q, k, v, positions, cos_sin, k_cache, v_cache, out_cache_loc, is_neox=True,
                  k_scale: float = 1.0, v_scale: float = 1.0) -> None:
    q.copy_(apply_rope(q, positions, cos_sin, is_neox))
    k.copy_(apply_rope(k, positions, cos_sin, is_neox))
    loc = out_cache_loc.long()
    if k_cache.dtype == torch.float8_e4m3fn:
        k_cache[loc] = (k.float() / k_scale).to(k_cache.dtype)
        v_cache[loc] = (v.float() / v_scale).to(v_cache.dtype)
    else:
        k_cache[loc] = k.to(k_cache.dtype)
        v_cache[loc] = v.to(v_cache.dtype)


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                    req_slots: torch.Tensor, seq_lens: torch.Tensor, q_lens: Optional[torch.Tensor], page_size: int,
                    scale: float, causal: bool = True, window: int = -1, logit_cap: float = 0.0,
                    k_scale: float = 1.0, v_scale: float = 1.0, custom_mask: Optional[torch.Tensor] = None,
                    return_lse: bool = False):
    """q [T, Hq, D] (ragged: request b owns q_lens[b] rows); caches [slots, Hkv, D].
    The KV of the current tokens is already in the cache (positions seq_len-q_len .. seq_len-1)."""
    T, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    g = Hq // Hkv
    B = req_slots.shape[0]
    out = q.new_empty(T, Hq, v_cache.shape[-1])          # (the value width may differ from the key width: MLA latent rows)
    lse = torch.empty(T, Hq, dtype=torch.float32, device=q.device)
    qs = 0
    mask_off = 0
    for b in range(B):
        L = int(seq_lens[b])
        ql = 1 if q_lens is None else int(q_lens[b])
        npg = (L + page_size - 1) // page_size
        pages = page_table[int(req_slots[b]), :npg].long()
        slots = (pages[:, None] * page_size + torch.arange(page_size, device=q.device)[None, :]).reshape(-1)[:L]
        K = k_cache[slots].float() * k_scale   # [L, Hkv, D]
        V = v_cache[slots].float() * v_scale
        Q = q[qs:qs + ql].float()              # [ql, Hq, D]
        Kx = K.repeat_interleave(g, dim=1)
        Vx = V.repeat_interleave(g, dim=1)
        s = torch.einsum("qhd,khd->hqk", Q, Kx) * scale
        if logit_cap > 0:
            s = logit_cap * torch.tanh(s / logit_cap)
        qpos = torch.arange(L - ql, L, device=q.device)[:, None]
        kpos = torch.arange(L, device=q.device)[None, :]
        if custom_mask is not None:
            m = custom_mask[mask_off:mask_off + ql * L].view(ql, L).bool()
            mask_off += ql * L
            s = s.masked_fill(~m[None], float("-inf"))
        else:
            if causal:
                s = s.masked_fill((kpos > qpos)[None], float("-inf"))
            if window > 0:
                s = s.masked_fill((kpos <= qpos - window)[None], float("-inf"))
        l = torch.logsumexp(s, dim=-1)         # [Hq, ql]
        p = torch.exp(s - l[..., None])
        o = torch.einsum("hqk,khd->qhd", p, Vx)
        out[qs:qs + ql] = o.to(q.dtype)
        lse[qs:qs + ql] = l.transpose(0, 1)
        qs += ql
    return (out, lse) if return_lse else out


def merge_attn_states(o1, lse1, o2, lse2):
    """LSE-weighted merge of two partial attention results (reference merge_attn_states.cu:126)"""
    m = torch.maximum(lse1, lse2)
    w1, w2 = torch.exp(lse1 - m), torch.exp(lse2 - m)
    o = (o1.float() * w1[..., None] + o2.float() * w2[..., None]) / (w1 + w2)[..., None]
    return o.to(o1.dtype), m + torch.log(w1 + w2)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return F.linear(x, w, bias)


# ------------------------------------------------------------------ sampling
def top_k_top_p_min_p_probs(probs: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor, min_p: torch.Tensor) -> torch.Tensor:
    """renormalised probabilities after top-k -> top-p -> min-p filtering (fp32)"""
    sp, idx = probs.sort(dim=-1, descending=True)
    csum = sp.cumsum(-1)
    V = probs.shape[-1]
    rank = torch.arange(V, device=probs.device)[None, :]
    keep = rank < top_k.clamp(max=V)[:, None]
    keep &= (csum - sp) < top_p[:, None]
    keep &= sp >= (sp[:, :1] * min_p[:, None])
    sp = torch.where(keep, sp, torch.zeros_like(sp))
    sp = sp / sp.sum(-1, keepdim=True)
    return torch.zeros_like(probs).scatter_(1, idx, sp)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor) -> torch.Tensor:
    """inverse-CDF sampling in sorted-prob order with one uniform per row; top_k==1 rows are argmax"""
    lf = logits.float()
    greedy = top_k == 1
    probs = torch.softmax(lf / temperature.clamp(min=1e-6)[:, None], dim=-1)
    p = top_k_top_p_min_p_probs(probs, top_k, top_p, min_p)
    sp, idx = p.sort(dim=-1, descending=True)
    c = sp.cumsum(-1)
    pick = (c < uniform[:, None] * c[:, -1:]).sum(-1).clamp(max=logits.shape[-1] - 1)
    tok = idx.gather(1, pick[:, None]).squeeze(1)
    return torch.where(greedy, lf.argmax(-1), tok)


def apply_token_bitmask(logits: torch.Tensor, bitmask: torch.Tensor) -> None:
    """bitmask int32 [B, ceil(V/32)], bit=1 allowed (xgrammar convention; reference
    apply_token_bitmask_inplace_cuda.cu:157)"""
    V = logits.shape[-1]
    bits = ((bitmask[:, :, None] >> torch.arange(32, device=bitmask.device, dtype=torch.int32)[None, None, :]) & 1)
    allowed = bits.reshape(bitmask.shape[0], -1)[:, :V].bool()
    logits.masked_fill_(~allowed, float("-inf"))


def apply_penalties(logits, output_counts, prompt_mask, freq_pen, pres_pen, rep_pen) -> None:
    lf = logits.float()
    seen = (output_counts > 0) | prompt_mask
    lf = torch.where(seen & (rep_pen[:, None] != 1.0), torch.where(lf > 0, lf / rep_pen[:, None], lf * rep_pen[:, None]), lf)
    lf = lf - freq_pen[:, None] * output_counts.float() - pres_pen[:, None] * (output_counts > 0).float()
    logits.copy_(lf.to(logits.dtype))


# ------------------------------------------------------------------ MoE
def moe_topk_softmax(router_logits: torch.Tensor, top_k: int, renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    p = torch.softmax(router_logits.float(), dim=-1)
    w, ids = p.topk(top_k, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, ids.to(torch.int32)


def fused_moe(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor,
              expert_offset: int = 0, act=None) -> torch.Tensor:
    """x [T,H]; w13 [E_local, 2I, H]; w2 [E_local, H, I]; ids are global expert ids; experts outside
    [expert_offset, expert_offset+E_local) contribute zero (EP)."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    E = w13.shape[0]
    for e in range(E):
        sel = (topk_ids == e + expert_offset)
        tok, kk = sel.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = F.linear(x[tok], w13[e])
        h = silu_and_mul(h) if act is None else act(h)
        y = F.linear(h, w2[e]).float()
        out.index_add_(0, tok, y * topk_w[tok, kk].float()[:, None])
    return out.to(x.dtype)


# ------------------------------------------------------------------ quantisation
FP8_MAX = 448.0


def per_token_group_quant_fp8(x: torch.Tensor, group: int = 128, ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    T, K = x.shape
    xg = x.float().view(T, K // group, group)
    amax = xg.abs().amax(-1).clamp(min=1e-10)
    s = amax / FP8_MAX
    if ue8m0:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    q = (xg / s[..., None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(T, K)
    return q, s


def block_quant_weight_fp8(w: torch.Tensor, block: int = 128, ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    wb = wp.view(nb, block, kb, block)
    amax = wb.abs().amax(dim=(1, 3)).clamp(min=1e-10)
    s = amax / FP8_MAX
    if ue8m0:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    q = (wb / s[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(nb * block, kb * block)[:N, :K]
    return q.contiguous(), s


def fp8_block_gemm(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, block: int = 128,
                   out_dtype=torch.bfloat16) -> torch.Tensor:
    T, K = xq.shape
    N = wq.shape[0]
    x = xq.float().view(T, K // block, block) * xs[..., None]
    wsf = ws.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    w = wq.float() * wsf
    return (x.view(T, K) @ w.t()).to(out_dtype)


def tree_anc_to_mask(tree_anc: torch.Tensor, q_lens: torch.Tensor, seq_lens: torch.Tensor) -> torch.Tensor:
    """dense custom mask (flat, per request [q_len, seq_len] row-major) from per-node ancestor bits: keys below the prefix are visible to
    every node, draft key ``prefix + k`` iff bit k of the node's word is set (speculative token-tree verification)"""
    out = []
    anc = tree_anc.to(torch.int64) & 0xFFFFFFFF
    off = 0
    for ql, L in zip(q_lens.tolist(), seq_lens.tolist()):
        p = L - ql
        m = torch.ones(ql, L, dtype=torch.bool, device=tree_anc.device)
        bits = (anc[off:off + ql, None] >> torch.arange(ql, device=tree_anc.device)[None, :]) & 1
        m[:, p:] = bits.bool()
        out.append(m.reshape(-1))
        off += ql
    return torch.cat(out) if out else torch.zeros(0, dtype=torch.bool, device=tree_anc.device)


def causal_conv1d(x: torch.Tensor, w: torch.Tensor, bias, conv_state: torch.Tensor, cu_q, req_slots: torch.Tensor, seq_lens: torch.Tensor,
                  silu: bool = True) -> torch.Tensor:
    """ragged causal depthwise conv with a rolling per-request state (in place): x [T, C], w [C, k], conv_state [slots, C, k-1] -> fp32 [T, C].
    ``cu_q`` None = decode (one token per request)."""
    import torch.nn.functional as F

    T, C = x.shape
    k = w.shape[1]
    out = torch.empty(T, C, dtype=torch.float32, device=x.device)
    B = req_slots.numel()
    cu = cu_q.tolist() if cu_q is not None else list(range(B + 1))
    sl = seq_lens.tolist()
    slots = req_slots.tolist()
    for b in range(B):
        q0, n = cu[b], cu[b + 1] - cu[b]
        if n <= 0:
            continue
        s = slots[b]
        prev = torch.zeros_like(conv_state[s]) if sl[b] - n == 0 else conv_state[s]
        seq = torch.cat([prev.t(), x[q0:q0 + n]], 0)                       # [k-1+n, C]
        conv_state[s] = seq[-(k - 1):].t()
        u = F.conv1d(seq.t().unsqueeze(0).float(), w.float().unsqueeze(1), bias.float() if bias is not None else None, groups=C)[0].t()
        out[q0:q0 + n] = F.silu(u) if silu else u
    return out


def selective_state_update(state: torch.Tensor, req_slots: torch.Tensor, x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, Bm: torch.Tensor,
                           Cm: torch.Tensor, D) -> torch.Tensor:
    """state fp32 [slots, H, P, N] (in place); x [B, H*P], dt [B, H], A [H], Bm / Cm [B, G*N], D [H] or None -> y fp32 [B, H, P]"""
    Bn = req_slots.numel()
    H, P, N = state.shape[1:]
    G = Bm.shape[1] // N
    rep = H // G
    sl = req_slots.long()
    st = state[sl]
    xh = x.float().view(Bn, H, P)
    dA = torch.exp(dt.float() * A.float()[None, :])
    Bh = Bm.float().reshape(Bn, G, N).repeat_interleave(rep, 1)
    Ch = Cm.float().reshape(Bn, G, N).repeat_interleave(rep, 1)
    st = st * dA[..., None, None] + (dt.float()[..., None] * xh)[..., None] * Bh[:, :, None, :]
    state[sl] = st
    y = torch.einsum("bhpn,bhn->bhp", st, Ch)
    if D is not None:
        y = y + D.float()[None, :, None] * xh
    return y


# ------------------------------------------------------------------ fp32 residual stream, latent attention, gated delta rule, clamped GLU
def add_rmsnorm_f32(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, zero_centred: bool,
                    out_dtype: torch.dtype) -> torch.Tensor:
    """residual (fp32, in place) += delta; returns norm(residual) * (1 + w | w) in ``out_dtype``"""
    if delta is not None:
        residual.add_(delta.float())
    y = residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + eps)
    w = weight.float().reshape(-1)          # one element: one gain for all coordinates
    return (y * (1.0 + w if zero_centred else w)).to(out_dtype)


def clamped_glu(gu: torch.Tensor, limit: float, alpha: float = 1.702) -> torch.Tensor:
    """gu [T, 2I] = [gate | up] -> min(g, limit) * sigmoid(alpha * g) * (clamp(u, -limit, limit) + 1)"""
    I = gu.shape[-1] // 2
    g = gu[..., :I].float().clamp(max=limit)
    u = gu[..., I:].float().clamp(-limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(gu.dtype)


def latent_attention(q_lat: torch.Tensor, cache: torch.Tensor, rank: int, page_table: torch.Tensor, req_slots: torch.Tensor, seq_lens: torch.Tensor,
                     q_lens: Optional[torch.Tensor], page_size: int, scale: float, window: int, sinks: Optional[torch.Tensor],
                     v_rank: Optional[int] = None) -> torch.Tensor:
    """absorbed multi-query attention over cached latent rows.  q_lat fp32 [T, H, rank] (query already multiplied into the key up-projection);
    cache [slots, 1, >= rank]; key j of a request is visible to its query i when ``0 <= i - j < window`` (``window <= 0``: all earlier keys);
    ``sinks`` fp32 [H]: exp(sink_h) joins the soft-max denominator only.  Returns the probability-weighted latent rows, fp32 [T, H, rank].
    ``v_rank < rank``: only the first ``v_rank`` columns of a row are its value (the rest, e.g. a rotary key part, only score); the result is
    [T, H, v_rank]."""
    T, H, R = q_lat.shape
    Rv = R if v_rank is None else int(v_rank)
    out = torch.empty(T, H, Rv, dtype=torch.float32, device=q_lat.device)
    qs = 0
    for b in range(req_slots.shape[0]):
        L = int(seq_lens[b])
        ql = 1 if q_lens is None else int(q_lens[b])
        if ql <= 0:
            continue
        lo = 0 if window <= 0 else max(0, L - ql - window + 1)
        pos = torch.arange(lo, L, device=q_lat.device)
        slots = page_table[int(req_slots[b]), (pos // page_size).long()].long() * page_size + pos % page_size
        C = cache[slots, 0, :R].float()                                    # [n, R]
        s = torch.einsum("qhr,kr->hqk", q_lat[qs:qs + ql].float(), C) * scale
        qpos = torch.arange(L - ql, L, device=q_lat.device)[:, None]
        hide = pos[None, :] > qpos
        if window > 0:
            hide = hide | (pos[None, :] <= qpos - window)
        s = s.masked_fill(hide[None], float("-inf"))
        if sinks is not None:
            s = torch.cat([s, sinks.float()[:, None, None].expand(H, ql, 1)], -1)
        p = torch.softmax(s, dim=-1)[..., : pos.numel()]
        out[qs:qs + ql] = torch.einsum("hqk,kr->qhr", p, C[:, :Rv])
        qs += ql
    return out


def gated_delta_rule(u: torch.Tensor, Hk: int, Dk: int, H: int, Dv: int, a_raw: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor,
                     b_raw: torch.Tensor, state: torch.Tensor, req_slots: torch.Tensor, seq_lens: torch.Tensor, q_lens: Optional[torch.Tensor],
                     gate_raw: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6,
                     gate_act: str = "silu", per_channel: Optional[bool] = None) -> torch.Tensor:
    """Gated delta rule over a ragged batch, token by token, state in place.

    u fp32 [T, 2*Hk*Dk + H*Dv] = short-conv outputs [q | k | v] (not yet normalised); value head h reads q/k head ``h // (H // Hk)``.
    a_raw [T, H] (one decay per head) or [T, H*Dk] (one per head and key channel): decay = exp(-exp(A_log_h) * softplus(a_raw + dt_bias)).
    b_raw [T, H]: beta = sigmoid(b_raw).  state fp32 [slots, H, Dk, Dv]; a request whose ``seq_len == q_len`` starts from zero.
    Per token: S <- decay * S (rows = key channels); w = beta * (v - S^T k); S <- S + k w^T; o = S^T q  (q, k unit vectors, q also / sqrt(Dk)).
    With ``norm_w``: o <- o / rms(o) * norm_w * act(gate_raw) per head (act = silu | sigmoid).  Returns fp32 [T, H, Dv]."""
    T = u.shape[0]
    kd = Hk * Dk
    rep = H // Hk
    q = u[:, :kd].float().view(T, Hk, Dk)
    k = u[:, kd:2 * kd].float().view(T, Hk, Dk)
    v = u[:, 2 * kd:].float().view(T, H, Dv)
    q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * Dk ** -0.5
    k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    if per_channel is None:
        per_channel = a_raw.shape[1] != H
    sp = F.softplus(a_raw.float() + dt_bias.float())
    if per_channel:
        g = torch.exp(-A_log.float().exp()[None, :, None] * sp.view(T, H, Dk))
    else:
        g = torch.exp(-A_log.float().exp()[None, :] * sp)[..., None].expand(T, H, Dk)
    beta = torch.sigmoid(b_raw.float())
    out = torch.empty(T, H, Dv, dtype=torch.float32, device=u.device)
    off = 0
    for b in range(req_slots.shape[0]):
        n = 1 if q_lens is None else int(q_lens[b])
        if n <= 0:
            continue
        slot = int(req_slots[b])
        S = torch.zeros_like(state[slot]) if int(seq_lens[b]) - n == 0 else state[slot].clone()
        for t in range(off, off + n):
            S = S * g[t][..., None]
            w = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
            S = S + k[t][..., None] * w[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, q[t])
        state[slot] = S
        off += n
    if norm_w is not None:
        out = out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
        z = gate_raw.float().view(T, H, Dv)
        out = out * (F.silu(z) if gate_act == "silu" else torch.sigmoid(z))
    return out


# ------------------------------------------------------------------ Zaparax mechanisms: bigram embedding, post-normed residual, Mamba-2 scan, biased window attention
def bigram_embedding(embed: torch.Tensor, bigram: Optional[torch.Tensor], ids: torch.Tensor, prev_tokens: Optional[torch.Tensor], cu_q,
                     req_slots: torch.Tensor, seq_lens: torch.Tensor, scale: float, mul_prev: int, mul_cur: int, buckets: int) -> torch.Tensor:
    """fp32 [T, width] = embed[id] * scale + bigram[(prev * mul_prev + id * mul_cur) mod buckets]; a sequence's first token takes row
    ``buckets``.  ``prev_tokens`` int32 [slots] holds every request's last token between calls (updated in place); ``cu_q`` None = one token per
    request."""
    x = embed[ids.long()].float() * scale
    if bigram is None:
        return x
    B = req_slots.numel()
    cu = cu_q.tolist() if cu_q is not None else list(range(B + 1))
    idl = ids.long()
    prev = torch.roll(idl, 1)
    first = torch.zeros_like(idl, dtype=torch.bool)
    for b in range(B):
        q0, n = cu[b], cu[b + 1] - cu[b]
        if n <= 0:
            continue
        s = int(req_slots[b])
        if int(seq_lens[b]) - n == 0:
            first[q0] = True
        else:
            prev[q0] = prev_tokens[s].long()
        prev_tokens[s] = idl[q0 + n - 1].to(prev_tokens.dtype)
    row = (prev * mul_prev + idl * mul_cur) % buckets
    row = torch.where(first, torch.full_like(row, buckets), row)
    return x + bigram[row].float()


def postnorm_add_rmsnorm_f32(residual: torch.Tensor, delta: Optional[torch.Tensor], post_weight: torch.Tensor, weight: torch.Tensor, eps: float,
                             out_dtype: torch.dtype, zero_centred: bool = True) -> torch.Tensor:
    """residual (fp32, in place) += rmsnorm(delta) * g(post_weight); returns rmsnorm(residual) * g(weight) in ``out_dtype``, with
    ``g(w) = 1 + w`` (``zero_centred``) or ``w``; a weight of one element is one gain for all coordinates"""
    g = (lambda w: 1.0 + w.float().reshape(-1)) if zero_centred else (lambda w: w.float().reshape(-1))
    d = delta.float()
    residual.add_(d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * g(post_weight))
    y = residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + eps)
    return (y * g(weight)).to(out_dtype)


def grouped_rmsnorm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, out_dtype: torch.dtype, gate: Optional[torch.Tensor] = None,
                    out_scale: float = 1.0) -> torch.Tensor:
    """x [T, C] cut into ``groups`` equal parts, each divided by its own root mean square, times weight [C]; with ``gate`` [T, C] also times
    ``sigmoid(gate)``; times ``out_scale``"""
    T, C = x.shape
    xf = x.float().view(T, groups, C // groups)
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).view(T, C) * weight.float()
    if gate is not None:
        y = y * torch.sigmoid(gate.float())
    return (y * out_scale if out_scale != 1.0 else y).to(out_dtype)


def mamba2_scan(u: torch.Tensor, z: Optional[torch.Tensor], dt_raw: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, D: Optional[torch.Tensor],
                state: torch.Tensor, req_slots: torch.Tensor, seq_lens: torch.Tensor, q_lens: Optional[torch.Tensor], H: int, P: int, N: int,
                G: int, decay: Optional[torch.Tensor] = None, gates: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Mamba-2 recurrence over a ragged batch, token by token, state in place.  ``decay`` fp32 [H] (then ``dt_raw``, ``dt_bias`` and ``A_log``
    are not read): the step size is 1 and every head's state shrinks by its constant, S <- decay_h S + B x^T (linear attention with decay).
    ``gates`` fp32 [T, H, >= 2] (likewise): every token brings its own decay ``gates[t, h, 0]`` and step ``gates[t, h, 1]``.

    u fp32 [T, H*P + 2*G*N] = short-conv outputs [x | B | C]; head h reads B / C group ``h // (H // G)``.  dt = softplus(dt_raw + dt_bias) [T, H]
    (no clamp).  state fp32 [slots, H, N, P]; a request whose ``seq_len == q_len`` starts from zero.  Per token and head:
    S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x;  with ``z``: y <- y * silu(z).  Returns fp32 [T, H*P]."""
    T = u.shape[0]
    inner = H * P
    rep = H // G
    x = u[:, :inner].float().view(T, H, P)
    Bm = u[:, inner:inner + G * N].float().view(T, G, N).repeat_interleave(rep, 1)
    Cm = u[:, inner + G * N:inner + 2 * G * N].float().view(T, G, N).repeat_interleave(rep, 1)
    if gates is not None:
        dA, dt = gates[:, :, 0].float(), gates[:, :, 1].float()
    elif decay is not None:
        dt = torch.ones(T, H, dtype=torch.float32, device=u.device)
        dA = decay.float()[None, :].expand(T, H)
    else:
        dt = F.softplus(dt_raw.float() + dt_bias.float(), threshold=1e9)
        dA = torch.exp(-A_log.float().exp()[None, :] * dt)
    out = torch.empty(T, H, P, dtype=torch.float32, device=u.device)
    off = 0
    for b in range(req_slots.shape[0]):
        n = 1 if q_lens is None else int(q_lens[b])
        if n <= 0:
            continue
        slot = int(req_slots[b])
        S = torch.zeros_like(state[slot]) if int(seq_lens[b]) - n == 0 else state[slot].clone()
        for t in range(off, off + n):
            S = S * dA[t][:, None, None] + (dt[t][:, None] * Bm[t])[:, :, None] * x[t][:, None, :]
            out[t] = torch.einsum("hnp,hn->hp", S, Cm[t])
        state[slot] = S
        off += n
    if D is not None:
        out = out + D.float()[None, :, None] * x
    out = out.reshape(T, inner)
    if z is not None:
        out = out * F.silu(z.float())
    return out


def qk_norm_cache_write(qkv: torch.Tensor, H: int, G: int, D: int, Dv: int, positions: torch.Tensor, eps: float, temp_coef: float, temp_every: int,
                        k_cache: torch.Tensor, v_cache: torch.Tensor, out_cache_loc: torch.Tensor, normalise: bool = True, pad: int = 0) -> torch.Tensor:
    """qkv [T, H*D + G*D + G*Dv] -> q [T, H, D] (cache dtype) with every head divided by its root mean square and multiplied by the
    position's query temperature ``1 + coef * ln(floor((p + 1) / every) + 1)``; the heads of k (same unit-RMS form) go to the first
    ``G*D`` columns of ``k_cache[loc]`` and v to the first ``G*Dv`` columns of ``v_cache[loc]`` (caches [slots, 1, width]).
    ``pad > 0``: every head of q, k and v occupies ``pad`` columns, zeros behind its values (q is [T, H, pad])."""
    T = qkv.shape[0]
    q = qkv[:, :H * D].float().view(T, H, D)
    k = qkv[:, H * D:H * D + G * D].float().view(T, G, D)
    v = qkv[:, H * D + G * D:].float()
    if normalise:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps)
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps)
    if temp_coef != 0.0:
        p1 = positions.long() + 1
        q = q * (1.0 + temp_coef * torch.log((p1 // int(temp_every)).float() + 1.0))[:, None, None]
    loc = out_cache_loc.long()
    if pad > 0:
        zp = lambda t, n: torch.nn.functional.pad(t, (0, pad - n))
        k_cache[loc, 0, :G * pad] = zp(k, D).reshape(T, G * pad).to(k_cache.dtype)
        v_cache[loc, 0, :G * pad] = zp(v.view(T, G, Dv), Dv).reshape(T, G * pad).to(v_cache.dtype)
        return zp(q, D).to(k_cache.dtype)
    k_cache[loc, 0, :G * D] = k.reshape(T, G * D).to(k_cache.dtype)
    v_cache[loc, 0, :G * Dv] = v.to(v_cache.dtype)
    return q.to(k_cache.dtype)


def window_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, G: int, Dv: int, page_table: torch.Tensor, req_slots: torch.Tensor,
                     seq_lens: torch.Tensor, q_lens: Optional[torch.Tensor], page_size: int, scale: float, softcap: float, window: int,
                     slopes: Optional[torch.Tensor], sinks: Optional[torch.Tensor], dim: int = 0, pad: int = 0, keep_first: int = 0,
                     log_rates: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> torch.Tensor:
    """grouped-query attention over a paged cache with a tanh score cap, a per-head distance bias, a sliding window and soft-max sinks.
    ``pad > 0``: q is [T, H, pad] and every key / value head occupies ``pad`` cache columns, of which the first ``dim`` / ``Dv`` count.
    ``keep_first``: with a window, the sequence's first ``keep_first`` positions stay visible to every later query.  ``log_rates`` fp32 [H]:
    the distance bias is ``slopes_h * ln(1 + log_rates_h * (i - j))`` instead of linear.  ``gate`` [T, H] or [T, H*Dv]: the output is
    multiplied by ``sigmoid(gate)`` per head or per element; ``out_scale`` multiplies it once more.

    q [T, H, D]; caches [slots, 1, width] with the G key heads in the first ``G*D`` columns (values: ``G*Dv``); query head h reads key head
    ``h // (H // G)``.  score_ij = cap(q_i . k_j * scale) - slopes_h * (i - j) with cap(s) = softcap * tanh(s / softcap) (``softcap <= 0``:
    none); key j is visible when ``0 <= i - j < window`` (``window <= 0``: all earlier keys); ``sinks`` fp32 [H]: exp(sink_h) joins the
    soft-max denominator only.  Returns fp32 [T, H, Dv]."""
    T, H, D = q.shape
    if pad > 0:
        D = dim
        q = q[:, :, :D]
    hk, hv = (pad, pad) if pad > 0 else (D, Dv)
    rep = H // G
    out = torch.empty(T, H, Dv, dtype=torch.float32, device=q.device)
    qs = 0
    for b in range(req_slots.shape[0]):
        L = int(seq_lens[b])
        ql = 1 if q_lens is None else int(q_lens[b])
        if ql <= 0:
            continue
        lo = 0 if window <= 0 else max(0, L - ql - window + 1)
        pos = torch.arange(lo, L, device=q.device)
        if keep_first > 0 and lo > 0:
            pos = torch.cat([torch.arange(0, min(keep_first, lo), device=q.device), pos])
        slots = page_table[int(req_slots[b]), (pos // page_size).long()].long() * page_size + pos % page_size
        K = k_cache[slots, 0, :G * hk].float().view(-1, G, hk)[:, :, :D].repeat_interleave(rep, 1)
        V = v_cache[slots, 0, :G * hv].float().view(-1, G, hv)[:, :, :Dv].repeat_interleave(rep, 1)
        s = torch.einsum("qhd,khd->hqk", q[qs:qs + ql].float(), K) * scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        qpos = torch.arange(L - ql, L, device=q.device)[:, None]
        dist = (qpos - pos[None, :]).float()
        if slopes is not None and log_rates is not None:
            s = s - slopes.float()[:, None, None] * torch.log(1.0 + log_rates.float()[:, None, None] * dist.clamp(min=0.0)[None])
        elif slopes is not None:
            s = s - slopes.float()[:, None, None] * dist[None]
        hide = dist < 0
        if window > 0:
            far = dist >= window
            hide = hide | (far & (pos[None, :] >= keep_first) if keep_first > 0 else far)
        s = s.masked_fill(hide[None], float("-inf"))
        if sinks is not None:
            s = torch.cat([s, sinks.float()[:, None, None].expand(H, ql, 1)], -1)
        p = torch.softmax(s, dim=-1)[..., : pos.numel()]
        out[qs:qs + ql] = torch.einsum("hqk,khd->qhd", p, V)
        qs += ql
    if gate is not None:
        g = torch.sigmoid(gate.float())
        out = out * (g[:, :, None] if g.shape[1] == H else g.view(T, H, Dv))
    return out * out_scale if out_scale != 1.0 else out


def softmax_bias_route(logits: torch.Tensor, correction: Optional[torch.Tensor], top_k: int, n_real: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """soft-max router with a choice-only correction: s = softmax(logits) over all columns; the ``top_k`` largest ``s + correction`` are chosen,
    weighted by their plain ``s`` (not renormalised).  Columns >= ``n_real`` are identity experts: their weights are summed into the third result.
    -> (weights fp32 [T, top_k] with identity picks zeroed, ids int32 [T, top_k], identity weight fp32 [T])"""
    s = torch.softmax(logits.float(), -1)
    choice = s + correction.float() if correction is not None else s
    ids = choice.topk(top_k, dim=-1).indices
    w = s.gather(1, ids)
    ident = ids >= n_real
    return w.masked_fill(ident, 0.0).contiguous(), ids.to(torch.int32).contiguous(), (w * ident).sum(-1)


# ------------------------------------------------------------------ Resatar mechanisms: attention preparation (projection-wide norm, partial rotation, value mixing), selective scan
def attention_prepare(qkv: torch.Tensor, H: int, G: int, D: int, Dv: int, positions: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      out_cache_loc: torch.Tensor, q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
                      inv_freq: Optional[torch.Tensor] = None, v_first: Optional[torch.Tensor] = None, v_lambda: float = 0.0, pad: int = 0,
                      v_inv_freq: Optional[torch.Tensor] = None, v_interleaved: bool = False) -> torch.Tensor:
    """rows of ``qkv`` [T, >= H*D + G*D + G*Dv] = [q | k | v | ...] -> q [T, H, D] in the cache dtype; k rows to ``k_cache[loc]`` (first
    ``G*D`` columns), v rows to ``v_cache[loc]`` (first ``G*Dv`` columns).  In this order:

    * ``q_norm_w`` [H*D] / ``k_norm_w`` [G*D]: q and k are RMS-normed over their WHOLE projection (all heads at once), times the weight;
    * ``inv_freq`` fp32 [R/2]: the first R coordinates of every q and k head are rotated by the angle ``position * inv_freq[i]``, coordinate
      ``i`` paired with ``i + R/2``;
    * ``v_first`` [T, G*Dv]: v <- (1 - v_lambda) v + v_lambda v_first before it is cached;
    * ``v_inv_freq`` fp32 [Dv/2]: every value head is rotated over its whole width by ``position * v_inv_freq[m]`` before it is cached, pair m
      = coordinates ``(m, m + Dv/2)``, or ``(2m, 2m + 1)`` with ``v_interleaved`` (``rotate_heads`` turns an attention output back).

    ``pad > 0``: every head of q, k and v occupies ``pad`` columns, zeros behind its values (q is [T, H, pad])."""
    T = qkv.shape[0]
    q = qkv[:, :H * D].float()
    k = qkv[:, H * D:H * D + G * D].float()
    v = qkv[:, H * D + G * D:H * D + G * D + G * Dv].float()
    if q_norm_w is not None:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_norm_w.float()
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_norm_w.float()
    q, k = q.reshape(T, H, D), k.reshape(T, G, D)
    if inv_freq is not None:
        half = inv_freq.numel()
        ang = positions.float()[:, None] * inv_freq.float()[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

        def rot(x):
            a, b = x[..., :half], x[..., half:2 * half]
            return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half:]], -1)

        q, k = rot(q), rot(k)
    if v_first is not None:
        v = (1.0 - v_lambda) * v + v_lambda * v_first.float()
    if v_inv_freq is not None:
        v = rotate_pairs(v.reshape(T, G, Dv), positions, v_inv_freq, v_interleaved).reshape(T, G * Dv)
    loc = out_cache_loc.long()
    if pad > 0:
        zp = lambda t, n: torch.nn.functional.pad(t, (0, pad - n))
        k_cache[loc, 0, :G * pad] = zp(k, D).reshape(T, G * pad).to(k_cache.dtype)
        v_cache[loc, 0, :G * pad] = zp(v.reshape(T, G, Dv), Dv).reshape(T, G * pad).to(v_cache.dtype)
        return zp(q, D).to(k_cache.dtype)
    k_cache[loc, 0, :G * D] = k.reshape(T, G * D).to(k_cache.dtype)
    v_cache[loc, 0, :G * Dv] = v.to(v_cache.dtype)
    return q.to(k_cache.dtype)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, interleaved: bool, inverse: bool = False,
                 mult: float = 1.0) -> torch.Tensor:
    """x fp32 [T, heads, n]: the first ``2 * len(inv_freq)`` coordinates of every head turned by ``position * inv_freq[m]`` (``inverse``: by the
    negative angle), pair m = coordinates ``(m, m + half)`` or, ``interleaved``, ``(2m, 2m + 1)``; sine and cosine both times ``mult``; the
    angle is the fp32 product"""
    half = inv_freq.numel()
    ang = positions.float()[:, None] * inv_freq.float()[None, :]
    c, s = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    if inverse:
        s = -s
    if interleaved:
        a, b = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        r = torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2)
        return torch.cat([r, x[..., 2 * half:]], -1)
    a, b = x[..., :half], x[..., half:2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half:]], -1)


def rotate_heads(o: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, Dv: int, interleaved: bool, inverse: bool,
                 lse: Optional[torch.Tensor], sinks: Optional[torch.Tensor]) -> torch.Tensor:
    """o [T, H, >= Dv] -> [T, H * Dv] in o's dtype: ``o[:, :, :Dv]``, times ``sigmoid(lse - sink_h)`` when the attention returned its
    log-sum-exp (a sink joins the denominator), every head then turned over its whole width by ``-+ position * inv_freq[m]``"""
    T, H = o.shape[0], o.shape[1]
    x = o[:, :, :Dv].float()
    if lse is not None:
        x = x * torch.sigmoid(lse.float() - sinks.float()[None, :]).unsqueeze(-1)
    return rotate_pairs(x, positions, inv_freq, interleaved, inverse).reshape(T, H * Dv).to(o.dtype)


def causal_softmax(scores: torch.Tensor, tq: int, first: int, scale: float, out_dtype: torch.dtype) -> torch.Tensor:
    """scores fp32 [R, n], row r = h * tq + i: the soft-max of ``scale * scores[r]`` over the keys ``j <= first + i`` (zero beyond them), in ``out_dtype``"""
    R, n = scores.shape
    i = torch.arange(R, device=scores.device) % tq
    hide = torch.arange(n, device=scores.device)[None, :] > (first + i)[:, None]
    return torch.softmax((scores.float() * scale).masked_fill(hide, float("-inf")), -1).to(out_dtype)


def parallel_add_rmsnorm_f32(residual: torch.Tensor, deltas, w1: torch.Tensor, w2: Optional[torch.Tensor], eps: float, zero_centred: bool,
                             out_dtype: torch.dtype):
    """residual (fp32, in place) += sum of ``deltas`` (fp32 sum of the deltas first); returns the RMS norm of the new residual under ``w1``
    and, when given, under ``w2`` (weights applied as ``1 + w`` when ``zero_centred``), both in ``out_dtype``"""
    if deltas:
        d = deltas[0].float()
        for t in deltas[1:]:
            d = d + t.float()
        residual.add_(d)
    y = residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + eps)
    g = (lambda w: 1.0 + w.float()) if zero_centred else (lambda w: w.float())
    return (y * g(w1)).to(out_dtype), ((y * g(w2)).to(out_dtype) if w2 is not None else None)


def glu_activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    """x [T, 2F] = [gate | up] -> act(gate) * up, fp32 math, x's dtype; ``kind``: ``silu`` or ``gelu_tanh``"""
    F_ = x.shape[-1] // 2
    g, u = x[..., :F_].float(), x[..., F_:].float()
    a = F.silu(g) if kind == "silu" else F.gelu(g, approximate="tanh")
    return (a * u).to(x.dtype)


def latent_prepare(x: torch.Tensor, q_rank: int, q_norm_w: Optional[torch.Tensor], rank: int, rot_dim: int, kv_norm_w: torch.Tensor, eps: float,
                   positions: torch.Tensor, inv_freq: Optional[torch.Tensor], mult: float, cache: torch.Tensor,
                   out_cache_loc: torch.Tensor) -> Optional[torch.Tensor]:
    """rows of ``x`` [T, >= q_rank + rank + rot_dim] = [query latent | key/value latent | shared rotary key]: the query latent RMS-normed times
    ``q_norm_w`` is returned in x's dtype (``q_rank = 0``: none); the key/value latent RMS-normed times ``kv_norm_w`` goes to the first ``rank``
    columns of ``cache[loc]`` and the rotary key, turned by ``position * inv_freq[m]`` on neighbouring pairs ``(2m, 2m + 1)`` with sine and
    cosine times ``mult``, to the next ``rot_dim`` columns (cache [slots, 1, width])"""
    T = x.shape[0]
    xf = x.float()
    nrm = lambda t: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)
    c = nrm(xf[:, q_rank:q_rank + rank]) * kv_norm_w.float()
    loc = out_cache_loc.long()
    cache[loc, 0, :rank] = c.to(cache.dtype)
    if rot_dim > 0:
        kr = xf[:, q_rank + rank:q_rank + rank + rot_dim].reshape(T, 1, rot_dim)
        if inv_freq is not None:
            kr = rotate_pairs(kr, positions, inv_freq, True, False, mult)
        cache[loc, 0, rank:rank + rot_dim] = kr.reshape(T, rot_dim).to(cache.dtype)
    if q_rank > 0:
        return (nrm(xf[:, :q_rank]) * q_norm_w.float()).to(x.dtype)
    return None


def latent_query(q: torch.Tensor, q_abs: torch.Tensor, dim: int, rot_dim: int, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                 mult: float) -> torch.Tensor:
    """the query of absorbed latent attention with a rotary part: q [T, H, dim + rot_dim] (per head: unrotated | rotary), ``q_abs`` fp32
    [H, T, rank] (the unrotated part already multiplied into the key up-projection) -> fp32 [T, H, rank + rot_dim] = [q_abs | rotary part
    turned by position (neighbouring pairs, sine and cosine times ``mult``)]"""
    qr = q[:, :, dim:dim + rot_dim].float()
    if inv_freq is not None:
        qr = rotate_pairs(qr, positions, inv_freq, True, False, mult)
    return torch.cat([q_abs.float().transpose(0, 1), qr], -1).contiguous()


def mlstm_prepare(proj: torch.Tensor, gates_raw: torch.Tensor, H: int, D: int, Dv: int, cap: float, mstate: torch.Tensor, req_slots: torch.Tensor,
                  seq_lens: torch.Tensor, q_lens: Optional[torch.Tensor]):
    """inputs of the matrix-memory recurrence with exponential gates and a running maximum (mLSTM), ragged over requests.

    ``proj`` [T, >= 2*H*D + H*Dv] = [q | k | v | ...]; ``gates_raw`` fp32 [T, 2H] = [input | forget] pre-activations.  Per head:
    ``i = cap tanh(raw_i / cap)``, ``f = logsigmoid(cap tanh(raw_f / cap))`` (``cap <= 0``: no cap), ``m_t = max(f + m_(t-1), i)`` with m = 0
    at the start of a sequence (``mstate`` fp32 [slots, H] carries it from call to call, in place).  Returns

    * u fp32 [T, H*(Dv+1) + 2*H*D] = [v with a column of ones behind every head | k | q / sqrt(D)]: the scan's [x | B | C] (the ones
      column accumulates the normaliser n alongside the memory);
    * gates fp32 [T, H, 3] = (exp(f + m_(t-1) - m_t), exp(i - m_t), exp(-m_t)): decay, input scale and the floor of the denominator."""
    T = proj.shape[0]
    q = proj[:, :H * D].float() * (D ** -0.5)
    k = proj[:, H * D:2 * H * D].float()
    v = proj[:, 2 * H * D:2 * H * D + H * Dv].float().view(T, H, Dv)
    x = torch.cat([v, torch.ones(T, H, 1, dtype=torch.float32, device=proj.device)], -1).reshape(T, H * (Dv + 1))
    u = torch.cat([x, k, q], -1).contiguous()
    raw = gates_raw.float()
    capf = (lambda t: cap * torch.tanh(t / cap)) if cap > 0 else (lambda t: t)
    ig = capf(raw[:, :H])
    fg = F.logsigmoid(capf(raw[:, H:2 * H]))
    gates = torch.empty(T, H, 3, dtype=torch.float32, device=proj.device)
    off = 0
    for b in range(req_slots.shape[0]):
        n = 1 if q_lens is None else int(q_lens[b])
        if n <= 0:
            continue
        slot = int(req_slots[b])
        m = torch.zeros(H, dtype=torch.float32, device=proj.device) if int(seq_lens[b]) - n == 0 else mstate[slot].clone()
        for t in range(off, off + n):
            m_new = torch.maximum(fg[t] + m, ig[t])
            gates[t, :, 0] = torch.exp(fg[t] + m - m_new)
            gates[t, :, 1] = torch.exp(ig[t] - m_new)
            gates[t, :, 2] = torch.exp(-m_new)
            m = m_new
        mstate[slot] = m
        off += n
    return u, gates


def mlstm_readout(y: torch.Tensor, gates: torch.Tensor, H: int, Dv: int, norm_w: torch.Tensor, eps: float, gate: Optional[torch.Tensor],
                  out_dtype: torch.dtype) -> torch.Tensor:
    """y fp32 [T, H*(Dv+1)]: per head the memory's read-out and, in the last column, the normaliser's (n . q).  Per head
    ``o = y[:Dv] / (max(|n . q|, gates[..., 2]) + 1e-6)``, divided by its root mean square, times ``norm_w`` [H*Dv], times ``sigmoid(gate)``
    ([T, H*Dv]) -> [T, H*Dv] in ``out_dtype``"""
    T = y.shape[0]
    yy = y.float().view(T, H, Dv + 1)
    den = torch.maximum(yy[..., Dv].abs(), gates[..., 2].float()) + 1e-6
    o = yy[..., :Dv] / den[..., None]
    o = (o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)).reshape(T, H * Dv) * norm_w.float()
    if gate is not None:
        o = o * torch.sigmoid(gate.float())
    return o.to(out_dtype)


def mamba1_scan(u: torch.Tensor, dt_raw: torch.Tensor, dt_bias: Optional[torch.Tensor], A_log: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
                D: Optional[torch.Tensor], z: Optional[torch.Tensor], state: torch.Tensor, req_slots: torch.Tensor, seq_lens: torch.Tensor,
                q_lens: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """selective scan (Mamba-1) over a ragged batch, token by token, state in place.

    u fp32 [T, C] short-conv outputs; dt = softplus(dt_raw + dt_bias) [T, C] (no clamp); Bm / Cm [T, N]; state fp32 [slots, 1, C, N]; a request
    whose ``seq_len == q_len`` starts from zero.  Per token, channel c and state n:  S[c, n] <- exp(-dt_c exp(A_log[c, n])) S[c, n] + dt_c u_c B_n;
    y_c = sum_n S[c, n] C_n + D_c u_c;  with ``z``: y <- y * silu(z).  Returns [T, C] in ``out_dtype``."""
    T, C = u.shape
    x = u.float()
    dt = dt_raw.float() + (dt_bias.float() if dt_bias is not None else 0.0)
    dt = F.softplus(dt, threshold=1e9)
    A = -torch.exp(A_log.float())
    Bf, Cf = Bm.float(), Cm.float()
    out = torch.empty(T, C, dtype=torch.float32, device=u.device)
    off = 0
    for b in range(req_slots.shape[0]):
        n = 1 if q_lens is None else int(q_lens[b])
        if n <= 0:
            continue
        slot = int(req_slots[b])
        S = torch.zeros_like(state[slot, 0]) if int(seq_lens[b]) - n == 0 else state[slot, 0].clone()
        for t in range(off, off + n):
            S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * Bf[t][None, :]
            out[t] = S @ Cf[t]
        state[slot, 0] = S
        off += n
    if D is not None:
        out = out + D.float()[None, :] * x
    if z is not None:
        out = out * F.silu(z.float())
    return out.to(out_dtype)
