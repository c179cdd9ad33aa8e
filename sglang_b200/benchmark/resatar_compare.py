"""Resatar beside the closest existing family at equal size (``python bench.py --hybrid-compare --hybrid-family resatar``).

Two parts, random weights, one GPU:

1. **engine**: prefill and decode throughput of a four-layer Resatar slice (rotary attention + dense, selective scan + MoE, parallel mixer + MoE,
   selective scan + MoE) and of a Jamba slice of the same width, head counts, head size, inner width, state size, step rank and taps (pattern
   ``*M*M``; its feed-forward width is chosen so that a token runs as many feed-forward columns as a Resatar token: ``top * expert ff + shared
   ff``), both through ``Scheduler.replay_step`` (the serving step).
2. **kernels**: each new kernel beside the like op of the closest model on the same shapes: the ragged selective scan vs the chunked PyTorch
   scan Jamba prompts run and vs the tensor expressions of its decode step; window attention with kept tokens, logarithmic bias and an
   element gate, on the tcgen05 kernels (bf16 serving) and on the general kernel (fp32 serving), vs the tcgen05 paged attention kernel with the
   same window alone; rotary gated attention on the tcgen05 kernels (+ gate) vs the same kernels alone; ``attention_prepare`` vs ``rope_kv_write``; the constant-decay scan vs the Mamba-2 scan it shares a kernel with; the
   scalar sandwich norm vs the vector one; the gated norm vs the plain one; the element-wise activation vs ``silu_and_mul``.
   Roofline: algorithmic bytes over the measured copy bandwidth; for prompt attention also FLOPs over the measured bf16 GEMM rate.

Timing: CUDA events on the launching stream, >= 3 warm-ups, an L2 flush (a 256 MB write) between timed iterations.
Prints one JSON line per measurement and a closing summary line.
"""
from __future__ import annotations

import json
from typing import List

import torch

from .hybrid_compare import _engine_numbers, _peaks, _Timer


def _resatar_cfg(width: int, heads: int, experts: int, top: int, eff: int, shared: int, window: int, state: int, ff: int) -> dict:
    rot = {"dims": 64, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    attn = {"type": "attention", "mixer": {"heads": heads, "kv_heads": max(1, heads // 8), "dim": 128, "vdim": 128, "rot": rot, "scale": 128 ** -0.5, "v_mix": True}}
    par = {"type": "parallel", "mixer": {"left": {"heads": heads // 2, "kv_heads": max(1, heads // 16), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                                  "mask": {"size": window, "keep_first": 4}},
                                         "right": {"heads": heads // 2, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-5 - 3 * i / max(1, heads // 2 - 1))
                                                                                                          for i in range(heads // 2)]},
                                         "left_scale": 1.0, "right_scale": 1.0}}
    m1 = {"type": "mamba1", "mixer": {"inner": 2 * width, "state": state, "dt_rank": width // 16, "conv": 4}}
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": experts, "top": top}, "shared": {"ff": shared}}
    return {"architecture": "Resatar", "width": width, "vocab": 32000, "norm": {"eps": 1e-6},
            "layers": [dict(attn, mlp={"kind": "dense", "ff": ff}), dict(m1, mlp=moe), dict(par, mlp=moe), dict(m1, mlp=moe)]}


def _jamba_cfg(width: int, heads: int, ff: int, experts: int, state: int) -> dict:
    return {"architectures": ["JambaForCausalLM"], "hidden_size": width, "num_hidden_layers": 4, "layers_block_type": ["attention", "mamba", "attention", "mamba"],
            "layers_num_experts": [1, experts, experts, experts], "num_experts_per_tok": 2, "mamba_expand": 2, "mamba_d_state": state, "mamba_d_conv": 4,
            "mamba_dt_rank": width // 16, "num_attention_heads": heads, "num_key_value_heads": max(1, heads // 8), "intermediate_size": ff,
            "vocab_size": 32000, "rms_norm_eps": 1e-6, "max_position_embeddings": 32768, "tie_word_embeddings": False}


def _kernel_numbers(timer: _Timer, hbm_gbs: float, tflops: float) -> List[dict]:
    import torch.nn.functional as F

    from .. import ops
    from ..layers.gated_attention import scaled_inv_freq
    from ..models.mamba import selective_scan_chunked

    dev, out = "cuda", []

    def rec(kernel, phase, shape, ms, nbytes, like=None, like_ms=None, like_bytes=None, flops=None):
        r = {"part": "kernel", "kernel": kernel, "phase": phase, "shape": shape, "ms": round(ms, 4), "algorithmic_mb": round(nbytes / 1e6, 2),
             "roofline_frac": round(nbytes / (ms * 1e-3) / (hbm_gbs * 1e9), 4)}
        if flops is not None:
            r["tensor_frac"] = round(flops / (ms * 1e-3) / (tflops * 1e12), 4)
        if like is not None:
            lb = nbytes if like_bytes is None else like_bytes
            r.update(like=like, like_ms=round(like_ms, 4), like_roofline_frac=round(lb / (like_ms * 1e-3) / (hbm_gbs * 1e9), 4))
            r["distance_ratio"] = round(r["like_roofline_frac"] / max(r["roofline_frac"], 1e-9), 3)
        out.append(r)

    g = torch.Generator(device=dev).manual_seed(0)
    bf = torch.bfloat16
    # ---- selective scan
    C, N, R = 4096, 16, 128
    dtb, A_log, D = torch.zeros(C, device=dev), torch.zeros(C, N, device=dev), torch.ones(C, device=dev)
    for B, S in ((4, 2048), (1, 4096)):
        T = B * S
        u, dt_raw = torch.randn(T, C, device=dev, generator=g), torch.randn(T, C, device=dev, generator=g)
        low = torch.randn(T, R + 2 * N, device=dev, generator=g).to(bf)
        xz = torch.randn(T, 2 * C, device=dev, generator=g).to(bf)
        state = torch.zeros(B + 1, 1, C, N, device=dev)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), S, dtype=torch.int32, device=dev)
        cu = torch.arange(0, T + 1, S, dtype=torch.int32, device=dev)
        ms = timer(lambda: ops.mamba1_scan(u, dt_raw, dtb, A_log, low[:, R:R + N], low[:, R + N:], D, xz[:, C:], state, slots, sl, cu, sl, bf))
        negA = -A_log.exp()

        def chunked():
            dt = F.softplus(dt_raw + dtb)
            for i in range(B):
                s = slice(i * S, (i + 1) * S)
                y, fin = selective_scan_chunked(u[s], dt[s], negA, low[s, R:R + N], low[s, R + N:], state[i, 0], 16)
                y = ((y + D[None] * u[s]) * F.silu(xz[s, C:].float())).to(bf)

        like = timer(chunked, iters=3, warmup=2)
        nbytes = T * C * (4 + 4 + 2 + 2) + low.numel() * 2 + 2 * state[:B].numel() * 4
        rec("mamba1_scan", "prefill", f"B{B} S{S} C{C} N{N}", ms, nbytes, "mamba.selective_scan_chunked + gate (torch)", like)
    for B in (32, 256):
        u, dt_raw = torch.randn(B, C, device=dev, generator=g), torch.randn(B, C, device=dev, generator=g)
        low = torch.randn(B, R + 2 * N, device=dev, generator=g).to(bf)
        xz = torch.randn(B, 2 * C, device=dev, generator=g).to(bf)
        state = torch.randn(B + 1, 1, C, N, device=dev, generator=g)
        st2 = state.clone()
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), 999, dtype=torch.int32, device=dev)
        ms = timer(lambda: ops.mamba1_scan(u, dt_raw, dtb, A_log, low[:, R:R + N], low[:, R + N:], D, xz[:, C:], state, slots, sl, None, None, bf))
        negA = -A_log.exp()
        sidx = slots.long()

        def upd():          # the decode step of models/mamba.py Mamba1Mixer
            dt = F.softplus(dt_raw + dtb)
            st = st2[sidx][:, 0]
            st = torch.exp(dt[:, :, None] * negA[None]) * st + (dt * u)[:, :, None] * low[:, None, R:R + N].float()
            st2[sidx] = st.unsqueeze(1)
            y = torch.einsum("bdn,bn->bd", st, low[:, R + N:].float())
            y = ((y + D[None] * u) * F.silu(xz[:, C:].float())).to(bf)

        like = timer(upd)
        rec("mamba1_scan", "decode", f"B{B} C{C} N{N}", ms, 2 * state[:B].numel() * 4, "Mamba1Mixer decode step (torch expressions)", like)
    # ---- constant-decay linear attention on the Mamba-2 scan kernel
    H, P, Nk = 16, 128, 128
    decay = torch.full((H,), 0.99, device=dev)
    dtb2, A2 = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
    for B, S in ((4, 2048), (32, 1)):
        T = B * S
        u = torch.randn(T, H * P + 2 * H * Nk, device=dev, generator=g) * 0.1
        dtr = torch.randn(T, H, device=dev, generator=g).to(bf)
        state = torch.zeros(B + 1, H, Nk, P, device=dev)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), S if S > 1 else 999, dtype=torch.int32, device=dev)
        cu = torch.arange(0, T + 1, S, dtype=torch.int32, device=dev) if S > 1 else None
        ql = sl if S > 1 else None
        ms = timer(lambda: ops.mamba2_scan(u, None, None, None, None, None, state, slots, sl, cu, ql, H, P, Nk, H, decay))
        like = timer(lambda: ops.mamba2_scan(u, None, dtr, dtb2, A2, None, state, slots, sl, cu, ql, H, P, Nk, H))
        nbytes = u.numel() * 4 + T * H * P * 4 + 2 * state[:B].numel() * 4
        rec("mamba2_scan(decay): linear attention with a constant decay", "prefill" if S > 1 else "decode", f"B{B} S{S} H{H} D{Nk} Dv{P}", ms, nbytes,
            "mamba2_scan (input-dependent step, same kernel)", like)
    # ---- attention
    H, Gk, Dh, ps, W = 32, 4, 128, 64, 1024
    r1, r2 = torch.full((H,), 0.5, device=dev), torch.full((H,), 0.1, device=dev)
    for B, S, Q in ((4, 2048, 2048), (64, 2048, 1)):
        pages = B * S // ps
        kc = torch.randn((pages + 1) * ps, 1, Gk * Dh, device=dev, generator=g).to(bf)
        vc = torch.randn((pages + 1) * ps, 1, Gk * Dh, device=dev, generator=g).to(bf)
        pt = (torch.arange(pages, dtype=torch.int32, device=dev) + 1).view(B, S // ps).contiguous()
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), S, dtype=torch.int32, device=dev)
        ql = torch.full((B,), Q, dtype=torch.int32, device=dev)
        cu = None if Q == 1 else torch.arange(0, B * Q + 1, Q, dtype=torch.int32, device=dev)
        q = torch.randn(B * Q, H, Dh, device=dev, generator=g).to(bf)
        ge, gh = torch.randn(B * Q, H * Dh, device=dev, generator=g).to(bf), torch.randn(B * Q, H, device=dev, generator=g).to(bf)
        ms = timer(lambda: ops.window_attention(q, kc, vc, Gk, Dh, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, 0.0, W, r1, None, Dh, 0, 4, r2, ge))
        k4, v4 = kc.view(-1, Gk, Dh), vc.view(-1, Gk, Dh)
        ns = 1 if Q > 1 else 4
        like = timer(lambda: ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, W, num_splits=ns))
        keys = sum(min(i + 1, W) for i in range(S - Q, S))
        nbytes = q.numel() * 2 * 3 + B * min(S, W + Q) * Gk * Dh * 2 * 2
        ph = "prefill" if Q > 1 else "decode"
        rec("window_attention (general kernel: fp32 serving and head sizes beyond 128) with kept tokens, logarithmic bias, element gate", ph, f"B{B} S{S} q{Q} H{H} G{Gk} D{Dh} window{W} keep4", ms, nbytes,
            "paged_attention (tcgen05 / split-KV decode kernel, same window)", like, like_bytes=nbytes - q.numel() * 2, flops=4.0 * B * keys * H * Dh)
        # the same window layer on the tcgen05 kernels (bf16 serving with heads up to 128 wide): window, kept tokens and logarithmic bias inside, gate pass behind

        def window_tc():
            o = ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, W, num_splits=ns, slopes=r1, log_rates=r2,
                                    keep_first=4)
            return ops.sigmoid_gate(o, ge, Dh)

        ms1 = timer(window_tc)
        rec("window attention on the tcgen05 kernels (kept tokens, logarithmic bias) + sigmoid_gate (element)", ph, f"B{B} S{S} q{Q} H{H} G{Gk} D{Dh} window{W} keep4 splits{ns}",
            ms1, nbytes + q.numel() * 2 * 2, "paged_attention (tcgen05 / split-KV decode kernel, same window)", like, like_bytes=nbytes - q.numel() * 2,
            flops=4.0 * B * keys * H * Dh)
        # rotary causal attention with a per-head gate: the tcgen05 kernels + the gate pass, beside the same kernels alone
        keys = sum(i + 1 for i in range(S - Q, S))
        nb2 = q.numel() * 2 * 2 + B * S * Gk * Dh * 2 * 2

        def gated():
            o = ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, -1, num_splits=ns)
            return ops.sigmoid_gate(o, gh, Dh)

        ms2 = timer(gated)
        like2 = timer(lambda: ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, -1, num_splits=ns))
        rec("causal attention on the tcgen05 kernels + sigmoid_gate", ph, f"B{B} S{S} q{Q} H{H} G{Gk} D{Dh} splits{ns}", ms2, nb2 + q.numel() * 2 * 2,
            "paged_attention (same kernels, no gate)", like2, like_bytes=nb2, flops=4.0 * B * keys * H * Dh)
    # ---- attention_prepare
    T = 8192
    qkv = torch.randn(T, (H + 2 * Gk) * Dh, device=dev, generator=g).to(bf)
    kc = torch.zeros(T + 64, 1, Gk * Dh, device=dev, dtype=bf)
    vc = torch.zeros_like(kc)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    loc = pos + 64
    fr = scaled_inv_freq(64, 10000.0, None).to(dev)
    vf = torch.randn(T, Gk * Dh, device=dev, generator=g).to(bf)
    ms = timer(lambda: ops.attention_prepare(qkv, H, Gk, Dh, Dh, pos, kc, vc, loc, None, None, 0.0, fr, vf, 0.3))
    q3 = qkv[:, :H * Dh].clone().view(T, H, Dh)
    k3, v3 = qkv[:, H * Dh:(H + Gk) * Dh].clone().view(T, Gk, Dh), qkv[:, (H + Gk) * Dh:].clone().view(T, Gk, Dh)
    cs = torch.randn(T, Dh, device=dev)
    like = timer(lambda: ops.rope_kv_write(q3, k3, v3, pos, cs, kc.view(-1, Gk, Dh), vc.view(-1, Gk, Dh), loc))
    rec("attention_prepare (partial rotation, angles computed in fp32, value blend)", "any", f"T{T} H{H} G{Gk} D{Dh} rot64", ms, qkv.numel() * 2 * 2 + vf.numel() * 2,
        "rope_kv_write (table of cos / sin)", like, like_bytes=qkv.numel() * 2 * 2)
    qw, kw = torch.ones(H * Dh, device=dev, dtype=bf), torch.ones(Gk * Dh, device=dev, dtype=bf)
    ms = timer(lambda: ops.attention_prepare(qkv, H, Gk, Dh, Dh, pos, kc, vc, loc, qw, kw, 1e-6))
    like = timer(lambda: ops.qk_norm_cache_write(qkv, H, Gk, Dh, Dh, pos, 1e-6, 0.0, 1, kc, vc, loc))
    rec("attention_prepare (norm over the whole projection, weights)", "any", f"T{T} H{H} G{Gk} D{Dh}", ms, qkv.numel() * 2 * 2, "qk_norm_cache_write (per-head norm)", like)
    # ---- norms on the fp32 residual, gated norm, activation
    Wd = 4096
    res, d16 = torch.randn(T, Wd, device=dev), torch.randn(T, Wd, device=dev).to(bf)
    w1, wv = torch.ones(1, device=dev, dtype=bf), torch.zeros(Wd, device=dev, dtype=bf)
    ms = timer(lambda: ops.add_rmsnorm_f32(res, d16, w1, 1e-6, False, bf, w1))
    like = timer(lambda: ops.add_rmsnorm_f32(res, d16, wv, 1e-6, True, bf, wv))
    rec("add_rmsnorm_f32(post_weight), one gain per norm", "any", f"T{T} W{Wd}", ms, T * Wd * 12, "add_rmsnorm_f32(post_weight), weight vectors", like)
    y32, gate = torch.randn(T, Wd, device=dev), torch.randn(T, Wd, device=dev).to(bf)
    ms = timer(lambda: ops.grouped_rmsnorm(y32, wv, 1, 1e-6, bf, gate))
    like = timer(lambda: ops.grouped_rmsnorm(y32, wv, 1, 1e-6, bf))
    rec("grouped_rmsnorm(gate)", "any", f"T{T} C{Wd} (fp32 in, gate in, 8 B/elem)", ms, T * Wd * 8, "grouped_rmsnorm (6 B/elem)", like, like_bytes=T * Wd * 6)
    x2 = torch.randn(T, 2 * Wd, device=dev).to(bf)
    ms = timer(lambda: ops.activation(x2, "gelu_tanh"))
    like = timer(lambda: ops.silu_and_mul(x2))
    rec("activation(gelu_tanh)", "any", f"T{T} n{2 * Wd} (4 B/elem)", ms, T * 2 * Wd * 4, "silu_and_mul (3 B per input elem)", like, like_bytes=T * Wd * 6)
    ms = timer(lambda: ops.activation(x2, "silu", torch.float32))
    rec("activation(silu) -> fp32 (the scan's input)", "any", f"T{T} n{2 * Wd} (6 B/elem)", ms, T * 2 * Wd * 6, "silu_and_mul (3 B per input elem)", like, like_bytes=T * Wd * 6)
    return out


def main(sizes: str = "2048,4096") -> None:
    pk = _peaks()
    timer = _Timer()
    rows: List[dict] = []
    for w in [int(x) for x in sizes.split(",") if x]:
        heads = w // 128
        experts, top, eff, shared = 16, 4, w // 2, w
        ff = (top * eff + shared) // 2                    # Jamba runs two experts of its one feed-forward width per token
        cfgs = (("resatar", _resatar_cfg(w, heads, experts, top, eff, shared, 1024, 16, 3 * ff // 2)), ("jamba", _jamba_cfg(w, heads, ff, experts, 16)))
        for name, cfg in cfgs:
            for r in _engine_numbers(name, cfg, 4, 2048, 32, 8, timer):
                r["width"] = w
                rows.append(r)
                print(json.dumps(r), flush=True)
    for r in _kernel_numbers(timer, pk["hbm_gbs"], pk["bf16_tflops"]):
        rows.append(r)
        print(json.dumps(r), flush=True)
    worst = max((r.get("distance_ratio", 0.0) for r in rows if r["part"] == "kernel"), default=0.0)
    print(json.dumps({"metric": "hybrid_compare", "family": "resatar", "roofline": f"{pk['hbm_gbs']} GB/s, {pk['bf16_tflops']} TFLOP/s ({pk['src']})",
                      "worst_kernel_distance_ratio": worst, "rows": len(rows), "data": "synthetic", "dtype": "bf16"}), flush=True)
