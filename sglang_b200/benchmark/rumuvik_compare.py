"""Rumuvik beside the closest existing family at equal size (``python bench.py --hybrid-compare --hybrid-family rumuvik``).

Two parts, random weights, one GPU:

1. **engine**: prefill and decode throughput of a four-layer Rumuvik slice (gated matrix memory, two rotary attention layers with rotated
   values, rotary latent attention; every layer with the gated GELU feed-forward) and of a Resatar slice of the same width, head counts and
   head sizes (parallel mixer = window attention beside decaying linear attention, then three rotary gated attention layers; dense GELU
   feed-forward of 1.5 times the width, so that a token multiplies as many feed-forward weights), both through ``Scheduler.replay_step``
   (the serving step).
2. **kernels**: each new or extended kernel beside the like op of the closest model on the same shapes: the scan with per-token gates
   (values one column wider: the normaliser) vs the constant-decay scan it shares a kernel with; ``mlstm_prepare`` vs the activation pass that
   feeds that scan; ``mlstm_readout`` vs the gated norm; causal attention on the tcgen05 kernels with a score cap + the sink / back-rotation
   pass vs the same kernels + the gate pass; the general kernel (fp32 serving, group sizes that do not divide 128) with cap and sink + the
   back-rotation pass vs the tcgen05 kernels; ``attention_prepare`` with rotated values vs with the value blend; the absorbed latent kernel
   with 64 score-only columns vs the same kernel over the latent alone; ``causal_softmax`` vs ``torch.softmax`` + cast; ``latent_prepare`` vs the bf16 RMS norm; ``latent_query`` vs the
   transposing copy it replaces; the two-norm residual kernel vs two calls of the one-norm kernel; the gated activation vs ``silu_and_mul``.
   Roofline: algorithmic bytes over the measured copy bandwidth; for prompt attention also FLOPs over the measured bf16 GEMM rate.

Timing: CUDA events on the launching stream, >= 3 warm-ups, an L2 flush (a 256 MB write) between timed iterations.
Prints one JSON line per measurement and a closing summary line.
"""
from __future__ import annotations

import json
from typing import List

import torch

from .hybrid_compare import _engine_numbers, _peaks, _Timer


def _rumuvik_cfg(width: int, heads: int, ff: int) -> dict:
    kv = max(1, heads // 8)
    attn = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "rot": {"base": 10000.0, "dims": 64}, "scale": 128 ** -0.5,
                                           "softcap": 30.0}}
    lat = {"type": "latent_attention", "mixer": {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "q_rank": 3 * width // 4,
                                                 "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
                                                 "scale": 192 ** -0.5}}
    mem = {"type": "mlstm", "mixer": {"heads": heads // 2, "dim": 128, "vdim": 128, "gate_cap": 15.0}}
    mlp = {"kind": "dense", "ff": ff}
    return {"architecture": "Rumuvik", "width": width, "vocab": 32000, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": [dict(mem, mlp=mlp), dict(attn, mlp=mlp), dict(attn, mlp=mlp), dict(lat, mlp=mlp)]}


def _resatar_cfg(width: int, heads: int, ff: int) -> dict:
    kv = max(1, heads // 8)
    rot = {"dims": 64, "base": 10000.0}
    attn = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "rot": rot, "scale": 128 ** -0.5, "v_mix": True}}
    par = {"type": "parallel", "mixer": {"left": {"heads": heads // 2, "kv_heads": max(1, heads // 16), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                                  "mask": {"size": 1024, "keep_first": 4}},
                                         "right": {"heads": heads // 2, "dim": 128, "vdim": 128, "decay": [0.99] * (heads // 2)},
                                         "left_scale": 1.0, "right_scale": 1.0}}
    mlp = {"kind": "dense", "ff": 3 * ff // 2}
    return {"architecture": "Resatar", "width": width, "vocab": 32000, "norm": {"eps": 1e-6},
            "layers": [dict(par, mlp=mlp), dict(attn, mlp=mlp), dict(attn, mlp=mlp), dict(attn, mlp=mlp)]}


def _kernel_numbers(timer: _Timer, hbm_gbs: float, tflops: float) -> List[dict]:
    from .. import ops
    from ..layers.gated_attention import scaled_inv_freq
    from ..layers.latent_attention import yarn_inv_freq

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
    # ---- the gated matrix memory: preparation, scan, read-out, beside the decaying linear attention of the closest model
    H, D, Dv = 16, 128, 128
    decay = torch.full((H,), 0.99, device=dev)
    nw = torch.ones(H * Dv, device=dev, dtype=bf)
    for B, S in ((4, 2048), (32, 1)):
        T = B * S
        ph = "prefill" if S > 1 else "decode"
        proj = (torch.randn(T, 2 * H * D + 2 * H * Dv, device=dev, generator=g) * 0.3).to(bf)
        raw = torch.randn(T, 2 * H, device=dev, generator=g) * 3
        raw[:, H:] += 3.0
        state = torch.zeros(B + 1, H, D, Dv + 1, device=dev)
        state2 = torch.zeros(B + 1, H, D, Dv, device=dev)
        mst = torch.zeros(B + 1, H, device=dev)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), S if S > 1 else 999, dtype=torch.int32, device=dev)
        cu = torch.arange(0, T + 1, S, dtype=torch.int32, device=dev) if S > 1 else None
        ql = sl if S > 1 else None
        n = 2 * H * D + H * Dv
        ms = timer(lambda: ops.mlstm_prepare(proj, raw, H, D, Dv, 15.0, mst, slots, sl, cu, ql))
        like = timer(lambda: ops.activation(proj[:, :n], "silu", torch.float32))
        rec("mlstm_prepare (scan input rows in fp32, capped gates, running maximum)", ph, f"B{B} S{S} H{H} D{D} Dv{Dv}", ms, T * n * 2 + T * (n + H) * 4 + T * H * 20,
            "activation(silu) -> fp32 (the linear-attention scan's input)", like, like_bytes=T * n * 6)
        u, gt = ops.mlstm_prepare(proj, raw, H, D, Dv, 15.0, mst, slots, sl, cu, ql)
        u2 = ops.activation(proj[:, :n], "silu", torch.float32)
        ms = timer(lambda: ops.mamba2_scan(u, None, None, None, None, None, state, slots, sl, cu, ql, H, Dv + 1, D, H, gates=gt))
        like = timer(lambda: ops.mamba2_scan(u2, None, None, None, None, None, state2, slots, sl, cu, ql, H, Dv, D, H, decay))
        nbytes = u.numel() * 4 + T * H * (Dv + 1) * 4 + 2 * state[:B].numel() * 4
        rec("mamba2_scan(gates): matrix memory and its normaliser", ph, f"B{B} S{S} H{H} D{D} Dv{Dv}+1", ms, nbytes,
            "mamba2_scan(decay) (constant decay, same kernel)", like, like_bytes=u2.numel() * 4 + T * H * Dv * 4 + 2 * state2[:B].numel() * 4)
        y = ops.mamba2_scan(u, None, None, None, None, None, state, slots, sl, cu, ql, H, Dv + 1, D, H, gates=gt)
        y2 = ops.mamba2_scan(u2, None, None, None, None, None, state2, slots, sl, cu, ql, H, Dv, D, H, decay)
        ms = timer(lambda: ops.mlstm_readout(y, gt, H, Dv, nw, 1e-6, proj[:, n:], bf))
        like = timer(lambda: ops.grouped_rmsnorm(y2, nw, 1, 1e-6, bf, proj[:, n:]))
        rec("mlstm_readout (floored normaliser, per-head norm, gate)", ph, f"T{T} H{H} Dv{Dv}", ms, T * H * Dv * 8, "grouped_rmsnorm(gate)", like)
    # ---- attention: score cap, unit sink, values turned back
    H, Gk, Dh, ps = 32, 4, 128, 64
    sinks = torch.zeros(H, device=dev)
    fv = scaled_inv_freq(Dh, 10000.0).to(dev)
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
        pos = (torch.arange(B * Q, dtype=torch.int32, device=dev) % Q) + (S - Q)
        gh = torch.randn(B * Q, H, device=dev, generator=g).to(bf)
        k4, v4 = kc.view(-1, Gk, Dh), vc.view(-1, Gk, Dh)
        ns = 1 if Q > 1 else 4
        ph = "prefill" if Q > 1 else "decode"
        keys = sum(i + 1 for i in range(S - Q, S))
        nb = q.numel() * 2 * 2 + B * S * Gk * Dh * 2 * 2
        lse = torch.empty(B * Q, H, dtype=torch.float32, device=dev)

        def capped():
            o = ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, -1, logit_cap=30.0, num_splits=ns, lse=lse)
            return ops.rotate_heads(o, pos, fv, Dh, False, True, lse, sinks)

        def gated():
            o = ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, -1, num_splits=ns)
            return ops.sigmoid_gate(o, gh, Dh)

        ms = timer(capped)
        like_attn = like = timer(gated)
        rec("causal attention on the tcgen05 kernels with a score cap + rotate_heads (sink share, back-rotation)", ph, f"B{B} S{S} q{Q} H{H} G{Gk} D{Dh} splits{ns}",
            ms, nb + q.numel() * 2 * 2, "paged_attention + sigmoid_gate (the closest model's attention)", like, flops=4.0 * B * keys * H * Dh)
        o0 = ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, -1, num_splits=ns)
        ms = timer(lambda: ops.rotate_heads(o0, pos, fv, Dh, False, True, lse, sinks))
        like = timer(lambda: ops.sigmoid_gate(o0, gh, Dh))
        rec("rotate_heads (sink share, back-rotation)", ph, f"T{B * Q} H{H} Dv{Dh}", ms, q.numel() * 4, "sigmoid_gate", like)

        def general():
            o = ops.window_attention(q, kc, vc, Gk, Dh, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, 30.0, -1, None, sinks, Dh, 0)
            return ops.rotate_heads(o.view(B * Q, H, Dh), pos, fv, Dh, False, True)

        ms = timer(general)
        rec("window_attention (general kernel: fp32 serving, other group sizes) with cap and sink + rotate_heads", ph, f"B{B} S{S} q{Q} H{H} G{Gk} D{Dh}", ms,
            nb + q.numel() * 2 * 2, "paged_attention + sigmoid_gate (tcgen05 kernels)", like_attn, flops=4.0 * B * keys * H * Dh)
    # ---- attention_prepare with rotated values
    T = 8192
    qkv = torch.randn(T, (H + 2 * Gk) * Dh, device=dev, generator=g).to(bf)
    kc = torch.zeros(T + 64, 1, Gk * Dh, device=dev, dtype=bf)
    vc = torch.zeros_like(kc)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    loc = pos + 64
    fr = scaled_inv_freq(64, 10000.0, None).to(dev)
    vf = torch.randn(T, Gk * Dh, device=dev, generator=g).to(bf)
    ms = timer(lambda: ops.attention_prepare(qkv, H, Gk, Dh, Dh, pos, kc, vc, loc, None, None, 0.0, fr, None, 0.0, 0, fv, False))
    like = timer(lambda: ops.attention_prepare(qkv, H, Gk, Dh, Dh, pos, kc, vc, loc, None, None, 0.0, fr, vf, 0.3))
    rec("attention_prepare (partial rotation of q / k, values rotated over their whole width)", "any", f"T{T} H{H} G{Gk} D{Dh} rot64", ms, qkv.numel() * 2 * 2,
        "attention_prepare (partial rotation, value blend)", like, like_bytes=qkv.numel() * 2 * 2 + vf.numel() * 2)
    # ---- latent attention with a rotary part
    Hl, R, Dr, Dn = 16, 512, 64, 128
    f, mult = yarn_inv_freq(Dr, 10000.0, {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0})
    f = f.to(dev)
    for B, S, Q in ((2, 2048, 2048), (32, 2048, 1)):
        pages = B * S // ps
        cache = (torch.randn((pages + 1) * ps, 1, R + Dr, device=dev, generator=g) * 0.3).to(bf)
        pt = (torch.arange(pages, dtype=torch.int32, device=dev) + 1).view(B, S // ps).contiguous()
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), S, dtype=torch.int32, device=dev)
        ql = torch.full((B,), Q, dtype=torch.int32, device=dev)
        cu = None if Q == 1 else torch.arange(0, B * Q + 1, Q, dtype=torch.int32, device=dev)
        qa = torch.randn(B * Q, Hl, R + Dr, device=dev, generator=g) * 0.1
        qb = qa[:, :, :R].contiguous()
        ph = "prefill" if Q > 1 else "decode"
        ms = timer(lambda: ops.latent_attention(qa, cache, R + Dr, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, 0.07, -1, None, S, v_rank=R), iters=3)
        like = timer(lambda: ops.latent_attention(qb, cache, R, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, 0.07, -1, None, S), iters=3)
        nb = B * S * (R + Dr) * 2 + qa.numel() * 4 + B * Q * Hl * R * 4
        rec("latent_attention (absorbed, 64 score-only rotary columns)", ph, f"B{B} S{S} q{Q} H{Hl} R{R}+{Dr}", ms, nb,
            "latent_attention (the latent alone, same kernel)", like, like_bytes=B * S * R * 2 + qb.numel() * 8)
    # the soft-max between the two matrix products of long latent prompt portions
    tq = 2048
    sc = torch.randn(Hl * tq, tq, device=dev, generator=g)
    ms = timer(lambda: ops.causal_softmax(sc, tq, 0, 0.07, bf))
    like = timer(lambda: torch.softmax(sc, -1).to(bf))
    rec("causal_softmax (fp32 scores in, bf16 weights out, causal limit)", "prefill", f"H{Hl} q{tq} keys{tq}", ms, sc.numel() * 4,
        "torch.softmax + cast (no mask; the same task's bytes)", like)
    T, Rq = 8192, 1536
    x = torch.randn(T, Rq + R + Dr, device=dev, generator=g).to(bf)
    wq, wk = torch.ones(Rq, device=dev, dtype=bf), torch.ones(R, device=dev, dtype=bf)
    cache = torch.zeros(T + 64, 1, R + Dr, device=dev, dtype=bf)
    ms = timer(lambda: ops.latent_prepare(x, Rq, wq, R, Dr, wk, 1e-6, pos, f, mult, cache, loc))
    xc, wqc = x[:, :Rq + R].contiguous(), torch.ones(Rq + R, device=dev, dtype=bf)
    like = timer(lambda: ops.rmsnorm(xc, wqc, 1e-6))
    rec("latent_prepare (two norms, rotary key, cache write)", "any", f"T{T} Rq{Rq} R{R} Dr{Dr}", ms, x.numel() * 4, "rmsnorm (bf16, one norm over the same columns)", like,
        like_bytes=xc.numel() * 4)
    q = torch.randn(T, Hl, Dn + Dr, device=dev, generator=g).to(bf)
    q_abs = torch.randn(Hl, T, R, device=dev, generator=g)
    ms = timer(lambda: ops.latent_query(q, q_abs, Dn, Dr, pos, f, mult))
    like = timer(lambda: q_abs.transpose(0, 1).contiguous())
    rec("latent_query (transpose + rotary query columns)", "any", f"T{T} H{Hl} R{R} Dr{Dr}", ms, q_abs.numel() * 8 + T * Hl * Dr * 6, "transposing copy (torch)", like,
        like_bytes=q_abs.numel() * 8)
    # ---- the residual stream with two norms, the gated activation
    Wd = 4096
    res = torch.randn(T, Wd, device=dev)
    d1, d2 = torch.randn(T, Wd, device=dev).to(bf), torch.randn(T, Wd, device=dev).to(bf)
    w1, w2 = torch.zeros(Wd, device=dev, dtype=bf), torch.zeros(Wd, device=dev, dtype=bf)
    ms = timer(lambda: ops.parallel_add_rmsnorm_f32(res, [d1, d2], w1, w2, 1e-6, True, bf))

    def twice():
        ops.add_rmsnorm_f32(res, d1, w1, 1e-6, True, bf)
        ops.add_rmsnorm_f32(res, d2, w2, 1e-6, True, bf)

    like = timer(twice)
    rec("parallel_add_rmsnorm_f32 (two deltas in, two norms out)", "any", f"T{T} W{Wd}", ms, T * Wd * 16, "add_rmsnorm_f32 twice (one delta, one norm each)", like,
        like_bytes=T * Wd * 20)
    x2 = torch.randn(T, 2 * Wd, device=dev).to(bf)
    ms = timer(lambda: ops.glu_activation(x2, "gelu_tanh"))
    like = timer(lambda: ops.silu_and_mul(x2))
    rec("activation(gelu_tanh, mul): gated feed-forward middle", "any", f"T{T} n{2 * Wd}", ms, T * Wd * 6, "silu_and_mul", like)
    return out


def main(sizes: str = "2048,4096") -> None:
    pk = _peaks()
    timer = _Timer()
    rows: List[dict] = []
    for w in [int(x) for x in sizes.split(",") if x]:
        heads = w // 128
        for name, cfg in (("rumuvik", _rumuvik_cfg(w, heads, 2 * w)), ("resatar", _resatar_cfg(w, heads, 2 * w))):
            for r in _engine_numbers(name, cfg, 4, 2048, 32, 8, timer):
                r["width"] = w
                rows.append(r)
                print(json.dumps(r), flush=True)
    for r in _kernel_numbers(timer, pk["hbm_gbs"], pk["bf16_tflops"]):
        rows.append(r)
        print(json.dumps(r), flush=True)
    worst = max((r.get("distance_ratio", 0.0) for r in rows if r["part"] == "kernel"), default=0.0)
    print(json.dumps({"metric": "hybrid_compare", "family": "rumuvik", "roofline": f"{pk['hbm_gbs']} GB/s, {pk['bf16_tflops']} TFLOP/s ({pk['src']})",
                      "worst_kernel_distance_ratio": worst, "rows": len(rows), "data": "synthetic", "dtype": "bf16"}), flush=True)
