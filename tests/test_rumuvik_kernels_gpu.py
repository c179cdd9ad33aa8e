"""Rumuvik CUDA kernels against their fp32 PyTorch references (``ops/torch_ref.py``) and the engine on CUDA against the plain oracle."""
import numpy as np
import pytest
import torch

from sglang_b200 import ops
from sglang_b200.layers.gated_attention import scaled_inv_freq
from sglang_b200.layers.latent_attention import yarn_inv_freq
from sglang_b200.ops import torch_ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _need():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    assert ops.load_native(), "the CUDA extension must be built on a GPU box"


def _i32(x, dev=DEV):
    return torch.tensor(x, dtype=torch.int32, device=dev)


def _tol(dtype, f32=(1e-5, 1e-5), bf=(2e-2, 2e-2)):
    r, a = bf if dtype == torch.bfloat16 else f32
    return dict(rtol=r, atol=a)


def _ragged(q_lens, cached):
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    return cu.tolist(), [c + q for c, q in zip(cached, q_lens)]


def _paged(n_req, max_len, ps, width, dtype, g):
    per = (max_len + ps - 1) // ps
    n_pages = n_req * per + 3
    pt = torch.zeros(n_req + 1, per + 1, dtype=torch.int32)
    perm = torch.randperm(n_pages - 1, generator=g) + 1
    for r in range(n_req):
        pt[r + 1, :per] = perm[r * per:(r + 1) * per].int()
    kc = (torch.randn(n_pages * ps, 1, width, generator=g) * 0.5).to(dtype)
    vc = (torch.randn(n_pages * ps, 1, width, generator=g) * 0.5).to(dtype)
    return pt, kc, vc


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [24, 250, 1024, 5000])
def test_parallel_add_and_two_norms(dtype, W):
    _need()
    g = torch.Generator().manual_seed(W)
    x = torch.randn(7, W, generator=g)
    d1, d2 = torch.randn(7, W, generator=g).to(dtype), torch.randn(7, W, generator=g).to(dtype)
    x0 = torch.randn(7, W, generator=g)
    w1, w2 = (torch.randn(W, generator=g) * 0.2).to(dtype), (torch.randn(W, generator=g) * 0.2).to(dtype)
    for deltas, extra, second, zc in (([d1, d2], None, True, True), ([d1], x0, True, True), ([], None, True, False), ([d1, d2], x0, False, True)):
        r1, r2 = x.clone(), x.clone().to(DEV)
        ref = torch_ref.parallel_add_rmsnorm_f32(r1, deltas + ([extra] if extra is not None else []), w1, w2 if second else None, 1e-6, zc, dtype)
        got = ops.parallel_add_rmsnorm_f32(r2, [d.to(DEV) for d in deltas], w1.to(DEV), w2.to(DEV) if second else None, 1e-6, zc, dtype,
                                           extra.to(DEV) if extra is not None else None)
        torch.testing.assert_close(r2.cpu(), r1, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(got[0].cpu().float(), ref[0].float(), **_tol(dtype))
        assert (got[1] is None) == (not second)
        if second:
            torch.testing.assert_close(got[1].cpu().float(), ref[1].float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("F", [8, 100, 1024, 333])
def test_gated_activation(dtype, F):
    _need()
    g = torch.Generator().manual_seed(F)
    x = (torch.randn(11, 2 * F, generator=g) * 2).to(dtype)
    for kind in ("gelu_tanh", "silu"):
        ref = torch_ref.glu_activation(x, kind)
        got = ops.glu_activation(x.to(DEV), kind)
        torch.testing.assert_close(got.cpu().float(), ref.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Dv,rot,inter,pad", [(12, 4, 64, 32, 24, False, 0), (4, 2, 40, 56, 8, False, 0), (3, 3, 16, 6, 0, False, 0), (5, 1, 10, 10, 10, True, 0),
                                                     (4, 1, 64, 32, 32, True, 128), (8, 2, 128, 128, 64, False, 128), (2, 2, 24, 18, 4, True, 0)])
def test_attention_prepare_rotates_values(H, G, D, Dv, rot, inter, pad, dtype):
    _need()
    g = torch.Generator().manual_seed(H * 100 + D)
    T, slots = 13, 64
    n = H * D + G * D + G * Dv
    qkv = torch.randn(T, n + 5, generator=g).to(dtype)
    pos = torch.randint(0, 3000, (T,), generator=g).int()
    loc = torch.randperm(slots, generator=g)[:T].int()
    f = scaled_inv_freq(rot, 3e4) if rot else None
    fv = scaled_inv_freq(Dv, 3e4)
    width = G * (pad if pad else max(D, Dv)) + 8
    kr, vr = torch.zeros(slots, 1, width, dtype=dtype), torch.zeros(slots, 1, width, dtype=dtype)
    kg, vg = kr.clone().to(DEV), vr.clone().to(DEV)
    ref = torch_ref.attention_prepare(qkv[:, :n], H, G, D, Dv, pos, kr, vr, loc, None, None, 0.0, f, None, 0.0, pad, fv, inter)
    got = ops.attention_prepare(qkv.to(DEV)[:, :n], H, G, D, Dv, pos.to(DEV), kg, vg, loc.to(DEV), None, None, 0.0, f.to(DEV) if rot else None, None, 0.0,
                                pad, fv.to(DEV), inter)
    torch.testing.assert_close(got.cpu().float(), ref.float(), **_tol(dtype, f32=(2e-4, 2e-4)))
    torch.testing.assert_close(kg.cpu().float(), kr.float(), **_tol(dtype, f32=(2e-4, 2e-4)))
    torch.testing.assert_close(vg.cpu().float(), vr.float(), **_tol(dtype, f32=(2e-4, 2e-4)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Dv,hs,inter,sink", [(5, 32, 32, False, False), (3, 10, 10, True, False), (4, 64, 128, False, True), (5, 128, 128, True, True), (2, 6, 9, False, False)])
def test_rotate_heads(H, Dv, hs, inter, sink, dtype):
    _need()
    g = torch.Generator().manual_seed(Dv)
    T = 17
    o = torch.randn(T, H, hs, generator=g).to(dtype)
    pos = torch.randint(0, 5000, (T,), generator=g).int()
    f = scaled_inv_freq(Dv, 1e4)
    lse = torch.randn(T, H, generator=g) if sink else None
    sinks = torch.randn(H, generator=g) * 0.3 if sink else None
    for inverse in (True, False):
        ref = torch_ref.rotate_heads(o, pos, f, Dv, inter, inverse, lse, sinks)
        got = ops.rotate_heads(o.to(DEV), pos.to(DEV), f.to(DEV), Dv, inter, inverse, lse.to(DEV) if sink else None, sinks.to(DEV) if sink else None)
        torch.testing.assert_close(got.cpu().float(), ref.float(), **_tol(dtype, f32=(3e-4, 3e-4)))
    # turning there and back is the identity
    there = ops.rotate_heads(o.to(DEV)[:, :, :Dv].contiguous().float(), pos.to(DEV), f.to(DEV), Dv, inter, False)
    back = ops.rotate_heads(there.view(T, H, Dv), pos.to(DEV), f.to(DEV), Dv, inter, True)
    torch.testing.assert_close(back.cpu().view(T, H, Dv), o[:, :, :Dv].float(), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Rq,R,Dr,scaled", [(96, 48, 24, True), (24, 40, 8, False), (0, 16, 0, False), (96, 512, 64, True), (7, 9, 2, True)])
def test_latent_prepare_and_query(Rq, R, Dr, scaled, dtype):
    _need()
    g = torch.Generator().manual_seed(R)
    T, slots, H, D = 11, 40, 3, 12
    x = torch.randn(T, Rq + R + Dr + 3, generator=g).to(dtype)
    pos = torch.randint(0, 4000, (T,), generator=g).int()
    loc = torch.randperm(slots, generator=g)[:T].int()
    f, mult = yarn_inv_freq(Dr, 2e5, {"factor": 4.0, "original": 256, "fast": 32.0, "slow": 1.0} if scaled else None) if Dr else (None, 1.0)
    wq, wk = (torch.randn(max(Rq, 1), generator=g) * 0.1 + 1).to(dtype), (torch.randn(R, generator=g) * 0.1 + 1).to(dtype)
    cr = torch.zeros(slots, 1, R + Dr + 8, dtype=dtype)
    cg = cr.clone().to(DEV)
    ref = torch_ref.latent_prepare(x, Rq, wq[:Rq], R, Dr, wk, 1e-6, pos, f, mult, cr, loc)
    got = ops.latent_prepare(x.to(DEV), Rq, wq[:Rq].to(DEV) if Rq else None, R, Dr, wk.to(DEV), 1e-6, pos.to(DEV), f.to(DEV) if Dr else None, mult, cg, loc.to(DEV))
    torch.testing.assert_close(cg.cpu().float(), cr.float(), **_tol(dtype, f32=(2e-4, 2e-4)))
    if Rq:
        torch.testing.assert_close(got.cpu().float(), ref.float(), **_tol(dtype))
    else:
        assert got is None and ref is None
    q = torch.randn(T, H, D + Dr, generator=g).to(dtype)
    q_abs = torch.randn(H, T, R, generator=g)
    ref = torch_ref.latent_query(q, q_abs, D, Dr, pos, f, mult)
    got = ops.latent_query(q.to(DEV), q_abs.to(DEV), D, Dr, pos.to(DEV), f.to(DEV) if Dr else None, mult)
    torch.testing.assert_close(got.cpu(), ref, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,Rv,ps", [(8, 96, 64, 64), (3, 24, 16, 16), (16, 576, 512, 64), (2, 9, 5, 8), (4, 40, 40, 32)])
def test_latent_attention_with_a_score_only_part(H, R, Rv, ps, dtype):
    _need()
    g = torch.Generator().manual_seed(R)
    for q_lens, cached in (([5, 130, 1, 33], [0, 70, 299, 31]), ([1, 1, 1], [0, 257, 63])):
        cu, seq = _ragged(q_lens, cached)
        pt, cache, _ = _paged(len(q_lens), max(seq), ps, R + 8, dtype, g)
        T = sum(q_lens)
        q = torch.randn(T, H, R, generator=g) * 0.5
        slots = _i32(list(range(1, len(q_lens) + 1)))
        dec = all(n == 1 for n in q_lens)
        ref = torch_ref.latent_attention(q, cache, R, pt, slots.cpu(), torch.tensor(seq), None if dec else torch.tensor(q_lens), ps, 0.2, -1, None, Rv)
        got = ops.latent_attention(q.to(DEV), cache.to(DEV), R, pt.to(DEV), slots, _i32(seq), None if dec else _i32(cu), None if dec else _i32(q_lens),
                                   max(q_lens), ps, 0.2, -1, None, max(seq), v_rank=Rv)
        assert got.shape == (T, H, Rv)
        torch.testing.assert_close(got.cpu(), ref, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Dv,cap", [(2, 48, 32, 9.0), (3, 5, 7, 0.0), (4, 128, 128, 15.0), (1, 17, 130, 8.0), (8, 64, 32, 11.0)])
def test_mlstm_prepare_scan_readout(H, D, Dv, cap, dtype):
    _need()
    g = torch.Generator().manual_seed(H * 7 + D)
    slots_n = 6
    state_r = torch.randn(slots_n, H, D, Dv + 1, generator=g) * 0.1
    m_r = torch.randn(slots_n, H, generator=g)
    state_g, m_g = state_r.clone().to(DEV), m_r.clone().to(DEV)
    nw = (torch.randn(H * Dv, generator=g) * 0.1 + 1).to(dtype)
    for q_lens, cached, slots in (([70, 3, 1, 40], [0, 5, 9, 0], [2, 1, 4, 5]), ([1, 1, 1], [70, 8, 0], [2, 1, 3]), ([2, 33], [71, 0], [2, 0])):
        cu, seq = _ragged(q_lens, cached)
        T = sum(q_lens)
        dec = all(n == 1 for n in q_lens)
        proj = torch.randn(T, 2 * H * D + 2 * H * Dv + 4, generator=g).to(dtype)
        raw = torch.randn(T, 2 * H, generator=g) * 6
        raw[:, H:] += 3.0
        sl = torch.tensor(slots, dtype=torch.int32)
        ql = None if dec else torch.tensor(q_lens)
        u_r, g_r = torch_ref.mlstm_prepare(proj, raw, H, D, Dv, cap, m_r, sl, torch.tensor(seq), ql)
        u_g, g_g = ops.mlstm_prepare(proj.to(DEV), raw.to(DEV), H, D, Dv, cap, m_g, sl.to(DEV), _i32(seq), None if dec else _i32(cu), None if dec else _i32(q_lens))
        torch.testing.assert_close(u_g.cpu(), u_r, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(g_g.cpu(), g_r, rtol=1e-4, atol=1e-6)
        torch.testing.assert_close(m_g.cpu(), m_r, rtol=1e-5, atol=1e-5)
        y_r = torch_ref.mamba2_scan(u_r, None, None, None, None, None, state_r, sl, torch.tensor(seq), ql, H, Dv + 1, D, H, None, g_r)
        y_g = ops.mamba2_scan(u_g, None, None, None, None, None, state_g, sl.to(DEV), _i32(seq), None if dec else _i32(cu), None if dec else _i32(q_lens),
                              H, Dv + 1, D, H, gates=g_g)
        torch.testing.assert_close(y_g.cpu(), y_r, rtol=2e-4, atol=2e-4)
        torch.testing.assert_close(state_g.cpu(), state_r, rtol=2e-4, atol=2e-4)
        n = 2 * H * D + H * Dv
        o_r = torch_ref.mlstm_readout(y_r, g_r, H, Dv, nw, 1e-6, proj[:, n:n + H * Dv], dtype)
        o_g = ops.mlstm_readout(y_g, g_g, H, Dv, nw.to(DEV), 1e-6, proj.to(DEV)[:, n:n + H * Dv], dtype)
        torch.testing.assert_close(o_g.cpu().float(), o_r.float(), **_tol(dtype, f32=(1e-3, 1e-3)))


# ------------------------------------------------------------------ a far key, a key at a page border and the sink on the kernels (both attention routes)
def _attend_cuda(H, G, D, Dv, qkv, ps, scale, cap, dtype, tc):
    """attention of ONE request on the kernels: preparation with rotated values, the general kernel or the tcgen05 kernels (heads laid out 128
    wide) with cap and unit sink over a paged cache whose pages lie in reverse order, back-rotation"""
    T = qkv.shape[0]
    n_pages = (T + ps - 1) // ps
    pt = torch.zeros(2, n_pages + 1, dtype=torch.int32)
    pt[1, :n_pages] = torch.arange(n_pages, 0, -1, dtype=torch.int32) + 2
    loc = torch.tensor([int(pt[1, t // ps]) * ps + t % ps for t in range(T)], dtype=torch.int32).to(DEV)
    pad = 128 if tc else 0
    width = G * (pad if pad else max(D, Dv))
    kc, vc = torch.zeros((n_pages + 4) * ps, 1, width, dtype=dtype, device=DEV), torch.zeros((n_pages + 4) * ps, 1, width, dtype=dtype, device=DEV)
    fv = scaled_inv_freq(Dv, 100.0).to(DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    q = ops.attention_prepare(qkv.to(dtype).to(DEV), H, G, D, Dv, pos, kc, vc, loc, None, None, 0.0, None, None, 0.0, pad, fv, False)
    sinks = torch.zeros(H, device=DEV)
    slots, seq, cu, ql = _i32([1]), _i32([T]), _i32([0, T]), _i32([T])
    if tc:
        k4, v4 = kc.view(-1, G, 128), vc.view(-1, G, 128)
        assert ops.tc_attention_ok(q, k4, v4, ps)
        lse = torch.empty(T, H, dtype=torch.float32, device=DEV)
        o = ops.paged_attention(q, k4, v4, pt.to(DEV), slots, seq, cu, ql, T, ps, scale, causal=True, logit_cap=cap, lse=lse)
        return ops.rotate_heads(o, pos, fv, Dv, False, True, lse, sinks).view(T, H, Dv).float().cpu()
    o = ops.window_attention(q, kc, vc, G, Dv, pt.to(DEV), slots, seq, cu, ql, T, ps, scale, cap, -1, None, sinks, D, 0)
    return ops.rotate_heads(o.view(T, H, Dv), pos, fv, Dv, False, True).view(T, H, Dv).float().cpu()


@pytest.mark.parametrize("tc,dtype", [(False, torch.float32), (False, torch.bfloat16), (True, torch.bfloat16)])
def test_far_key_page_border_and_sink_on_the_kernels(tc, dtype):
    _need()
    import rumuvik_oracle as O

    H, G, D, Dv, ps = 2, 1, 8, 6, 16
    tol = 2e-3 if dtype == torch.float32 else 5e-2
    for T, far in ((300, 3), (300, 15), (300, 16), (129, 127), (64, 0)):
        g = torch.Generator().manual_seed(T + far)
        qkv = torch.randn(T, H * D + G * D + G * Dv, generator=g) * 0.1
        kdir = torch.randn(D, generator=g)
        kdir = kdir / kdir.norm()
        qkv[far, H * D:H * D + D] = 6.0 * kdir
        qkv[T - 1, :D] = 6.0 * kdir
        val = torch.randn(Dv, generator=g)
        qkv[far, H * D + D:] = val
        o = _attend_cuda(H, G, D, Dv, qkv, ps, 1.0, 0.0, dtype, tc)
        want = O.turn(val.double()[None, None, :], [T - 1 - far], O.frequencies(100.0, Dv), "halves", back=True)[0, 0]
        torch.testing.assert_close(o[T - 1, 0].double(), want, rtol=tol, atol=tol)
        assert float((o[T - 1, 1].double() - want).abs().max()) > 0.1
    # one key and the sink: the key's share of the value
    for qv, scale, cap in ((1.0, 1.0, 0.0), (1.0, 0.25, 0.0), (1.0, 5.0, 3.0), (-1.0, 4.0, 0.0), (-1.0, 4.0, 2.0)):
        qkv = torch.zeros(1, H * D + G * D + G * Dv)
        qkv[0, 0], qkv[0, H * D], qkv[0, H * D + D:H * D + D + 2] = qv, 2.0, torch.tensor([3.0, -1.0])
        s = 2.0 * qv * scale
        if cap:
            s = cap * np.tanh(s / cap)
        share = np.exp(s) / (1.0 + np.exp(s))
        o = _attend_cuda(H, G, D, Dv, qkv, ps, scale, cap, dtype, tc)
        torch.testing.assert_close(o[0, 0, :2], torch.tensor([3.0, -1.0]) * share, rtol=tol, atol=tol * 0.1)


# ------------------------------------------------------------------ the engine on CUDA against the oracle
def _engine_case(tmp_path, dtype, cfg, seed, tol, gen=True, spikes=False):
    """``spikes``: tiny or drawn stacks, where single positions are badly conditioned in bf16 whatever kernel runs (a normaliser or a norm over a
    handful of numbers near zero; the same positions stand out with the tcgen05 route, the expanded route or neither): those cases bound a
    high quantile and the mean over all compared positions, the fixed lane-friendly configuration bounds the maximum"""
    from test_rumuvik import Harness, _tokens

    h = Harness(tmp_path, cfg, seed=seed, slots=4, max_tokens=1024, device="cuda", dtype=dtype, page=16)
    V = cfg["vocab"]
    a, b, c = _tokens(150, V, 1), _tokens(41, V, 2), _tokens(3, V, 3)
    ra, rb, rc = h.oracle(a), h.oracle(b), h.oracle(c)
    scale = float(np.abs(ra).mean()) + 1e-6
    errs = []

    def close(x, y):
        if dtype == "float32":
            err = np.abs(x - y).max(-1) / scale
            assert float(err.max()) < tol, float(err.max())
            return
        # bf16: per position, the root mean square over the vocabulary of the difference against that of the logits (means taken off)
        d, r = x - y, y - y.mean(-1, keepdims=True)
        d = d - d.mean(-1, keepdims=True)
        errs.append(np.sqrt((d ** 2).mean(-1)) / np.sqrt((r ** 2).mean(-1) + 1e-12))

    close(h.step([("a", a, range(len(a)))], ["a"]), ra)                                            # whole
    close(h.run_cut("a2", a, [100, 2, 17]), ra)                                                    # portions, then token by token
    out = h.step([("a", a[:90], range(90)), ("b", b[:7], range(7)), ("c", c, range(3))], ["c"])    # unequal batch
    close(out[:90], ra[:90]); close(out[90:97], rb[:7]); close(out[97:], rc)
    out = h.step([("a", a[90:], range(60)), ("b", b[7:8], range(1))], ["a"])
    close(out[:60], ra[90:]); close(out[60:], rb[7:8])
    out = h.step([("b", b[8:], range(len(b) - 8)), ("d", c, range(3))], ["b", "d"])                # "d" reuses a freed slot and pages
    close(out[:len(b) - 8], rb[8:]); close(out[len(b) - 8:], rc)
    if errs:
        err = np.concatenate(errs)
        if spikes:
            assert float(np.quantile(err, 0.9)) < tol and float(err.mean()) < 0.5 * tol and float(err.max()) < 1.0, (float(np.quantile(err, 0.9)), float(err.mean()), float(err.max()))
        else:
            assert float(err.max()) < tol and float(err.mean()) < 0.4 * tol, (float(err.max()), float(err.mean()))
    if dtype == "float32" and gen:  # greedy generation through the engine's own entry point, scheduler and sampler
        prompts = [b[:9], c]
        outs = h.eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 6, "temperature": 0, "ignore_eos": True})
        for pr, o in zip(prompts, outs):
            seq = list(pr)
            for _ in range(6):
                seq.append(int(h.oracle(seq)[-1].argmax()))
            assert o["output_ids"] == seq[len(pr):]
    h.close()


def _wide():
    """lane-friendly sizes: bf16 attention layers with group sizes 4 and 1 take the tcgen05 kernels (heads laid out 128 wide), the layer with
    three query heads per key head the general kernel"""
    from test_rumuvik import L, _attn, _cfg, _dense, _lat, _ml

    return _cfg([L(_ml(heads=2, dim=32, vdim=64, gate_cap=10.0), _dense(128)), L(_attn(heads=8, kv_heads=2, dim=64, vdim=64, rot_dims=32, base=1e4, scale=0.2, softcap=20.0), _dense(64)),
                 L(_lat(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=48, scale=0.15), _dense(64)),
                 L(_attn(heads=2, kv_heads=2, dim=128, vdim=32, rot_dims=128, base=50.0, scale=0.1, softcap=0), None),
                 L(_attn(heads=6, kv_heads=2, dim=32, vdim=48, rot_dims=8, scale=0.25), _dense(32))], width=128, vocab=256, loop=(1, 4, 2), scale=4.0)


def test_engine_on_cuda_fp32(tmp_path):
    from test_rumuvik import MIXED

    _need()
    _engine_case(tmp_path, "float32", MIXED, 1, 3e-4)


def test_engine_on_cuda_bf16(tmp_path):
    from test_rumuvik import MIXED

    _need()
    _engine_case(tmp_path, "bfloat16", MIXED, 2, 0.12, spikes=True)


def test_engine_on_cuda_lane_friendly_sizes_fp32(tmp_path):
    _need()
    _engine_case(tmp_path, "float32", _wide(), 3, 3e-4)


def test_engine_on_cuda_lane_friendly_sizes_bf16(tmp_path):
    _need()
    _engine_case(tmp_path, "bfloat16", _wide(), 4, 0.12)


def test_tensor_core_route_agrees_with_the_general_kernel(tmp_path, monkeypatch):
    """the same bf16 model with and without the tcgen05 route: both within the bf16 tolerance of the oracle (the route is taken: its layers are padded)"""
    from sglang_b200.layers.gated_attention import GatedAttention
    from test_rumuvik import Harness

    _need()
    h = Harness(tmp_path, _wide(), seed=5, slots=2, max_tokens=512, device="cuda", dtype="bfloat16", page=16)
    pads = [b.mix.pad for b in h.model.model.all_layers if b.kind == "attention"]
    h.close()
    assert pads == [128, 128, 0]
    monkeypatch.setattr(GatedAttention, "tc_route", False)
    _engine_case(tmp_path / "general", "bfloat16", _wide(), 5, 0.12)


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
def test_engine_on_cuda_randomly_drawn_stacks_fp32(tmp_path, seed):
    from test_rumuvik import drawn_config

    _need()
    _engine_case(tmp_path, "float32", drawn_config(seed, friendly=seed % 2 == 0), seed, 2e-3, gen=False)


@pytest.mark.parametrize("seed", [21, 22, 23])
def test_engine_on_cuda_randomly_drawn_stacks_bf16(tmp_path, seed):
    from test_rumuvik import drawn_config

    _need()
    _engine_case(tmp_path, "bfloat16", drawn_config(seed, friendly=True), seed, 0.15, spikes=True)


@pytest.mark.parametrize("seed", [31, 32, 33])
def test_engine_on_cuda_randomly_drawn_stacks_of_odd_sizes_bf16(tmp_path, seed):
    """widths, head sizes, ranks and vocabularies that are no multiples of the vector widths: every kernel takes its scalar path, the GEMMs
    their general one"""
    from test_rumuvik import drawn_config

    _need()
    _engine_case(tmp_path, "bfloat16", drawn_config(seed), seed, 0.25, spikes=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,tq,n,first", [(3, 5, 9, 2), (2, 64, 300, 236), (4, 33, 33, 0), (1, 7, 1000, 10), (2, 3, 5000, 4996)])
def test_causal_softmax(H, tq, n, first, dtype):
    _need()
    g = torch.Generator().manual_seed(n)
    s = torch.randn(H * tq, n, generator=g) * 4
    for scale in (0.3, 1.0):
        ref = torch_ref.causal_softmax(s, tq, first, scale, dtype)
        got = ops.causal_softmax(s.to(DEV), tq, first, scale, dtype)
        torch.testing.assert_close(got.cpu().float(), ref.float(), **_tol(dtype, f32=(1e-5, 1e-6), bf=(1e-2, 1e-3)))
        assert float(got[:, min(n, first + tq):].abs().max()) == 0.0 if first + tq < n else True


def test_latent_prompts_as_two_matrix_products(tmp_path, monkeypatch):
    """long bf16 prompt portions of latent attention run Q K^T and P V as batched GEMMs around the soft-max kernel: against the oracle, beside the
    attention-kernel form of the same route, alone, over cached rows, and beside short portions and decode tokens of other requests"""
    from sglang_b200.layers.latent_attention import RotaryLatentAttention
    from test_rumuvik import Harness, L, _cfg, _dense, _lat, _tokens

    _need()
    calls = []
    real = RotaryLatentAttention._attend_by_gemms
    monkeypatch.setattr(RotaryLatentAttention, "_attend_by_gemms", lambda self, *a: (calls.append(1), real(self, *a))[1])
    monkeypatch.setattr(RotaryLatentAttention, "GEMM_SCORE_BYTES", 1 << 18)              # several query chunks per request
    cfg = _cfg([L(_lat(heads=4, dim=32, rot_dim=16, vdim=48, kv_rank=64, q_rank=48, scale=0.15), _dense(64)),
                L(_lat(heads=2, dim=64, rot_dim=0, vdim=32, kv_rank=96, q_rank=32, scaling=None, scale=0.12), None)], width=128, vocab=256, scale=4.0)
    h = Harness(tmp_path, cfg, seed=7, slots=4, max_tokens=2048, device="cuda", dtype="bfloat16", page=16)
    a, b, c = _tokens(700, 256, 1), _tokens(300, 256, 2), _tokens(40, 256, 3)
    ra, rb, rc = h.oracle(a), h.oracle(b), h.oracle(c)

    def err(x, y):
        d, r = x - y, y - y.mean(-1, keepdims=True)
        d = d - d.mean(-1, keepdims=True)
        return np.sqrt((d ** 2).mean(-1)) / np.sqrt((r ** 2).mean(-1) + 1e-12)

    e1 = err(h.step([("a", a, range(len(a)))], ["a"]), ra)                                # one long prompt
    assert len(calls) == 2
    out = h.step([("a", a[:300], range(300)), ("b", b[:5], range(5)), ("c", c, range(40))], ["c"])
    e2 = np.concatenate([err(out[:300], ra[:300]), err(out[300:305], rb[:5]), err(out[305:], rc)])
    out = h.step([("a", a[300:], range(400)), ("b", b[5:6], range(1))], ["a"])           # 400 more over 300 cached rows, beside a decode token
    e3 = np.concatenate([err(out[:400], ra[300:]), err(out[400:], rb[5:6])])
    out = h.step([("b", b[6:], range(294))], ["b"])
    e4 = err(out, rb[6:])
    assert len(calls) == 8
    monkeypatch.setattr(RotaryLatentAttention, "gemm_prefill", False)
    e0 = err(h.step([("a", a, range(len(a)))], ["a"]), ra)                                # the same route on the attention kernel
    assert len(calls) == 8
    h.close()
    for e in (e1, e2, e3, e4):
        assert float(e.max()) < 0.1 and float(e.mean()) < 1.5 * float(e0.mean()) + 0.005, (float(e.max()), float(e.mean()), float(e0.mean()))
