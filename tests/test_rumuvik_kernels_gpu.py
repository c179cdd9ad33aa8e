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
@pytest.mark.parametrize("H,G,D,Dv,rot,inter,pad", [(6, 2, 64, 64, 16, False, 0), (4, 2, 40, 56, 8, False, 0), (3, 3, 16, 6, 0, False, 0), (5, 1, 10, 10, 10, True, 0),
                                                     (4, 1, 64, 32, 32, True, 128), (8, 2, 128, 128, 64, False, 128), (2, 2, 24, 18, 4, True, 0)])
def test_attention_prepare_rotates_values(H, G, D, Dv, rot, inter, pad, dtype):
    _need()
    g = torch.Generator().manual_seed(H * 100 + D)
    T, slots = 13, 64
    n = H * D + G * D + G * Dv
    qkv = torch.randn(T, n + 5, generator=g).to(dtype)
    pos = torch.randint(0, 3000, (T,), generator=g).int()
    loc = torch.randperm(slots, generator=g)[:T].int()
    f = scaled_inv_freq(rot, 5e4) if rot else None
    fv = scaled_inv_freq(Dv, 5e4)
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
@pytest.mark.parametrize("H,Dv,hs,inter,sink", [(6, 64, 64, False, False), (3, 10, 10, True, False), (4, 64, 128, False, True), (5, 128, 128, True, True), (2, 6, 9, False, False)])
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
@pytest.mark.parametrize("Rq,R,Dr,scaled", [(128, 64, 16, True), (24, 40, 8, False), (0, 16, 0, False), (96, 512, 64, True), (7, 9, 2, True)])
def test_latent_prepare_and_query(Rq, R, Dr, scaled, dtype):
    _need()
    g = torch.Generator().manual_seed(R)
    T, slots, H, D = 11, 40, 3, 12
    x = torch.randn(T, Rq + R + Dr + 3, generator=g).to(dtype)
    pos = torch.randint(0, 4000, (T,), generator=g).int()
    loc = torch.randperm(slots, generator=g)[:T].int()
    f, mult = yarn_inv_freq(Dr, 1e6, {"factor": 4.0, "original": 256, "fast": 32.0, "slow": 1.0} if scaled else None) if Dr else (None, 1.0)
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
@pytest.mark.parametrize("H,R,Rv,ps", [(6, 80, 64, 64), (3, 24, 16, 16), (16, 576, 512, 64), (2, 9, 5, 8), (4, 40, 40, 32)])
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
@pytest.mark.parametrize("H,D,Dv,cap", [(2, 32, 64, 12.0), (3, 5, 7, 0.0), (4, 128, 128, 15.0), (1, 17, 130, 8.0), (8, 64, 32, 12.0)])
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
