"""Resatar CUDA kernels against their fp32 PyTorch references (``ops/torch_ref.py``) and the engine on CUDA against the plain oracle."""
import numpy as np
import pytest
import torch

from sglang_b200 import ops
from sglang_b200.layers.gated_attention import GatedAttention, scaled_inv_freq
from sglang_b200.ops import moe_ops, torch_ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _need():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    assert ops.load_native(), "the CUDA extension must be built on a GPU box"


def _i32(x, dev=DEV):
    return torch.tensor(x, dtype=torch.int32, device=dev)


def _ragged(q_lens, cached):
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    seq = [c + q for c, q in zip(cached, q_lens)]
    return cu.tolist(), seq


def _tol(dtype, f32=(1e-5, 1e-5), bf=(2e-2, 2e-2)):
    r, a = bf if dtype == torch.bfloat16 else f32
    return dict(rtol=r, atol=a)


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
@pytest.mark.parametrize("W", [24, 256, 1000])
def test_scalar_sandwich_norm_and_gated_norm(dtype, W):
    _need()
    g = torch.Generator().manual_seed(0)
    x, d = torch.randn(9, W, generator=g), torch.randn(9, W, generator=g).to(dtype)
    pw, w = torch.tensor([1.3]).to(dtype), torch.tensor([0.7]).to(dtype)
    for zc in (False, True):
        r1, r2 = x.clone(), x.clone().to(DEV)
        ref = torch_ref.postnorm_add_rmsnorm_f32(r1, d, pw, w, 1e-5, dtype, zc)
        got = ops.add_rmsnorm_f32(r2, d.to(DEV), w.to(DEV), 1e-5, zc, dtype, pw.to(DEV))
        torch.testing.assert_close(r2.cpu(), r1, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(got.cpu().float(), ref.float(), **_tol(dtype))
        r1, r2 = x.clone(), x.clone().to(DEV)                   # no post-norm: plain add, scalar gain
        ref = torch_ref.add_rmsnorm_f32(r1, d, w, 1e-5, zc, dtype)
        got = ops.add_rmsnorm_f32(r2, d.to(DEV), w.to(DEV), 1e-5, zc, dtype)
        torch.testing.assert_close(got.cpu().float(), ref.float(), **_tol(dtype))
    # vector weights still work next to scalar ones
    wv, pv = torch.randn(W, generator=g).to(dtype), torch.randn(W, generator=g).to(dtype)
    r1, r2 = x.clone(), x.clone().to(DEV)
    ref = torch_ref.postnorm_add_rmsnorm_f32(r1, d, pv, wv, 1e-5, dtype, False)
    got = ops.add_rmsnorm_f32(r2, d.to(DEV), wv.to(DEV), 1e-5, False, dtype, pv.to(DEV))
    torch.testing.assert_close(got.cpu().float(), ref.float(), **_tol(dtype))
    # gated norm into a column block of a wider buffer
    y, gate, nw = torch.randn(9, W, generator=g), torch.randn(9, W + 16, generator=g).to(dtype), torch.randn(W, generator=g).to(dtype)
    ref = torch_ref.grouped_rmsnorm(y, nw, 1, 1e-5, dtype, gate[:, 8:8 + W], 1.1)
    buf = torch.zeros(9, W + 40, dtype=dtype, device=DEV)
    ops.grouped_rmsnorm(y.to(DEV), nw.to(DEV), 1, 1e-5, dtype, gate.to(DEV)[:, 8:8 + W], 1.1, buf[:, 24:24 + W])
    torch.testing.assert_close(buf[:, 24:24 + W].cpu().float(), ref.float(), **_tol(dtype))
    assert float(buf[:, :24].abs().max()) == 0.0 and float(buf[:, 24 + W:].abs().max()) == 0.0


@pytest.mark.parametrize("kind", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activation(kind, dtype):
    _need()
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(13, 77, generator=g) * 3).to(dtype)
    xf = x[:, 5:60].float()
    want = torch.nn.functional.silu(xf) if kind == "silu" else 0.5 * xf * (1 + torch.tanh(0.7978845608028654 * (xf + 0.044715 * xf ** 3)))
    for od in (torch.float32, dtype):
        got = ops.activation(x.to(DEV)[:, 5:60], kind, od)
        assert got.dtype == od and got.is_contiguous()
        torch.testing.assert_close(got.cpu().float(), want, **_tol(od, (1e-5, 1e-6)))


@pytest.mark.parametrize("C,N", [(256, 20), (7, 1), (33, 4), (20, 9), (130, 16), (64, 33), (12, 100), (5, 200), (5000, 16), (2600, 12), (1300, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selective_scan(C, N, dtype):
    _need()
    g = torch.Generator().manual_seed(2)
    q_lens, cached = [37, 1, 2, 50], [12, 9, 0, 0]
    cu, seq = _ragged(q_lens, cached)
    T = sum(q_lens)
    u, dt_raw = torch.randn(T, C, generator=g), torch.randn(T, C, generator=g)
    low = torch.randn(T, 3 + 2 * N, generator=g).to(dtype)      # B and C are column views of a wider projection
    zz = torch.randn(T, 2 * C, generator=g).to(dtype)
    dtb, A_log, D = torch.randn(C, generator=g), torch.randn(C, N, generator=g) * 0.5, torch.randn(C, generator=g)
    state = torch.randn(6, 1, C, N, generator=g)
    slots = [4, 1, 3, 2]
    s1, s2 = state.clone(), state.clone().to(DEV)
    ref = torch_ref.mamba1_scan(u, dt_raw, dtb, A_log, low[:, 3:3 + N], low[:, 3 + N:], D, zz[:, C:], s1, _i32(slots, "cpu"), _i32(seq, "cpu"), _i32(q_lens, "cpu"),
                                dtype)
    lg, zg = low.to(DEV), zz.to(DEV)
    got = ops.mamba1_scan(u.to(DEV), dt_raw.to(DEV), dtb.to(DEV), A_log.to(DEV), lg[:, 3:3 + N], lg[:, 3 + N:], D.to(DEV), zg[:, C:], s2, _i32(slots), _i32(seq),
                          _i32(cu), _i32(q_lens), dtype)
    torch.testing.assert_close(got.cpu().float(), ref.float(), **_tol(dtype, (2e-4, 2e-4), (3e-2, 3e-2)))
    torch.testing.assert_close(s2.cpu(), s1, rtol=2e-4, atol=2e-4)
    # decode form on the continued state, no gate, no skip, no bias
    B = 4
    ref = torch_ref.mamba1_scan(u[:B], dt_raw[:B], None, A_log, low[:B, 3:3 + N], low[:B, 3 + N:], None, None, s1, _i32(slots, "cpu"),
                                _i32([s + 1 for s in seq], "cpu"), None, torch.float32)
    got = ops.mamba1_scan(u[:B].to(DEV), dt_raw[:B].to(DEV), None, A_log.to(DEV), lg[:B, 3:3 + N], lg[:B, 3 + N:], None, None, s2, _i32(slots),
                          _i32([s + 1 for s in seq]), None, None, torch.float32)
    torch.testing.assert_close(got.cpu(), ref, rtol=3e-4, atol=3e-4)
    torch.testing.assert_close(s2.cpu(), s1, rtol=3e-4, atol=3e-4)


@pytest.mark.parametrize("H,D,Dv", [(2, 64, 64), (3, 5, 7), (4, 128, 32), (1, 17, 130)])
def test_constant_decay_mode_of_the_scan(H, D, Dv):
    _need()
    g = torch.Generator().manual_seed(3)
    q_lens, cached = [45, 1, 3, 70], [8, 30, 0, 0]
    cu, seq = _ragged(q_lens, cached)
    T = sum(q_lens)
    u = torch.randn(T, H * Dv + 2 * H * D, generator=g) * 0.5
    decay = torch.rand(H, generator=g) * 0.5 + 0.5
    decay[0] = 1.0
    state = torch.randn(6, H, D, Dv, generator=g)
    slots = [2, 5, 1, 3]
    s1, s2 = state.clone(), state.clone().to(DEV)
    ref = torch_ref.mamba2_scan(u, None, None, None, None, None, s1, _i32(slots, "cpu"), _i32(seq, "cpu"), _i32(q_lens, "cpu"), H, Dv, D, H, decay)
    got = ops.mamba2_scan(u.to(DEV), None, None, None, None, None, s2, _i32(slots), _i32(seq), _i32(cu), _i32(q_lens), H, Dv, D, H, decay.to(DEV))
    torch.testing.assert_close(got.cpu(), ref, rtol=3e-4, atol=3e-4)
    torch.testing.assert_close(s2.cpu(), s1, rtol=3e-4, atol=3e-4)


@pytest.mark.parametrize("H,G,D,Dv,rot", [(5, 1, 80, 48, 80), (6, 2, 10, 7, 4), (4, 2, 40, 56, 0), (3, 3, 128, 128, 64), (8, 2, 20, 36, 20)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_prepare(H, G, D, Dv, rot, dtype):
    _need()
    g = torch.Generator().manual_seed(4)
    T, ps = 75, 16
    pos = torch.randint(0, 3000, (T,), generator=g).int()
    loc = torch.randperm(200, generator=g)[:T].int()
    qkv = torch.randn(T, (H + G) * D + G * Dv + 11, generator=g).to(dtype)
    vf = torch.randn(T, G * Dv + 5, generator=g).to(dtype)
    qw, kw = torch.randn(H * D, generator=g).to(dtype), torch.randn(G * D, generator=g).to(dtype)
    fr = scaled_inv_freq(rot, 10000.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}) if rot else None
    for norm, mix, pad in ((True, True, 0), (False, False, 0), (True, False, 0), (False, True, 128 if max(D, Dv) <= 128 else 0)):
        w = G * (pad if pad else max(D, Dv)) + 8
        k1, v1 = torch.full((200, 1, w), 3.0, dtype=dtype), torch.full((200, 1, w), 3.0, dtype=dtype)
        k2, v2 = k1.clone().to(DEV), v1.clone().to(DEV)
        a = (qw, kw, 1e-5) if norm else (None, None, 0.0)
        b = (vf[:, 2:2 + G * Dv], 0.35) if mix else (None, 0.0)
        q_ref = torch_ref.attention_prepare(qkv, H, G, D, Dv, pos, k1, v1, loc, *a, fr, *b, pad)
        dv = lambda t: None if t is None else t.to(DEV)
        q_got = ops.attention_prepare(qkv.to(DEV), H, G, D, Dv, pos.to(DEV), k2, v2, loc.to(DEV), dv(a[0]), dv(a[1]), a[2], dv(fr),
                                      None if b[0] is None else vf.to(DEV)[:, 2:2 + G * Dv], b[1], pad)
        tol = _tol(dtype, (2e-4, 2e-4), (2e-2, 3e-2))             # angles up to 3000 rad in fp32
        torch.testing.assert_close(q_got.cpu().float(), q_ref.float(), **tol)
        torch.testing.assert_close(k2.cpu().float(), k1.float(), **tol)
        torch.testing.assert_close(v2.cpu().float(), v1.float(), **tol)


@pytest.mark.parametrize("H,G,D,Dv,window,keep", [(4, 2, 40, 56, 60, 5), (6, 2, 10, 7, 5, 9), (4, 4, 32, 48, -1, 3), (32, 1, 16, 16, 33, 1), (3, 3, 128, 128, 70, 64),
                                                  (2, 1, 200, 256, 17, 0), (40, 1, 8, 8, 1, 2), (7, 1, 24, 40, 130, 100)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_window_attention_with_kept_tokens_log_bias_and_gate(H, G, D, Dv, window, keep, dtype):
    _need()
    g = torch.Generator().manual_seed(5)
    ps = 16
    q_lens, cached = [45, 1, 2, 130, 1], [100, 77, 0, 0, 300]
    cu, seq = _ragged(q_lens, cached)
    T = sum(q_lens)
    pt, kc, vc = _paged(5, max(seq), ps, G * max(D, Dv) + 8, dtype, g)
    slots = [1, 2, 3, 4, 5]
    q = torch.randn(T, H, D, generator=g).to(dtype)
    r1, r2 = torch.rand(H, generator=g) + 0.1, torch.rand(H, generator=g) * 2
    gh, ge = torch.randn(T, H + 3, generator=g).to(dtype), torch.randn(T, H * Dv + 3, generator=g).to(dtype)
    tol = _tol(dtype, (2e-4, 2e-5))
    for gate, scale_out in ((None, 1.0), (gh[:, 1:1 + H], 0.8), (ge[:, 2:2 + H * Dv], 1.0)):
        ref = torch_ref.window_attention(q, kc, vc, G, Dv, pt, _i32(slots, "cpu"), _i32(seq, "cpu"), _i32(q_lens, "cpu"), ps, 0.3, 0.0, window, r1, None, 0, 0,
                                         keep, r2, gate, scale_out)
        gg = None if gate is None else (gh.to(DEV)[:, 1:1 + H] if gate.shape[1] == H else ge.to(DEV)[:, 2:2 + H * Dv])
        buf = torch.zeros(T, H * Dv + 24, dtype=dtype, device=DEV)
        got = ops.window_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), G, Dv, pt.to(DEV), _i32(slots), _i32(seq), _i32(cu), _i32(q_lens), max(q_lens), ps, 0.3,
                                   0.0, window, r1.to(DEV), None, 0, 0, keep, r2.to(DEV), gg, scale_out, buf[:, 8:8 + H * Dv])
        torch.testing.assert_close(got.cpu().float().view(T, H, Dv), ref, **tol)
        assert float(buf[:, :8].abs().max()) == 0.0 and float(buf[:, 8 + H * Dv:].abs().max()) == 0.0
    # decode form: the last token of every request alone
    last = torch.tensor([c - 1 for c in cu[1:]])
    qd = q[last].contiguous()
    ref = torch_ref.window_attention(qd, kc, vc, G, Dv, pt, _i32(slots, "cpu"), _i32(seq, "cpu"), None, ps, 0.3, 0.0, window, r1, None, 0, 0, keep, r2)
    got = ops.window_attention(qd.to(DEV), kc.to(DEV), vc.to(DEV), G, Dv, pt.to(DEV), _i32(slots), _i32(seq), None, None, 1, ps, 0.3, 0.0, window, r1.to(DEV),
                               None, 0, 0, keep, r2.to(DEV))
    torch.testing.assert_close(got.cpu().float(), ref, **tol)


def test_window_and_kept_token_edges_on_the_kernel():
    """a standout value at the window's far edge, at the last kept position and at the first position behind the kept ones: seen or not, to the
    token, in a prompt portion and in a decode step"""
    _need()
    H, G, D, Dv, W, keep, ps = 2, 1, 8, 4, 68, 5, 16
    g = torch.Generator().manual_seed(6)
    for mark, seen_at, hidden_at in ((40, 40 + W - 1, 40 + W), (keep - 1, 400, None), (keep, keep + W - 1, keep + W)):
        pt, kc, vc = _paged(1, 420, ps, 16, torch.float32, g)
        kc, vc = kc * 0.1, vc * 0.1
        s = int(pt[1, mark // ps]) * ps + mark % ps
        kc[s, 0, :D] = 0.0
        kc[s, 0, 0] = 6.0
        vc[s, 0, :Dv] = 50.0
        for qpos in [p for p in (seen_at, hidden_at) if p is not None]:
            q = torch.zeros(1, H, D)
            q[0, :, 0] = 3.0
            for n_q in (1, 5):                                  # decode step / the last query of a five-token portion
                qq = torch.cat([torch.zeros(n_q - 1, H, D), q]).to(DEV)
                out = ops.window_attention(qq, kc.to(DEV), vc.to(DEV), G, Dv, pt.to(DEV), _i32([1]), _i32([qpos + 1]), _i32([0, n_q]) if n_q > 1 else None,
                                           _i32([n_q]) if n_q > 1 else None, n_q, ps, 1.0, 0.0, W, torch.full((H,), 0.1, device=DEV), None, 0, 0, keep,
                                           torch.full((H,), 0.5, device=DEV))
                assert (float(out.view(n_q, H, Dv)[-1, 0, 0]) > 5.0) == (qpos == seen_at), (mark, qpos, n_q)


def test_tensor_core_route_of_gated_attention_against_the_general_kernel():
    """bf16, heads padded to 128 columns: rotary causal attention with value blend and a per-head gate, and window attention with kept tokens,
    the logarithmic bias, projection-wide norms, biases and an element gate, on the tcgen05 kernels and on the general kernel give the same
    output (prompt portions and decode steps)"""
    _need()
    from types import SimpleNamespace

    g = torch.Generator().manual_seed(7)
    W, H, G, D, Dv, ps = 64, 8, 1, 80, 48, 64
    dt = torch.bfloat16
    mix = GatedAttention(W, H, G, D, Dv, 0.1, 1e-5, dt, rotary=(80, scaled_inv_freq(80, 10000.0, None)), gate="head", value_mix=True).to(DEV)
    mix.vmix = 0.3
    win = GatedAttention(W, H, G, D, Dv, 0.1, 1e-5, dt, bias=True, qk_norm=True, window=70, keep_first=3, log_bias=True, gate="element").to(DEV)
    win.r1.data.copy_(torch.rand(H, generator=g) + 0.1)
    win.r2.data.copy_(torch.rand(H, generator=g) * 2)
    for m in (mix, win):
        for p in (m.in_weight, m.o_weight):
            p.data.copy_((torch.randn(p.shape, generator=g) * p.shape[1] ** -0.5).to(dt))
        for p in (m.q_norm, m.k_norm, m.in_bias, m.o_bias):
            if p is not None:
                p.data.copy_((torch.rand(p.shape, generator=g) + 0.5).to(dt))
        assert m.wants_padding(dt)
        m.pad = 128
    for mix, q_lens, cached in ((mix, [130, 70], [0, 64]), (mix, [1, 1], [200, 134]), (win, [130, 70], [0, 64]), (win, [1, 1], [200, 134])):
        cu, seq = _ragged(q_lens, cached)
        T = sum(q_lens)
        pt, kc, vc = _paged(2, 260, ps, G * 128 + (72 if mix is win else 0), dt, g)       # also as the leading columns of wider pool rows
        pos = torch.cat([torch.arange(c, c + q) for c, q in zip(cached, q_lens)]).int()
        req = torch.cat([torch.full((q,), s) for s, q in zip([1, 2], q_lens)])
        loc = (pt[req.long(), (pos // ps).long()] * ps + pos % ps).int()
        dec = max(q_lens) == 1
        outs = []
        for route in (True, False):
            pool = SimpleNamespace(k=lambda i, kc=kc.clone().to(DEV): kc, v=lambda i, vc=vc.clone().to(DEV): vc)
            fb = SimpleNamespace(kv_pool=pool, positions=pos.to(DEV), out_cache_loc=loc.to(DEV), page_table=pt.to(DEV), req_slots=_i32([1, 2]), seq_lens=_i32(seq),
                                 cu_q=None if dec else _i32(cu), q_lens=None if dec else _i32(q_lens), max_q_len=max(q_lens), page_size=ps, num_splits=1,
                                 attn_workspace=None)
            h = (torch.randn(T, W, generator=torch.Generator().manual_seed(8))).to(dt).to(DEV)
            vf = (torch.randn(T, G * Dv, generator=torch.Generator().manual_seed(9))).to(dt).to(DEV)
            GatedAttention.tc_route = route
            try:
                if route:
                    assert ops.tc_attention_ok(torch.empty(T, H, 128, dtype=dt, device=DEV), pool.k(0)[:, 0, :G * 128].unflatten(-1, (G, 128)),
                                               pool.v(0)[:, 0, :G * 128].unflatten(-1, (G, 128)), ps)
                outs.append(mix.forward(h, fb, 0, vf).float().cpu())
            finally:
                GatedAttention.tc_route = True
        torch.testing.assert_close(outs[0], outs[1], rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("window,keep", [(100, 4), (300, 130), (64, 0), (1, 2), (500, 1), (129, 128), (-1, 3)])
@pytest.mark.parametrize("G,rep,ps", [(1, 8, 16), (2, 4, 64), (3, 1, 32), (1, 16, 128)])
def test_tensor_core_attention_with_window_kept_tokens_and_log_bias(window, keep, G, rep, ps, monkeypatch):
    """``paged_attention`` on the tcgen05 kernels (classic and persistent prompt kernels, decode kernel with one and several key splits)
    against the fp32 reference: windows that start inside a key tile, kept tokens inside the first tile, filling it and reaching into the
    second, requests shorter than the window, ragged portions beside single tokens"""
    _need()
    from sglang_b200.environ import envs

    g = torch.Generator().manual_seed(11)
    H, D, dt = G * rep, 128, torch.bfloat16
    q_lens, cached = [300, 1, 2, 200, 70], [150, 600, 0, 0, 513]
    cu, seq = _ragged(q_lens, cached)
    T = sum(q_lens)
    pt, kc, vc = _paged(5, max(seq), ps, G * D, dt, g)
    slots = [1, 2, 3, 4, 5]
    q = torch.randn(T, H, D, generator=g).to(dt)
    r1, r2 = torch.rand(H, generator=g) + 0.1, torch.rand(H, generator=g) * 2
    scale = 0.12
    k3, v3 = kc.to(DEV).view(-1, G, D), vc.to(DEV).view(-1, G, D)
    assert ops.tc_attention_ok(q.to(DEV), k3, v3, ps)
    ref = torch_ref.window_attention(q, kc, vc, G, D, pt, _i32(slots, "cpu"), _i32(seq, "cpu"), _i32(q_lens, "cpu"), ps, scale, 0.0, window, r1, None, 0, 0, keep, r2)
    for persist in ("1", "0"):
        monkeypatch.setenv(envs.SGLB_ATTN_PERSIST.name, persist)
        got = ops.paged_attention(q.to(DEV), k3, v3, pt.to(DEV), _i32(slots), _i32(seq), _i32(cu), _i32(q_lens), max(q_lens), ps, scale, causal=True,
                                  window=window, slopes=r1.to(DEV), log_rates=r2.to(DEV), keep_first=keep)
        torch.testing.assert_close(got.cpu().float(), ref, rtol=2e-2, atol=2e-2)
    # without a bias: the kept tokens and the window alone (the instance of the kernels without score rewriting)
    ref0 = torch_ref.window_attention(q, kc, vc, G, D, pt, _i32(slots, "cpu"), _i32(seq, "cpu"), _i32(q_lens, "cpu"), ps, scale, 0.0, window, None, None, 0, 0, keep)
    got0 = ops.paged_attention(q.to(DEV), k3, v3, pt.to(DEV), _i32(slots), _i32(seq), _i32(cu), _i32(q_lens), max(q_lens), ps, scale, causal=True,
                               window=window, keep_first=keep)
    torch.testing.assert_close(got0.cpu().float(), ref0, rtol=2e-2, atol=2e-2)
    # decode: the last token of every request alone
    last = torch.tensor([c - 1 for c in cu[1:]])
    qd = q[last].contiguous()
    refd = torch_ref.window_attention(qd, kc, vc, G, D, pt, _i32(slots, "cpu"), _i32(seq, "cpu"), None, ps, scale, 0.0, window, r1, None, 0, 0, keep, r2)
    for splits in (1, 3):
        gotd = ops.paged_attention(qd.to(DEV), k3, v3, pt.to(DEV), _i32(slots), _i32(seq), None, None, 1, ps, scale, causal=True, window=window,
                                   num_splits=splits, slopes=r1.to(DEV), log_rates=r2.to(DEV), keep_first=keep)
        torch.testing.assert_close(gotd.cpu().float(), refd, rtol=2e-2, atol=2e-2)


def test_window_and_kept_token_edges_on_the_tensor_core_kernels():
    """the standout value of the edge test above, on the tcgen05 kernels: seen or not to the token at the window's far edge, at the last kept
    position and at the first position behind the kept ones, with the mark inside the first key tile, at its end and in the second"""
    _need()
    H, G, D, ps, dt = 2, 1, 128, 16, torch.bfloat16
    g = torch.Generator().manual_seed(12)
    for W, keep in ((68, 5), (200, 128), (150, 131)):
        for mark, seen_at, hidden_at in ((keep + 35, keep + 35 + W - 1, keep + 35 + W), (keep - 1, 700, None), (keep, keep + W - 1, keep + W), (300, 300 + W - 1, 300 + W)):
            pt, kc, vc = _paged(1, 720, ps, D, dt, g)
            kc, vc = kc * 0.1, vc * 0.1
            s = int(pt[1, mark // ps]) * ps + mark % ps
            kc[s, 0] = 0.0
            kc[s, 0, 0] = 6.0
            vc[s, 0] = 50.0
            k3, v3 = kc.to(DEV).view(-1, G, D), vc.to(DEV).view(-1, G, D)
            for qpos in [p for p in (seen_at, hidden_at) if p is not None]:
                q = torch.zeros(1, H, D)
                q[0, :, 0] = 3.0
                for n_q in (1, 5, 140):                         # decode step / the last query of a short and of a two-tile portion
                    if n_q > qpos + 1:
                        continue
                    qq = torch.cat([torch.zeros(n_q - 1, H, D), q]).to(dt).to(DEV)
                    out = ops.paged_attention(qq, k3, v3, pt.to(DEV), _i32([1]), _i32([qpos + 1]), _i32([0, n_q]) if n_q > 1 else None,
                                              _i32([n_q]) if n_q > 1 else None, n_q, ps, 1.0, causal=True, window=W, slopes=torch.full((H,), 0.1, device=DEV),
                                              log_rates=torch.full((H,), 0.5, device=DEV), keep_first=keep)
                    assert (float(out[-1, 0, 0]) > 5.0) == (qpos == seen_at), (W, keep, mark, qpos, n_q)


def test_router_and_ungated_shared_combine():
    _need()
    g = torch.Generator().manual_seed(10)
    for E, K in ((16, 3), (5, 5), (7, 1), (600, 4)):
        z = torch.randn(50, E, generator=g) * 2
        w1, i1 = torch_ref.moe_topk_softmax(z, K, True)
        w2, i2 = moe_ops.topk_softmax(z.to(DEV), K, True)
        o1, o2 = i1.long().sort(-1), i2.cpu().long().sort(-1)
        assert torch.equal(o1.values, o2.values)
        torch.testing.assert_close(w2.cpu().gather(1, o2.indices), w1.gather(1, o1.indices), rtol=1e-5, atol=1e-6)
        want = torch.softmax(z.gather(1, i1.long()), -1)         # the definition: soft-max over the chosen logits only
        torch.testing.assert_close(w1, want, rtol=1e-5, atol=1e-6)
    for dtype in (torch.float32, torch.bfloat16):
        y, h, sh = (torch.randn(9, 40, generator=g).to(dtype) for _ in range(3))
        got = moe_ops.moe_identity_shared_combine(y.clone().to(DEV), h.to(DEV), None, sh.to(DEV), None)
        torch.testing.assert_close(got.cpu().float(), (y.float() + sh.float()).to(dtype).float(), **_tol(dtype))


# ------------------------------------------------------------------ the engine on CUDA against the oracle
def _engine_case(tmp_path, dtype, cfg, seed, tol, spikes=False):
    from test_resatar import Harness, _tokens

    h = Harness(tmp_path, cfg, seed=seed, slots=4, max_tokens=1024, device="cuda", dtype=dtype, page=16)
    V = cfg["vocab"]
    a, b, c = _tokens(150, V, 1), _tokens(41, V, 2), _tokens(3, V, 3)
    ra, rb, rc = h.oracle(a), h.oracle(b), h.oracle(c)
    scale = float(np.abs(ra).mean()) + 1e-6

    def close(x, y):
        if dtype == "float32":
            err = np.abs(x - y).max(-1) / scale
            if spikes:      # tiny drawn widths: single positions where a norm over a handful of numbers amplifies fp32 rounding (the reference ops too)
                assert float(np.quantile(err, 0.95)) < tol and float(err.max()) < 4 * tol, (float(np.quantile(err, 0.95)), float(err.max()))
                return
            assert float(err.max()) < tol, float(err.max())
            return
        # bf16: per position, the root mean square over the vocabulary of the difference against that of the logits (means taken off)
        d, r = x - y, y - y.mean(-1, keepdims=True)
        d = d - d.mean(-1, keepdims=True)
        err = np.sqrt((d ** 2).mean(-1)) / np.sqrt((r ** 2).mean(-1) + 1e-12)
        if spikes:          # tiny widths: a norm over a handful of numbers amplifies bf16 rounding at single positions (the reference ops do the same)
            assert float(np.quantile(err, 0.9)) < tol and float(err.mean()) < tol, (float(np.quantile(err, 0.9)), float(err.mean()))
            return
        assert float(err.max()) < tol and float(err.mean()) < 0.4 * tol, (float(err.max()), float(err.mean()))

    close(h.step([("a", a, range(len(a)))], ["a"]), ra)                                            # whole
    close(h.run_cut("a2", a, [100, 2, 17]), ra)                                                    # portions, then token by token
    out = h.step([("a", a[:90], range(90)), ("b", b[:7], range(7)), ("c", c, range(3))], ["c"])    # unequal batch
    close(out[:90], ra[:90]); close(out[90:97], rb[:7]); close(out[97:], rc)
    out = h.step([("a", a[90:], range(60)), ("b", b[7:8], range(1))], ["a"])
    close(out[:60], ra[90:]); close(out[60:], rb[7:8])
    out = h.step([("b", b[8:], range(len(b) - 8)), ("d", c, range(3))], ["b", "d"])                # "d" reuses a freed slot and pages
    close(out[:len(b) - 8], rb[8:]); close(out[len(b) - 8:], rc)
    if dtype == "float32":          # greedy generation through the engine's own entry point, scheduler and sampler
        prompts = [b[:9], c]
        outs = h.eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 6, "temperature": 0, "ignore_eos": True})
        for pr, o in zip(prompts, outs):
            seq = list(pr)
            for _ in range(6):
                seq.append(int(h.oracle(seq)[-1].argmax()))
            assert o["output_ids"] == seq[len(pr):]
    h.close()


def _wide(every):
    from test_resatar import L, SCALING, _attn, _cfg, _dense, _m1, _moe, _par

    moe = lambda: _moe(experts=4, top=4 if every else 2, ff=64, shared=128)
    return _cfg([L(_attn(heads=4, kv_heads=1, dim=64, vdim=32, rot_dims=32, base=10000.0, scaling=SCALING, scale=0.125), _dense(256)),
                 L(_par(heads=4, kv_heads=2, dim=32, vdim=64, window=40, keep=3, scale=0.17, rh=2, rd=64, rv=32, decay=(0.7, 0.995)), moe()),
                 L(_m1(inner=256, state=16, dt_rank=8, conv=4), moe()),
                 L(_attn(heads=8, kv_heads=1, dim=128, vdim=32, rot_dims=128, base=10000.0, scaling=None, scale=0.09), None)], width=128, vocab=192)


def test_engine_on_cuda_fp32(tmp_path):
    _need()
    from test_resatar import MIXED

    _engine_case(tmp_path, "float32", MIXED, 21, 2e-4)


def test_engine_on_cuda_bf16(tmp_path):
    _need()
    from test_resatar import EVERY_EXPERT

    _engine_case(tmp_path, "bfloat16", EVERY_EXPERT, 22, 0.1, spikes=True)


def test_engine_on_cuda_lane_friendly_sizes_fp32(tmp_path):
    """sizes the vectorised and tensor-core routes accept, so that those routes are the ones checked"""
    _need()
    _engine_case(tmp_path, "float32", _wide(False), 23, 2e-4)


def test_engine_on_cuda_lane_friendly_sizes_bf16(tmp_path):
    """bf16 with heads up to 128 wide and one key head: the rotary layers run the tcgen05 attention kernels on padded heads"""
    _need()
    _engine_case(tmp_path, "bfloat16", _wide(True), 24, 6e-2)


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
def test_engine_on_cuda_randomly_drawn_stacks_fp32(tmp_path, seed):
    _need()
    from test_resatar import drawn_config

    _engine_case(tmp_path, "float32", drawn_config(seed, friendly=seed % 2 == 0), 60 + seed, 5e-4, spikes=True)


@pytest.mark.parametrize("seed", [21, 22])
def test_engine_on_cuda_randomly_drawn_stacks_bf16(tmp_path, seed):
    _need()
    from test_resatar import drawn_config

    # small random stacks are badly conditioned in bf16 (RMS norms over a handful of numbers amplify the rounding of their inputs), so this
    # run only has to stay near the oracle; the sharp comparisons are the fp32 ones
    _engine_case(tmp_path, "bfloat16", drawn_config(seed, every_expert=True, friendly=True), 70 + seed, 0.3)
