"""Resatar through the serving engine (CPU tier, fp32) against the plain oracle in ``resatar_oracle.py``: every mechanism alone, prefill against
token-by-token decoding, prompt portions down to two tokens, unequal batches, page and slot reuse, window / kept-token / page edges, far keys
and far memory, the first tokens, long decoding, sizes that differ from layer to layer, and greedy generation through ``Engine.generate``."""
import json
import math
import os

import numpy as np
import pytest
import torch

import resatar_oracle as O
import sglang_b200 as sgl
from sglang_b200.layers.gated_attention import scaled_inv_freq
from sglang_b200.layers.moe import select_experts
from sglang_b200.ops import torch_ref

PAGE = 8
SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}


def _attn(heads=4, kv_heads=2, dim=8, vdim=6, rot_dims=4, base=100.0, scaling=SCALING, scale=0.5, v_mix=True):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, v_mix=v_mix)
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base, "scaling": scaling}
    return {"type": "attention", "mixer": m}


def _par(heads=4, kv_heads=2, dim=6, vdim=5, window=7, keep=2, scale=0.7, rh=3, rd=5, rv=4, decay=(0.5, 0.9, 0.99), ls=0.7, rs=1.3):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, mask={"size": window, "keep_first": keep})
    right = dict(heads=rh, dim=rd, vdim=rv, decay=list(decay))
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}}


def _m1(inner=12, state=5, dt_rank=3, conv=3):
    return {"type": "mamba1", "mixer": dict(inner=inner, state=state, dt_rank=dt_rank, conv=conv)}


def _moe(experts=5, top=2, ff=10, shared=14):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _dense(ff=20):
    return {"kind": "dense", "ff": ff}


def _cfg(layers, width=24, vocab=50, eps=1e-5):
    return {"architecture": "Resatar", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def L(mix, mlp):
    return dict(mix, mlp=mlp)


# sizes differ from layer to layer; three value-mixing layers (the first only lends its values) and one attention layer that does not mix
MIXED = _cfg([L(_attn(), _dense()), L(_par(), _moe()), L(_m1(), _moe(experts=3, top=1, shared=0)),
              L(_attn(heads=2, kv_heads=2, dim=10, vdim=6, rot_dims=10, scaling=None, scale=0.3), None),
              L(_par(heads=3, kv_heads=3, dim=4, vdim=8, window=19, keep=0, rh=1, rd=7, rv=7, decay=(0.8,), ls=1.0, rs=1.0), _dense(9)),
              L(_m1(inner=8, state=9, dt_rank=2, conv=4), None),
              L(_attn(heads=6, kv_heads=2, dim=4, vdim=6, rot_dims=2, v_mix=True), _moe(experts=4, top=3, ff=6, shared=5)),
              L(_attn(heads=2, kv_heads=1, dim=8, vdim=8, rot_dims=0, v_mix=False), None)])
# every expert is chosen: nothing depends on which side of a near-tie a rounded router input falls (bf16 runs)
EVERY_EXPERT = _cfg([L(_m1(), _moe(experts=3, top=3)), L(_par(window=5, keep=3), _moe(experts=2, top=2, shared=0)),
                     L(_attn(heads=2, kv_heads=2, dim=8, vdim=4, rot_dims=8), _dense())])


def drawn_config(seed, every_expert=False, friendly=False):
    """a randomly drawn stack: order of layers, head counts and sizes, state sizes, taps, windows from 1 to beyond the prompt, kept tokens,
    decays, rotary widths and scalings, expert counts, shared experts.  ``friendly``: sizes in multiples of 16 (vector lanes, GEMM tiles)"""
    rng = np.random.default_rng(seed)
    pick = lambda *a: a[int(rng.integers(len(a)))]
    layers = []
    vshape = (pick(1, 2), pick(16, 32) if friendly else pick(3, 6, 9))           # value-mixing layers share their value shape
    for _ in range(int(rng.integers(2, 7))):
        r = rng.random()
        if r < 0.4:
            mixes = rng.random() < 0.7
            g, vd = vshape if mixes else (pick(1, 2, 3), pick(16, 48) if friendly else pick(2, 5, 8))
            dim = pick(16, 32) if friendly else pick(2, 6, 8, 12)
            mix = _attn(heads=g * pick(1, 2, 3, 5), kv_heads=g, dim=dim, vdim=vd, rot_dims=pick(0, 2, dim, dim // 2 * 2),
                        base=pick(10.0, 10000.0), scaling=pick(None, SCALING, {"factor": 2.0, "low": 2.0, "high": 8.0, "original": 32}),
                        scale=pick(0.2, 0.6), v_mix=mixes)
        elif r < 0.7:
            g, rh = pick(1, 2, 3), pick(1, 2, 4)
            mix = _par(heads=g * pick(1, 2, 4), kv_heads=g, dim=pick(16, 32) if friendly else pick(2, 5, 8), vdim=pick(16, 48) if friendly else pick(3, 6, 9),
                       window=pick(1, 2, 5, 16, 33, 200), keep=pick(0, 1, 3, 9), scale=pick(0.3, 0.9), rh=rh,
                       rd=pick(16, 32) if friendly else pick(3, 8, 17), rv=pick(16, 32) if friendly else pick(2, 8, 11),
                       decay=[pick(0.3, 0.9, 0.995, 1.0) for _ in range(rh)], ls=pick(1.0, 0.6), rs=pick(1.0, 1.4))
        else:
            mix = _m1(inner=pick(32, 64) if friendly else pick(6, 12, 20), state=pick(16, 24) if friendly else pick(1, 2, 5, 9, 17, 33),
                      dt_rank=pick(1, 2, 4, 8), conv=pick(1, 2, 3, 4, 5))
        r = rng.random()
        if r < 0.2:
            layers.append(L(mix, None))
        elif r < 0.4:
            layers.append(L(mix, _dense(pick(16, 64) if friendly else pick(5, 12, 30))))
        else:
            E = pick(1, 2, 4, 7)
            layers.append(L(mix, _moe(experts=E, top=E if every_expert else int(rng.integers(1, E + 1)), ff=pick(16, 32) if friendly else pick(3, 8, 11),
                                      shared=pick(0, 16 if friendly else 5, 32 if friendly else 12))))
    return _cfg(layers, width=pick(32, 64) if friendly else pick(10, 24, 36), vocab=pick(64, 128) if friendly else pick(19, 50, 131), eps=pick(1e-5, 1e-6))


class Harness:
    """a model folder with random weights, an engine on it, and the oracle's logits for any token sequence"""

    def __init__(self, tmp, cfg, seed=0, slots=4, max_tokens=512, device="cpu", dtype="float32", page=PAGE):
        from safetensors.torch import save_file

        self.cfg = cfg
        self.W = O.random_weights(cfg, seed)
        d = os.path.join(str(tmp), f"m{seed}")
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump({**cfg, "dtype": dtype}, f)
        if dtype == "bfloat16":          # the oracle sees the rounded weights the engine serves
            self.W = {k: v.to(torch.bfloat16).float() for k, v in self.W.items()}
        save_file({k: v.contiguous() for k, v in self.W.items()}, os.path.join(d, "model.safetensors"))
        self.dir = d
        self.eng = sgl.Engine(model_path=d, device=device, skip_tokenizer_init=True, page_size=page, max_total_tokens=max_tokens,
                              max_running_requests=slots, context_length=max_tokens, disable_radix_cache=True, chunked_prefill_size=-1,
                              max_prefill_tokens=max_tokens, log_level="warning")
        self.sched = self.eng.scheduler
        self._oracle = {}

    @property
    def model(self):
        w = self.sched.worker
        return w.runner.model if hasattr(w, "runner") else w.model

    def oracle(self, tokens):
        k = tuple(tokens)
        if k not in self._oracle:
            self._oracle[k] = O.forward(self.cfg, self.W, list(tokens)).float().numpy()
        return self._oracle[k]

    def step(self, entries, end=()):
        return self.sched.replay_step([(i, list(t), list(w)) for i, t, w in entries], list(end))

    def run_cut(self, rid, tokens, cuts):
        """feed one request in portions of the given sizes (the rest token by token); returns logits of every position"""
        out, at = [], 0
        sizes = list(cuts) + [1] * (len(tokens) - sum(cuts))
        for n in sizes:
            last = at + n == len(tokens)
            out.append(self.step([(rid, tokens[at:at + n], range(n))], [rid] if last else []))
            at += n
        return np.concatenate(out, 0)

    def close(self):
        self.eng.shutdown()


def _tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def _close(a, b, tol=2e-4):
    err = np.abs(a - b).max()
    assert err < tol, err


# ------------------------------------------------------------------ mechanisms alone (functions of the serving path against the oracle's)
def test_router_against_oracle():
    g = torch.Generator().manual_seed(0)
    for E, top in ((5, 2), (3, 1), (4, 4), (1, 1), (16, 3)):
        h, wr, b = torch.randn(40, 16, generator=g), torch.randn(E, 16, generator=g), torch.randn(E, generator=g)
        W = {"r.router": wr.double(), "r.router.b": b.double()}
        w1, i1 = select_experts(torch.nn.functional.linear(h, wr, b), top, True)
        w2, i2 = O.route(h.double(), W, "r.", top)
        o1, o2 = i1.long().sort(-1), i2.sort(-1)
        assert torch.equal(o1.values, o2.values)
        torch.testing.assert_close(w1.gather(1, o1.indices).double(), w2.gather(1, o2.indices), rtol=1e-5, atol=1e-6)
    # the bias takes part in the choice AND in the weights: soft-max over the chosen biased logits only
    z, b = torch.tensor([[1.0, 0.5, -3.0]]), torch.tensor([0.0, 0.0, 5.0])
    w, i = select_experts(z + b, 2, True)
    assert sorted(i[0].tolist()) == [0, 2]
    want = torch.softmax(torch.tensor([2.0, 1.0]), -1)          # logits 2.0 (expert 2) and 1.0 (expert 0)
    got = {int(e): float(x) for e, x in zip(i[0], w[0])}
    assert abs(got[2] - float(want[0])) < 1e-6 and abs(got[0] - float(want[1])) < 1e-6


def test_rotary_frequency_bands():
    """the three bands of the rescaling: short waves kept, long waves divided, the blend between; and no rescaling at all"""
    for dims, base, sc in ((16, 10000.0, SCALING), (8, 50.0, {"factor": 3.0, "low": 2.0, "high": 5.0, "original": 20}), (6, 100.0, None)):
        want = O.rotary_frequencies({"dims": dims, "base": base, "scaling": sc})
        got = scaled_inv_freq(dims, base, sc)
        torch.testing.assert_close(got.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-6, atol=0)
    f = scaled_inv_freq(16, 10000.0, SCALING).double()
    plain = scaled_inv_freq(16, 10000.0, None).double()
    ratio = f / plain
    assert float(ratio[0]) == 1.0 and abs(float(ratio[-1]) - 1 / 8.0) < 1e-6 and any(1 / 8.0 + 1e-3 < float(r) < 1 - 1e-3 for r in ratio)


def test_attention_prepare_reference_op():
    """whole-projection norm, partial rotation and value blend, each against the oracle's functions, and what lands in the cache"""
    g = torch.Generator().manual_seed(1)
    H, G, D, Dv, T, ps = 4, 2, 6, 5, 9, 4
    extra = 7                                                   # gate columns behind v: the op reads a wider projection
    qkv = torch.randn(T, (H + G) * D + G * Dv + extra, generator=g)
    pos = torch.arange(30, 30 + T, dtype=torch.int32)
    loc = torch.randperm(40, generator=g)[:T].int()
    kc, vc = torch.full((40, 1, 14), 9.0), torch.full((40, 1, 14), 9.0)
    qw, kw = torch.randn(H * D, generator=g), torch.randn(G * D, generator=g)
    # (1) norm over the whole projection
    q = torch_ref.attention_prepare(qkv, H, G, D, Dv, pos, kc, vc, loc, qw, kw, 1e-5)
    want = (O.rms(qkv[:, :H * D].double(), 1e-5) * qw.double()).view(T, H, D)
    torch.testing.assert_close(q.double(), want, rtol=1e-5, atol=1e-6)
    wk = O.rms(qkv[:, H * D:(H + G) * D].double(), 1e-5) * kw.double()
    torch.testing.assert_close(kc[loc.long(), 0, :G * D].double(), wk, rtol=1e-5, atol=1e-6)
    assert float(kc[loc.long(), 0, G * D:].min()) == 9.0       # columns beyond this layer's are not touched
    # (2) rotation of the first 4 of 6 coordinates
    fr = scaled_inv_freq(4, 100.0, SCALING)
    q = torch_ref.attention_prepare(qkv, H, G, D, Dv, pos, kc, vc, loc, inv_freq=fr)
    for t in range(T):
        want = O.rotate(qkv[t, :H * D].double().view(H, D), int(pos[t]), [float(x) for x in fr.double()], 4)
        torch.testing.assert_close(q[t].double(), want, rtol=1e-5, atol=1e-5)
        wk = O.rotate(qkv[t, H * D:(H + G) * D].double().view(G, D), int(pos[t]), [float(x) for x in fr.double()], 4)
        torch.testing.assert_close(kc[int(loc[t]), 0, :G * D].double().view(G, D), wk, rtol=1e-5, atol=1e-5)
    assert torch.equal(q[:, :, 4:], qkv[:, :H * D].view(T, H, D)[:, :, 4:])
    # (3) value blend: what is cached is the blend
    vf = torch.randn(T, G * Dv, generator=g)
    torch_ref.attention_prepare(qkv, H, G, D, Dv, pos, kc, vc, loc, v_first=vf, v_lambda=0.3)
    v = qkv[:, (H + G) * D:(H + G) * D + G * Dv]
    torch.testing.assert_close(vc[loc.long(), 0, :G * Dv], 0.7 * v + 0.3 * vf, rtol=1e-6, atol=1e-6)
    # (4) padded layout: same numbers, zeros behind them
    k2, v2 = torch.full((40, 1, G * 16), 9.0), torch.full((40, 1, G * 16), 9.0)
    q2 = torch_ref.attention_prepare(qkv, H, G, D, Dv, pos, k2, v2, loc, qw, kw, 1e-5, fr, vf, 0.3, pad=16)
    q1 = torch_ref.attention_prepare(qkv, H, G, D, Dv, pos, kc, vc, loc, qw, kw, 1e-5, fr, vf, 0.3)
    assert torch.equal(q2[:, :, :D], q1) and float(q2[:, :, D:].abs().max()) == 0.0
    assert torch.equal(k2[loc.long(), 0].view(T, G, 16)[:, :, :D], kc[loc.long(), 0, :G * D].view(T, G, D))
    assert float(v2[loc.long(), 0].view(T, G, 16)[:, :, Dv:].abs().max()) == 0.0


def _paged(g, n_pos, ps, width, n_pages=64):
    kc, vc = torch.randn(n_pages * ps, 1, width, generator=g) * 0.1, torch.randn(n_pages * ps, 1, width, generator=g) * 0.1
    need = (n_pos + ps - 1) // ps
    pages = torch.randperm(n_pages - 1, generator=g)[:need] + 1
    pt = torch.zeros(3, need + 2, dtype=torch.int32)
    pt[1, :need] = pages.int()
    return kc, vc, pt, (lambda pos: int(pages[pos // ps]) * ps + pos % ps)


def test_window_edges_kept_tokens_and_log_bias():
    """one key's value stands out.  As the oldest key inside the window it counts and one step later it is gone, in a prompt portion and in a
    decode step, across a page border; a key among the kept first tokens counts at any distance and the first one behind them does not; the
    logarithmic bias and the gates against sums written out by hand"""
    H, G, D, Dv, W, keep, ps = 2, 1, 6, 3, 11, 3, 4
    g = torch.Generator().manual_seed(2)
    r1, r2 = torch.tensor([0.9, 0.2]), torch.tensor([0.5, 2.0])
    for mark, visible_at, hidden_at in ((19, 19 + W - 1, 19 + W), (keep - 1, 150, None), (keep, keep + W - 1, keep + W)):
        kc, vc, pt, slot_of = _paged(g, 160, ps, 8)
        kc[slot_of(mark), 0, :D] = torch.tensor([5.0, 0, 0, 0, 0, 0])
        vc[slot_of(mark), 0, :Dv] = 50.0
        for qpos in [p for p in (visible_at, hidden_at) if p is not None]:
            q = torch.zeros(1, H, D)
            q[0, :, 0] = 3.0
            L_ = qpos + 1
            args = (kc, vc, G, Dv, pt, torch.tensor([1]), torch.tensor([L_]))
            kw = dict(keep_first=keep, log_rates=r2)
            out = torch_ref.window_attention(q, *args, None, ps, 0.7, 0.0, W, r1, None, **kw)                                      # decode step
            out2 = torch_ref.window_attention(torch.cat([torch.zeros(3, H, D), q]), *args, torch.tensor([4]), ps, 0.7, 0.0, W, r1, None, **kw)[-1:]
            torch.testing.assert_close(out, out2)
            seen = [j for j in range(L_) if qpos - j < W or j < keep]
            K = torch.stack([kc[slot_of(p), 0, :D] for p in seen]).double()
            V = torch.stack([vc[slot_of(p), 0, :Dv] for p in seen]).double()
            dist = torch.tensor([float(qpos - j) for j in seen], dtype=torch.float64)
            for h in range(H):
                s = K @ q[0, h].double() * 0.7 - r1[h].double() * torch.log(1 + r2[h].double() * dist)
                torch.testing.assert_close(out[0, h].double(), O.softmax_rows(s, V), rtol=1e-5, atol=1e-6)
            assert (out[0, 1, 0].item() > 1.0) == (qpos == visible_at), (mark, qpos)
    # gates: one number per head, one per element; and the constant
    q = torch.randn(5, H, D, generator=g)
    args = (kc, vc, G, Dv, pt, torch.tensor([1]), torch.tensor([40]), torch.tensor([5]), ps, 0.7, 0.0, W, r1, None)
    base = torch_ref.window_attention(q, *args, keep_first=keep, log_rates=r2)
    gh, ge = torch.randn(5, H, generator=g), torch.randn(5, H * Dv, generator=g)
    torch.testing.assert_close(torch_ref.window_attention(q, *args, keep_first=keep, log_rates=r2, gate=gh, out_scale=0.8),
                               base * torch.sigmoid(gh)[:, :, None] * 0.8)
    torch.testing.assert_close(torch_ref.window_attention(q, *args, keep_first=keep, log_rates=r2, gate=ge), base * torch.sigmoid(ge).view(5, H, Dv))


def test_far_key_with_full_attention():
    """no window: a key 300 positions back wins when its score stands out"""
    H, G, D, Dv, ps, n = 2, 1, 4, 2, 8, 330
    g = torch.Generator().manual_seed(3)
    kc, vc, pt, slot_of = _paged(g, n, ps, 4)
    kc[slot_of(9), 0, :D] = torch.tensor([9.0, 0, 0, 0])
    vc[slot_of(9), 0, :Dv] = 10.0
    q = torch.zeros(1, H, D)
    q[0, 0, 0], q[0, 1, 0] = 2.0, -2.0
    out = torch_ref.window_attention(q, kc, vc, G, Dv, pt, torch.tensor([1]), torch.tensor([n]), None, ps, 1.0, 0.0, -1, None, None)
    assert out[0, 0, 0].item() > 9.0 and abs(out[0, 1, 0].item()) < 0.5


def test_decay_linear_attention_reference_op_and_far_memory():
    """the constant-decay mode of the scan op in two portions against sums written out by hand; then a write at t = 3 read back 400 tokens later"""
    g = torch.Generator().manual_seed(4)
    H, D, Dv, T = 3, 5, 4, 40
    u = torch.randn(T, H * Dv + 2 * H * D, generator=g)        # [v | k | q]
    decay = torch.tensor([0.5, 0.97, 1.0])
    state = torch.randn(3, H, D, Dv, generator=g)              # a used slot: a fresh request must not see it
    outs = []
    for lo, hi in ((0, 13), (13, 40)):
        outs.append(torch_ref.mamba2_scan(u[lo:hi], None, None, None, None, None, state, torch.tensor([2]), torch.tensor([hi]), torch.tensor([hi - lo]),
                                          H, Dv, D, H, decay))
    got = torch.cat(outs).view(T, H, Dv)
    v, k, q = u[:, :H * Dv].double().view(T, H, Dv), u[:, H * Dv:H * Dv + H * D].double().view(T, H, D), u[:, H * Dv + H * D:].double().view(T, H, D)
    S = torch.zeros(H, D, Dv, dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            S[h] = float(decay[h]) * S[h] + torch.outer(k[t, h], v[t, h])
            torch.testing.assert_close(got[t, h].double(), S[h].t() @ q[t, h], rtol=1e-4, atol=1e-5)
    T = 404
    u = torch.randn(T, H * Dv + 2 * H * D, generator=g) * 0.01
    u[3, H * Dv] = 6.0                     # k, head 0, coordinate 0
    u[3, 0:Dv] = torch.tensor([5.0, -4.0, 3.0, 1.0])
    u[-1, H * Dv + H * D] = 7.0            # q, head 0, coordinate 0
    y = torch_ref.mamba2_scan(u, None, None, None, None, None, torch.zeros(1, H, D, Dv), torch.tensor([0]), torch.tensor([T]), torch.tensor([T]), H, Dv, D, H,
                              torch.tensor([0.999, 0.5, 0.5]))
    want = 6.0 * 7.0 * torch.tensor([5.0, -4.0, 3.0, 1.0]) * 0.999 ** (T - 4)
    assert (y[-1, :Dv] - want).abs().max() < 0.02 * want.abs().max()


def test_selective_scan_reference_op_and_far_memory():
    g = torch.Generator().manual_seed(5)
    C, N, T = 7, 4, 30
    u, dt_raw, z = torch.randn(T, C, generator=g), torch.randn(T, C, generator=g), torch.randn(T, C, generator=g)
    Bm, Cm = torch.randn(T, N, generator=g), torch.randn(T, N, generator=g)
    dtb, A_log, D = torch.randn(C, generator=g), torch.randn(C, N, generator=g) * 0.5, torch.randn(C, generator=g)
    state = torch.randn(3, 1, C, N, generator=g)
    outs = []
    for lo, hi in ((0, 2), (2, 19), (19, 30)):
        outs.append(torch_ref.mamba1_scan(u[lo:hi], dt_raw[lo:hi], dtb, A_log, Bm[lo:hi], Cm[lo:hi], D, z[lo:hi], state, torch.tensor([1]), torch.tensor([hi]),
                                          torch.tensor([hi - lo]), torch.float32))
    got = torch.cat(outs).double()
    dt = torch.nn.functional.softplus(dt_raw.double() + dtb.double())
    S = torch.zeros(C, N, dtype=torch.float64)
    for t in range(T):
        for c in range(C):
            for n in range(N):
                S[c, n] = math.exp(-float(dt[t, c]) * math.exp(float(A_log[c, n]))) * S[c, n] + float(dt[t, c]) * float(u[t, c]) * float(Bm[t, n])
            y = float(S[c] @ Cm[t].double()) + float(D[c]) * float(u[t, c])
            zz = float(z[t, c])
            assert abs(float(got[t, c]) - y * zz / (1 + math.exp(-zz))) < 1e-4 * (1 + abs(y))
    # far memory: slow decay, one large write at t = 3 into state 0 of channel 2, read back only at the end
    T = 404
    u, Bm, Cm = torch.randn(T, C, generator=g) * 0.01, torch.randn(T, N, generator=g) * 0.01, torch.zeros(T, N)
    u[3, 2], Bm[3, 0], Cm[-1, 0] = 5.0, 6.0, 7.0
    y = torch_ref.mamba1_scan(u, torch.zeros(T, C), None, torch.full((C, N), -9.0), Bm, Cm, None, None, torch.zeros(1, 1, C, N), torch.tensor([0]),
                              torch.tensor([T]), torch.tensor([T]), torch.float32)
    want = math.log(2.0) * 5.0 * 6.0 * 7.0 * math.exp(-math.exp(-9.0) * math.log(2.0) * (T - 4))
    assert abs(float(y[-1, 2]) - want) < 0.02 * want


def test_scalar_sandwich_norm_reference_op():
    g = torch.Generator().manual_seed(6)
    x, d = torch.randn(5, 12, generator=g), torch.randn(5, 12, generator=g)
    pw, w = torch.tensor([1.3]), torch.tensor([0.7])
    res = x.clone()
    out = torch_ref.postnorm_add_rmsnorm_f32(res, d, pw, w, 1e-5, torch.float32, False)
    want_res = x.double() + O.scalar_norm(d.double(), pw.double(), 1e-5)
    torch.testing.assert_close(res.double(), want_res, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(out.double(), O.scalar_norm(want_res, w.double(), 1e-5), rtol=1e-5, atol=1e-6)


def test_config_reader(tmp_path):
    from sglang_b200.configs.model_config import load_model_config

    d = tmp_path / "cfg"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(MIXED))
    c = load_model_config(str(d))
    assert c.architecture == "Resatar" and c.hidden_size == 24 and c.vocab_size == 50 and c.num_hidden_layers == 8 and c.rms_norm_eps == 1e-5
    assert c.hybrid["layers"][1]["mixer"]["left"]["mask"] == {"size": 7, "keep_first": 2} and c.hybrid["layers"][1]["mixer"]["right"]["decay"][2] == 0.99


# ------------------------------------------------------------------ single mechanisms through the engine
@pytest.mark.parametrize("cfg", [
    _cfg([L(_attn(), None)]), _cfg([L(_attn(heads=6, kv_heads=1, rot_dims=8, scaling=None), _dense())]),
    _cfg([L(_attn(rot_dims=0, v_mix=False), None), L(_attn(heads=2, dim=4), None), L(_attn(heads=2, dim=6, rot_dims=6), _moe())]),
    _cfg([L(_par(), None)]), _cfg([L(_par(window=1, keep=0), _moe(shared=0))]), _cfg([L(_par(heads=3, kv_heads=3, window=4, keep=6, rh=1, decay=(1.0,)), None)]),
    _cfg([L(_m1(), None)]), _cfg([L(_m1(inner=9, state=1, dt_rank=1, conv=1), _dense(7))]), _cfg([L(_m1(inner=6, state=33, dt_rank=5, conv=5), _moe(experts=6, top=1))])])
def test_one_layer_models(tmp_path, cfg):
    h = Harness(tmp_path, cfg)
    toks = _tokens(37, 50, 5)
    ref = h.oracle(toks)
    _close(h.step([("a", toks, range(len(toks)))], ["a"]), ref)                    # whole prompt
    _close(h.run_cut("b", toks, []), ref)                                          # token by token from the first token
    h.close()


# ------------------------------------------------------------------ the mixed model: cuts, batches, reuse
@pytest.fixture(scope="module")
def mixed(tmp_path_factory):
    h = Harness(tmp_path_factory.mktemp("resatar"), MIXED, seed=3, slots=4, max_tokens=40 * PAGE)
    yield h
    h.close()


def test_residual_after_every_layer(mixed):
    toks = _tokens(17, 50, 6)
    want, got = [], []
    O.forward(mixed.cfg, mixed.W, toks, tap=lambda i, x: want.append(x.float()))
    mixed.model.layer_tap = lambda i, x: got.append(x.clone())
    try:
        mixed.step([("t", toks, [])], ["t"])
    finally:
        mixed.model.layer_tap = None
    assert len(got) == len(want) == 8
    for a, b in zip(got, want):
        torch.testing.assert_close(a.cpu(), b, rtol=1e-4, atol=1e-4)


def test_first_tokens_and_prefill_against_decode(mixed):
    toks = _tokens(61, 50, 7)
    ref = mixed.oracle(toks)
    whole = mixed.step([("w", toks, range(len(toks)))], ["w"])
    _close(whole, ref)
    _close(whole[:3], ref[:3], 1e-4)                                               # positions 0, 1, 2: zero history, zero state, kept tokens only
    _close(mixed.run_cut("d", toks, [30]), ref)                                    # 30 at once, then 31 decode steps (windows 7 and 19 pass over them)


@pytest.mark.parametrize("cuts", [[2, 2, 2, 3, 2], [7, 8, 9, 2, 16], [1, 2, 17, 2, 2, 23], [PAGE, PAGE, 2 * PAGE], [PAGE - 1, 2, PAGE + 1, 19]])
def test_portions_of_many_sizes(mixed, cuts):
    toks = _tokens(70, 50, 11)
    _close(mixed.run_cut("c", toks, cuts), mixed.oracle(toks))


def test_unequal_batches_and_reuse_of_pages_and_slots(mixed):
    rng = np.random.default_rng(5)
    lens = [53, 9, 31, 2, 44, 18, 27]
    seqs = [_tokens(n, 50, 100 + i) for i, n in enumerate(lens)]
    at = [0] * len(seqs)
    got = [[] for _ in seqs]
    waiting, live = list(range(len(seqs))), []
    rounds = 0
    while waiting or live:
        while waiting and len(live) < 4:                                           # four slots: later requests take over freed slots and pages
            live.append(waiting.pop(0))
        entries, end = [], []
        for i in live:
            left = len(seqs[i]) - at[i]
            n = int(min(left, rng.choice([1, 1, 2, 3, 5, 11, 16])))
            if at[i] and rng.random() < 0.2:
                continue                                                           # a request may sit a step out
            entries.append((f"r{i}", seqs[i][at[i]:at[i] + n], range(n)))
        if not entries:
            continue
        for rid, t, _ in entries:
            i = int(rid[1:])
            if at[i] + len(t) == len(seqs[i]):
                end.append(rid)
        out = mixed.step(entries, end)
        o = 0
        for rid, t, _ in entries:
            i = int(rid[1:])
            got[i].append(out[o:o + len(t)])
            o += len(t)
            at[i] += len(t)
            if at[i] == len(seqs[i]):
                live.remove(i)
        rounds += 1
    assert rounds > 10
    for i, s in enumerate(seqs):
        _close(np.concatenate(got[i], 0), mixed.oracle(s))
    assert mixed.sched.kv.allocator.available_pages() == mixed.sched.kv.allocator.total_pages        # everything was given back
    assert mixed.sched.kv.slots.available() == 4


def test_long_decoding_past_every_window(mixed):
    toks = _tokens(5 + 90, 50, 13)
    _close(mixed.run_cut("l", toks, [5]), mixed.oracle(toks), 3e-4)


def test_greedy_generation_through_the_engine(mixed):
    prompts = [_tokens(n, 50, 40 + n) for n in (12, 3, 25)]
    outs = mixed.eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 10, "temperature": 0, "ignore_eos": True})
    for p, o in zip(prompts, outs):
        seq = list(p)
        for _ in range(10):
            seq.append(int(mixed.oracle(seq)[-1].argmax()))
        assert o["output_ids"] == seq[len(p):]
    mixed.sched.check_invariants()


def test_other_sizes_whole_portions_and_batch(tmp_path):
    h = Harness(tmp_path, EVERY_EXPERT, seed=9, max_tokens=30 * PAGE)
    a, b = _tokens(58, 50, 1), _tokens(21, 50, 2)
    ra, rb = h.oracle(a), h.oracle(b)
    _close(h.run_cut("a", a, [29, 2, 2]), ra)
    out = h.step([("a", a[:40], range(40)), ("b", b, range(len(b)))], ["b"])
    _close(out[:40], ra[:40]); _close(out[40:], rb)
    _close(h.step([("a", a[40:], range(18))], ["a"]), ra[40:])
    h.close()


def test_text_prompts_on_a_weights_only_folder(tmp_path):
    """a folder with only config.json and model.safetensors serves text through the byte tokenizer (what `cli generate` and the HTTP server do)"""
    h = Harness(tmp_path, _cfg([L(_m1(), _moe()), L(_par(), None), L(_attn(), _dense())], vocab=300), seed=8)
    h.close()
    eng = sgl.Engine(model_path=h.dir, device="cpu", page_size=PAGE, max_total_tokens=256, max_running_requests=2, log_level="warning")
    out = eng.generate("hello there", {"max_new_tokens": 4, "temperature": 0.7, "top_k": 5, "ignore_eos": True})
    assert len(out["output_ids"]) == 4 and isinstance(out["text"], str)
    eng.shutdown()


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_randomly_drawn_stacks(tmp_path, seed):
    cfg = drawn_config(seed)
    h = Harness(tmp_path, cfg, seed=50 + seed, max_tokens=30 * PAGE)
    V = cfg["vocab"]
    a, b = _tokens(45, V, 1), _tokens(14, V, 2)
    ra, rb = h.oracle(a), h.oracle(b)
    _close(h.step([("w", a, range(len(a)))], ["w"]), ra, 3e-4)
    _close(h.run_cut("c", a, [19, 2, 9, 2]), ra, 3e-4)
    out = h.step([("a", a[:30], range(30)), ("b", b, range(len(b)))], ["b"])
    _close(out[:30], ra[:30], 3e-4); _close(out[30:], rb, 3e-4)
    _close(h.step([("a", a[30:], range(15))], ["a"]), ra[30:], 3e-4)
    h.close()
