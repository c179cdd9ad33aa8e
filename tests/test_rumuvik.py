"""Rumuvik through the serving engine (CPU tier, fp32) against the plain oracle in ``rumuvik_oracle.py``: every mechanism alone, prefill against
token-by-token decoding, prompt portions down to two tokens, unequal batches, page and slot reuse, far keys and keys at page borders, the
sink, rotated values, far memory of the gated matrix memory, the first tokens, long decoding, looped passes, sizes that differ from layer to
layer, and greedy generation through ``Engine.generate``."""
import json
import math
import os

import numpy as np
import pytest
import torch

import rumuvik_oracle as O
import sglang_b200 as sgl
from sglang_b200.layers.gated_attention import scaled_inv_freq
from sglang_b200.layers.latent_attention import yarn_inv_freq
from sglang_b200.models.zaparax import layer_passes
from sglang_b200.ops import torch_ref

PAGE = 8
YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}


def _attn(heads=4, kv_heads=2, dim=8, vdim=6, rot_dims=4, base=100.0, scale=0.5, softcap=5.0):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot={"base": base, "dims": rot_dims})
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def _lat(heads=3, dim=6, rot_dim=4, vdim=5, kv_rank=7, q_rank=9, base=1000.0, scaling=YARN, scale=0.4):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "latent_attention", "mixer": dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale, rot=rot)}


def _ml(heads=2, dim=5, vdim=7, gate_cap=6.0):
    return {"type": "mlstm", "mixer": dict(heads=heads, dim=dim, vdim=vdim, gate_cap=gate_cap)}


def _dense(ff=20):
    return {"kind": "dense", "ff": ff}


def L(mix, mlp):
    return dict(mix, mlp=mlp)


def _cfg(layers, width=24, vocab=50, eps=1e-5, loop=None, scale=3.0):
    c = {"architecture": "Rumuvik", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# sizes differ from layer to layer; the loop covers an attention, a latent and a memory layer, runs three times and does not start at layer 0
MIXED = _cfg([L(_attn(), _dense()), L(_ml(), _dense(9)), L(_lat(), None), L(_attn(heads=3, kv_heads=3, dim=4, vdim=8, rot_dims=4, softcap=0), _dense(11)),
              L(_lat(heads=2, dim=4, rot_dim=6, vdim=4, kv_rank=5, q_rank=3, scaling=None), _dense(6)), L(_ml(heads=3, dim=4, vdim=4, gate_cap=0), None)],
             loop=(1, 4, 3))


def drawn_config(seed, friendly=False):
    """a randomly drawn stack: order of layers, head counts and sizes, ranks, rotary widths, caps, loop position and count.  ``friendly``:
    sizes in multiples of 16 (vector lanes, GEMM tiles)"""
    rng = np.random.default_rng(seed)
    pick = lambda *a: a[int(rng.integers(len(a)))]
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        r = rng.random()
        if r < 0.4:
            g = pick(1, 2, 3)
            dim = pick(16, 32, 64) if friendly else pick(2, 6, 8, 12)
            mix = _attn(heads=g * pick(1, 2, 3, 4), kv_heads=g, dim=dim, vdim=pick(16, 32, 64) if friendly else pick(2, 4, 6, 10),
                        rot_dims=pick(2, dim, max(2, dim // 4 * 2)), base=pick(10.0, 30000.0), scale=pick(0.2, 0.6), softcap=pick(0, 3.0, 30.0))
        elif r < 0.7:
            mix = _lat(heads=pick(1, 2, 5), dim=pick(16, 32) if friendly else pick(3, 8), rot_dim=pick(16, 32) if friendly else pick(2, 4, 10),
                       vdim=pick(16, 48) if friendly else pick(3, 6, 9), kv_rank=pick(32, 64) if friendly else pick(4, 11, 16),
                       q_rank=pick(16, 48) if friendly else pick(2, 9), base=pick(100.0, 2e5),
                       scaling=pick(None, YARN, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5}), scale=pick(0.2, 0.5))
        else:
            mix = _ml(heads=pick(1, 2, 4), dim=pick(16, 32) if friendly else pick(1, 3, 8, 17), vdim=pick(16, 32) if friendly else pick(2, 8, 11),
                      gate_cap=pick(0, 4.0, 15.0))
        layers.append(L(mix, None if rng.random() < 0.25 else _dense(pick(16, 64) if friendly else pick(5, 12, 30))))
    n = len(layers)
    loop = None
    if rng.random() < 0.7:
        a = int(rng.integers(0, n))
        loop = (a, int(rng.integers(a + 1, n + 1)), pick(1, 2, 3))
    return _cfg(layers, width=pick(32, 64) if friendly else pick(10, 24, 36), vocab=pick(64, 128) if friendly else pick(19, 50, 131), eps=pick(1e-5, 1e-6),
                loop=loop, scale=pick(1.0, 2.5, 8.0))


class Harness:
    """a model folder with random weights, an engine on it, and the oracle's logits for any token sequence"""

    def __init__(self, tmp, cfg, seed=0, slots=4, max_tokens=512, device="cpu", dtype="float32", page=PAGE, weights=None):
        from safetensors.torch import save_file

        self.cfg = cfg
        self.W = weights if weights is not None else O.random_weights(cfg, seed)
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


# ------------------------------------------------------------------ mechanisms alone (functions of the serving path against the oracle's or hand-written sums)
def test_rotary_frequencies_and_yarn_blend():
    for dims, base, sc in ((24, 2e5, {"factor": 3.0, "original": 1024, "fast": 24.0, "slow": 2.0}), (8, 100.0, YARN), (6, 50.0, None), (2, 10.0, YARN)):
        want, wm = O.yarn_frequencies(base, dims, sc)
        got, gm = yarn_inv_freq(dims, base, sc)
        torch.testing.assert_close(got.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-6, atol=0)
        assert abs(gm - wm) < 1e-12
    f, mult = yarn_inv_freq(32, 10000.0, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0})
    ratio = f.double() / scaled_inv_freq(32, 10000.0).double()
    assert float(ratio[0]) == 1.0 and abs(float(ratio[-1]) - 1 / 8.0) < 1e-6 and any(0.13 < float(r) < 0.99 for r in ratio)          # fast kept, slow divided, a blend between
    assert abs(mult - (0.1 * math.log(8.0) + 1.0)) < 1e-12


def test_layer_passes_mark_where_a_later_pass_starts():
    assert layer_passes(4, {"start": 1, "stop": 3, "times": 3}) == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert layer_passes(3, {"start": 0, "stop": 1, "times": 3}) == [(0, False), (0, True), (0, True), (1, False), (2, False)]
    assert layer_passes(2, None) == [(0, False), (1, False)] and layer_passes(2, {"start": 0, "stop": 2, "times": 1}) == [(0, False), (1, False)]
    for n, lp in ((5, (1, 3, 3)), (3, (0, 3, 2)), (4, (3, 4, 4))):
        cfg = _cfg([None] * n, loop=lp)
        assert layer_passes(n, cfg["loop"]) == O.run_order(cfg)


def test_two_norm_residual_reference_op():
    g = torch.Generator().manual_seed(0)
    x, a, b, e = (torch.randn(5, 12, generator=g) for _ in range(4))
    w1, w2 = torch.randn(12, generator=g) * 0.2, torch.randn(12, generator=g) * 0.2
    res = x.clone()
    h1, h2 = torch_ref.parallel_add_rmsnorm_f32(res, [a, b, e], w1, w2, 1e-5, True, torch.float32)
    want = x.double() + a.double() + b.double() + e.double()
    torch.testing.assert_close(res.double(), want, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(h1.double(), O.centred_norm(want, w1.double(), 1e-5), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(h2.double(), O.centred_norm(want, w2.double(), 1e-5), rtol=1e-5, atol=1e-6)


def _attend_ref(H, G, D, Dv, rot, qkv, positions, ps, scale, cap, inter=False):
    """attention of ONE request through the serving path's ops (reference tier): preparation with rotated values, scores with cap and unit
    sink over a paged cache, back-rotation"""
    T = qkv.shape[0]
    n_pages = (T + ps - 1) // ps
    pt = torch.zeros(2, n_pages + 1, dtype=torch.int32)
    pt[1, :n_pages] = torch.arange(n_pages, 0, -1, dtype=torch.int32) + 2                  # pages in reverse order: position and row differ
    loc = torch.tensor([int(pt[1, t // ps]) * ps + t % ps for t in range(T)], dtype=torch.int32)
    kc, vc = torch.zeros((n_pages + 4) * ps, 1, G * max(D, Dv)), torch.zeros((n_pages + 4) * ps, 1, G * max(D, Dv))
    fv = scaled_inv_freq(Dv, 100.0)
    q = torch_ref.attention_prepare(qkv, H, G, D, Dv, positions, kc, vc, loc, None, None, 0.0, scaled_inv_freq(rot, 100.0) if rot else None, None, 0.0, 0, fv, inter)
    o = torch_ref.window_attention(q, kc, vc, G, Dv, pt, torch.tensor([1]), torch.tensor([T]), torch.tensor([T]), ps, scale, cap, -1, None, torch.zeros(H))
    return torch_ref.rotate_heads(o, positions, fv, Dv, inter, True, None, None).view(T, H, Dv)


def test_a_far_key_among_hundreds_brings_its_value_turned_by_the_distance():
    """one key far back (and one right at a page border) stands out for the last query: the output is that key's value turned by the
    distance between the two positions, in a prompt; the other keys are noise"""
    H, G, D, Dv, ps = 2, 1, 8, 6, 16
    for T, far in ((300, 3), (300, 15), (300, 16), (129, 127), (64, 0)):
        g = torch.Generator().manual_seed(T + far)
        qkv = torch.randn(T, H * D + G * D + G * Dv, generator=g) * 0.1
        kdir = torch.randn(D, generator=g)
        kdir = kdir / kdir.norm()
        qkv[far, H * D:H * D + D] = 6.0 * kdir                                             # the key
        qkv[T - 1, :D] = 6.0 * kdir                                                        # head 0 of the last query looks for it
        val = torch.randn(Dv, generator=g)
        qkv[far, H * D + D:] = val
        pos = torch.arange(T, dtype=torch.int32)
        o = _attend_ref(H, G, D, Dv, 0, qkv, pos, ps, 1.0, 0.0)
        want = O.turn(val.double()[None, None, :], [T - 1 - far], O.frequencies(100.0, Dv), "halves", back=True)[0, 0]
        torch.testing.assert_close(o[T - 1, 0].double(), want, rtol=2e-3, atol=2e-3)           # exp(36) dwarfs the other keys and the sink
        assert float((o[T - 1, 1].double() - want).abs().max()) > 0.1                         # head 1 did not look for it


def test_the_sink_takes_its_share_and_the_cap_bounds_a_score():
    H, G, D, Dv = 1, 1, 4, 2
    qkv = torch.zeros(1, H * D + G * D + G * Dv)
    qkv[0, :D], qkv[0, D:2 * D], qkv[0, 2 * D:] = torch.tensor([1.0, 0, 0, 0]), torch.tensor([2.0, 0, 0, 0]), torch.tensor([3.0, -1.0])
    pos = torch.zeros(1, dtype=torch.int32)
    for scale, cap in ((1.0, 0.0), (0.25, 0.0), (5.0, 3.0), (-4.0, 0.0)):
        s = 2.0 * scale
        if cap:
            s = cap * math.tanh(s / cap)
        share = math.exp(s) / (1.0 + math.exp(s))                                          # one key, and one more in the denominator
        o = _attend_ref(H, G, D, Dv, 0, qkv, pos, 8, scale, cap)
        torch.testing.assert_close(o[0, 0], torch.tensor([3.0, -1.0]) * share, rtol=1e-5, atol=1e-6)


def test_rotated_values_in_both_layouts_against_the_oracle():
    g = torch.Generator().manual_seed(3)
    H, G, D, Dv, T = 4, 2, 6, 8, 21
    qkv = torch.randn(T, H * D + G * D + G * Dv, generator=g)
    pos = torch.arange(T, dtype=torch.int32)
    for inter, layout in ((False, "halves"), (True, "neighbours")):
        o = _attend_ref(H, G, D, Dv, 4, qkv, pos, 8, 0.4, 2.0, inter)
        q = O.turn(qkv[:, :H * D].double().view(T, H, D), range(T), O.frequencies(100.0, 4), "halves")
        k = O.turn(qkv[:, H * D:H * D + G * D].double().view(T, G, D), range(T), O.frequencies(100.0, 4), "halves")
        v = O.turn(qkv[:, H * D + G * D:].double().view(T, G, Dv), range(T), O.frequencies(100.0, Dv), layout)
        want = torch.zeros(T, H, Dv, dtype=torch.float64)
        for h in range(H):
            for i in range(T):
                s = 2.0 * torch.tanh((k[:i + 1, h // 2] @ q[i, h]) * 0.4 / 2.0)
                e = torch.exp(s)
                want[i, h] = (e / (1.0 + e.sum())) @ v[:i + 1, h // 2]
        want = O.turn(want, range(T), O.frequencies(100.0, Dv), layout, back=True)
        torch.testing.assert_close(o.double(), want, rtol=1e-4, atol=1e-5)


def test_latent_preparation_query_and_score_only_columns():
    g = torch.Generator().manual_seed(4)
    T, Rq, R, Dr, H, D, ps = 19, 5, 6, 4, 2, 3, 8
    x = torch.randn(T, Rq + R + Dr, generator=g)
    wq, wk = torch.randn(Rq, generator=g), torch.randn(R, generator=g)
    f, mult = yarn_inv_freq(Dr, 50.0, YARN)
    pos = torch.arange(T, dtype=torch.int32)
    cache = torch.zeros(5 * ps, 1, R + Dr + 2)
    pt = torch.tensor([[0, 0, 0, 0], [3, 1, 2, 0]], dtype=torch.int32)
    loc = torch.tensor([int(pt[1, t // ps]) * ps + t % ps for t in range(T)], dtype=torch.int32)
    cq = torch_ref.latent_prepare(x, Rq, wq, R, Dr, wk, 1e-5, pos, f, mult, cache, loc)
    torch.testing.assert_close(cq.double(), O.unit_rms(x[:, :Rq].double(), 1e-5) * wq.double(), rtol=1e-5, atol=1e-6)
    rows = cache[loc.long(), 0]
    torch.testing.assert_close(rows[:, :R].double(), O.unit_rms(x[:, Rq:Rq + R].double(), 1e-5) * wk.double(), rtol=1e-5, atol=1e-6)
    fo, mo = O.yarn_frequencies(50.0, Dr, YARN)
    kr = O.turn(x[:, Rq + R:].double(), range(T), fo, "neighbours", mo)
    torch.testing.assert_close(rows[:, R:R + Dr].double(), kr, rtol=1e-4, atol=1e-5)
    assert float(rows[:, R + Dr:].abs().max()) == 0.0
    q = torch.randn(T, H, D + Dr, generator=g)
    q_abs = torch.randn(H, T, R, generator=g)
    ql = torch_ref.latent_query(q, q_abs, D, Dr, pos, f, mult)
    torch.testing.assert_close(ql[:, :, :R], q_abs.transpose(0, 1))
    torch.testing.assert_close(ql[:, :, R:].double(), O.turn(q[:, :, D:].double(), range(T), fo, "neighbours", mo), rtol=1e-4, atol=1e-5)
    # the rotary columns score but are no part of the value
    out = torch_ref.latent_attention(ql, cache, R + Dr, pt, torch.tensor([1]), torch.tensor([T]), torch.tensor([T]), ps, 0.3, -1, None, R)
    assert out.shape == (T, H, R)
    C = rows[:, :R + Dr].double()
    for h in range(H):
        for i in (0, 1, 7, 8, T - 1):
            p = torch.softmax((C[:i + 1] @ ql[i, h].double()) * 0.3, 0)
            torch.testing.assert_close(out[i, h].double(), p @ C[:i + 1, :R], rtol=1e-4, atol=1e-5)


def test_gated_memory_in_portions_and_a_write_read_back_far_later():
    g = torch.Generator().manual_seed(5)
    H, D, Dv, T, cap = 2, 3, 4, 30, 6.0
    proj = torch.randn(T, 2 * H * D + 2 * H * Dv, generator=g)
    raw = torch.randn(T, 2 * H, generator=g) * 4
    nw = torch.randn(H * Dv, generator=g)
    state, ms = torch.randn(3, H, D, Dv + 1, generator=g), torch.randn(3, H, generator=g)          # a used slot: a new request must not see it
    outs = []
    n = 2 * H * D + H * Dv
    for lo, hi in ((0, 2), (2, 19), (19, 30)):
        sl, sq, ql = torch.tensor([1]), torch.tensor([hi]), torch.tensor([hi - lo])
        u, gt = torch_ref.mlstm_prepare(proj[lo:hi], raw[lo:hi], H, D, Dv, cap, ms, sl, sq, ql)
        y = torch_ref.mamba2_scan(u, None, None, None, None, None, state, sl, sq, ql, H, Dv + 1, D, H, None, gt)
        outs.append(torch_ref.mlstm_readout(y, gt, H, Dv, nw, 1e-5, proj[lo:hi, n:], torch.float32))
    got = torch.cat(outs).double()
    # the same thing written out from the recurrence
    q, k = proj[:, :H * D].double().view(T, H, D) / math.sqrt(D), proj[:, H * D:2 * H * D].double().view(T, H, D)
    v, gate = proj[:, 2 * H * D:n].double().view(T, H, Dv), proj[:, n:].double()
    want = torch.zeros(T, H, Dv, dtype=torch.float64)
    for h in range(H):
        S, nn, m = torch.zeros(D, Dv, dtype=torch.float64), torch.zeros(D, dtype=torch.float64), 0.0
        for t in range(T):
            li = cap * math.tanh(float(raw[t, h]) / cap)
            lf = cap * math.tanh(float(raw[t, H + h]) / cap)
            lf = -math.log1p(math.exp(-lf))
            new = max(lf + m, li)
            S = math.exp(lf + m - new) * S + math.exp(li - new) * torch.outer(k[t, h], v[t, h])
            nn = math.exp(lf + m - new) * nn + math.exp(li - new) * k[t, h]
            m = new
            want[t, h] = S.T @ q[t, h] / (max(abs(float(nn @ q[t, h])), math.exp(-m)) + 1e-6)
    want = (O.unit_rms(want, 1e-5).reshape(T, H * Dv) * nw.double()) * torch.sigmoid(gate)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    # far memory: the forget gate stays open, one write at t = 3, the matching query 400 tokens later; every other key is orthogonal
    T = 404
    proj = torch.zeros(T, 2 * D + 2 * Dv)
    proj[:, D + 1] = 1.0                                            # all keys along axis 1 ...
    proj[3, D:2 * D] = torch.tensor([2.0, 0.0, 0.0])                # ... but the one at t = 3, along axis 0
    proj[:, 2 * D:2 * D + Dv] = 0.5
    proj[3, 2 * D:2 * D + Dv] = torch.tensor([1.0, -2.0, 3.0, 0.5])
    proj[-1, :D] = torch.tensor([math.sqrt(D), 0.0, 0.0])           # the last query reads axis 0
    raw = torch.zeros(T, 2)
    raw[:, 1] = 30.0                                                # log forget gate = -1e-13
    state, ms = torch.zeros(1, 1, D, Dv + 1), torch.zeros(1, 1)
    u, gt = torch_ref.mlstm_prepare(proj, raw, 1, D, Dv, 0.0, ms, torch.tensor([0]), torch.tensor([T]), torch.tensor([T]))
    y = torch_ref.mamba2_scan(u, None, None, None, None, None, state, torch.tensor([0]), torch.tensor([T]), torch.tensor([T]), 1, Dv + 1, D, 1, None, gt)
    num, den = y[-1, :Dv], y[-1, Dv]
    torch.testing.assert_close(num / den, torch.tensor([1.0, -2.0, 3.0, 0.5]), rtol=1e-4, atol=1e-4)          # S^T q / (n . q): exactly the written value
    # a large input gate moves the running maximum: the floor exp(-m) shrinks and the state stays of order one
    raw2 = torch.zeros(6, 2)
    raw2[2, 0] = 50.0
    ms2 = torch.zeros(1, 1)
    _, g2 = torch_ref.mlstm_prepare(torch.zeros(6, 2 * D + 2 * Dv), raw2, 1, D, Dv, 0.0, ms2, torch.tensor([0]), torch.tensor([6]), torch.tensor([6]))
    assert float(g2[2, 0, 1]) == 1.0 and float(g2[2, 0, 2]) < 1e-20 and float(g2[:, 0, :2].max()) <= 1.0 and abs(float(ms2) - (50.0 + 3 * math.log(0.5))) < 1e-4


def test_causal_softmax_reference_op():
    g = torch.Generator().manual_seed(9)
    H, tq, n, first = 3, 5, 9, 2
    s = torch.randn(H * tq, n, generator=g) * 3
    p = torch_ref.causal_softmax(s, tq, first, 0.7, torch.float32)
    for r in range(H * tq):
        lim = min(n, first + r % tq + 1)
        e = [math.exp(0.7 * float(s[r, j])) for j in range(lim)]
        for j in range(n):
            want = e[j] / sum(e) if j < lim else 0.0
            assert abs(float(p[r, j]) - want) < 1e-6


def test_config_reader(tmp_path):
    from sglang_b200.configs.model_config import load_model_config

    d = tmp_path / "cfg"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(MIXED))
    c = load_model_config(str(d))
    assert c.architecture == "Rumuvik" and c.hidden_size == 24 and c.vocab_size == 50 and c.num_hidden_layers == 6 and c.rms_norm_eps == 1e-5
    assert c.hybrid["loop"] == {"start": 1, "stop": 4, "times": 3} and c.hybrid["embedding"]["scale"] == 3.0
    assert c.hybrid["layers"][2]["mixer"]["rot"]["scaling"] == YARN


# ------------------------------------------------------------------ single mechanisms through the engine
@pytest.mark.parametrize("cfg", [
    _cfg([L(_attn(), None)]), _cfg([L(_attn(heads=6, kv_heads=1, rot_dims=8, softcap=0), _dense())]), _cfg([L(_attn(heads=1, kv_heads=1, dim=2, vdim=2, rot_dims=2), None)]),
    _cfg([L(_lat(), None)]), _cfg([L(_lat(heads=1, dim=2, rot_dim=2, vdim=3, kv_rank=2, q_rank=1, scaling=None), _dense(7))]),
    _cfg([L(_lat(heads=4, dim=5, rot_dim=8, vdim=5, kv_rank=12, q_rank=12), None)], scale=1.0),
    _cfg([L(_ml(), None)]), _cfg([L(_ml(heads=1, dim=1, vdim=2, gate_cap=0), _dense(7))]), _cfg([L(_ml(heads=3, dim=9, vdim=4, gate_cap=2.0), None)]),
    _cfg([L(_attn(), _dense())], loop=(0, 1, 3)), _cfg([L(_ml(), _dense()), L(_lat(), None)], loop=(0, 2, 2))])
def test_one_and_two_layer_models(tmp_path, cfg):
    h = Harness(tmp_path, cfg)
    toks = _tokens(37, 50, 5)
    ref = h.oracle(toks)
    _close(h.step([("a", toks, range(len(toks)))], ["a"]), ref)                    # whole prompt
    _close(h.run_cut("b", toks, []), ref)                                          # token by token from the first token
    h.close()


def test_expanded_prompt_route_of_latent_attention(tmp_path, monkeypatch):
    """large prompt portions up-project the rows they see and run the general attention kernel; small ones and decode tokens stay absorbed:
    both against the oracle, alone and in one batch, and the route is really taken"""
    from sglang_b200.layers.latent_attention import RotaryLatentAttention

    calls = []
    real = RotaryLatentAttention._forward_expanded
    monkeypatch.setattr(RotaryLatentAttention, "_forward_expanded", lambda self, q, cache, fb: (calls.append(q.shape[0]), real(self, q, cache, fb))[1])
    h = Harness(tmp_path, _cfg([L(_lat(), _dense()), L(_lat(heads=2, dim=4, rot_dim=0, vdim=4, kv_rank=5, q_rank=3, scaling=None), None)]), max_tokens=60 * PAGE)
    a, b = _tokens(150, 50, 1), _tokens(90, 50, 2)
    ra, rb = h.oracle(a), h.oracle(b)
    _close(h.step([("a", a, range(len(a)))], ["a"]), ra)
    assert calls == [150, 150]
    _close(h.run_cut("a2", a, [70, 3, 66]), ra)                                    # expanded, absorbed, expanded over cached rows, then token by token
    assert calls[2:] == [70, 70, 66, 66]
    out = h.step([("a", a[:80], range(80)), ("b", b[:5], range(5))], [])           # a large and a small portion in one batch
    _close(out[:80], ra[:80]); _close(out[80:], rb[:5])
    out = h.step([("a", a[80:81], range(1)), ("b", b[5:], range(85))], ["b"])      # a decode token beside a large portion
    _close(out[:1], ra[80:81]); _close(out[1:], rb[5:])
    n = len(calls)
    _close(h.step([("a", a[81:], range(69))], ["a"]), ra[81:])
    assert len(calls) == n + 2
    monkeypatch.setattr(RotaryLatentAttention, "expand_prefill", False)
    _close(h.step([("c", a, range(len(a)))], ["c"]), ra)
    assert len(calls) == n + 2
    h.close()


# ------------------------------------------------------------------ the mixed model: cuts, batches, reuse
@pytest.fixture(scope="module")
def mixed(tmp_path_factory):
    h = Harness(tmp_path_factory.mktemp("rumuvik"), MIXED, seed=3, slots=4, max_tokens=40 * PAGE)
    yield h
    h.close()


def test_residual_after_every_layer_run(mixed):
    toks = _tokens(17, 50, 6)
    want, got = [], []
    O.forward(mixed.cfg, mixed.W, toks, tap=lambda i, x: want.append(x.float()))
    mixed.model.layer_tap = lambda i, x: got.append(x.clone())
    try:
        mixed.step([("t", toks, [])], ["t"])
    finally:
        mixed.model.layer_tap = None
    assert len(got) == len(want) == 1 + 3 * 3 + 2
    for a, b in zip(got, want):
        torch.testing.assert_close(a.cpu(), b, rtol=1e-4, atol=1e-4)


def test_first_tokens_and_prefill_against_decode(mixed):
    toks = _tokens(61, 50, 7)
    ref = mixed.oracle(toks)
    whole = mixed.step([("w", toks, range(len(toks)))], ["w"])
    _close(whole, ref)
    _close(whole[:3], ref[:3], 1e-4)                                               # positions 0, 1, 2: one key and the sink, zero state, zero maximum
    _close(mixed.run_cut("d", toks, [30]), ref)                                    # 30 at once, then 31 decode steps


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


def test_long_decoding(mixed):
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


def test_text_prompts_on_a_weights_only_folder(tmp_path):
    """a folder with only config.json and model.safetensors serves text through the byte tokenizer (what `cli generate` and the HTTP server do)"""
    h = Harness(tmp_path, _cfg([L(_ml(), _dense()), L(_lat(), None), L(_attn(), _dense())], vocab=300, loop=(1, 3, 2)), seed=8)
    h.close()
    eng = sgl.Engine(model_path=h.dir, device="cpu", page_size=PAGE, max_total_tokens=256, max_running_requests=2, log_level="warning")
    out = eng.generate("hello there", {"max_new_tokens": 4, "temperature": 0.7, "top_k": 5, "ignore_eos": True})
    assert len(out["output_ids"]) == 4 and isinstance(out["text"], str)
    eng.shutdown()


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5])
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
