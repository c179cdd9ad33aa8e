"""A plain, slow restatement of the Resatar decoder, written from its equations with one function per mechanism.  It shares no code with the
serving path: every token is visited one by one, every sum is spelled out, everything is float64 but the rotary angle (see ``rotate``).  The tests compare the engine with it.

Notation: ``h`` the normed input of a sublayer, ``p`` a position (from 0), ``W x`` a stored [out, in] matrix applied to a vector.
"""
import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """one gain for all coordinates"""
    return rms(x, eps) * g.reshape(())


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softmax_rows(scores, values):
    """scores [n], values [n, d] -> sum_j softmax(scores)_j values_j"""
    e = torch.exp(scores - scores.max())
    return (e[:, None] * values).sum(0) / e.sum()


# ---------------------------------------------------------------- rotary positions
def rotary_frequencies(rot):
    """f_i = base^(-2 i / dims), i < dims / 2, with the three-band rescaling by wavelength when ``scaling`` is given"""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f:
            wavelength = 2.0 * math.pi / fi
            if wavelength < orig / high:
                out.append(fi)
            elif wavelength > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wavelength - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return f


def rotate(x, p, freqs, dims):
    """x [heads, dim] at position p: coordinate i pairs with i + dims/2 inside the first ``dims`` coordinates of every head.  The design
    keeps frequencies and angles in 32-bit floats, so the angle is the rounded product of the rounded frequency: at position 1000 that
    rounding moves an angle by up to 3e-5, which a float64 angle would count as an error of the engine"""
    y = x.clone()
    half = dims // 2
    for i in range(half):
        a = float(torch.tensor(float(p), dtype=torch.float32) * torch.tensor(freqs[i], dtype=torch.float32))
        c, s = math.cos(a), math.sin(a)
        u, v = x[:, i], x[:, i + half]
        y[:, i] = u * c - v * s
        y[:, i + half] = v * c + u * s
    return y


# ---------------------------------------------------------------- mixers
def attention(h, m, W, pre, v_first):
    """rotary grouped-query attention with cross-layer value mixing and a per-head output gate.  ``v_first``: the values of the first
    value-mixing layer (None in that layer and in layers that do not mix).  -> (output [T, width], this layer's cached values)"""
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W[pre + "q"].t()).reshape(T, H, D)
    k = (h @ W[pre + "k"].t()).reshape(T, G, D)
    v = (h @ W[pre + "v"].t()).reshape(T, G, Dv)
    rot = m.get("rot")
    if rot:
        fr, dims = rotary_frequencies(rot), int(rot["dims"])
        q = torch.stack([rotate(q[t], t, fr, dims) for t in range(T)])
        k = torch.stack([rotate(k[t], t, fr, dims) for t in range(T)])
    if v_first is not None:
        lam = W[pre + "vmix"].reshape(())
        v = (1.0 - lam) * v + lam * v_first
    gate = torch.sigmoid(h @ W[pre + "g"].t())                     # [T, H]
    scale = float(m["scale"])
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for i in range(T):
        for hd in range(H):
            g = hd // (H // G)
            s = (k[: i + 1, g] @ q[i, hd]) * scale
            out[i, hd] = softmax_rows(s, v[: i + 1, g]) * gate[i, hd]
    return out.reshape(T, H * Dv) @ W[pre + "o"].t(), v


def window_attention(h, m, W, pre, eps):
    """position-free attention: q / k normed over their whole projection, a logarithmic distance penalty, a sliding window that also keeps
    the sequence's first tokens, an element-wise output gate"""
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = h @ W[pre + "q"].t() + W[pre + "q.b"]
    k = h @ W[pre + "k"].t() + W[pre + "k.b"]
    v = (h @ W[pre + "v"].t() + W[pre + "v.b"]).reshape(T, G, Dv)
    q = (rms(q, eps) * W[pre + "q.norm"]).reshape(T, H, D)
    k = (rms(k, eps) * W[pre + "k.norm"]).reshape(T, G, D)
    mask = m.get("mask") or {}
    size, keep = int(mask.get("size") or 0), int(mask.get("keep_first") or 0)
    r1, r2 = W[pre + "r1"], W[pre + "r2"]
    scale = float(m["scale"])
    gate = torch.sigmoid(h @ W[pre + "g"].t())                     # [T, H * Dv]
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for i in range(T):
        seen = [j for j in range(i + 1) if size <= 0 or i - j < size or j < keep]
        dist = torch.tensor([float(i - j) for j in seen], dtype=h.dtype)
        for hd in range(H):
            g = hd // (H // G)
            s = (k[seen, g] @ q[i, hd]) * scale - r1[hd] * torch.log(1.0 + r2[hd] * dist)
            out[i, hd] = softmax_rows(s, v[seen, g])
    return (out.reshape(T, H * Dv) * gate) @ W[pre + "o"].t() + W[pre + "o.b"]


def decay_linear_attention(h, m, W, pre, eps):
    """per head S <- decay S + k v^T, o = S^T q on SiLU-activated projections; the heads' outputs normed together, gated, projected"""
    T = h.shape[0]
    H, D, Dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ W[pre + "q"].t()).reshape(T, H, D)
    k = silu(h @ W[pre + "k"].t()).reshape(T, H, D)
    v = silu(h @ W[pre + "v"].t()).reshape(T, H, Dv)
    decay = [float(d) for d in m["decay"]]
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    o = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            S[hd] = decay[hd] * S[hd] + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].t() @ q[t, hd]
    o = rms(o.reshape(T, H * Dv), eps) * W[pre + "norm"]
    return (o * torch.sigmoid(h @ W[pre + "g"].t())) @ W[pre + "o"].t()


def parallel(h, m, W, pre, eps):
    left = window_attention(h, m["left"], W, pre + "left.", eps)
    right = decay_linear_attention(h, m["right"], W, pre + "right.", eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def mamba1(h, m, W, pre):
    """selective scan: a state of ``state`` numbers per channel, step size, input and read-out vectors all functions of the token"""
    T = h.shape[0]
    inner, N, R, taps = int(m["inner"]), int(m["state"]), int(m["dt_rank"]), int(m["conv"])
    proj = h @ W[pre + "in"].t()
    xin, z = proj[:, :inner], proj[:, inner:]
    cw, cb = W[pre + "conv"], W[pre + "conv.b"]
    x = torch.zeros_like(xin)
    for t in range(T):
        acc = cb.clone()
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                acc = acc + cw[:, j] * xin[src]
        x[t] = silu(acc)
    low = x @ W[pre + "x"].t()
    dt = torch.nn.functional.softplus(low[:, :R] @ W[pre + "dt"].t() + W[pre + "dt.b"], threshold=1e9)      # [T, inner]
    B, C = low[:, R:R + N], low[:, R + N:R + 2 * N]
    A = -torch.exp(W[pre + "A_log"])                               # [inner, N]
    S = torch.zeros(inner, N, dtype=h.dtype)
    y = torch.zeros(T, inner, dtype=h.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + W[pre + "D"] * x[t]
    return (y * silu(z)) @ W[pre + "o"].t()


# ---------------------------------------------------------------- feed-forward
def dense(h, W, pre):
    return gelu_tanh(h @ W[pre + "up"].t()) @ W[pre + "down"].t()


def glu(h, W, pre):
    return (silu(h @ W[pre + "gate"].t()) * (h @ W[pre + "up"].t())) @ W[pre + "down"].t()


def route(h, W, pre, top):
    """-> (weights [T, top], chosen [T, top]): the largest logits, soft-max over the chosen ones only"""
    z = h @ W[pre + "router"].t() + W[pre + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return torch.softmax(val, -1), idx


def moe(h, mlp, W, pre):
    w, idx = route(h, W, pre, int(mlp["router"]["top"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            out[t] = out[t] + w[t, j] * glu(h[t:t + 1], W, pre + f"e{int(idx[t, j])}.")[0]
    if mlp.get("shared"):
        out = out + glu(h, W, pre + "shared.")
    return out


# ---------------------------------------------------------------- the model
def forward(cfg, W, tokens, tap=None, dtype=F64):
    """logits [T, vocab] of one sequence; ``tap(layer, x)`` sees the residual stream after every layer"""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][list(tokens)]
    v_first = None
    for i, sp in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", sp["mixer"], sp["type"]
        h = scalar_norm(x, W[p + "norm1"], eps)
        if kind == "attention":
            mixes = bool(m.get("v_mix"))
            y, v = attention(h, m, W, p + "mix.", v_first if mixes else None)
            if mixes and v_first is None:
                v_first = v
        elif kind == "parallel":
            y = parallel(h, m, W, p + "mix.", eps)
        elif kind == "mamba1":
            y = mamba1(h, m, W, p + "mix.")
        else:
            raise ValueError(kind)
        x = x + scalar_norm(y, W[p + "norm1b"], eps)
        mlp = sp.get("mlp")
        if mlp:
            h = scalar_norm(x, W[p + "norm2"], eps)
            y = dense(h, W, p + "mlp.") if mlp["kind"] == "dense" else moe(h, mlp, W, p + "mlp.")
            x = x + scalar_norm(y, W[p + "norm2b"], eps)
        if tap is not None:
            tap(i, x)
    return scalar_norm(x, W["final.norm"], eps) @ W["head"].t()


def random_weights(cfg, seed=0):
    """random tensors under the checkpoint names, scaled so that every mechanism matters in the logits"""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, sc=1.0, off=0.0: torch.randn(*s, generator=g) * sc + off
    lin = lambda o, i, sc=1.0: rn(o, i, sc=sc * i ** -0.5)
    one = lambda sc=0.2, off=1.0: rn(1, sc=sc, off=off).reshape(())
    Wd, V = int(cfg["width"]), int(cfg["vocab"])
    W = {"embed": rn(V, Wd, sc=0.5), "final.norm": one(), "head": lin(V, Wd)}
    for i, sp in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", sp["mixer"], sp["type"]
        for nm in ("norm1", "norm1b") + (("norm2", "norm2b") if sp.get("mlp") else ()):
            W[p + nm] = one()
        q = p + "mix."
        if kind == "attention":
            H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            W[q + "q"], W[q + "k"], W[q + "v"] = lin(H * D, Wd, 2.0), lin(G * D, Wd, 2.0), lin(G * Dv, Wd)
            W[q + "vmix"] = rn(1, sc=0.1, off=0.4).reshape(())
            W[q + "g"], W[q + "o"] = lin(H, Wd, 2.0), lin(Wd, H * Dv)
        elif kind == "parallel":
            a, b = m["left"], m["right"]
            H, G, D, Dv = int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"])
            l = q + "left."
            W[l + "q"], W[l + "q.b"] = lin(H * D, Wd, 2.0), rn(H * D, sc=0.3)
            W[l + "k"], W[l + "k.b"] = lin(G * D, Wd, 2.0), rn(G * D, sc=0.3)
            W[l + "v"], W[l + "v.b"] = lin(G * Dv, Wd), rn(G * Dv, sc=0.3)
            W[l + "q.norm"], W[l + "k.norm"] = rn(H * D, sc=0.3, off=1.5), rn(G * D, sc=0.3, off=1.5)
            W[l + "r1"], W[l + "r2"] = rn(H, sc=0.2, off=0.8).abs(), rn(H, sc=0.2, off=0.6).abs()
            W[l + "g"], W[l + "o"], W[l + "o.b"] = lin(H * Dv, Wd, 2.0), lin(Wd, H * Dv), rn(Wd, sc=0.2)
            H, D, Dv = int(b["heads"]), int(b["dim"]), int(b["vdim"])
            r = q + "right."
            W[r + "q"], W[r + "k"], W[r + "v"] = lin(H * D, Wd, 2.0), lin(H * D, Wd, 2.0), lin(H * Dv, Wd, 2.0)
            W[r + "g"], W[r + "o"], W[r + "norm"] = lin(H * Dv, Wd, 2.0), lin(Wd, H * Dv), rn(H * Dv, sc=0.2, off=1.0)
        elif kind == "mamba1":
            inner, N, R, taps = int(m["inner"]), int(m["state"]), int(m["dt_rank"]), int(m["conv"])
            W[q + "in"] = lin(2 * inner, Wd, 1.5)
            W[q + "conv"], W[q + "conv.b"] = rn(inner, taps, sc=0.6), rn(inner, sc=0.2)
            W[q + "x"] = lin(R + 2 * N, inner, 1.5)
            W[q + "dt"], W[q + "dt.b"] = lin(inner, R, 1.0), rn(inner, sc=0.7, off=-1.5)
            W[q + "A_log"] = rn(inner, N, sc=0.7, off=-0.5)
            W[q + "D"] = rn(inner, sc=0.5, off=0.5)
            W[q + "o"] = lin(Wd, inner)
        mlp = sp.get("mlp")
        if not mlp:
            continue
        q = p + "mlp."
        if mlp["kind"] == "dense":
            ff = int(mlp["ff"])
            W[q + "up"], W[q + "down"] = lin(ff, Wd, 2.0), lin(Wd, ff, 2.0)
            continue
        E, ff = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
        for e in range(E):
            W[q + f"e{e}.gate"], W[q + f"e{e}.up"], W[q + f"e{e}.down"] = lin(ff, Wd, 2.0), lin(ff, Wd, 2.0), lin(Wd, ff, 2.0)
        W[q + "router"], W[q + "router.b"] = lin(E, Wd, 3.0), rn(E, sc=0.3)
        if mlp.get("shared"):
            fs = int(mlp["shared"]["ff"])
            W[q + "shared.gate"], W[q + "shared.up"], W[q + "shared.down"] = lin(fs, Wd, 2.0), lin(fs, Wd, 2.0), lin(Wd, fs, 2.0)
    return W
