"""Plain float64 oracle of the Rumuvik design, written from its equations: one function per mechanism, whole sequences at once where a
mechanism is a sum over earlier positions and token by token where it is a recurrence.  Shares no code with the serving path."""
import math
import zlib

import torch

F64 = torch.float64


# ------------------------------------------------------------------ small pieces
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def centred_norm(x, w, eps):
    """RMS norm whose weight is stored around zero"""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def frequencies(base, dims):
    return [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]


def yarn_frequencies(base, dims, sc):
    """-> (frequencies, factor on sine and cosine)"""
    f = frequencies(base, dims)
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def turn(x, pos, freqs, layout, mult=1.0, back=False):
    """x [T, ..., n]: the first 2 * len(freqs) coordinates of the last axis turned by pos * freqs (``back``: the other way); ``layout``
    "halves" pairs coordinate i with i + len(freqs), "neighbours" pairs 2i with 2i + 1"""
    out = x.clone()
    h = len(freqs)
    for t in range(x.shape[0]):
        for i, f in enumerate(freqs):
            a = float(pos[t]) * f * (-1.0 if back else 1.0)
            c, s = math.cos(a) * mult, math.sin(a) * mult
            ia, ib = (i, i + h) if layout == "halves" else (2 * i, 2 * i + 1)
            u, v = x[t, ..., ia], x[t, ..., ib]
            out[t, ..., ia] = u * c - v * s
            out[t, ..., ib] = v * c + u * s
    return out


# ------------------------------------------------------------------ mixers
def attention(h, W, p, m):
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"])
    Dv = int(m.get("vdim", D))
    pos = list(range(T))
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, Dv)
    rot = m.get("rot") or {}
    base = float(rot.get("base", 10000.0))
    if rot.get("dims"):
        f = frequencies(base, int(rot["dims"]))
        q, k = turn(q, pos, f, "halves"), turn(k, pos, f, "halves")
    fv = frequencies(base, Dv)
    v = turn(v, pos, fv, "halves")                      # a value carries its own position
    cap = float(m.get("softcap") or 0.0)
    o = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, hd]) * float(m["scale"])
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            e = torch.exp(s)
            o[i, hd] = (e / (1.0 + e.sum())) @ v[: i + 1, g]          # one more in the denominator: a sink with score 0 and no value
    o = turn(o, pos, fv, "halves", back=True)               # ... and the sum is turned back by the query's
    return o.reshape(T, H * Dv) @ W[p + "o"].T


def latent_attention(h, W, p, m, eps):
    T = h.shape[0]
    H, D, Dv, R = int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = m.get("rot") or {}
    Dr = int(m.get("rot_dim", rot.get("dims", 0)))
    pos = list(range(T))
    cq = unit_rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(T, H, D + Dr)
    down = h @ W[p + "dkv"].T
    c = unit_rms(down[:, :R], eps) * W[p + "dkv.norm"]
    kr = down[:, R:R + Dr]
    if Dr:
        f, mult = yarn_frequencies(float(rot.get("base", 10000.0)), Dr, rot.get("scaling"))
        qr = turn(q[:, :, D:], pos, f, "neighbours", mult)
        kr = turn(kr, pos, f, "neighbours", mult)
    else:
        qr = q[:, :, D:]
    k0 = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, Dv)
    o = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        for i in range(T):
            s = (k0[: i + 1, hd] @ q[i, hd, :D] + kr[: i + 1] @ qr[i, hd]) * float(m["scale"])
            o[i, hd] = torch.softmax(s, 0) @ v[: i + 1, hd]
    return o.reshape(T, H * Dv) @ W[p + "o"].T


def mlstm(h, W, p, m, eps):
    T = h.shape[0]
    H, D = int(m["heads"]), int(m["dim"])
    Dv = int(m.get("vdim", D))
    cap = float(m.get("gate_cap") or 0.0)
    q = (h @ W[p + "q"].T).view(T, H, D) / math.sqrt(D)
    k = (h @ W[p + "k"].T).view(T, H, D)
    v = (h @ W[p + "v"].T).view(T, H, Dv)
    ri, rf = h @ W[p + "i"].T + W[p + "i.b"], h @ W[p + "f"].T + W[p + "f.b"]
    if cap > 0:
        ri, rf = cap * torch.tanh(ri / cap), cap * torch.tanh(rf / cap)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        S, n, mx = torch.zeros(D, Dv, dtype=F64), torch.zeros(D, dtype=F64), 0.0
        for t in range(T):
            li = float(ri[t, hd])
            lf = -math.log1p(math.exp(-float(rf[t, hd])))                # log sigmoid
            new = max(lf + mx, li)
            a, b = math.exp(lf + mx - new), math.exp(li - new)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = new
            den = max(abs(float(n @ q[t, hd])), math.exp(-mx)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
    o = unit_rms(out, eps).reshape(T, H * Dv) * W[p + "norm"]
    return (o * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def feed_forward(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


# ------------------------------------------------------------------ the model
def run_order(cfg):
    """[(layer, whether a later pass of the loop starts here)]"""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp or int(lp["stop"]) <= int(lp["start"]):
        return [(i, False) for i in range(n)]
    a, b = int(lp["start"]), int(lp["stop"])
    order = [(i, False) for i in range(a)]
    for t in range(int(lp["times"])):
        order += [(i, t > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg, W, tokens, tap=None):
    """logits [T, vocab] (float64) of one sequence; ``tap(run, x)`` sees the residual stream after every layer run"""
    W = {k: v.to(F64) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.tensor(list(tokens))] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    first = x.clone()
    for run, (i, again) in enumerate(run_order(cfg)):
        if again:
            x = x + first
        sp, p = cfg["layers"][i], f"l{i}."
        h = centred_norm(x, W[p + "norm1"], eps)
        if sp["type"] == "attention":
            y = attention(h, W, p + "mix.", sp["mixer"])
        elif sp["type"] == "latent_attention":
            y = latent_attention(h, W, p + "mix.", sp["mixer"], eps)
        elif sp["type"] == "mlstm":
            y = mlstm(h, W, p + "mix.", sp["mixer"], eps)
        else:
            raise ValueError(sp["type"])
        if sp.get("mlp"):
            y = y + feed_forward(centred_norm(x, W[p + "norm2"], eps), W, p + "mlp.")
        x = x + y
        if tap is not None:
            tap(run, x)
    return centred_norm(x, W["final.norm"], eps) @ W["head"].T


def random_weights(cfg, seed):
    """fp32 tensors under the checkpoint's names, drawn so that scores, gates and states are of order one"""
    def rnd(name, *shape, s=1.0, off=0.0):
        g = torch.Generator().manual_seed((seed * 7919 + zlib.crc32(name.encode())) & 0x7FFFFFFF)
        return torch.randn(*shape, generator=g) * s + off

    lin = lambda name, o, i, s=1.0: rnd(name, o, i, s=s / math.sqrt(i))
    Wd = int(cfg["width"])
    W = {"embed": rnd("embed", int(cfg["vocab"]), Wd, s=0.3), "final.norm": rnd("fn", Wd, s=0.2), "head": lin("head", int(cfg["vocab"]), Wd, 2.0)}
    for i, sp in enumerate(cfg["layers"]):
        p, m = f"l{i}.", sp["mixer"]
        W[p + "norm1"] = rnd(p + "n1", Wd, s=0.2)
        q = p + "mix."
        if sp["type"] == "attention":
            H, G, D = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"])
            Dv = int(m.get("vdim", D))
            for nm, n, s in (("q", H * D, 2.5), ("k", G * D, 2.5), ("v", G * Dv, 1.0)):
                W[q + nm] = lin(q + nm, n, Wd, s)
                W[q + nm + ".b"] = rnd(q + nm + "b", n, s=0.3)
            W[q + "o"] = lin(q + "o", Wd, H * Dv)
        elif sp["type"] == "latent_attention":
            H, D, Dv, R, Rq = int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"]), int(m["q_rank"])
            Dr = int(m.get("rot_dim", (m.get("rot") or {}).get("dims", 0)))
            W[q + "dq"], W[q + "dq.norm"] = lin(q + "dq", Rq, Wd), rnd(q + "dqn", Rq, s=0.2, off=1.0)
            W[q + "uq"] = lin(q + "uq", H * (D + Dr), Rq, 2.0)
            W[q + "dkv"], W[q + "dkv.norm"] = lin(q + "dkv", R + Dr, Wd, 1.5), rnd(q + "dkvn", R, s=0.2, off=1.0)
            W[q + "uk"], W[q + "uv"] = lin(q + "uk", H * D, R, 2.0), lin(q + "uv", H * Dv, R)
            W[q + "o"] = lin(q + "o", Wd, H * Dv)
        else:
            H, D = int(m["heads"]), int(m["dim"])
            Dv = int(m.get("vdim", D))
            for nm, n in (("q", H * D), ("k", H * D), ("v", H * Dv), ("g", H * Dv)):
                W[q + nm] = lin(q + nm, n, Wd, 1.5)
            W[q + "i"], W[q + "i.b"] = lin(q + "i", H, Wd, 3.0), rnd(q + "ib", H, s=1.0)
            W[q + "f"], W[q + "f.b"] = lin(q + "f", H, Wd, 3.0), rnd(q + "fb", H, s=1.0, off=2.0)
            W[q + "norm"] = rnd(q + "n", H * Dv, s=0.2, off=1.0)
            W[q + "o"] = lin(q + "o", Wd, H * Dv)
        if sp.get("mlp"):
            ff = int(sp["mlp"]["ff"])
            W[p + "norm2"] = rnd(p + "n2", Wd, s=0.2)
            W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"] = lin(p + "g", ff, Wd, 1.5), lin(p + "u", ff, Wd), lin(p + "d", Wd, ff)
    return W
