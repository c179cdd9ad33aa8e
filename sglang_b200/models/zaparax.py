"""Zaparax: a decoder whose configuration lists its layers one by one and may run a stretch of them several times with the same weights.
Every layer is sandwich-normed,

    x <- x + norm1b(mixer(norm1(x)));   x <- x + norm2b(ff(norm2(x)))        (no second half when the layer has no feed-forward)

with the mixer one of

* ``mamba2``:    Mamba-2 state-space mixer with a gated, group-wise RMS-normed read-out (``layers/mamba2_scan.py``);
* ``attention``: grouped-query attention without rotation — unit-RMS q / k, query temperature, capped scores, a per-head distance bias,
  a sliding window and soft-max sinks (``layers/window_attention.py``);

and the feed-forward a mixture of SiLU-GLU experts behind a soft-max router with a choice-only correction, identity experts (the last
router columns: they return their input) and an always-on shared expert scaled by a sigmoid of one number per token
(``layers/moe.py`` ``softmax_bias_route``).  Norms are RMS norms with weights stored around zero (``1 + w``).  The embedding is the token row
times a constant plus a hashed (previous token, token) row.

How it sits in the engine: the residual stream is fp32 on every path; ``ops.add_rmsnorm_f32(post_weight=...)`` norms a branch's output, adds
it and emits the next pre-norm in the GEMM dtype in one kernel.  ``loop = {start, stop, times}`` unrolls into a list of layer *runs*: a run
pairs a block (weights) with its own cache or state index, so attention runs each own a layer of the paged pool and Mamba-2 runs an entry of
the ``LayeredStatePool``; the pool also keeps every request's last token for the bigram row.  Prompt portions, decode steps and mixed
batches are the same forward: every kernel is ragged over ``cu_q`` / ``seq_lens``.  Prefix caching is off (recurrent state has no
page-aligned snapshot); tensor parallelism is not split for this family.

Checkpoint names: ``embed``, ``bigram``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.e<j>.{gate,up,down}``,
``l<i>.mlp.{router,correction}``, ``l<i>.mlp.shared.{gate,up,down,sg}``, ``final.norm``, ``head``; linear weights are [out, in].
"""
from __future__ import annotations

import zlib
from typing import Iterable, List, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..configs.model_config import ModelConfig
from ..layers.mamba2_scan import Mamba2ScanMixer
from ..layers.moe import FusedMoE, softmax_bias_route
from ..layers.window_attention import BiasedWindowAttention, FlatCacheSpec
from ..mem_cache.memory_pool import LayeredStatePool
from ..model_executor.forward_batch import ForwardBatch
from ..ops import moe_ops
from ..parallel.parallel_state import get_pp_group, get_tp_group
from .llama import _DT
from .rirotar import ZeroCentredNorm


def layer_runs(n_layers: int, loop: Optional[dict]) -> List[int]:
    """the order in which the layers run: layers ``start .. stop - 1`` repeat ``times`` times in a row, the rest follow"""
    if not loop:
        return list(range(n_layers))
    a, b, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
    if b <= a:
        return list(range(n_layers))
    assert 0 <= a < b <= n_layers and times >= 1, loop
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n_layers))


def layer_passes(n_layers: int, loop: Optional[dict]) -> List[Tuple[int, bool]]:
    """``layer_runs`` with a mark on every run that opens a pass of the loop after the first (where a design adds something between passes)"""
    order = layer_runs(n_layers, loop)
    if not loop or len(order) == n_layers:
        return [(i, False) for i in order]
    a, b = int(loop.get("start", 0)), int(loop.get("stop", 0))
    return [(i, a <= r < a + (b - a) * int(loop.get("times", 1)) and r > a and (r - a) % (b - a) == 0) for r, i in enumerate(order)]


class SiluGLU(nn.Module):
    def __init__(self, width: int, ff: int, dtype):
        super().__init__()
        self.gate_up = nn.Parameter(torch.zeros(2 * ff, width, dtype=dtype), requires_grad=False)        # rows [gate | up]: one GEMM
        self.down = nn.Parameter(torch.zeros(width, ff, dtype=dtype), requires_grad=False)
        self.ff = ff

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "gate":
            self.gate_up.data[: self.ff].copy_(w)
        elif leaf == "up":
            self.gate_up.data[self.ff:].copy_(w)
        elif leaf == "down":
            self.down.data.copy_(w)
        else:
            return False
        return True

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.silu_and_mul(ops.linear(h, self.gate_up)), self.down)


class IdentitySharedMoE(nn.Module):
    """experts + identity experts behind ``softmax_bias_route``, plus an optional always-on expert behind a sigmoid gate"""

    def __init__(self, width: int, mlp: dict, dtype, layer_id: int):
        super().__init__()
        r = mlp["router"]
        self.E, self.n_id, self.top = int(r["experts"]), int(r.get("identity", 0) or 0), int(r["top"])
        self.router = nn.Parameter(torch.zeros(self.E + self.n_id, width, dtype=dtype), requires_grad=False)
        self.correction = nn.Parameter(torch.zeros(self.E + self.n_id, dtype=torch.float32), requires_grad=False)
        self.experts = FusedMoE(self.E, self.top, width, int(mlp["expert"]["ff"]), dtype, False, 1, None, layer_id)
        sh = mlp.get("shared")
        self.shared = SiluGLU(width, int(sh["ff"]), dtype) if sh else None
        self.shared_gate = nn.Parameter(torch.zeros(1, width, dtype=dtype), requires_grad=False) if sh else None
        self._router32 = None            # [router rows | shared gate row] in fp32: one small fp32 GEMM gives both

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "router":
            self.router.data.copy_(w)
        elif leaf == "correction":
            self.correction.data.copy_(w.float())
        elif leaf == "shared.sg" and self.shared is not None:
            self.shared_gate.data.copy_(w.reshape(1, -1))
        elif leaf.startswith("shared.") and self.shared is not None:
            return self.shared.load(leaf[7:], w)
        else:
            head, _, proj = leaf.partition(".")
            if not (head[:1] == "e" and head[1:].isdigit() and int(head[1:]) < self.E and proj in ("gate", "up", "down")):
                return False
            ex = self.experts
            ex.weight_loader(ex.w2 if proj == "down" else ex.w13, w, int(head[1:]), {"gate": "w1", "up": "w3", "down": "w2"}[proj])
            return True
        self._router32 = None
        return True

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if self._router32 is None or self._router32.device != h.device:
            rows = [self.router.detach().float()] + ([self.shared_gate.detach().float()] if self.shared is not None else [])
            self._router32 = torch.cat(rows, 0).contiguous()
        n = self.E + self.n_id
        z = torch.nn.functional.linear(h.float(), self._router32)              # router (and shared gate) in fp32 on the (possibly bf16-rounded) input
        w, ids, ident = softmax_bias_route(z[:, :n], self.correction, self.top, self.E)
        y = self.experts.forward_routed(h, w, ids)                             # identity picks carry weight 0 and an id no expert owns
        y = y.resolve() if hasattr(y, "resolve") else y
        sh = self.shared(h) if self.shared is not None else None
        return moe_ops.moe_identity_shared_combine(y.contiguous(), h, ident if self.n_id else None, sh, z[:, n] if sh is not None else None)


class ZaparaxBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, spec: dict, idx: int, dtype):
        super().__init__()
        W, m, eps = cfg.hidden_size, spec["mixer"], cfg.rms_norm_eps
        kind = spec["type"]
        self.norm1, self.norm1b = ZeroCentredNorm(W, dtype), ZeroCentredNorm(W, dtype)
        if kind == "attention":
            self.kind = "attention"
            qt = m.get("q_temp") or {}
            self.mix = BiasedWindowAttention(W, int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"])), m.get("scale"),
                                             float(m.get("softcap") or 0.0), int((m.get("mask") or {}).get("size") or -1), eps, dtype,
                                             float(qt.get("coef", 0.0)), int(qt.get("every", 1)))
        elif kind == "mamba2":
            self.kind = "mamba"
            self.mix = Mamba2ScanMixer(W, int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m.get("groups", 1)), int(m.get("conv", 1)),
                                       int(m.get("norm_groups", 1)), eps, dtype)
        else:
            raise ValueError(f"Zaparax: unknown mixer type {kind!r} in layer {idx}")
        mlp = spec.get("mlp")
        self.norm2 = self.norm2b = self.mlp = None
        if mlp:
            if mlp.get("kind", "moe") != "moe":
                raise ValueError(f"Zaparax: unknown feed-forward kind {mlp.get('kind')!r} in layer {idx}")
            self.norm2, self.norm2b = ZeroCentredNorm(W, dtype), ZeroCentredNorm(W, dtype)
            self.mlp = IdentitySharedMoE(W, mlp, dtype, idx)


class _CacheLayer:
    """one attention run as the model runner sees it when it sizes the paged pool"""

    def __init__(self, spec: FlatCacheSpec):
        self.self_attn = type("_Attn", (), {"attn": spec})()


class ZaparaxForCausalLM(nn.Module):
    supports_cuda_graph = False          # the expert loop of fp32 serving syncs on the host
    disable_radix_cache = True           # recurrent state and token history per request: no page-aligned prefix to share

    def __init__(self, cfg: ModelConfig, quant_name: Optional[str] = None, device="cpu"):
        super().__init__()
        assert get_tp_group().world_size == 1 and get_pp_group().world_size == 1, "Zaparax runs on one rank"
        assert cfg.hybrid and cfg.hybrid.get("layers") is not None, "Zaparax needs the per-layer list of its configuration"
        self.cfg = cfg
        dtype = _DT[cfg.dtype]
        self.dtype = dtype
        specs = cfg.hybrid["layers"]
        emb = cfg.hybrid.get("embedding") or {}
        self.embed_scale = float(emb.get("scale", 1.0))
        self.bigram_cfg = emb.get("bigram") or None
        bb = nn.Module()
        bb.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype)
        bb.embed_tokens.weight.requires_grad_(False)
        if self.bigram_cfg:
            bb.bigram = nn.Parameter(torch.zeros(int(self.bigram_cfg["buckets"]) + 1, cfg.hidden_size, dtype=dtype), requires_grad=False)
        bb.all_layers = nn.ModuleList([ZaparaxBlock(cfg, s, i, dtype) for i, s in enumerate(specs)])
        # runs: (block index, index of the run's cache layer or state entry); what is looped gets a fresh index every pass
        self.runs: List[Tuple[int, int]] = []
        # bf16 layers whose heads fit the tcgen05 kernels lay them out 128 columns wide, when that is also the pool's row width (the widest layer's)
        attn = [b.mix for b in bb.all_layers if b.kind == "attention"]
        widest = max([m.G * 128 if m.wants_padding(dtype) else m.cache_width for m in attn] or [0])
        for m in attn:
            if m.wants_padding(dtype) and m.G * 128 == widest:
                m.pad = 128
        cache_width = max([m.cache_width for m in attn] or [0])
        bb.layers, n_rec = [], 0           # ``layers``: what the runner sizes the paged pool from (one entry per attention run)
        for i in layer_runs(len(specs), cfg.hybrid.get("loop")):
            blk = bb.all_layers[i]
            if blk.kind == "attention":
                self.runs.append((i, len(bb.layers)))
                bb.layers.append(_CacheLayer(FlatCacheSpec(blk.mix.H, cache_width, len(bb.layers), blk.mix.scale, blk.mix.window)))
            else:
                self.runs.append((i, n_rec))
                n_rec += 1
        bb.norm = ZeroCentredNorm(cfg.hidden_size, dtype)
        self.model = bb
        self.lm_head = nn.Parameter(torch.zeros(cfg.vocab_size, cfg.hidden_size, dtype=dtype), requires_grad=False)
        self.layer_tap = None            # callable(run index, fp32 residual [T, width]) after every layer run (debugging / tests)
        if dtype == torch.float32:
            torch.backends.cuda.matmul.allow_tf32 = False          # fp32 serving means fp32 products

    # ---- forward: fp32 residual stream; every post-norm + residual add + next pre-norm is one kernel
    def forward(self, fb: ForwardBatch, inputs_embeds=None):
        m, eps, dt = self.model, self.cfg.rms_norm_eps, self.dtype
        if inputs_embeds is None:
            # decode reads every request's input token from the device-side token buffer (where sampling leaves it)
            ids = fb.input_ids if fb.input_ids is not None else fb.next_token_buf[fb.req_slots.long()]
            bg = self.bigram_cfg
            x = ops.bigram_embedding(m.embed_tokens.weight, m.bigram if bg else None, ids, fb.kv_pool.mamba.tokens if bg else None, fb.cu_q,
                                     fb.req_slots, fb.seq_lens, fb.max_q_len, self.embed_scale, int(bg["mul_prev"]) if bg else 0,
                                     int(bg["mul_cur"]) if bg else 0, int(bg["buckets"]) if bg else 0)
        else:
            x = inputs_embeds.float().contiguous()
        y = post = None                   # branch output not yet added to the residual, and the weight of its post-norm
        for run, (i, idx) in enumerate(self.runs):
            blk = m.all_layers[i]
            h = ops.add_rmsnorm_f32(x, y, blk.norm1.weight, eps, True, dt, post)
            y, post = blk.mix(h, fb, idx), blk.norm1b.weight
            if blk.mlp is not None:
                h = ops.add_rmsnorm_f32(x, y, blk.norm2.weight, eps, True, dt, post)
                y, post = blk.mlp(h), blk.norm2b.weight
            if self.layer_tap is not None:
                yf = y.float()
                self.layer_tap(run, x + yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + post.float()))
        return ops.add_rmsnorm_f32(x, y, m.norm.weight, eps, True, dt, post)

    def compute_logits(self, hidden: torch.Tensor, key: str = "logits") -> torch.Tensor:
        return ops.linear(hidden, self.lm_head).float()

    # ---- recurrent state (and the token history of the bigram embedding)
    def make_mamba_pool(self, slots: int, device) -> Optional[LayeredStatePool]:
        geo = [self.model.all_layers[i].mix.state_geometry() for i, _ in self.runs if self.model.all_layers[i].kind == "mamba"]
        if not geo and not self.bigram_cfg:
            return None
        return LayeredStatePool(slots, geo, self.dtype, device, token_history=bool(self.bigram_cfg))

    # ---- weights
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> List[str]:
        loaded = []
        L = self.model.all_layers
        for name, w in weights:
            ok = False
            if name == "embed":
                self.model.embed_tokens.weight.data.copy_(w)
                ok = True
            elif name == "bigram" and self.bigram_cfg:
                self.model.bigram.data.copy_(w)
                ok = True
            elif name == "head":
                self.lm_head.data.copy_(w)
                ok = True
            elif name == "final.norm":
                self.model.norm.weight.data.copy_(w)
                ok = True
            elif name[:1] == "l" and "." in name and name[1:name.index(".")].isdigit():
                i, rest = int(name[1:name.index(".")]), name[name.index(".") + 1:]
                if i < len(L):
                    blk = L[i]
                    if rest in ("norm1", "norm1b", "norm2", "norm2b") and getattr(blk, rest) is not None:
                        getattr(blk, rest).weight.data.copy_(w)
                        ok = True
                    elif rest.startswith("mix."):
                        ok = blk.mix.load(rest[4:], w)
                    elif rest.startswith("mlp.") and blk.mlp is not None:
                        ok = blk.mlp.load(rest[4:], w)
            if ok:
                loaded.append(name)
        return loaded

    @staticmethod
    def dummy_checkpoint(cfg: ModelConfig, device, dtype, seed: int = 0, scale: float = 0.02):
        """random tensors under the checkpoint names (name-seeded), scaled so that activations stay O(1) through many layers"""
        def rnd(name: str, *shape: int, s: float = 1.0, off: float = 0.0) -> torch.Tensor:
            g = torch.Generator(device="cpu").manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFF)
            return (torch.randn(*shape, generator=g) * s + off).to(dtype)

        lin = lambda name, o, i, s=1.0: rnd(name, o, i, s=s * i ** -0.5)
        W = cfg.hidden_size
        yield "embed", rnd("embed", cfg.vocab_size, W, s=0.1)
        bg = (cfg.hybrid.get("embedding") or {}).get("bigram")
        if bg:
            yield "bigram", rnd("bigram", int(bg["buckets"]) + 1, W)
        for i, sp in enumerate(cfg.hybrid["layers"]):
            p, m = f"l{i}.", sp["mixer"]
            for nm in ("norm1", "norm1b"):
                yield p + nm, rnd(p + nm, W, s=0.1)
            if sp["type"] == "attention":
                H, G, D = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"])
                Dv = int(m.get("vdim", D))
                for nm, n, s in (("q", H * D, 2.0), ("k", G * D, 2.0), ("v", G * Dv, 1.0)):
                    yield p + "mix." + nm, lin(p + nm, n, W, s)
                    yield p + f"mix.{nm}.b", rnd(p + nm + "b", n, s=0.1)
                yield p + "mix.sink", rnd(p + "sink", H).float()
                yield p + "mix.o", lin(p + "o", W, H * Dv)
            else:
                H, P, N, G, taps = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m.get("groups", 1)), int(m.get("conv", 1))
                inner, ch = H * P, H * P + 2 * G * N
                yield p + "mix.in", lin(p + "in", 2 * inner + 2 * G * N + H, W)
                yield p + "mix.conv", rnd(p + "c", ch, taps, s=0.5)
                yield p + "mix.conv.b", rnd(p + "cb", ch, s=0.1)
                yield p + "mix.dt_bias", rnd(p + "dt", H, s=0.5, off=-1.0).float()
                yield p + "mix.A_log", rnd(p + "A", H, s=0.5, off=-1.0).float()
                yield p + "mix.D", rnd(p + "D", H, s=0.3, off=1.0).float()
                yield p + "mix.norm", rnd(p + "n", inner, s=0.1, off=1.0)
                yield p + "mix.o", lin(p + "o", W, inner)
            mlp = sp.get("mlp")
            if not mlp:
                continue
            for nm in ("norm2", "norm2b"):
                yield p + nm, rnd(p + nm, W, s=0.1)
            r = mlp["router"]
            E, n_id, ff = int(r["experts"]), int(r.get("identity", 0) or 0), int(mlp["expert"]["ff"])
            for e in range(E):
                q = p + f"mlp.e{e}."
                yield q + "gate", lin(q + "g", ff, W)
                yield q + "up", lin(q + "u", ff, W)
                yield q + "down", lin(q + "d", W, ff)
            yield p + "mlp.router", lin(p + "r", E + n_id, W, 2.0)
            yield p + "mlp.correction", rnd(p + "corr", E + n_id, s=0.02).float()
            if mlp.get("shared"):
                fs, q = int(mlp["shared"]["ff"]), p + "mlp.shared."
                yield q + "gate", lin(q + "g", fs, W)
                yield q + "up", lin(q + "u", fs, W)
                yield q + "down", lin(q + "d", W, fs)
                yield q + "sg", lin(q + "sg", 1, W)
        yield "final.norm", rnd("fn", W, s=0.1)
        yield "head", lin("head", cfg.vocab_size, W)
