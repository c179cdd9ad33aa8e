"""Resatar: a decoder whose configuration lists its layers one by one.  Every layer is sandwich-normed,

    x <- x + norm1b(mixer(norm1(x)));   x <- x + norm2b(ff(norm2(x)))        (no second half when the layer has no feed-forward)

where a norm is an RMS norm times ONE stored number, and the mixer is one of

* ``attention``: rotary grouped-query attention (partial rotation, three-band frequency rescaling), causal, with the values of every
  ``v_mix`` layer but the first blended with the first one's, and one sigmoid output gate per head (``layers/gated_attention.py``);
* ``parallel``:  two mixers side by side on the same input, summed with two constants: a position-free sliding-window attention that keeps
  the sequence's first tokens visible, norms q and k over their whole projection, subtracts a logarithmic distance penalty from the scores
  and gates its output element by element (``layers/gated_attention.py``); and linear attention with a constant decay per head, whose
  heads are normed together and gated (``layers/linear_attention.py``);
* ``mamba1``:    selective scan (``layers/mamba1_scan.py``);

and the feed-forward either dense (``W_down gelu_tanh(W_up h)``) or a mixture of SiLU-GLU experts behind a biased router whose weights are
the soft-max over the chosen logits, plus an optional always-on expert (``layers/moe.py``).

How it sits in the engine: the residual stream is fp32 on every path; ``ops.add_rmsnorm_f32(post_weight=...)`` norms a branch's output, adds
it and emits the next pre-norm in the GEMM dtype in one kernel.  Attention layers (both kinds) each own a layer of the paged pool, laid out
as flat rows (``FlatCacheSpec``) as wide as the widest layer needs; linear-attention and selective-scan layers each own an entry of the
``LayeredStatePool`` (matrix state, and convolution history where there is one), indexed by request slot.  The ``parallel`` mixer feeds both
its sides from one projection GEMM and sums them in one output GEMM over the concatenated, pre-scaled heads.  Prompt portions, decode steps
and mixed batches are the same forward: every kernel is ragged over ``cu_q`` / ``seq_lens``.  Prefix caching is off (recurrent state has no
page-aligned snapshot); tensor parallelism is not split for this family.

Checkpoint names: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b`` (one number each), ``l<i>.mix.*`` (``left.*`` / ``right.*`` under a parallel
mixer), ``l<i>.mlp.{up,down}`` or ``l<i>.mlp.e<j>.{gate,up,down}`` + ``l<i>.mlp.{router,router.b}`` + ``l<i>.mlp.shared.{gate,up,down}``,
``final.norm``, ``head``; linear weights are [out, in].
"""
from __future__ import annotations

import zlib
from typing import Iterable, List, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..configs.model_config import ModelConfig
from ..layers.gated_attention import GatedAttention, scaled_inv_freq
from ..layers.linear_attention import DecayLinearAttention
from ..layers.mamba1_scan import Mamba1ScanMixer
from ..layers.moe import FusedMoE, select_experts
from ..layers.window_attention import FlatCacheSpec
from ..mem_cache.memory_pool import LayeredStatePool
from ..model_executor.forward_batch import ForwardBatch
from ..ops import moe_ops
from ..parallel.parallel_state import get_pp_group, get_tp_group
from .llama import _DT
from .zaparax import SiluGLU, _CacheLayer


class ScalarNorm(nn.Module):
    """one gain for all coordinates; the norm itself runs fused with the residual update (``ops.add_rmsnorm_f32``)"""

    def __init__(self, dtype):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(1, dtype=dtype), requires_grad=False)


class GeluMLP(nn.Module):
    def __init__(self, width: int, ff: int, dtype):
        super().__init__()
        self.up = nn.Parameter(torch.zeros(ff, width, dtype=dtype), requires_grad=False)
        self.down = nn.Parameter(torch.zeros(width, ff, dtype=dtype), requires_grad=False)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf not in ("up", "down"):
            return False
        getattr(self, leaf).data.copy_(w)
        return True

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.activation(ops.linear(h, self.up), "gelu_tanh"), self.down)


class BiasedTopKMoE(nn.Module):
    """experts behind a router with a bias: the ``top`` largest logits win, weighted by the soft-max over the winners only; plus an optional
    always-on expert of the same form"""

    def __init__(self, width: int, mlp: dict, dtype, layer_id: int):
        super().__init__()
        r = mlp["router"]
        self.E, self.top = int(r["experts"]), int(r["top"])
        self.router = nn.Parameter(torch.zeros(self.E, width, dtype=dtype), requires_grad=False)
        self.router_bias = nn.Parameter(torch.zeros(self.E, dtype=torch.float32), requires_grad=False)
        self.experts = FusedMoE(self.E, self.top, width, int(mlp["expert"]["ff"]), dtype, True, 1, None, layer_id)
        sh = mlp.get("shared")
        self.shared = SiluGLU(width, int(sh["ff"]), dtype) if sh else None
        self._router32 = None

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "router":
            self.router.data.copy_(w)
            self._router32 = None
            return True
        if leaf == "router.b":
            self.router_bias.data.copy_(w.float())
            return True
        if leaf.startswith("shared.") and self.shared is not None:
            return self.shared.load(leaf[7:], w)
        head, _, proj = leaf.partition(".")
        if head[:1] == "e" and head[1:].isdigit() and int(head[1:]) < self.E and proj in ("gate", "up", "down"):
            ex = self.experts
            ex.weight_loader(ex.w2 if proj == "down" else ex.w13, w, int(head[1:]), {"gate": "w1", "up": "w3", "down": "w2"}[proj])
            return True
        return False

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if self._router32 is None or self._router32.device != h.device:
            self._router32 = self.router.detach().float()
        z = torch.nn.functional.linear(h.float(), self._router32, self.router_bias)          # router in fp32 on the (possibly bf16-rounded) input
        w, ids = select_experts(z, self.top, True)                 # soft-max, top-k, renormalised = soft-max over the chosen logits
        y = self.experts.forward_routed(h, w, ids)
        y = y.resolve() if hasattr(y, "resolve") else y
        if self.shared is None:
            return y
        return moe_ops.moe_identity_shared_combine(y.contiguous(), h, None, self.shared(h), None)


class ParallelMixer(nn.Module):
    """``left_scale * window attention + right_scale * decaying linear attention`` on the same input: one projection GEMM with rows
    [left q | k | v | g | right v | k | q | g], and one output GEMM over the two sides' gated heads side by side (the constants folded into
    the epilogues that produce them, the left output bias times its constant added by the GEMM)"""

    def __init__(self, width: int, m: dict, eps: float, dtype):
        super().__init__()
        a, b = m["left"], m["right"]
        mask = a.get("mask") or {}
        self.left = GatedAttention(width, int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a.get("vdim", a["dim"])), a.get("scale"),
                                   eps, dtype, bias=True, qk_norm=True, window=int(mask.get("size") or -1), keep_first=int(mask.get("keep_first") or 0),
                                   log_bias=True, gate="element", own_projection=False)
        self.right = DecayLinearAttention(width, int(b["heads"]), int(b["dim"]), int(b.get("vdim", b["dim"])), b["decay"], eps, dtype, own_projection=False)
        self.left.out_scale, self.right.out_scale = float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0))
        self.left.o_weight = self.left.o_bias = self.right.o_weight = None          # they live in ``o_weight`` / ``o_bias`` below
        nl, nr = self.left.rows, self.right.rows
        self.in_weight = nn.Parameter(torch.zeros(nl + nr, width, dtype=dtype), requires_grad=False)
        self.in_bias = nn.Parameter(torch.zeros(nl + nr, dtype=dtype), requires_grad=False)
        self.n_ol, self.n_or = self.left.H * self.left.Dv, self.right.n_v
        self.o_weight = nn.Parameter(torch.zeros(width, self.n_ol + self.n_or, dtype=dtype), requires_grad=False)
        self.o_bias = nn.Parameter(torch.zeros(width, dtype=dtype), requires_grad=False)       # left output bias times left_scale

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        side, _, rest = leaf.partition(".")
        if side == "left":
            if rest == "o":
                self.o_weight.data[:, :self.n_ol].copy_(w)
                return True
            if rest == "o.b":
                self.o_bias.data.copy_((w.float() * self.left.out_scale).to(self.o_bias.dtype))
                return True
            return self.left.load_in(rest, w, self.in_weight, self.in_bias, 0) or self.left.load(rest, w)
        if side == "right":
            if rest == "o":
                self.o_weight.data[:, self.n_ol:].copy_(w)
                return True
            return self.right.load_in(rest, w, self.in_weight, None, self.left.rows) or self.right.load(rest, w)
        return False

    def forward(self, h: torch.Tensor, fb: ForwardBatch, cache_idx: int, state_idx: int) -> torch.Tensor:
        proj = ops.linear(h, self.in_weight, self.in_bias)
        cat = torch.empty(h.shape[0], self.n_ol + self.n_or, dtype=h.dtype, device=h.device)
        self.left.attend(proj[:, :self.left.rows], fb, cache_idx, None, cat[:, :self.n_ol])
        self.right.attend(proj[:, self.left.rows:], fb, state_idx, cat[:, self.n_ol:])
        return ops.linear(cat, self.o_weight, self.o_bias)


class ResatarBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, spec: dict, idx: int, dtype):
        super().__init__()
        W, m, eps = cfg.hidden_size, spec["mixer"], cfg.rms_norm_eps
        kind = spec["type"]
        self.kind = kind
        self.norm1, self.norm1b = ScalarNorm(dtype), ScalarNorm(dtype)
        if kind == "attention":
            rot = m.get("rot")
            rotary = (int(rot["dims"]), scaled_inv_freq(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))) if rot else None
            self.mix = GatedAttention(W, int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"])), m.get("scale"),
                                      eps, dtype, rotary=rotary, gate="head", value_mix=bool(m.get("v_mix")))
        elif kind == "parallel":
            self.mix = ParallelMixer(W, m, eps, dtype)
        elif kind == "mamba1":
            self.mix = Mamba1ScanMixer(W, int(m["inner"]), int(m["state"]), int(m["dt_rank"]), int(m.get("conv", 1)), dtype)
        else:
            raise ValueError(f"Resatar: unknown mixer type {kind!r} in layer {idx}")
        mlp = spec.get("mlp")
        self.norm2 = self.norm2b = self.mlp = None
        if mlp:
            self.norm2, self.norm2b = ScalarNorm(dtype), ScalarNorm(dtype)
            if mlp.get("kind") == "dense":
                self.mlp = GeluMLP(W, int(mlp["ff"]), dtype)
            elif mlp.get("kind") == "moe":
                self.mlp = BiasedTopKMoE(W, mlp, dtype, idx)
            else:
                raise ValueError(f"Resatar: unknown feed-forward kind {mlp.get('kind')!r} in layer {idx}")

    def attention(self) -> Optional[GatedAttention]:
        return self.mix if self.kind == "attention" else self.mix.left if self.kind == "parallel" else None


class ResatarForCausalLM(nn.Module):
    supports_cuda_graph = False          # the expert loop of fp32 serving syncs on the host
    disable_radix_cache = True           # recurrent state per request: no page-aligned prefix to share

    def __init__(self, cfg: ModelConfig, quant_name: Optional[str] = None, device="cpu"):
        super().__init__()
        assert get_tp_group().world_size == 1 and get_pp_group().world_size == 1, "Resatar runs on one rank"
        assert cfg.hybrid and cfg.hybrid.get("layers") is not None, "Resatar needs the per-layer list of its configuration"
        self.cfg = cfg
        dtype = _DT[cfg.dtype]
        self.dtype = dtype
        specs = cfg.hybrid["layers"]
        bb = nn.Module()
        bb.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype)
        bb.embed_tokens.weight.requires_grad_(False)
        bb.all_layers = nn.ModuleList([ResatarBlock(cfg, s, i, dtype) for i, s in enumerate(specs)])
        # bf16 layers whose heads fit the tcgen05 kernels lay them out 128 columns wide in the leading columns of the pool's rows (the widest layer's width)
        attn = [b.attention() for b in bb.all_layers if b.attention() is not None]
        for m in attn:
            if m.wants_padding(dtype):
                m.pad = 128
        cache_width = -(-max([m.cache_width for m in attn] or [0]) // 8) * 8          # rows in multiples of 16 bytes (tensor maps over the pool)
        # per block: (index of its layer in the paged pool, index of its entry in the state pool); -1 where it has none
        self.slots_of: List[Tuple[int, int]] = []
        bb.layers, n_rec = [], 0           # ``layers``: what the runner sizes the paged pool from (one entry per attention layer)
        first_mix = None
        for i, blk in enumerate(bb.all_layers):
            a = blk.attention()
            ci = si = -1
            if a is not None:
                ci = len(bb.layers)
                bb.layers.append(_CacheLayer(FlatCacheSpec(a.H, cache_width, ci, a.scale, a.window)))
            if blk.kind in ("parallel", "mamba1"):
                si, n_rec = n_rec, n_rec + 1
            self.slots_of.append((ci, si))
            if blk.kind == "attention" and blk.mix.value_mix:
                if first_mix is None:
                    first_mix = i
                else:
                    f = bb.all_layers[first_mix].mix
                    assert (f.G, f.Dv) == (blk.mix.G, blk.mix.Dv), "value mixing needs equal value shapes in all mixing layers"
        self.first_mix = first_mix
        bb.norm = ScalarNorm(dtype)
        self.model = bb
        self.lm_head = nn.Parameter(torch.zeros(cfg.vocab_size, cfg.hidden_size, dtype=dtype), requires_grad=False)
        self.layer_tap = None            # callable(layer index, fp32 residual [T, width]) after every layer (debugging / tests)
        if dtype == torch.float32:
            torch.backends.cuda.matmul.allow_tf32 = False          # fp32 serving means fp32 products

    # ---- forward: fp32 residual stream; every post-norm + residual add + next pre-norm is one kernel
    def forward(self, fb: ForwardBatch, inputs_embeds=None):
        m, eps, dt = self.model, self.cfg.rms_norm_eps, self.dtype
        if inputs_embeds is None:          # decode gathers the last sampled token of every request slot on the device
            inputs_embeds = ops.embedding(m.embed_tokens.weight, fb.next_token_buf, fb.req_slots) if fb.input_ids is None \
                else ops.embedding(m.embed_tokens.weight, fb.input_ids)
        x = inputs_embeds.float().contiguous()
        y = post = None                   # branch output not yet added to the residual, and the gain of its post-norm
        v_first = None                    # the first value-mixing layer's values of this step's tokens
        for i, blk in enumerate(m.all_layers):
            ci, si = self.slots_of[i]
            h = ops.add_rmsnorm_f32(x, y, blk.norm1.weight, eps, False, dt, post)
            if blk.kind == "attention":
                proj = ops.linear(h, blk.mix.in_weight)
                y = blk.mix.forward_projected(proj, fb, ci, v_first if i != self.first_mix else None)
                if i == self.first_mix:
                    v_first = blk.mix.values_of(proj)
            elif blk.kind == "parallel":
                y = blk.mix(h, fb, ci, si)
            else:
                y = blk.mix(h, fb, si)
            post = blk.norm1b.weight
            if blk.mlp is not None:
                h = ops.add_rmsnorm_f32(x, y, blk.norm2.weight, eps, False, dt, post)
                y, post = blk.mlp(h), blk.norm2b.weight
            if self.layer_tap is not None:
                yf = y.float()
                self.layer_tap(i, x + yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + eps) * post.float())
        return ops.add_rmsnorm_f32(x, y, m.norm.weight, eps, False, dt, post)

    def compute_logits(self, hidden: torch.Tensor, key: str = "logits") -> torch.Tensor:
        return ops.linear(hidden, self.lm_head).float()

    # ---- recurrent state
    def make_mamba_pool(self, slots: int, device) -> Optional[LayeredStatePool]:
        geo = []
        for blk in self.model.all_layers:
            if blk.kind == "parallel":
                geo.append(blk.mix.right.state_geometry())
            elif blk.kind == "mamba1":
                geo.append(blk.mix.state_geometry())
        return LayeredStatePool(slots, geo, self.dtype, device) if geo else None

    # ---- weights
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> List[str]:
        loaded = []
        L = self.model.all_layers
        for name, w in weights:
            ok = False
            if name == "embed":
                self.model.embed_tokens.weight.data.copy_(w)
                ok = True
            elif name == "head":
                self.lm_head.data.copy_(w)
                ok = True
            elif name == "final.norm":
                self.model.norm.weight.data.copy_(w.reshape(1))
                ok = True
            elif name[:1] == "l" and "." in name and name[1:name.index(".")].isdigit():
                i, rest = int(name[1:name.index(".")]), name[name.index(".") + 1:]
                if i < len(L):
                    blk = L[i]
                    if rest in ("norm1", "norm1b", "norm2", "norm2b") and getattr(blk, rest) is not None:
                        getattr(blk, rest).weight.data.copy_(w.reshape(1))
                        ok = True
                    elif rest.startswith("mix."):
                        ok = blk.mix.load(rest[4:], w) or (rest == "mix.vmix" and blk.kind == "attention")      # an unused blend weight may be stored
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
        one = lambda name: rnd(name, 1, s=0.05, off=1.0).reshape(())
        W = cfg.hidden_size
        yield "embed", rnd("embed", cfg.vocab_size, W, s=0.5)
        for i, sp in enumerate(cfg.hybrid["layers"]):
            p, m, kind = f"l{i}.", sp["mixer"], sp["type"]
            for nm in ("norm1", "norm1b"):
                yield p + nm, one(p + nm)
            q = p + "mix."
            if kind == "attention":
                H, G, D = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"])
                Dv = int(m.get("vdim", D))
                for nm, n, s in (("q", H * D, 2.0), ("k", G * D, 2.0), ("v", G * Dv, 1.0), ("g", H, 1.0)):
                    yield q + nm, lin(q + nm, n, W, s)
                yield q + "vmix", rnd(q + "vmix", 1, s=0.05, off=0.3).reshape(())
                yield q + "o", lin(q + "o", W, H * Dv)
            elif kind == "parallel":
                a, b = m["left"], m["right"]
                H, G, D = int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"])
                Dv = int(a.get("vdim", D))
                l = q + "left."
                for nm, n, s in (("q", H * D, 2.0), ("k", G * D, 2.0), ("v", G * Dv, 1.0)):
                    yield l + nm, lin(l + nm, n, W, s)
                    yield l + nm + ".b", rnd(l + nm + "b", n, s=0.1)
                yield l + "q.norm", rnd(l + "qn", H * D, s=0.1, off=1.0)
                yield l + "k.norm", rnd(l + "kn", G * D, s=0.1, off=1.0)
                yield l + "r1", rnd(l + "r1", H, s=0.1, off=0.5).abs().float()
                yield l + "r2", rnd(l + "r2", H, s=0.1, off=0.5).abs().float()
                yield l + "g", lin(l + "g", H * Dv, W)
                yield l + "o", lin(l + "o", W, H * Dv)
                yield l + "o.b", rnd(l + "ob", W, s=0.1)
                H, D = int(b["heads"]), int(b["dim"])
                Dv = int(b.get("vdim", D))
                r = q + "right."
                for nm, n in (("q", H * D), ("k", H * D), ("v", H * Dv), ("g", H * Dv)):
                    yield r + nm, lin(r + nm, n, W)
                yield r + "norm", rnd(r + "n", H * Dv, s=0.1, off=1.0)
                yield r + "o", lin(r + "o", W, H * Dv)
            else:
                inner, N, R, taps = int(m["inner"]), int(m["state"]), int(m["dt_rank"]), int(m.get("conv", 1))
                yield q + "in", lin(q + "in", 2 * inner, W)
                yield q + "conv", rnd(q + "c", inner, taps, s=0.5)
                yield q + "conv.b", rnd(q + "cb", inner, s=0.1)
                yield q + "x", lin(q + "x", R + 2 * N, inner)
                yield q + "dt", lin(q + "dt", inner, R)
                yield q + "dt.b", rnd(q + "dtb", inner, s=0.5, off=-1.5).float()
                yield q + "A_log", rnd(q + "A", inner, N, s=0.5, off=-0.5).float()
                yield q + "D", rnd(q + "D", inner, s=0.3, off=1.0).float()
                yield q + "o", lin(q + "o", W, inner)
            mlp = sp.get("mlp")
            if not mlp:
                continue
            for nm in ("norm2", "norm2b"):
                yield p + nm, one(p + nm)
            q = p + "mlp."
            if mlp["kind"] == "dense":
                yield q + "up", lin(q + "up", int(mlp["ff"]), W)
                yield q + "down", lin(q + "down", W, int(mlp["ff"]))
                continue
            E, ff = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            for e in range(E):
                for nm, o, n in (("gate", ff, W), ("up", ff, W), ("down", W, ff)):
                    yield q + f"e{e}.{nm}", lin(q + f"e{e}{nm}", o, n)
            yield q + "router", lin(q + "r", E, W, 2.0)
            yield q + "router.b", rnd(q + "rb", E, s=0.1).float()
            if mlp.get("shared"):
                fs = int(mlp["shared"]["ff"])
                for nm, o, n in (("gate", fs, W), ("up", fs, W), ("down", W, fs)):
                    yield q + "shared." + nm, lin(q + "sh" + nm, o, n)
        yield "final.norm", one("fn")
        yield "head", lin("head", cfg.vocab_size, W)
