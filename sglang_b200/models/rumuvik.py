"""Rumuvik: a decoder whose configuration lists its layers one by one and may run a stretch of them several times with the same weights.
Every layer is a parallel block with two pre-norms of the SAME input,

    x <- x + (mixer(norm1(x)) + ff(norm2(x)))                  (no ff term when the layer has no feed-forward)

with the mixer one of

* ``attention``:        grouped-query attention with projection biases, partial rotation of q / k (pairs half a rotary width apart), values
  that are rotated by their own position over their whole width and turned back by the query's behind the soft-max, a tanh score cap and a
  soft-max with one more in the denominator (``layers/gated_attention.py`` with ``softcap``, ``sinks``, ``value_rotary``, no gate);
* ``latent_attention``: latent attention with a normed query latent and a decoupled rotary part shared by all heads (neighbouring
  coordinates paired, YaRN-blended frequencies), ordinary soft-max (``layers/latent_attention.py`` ``RotaryLatentAttention``);
* ``mlstm``:            matrix memory with exponential gates and a running maximum (``layers/mlstm.py``);

and the feed-forward ``W_down (gelu_tanh(W_gate h) * W_up h)``.  Norms are RMS norms with weights stored around zero (``1 + w``).  The
embedding is the token row times a constant.  ``loop = {start, stop, times}``: layers ``start .. stop - 1`` run ``times`` times in a row;
before every pass but the first the embedding output is added to the stream again.

How it sits in the engine: the residual stream is fp32 on every path; ``ops.parallel_add_rmsnorm_f32`` adds a block's two branch outputs
(and, at a pass boundary, the embedding output) to it and emits the next block's two pre-norms in the GEMM dtype in one kernel.  The loop
unrolls into a list of layer *runs*; a run pairs a block (weights) with its own cache or state: an attention run owns a layer (key and value
plane) of the paged pool, a latent-attention run ONE plane of a pool layer (two latent runs share a layer), laid out as flat rows as wide
as the widest run needs; an mLSTM run owns an entry of the ``LayeredStatePool`` by request slot.  Prompt portions, decode steps and mixed
batches are the same forward: every kernel is ragged over ``cu_q`` / ``seq_lens``.  Prefix caching is off (recurrent state has no
page-aligned snapshot); tensor parallelism is not split for this family.

Checkpoint names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*`` (``q|k|v`` + ``.b`` and ``o`` / ``dq|dq.norm|uq|dkv|dkv.norm|uk|uv|o`` /
``q|k|v|g|o|norm|i|i.b|f|f.b``), ``l<i>.mlp.{gate,up,down}``, ``final.norm``, ``head``; linear weights are [out, in].
"""
from __future__ import annotations

import zlib
from typing import Iterable, List, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..configs.model_config import ModelConfig
from ..layers.gated_attention import GatedAttention, scaled_inv_freq
from ..layers.latent_attention import RotaryLatentAttention, yarn_inv_freq
from ..layers.mlstm import MLSTMMixer
from ..layers.window_attention import FlatCacheSpec
from ..mem_cache.memory_pool import LayeredStatePool
from ..model_executor.forward_batch import ForwardBatch
from ..parallel.parallel_state import get_pp_group, get_tp_group
from .llama import _DT
from .rirotar import ZeroCentredNorm
from .zaparax import _CacheLayer, layer_passes


class GeluGLU(nn.Module):
    """``W_down (gelu_tanh(W_gate h) * W_up h)``"""

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
        return ops.linear(ops.glu_activation(ops.linear(h, self.gate_up), "gelu_tanh"), self.down)


class RumuvikBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, spec: dict, idx: int, dtype):
        super().__init__()
        W, m, eps = cfg.hidden_size, spec["mixer"], cfg.rms_norm_eps
        kind = spec["type"]
        self.kind = kind
        self.norm1 = ZeroCentredNorm(W, dtype)
        if kind == "attention":
            D, Dv = int(m["dim"]), int(m.get("vdim", m["dim"]))
            rot = m.get("rot") or {}
            base = float(rot.get("base", 10000.0))
            rotary = (int(rot["dims"]), scaled_inv_freq(int(rot["dims"]), base)) if rot.get("dims") else None
            self.mix = GatedAttention(W, int(m["heads"]), int(m.get("kv_heads", m["heads"])), D, Dv, m.get("scale"), eps, dtype, bias=True, rotary=rotary,
                                      gate=None, softcap=float(m.get("softcap") or 0.0), sinks=True, value_rotary=(scaled_inv_freq(Dv, base), False))
            self.mix.o_bias = None                   # biases on q, k and v only
        elif kind == "latent_attention":
            rot = m.get("rot") or {}
            Dr = int(m.get("rot_dim", rot.get("dims", 0)))
            rotary = yarn_inv_freq(Dr, float(rot.get("base", 10000.0)), rot.get("scaling")) if Dr else None
            self.mix = RotaryLatentAttention(W, int(m["heads"]), int(m["dim"]), Dr, int(m["vdim"]), int(m["kv_rank"]), int(m["q_rank"]), m.get("scale"),
                                             eps, dtype, rotary)
        elif kind == "mlstm":
            self.mix = MLSTMMixer(W, int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])), float(m.get("gate_cap") or 0.0), eps, dtype)
        else:
            raise ValueError(f"Rumuvik: unknown mixer type {kind!r} in layer {idx}")
        mlp = spec.get("mlp")
        self.norm2 = self.mlp = None
        if mlp:
            if mlp.get("kind", "dense") != "dense":
                raise ValueError(f"Rumuvik: unknown feed-forward kind {mlp.get('kind')!r} in layer {idx}")
            self.norm2 = ZeroCentredNorm(W, dtype)
            self.mlp = GeluGLU(W, int(mlp["ff"]), dtype)


class RumuvikForCausalLM(nn.Module):
    supports_cuda_graph = False          # the hybrid families run eagerly (ragged launches sized on the host)
    disable_radix_cache = True           # recurrent state per request: no page-aligned prefix to share

    def __init__(self, cfg: ModelConfig, quant_name: Optional[str] = None, device="cpu"):
        super().__init__()
        assert get_tp_group().world_size == 1 and get_pp_group().world_size == 1, "Rumuvik runs on one rank"
        assert cfg.hybrid and cfg.hybrid.get("layers") is not None, "Rumuvik needs the per-layer list of its configuration"
        self.cfg = cfg
        dtype = _DT[cfg.dtype]
        self.dtype = dtype
        specs = cfg.hybrid["layers"]
        self.embed_scale = float((cfg.hybrid.get("embedding") or {}).get("scale", 1.0))
        bb = nn.Module()
        bb.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype)
        bb.embed_tokens.weight.requires_grad_(False)
        bb.all_layers = nn.ModuleList([RumuvikBlock(cfg, s, i, dtype) for i, s in enumerate(specs)])
        # bf16 attention layers whose heads fit the tcgen05 kernels lay them out 128 columns wide in the leading columns of the pool's rows
        flat = [b.mix for b in bb.all_layers if b.kind == "attention"]
        for m in flat:
            if m.wants_padding(dtype):
                m.pad = 128
        widths = [m.cache_width for m in flat] + [b.mix.cache_width for b in bb.all_layers if b.kind == "latent_attention"]
        cache_width = -(-max(widths or [0]) // 8) * 8          # rows in multiples of 16 bytes (tensor maps over the pool)
        # runs: (block index, what the run owns, whether the embedding output joins the stream before it).  What a run owns: an attention
        # run a pool layer; a latent run (pool layer, plane); an mLSTM run an entry of the state pool.  Looped layers get fresh ones every pass.
        order = layer_passes(len(specs), cfg.hybrid.get("loop"))
        n_flat = sum(1 for i, _ in order if bb.all_layers[i].kind == "attention")
        self.runs: List[Tuple[int, object, bool]] = []
        bb.layers, n_lat, n_rec = [], 0, 0           # ``layers``: what the runner sizes the paged pool from
        for i, again in order:
            blk = bb.all_layers[i]
            if blk.kind == "attention":
                self.runs.append((i, len(bb.layers), again))
                bb.layers.append(_CacheLayer(FlatCacheSpec(blk.mix.H, cache_width, len(bb.layers), blk.mix.scale, -1)))
            elif blk.kind == "latent_attention":
                self.runs.append((i, (n_flat + n_lat // 2, n_lat % 2), again))
                n_lat += 1
            else:
                self.runs.append((i, n_rec, again))
                n_rec += 1
        for j in range((n_lat + 1) // 2):
            bb.layers.append(_CacheLayer(FlatCacheSpec(1, cache_width, n_flat + j, 1.0, -1)))
        bb.norm = ZeroCentredNorm(cfg.hidden_size, dtype)
        self.model = bb
        self.lm_head = nn.Parameter(torch.zeros(cfg.vocab_size, cfg.hidden_size, dtype=dtype), requires_grad=False)
        self.layer_tap = None            # callable(run index, fp32 residual [T, width]) after every layer run (debugging / tests)
        if dtype == torch.float32:
            torch.backends.cuda.matmul.allow_tf32 = False          # fp32 serving means fp32 products

    # ---- forward: fp32 residual stream; a block's residual add and the next block's two pre-norms are one kernel
    def forward(self, fb: ForwardBatch, inputs_embeds=None):
        m, eps, dt = self.model, self.cfg.rms_norm_eps, self.dtype
        if inputs_embeds is None:
            # decode reads every request's input token from the device-side token buffer (where sampling leaves it)
            ids = fb.input_ids if fb.input_ids is not None else fb.next_token_buf[fb.req_slots.long()]
            x = ops.bigram_embedding(m.embed_tokens.weight, None, ids, None, fb.cu_q, fb.req_slots, fb.seq_lens, fb.max_q_len, self.embed_scale)
        else:
            x = inputs_embeds.float().contiguous() * self.embed_scale
        x0 = x.clone() if any(again for _, _, again in self.runs) else None
        pending: List[torch.Tensor] = []          # branch outputs not yet added to the residual
        for run, (i, own, again) in enumerate(self.runs):
            blk = m.all_layers[i]
            h1, h2 = ops.parallel_add_rmsnorm_f32(x, pending, blk.norm1.weight, blk.norm2.weight if blk.mlp is not None else None, eps, True, dt,
                                                  x0 if again else None)
            if blk.kind == "attention":
                y = blk.mix(h1, fb, own)
            elif blk.kind == "latent_attention":
                y = blk.mix(h1, fb, fb.kv_pool.k(own[0]) if own[1] == 0 else fb.kv_pool.v(own[0]))
            else:
                y = blk.mix(h1, fb, own)
            pending = [y, blk.mlp(h2)] if blk.mlp is not None else [y]
            if self.layer_tap is not None:
                self.layer_tap(run, x + sum(t.float() for t in pending))
        h, _ = ops.parallel_add_rmsnorm_f32(x, pending, m.norm.weight, None, eps, True, dt)
        return h

    def compute_logits(self, hidden: torch.Tensor, key: str = "logits") -> torch.Tensor:
        return ops.linear(hidden, self.lm_head).float()

    # ---- recurrent state
    def make_mamba_pool(self, slots: int, device) -> Optional[LayeredStatePool]:
        geo = [self.model.all_layers[i].mix.state_geometry() for i, _, _ in self.runs if self.model.all_layers[i].kind == "mlstm"]
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
                self.model.norm.weight.data.copy_(w)
                ok = True
            elif name[:1] == "l" and "." in name and name[1:name.index(".")].isdigit():
                i, rest = int(name[1:name.index(".")]), name[name.index(".") + 1:]
                if i < len(L):
                    blk = L[i]
                    if rest in ("norm1", "norm2") and getattr(blk, rest) is not None:
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
        for i, sp in enumerate(cfg.hybrid["layers"]):
            p, m, kind = f"l{i}.", sp["mixer"], sp["type"]
            yield p + "norm1", rnd(p + "norm1", W, s=0.1)
            q = p + "mix."
            if kind == "attention":
                H, G, D = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"])
                Dv = int(m.get("vdim", D))
                for nm, n, s in (("q", H * D, 2.0), ("k", G * D, 2.0), ("v", G * Dv, 1.0)):
                    yield q + nm, lin(q + nm, n, W, s)
                    yield q + nm + ".b", rnd(q + nm + "b", n, s=0.1)
                yield q + "o", lin(q + "o", W, H * Dv)
            elif kind == "latent_attention":
                H, D, Dv, R, Rq = int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"]), int(m["q_rank"])
                Dr = int(m.get("rot_dim", (m.get("rot") or {}).get("dims", 0)))
                yield q + "dq", lin(q + "dq", Rq, W)
                yield q + "dq.norm", rnd(q + "dqn", Rq, s=0.1, off=1.0)
                yield q + "uq", lin(q + "uq", H * (D + Dr), Rq, 2.0)
                yield q + "dkv", lin(q + "dkv", R + Dr, W)
                yield q + "dkv.norm", rnd(q + "dkvn", R, s=0.1, off=1.0)
                yield q + "uk", lin(q + "uk", H * D, R, 2.0)
                yield q + "uv", lin(q + "uv", H * Dv, R)
                yield q + "o", lin(q + "o", W, H * Dv)
            else:
                H, D = int(m["heads"]), int(m["dim"])
                Dv = int(m.get("vdim", D))
                for nm, n in (("q", H * D), ("k", H * D), ("v", H * Dv), ("g", H * Dv)):
                    yield q + nm, lin(q + nm, n, W)
                yield q + "i", lin(q + "i", H, W)
                yield q + "i.b", rnd(q + "ib", H, s=0.5)
                yield q + "f", lin(q + "f", H, W)
                yield q + "f.b", rnd(q + "fb", H, s=0.5, off=3.0)
                yield q + "norm", rnd(q + "n", H * Dv, s=0.1, off=1.0)
                yield q + "o", lin(q + "o", W, H * Dv)
            mlp = sp.get("mlp")
            if not mlp:
                continue
            yield p + "norm2", rnd(p + "norm2", W, s=0.1)
            ff = int(mlp["ff"])
            yield p + "mlp.gate", lin(p + "g", ff, W)
            yield p + "mlp.up", lin(p + "u", ff, W)
            yield p + "mlp.down", lin(p + "d", W, ff)
        yield "final.norm", rnd("fn", W, s=0.1)
        yield "head", lin("head", cfg.vocab_size, W)
