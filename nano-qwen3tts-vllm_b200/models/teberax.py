"""Teberax: a decoder-only token model over one 32-bit residual stream whose sublayers are normed on the way in and on
the way out, each norm a single-gain RMS norm n_g(v) = g v / sqrt(mean(v^2) + eps).

    x = n_e(embed[token])
    layer:  x <- x + n_1b(mixer(n_1(x)));   x <- x + n_2b(ff(n_2(x)))                         (the second line optional)
    mixers: "attention"         differential attention: two softmax maps per head over the same values, no positions,
                                sliding window with kept first keys; optionally on another layer's keys and values
            "parallel"          biased rotary attention (pair rotation with linearly scaled frequencies, soft-capped
                                scores, causal, a zero sink in the denominator)  beside  gated linear attention (a decay
                                per key channel); (N(left) * w_l + N(right) * w_r) / 2 with N the RMS norm over the width
            "latent_attention"  keys and values expanded from one normed latent per token plus one rotated key part
                                shared by the heads; sliding window; ordinary softmax
    ff:     W_down polynorm(W_up h);  or a mixture of SiLU-gated experts routed by a softmax over all router outputs
            (choice on score + correction, weights = scores), whose last outputs are identity experts;  or absent
    logits = cap tanh(head n_f(x) / cap)

Every layer carries its own sizes (``config.TeberaxLayerSpec``).  One forward runs a whole engine step: prompt portions
and single decoded tokens side by side, described by the step layout in the global Context.  Launches per layer: ONE
merged input GEMM per mixer, attention preparation (bias / rotation / cache write), attention [+ map combination], [decay
GEMM, the recurrence, gate + norm], output GEMM(s), ONE launch for the residual update fused with the next input norm
(the two branch norms of a parallel mixer and the weighted sum over experts ride in it), and the feed-forward's GEMMs with
their activation.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import _native as nat
from ..config import DiffAttentionSpec, GatedLinearSpec, SinkAttentionSpec, TeberaxConfig, TeberaxLayerSpec
from ..layers.activation import PolyNorm
from ..layers.attention import DifferentialAttention, SinkSoftmaxAttention
from ..layers.embed_head import NormedTokenEmbedding
from ..layers.layernorm import GainRMSNorm, SandwichNorm
from ..layers.linear import ColumnParallelLinear, MergedColumnParallelLinear, RowParallelLinear, linear
from ..layers.moe import SoftmaxIdentityMoE
from ..layers.recurrent import GatedLinearAttention
from ..layers.rotary_embedding import PairRotary
from .ridevik import LatentAttentionMixer

F32 = dict(dtype=torch.float32)


class DiffAttentionMixer(nn.Module):
    """q | k | v behind one merged projection (q alone for a layer that borrows keys and values), rows of q and k stored
    map-major (``DifferentialAttention.map_major``); attention over the paged cache; output projection."""

    def __init__(self, width: int, spec: DiffAttentionSpec, eps: float):
        super().__init__()
        m = self.spec = spec
        self.own = m.kv_from is None
        self.attn = DifferentialAttention(m.heads, m.kv_heads, m.dim, m.vdim, m.window, m.keep_first, m.scale, m.diff, eps, own_cache=self.own)
        self.nq, self.nk, self.nv = m.heads * 2 * m.dim, m.kv_heads * 2 * m.dim, m.kv_heads * m.vdim
        self.in_proj = MergedColumnParallelLinear(width, [self.nq, self.nk, self.nv] if self.own else [self.nq])
        self.o_proj = RowParallelLinear(m.heads * m.vdim, width)

    def cache_plan(self):
        return {"paged": [self.nk, self.nv] if self.own else [], "state": []}

    def bind(self, paged, state):
        self.attn.k_cache, self.attn.v_cache = paged

    def forward(self, h: torch.Tensor):
        u = self.in_proj(h)
        q = self.attn.prepare(u, 0, self.nq if self.own else 0, self.nq + self.nk if self.own else 0)
        return self.o_proj(self.attn(q))


class BiasedRotaryBranch(nn.Module):
    """The attention half of a parallel mixer: reads q | k | v from the mixer's merged projection."""

    def __init__(self, spec: SinkAttentionSpec, eps: float):
        super().__init__()
        m = self.spec = spec
        rot = PairRotary(m.rot.dims, m.rot.base, m.rot.scaling) if m.rot is not None else None
        self.attn = SinkSoftmaxAttention(m.heads, m.kv_heads, m.dim, m.vdim, m.mask_kind, m.mask_size, m.scale, bias=m.bias,
                                         rotary=rot, eps=eps, sink=m.sink, softcap=m.softcap, keep_first=m.keep_first)

    def proj_parts(self):
        m = self.spec
        return [("q", m.heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim)]

    def forward(self, u: torch.Tensor, cols: dict) -> torch.Tensor:
        return self.attn(self.attn.prepare(u, cols["q"], cols["k"], cols["v"]))


class AttentionLinearMixer(nn.Module):
    """Biased rotary attention beside gated linear attention behind ONE merged input projection; each branch has its
    output projection and a weight vector for the RMS norm over the width that precedes their half sum (the norms and the
    sum ride in the residual launch: ``forward`` returns both branch outputs)."""

    def __init__(self, width: int, spec, eps: float):
        super().__init__()
        self.spec = spec
        self.left = BiasedRotaryBranch(spec.left, eps)
        self.right = GatedLinearAttention(spec.right, eps)
        self.parts = [("left." + n, w) for n, w in self.left.proj_parts()] + [("right." + n, w) for n, w in self.right.proj_parts()]
        self.in_proj = MergedColumnParallelLinear(width, [w for _, w in self.parts])
        off, self.cols = 0, {"left": {}, "right": {}}
        for name, w in self.parts:
            side, key = name.split(".", 1)
            self.cols[side][key] = off
            off += w
        lm, r = spec.left, spec.right
        self.left_o = RowParallelLinear(lm.heads * lm.vdim, width, bias=lm.bias)
        self.right_o = RowParallelLinear(r.heads * r.vdim, width)
        self.left_out = nn.Parameter(torch.ones(width, **F32), requires_grad=False)
        self.right_out = nn.Parameter(torch.ones(width, **F32), requires_grad=False)

    def shard(self, name: str) -> int:
        return [n for n, _ in self.parts].index(name)

    def cache_plan(self):
        lm = self.spec.left
        return {"paged": [lm.kv_heads * lm.dim, lm.kv_heads * lm.vdim], "state": self.right.state_plan()}

    def bind(self, paged, state):
        self.left.attn.k_cache, self.left.attn.v_cache = paged
        self.right.bind(state)

    def forward(self, h: torch.Tensor):
        u = self.in_proj(h)
        a = self.left_o(self.left(u, self.cols["left"]))
        b = self.right_o(self.right(u, self.cols["right"]))
        return a, b


class LatentMixer(nn.Module):
    """Windowed latent attention with an ordinary softmax: the package's latent attention mixer without a sink."""

    def __init__(self, width: int, spec, eps: float):
        super().__init__()
        self.spec = spec
        self.core = LatentAttentionMixer(width, spec, eps)
        self.core.attn.sink = None                                              # no extra term in the denominator
        self.cache = None

    def cache_plan(self):
        return {"paged": [self.spec.cache_width], "state": []}

    def bind(self, paged, state):
        (self.cache,) = paged

    def forward(self, h: torch.Tensor):
        return self.core(h, self.cache)


class PolyNormFF(nn.Module):
    """W_down polynorm(W_up h)."""

    def __init__(self, width: int, ff: int, eps: float):
        super().__init__()
        self.up = ColumnParallelLinear(width, ff)
        self.act = PolyNorm(eps)
        self.down = RowParallelLinear(ff, width)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.down(self.act(self.up(h)))


class TeberaxLayer(nn.Module):
    def __init__(self, width: int, spec: TeberaxLayerSpec, eps: float):
        super().__init__()
        self.kind = spec.type
        self.norm1 = SandwichNorm(eps)
        if spec.type == "attention":
            self.mix = DiffAttentionMixer(width, spec.mixer, eps)
        elif spec.type == "parallel":
            self.mix = AttentionLinearMixer(width, spec.mixer, eps)
        else:
            self.mix = LatentMixer(width, spec.mixer, eps)
        f = spec.mlp
        self.mlp_kind = None if f is None else f.kind
        if f is None:
            self.mlp = self.norm2 = None
        else:
            self.norm2 = SandwichNorm(eps)
            self.mlp = PolyNormFF(width, f.ff, eps) if f.kind == "dense" else SoftmaxIdentityMoE(width, f.ff, f.experts, f.top, f.identity)

    def forward(self, x: torch.Tensor, h: torch.Tensor, nxt: GainRMSNorm | None):
        """x [n, width] float, updated in place; h = norm1.pre(x) in the activation type.  Returns the next layer's input
        ``nxt(x)`` (None after the last layer)."""
        after = self.norm2.pre if self.mlp is not None else nxt
        if self.kind == "parallel":
            a, b = self.mix(h)
            h = self.norm1.add(x, after, a=a, b=b, wa=self.mix.left_out, wb=self.mix.right_out, branch_scale=0.5)
        else:
            h = self.norm1.add(x, after, a=self.mix(h))
        if self.mlp_kind == "dense":
            h = self.norm2.add(x, nxt, a=self.mlp(h))
        elif self.mlp_kind == "moe":
            z, zw = self.mlp(h)
            h = self.norm2.add(x, nxt, z=z, zw=zw, z_idx=self.mlp.last_choice, n_real=self.mlp.experts, hin=h)
        return h


class TeberaxForCausalLM(nn.Module):
    def __init__(self, config: TeberaxConfig):
        super().__init__()
        self.config = c = config
        self.embed = NormedTokenEmbedding(c.vocab, c.width, c.norm_eps)
        self.layers = nn.ModuleList([TeberaxLayer(c.width, spec, c.norm_eps) for spec in c.layers])
        self.final_norm = GainRMSNorm(c.norm_eps)
        self.head = nn.Parameter(torch.empty(c.vocab, c.width), requires_grad=False)
        self.trace_layers = None               # a list: forward() appends a copy of the residual stream after every layer

    @property
    def dtype(self) -> torch.dtype:
        return self.head.dtype

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """One engine step over the packed tokens of the batch -> the residual stream [n, width] (float)."""
        layers = self.layers
        x, h = self.embed(tokens, layers[0].norm1.pre if len(layers) else None)
        for i, layer in enumerate(layers):
            h = layer(x, h, layers[i + 1].norm1.pre if i + 1 < len(layers) else None)
            if self.trace_layers is not None:
                self.trace_layers.append(x.clone())
        return x

    def compute_logits(self, x: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        logits = linear(self.final_norm(x, self.dtype, rows), self.head).float()
        cap = self.config.logit_softcap
        return nat.tanh_cap_(logits.contiguous(), cap) if cap > 0 else logits

    # ------------------------------------------------------------------ cache and state
    def cache_plan(self) -> list[dict]:
        """Per layer: widths of its paged tensors and shapes (after the slot axis) / dtypes of its state tensors.  A layer
        that borrows keys and values has none of its own."""
        return [layer.mix.cache_plan() for layer in self.layers]

    def bind_cache(self, run: int, paged: list, state: list):
        spec = self.config.layers[run]
        if spec.type == "attention" and spec.mixer.kv_from is not None:
            src = self.layers[spec.mixer.kv_from].mix.attn              # bound before: the source is an earlier layer
            paged = [src.k_cache, src.v_cache]
        self.layers[run].mix.bind(paged, state)

    # ------------------------------------------------------------------ weights
    def _targets(self) -> dict:
        """Checkpoint name -> (parameter, shard of a merged weight or None, transform of the stored tensor or None)."""
        t = {"embed": (self.embed.embed, None, None), "embed.norm": (self.embed.norm.weight, None, None),
             "final.norm": (self.final_norm.weight, None, None), "head": (self.head, None, None)}
        for i, (layer, spec) in enumerate(zip(self.layers, self.config.layers)):
            p = f"l{i}."
            t[p + "norm1"], t[p + "norm1b"] = (layer.norm1.pre.weight, None, None), (layer.norm1.post.weight, None, None)
            mix, m = layer.mix, spec.mixer
            M = p + "mix."
            if spec.type == "attention":
                a = mix.attn
                t[M + "q"] = (mix.in_proj.weight, 0, lambda w, m=m: DifferentialAttention.map_major(w, m.heads, m.dim))
                if mix.own:
                    t[M + "k"] = (mix.in_proj.weight, 1, lambda w, m=m: DifferentialAttention.map_major(w, m.kv_heads, m.dim))
                    t[M + "v"] = (mix.in_proj.weight, 2, None)
                for name in ("lq1", "lk1", "lq2", "lk2"):
                    t[M + name] = (getattr(a, name), None, None)
                t[M + "o"] = (mix.o_proj.weight, None, None)
            elif spec.type == "parallel":
                L, R, a, r = M + "left.", M + "right.", mix.left.attn, mix.right
                for name, _ in mix.left.proj_parts():
                    t[L + name] = (mix.in_proj.weight, mix.shard("left." + name), None)
                t[L + "q.b"], t[L + "k.b"], t[L + "v.b"] = (a.q_bias, None, None), (a.k_bias, None, None), (a.v_bias, None, None)
                t[L + "o"], t[L + "o.b"], t[L + "out"] = (mix.left_o.weight, None, None), (mix.left_o.bias, None, None), (mix.left_out, None, None)
                for name, _ in r.proj_parts():
                    t[R + name] = (mix.in_proj.weight, mix.shard("right." + name), None)
                t[R + "a2"], t[R + "a2.b"], t[R + "norm"] = (r.a2, None, None), (r.a2_bias, None, None), (r.norm, None, None)
                t[R + "o"], t[R + "out"] = (mix.right_o.weight, None, None), (mix.right_out, None, None)
            else:
                c = mix.core
                t[M + "q"], t[M + "dkv"] = (c.in_proj.weight, 0, None), (c.in_proj.weight, 1, None)
                t[M + "dkv.norm"], t[M + "uk"], t[M + "uv"] = (c.kv_norm, None, None), (c.uk, None, None), (c.uv, None, None)
                t[M + "o"] = (c.o_proj.weight, None, None)
            if layer.mlp is None:
                continue
            t[p + "norm2"], t[p + "norm2b"] = (layer.norm2.pre.weight, None, None), (layer.norm2.post.weight, None, None)
            F = p + "mlp."
            if layer.mlp_kind == "dense":
                t[F + "up"], t[F + "down"] = (layer.mlp.up.weight, None, None), (layer.mlp.down.weight, None, None)
                t[F + "act"] = (layer.mlp.act.coef, None, None)
            else:
                e = layer.mlp
                t[F + "router"], t[F + "correction"] = (e.router, None, None), (e.router_bias, None, None)
                for j in range(e.experts):
                    t[f"{F}e{j}.gate"], t[f"{F}e{j}.up"] = (e.up[j, :e.ff], None, None), (e.up[j, e.ff:], None, None)
                    t[f"{F}e{j}.down"] = (e.down[j], None, None)
        return t

    def checkpoint_names(self) -> list[str]:
        return sorted(self._targets())

    def load_state_dict(self, state_dict, strict=True):
        """Checkpoint names: ``embed``, ``embed.norm``, ``final.norm``, ``head``, per layer ``l<i>.norm1|norm1b|norm2|norm2b``,
        the mixer's tensors under ``l<i>.mix.`` (a parallel mixer's under ``.left.`` / ``.right.``) and the feed-forward's
        under ``l<i>.mlp.`` (experts ``.e<j>.``).  Tensors are bfloat16 in the file; what the kernels keep in float (norm
        gains and weights, biases of the attention, routers, the numbers of activations and of lambda) is widened exactly."""
        targets, seen = self._targets(), set()
        for name, value in state_dict.items():
            if name not in targets:
                if strict:
                    raise KeyError(f"unexpected tensor {name!r} in the checkpoint")
                continue
            param, shard, transform = targets[name]
            if transform is not None:
                value = transform(value)
            with torch.no_grad():
                if shard is not None:
                    param.weight_loader(param, value.to(param.dtype), shard)
                else:
                    if param.numel() != value.numel() or (param.dim() == value.dim() and tuple(param.shape) != tuple(value.shape)):
                        raise ValueError(f"{name}: shape {tuple(value.shape)} does not fit {tuple(param.shape)}")
                    param.copy_(value.to(param.dtype).reshape(param.shape))
            seen.add(name)
        for layer in self.layers:
            if layer.kind == "attention":
                layer.mix.attn._lam = None
        if strict:
            missing = sorted(set(targets) - seen)
            if missing:
                raise KeyError(f"missing tensors: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
        return seen


def checkpoint_shapes(config: TeberaxConfig) -> dict:
    """Checkpoint name -> shape, from the configuration alone."""
    D, sh = config.width, {}
    sh.update({"embed": (config.vocab, D), "embed.norm": (), "final.norm": (), "head": (config.vocab, D)})
    for i, spec in enumerate(config.layers):
        p, m = f"l{i}.", spec.mixer
        for n in ("norm1", "norm1b"):
            sh[p + n] = ()
        M = p + "mix."
        if spec.type == "attention":
            sh[M + "q"] = (m.heads * 2 * m.dim, D)
            if m.kv_from is None:
                sh[M + "k"], sh[M + "v"] = (m.kv_heads * 2 * m.dim, D), (m.kv_heads * m.vdim, D)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                sh[M + n] = (m.dim,)
            sh[M + "o"] = (D, m.heads * m.vdim)
        elif spec.type == "parallel":
            lm, r = m.left, m.right
            L, R = M + "left.", M + "right."
            for n, rows in (("q", lm.heads * lm.dim), ("k", lm.kv_heads * lm.dim), ("v", lm.kv_heads * lm.vdim)):
                sh[L + n], sh[L + n + ".b"] = (rows, D), (rows,)
            sh[L + "o"], sh[L + "o.b"], sh[L + "out"] = (D, lm.heads * lm.vdim), (D,), (D,)
            for n, rows in (("q", r.heads * r.dim), ("k", r.heads * r.dim), ("v", r.heads * r.vdim), ("g", r.heads * r.vdim),
                            ("a1", r.decay_rank)):
                sh[R + n] = (rows, D)
            sh[R + "a2"], sh[R + "a2.b"], sh[R + "norm"] = (r.heads * r.dim, r.decay_rank), (r.heads * r.dim,), (r.vdim,)
            sh[R + "o"], sh[R + "out"] = (D, r.heads * r.vdim), (D,)
        else:
            sh[M + "q"], sh[M + "dkv"] = (m.heads * (m.dim + m.rot_dim), D), (m.kv_rank + m.rot_dim, D)
            sh[M + "dkv.norm"], sh[M + "uk"], sh[M + "uv"] = (m.kv_rank,), (m.heads * m.dim, m.kv_rank), (m.heads * m.vdim, m.kv_rank)
            sh[M + "o"] = (D, m.heads * m.vdim)
        f = spec.mlp
        if f is None:
            continue
        for n in ("norm2", "norm2b"):
            sh[p + n] = ()
        F = p + "mlp."
        if f.kind == "dense":
            sh[F + "up"], sh[F + "down"], sh[F + "act"] = (f.ff, D), (D, f.ff), (4,)
        else:
            sh[F + "router"], sh[F + "correction"] = (f.experts + f.identity, D), (f.experts + f.identity,)
            for j in range(f.experts):
                sh[f"{F}e{j}.gate"], sh[f"{F}e{j}.up"], sh[f"{F}e{j}.down"] = (f.ff, D), (f.ff, D), (D, f.ff)
    return sh


def random_state_dict(config: TeberaxConfig, seed: int = 0) -> dict:
    """Random bfloat16 tensors under the checkpoint's names (benchmarks, tests and smoke runs; no trained weights exist)."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in sorted(checkpoint_shapes(config).items()):
        leaf = name.rsplit(".", 1)[-1]
        t = torch.randn(shape, generator=g)
        if len(shape) == 0:
            t = 1.0 + 0.1 * t                                     # norm gains
        elif len(shape) == 2:
            t = t * shape[1] ** -0.5
        elif leaf in ("norm", "out"):
            t = 1.0 + 0.1 * t
        elif leaf == "act":
            t = torch.tensor([1.0, 0.3, 0.1, 0.0]) + 0.1 * t
        elif leaf == "correction":
            t = 0.02 * t
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.3 * t
        else:
            t = 0.3 * t                                           # biases
        sd[name] = t.to(torch.bfloat16)
    return sd
