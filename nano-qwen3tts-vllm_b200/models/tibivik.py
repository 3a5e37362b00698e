"""Tibivik: a decoder-only token model over several residual streams, with mixers that pair attention with a recurrence.

    x_s = embed[token] + bigram[hash(previous token, token)]              (every stream s starts as the same vector)
    sublayer f (mixer, then feed-forward) of a layer, with its stream connection (in, out, mix) and RMS norm:
        u = sum_s in[s] x_s;   y = f(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y
    mixers: "mamba2"      a selective state space (short convolution, scalar decay per head, gated grouped norm)
            "parallel"    sliding-window sink attention (q/k normed over the whole projection, half-split rotation, values
                          = the raw keys)  beside  a matrix memory with exponential gates
            "parallel_2"  chunked sink attention (biased projections, no positions, per-head output gate)  beside  a
                          gated delta rule (short convolutions, unit q/k)
            a parallel mixer returns left_scale * left + right_scale * right
    ff:     W_down (silu(W_gate h) * W_up h), or absent
    logits = embed . norm(sum_s x_s)                                        (the head is the embedding table)

Every layer carries its own sizes (``config.TibivikLayerSpec``).  ``loop`` runs a range of layers several times in a
row with the same modules; every layer RUN has a K/V cache and state of its own.  One forward runs a whole engine step:
prompt portions and single decoded tokens side by side, described by the step layout in the global Context.  Launches
per layer run: ONE merged input GEMM for both branches, attention preparation (bias / norm / rotation / cache write),
attention, [convolution,] the recurrence, gate + norm, two output GEMMs, the stream update fused with the next read-out
and norm, the feed-forward (merged gate|up GEMM with the activation, down GEMM), and the next stream update.
"""
from __future__ import annotations

import re

import torch
from torch import nn

from .. import _native as nat
from ..config import (DeltaRuleSpec, MatrixMemorySpec, ParallelMixerSpec, SinkAttentionSpec, StateSpaceSpec, TibivikConfig,
                      TibivikLayerSpec)
from ..layers import hyper_connection as hc
from ..layers.attention import SinkSoftmaxAttention
from ..layers.embed_head import BigramTokenEmbedding
from ..layers.layernorm import StreamRMSNorm
from ..layers.linear import MergedColumnParallelLinear, RowParallelLinear, linear, linear_silu_mul
from ..layers.recurrent import DeltaRuleMemory, MatrixMemory, StateSpaceMemory
from ..layers.rotary_embedding import HalfRotary


class SinkAttentionBranch(nn.Module):
    """The attention half of a parallel mixer; told apart by its spec alone."""

    def __init__(self, spec: SinkAttentionSpec, eps: float):
        super().__init__()
        m = self.spec = spec
        rot = HalfRotary(m.rot.dims, m.rot.base) if m.rot is not None else None
        self.attn = SinkSoftmaxAttention(m.heads, m.kv_heads, m.dim, m.vdim, m.mask_kind, m.mask_size, m.scale, bias=m.bias,
                                         qk_norm=m.qk_norm, rotary=rot, eps=eps)

    def proj_parts(self):
        m = self.spec
        parts = [("q", m.heads * m.dim), ("k", m.kv_heads * m.dim)]
        if not m.tied_values:
            parts.append(("v", m.kv_heads * m.vdim))
        if m.gate:
            parts.append(("g", m.heads))
        return parts

    def cache_plan(self):
        m = self.spec
        return [m.kv_heads * m.dim, m.kv_heads * m.vdim]

    def bind(self, paged):
        self.attn.k_cache, self.attn.v_cache = paged

    def forward(self, u: torch.Tensor, cols: dict) -> torch.Tensor:
        m = self.spec
        q = self.attn.prepare(u, cols["q"], cols["k"], -1 if m.tied_values else cols["v"])
        return self.attn(q, u[:, cols["g"]:cols["g"] + m.heads] if m.gate else None)


class ParallelMixer(nn.Module):
    """An attention branch and a recurrent branch behind ONE merged input projection; each has its output projection."""

    def __init__(self, width: int, spec: ParallelMixerSpec, eps: float):
        super().__init__()
        self.spec = spec
        self.left = SinkAttentionBranch(spec.left, eps)
        r = spec.right
        self.right = MatrixMemory(r, eps) if isinstance(r, MatrixMemorySpec) else DeltaRuleMemory(r, eps)
        self.parts = [("left." + n, w) for n, w in self.left.proj_parts()] + [("right." + n, w) for n, w in self.right.proj_parts()]
        self.in_proj = MergedColumnParallelLinear(width, [w for _, w in self.parts])
        off, self.cols = 0, {"left": {}, "right": {}}
        for name, w in self.parts:
            side, key = name.split(".", 1)
            self.cols[side][key] = off
            off += w
        self.left_o = RowParallelLinear(spec.left.heads * spec.left.vdim, width)
        self.right_o = RowParallelLinear(r.heads * r.vdim, width)

    def shard(self, name: str) -> int:
        return [n for n, _ in self.parts].index(name)

    def cache_plan(self):
        return {"paged": self.left.cache_plan(), "state": self.right.state_plan()}

    def bind(self, paged, state):
        self.left.bind(paged)
        self.right.bind(state)

    def forward(self, h: torch.Tensor):
        u = self.in_proj(h)
        a = self.left_o(self.left(u, self.cols["left"]))
        b = self.right_o(self.right(u, self.cols["right"]))
        return a, b, self.spec.left_scale, self.spec.right_scale


class StateSpaceMixer(nn.Module):
    def __init__(self, width: int, spec: StateSpaceSpec, eps: float):
        super().__init__()
        self.spec = spec
        self.core = StateSpaceMemory(spec, eps)
        self.in_proj = MergedColumnParallelLinear(width, [w for _, w in self.core.proj_parts()])
        self.o_proj = RowParallelLinear(spec.inner, width)

    def cache_plan(self):
        return {"paged": [], "state": self.core.state_plan()}

    def bind(self, paged, state):
        self.core.bind(state)

    def forward(self, h: torch.Tensor):
        return self.o_proj(self.core(self.in_proj(h), {"in": 0})), None, 1.0, 0.0


class GatedSiluFF(nn.Module):
    """W_down (silu(W_gate h) * W_up h) over a merged [gate; up] weight."""

    def __init__(self, width: int, ff: int):
        super().__init__()
        self.gate_up = MergedColumnParallelLinear(width, [ff, ff])
        self.down = RowParallelLinear(ff, width)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if h.dtype == torch.bfloat16:
            return self.down(linear_silu_mul(h, self.gate_up.weight))
        return self.down(nat.silu_mul(linear(h, self.gate_up.weight)))


class TibivikLayer(nn.Module):
    def __init__(self, width: int, spec: TibivikLayerSpec, eps: float, streams: int):
        super().__init__()
        self.norm1 = StreamRMSNorm(width, eps)
        self.hc1 = hc.StreamConnection(streams)
        self.mix = StateSpaceMixer(width, spec.mixer, eps) if spec.type == "mamba2" else ParallelMixer(width, spec.mixer, eps)
        if spec.mlp is None:
            self.mlp = self.norm2 = self.hc2 = None
        else:
            self.mlp = GatedSiluFF(width, spec.mlp.ff)
            self.norm2 = StreamRMSNorm(width, eps)
            self.hc2 = hc.StreamConnection(streams)


class TibivikForCausalLM(nn.Module):
    def __init__(self, config: TibivikConfig):
        super().__init__()
        self.config = c = config
        self.streams = max(c.streams, 1)
        bg = c.bigram or {}
        self.embed = BigramTokenEmbedding(c.vocab, c.width, self.streams, bg.get("buckets", 0), bg.get("mul_prev", 0), bg.get("mul_cur", 0))
        self.layers = nn.ModuleList([TibivikLayer(c.width, spec, c.norm_eps, self.streams) for spec in c.layers])
        self.runs = c.runs()
        self.final_norm = StreamRMSNorm(c.width, c.norm_eps)
        self.caches: list = [None] * len(self.runs)          # per layer RUN: (paged tensors, state tensors)
        self.trace_layers = None               # a list: forward() appends the sum of the streams after every layer run

    @property
    def dtype(self) -> torch.dtype:
        return self.embed.embed.dtype

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """One engine step over the packed tokens of the batch -> the residual streams [n, streams, width] (float)."""
        from ..utils.context import get_context
        dt = self.dtype
        xs = self.embed(tokens, get_context().step_layout.prev_tokens)
        runs = self.runs
        if not runs:
            return xs
        first = self.layers[runs[0]]
        h = hc.step(xs, None, None, first.hc1, first.norm1, dt)
        for r, li in enumerate(runs):
            layer = self.layers[li]
            nxt = self.layers[runs[r + 1]] if r + 1 < len(runs) else None
            layer.mix.bind(*self.caches[r])
            y = layer.mix(h)
            if layer.mlp is not None:
                h = hc.step(xs, y, layer.hc1, layer.hc2, layer.norm2, dt)
                y, post = (layer.mlp(h), None, 1.0, 0.0), layer.hc2
            else:
                post = layer.hc1
            h = hc.step(xs, y, post, nxt.hc1 if nxt is not None else None, nxt.norm1 if nxt is not None else None, dt)
            if self.trace_layers is not None:
                self.trace_layers.append(xs.sum(1))
        return xs

    def compute_logits(self, xs: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        """Logits (float) of the rows ``rows`` (all rows if None): the streams' sum, final norm, then the embedding table."""
        return linear(self.final_norm(xs, self.dtype, rows), self.embed.embed).float()

    # ------------------------------------------------------------------ cache and state
    def cache_plan(self) -> list[dict]:
        """Per layer run: widths of its paged tensors and shapes (after the slot axis) / dtypes of its state tensors."""
        return [self.layers[li].mix.cache_plan() for li in self.runs]

    def bind_cache(self, run: int, paged: list, state: list):
        self.caches[run] = (paged, state)

    # ------------------------------------------------------------------ weights
    def _targets(self) -> dict:
        """Checkpoint name -> (parameter, shard of a merged weight or None)."""
        t = {"embed": (self.embed.embed, None), "final.norm": (self.final_norm.weight, None)}
        if self.embed.bigram is not None:
            t["bigram"] = (self.embed.bigram, None)
        for i, (layer, spec) in enumerate(zip(self.layers, self.config.layers)):
            p = f"l{i}."
            t[p + "norm1"] = (layer.norm1.weight, None)
            subs = [(1, layer.hc1)]
            if layer.mlp is not None:
                t[p + "norm2"] = (layer.norm2.weight, None)
                t[p + "mlp.gate"] = (layer.mlp.gate_up.weight, 0)
                t[p + "mlp.up"] = (layer.mlp.gate_up.weight, 1)
                t[p + "mlp.down"] = (layer.mlp.down.weight, None)
                subs.append((2, layer.hc2))
            if self.config.streams:
                for q, conn in subs:
                    t[f"{p}hc{q}.in"], t[f"{p}hc{q}.out"], t[f"{p}hc{q}.mix"] = (conn.in_w, None), (conn.out_w, None), (conn.mix, None)
            mix = layer.mix
            if spec.type == "mamba2":
                core = mix.core
                t.update({p + "mix.in": (mix.in_proj.weight, None), p + "mix.conv": (core.conv.weight, None),
                          p + "mix.conv.b": (core.conv.bias, None), p + "mix.dt_bias": (core.dt_bias, None),
                          p + "mix.A_log": (core.A_log, None), p + "mix.D": (core.D, None), p + "mix.norm": (core.norm, None),
                          p + "mix.o": (mix.o_proj.weight, None)})
                continue
            a, m = mix.left.attn, spec.mixer.left
            L = p + "mix.left."
            for name, _ in mix.left.proj_parts():
                t[L + name] = (mix.in_proj.weight, mix.shard("left." + name))
            t[L + "sink"], t[L + "o"] = (a.sink, None), (mix.left_o.weight, None)
            if m.bias:
                t[L + "q.b"], t[L + "k.b"] = (a.q_bias, None), (a.k_bias, None)
                if not m.tied_values:
                    t[L + "v.b"] = (a.v_bias, None)
            if m.qk_norm:
                t[L + "q.norm"], t[L + "k.norm"] = (a.q_norm, None), (a.k_norm, None)
            R, right = p + "mix.right.", mix.right
            for name, _ in right.proj_parts():
                t[R + name] = (mix.in_proj.weight, mix.shard("right." + name))
            t[R + "norm"], t[R + "o"] = (right.norm, None), (mix.right_o.weight, None)
            if isinstance(spec.mixer.right, MatrixMemorySpec):
                t[R + "i.b"], t[R + "f.b"] = (right.i_bias, None), (right.f_bias, None)
            else:
                rs, off = spec.mixer.right, 0
                for ch, rows in (("q", rs.kv_heads * rs.dim), ("k", rs.kv_heads * rs.dim), ("v", rs.heads * rs.vdim)):
                    t[f"{R}{ch}.conv"] = (right.conv.weight[off:off + rows], None)
                    off += rows
                t[R + "A_log"], t[R + "dt_bias"] = (right.A_log, None), (right.dt_bias, None)
        return t

    def checkpoint_names(self) -> list[str]:
        return sorted(self._targets())

    def load_state_dict(self, state_dict, strict=True):
        """Checkpoint names: ``embed``, ``bigram``, ``final.norm``, and per layer ``l<i>.norm1|norm2``,
        ``l<i>.hc1|hc2.{in,out,mix}``, ``l<i>.mlp.{gate,up,down}`` and the mixer's tensors under ``l<i>.mix.`` (a parallel
        mixer's under ``.left.`` and ``.right.``).  Tensors are bfloat16 in the file; what the kernels keep in float (norm
        weights, stream matrices, sinks, biases of the attention, filters, per-head constants) is widened exactly."""
        targets, seen = self._targets(), set()
        for name, value in state_dict.items():
            if name not in targets:
                if strict:
                    raise KeyError(f"unexpected tensor {name!r} in the checkpoint")
                continue
            param, shard = targets[name]
            with torch.no_grad():
                if shard is not None:
                    param.weight_loader(param, value.to(param.dtype), shard)
                else:
                    if tuple(param.shape) != tuple(value.shape):
                        raise ValueError(f"{name}: shape {tuple(value.shape)} does not fit {tuple(param.shape)}")
                    param.copy_(value.to(param.dtype))
            seen.add(name)
        if strict:
            missing = sorted(set(targets) - seen)
            if missing:
                raise KeyError(f"missing tensors: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
        return seen


def random_state_dict(config: TibivikConfig, seed: int = 0) -> dict:
    """Random bfloat16 tensors under the checkpoint's names (benchmarks, tests and smoke runs; no trained weights exist)."""
    g = torch.Generator().manual_seed(seed)
    with torch.device("meta"):
        shapes = {k: tuple(p.shape) for k, (p, _) in TibivikForCausalLM(config)._targets().items()}
    # a shard of a merged weight: its own rows
    model_parts = {}
    for i, spec in enumerate(config.layers):
        p = f"l{i}."
        if spec.mlp is not None:
            model_parts[p + "mlp.gate"] = model_parts[p + "mlp.up"] = (spec.mlp.ff, config.width)
        if spec.type != "mamba2":
            lm, r = spec.mixer.left, spec.mixer.right
            rows = {"left.q": lm.heads * lm.dim, "left.k": lm.kv_heads * lm.dim, "left.v": lm.kv_heads * lm.vdim, "left.g": lm.heads}
            if isinstance(r, MatrixMemorySpec):
                rows.update({"right.q": r.heads * r.dim, "right.k": r.heads * r.dim, "right.v": r.heads * r.vdim,
                             "right.g": r.heads * r.vdim, "right.i": r.heads, "right.f": r.heads})
            else:
                rows.update({"right.q": r.kv_heads * r.dim, "right.k": r.kv_heads * r.dim, "right.v": r.heads * r.vdim,
                             "right.g": r.heads * r.vdim, "right.b": r.heads, "right.a": r.heads})
            for k, n in rows.items():
                model_parts[p + "mix." + k] = (n, config.width)
    sd = {}
    for name, shape in sorted(shapes.items()):
        shape = model_parts.get(name, shape)
        leaf = name.rsplit(".", 1)[-1]
        t = torch.randn(shape, generator=g)
        if re.search(r"norm\d?$", name) or leaf == "norm":
            t = 1.0 + 0.1 * t
        elif leaf == "mix" and ".hc" in name:
            t = torch.eye(shape[0]) + 0.2 * t
        elif leaf in ("in", "out") and ".hc" in name:
            t = 0.7 + 0.2 * t
        elif leaf in ("A_log", "dt_bias", "D", "sink", "b") and len(shape) == 1:
            t = 0.5 * t
        elif len(shape) == 2 and leaf != "conv":
            t = t * shape[1] ** -0.5
        elif leaf == "conv":
            t = 0.5 * t
        sd[name] = t.to(torch.bfloat16)
    return sd
