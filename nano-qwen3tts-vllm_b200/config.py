"""Engine and model configuration for the hot path.

``Config`` keeps the field names of the reference's engine dataclass (config.py:41-66) so the
``TalkerLLM(model_path, enforce_eager=..., gpu_memory_utilization=...)`` call is unchanged; unlike the
reference it does NOT overwrite ``max_model_len`` with 1024 (config.py:64): the decode block-table
buffers are sized from the real value, so voice-clone prompts (~4k tokens, BASELINE config 4) run
on the graph path.  ``StackConfig`` is the subset of the HF ``config.json`` the decoder stacks read
(``talker_config`` and its nested ``code_predictor_config``, config.py:171-360,362-560).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field


@dataclass
class StackConfig:
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 3072
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_scaling: dict | None = None          # {"mrope_section": [24,20,20], "interleaved": true}
    max_position_embeddings: int = 32768
    num_code_groups: int = 16
    text_vocab_size: int = 0
    text_hidden_size: int = 0

    @classmethod
    def from_dict(cls, d: dict) -> "StackConfig":
        known = {k: d[k] for k in cls.__dataclass_fields__ if k in d and (d[k] is not None or k == "rope_scaling")}
        c = cls(**known)
        if d.get("head_dim") is None:
            c.head_dim = c.hidden_size // c.num_attention_heads          # qwen3_tts_share.py:34
        return c

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim


@dataclass
class ModelConfig:
    """Parsed ``config.json`` of a Qwen3-TTS checkpoint (Qwen3TTSConfig, config.py:564-609)."""
    talker: StackConfig
    predictor: StackConfig
    codec_eos_token_id: int = 2150            # hard-coded in the reference's frame loop, interface.py:1233

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        t = d.get("talker_config", d)
        p = t.get("code_predictor_config", {})
        talker = StackConfig.from_dict(t)
        pd = dict(p)
        pd.setdefault("num_code_groups", talker.num_code_groups)
        predictor = StackConfig.from_dict(pd)
        return cls(talker=talker, predictor=predictor)

    @classmethod
    def from_pretrained(cls, model_dir: str) -> "ModelConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        t = {k: getattr(self.talker, k) for k in StackConfig.__dataclass_fields__}
        t["code_predictor_config"] = {k: getattr(self.predictor, k) for k in StackConfig.__dataclass_fields__}
        return {"talker_config": t}


def qwen3_tts_config(size: str = "1.7B") -> ModelConfig:
    """The shipped model shapes; weights are random-init in every BASELINE
    config, so these numbers define the workload."""
    mrope = {"mrope_section": [24, 20, 20], "interleaved": True}
    if size in ("1.7B", "1.7b"):
        talker = StackConfig(hidden_size=2048, intermediate_size=6144, num_hidden_layers=28, vocab_size=3072,
                             rope_scaling=mrope, text_vocab_size=151936, text_hidden_size=2048)
    elif size in ("0.6B", "0.6b"):
        talker = StackConfig(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, vocab_size=3072,
                             rope_scaling=mrope, text_vocab_size=151936, text_hidden_size=2048)
    elif size == "tiny":                      # test-sized: same kernels, seconds on the CPU oracle
        talker = StackConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, vocab_size=3072,
                             rope_scaling=mrope)
        return ModelConfig(talker, StackConfig(hidden_size=128, intermediate_size=384, num_hidden_layers=2,
                                               vocab_size=2048))
    else:
        raise ValueError(f"unknown model size {size!r}")
    predictor = StackConfig(hidden_size=1024, intermediate_size=3072, num_hidden_layers=5, vocab_size=2048)
    return ModelConfig(talker, predictor)


@dataclass
class MixerSpec:
    """One token mixer of a layered decoder: windowed attention over ``kv_heads`` shared key/value heads with a short
    causal convolution (``conv`` taps) after the projections."""
    heads: int
    kv_heads: int
    dim: int                       # query / key size per head
    vdim: int                      # value size per head
    conv: int                      # taps of the short convolution (1 = none)
    window: int                    # keys a position sees, itself included
    scale: float                   # score multiplier

    @property
    def channels(self) -> int:
        return self.heads * self.dim + self.kv_heads * (self.dim + self.vdim)


@dataclass
class FeedForwardSpec:
    kind: str                      # "dense" | "moe"
    ff: int                        # inner size (of one expert for "moe")
    experts: int = 0
    top: int = 0
    router_scale: float = 1.0
    act: str = "relu2"             # "relu2": relu(up)^2;  "xielu": two learned numbers;  "silu_gate": silu(gate) * up;
                                   # "polynorm": a N(z) + b N(z^2) + c N(z^3) + e with four learned numbers
    bias: bool = False             # dense projections carry biases
    router: str = "sigmoid"        # "sigmoid": scores / their sum;  "softmax_chosen": logits + bias, softmax over the chosen;
                                   # "softmax_all": softmax over all outputs, a correction enters the choice only
    identity: int = 0              # router outputs beyond ``experts`` that stand for experts returning their input


@dataclass
class LayerSpec:
    type: str                      # which mixer ("attention")
    mixer: MixerSpec
    mlp: FeedForwardSpec | None


@dataclass
class BokenexConfig:
    """``config.json`` of a Bokenex checkpoint: a decoder-only token model whose layers are listed one by one, each
    with its own mixer sizes and feed-forward (dense, mixture of experts, or none).  Every size and every constant
    that can differ between checkpoints is read here; nothing is assumed equal across layers."""
    architecture: str
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    residual_mult: float
    layers: list

    page_multiple = 16             # KV pages of this family may be any multiple of 16 tokens

    @classmethod
    def from_dict(cls, d: dict) -> "BokenexConfig":
        layers = []
        for i, ld in enumerate(d["layers"]):
            if ld["type"] != "attention":
                raise ValueError(f"layer {i}: unknown mixer type {ld['type']!r}")
            m = ld["mixer"]
            mixer = MixerSpec(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                              conv=int(m.get("conv", 1)), window=int(m["mask"]["size"]), scale=float(m["scale"]))
            if mixer.heads % mixer.kv_heads:
                raise ValueError(f"layer {i}: {mixer.heads} heads over {mixer.kv_heads} key/value heads")
            f = ld.get("mlp")
            mlp = None
            if f is not None:
                if f["kind"] == "dense":
                    mlp = FeedForwardSpec("dense", int(f["ff"]))
                elif f["kind"] == "moe":
                    r = f["router"]
                    mlp = FeedForwardSpec("moe", int(f["expert"]["ff"]), int(r["experts"]), int(r["top"]), float(r["scale"]))
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {f['kind']!r}")
            layers.append(LayerSpec(ld["type"], mixer, mlp))
        return cls(architecture=d["architecture"], vocab=int(d["vocab"]), width=int(d["width"]),
                   max_positions=int(d["max_positions"]), norm_eps=float(d["norm"]["eps"]),
                   residual_mult=float(d["residual_mult"]), layers=layers)

    @classmethod
    def from_pretrained(cls, model_dir: str) -> "BokenexConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        out = []
        for l in self.layers:
            m = l.mixer
            mlp = None
            if l.mlp is not None and l.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": l.mlp.ff}
            elif l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff},
                       "router": {"experts": l.mlp.experts, "top": l.mlp.top, "scale": l.mlp.router_scale}}
            out.append({"type": l.type, "mlp": mlp,
                        "mixer": {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv,
                                  "mask": {"size": m.window}, "scale": m.scale}})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "layers": out}


@dataclass
class RotarySpec:
    """Pair rotation of the first ``dims`` coordinates (2i with 2i+1) by position * base^(-2i/dims); ``scaling``
    {factor, original, fast, slow} blends each frequency with its ``1/factor`` multiple over a ramp (YaRN), ``scaling``
    {factor} alone divides every frequency by it (linear)."""
    dims: int
    base: float
    scaling: dict | None = None


@dataclass
class LatentMixerSpec:
    """Attention whose keys and values are expanded per head from one cached latent per token, plus one rotated key
    part shared by all heads.  ``q_rank`` 0: queries come straight from the input; otherwise through a normed latent.
    ``window`` 0: every earlier key is visible.  ``gate``: the heads' outputs are multiplied by a sigmoid gate."""
    heads: int
    dim: int                       # un-rotated query / key size per head
    rot_dim: int                   # rotated query / key size per head (the key part is shared by the heads)
    vdim: int
    kv_rank: int
    q_rank: int
    window: int
    scale: float
    rot: RotarySpec
    gate: bool

    @property
    def cache_width(self) -> int:
        return self.kv_rank + self.rot_dim


@dataclass
class RidevikLayerSpec:
    type: str                      # "latent_attention" | "latent_attention_2"
    mixer: LatentMixerSpec
    mlp: FeedForwardSpec | None
    weights_of: int | None = None  # this layer runs another layer's tensors over a cache and state of its own


@dataclass
class RidevikConfig:
    """``config.json`` of a Ridevik checkpoint: a decoder-only token model whose layers (listed one by one, each with
    its own sizes) read the 32-bit residual stream itself, token-shifted for the mixer, and add their output after a
    grouped RMS norm.  Mixers are latent attentions in two variants; feed-forwards are dense (xIELU, biases) or a
    softmax-over-chosen mixture of gated experts, or absent.  A layer may reuse an earlier layer's tensors."""
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    norm_groups: int
    layers: list
    max_positions = None           # positions enter through rotations only: no table bounds them

    page_multiple = 16

    MIXER_TYPES = ("latent_attention", "latent_attention_2")

    @classmethod
    def from_dict(cls, d: dict) -> "RidevikConfig":
        layers = []
        for i, ld in enumerate(d["layers"]):
            if ld["type"] not in cls.MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {ld['type']!r}")
            m = ld["mixer"]
            r = m["rot"]
            rot = RotarySpec(int(r["dims"]), float(r["base"]), dict(r["scaling"]) if r.get("scaling") else None)
            mixer = LatentMixerSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                                    kv_rank=int(m["kv_rank"]), q_rank=int(m.get("q_rank") or 0),
                                    window=int(m["mask"]["size"]) if m.get("mask") else 0, scale=float(m["scale"]), rot=rot,
                                    gate=ld["type"] == "latent_attention")
            if rot.dims > mixer.rot_dim or rot.dims % 2:
                raise ValueError(f"layer {i}: {rot.dims} rotated dimensions in a part of {mixer.rot_dim}")
            f = ld.get("mlp")
            mlp = None
            if f is not None:
                if f["kind"] == "dense":
                    mlp = FeedForwardSpec("dense", int(f["ff"]), act="xielu", bias=True)
                elif f["kind"] == "moe":
                    ro = f["router"]
                    mlp = FeedForwardSpec("moe", int(f["expert"]["ff"]), int(ro["experts"]), int(ro["top"]), act="silu_gate",
                                          router="softmax_chosen")
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {f['kind']!r}")
            src = ld.get("weights_of")
            if src is not None and not (0 <= int(src) < len(d["layers"]) and int(src) != i
                                        and d["layers"][int(src)].get("weights_of") is None):
                raise ValueError(f"layer {i}: weights_of {src} must name another layer with tensors of its own")
            layers.append(RidevikLayerSpec(ld["type"], mixer, mlp, None if src is None else int(src)))
        c = cls(architecture=d["architecture"], vocab=int(d["vocab"]), width=int(d["width"]),
                embedding_scale=float(d["embedding"]["scale"]), norm_eps=float(d["norm"]["eps"]),
                norm_groups=int(d["norm"].get("groups", 1)), layers=layers)
        if c.width % c.norm_groups:
            raise ValueError(f"width {c.width} does not split into {c.norm_groups} norm groups")
        return c

    @classmethod
    def from_pretrained(cls, model_dir: str) -> "RidevikConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        out = []
        for l in self.layers:
            m = l.mixer
            mix = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale,
                   "rot": {"dims": m.rot.dims, "base": m.rot.base}}
            if m.rot.scaling:
                mix["rot"]["scaling"] = dict(m.rot.scaling)
            if m.q_rank:
                mix["q_rank"] = m.q_rank
            if m.window:
                mix["mask"] = {"size": m.window}
            mlp = None
            if l.mlp is not None and l.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": l.mlp.ff}
            elif l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff}, "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
            entry = {"type": l.type, "mixer": mix, "mlp": mlp}
            if l.weights_of is not None:
                entry["weights_of"] = l.weights_of
            out.append(entry)
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                "layers": out}


@dataclass
class HalfRotarySpec:
    """Rotation of the first ``dims`` coordinates of a head, coordinate i paired with i + dims/2, by position *
    base^(-2i/dims)."""
    dims: int
    base: float


@dataclass
class SinkAttentionSpec:
    """Softmax attention over ``kv_heads`` shared key/value heads with a learned per-head sink in the denominator, under a
    mask that is a sliding window or a chunk of ``mask_size`` positions.  Switches: ``bias`` on the q/k/v projections,
    ``qk_norm`` (RMS norm over the whole q and the whole k projection), ``rot`` (or no positions at all), ``tied_values``
    (no value projection: the values are the keys as projected, before norm and rotation), ``gate`` (one sigmoid gate
    per head on the output)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    mask_kind: str                 # "window" | "chunk"
    mask_size: int
    scale: float
    rot: object | None = None      # HalfRotarySpec (i with i + dims/2) | RotarySpec (2i with 2i + 1)
    qk_norm: bool = False
    bias: bool = False
    gate: bool = False
    tied_values: bool = False
    softcap: float = 0.0           # c > 0: scaled scores become c tanh(s / c)
    keep_first: int = 0            # keys below this position stay visible behind the mask
    sink: str = "learned"          # "learned": exp(sink_h) in the denominator;  "zero": exp(0);  "none": an ordinary softmax


@dataclass
class MatrixMemorySpec:
    """Matrix memory with exponential input and forget gates (log gates capped by ``gate_cap`` * tanh(. / ``gate_cap``))."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass
class DeltaRuleSpec:
    """Gated delta-rule memory: ``kv_heads`` query/key heads shared by ``heads`` value heads, a short convolution of
    ``conv`` taps on q, k and v."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass
class StateSpaceSpec:
    """Selective state space with a scalar decay per head: ``heads`` x ``vdim`` inner channels, ``state`` numbers per
    channel, B and C shared by the heads of a group, output norm in ``norm_groups`` parts."""
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state


@dataclass
class ParallelMixerSpec:
    """An attention branch and a recurrent branch that read the same input; their outputs are added with two weights."""
    left: SinkAttentionSpec
    right: object                  # MatrixMemorySpec | DeltaRuleSpec
    left_scale: float
    right_scale: float


@dataclass
class TibivikLayerSpec:
    type: str                      # "mamba2" | "parallel" | "parallel_2"
    mixer: object                  # StateSpaceSpec | ParallelMixerSpec
    mlp: FeedForwardSpec | None
    raw: dict = field(default_factory=dict, repr=False)      # the layer's entry as read (kept for to_dict)


@dataclass
class TibivikConfig:
    """``config.json`` of a Tibivik checkpoint: a decoder-only token model over ``streams`` copies of the residual
    stream that small learned matrices mix around every sublayer (0: one plain residual stream).  The embedding adds a
    hashed (previous token, token) row.  Layers are listed one by one with their own sizes: a state-space mixer, or an
    attention branch beside a recurrent branch (sliding window + matrix memory, or chunks + delta rule); feed-forwards are
    SiLU-gated or absent.  ``loop`` repeats a range of layers with the same weights, each pass over a cache and state of
    its own.  The output head is the embedding table."""
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    streams: int
    bigram: dict | None            # {"buckets", "mul_prev", "mul_cur"}
    layers: list
    loop: dict | None              # {"start", "stop", "times"}
    max_positions = None           # positions enter through rotations only: no table bounds them

    page_multiple = 16

    @staticmethod
    def _attention(m: dict, kind: str, i: int) -> SinkAttentionSpec:
        r = m.get("rot")
        rot = HalfRotarySpec(int(r["dims"]), float(r["base"])) if r else None
        window = kind == "parallel"
        spec = SinkAttentionSpec(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                 mask_kind="window" if window else "chunk", mask_size=int(m["mask"]["size"]),
                                 scale=float(m["scale"]), rot=rot, qk_norm=window, bias=not window, gate=not window,
                                 tied_values=window)
        if spec.heads % spec.kv_heads:
            raise ValueError(f"layer {i}: {spec.heads} heads over {spec.kv_heads} key/value heads")
        if spec.tied_values and spec.vdim != spec.dim:
            raise ValueError(f"layer {i}: values that are the keys need vdim == dim ({spec.vdim} != {spec.dim})")
        if rot is not None and (rot.dims % 2 or rot.dims > spec.dim):
            raise ValueError(f"layer {i}: {rot.dims} rotated coordinates in a head of {spec.dim}")
        if spec.mask_size < 1:
            raise ValueError(f"layer {i}: mask size {spec.mask_size}")
        return spec

    @classmethod
    def from_dict(cls, d: dict) -> "TibivikConfig":
        layers = []
        for i, ld in enumerate(d["layers"]):
            kind, m = ld["type"], ld["mixer"]
            if kind == "mamba2":
                mixer = StateSpaceSpec(heads=int(m["heads"]), vdim=int(m["vdim"]), state=int(m["state"]), groups=int(m["groups"]),
                                       conv=int(m["conv"]), norm_groups=int(m["norm_groups"]))
                if mixer.heads % mixer.groups or mixer.inner % mixer.norm_groups:
                    raise ValueError(f"layer {i}: heads, groups and norm groups do not divide")
            elif kind == "parallel":
                rt = m["right"]
                right = MatrixMemorySpec(heads=int(rt["heads"]), dim=int(rt["dim"]), vdim=int(rt["vdim"]), gate_cap=float(rt["gate_cap"]))
                mixer = ParallelMixerSpec(cls._attention(m["left"], kind, i), right, float(m["left_scale"]), float(m["right_scale"]))
            elif kind == "parallel_2":
                rt = m["right"]
                right = DeltaRuleSpec(heads=int(rt["heads"]), kv_heads=int(rt["kv_heads"]), dim=int(rt["dim"]), vdim=int(rt["vdim"]),
                                      conv=int(rt["conv"]))
                if right.heads % right.kv_heads:
                    raise ValueError(f"layer {i}: {right.heads} value heads over {right.kv_heads} key heads")
                mixer = ParallelMixerSpec(cls._attention(m["left"], kind, i), right, float(m["left_scale"]), float(m["right_scale"]))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            f = ld.get("mlp")
            mlp = None
            if f is not None:
                if f["kind"] != "dense":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {f['kind']!r}")
                mlp = FeedForwardSpec("dense", int(f["ff"]), act="silu_gate")
            layers.append(TibivikLayerSpec(kind, mixer, mlp, raw=ld))
        bg = (d.get("embedding") or {}).get("bigram")
        bigram = {k: int(bg[k]) for k in ("buckets", "mul_prev", "mul_cur")} if bg else None
        lp = d.get("loop")
        loop = {k: int(lp[k]) for k in ("start", "stop", "times")} if lp else None
        if loop is not None and not (0 <= loop["start"] <= loop["stop"] <= len(layers) and loop["times"] >= 1):
            raise ValueError(f"loop {loop} does not fit {len(layers)} layers")
        streams = int(d.get("streams") or 0)
        if streams > 8:
            raise ValueError(f"{streams} streams (at most 8)")
        return cls(architecture=d["architecture"], vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                   streams=streams, bigram=bigram, layers=layers, loop=loop)

    @classmethod
    def from_pretrained(cls, model_dir: str) -> "TibivikConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def runs(self) -> list[int]:
        """Layer index of every layer run, in order: the looped range repeats in a row."""
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        a, b, t = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(a)) + list(range(a, b)) * t + list(range(b, n))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [dict(l.raw) for l in self.layers]}
        if self.streams:
            out["streams"] = self.streams
        if self.bigram:
            out["embedding"] = {"bigram": dict(self.bigram)}
        if self.loop:
            out["loop"] = dict(self.loop)
        return out


@dataclass
class DiffAttentionSpec:
    """Differential attention: every head runs two softmax maps (their queries and keys stored side by side) over the
    same values and returns map 1 - lambda * map 2, divided by its root mean square and multiplied by 1 - ``diff``.
    ``window`` 0: causal; ``keep_first``: first keys that stay visible behind the window.  ``kv_from``: the layer has no
    key/value projections and reads the cache of that (earlier) layer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    window: int = 0
    keep_first: int = 0
    kv_from: int | None = None


@dataclass
class GatedLinearSpec:
    """Gated linear attention: a matrix state per head with one decay per key channel and token,
    sigmoid(W_a2 W_a1 h + b)^(1/tau); ``decay_rank`` is the inner size of that two-step projection (0: not known yet,
    read from the checkpoint's tensor shapes)."""
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int = 0


@dataclass
class TeberaxLayerSpec:
    type: str                      # "attention" | "parallel" | "latent_attention"
    mixer: object                  # DiffAttentionSpec | ParallelMixerSpec | LatentMixerSpec
    mlp: FeedForwardSpec | None
    raw: dict = field(default_factory=dict, repr=False)      # the layer's entry as read (kept for to_dict)


@dataclass
class TeberaxConfig:
    """``config.json`` of a Teberax checkpoint: a decoder-only token model over one 32-bit residual stream whose
    sublayers are normed on the way in and on the way out with single-gain RMS norms.  Layers are listed one by one with
    their own sizes: differential window attention (optionally on another layer's keys and values), biased rotary
    attention with a zero sink beside gated linear attention, or windowed latent attention; feed-forwards are dense with
    PolyNorm, a softmax-routed mixture of SiLU-gated experts with identity experts, or absent.  Logits pass a tanh cap."""
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float
    layers: list
    max_positions = None           # positions enter through rotations only: no table bounds them

    page_multiple = 16

    @staticmethod
    def _rot(r: dict | None):
        if not r:
            return None
        sc = r.get("scaling")
        return RotarySpec(int(r["dims"]), float(r["base"]), {"factor": float(sc["factor"])} if sc else None)

    @classmethod
    def from_dict(cls, d: dict) -> "TeberaxConfig":
        layers = []
        for i, ld in enumerate(d["layers"]):
            kind, m = ld["type"], ld["mixer"]
            mask = m.get("mask") or {}
            if kind == "attention":
                src = m.get("kv_from")
                mixer = DiffAttentionSpec(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                          scale=float(m["scale"]), diff=float(m["diff"]), window=int(mask.get("size") or 0),
                                          keep_first=int(mask.get("keep_first") or 0), kv_from=None if src is None else int(src))
                if mixer.heads % mixer.kv_heads:
                    raise ValueError(f"layer {i}: {mixer.heads} heads over {mixer.kv_heads} key/value heads")
                if mixer.kv_from is not None:
                    s = layers[mixer.kv_from].mixer if 0 <= mixer.kv_from < i else None
                    if not isinstance(s, DiffAttentionSpec) or s.kv_from is not None or \
                            (s.kv_heads, s.dim, s.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                        raise ValueError(f"layer {i}: kv_from {mixer.kv_from} must name an earlier attention layer with key/value "
                                         "projections of its own and the same key/value sizes")
            elif kind == "parallel":
                lm, rt = m["left"], m["right"]
                left = SinkAttentionSpec(heads=int(lm["heads"]), kv_heads=int(lm["kv_heads"]), dim=int(lm["dim"]), vdim=int(lm["vdim"]),
                                         mask_kind="window", mask_size=0, scale=float(lm["scale"]), rot=cls._rot(lm.get("rot")),
                                         bias=True, softcap=float(lm.get("softcap") or 0.0), sink="zero")
                if left.heads % left.kv_heads:
                    raise ValueError(f"layer {i}: {left.heads} heads over {left.kv_heads} key/value heads")
                if left.rot is not None and (left.rot.dims % 2 or left.rot.dims > left.dim):
                    raise ValueError(f"layer {i}: {left.rot.dims} rotated coordinates in a head of {left.dim}")
                right = GatedLinearSpec(heads=int(rt["heads"]), dim=int(rt["dim"]), vdim=int(rt["vdim"]), tau=float(rt["tau"]),
                                        decay_rank=int(rt.get("decay_rank") or 0))
                mixer = ParallelMixerSpec(left, right, 0.5, 0.5)
            elif kind == "latent_attention":
                rot = cls._rot(m["rot"])
                mixer = LatentMixerSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                                        kv_rank=int(m["kv_rank"]), q_rank=0, window=int(mask.get("size") or 0),
                                        scale=float(m["scale"]), rot=rot, gate=False)
                if rot.dims > mixer.rot_dim or rot.dims % 2:
                    raise ValueError(f"layer {i}: {rot.dims} rotated dimensions in a part of {mixer.rot_dim}")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            f = ld.get("mlp")
            mlp = None
            if f is not None:
                if f["kind"] == "dense":
                    mlp = FeedForwardSpec("dense", int(f["ff"]), act="polynorm")
                elif f["kind"] == "moe":
                    ro = f["router"]
                    mlp = FeedForwardSpec("moe", int(f["expert"]["ff"]), int(ro["experts"]), int(ro["top"]), act="silu_gate",
                                          router="softmax_all", identity=int(ro.get("identity") or 0))
                    if not 1 <= mlp.top <= mlp.experts + mlp.identity:
                        raise ValueError(f"layer {i}: top {mlp.top} of {mlp.experts} + {mlp.identity} experts")
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {f['kind']!r}")
            layers.append(TeberaxLayerSpec(kind, mixer, mlp, raw=ld))
        return cls(architecture=d["architecture"], vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                   logit_softcap=float(d.get("logit_softcap") or 0.0), layers=layers)

    def complete_from_checkpoint(self, model_dir: str) -> None:
        """Sizes that only a tensor's shape gives (the inner size of the decay projection) are read from the header of
        ``model.safetensors``: 8 bytes of little-endian length, then that many bytes of JSON."""
        todo = [i for i, l in enumerate(self.layers) if l.type == "parallel" and not l.mixer.right.decay_rank]
        path = os.path.join(model_dir, "model.safetensors")
        if not todo or not os.path.exists(path):
            return
        import struct
        with open(path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            header = json.loads(f.read(n))
        for i in todo:
            self.layers[i].mixer.right.decay_rank = int(header[f"l{i}.mix.right.a1"]["shape"][0])

    @classmethod
    def from_pretrained(cls, model_dir: str) -> "TeberaxConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            c = cls.from_dict(json.load(f))
        c.complete_from_checkpoint(model_dir)
        return c

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            e = json.loads(json.dumps(l.raw))
            if l.type == "parallel" and l.mixer.right.decay_rank:
                e["mixer"]["right"]["decay_rank"] = l.mixer.right.decay_rank
            layers.append(e)
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": layers}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out


def load_model_config(model_dir: str):
    """Parse ``config.json`` with the configuration class its architecture is registered under; a class that needs sizes
    only the checkpoint's tensor shapes give completes itself from the file's header."""
    from .models.registry import resolve
    with open(os.path.join(model_dir, "config.json")) as f:
        d = json.load(f)
    cfg = resolve(d).config_cls.from_dict(d)
    if hasattr(cfg, "complete_from_checkpoint"):
        cfg.complete_from_checkpoint(model_dir)
    return cfg


@dataclass
class Config:
    """Engine configuration; field names follow the reference's ``Config`` (config.py:41-66)."""
    model: str = ""
    max_num_batched_tokens: int = 16384
    max_num_seqs: int = 512
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.9
    tensor_parallel_size: int = 1
    enforce_eager: bool = False
    hf_config: object | None = None            # ModelConfig, or the configuration class of a registered architecture
    eos: int = -1
    kvcache_block_size: int = 256
    num_kvcache_blocks: int = -1
    distributed_port: int = 29500
    process_gpu_memory_fraction: float | None = None
    # additions (not in the reference)
    device: str = "cuda:0"
    rounding: int = 0                          # _native.ROUND_EAGER | ROUND_FUSED, see DESIGN.md
    graph_batch_sizes: list = field(default_factory=list)   # [] = reference's schedule

    max_state_slots: int = 0                   # per-sequence recurrent / convolution state slots (0 = max_num_seqs)
    dtype: str = "bfloat16"                    # activation and cache type: "bfloat16", or "float32" where a model has it

    def __post_init__(self):
        assert self.tensor_parallel_size == 1, "replicas only: the hot path never shards a model"
        assert self.max_num_batched_tokens >= self.max_model_len
        if self.hf_config is None and self.model:
            assert os.path.isdir(self.model), self.model               # config.py:59
            self.hf_config = load_model_config(self.model)
        # the reference's pages are multiples of 256 tokens (config.py:60); a model family may allow finer ones
        assert self.kvcache_block_size % getattr(self.hf_config, "page_multiple", 256) == 0
        assert self.dtype in ("bfloat16", "float32")
