"""RoPE modules with the reference's surface (layers/rotary_embedding.py:87-237):
``get_rope(head_size, rotary_dim, max_position, base, rope_scaling)`` -> module with buffer
``inv_freq`` and ``forward(positions, query, key) -> (query, key)``.

cos/sin are recomputed from ``positions`` inside the kernel (fp32 angle -> bf16 cos/sin) and the
rotation keeps the three bf16 roundings of the reference's eager expression.  The talker's 3-D
M-RoPE is a per-column choice of position row (``modality``); with the 1-D positions the runner
feeds (talker_mode_runner.py:134) it collapses to plain RoPE."""
import torch
from torch import nn

from .. import _native as nat


def mrope_dim_modality(head_dim: int, mrope_section, interleaved: bool) -> list[int]:
    """Position row (0..2) read by each of the ``head_dim`` cos/sin columns
    (apply_multimodal_rotary_pos_emb, rotary_embedding.py:52-80)."""
    half = head_dim // 2
    if interleaved:
        m = [0] * half
        n_mod = len(mrope_section)
        for i, n in enumerate(mrope_section[1:], 1):
            for f in range(i, min(n * n_mod, half), n_mod):
                m[f] = i
        return m + m
    out = []
    for i, n in enumerate(mrope_section):          # sections doubled in WIDTH, rotary_embedding.py:74
        out += [i % 3] * (2 * n)
    assert len(out) == head_dim, (len(out), head_dim)
    return out


class RotaryEmbedding(nn.Module):
    def __init__(self, head_size: int, rotary_dim: int, max_position_embeddings: int, base: float) -> None:
        super().__init__()
        assert rotary_dim == head_size
        self.head_size = head_size
        inv_freq = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float) / rotary_dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self.attention_scaling = 1.0
        self.register_buffer("modality", None, persistent=False)

    def forward(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor):
        """query [N, heads*hd] or [N, heads, hd]; key likewise.  Returns tensors of the same shape."""
        hd = self.head_size
        q3, k3 = query.view(query.shape[0], -1, hd), key.view(key.shape[0], -1, hd)
        pos = positions
        if pos.dim() == 3:                      # [3, 1, N] as TalkerRotaryEmbedding accepts
            pos = pos[:, 0]
        q, k = nat.qknorm_rope_kvwrite(q3, k3, None, None, None, 0.0, pos, self.inv_freq, modality=self.modality,
                                       attention_scaling=self.attention_scaling)
        return q.view(query.shape), k.view(key.shape)


class TalkerRotaryEmbedding(RotaryEmbedding):
    def __init__(self, head_size, rotary_dim, max_position_embeddings, base, mrope_section, mrope_interleaved=False):
        super().__init__(head_size, rotary_dim, max_position_embeddings, base)
        self.mrope_section = list(mrope_section)
        self.mrope_interleaved = mrope_interleaved
        mod = torch.tensor(mrope_dim_modality(head_size, self.mrope_section, mrope_interleaved), dtype=torch.int32)
        self.modality = mod


def get_rope(head_size: int, rotary_dim: int, max_position: int, base: float, rope_scaling: dict | None = None):
    if rope_scaling and "mrope_section" in rope_scaling:
        return TalkerRotaryEmbedding(head_size, rotary_dim, max_position, base, rope_scaling["mrope_section"],
                                     rope_scaling.get("interleaved", rope_scaling.get("mrope_interleaved", False)))
    return RotaryEmbedding(head_size, rotary_dim, max_position, base)


class PairRotary(nn.Module):
    """Frequencies of a pair rotation (coordinate 2i with 2i+1) of the first ``dims`` coordinates of a vector:
    f_i = base^(-2i/dims).  With ``scaling`` = {factor, original, fast, slow} (YaRN): with
    turns(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(turns(fast)), 0),
    hi = min(ceil(turns(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency is
    f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are multiplied by ``mult`` = 0.1 ln(factor) + 1.
    With ``scaling`` = {factor} alone (linear): f_i / factor, ``mult`` stays 1.
    The table is computed in float64 and kept as float; the kernels that rotate (``nat.latent_prep`` for keys,
    ``nat.latent_attn`` for queries) form the angle position * f_i in float."""

    def __init__(self, dims: int, base: float, scaling: dict | None = None):
        super().__init__()
        import math
        assert dims % 2 == 0
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = torch.as_tensor(float(base), dtype=torch.float64) ** (-2.0 * i / max(dims, 1))
        self.dims, self.mult = dims, 1.0
        if scaling and "original" not in scaling:
            f = f / float(scaling["factor"])
        elif scaling:
            factor, orig = float(scaling["factor"]), float(scaling["original"])
            turns = lambda t: dims * math.log(orig / (2 * math.pi * t)) / (2 * math.log(base))
            lo = max(math.floor(turns(float(scaling["fast"]))), 0)
            hi = min(math.ceil(turns(float(scaling["slow"]))), dims - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
            f = f / factor * ramp + f * (1 - ramp)
            self.mult = 0.1 * math.log(factor) + 1.0
        self.register_buffer("freq", f.to(torch.float32), persistent=False)

    interleaved = True


class HalfRotary(nn.Module):
    """Frequencies of a rotation that pairs coordinate i with i + dims/2 (i < dims/2) of the first ``dims`` coordinates
    of a head: f_i = base^(-2i/dims).  Computed in float64, kept as float; the kernel that rotates
    (``nat.attn_prep``) forms the angle position * f_i in float."""

    def __init__(self, dims: int, base: float):
        super().__init__()
        assert dims % 2 == 0
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = torch.as_tensor(float(base), dtype=torch.float64) ** (-2.0 * i / max(dims, 1))
        self.dims = dims
        self.register_buffer("freq", f.to(torch.float32), persistent=False)

    interleaved = False
