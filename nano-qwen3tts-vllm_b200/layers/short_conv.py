"""Short causal convolution over time on the channels of a merged q|k|v projection, with the state it carries from
step to step (the last ``taps - 1`` projections of every live sequence, one slot per sequence).

The convolution is fused with what follows it in the attention mixer: the per-head RMS norm of q and k and the write
of k and v into the paged cache (``b2tts_conv_headnorm_kvwrite``), as the rotary models of this package fuse
head norm, rotation and cache write.  Weights are float [channels, taps]; tap ``taps - 1`` multiplies the token itself."""
import torch
from torch import nn

from .. import _native as nat
from ..utils.context import get_context


class ShortConvQKV(nn.Module):
    def __init__(self, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float):
        super().__init__()
        self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.eps = heads, kv_heads, dim, vdim, taps, eps
        channels = heads * dim + kv_heads * (dim + vdim)
        f32 = dict(dtype=torch.float32)
        self.weight = nn.Parameter(torch.zeros(channels, taps, **f32), requires_grad=False)
        self.q_norm = nn.Parameter(torch.ones(dim, **f32), requires_grad=False)
        self.k_norm = nn.Parameter(torch.ones(dim, **f32), requires_grad=False)
        self.state = None                      # [slots, taps - 1, channels], bound by the model runner

    def forward(self, u: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> torch.Tensor:
        """u [n, channels] -> q [n, heads * dim] (convolved and normed); k, v go to their cache slots; the state of
        every sequence in the step advances."""
        lay = get_context().step_layout
        q = torch.empty(u.shape[0], self.heads * self.dim, dtype=u.dtype, device=u.device)
        nat.conv_headnorm_kvwrite(u, self.weight, self.state, lay, self.q_norm, self.k_norm, q, k_cache, v_cache,
                                  self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.eps)
        return q


F32 = dict(dtype=torch.float32)


class ShortConvAct(nn.Module):
    """Causal convolution over time, one filter of ``taps`` numbers per channel (the last tap multiplies the token
    itself), optional bias, then SiLU.  The last ``taps - 1`` inputs of every live sequence are its carried state."""

    def __init__(self, channels: int, taps: int, bias: bool):
        super().__init__()
        self.channels, self.taps = channels, taps
        self.weight = nn.Parameter(torch.zeros(channels, taps, **F32), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(channels, **F32), requires_grad=False) if bias else None
        self.state = None                      # [slots, max(taps - 1, 1), channels] in the activation type

    def state_plan(self):
        return ((max(self.taps - 1, 1), self.channels), None)

    def forward(self, u: torch.Tensor, c_off: int) -> torch.Tensor:
        out = torch.empty(u.shape[0], self.channels, dtype=u.dtype, device=u.device)
        nat.short_conv_act(u, c_off, self.channels, self.weight, self.bias, self.state, get_context().step_layout, out, self.taps, 1)
        return out
