"""``Qwen3TTSRMSNorm`` (layers/layernorm.py:7-53 of the reference) on libb200tts.

``forward(x)`` -> y;  ``forward(x, residual)`` -> (y, residual + x) with the reference's
add_rms_forward semantics (fp32 sum feeds the norm, layernorm.py:35-38)."""
import torch
from torch import nn

from .. import _native as nat


class Qwen3TTSRMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, rounding: int = nat.ROUND_EAGER) -> None:
        super().__init__()
        self.eps = eps
        self.rounding = rounding
        self.weight = nn.Parameter(torch.ones(hidden_size), requires_grad=False)

    def rms_forward(self, x: torch.Tensor) -> torch.Tensor:
        return nat.rmsnorm(x, self.weight, self.eps, self.rounding)

    def add_rms_forward(self, x: torch.Tensor, residual: torch.Tensor):
        return nat.add_rmsnorm(x, residual, self.weight, self.eps, self.rounding, round_sum_first=False)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        if residual is None:
            return self.rms_forward(x)
        return self.add_rms_forward(x, residual)


class GainRMSNorm(nn.Module):
    """RMS norm with ONE learned gain for all coordinates, over a 32-bit residual stream:
    y = x / sqrt(mean(x^2) + eps) * g.  The gain is kept in float; the output takes the activation dtype.
    In a model the norm rides in the kernel that produces x (``nat.embed_pos_norm`` / ``nat.residual_norm``);
    ``forward`` is the stand-alone form, optionally over a subset of rows."""

    def __init__(self, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones((), dtype=torch.float32), requires_grad=False)

    def gain(self) -> torch.Tensor:
        return self.weight.view(1)

    def forward(self, x: torch.Tensor, dtype: torch.dtype, rows: torch.Tensor | None = None) -> torch.Tensor:
        return nat.gather_gain_norm(x, rows, self.gain(), self.eps, dtype)


class SandwichNorm(nn.Module):
    """The pair of single-gain RMS norms around a sublayer whose output is normed before it joins a 32-bit residual
    stream: ``self.pre`` on the way in, ``self.post`` on the way out.  ``add`` does x += post(y) and returns the NEXT
    sublayer's input ``nxt.pre(x)`` from the same launch (``nat.sandwich_residual``).  y is a dense output ``a``; two
    branch outputs ``a``, ``b`` that are first RMS-normed over the row with weight vectors ``wa``, ``wb`` and summed with
    ``branch_scale``; or per-choice expert outputs ``z`` with weights ``zw``, where choices ``z_idx`` >= ``n_real`` stand
    for identity experts and contribute the sublayer's input ``hin``."""

    def __init__(self, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.pre, self.post = GainRMSNorm(eps), GainRMSNorm(eps)

    def add(self, x: torch.Tensor, nxt: "GainRMSNorm | None", **y) -> torch.Tensor | None:
        return nat.sandwich_residual(x, self.post.gain(), g_in=nxt.gain() if nxt is not None else None, eps=self.eps, **y)


class GroupRMSNorm(nn.Module):
    """RMS norm in groups: the vector is cut into ``groups`` equal consecutive parts, each divided by its own
    sqrt(mean(part^2) + eps), the whole multiplied by a weight vector (kept in float).  In a model it sits on a
    sublayer's OUTPUT and rides in the residual update: ``add_to`` does x += norm(y) on a 32-bit stream, with y a
    dense output ``a`` and / or the weighted sum of per-choice expert outputs ``z`` (weights ``zw``).  ``forward`` is
    the stand-alone form over a subset of rows (the final norm before the head)."""

    def __init__(self, width: int, groups: int = 1, eps: float = 1e-6):
        super().__init__()
        assert width % groups == 0
        self.groups, self.eps = groups, eps
        self.weight = nn.Parameter(torch.ones(width, dtype=torch.float32), requires_grad=False)

    def add_to(self, x: torch.Tensor, a=None, z=None, zw=None, copy_dtype: torch.dtype | None = None, dtype=None):
        """x [n, width] float, updated in place.  Returns the new x in ``copy_dtype`` (or None)."""
        dtype = dtype or (a.dtype if a is not None else z.dtype)
        copy = torch.empty(x.shape, dtype=copy_dtype, device=x.device) if copy_dtype is not None else None
        nat.group_norm_residual(x, a, z, zw, self.weight, self.groups, self.eps, copy, dtype)
        return copy

    def forward(self, x: torch.Tensor, dtype: torch.dtype, rows: torch.Tensor | None = None) -> torch.Tensor:
        return nat.gather_group_norm(x, rows, self.weight, self.groups, self.eps, dtype)


class StreamRMSNorm(nn.Module):
    """RMS norm with a weight vector kept in float, applied to what is read out of the residual streams: it rides in
    the stream kernels (``layers/hyper_connection.step``); ``forward`` is the stand-alone form on the sum of the streams
    of gathered rows (the final norm in front of the head)."""

    def __init__(self, width: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(width, dtype=torch.float32), requires_grad=False)

    def forward(self, xs: torch.Tensor, dtype: torch.dtype, rows: torch.Tensor | None = None) -> torch.Tensor:
        return nat.stream_gather_norm(xs, rows, None, self.weight, self.eps, dtype)
