"""``Silu`` (layers/activation.py:7-13) and the gated product of the MLP
(models/qwen3_tts_share.py:131-135) as one kernel over a fused gate_up tensor."""
import torch
from torch import nn

from .. import _native as nat


class Silu(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return nat.silu_and_mul(x, None)


class SiluAndMul(nn.Module):
    """x = [gate | up] along the last dim (the output of a merged gate_up projection)."""

    def __init__(self, rounding: int = nat.ROUND_EAGER):
        super().__init__()
        self.rounding = rounding

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        inter = x.shape[-1] // 2
        x2 = x.view(-1, x.shape[-1])
        out = nat.silu_and_mul(x2[:, :inter], x2[:, inter:], self.rounding)
        return out.view(*x.shape[:-1], inter)


class ReluSquared(nn.Module):
    """max(x, 0)^2, in place (bf16 or float32)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return nat.relu_sq_(x)


class XIELU(nn.Module):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2, with two learned numbers
    (p, q) kept in float; in place, a bias may be added first (in float, before the activation)."""

    def __init__(self):
        super().__init__()
        self.pq = nn.Parameter(torch.zeros(2, dtype=torch.float32), requires_grad=False)

    def forward(self, y: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        return nat.xielu_(y, bias, self.pq)


class PolyNorm(nn.Module):
    """a N(z) + b N(z^2) + c N(z^3) + e with four learned numbers kept in float; powers element by element, N divides a
    row by its root mean square (eps inside the root); in place."""

    def __init__(self, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.coef = nn.Parameter(torch.zeros(4, dtype=torch.float32), requires_grad=False)

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        return nat.polynorm_(y, self.coef, self.eps)


class GatedSilu(nn.Module):
    """[gate | up] along the last axis -> silu(gate) * up (bf16 or float32)."""

    def forward(self, gu: torch.Tensor) -> torch.Tensor:
        return nat.silu_mul(gu)
