"""Recurrent token mixers with a matrix state per head (``nat.ssm_scan``, ``nat.matrix_memory_scan``,
``nat.delta_rule_scan``): the state lives in float in one slot per live sequence, starts at zero at position 0 and is
carried from step to step, so prompt portions and single decoded tokens run through the same launch.

Each module owns the per-head constants of its recurrence and the gate + norm that follows it, and reads its inputs as
column ranges of the mixer's merged input projection ``u`` (``cols``: name -> first column).  ``bind(state)`` receives
the tensors the model runner allocated from ``state_plan()``."""
import torch
from torch import nn

from .. import _native as nat
from ..utils.context import get_context
from .short_conv import ShortConvAct

F32 = dict(dtype=torch.float32)


class StateSpaceMemory(nn.Module):
    """u = [z | x | B | C | dt]: x, B, C pass the short convolution and SiLU; dt = softplus(dt + dt_bias);
    S <- exp(-exp(A_log) dt) S + dt B x^T; y = S^T C + D x; then y * silu(z), RMS norm in ``norm_groups`` parts, weight."""

    def __init__(self, spec, eps: float):
        super().__init__()
        m = self.spec = spec
        self.eps = eps
        self.conv = ShortConvAct(m.conv_channels, m.conv, bias=True)
        self.dt_bias = nn.Parameter(torch.zeros(m.heads, **F32), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(m.heads, **F32), requires_grad=False)
        self.D = nn.Parameter(torch.zeros(m.heads, **F32), requires_grad=False)
        self.norm = nn.Parameter(torch.ones(m.inner, **F32), requires_grad=False)
        self.S = None

    def proj_parts(self):
        m = self.spec
        return [("in", 2 * m.inner + 2 * m.groups * m.state + m.heads)]

    def state_plan(self):
        m = self.spec
        return [self.conv.state_plan(), ((m.heads, m.state, m.vdim), torch.float32)]

    def bind(self, state):
        self.conv.state, self.S = state

    def forward(self, u: torch.Tensor, cols: dict) -> torch.Tensor:
        m, lay = self.spec, get_context().step_layout
        base = cols["in"]
        xbc = self.conv(u, base + m.inner)
        dt0 = base + m.inner + m.conv_channels
        y = torch.empty(u.shape[0], m.inner, dtype=torch.float32, device=u.device)
        nat.ssm_scan(xbc, u[:, dt0:dt0 + m.heads], self.dt_bias, self.A_log, self.D, self.S, y, lay, m.heads, m.groups, m.vdim, m.state)
        out = torch.empty(u.shape[0], m.inner, dtype=u.dtype, device=u.device)
        nat.gated_group_norm(y, u[:, base:base + m.inner], self.norm, m.norm_groups, nat.GATE_SILU, True, self.eps, out)
        return out


class MatrixMemory(nn.Module):
    """Matrix memory with exponential gates and a running maximum; each head's read-out is divided by its root mean
    square, then weight and sigmoid gate."""

    def __init__(self, spec, eps: float):
        super().__init__()
        m = self.spec = spec
        self.eps = eps
        self.i_bias = nn.Parameter(torch.zeros(m.heads, **F32), requires_grad=False)
        self.f_bias = nn.Parameter(torch.zeros(m.heads, **F32), requires_grad=False)
        self.norm = nn.Parameter(torch.ones(m.heads * m.vdim, **F32), requires_grad=False)
        self.S = self.nm = None

    def proj_parts(self):
        m = self.spec
        return [("q", m.heads * m.dim), ("k", m.heads * m.dim), ("v", m.heads * m.vdim), ("g", m.heads * m.vdim),
                ("i", m.heads), ("f", m.heads)]

    def state_plan(self):
        m = self.spec
        return [((m.heads, m.dim, m.vdim), torch.float32), ((m.heads, m.dim + 1), torch.float32)]

    def bind(self, state):
        self.S, self.nm = state

    def forward(self, u: torch.Tensor, cols: dict) -> torch.Tensor:
        m, lay = self.spec, get_context().step_layout
        n, hd, hv = u.shape[0], m.heads * m.dim, m.heads * m.vdim
        cut = lambda name, w: u[:, cols[name]:cols[name] + w]
        gates = torch.empty(n, m.heads, 3, dtype=torch.float32, device=u.device)
        o = torch.empty(n, hv, dtype=torch.float32, device=u.device)
        nat.matrix_memory_scan(cut("q", hd), cut("k", hd), cut("v", hv), cut("i", m.heads), cut("f", m.heads), self.i_bias,
                               self.f_bias, m.gate_cap, self.S, self.nm, gates, o, lay, m.heads, m.dim, m.vdim)
        out = torch.empty(n, hv, dtype=u.dtype, device=u.device)
        nat.gated_group_norm(o, cut("g", hv), self.norm, m.heads, nat.GATE_SIGMOID, False, self.eps, out)
        return out


class DeltaRuleMemory(nn.Module):
    """Gated delta rule: q, k, v pass a short convolution and SiLU, q and k become unit vectors, one decay and one
    write strength per head; each head's read-out is RMS-normed with a weight shared by the heads, then a SiLU gate."""

    def __init__(self, spec, eps: float):
        super().__init__()
        m = self.spec = spec
        self.eps = eps
        self.channels = 2 * m.kv_heads * m.dim + m.heads * m.vdim
        self.conv = ShortConvAct(self.channels, m.conv, bias=False)
        self.A_log = nn.Parameter(torch.zeros(m.heads, **F32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(m.heads, **F32), requires_grad=False)
        self.norm = nn.Parameter(torch.ones(m.vdim, **F32), requires_grad=False)
        self.S = None

    def proj_parts(self):
        m = self.spec
        return [("q", m.kv_heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.heads * m.vdim), ("g", m.heads * m.vdim),
                ("b", m.heads), ("a", m.heads)]

    def state_plan(self):
        m = self.spec
        return [self.conv.state_plan(), ((m.heads, m.dim, m.vdim), torch.float32)]

    def bind(self, state):
        self.conv.state, self.S = state

    def forward(self, u: torch.Tensor, cols: dict) -> torch.Tensor:
        m, lay = self.spec, get_context().step_layout
        n, hv = u.shape[0], m.heads * m.vdim
        qkv = self.conv(u, cols["q"])                                            # q | k | v are adjacent columns of u
        o = torch.empty(n, hv, dtype=torch.float32, device=u.device)
        nat.delta_rule_scan(qkv, u[:, cols["b"]:cols["b"] + m.heads], u[:, cols["a"]:cols["a"] + m.heads], self.A_log, self.dt_bias,
                            self.S, o, lay, m.heads, m.kv_heads, m.dim, m.vdim)
        out = torch.empty(n, hv, dtype=u.dtype, device=u.device)
        nat.gated_group_norm(o, u[:, cols["g"]:cols["g"] + hv], self.norm, m.heads, nat.GATE_SILU, False, self.eps, out)
        return out


class GatedLinearAttention(nn.Module):
    """Gated linear attention: S <- diag(alpha) S + k v^T, o = S^T q per head, q scaled by dim^(-1/2), with one decay per
    key channel and token alpha = sigmoid(W_a2 (W_a1 h) + b)^(1/tau).  The first step of the decay projection rides in
    the mixer's merged input projection (part ``a1``), the second is a small GEMM of this module; bias, logsigmoid,
    the division by tau and the exponential are float.  Each head's read-out is RMS-normed with a weight shared by the
    heads, then multiplied by silu(W_g h)."""

    def __init__(self, spec, eps: float):
        super().__init__()
        m = self.spec = spec
        assert m.decay_rank > 0, "the decay projection's inner size is unknown (read it from the checkpoint's tensor shapes)"
        self.eps = eps
        self.a2 = nn.Parameter(torch.empty(m.heads * m.dim, m.decay_rank), requires_grad=False)
        self.a2_bias = nn.Parameter(torch.zeros(m.heads * m.dim, **F32), requires_grad=False)
        self.norm = nn.Parameter(torch.ones(m.vdim, **F32), requires_grad=False)
        self.S = None

    def proj_parts(self):
        m = self.spec
        return [("q", m.heads * m.dim), ("k", m.heads * m.dim), ("v", m.heads * m.vdim), ("g", m.heads * m.vdim), ("a1", m.decay_rank)]

    def state_plan(self):
        m = self.spec
        return [((m.heads, m.dim, m.vdim), torch.float32)]

    def bind(self, state):
        (self.S,) = state

    def forward(self, u: torch.Tensor, cols: dict) -> torch.Tensor:
        from .linear import linear
        m, lay = self.spec, get_context().step_layout
        n, hd, hv = u.shape[0], m.heads * m.dim, m.heads * m.vdim
        cut = lambda name, w: u[:, cols[name]:cols[name] + w]
        z = linear(cut("a1", m.decay_rank).contiguous(), self.a2)
        o = torch.empty(n, hv, dtype=torch.float32, device=u.device)
        nat.gated_linear_scan(cut("q", hd), cut("k", hd), cut("v", hv), z, self.a2_bias, m.tau, self.S, o, lay, m.heads, m.dim, m.vdim)
        out = torch.empty(n, hv, dtype=u.dtype, device=u.device)
        nat.gated_group_norm(o, cut("g", hv), self.norm, m.heads, nat.GATE_SILU, False, self.eps, out)
        return out
