"""Mixture-of-experts feed-forwards with a top-k router.

Router scores are computed in float.  Three routers: sigmoid scores, the chosen ones divided by their sum (+ 1e-20)
times ``scale``; logits (plus a bias) whose chosen ones are soft-maxed among themselves; or a softmax over all router
outputs, chosen by score + correction and weighted by the score itself, whose last ``identity`` outputs stand for experts
that return their input.  Two experts: two matrices
with a squared ReLU, or three with a SiLU gate.  Experts are stored stacked ([experts, ff or 2 ff, width] /
[experts, width, ff]) so that ONE grouped launch runs all of them over the (token, choice) pairs sorted by expert -
for a prompt portion of thousands of tokens and for a decode step of a few rows per expert alike, with no group size
ever read back to the host.  ``forward`` returns the per-pair outputs and weights; the weighted sum over a token's
choices is taken, in a fixed order, by the residual kernel that consumes them."""
import torch
from torch import nn

from .. import _native as nat


class TopKMoE(nn.Module):
    """The shared machinery: route, group by expert, two grouped launches.  ``router_kind`` "sigmoid" (scores divided
    by the sum of the chosen, times ``scale``) or "softmax_chosen" (logits plus an optional bias; weights are the
    softmax over the chosen logits only).  ``gated``: an expert is W_down (silu(W_gate h) * (W_up h)) with gate and up
    stacked in one [experts, 2 ff, width] tensor; otherwise W_down relu(W_up h)^2."""

    ROUTES = {"sigmoid": nat.ROUTE_SIGMOID, "softmax_chosen": nat.ROUTE_SOFTMAX_CHOSEN, "softmax_all": nat.ROUTE_SOFTMAX_ALL}

    def __init__(self, width: int, ff: int, experts: int, top: int, scale: float = 1.0, router_kind: str = "sigmoid",
                 router_bias: bool = False, gated: bool = False, identity: int = 0):
        super().__init__()
        assert router_kind in self.ROUTES
        self.width, self.ff, self.experts, self.top, self.scale = width, ff, experts, top, scale
        self.router_kind, self.gated, self.identity = router_kind, gated, identity
        # the router has one output per expert and per identity expert; only the former have matrices and reach the
        # grouped launches (the groups of the latter lie behind offsets[experts])
        self.router = nn.Parameter(torch.zeros(experts + identity, width, dtype=torch.float32), requires_grad=False)
        if router_bias:
            self.router_bias = nn.Parameter(torch.zeros(experts + identity, dtype=torch.float32), requires_grad=False)
        else:
            self.register_parameter("router_bias", None)
        self.up = nn.Parameter(torch.empty(experts, (2 if gated else 1) * ff, width), requires_grad=False)
        self.down = nn.Parameter(torch.empty(experts, width, ff), requires_grad=False)

    def route(self, h: torch.Tensor):
        n, dev = h.shape[0], h.device
        top_idx = torch.empty(n, self.top, dtype=torch.int32, device=dev)
        top_w = torch.empty(n, self.top, dtype=torch.float32, device=dev)
        offsets = torch.empty(self.experts + self.identity + 1, dtype=torch.int32, device=dev)
        sorted_pair = torch.empty(n * self.top, dtype=torch.int32, device=dev)
        nat.moe_route(h, self.router, top_idx, top_w, offsets, sorted_pair, self.top, self.scale, bias=self.router_bias,
                      mode=self.ROUTES[self.router_kind])
        return top_idx, top_w, offsets, sorted_pair

    def forward(self, h: torch.Tensor):
        """h [n, width] -> (z [n * top, width], weights [n, top]): z[t * top + k] is the output of token t's k-th expert."""
        n = h.shape[0]
        pairs = n * self.top
        top_idx, top_w, offsets, sorted_pair = self.route(h)
        self.last_choice = top_idx                      # with identity experts the consumer needs to know which pairs they are
        if self.gated:
            gu = torch.empty(pairs, 2 * self.ff, dtype=h.dtype, device=h.device)
            nat.grouped_gemm(h, self.up, gu, offsets, sorted_pair, pairs, self.top, in_by_token=True, out_by_pair=False, act=0)
            y = nat.silu_mul(gu)
        else:
            y = torch.empty(pairs, self.ff, dtype=h.dtype, device=h.device)
            nat.grouped_gemm(h, self.up, y, offsets, sorted_pair, pairs, self.top, in_by_token=True, out_by_pair=False, act=1)
        z = torch.empty(pairs, self.width, dtype=h.dtype, device=h.device)
        nat.grouped_gemm(y, self.down, z, offsets, sorted_pair, pairs, self.top, in_by_token=False, out_by_pair=True, act=0)
        return z, top_w


class SoftmaxIdentityMoE(TopKMoE):
    """Router scores softmax(W_r h) over ``experts`` + ``identity`` outputs in float; the ``top`` largest of score +
    correction are chosen; the weights are the chosen scores, not renormalised; gated SiLU experts.  The rows of ``z`` that
    belong to identity experts are not written: the consumer reads ``last_choice`` and substitutes its input."""

    def __init__(self, width: int, ff: int, experts: int, top: int, identity: int):
        super().__init__(width, ff, experts, top, 1.0, "softmax_all", True, True, identity)


class SigmoidTopKMoE(TopKMoE):
    def __init__(self, width: int, ff: int, experts: int, top: int, scale: float):
        super().__init__(width, ff, experts, top, scale, "sigmoid", False, False)


class SoftmaxTopKGatedMoE(TopKMoE):
    """Router logits W_r h + b in float, the ``top`` largest chosen, weights = softmax over the chosen; gated SiLU experts."""

    def __init__(self, width: int, ff: int, experts: int, top: int):
        super().__init__(width, ff, experts, top, 1.0, "softmax_chosen", True, True)
