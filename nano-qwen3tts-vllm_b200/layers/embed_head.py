"""``ParallelLMHead`` (layers/embed_head.py:45-66): in prefill only the last token of every
sequence (``cu_seqlens_q[1:] - 1``) reaches the head GEMM."""
import torch
from torch import nn

from .. import _native as nat
from ..utils.context import get_context
from .linear import linear


class ParallelLMHead(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, bias: bool = False):
        super().__init__()
        assert not bias
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ctx = get_context()
        if ctx.is_prefill:
            last = (ctx.cu_seqlens_q[1:] - 1).to(torch.int64)
            x = nat.gather_rows(x, last)
        return linear(x, self.weight)


class TokenPositionEmbedding(nn.Module):
    """Token embedding plus a learned, unscaled position vector, summed in float into a 32-bit residual stream; the
    first layer's norm is applied in the same launch when ``norm`` is given."""

    def __init__(self, vocab: int, max_positions: int, width: int):
        super().__init__()
        self.embed = nn.Parameter(torch.empty(vocab, width), requires_grad=False)
        self.pos = nn.Parameter(torch.empty(max_positions, width), requires_grad=False)

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, norm=None):
        n, width = tokens.shape[0], self.embed.shape[1]
        x = torch.empty(n, width, dtype=torch.float32, device=tokens.device)
        h = torch.empty(n, width, dtype=self.embed.dtype, device=tokens.device) if norm is not None else None
        nat.embed_pos_norm(tokens, positions, self.embed, self.pos, x, h, norm.gain() if norm is not None else None,
                           norm.eps if norm is not None else 0.0)
        return x, h


class ScaledTokenEmbedding(nn.Module):
    """Token embedding times a constant, written as floats into a 32-bit residual stream."""

    def __init__(self, vocab: int, width: int, scale: float):
        super().__init__()
        self.scale = scale
        self.embed = nn.Parameter(torch.empty(vocab, width), requires_grad=False)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        x = torch.empty(tokens.shape[0], self.embed.shape[1], dtype=torch.float32, device=tokens.device)
        nat.embed_scale(tokens, self.embed, self.scale, x)
        return x


class NormedTokenEmbedding(nn.Module):
    """Token embedding followed by a single-gain RMS norm, written as floats into a 32-bit residual stream; the first
    layer's input norm rides in the same launch."""

    def __init__(self, vocab: int, width: int, eps: float = 1e-6):
        super().__init__()
        from .layernorm import GainRMSNorm
        self.embed = nn.Parameter(torch.empty(vocab, width), requires_grad=False)
        self.norm = GainRMSNorm(eps)

    def forward(self, tokens: torch.Tensor, next_norm=None):
        """-> (x [n, width] float, the next sublayer's input in the table's dtype or None)."""
        x = torch.empty(tokens.shape[0], self.embed.shape[1], dtype=torch.float32, device=tokens.device)
        h = nat.sandwich_residual(x, self.norm.gain(), a=self.embed, a_index=tokens, init=True, eps=self.norm.eps,
                                  g_in=next_norm.gain() if next_norm is not None else None)
        return x, h


class BigramTokenEmbedding(nn.Module):
    """Token embedding plus a row of a hashed bigram table, row (previous token * mul_prev + token * mul_cur) mod
    ``buckets`` (the table's extra last row for a sequence's first token), written as floats into every one of
    ``streams`` residual streams [n, streams, width].  ``buckets`` 0: no bigram table."""

    def __init__(self, vocab: int, width: int, streams: int, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0):
        super().__init__()
        self.streams, self.buckets, self.mul_prev, self.mul_cur = streams, buckets, mul_prev, mul_cur
        self.embed = nn.Parameter(torch.empty(vocab, width), requires_grad=False)
        self.bigram = nn.Parameter(torch.empty(buckets + 1, width), requires_grad=False) if buckets else None

    def forward(self, tokens: torch.Tensor, prev_tokens: torch.Tensor) -> torch.Tensor:
        xs = torch.empty(tokens.shape[0], self.streams, self.embed.shape[1], dtype=torch.float32, device=tokens.device)
        nat.embed_bigram_streams(tokens, prev_tokens, self.embed, self.bigram, xs, self.buckets, self.mul_prev, self.mul_cur)
        return xs
