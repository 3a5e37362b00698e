"""``store_kvcache`` and ``Attention`` with the reference's surface (layers/attention.py:33-96):
``Attention(num_heads, head_dim, scale, num_kv_heads)`` owns ``k_cache`` / ``v_cache`` (empty until
the model runner binds views of the paged pool, base.py:160-164) and ``forward(q, k, v)`` reads the
batch layout from the global Context."""
import torch
from torch import nn

from .. import _native as nat
from ..utils.context import get_context


def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping: torch.Tensor) -> None:
    n, num_heads, head_dim = key.shape
    d = num_heads * head_dim
    assert key.stride(-1) == 1 and value.stride(-1) == 1
    assert key.stride(1) == head_dim and value.stride(1) == head_dim
    assert k_cache.stride(1) == d and v_cache.stride(1) == d
    assert slot_mapping.numel() == n
    nat.store_kvcache(key, value, k_cache, v_cache, slot_mapping)


class Attention(nn.Module):
    def __init__(self, num_heads, head_dim, scale, num_kv_heads):
        super().__init__()
        self.num_heads, self.head_dim, self.scale, self.num_kv_heads = num_heads, head_dim, scale, num_kv_heads
        self.k_cache = self.v_cache = torch.tensor([])
        self.workspace = None                     # split-KV scratch, bound by the runner
        self.fused_workspace = None               # zero-filled scratch of the fused decode kernel, bound by the runner

    def attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor | None = None):
        """Attention only (the KV rows of this step are already in the cache)."""
        ctx = get_context()
        if ctx.is_prefill:
            if ctx.block_tables is not None:      # prefix-cache hit: read K/V through the block table
                return nat.varlen_attn_prefill(q, self.k_cache, self.v_cache, ctx.cu_seqlens_q, ctx.cu_seqlens_k,
                                               ctx.max_seqlen_q, ctx.max_seqlen_k, self.scale,
                                               block_table=ctx.block_tables, out=out)
            return nat.varlen_attn_prefill(q, k, v, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.max_seqlen_q,
                                           ctx.max_seqlen_k, self.scale, out=out)
        max_ctx = ctx.max_context_len or ctx.block_tables.shape[1] * self.k_cache.shape[1]
        return nat.paged_attn_decode(q, self.k_cache, self.v_cache, ctx.block_tables, ctx.context_lens, self.scale,
                                     max_ctx, out=out, workspace=self.workspace)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        ctx = get_context()
        if self.k_cache.numel() and self.v_cache.numel():
            store_kvcache(k, v, self.k_cache, self.v_cache, ctx.slot_mapping)
        return self.attend(q, k, v)


class WindowSigmoidAttention(nn.Module):
    """Sliding-window attention whose weights are sigmoids of the biased score, not a softmax:

        w(i, j) = sigmoid(q_i . k_j * scale - r1_h * ln(1 + r2_h * (i - j)) + pb_h)    for 0 <= i - j < window

    The cache holds this step's keys already (the convolution kernel wrote them), so prompt portions and decoded
    tokens run through the same launch; the step's layout comes from the global Context.  ``r1``, ``r2``, ``pb`` are
    per-head floats.  ``k_cache`` [pages, page, kv_heads * dim] and ``v_cache`` [pages, page, kv_heads * vdim] are bound
    by the model runner."""

    def __init__(self, heads: int, kv_heads: int, dim: int, vdim: int, window: int, scale: float):
        super().__init__()
        self.heads, self.kv_heads, self.dim, self.vdim, self.window, self.scale = heads, kv_heads, dim, vdim, window, scale
        f32 = dict(dtype=torch.float32)
        self.r1 = nn.Parameter(torch.zeros(heads, **f32), requires_grad=False)
        self.r2 = nn.Parameter(torch.zeros(heads, **f32), requires_grad=False)
        self.pb = nn.Parameter(torch.zeros(heads, **f32), requires_grad=False)
        self.k_cache = self.v_cache = torch.tensor([])

    def forward(self, q: torch.Tensor) -> torch.Tensor:
        lay = get_context().step_layout
        out = torch.empty(q.shape[0], self.heads * self.vdim, dtype=q.dtype, device=q.device)
        nat.window_sigmoid_attn(q, self.k_cache, self.v_cache, out, lay, self.r1, self.r2, self.pb, self.heads,
                                self.kv_heads, self.dim, self.vdim, self.k_cache.shape[1], self.window, self.scale)
        return out


class LatentSinkAttention(nn.Module):
    """Softmax attention over a paged cache of latents, with a learned per-head sink in the denominator.

    A cached row is [c | kr]: the normed key/value latent (``kv_rank``) and the rotated key part all heads share
    (``rot_dim``).  Head h's key is [W_uk,h c | kr], its value W_uv,h c.  Neither is materialised: the caller hands in
    queries already multiplied by W_uk,h^T (``ql`` [heads, n, kv_rank]) and gets back the attention-weighted sums of
    latents ([heads, n, kv_rank]), to which it applies W_uv,h.  ``window`` 0 = causal without a window.  The cache holds
    this step's rows already (``nat.latent_prep`` wrote them), so prompt portions and decoded tokens run in one launch."""

    def __init__(self, heads: int, kv_rank: int, rot_dim: int, window: int, scale: float, rotary):
        super().__init__()
        self.heads, self.kv_rank, self.rot_dim, self.window, self.scale, self.rotary = heads, kv_rank, rot_dim, window, scale, rotary
        self.sink = nn.Parameter(torch.zeros(heads, dtype=torch.float32), requires_grad=False)
        self.path = nat.LATENT_ATTN_AUTO

    def forward(self, ql: torch.Tensor, qr: torch.Tensor, qr_strides, cache: torch.Tensor) -> torch.Tensor:
        """ql [heads, n, kv_rank] contiguous; qr: any tensor whose element (t, h, :rot_dim) lies at
        t * qr_strides[0] + h * qr_strides[1] (the rotary query parts, not yet rotated)."""
        lay = get_context().step_layout
        n = ql.shape[1]
        out = torch.empty_like(ql)
        nat.latent_attn(ql, (self.kv_rank, n * self.kv_rank), qr, qr_strides, cache, out, (self.kv_rank, n * self.kv_rank),
                        self.sink, self.rotary.freq, self.rotary.mult, self.rotary.dims, lay, self.heads, self.kv_rank,
                        self.rot_dim, cache.shape[1], self.window, self.scale, self.path)
        return out


class SinkSoftmaxAttention(nn.Module):
    """Softmax attention over paged K/V with a learned per-head sink in the denominator (it has no key and no value and
    is not scaled), under a sliding window (``mask_kind`` "window": the token itself and the ``mask`` - 1 before it) or
    chunks (``"chunk"``: earlier tokens of the same block of ``mask`` positions, counted from position 0).

    ``prepare`` turns the mixer's merged projection into queries and cache rows: optional biases, optional RMS norm over
    the whole q and the whole k projection, optional half-split rotation; the values are a projection of their own or,
    with ``v_off`` < 0, the keys as projected.  ``forward`` attends; an optional per-head sigmoid gate rides in the same
    launch.  The cache holds this step's keys already, so prompt portions and decoded tokens share the launch.

    Further switches: ``sink`` "learned" (a parameter per head), "zero" (the denominator gets exp(0) = 1: the parameter
    stays zero and is not part of a checkpoint) or "none" (an ordinary softmax); ``softcap`` c > 0 turns a scaled score s
    into c tanh(s / c); ``keep_first`` keys stay visible behind the mask; ``mask`` 0 is plain causal attention; the
    rotation pairs coordinate i with i + dims/2 or 2i with 2i + 1 as the ``rotary`` module says; ``v_heads`` < ``kv_heads``
    value heads are shared by the key heads (key head g reads value head g mod v_heads); ``own_cache`` False: the
    module projects no keys and values and reads a cache another module writes."""

    MASKS = {"window": nat.MASK_WINDOW, "chunk": nat.MASK_CHUNK}

    def __init__(self, heads: int, kv_heads: int, dim: int, vdim: int, mask_kind: str, mask: int, scale: float, *,
                 bias: bool = False, qk_norm: bool = False, rotary=None, eps: float = 1e-6, sink: str = "learned",
                 softcap: float = 0.0, keep_first: int = 0, v_heads: int | None = None, own_cache: bool = True):
        super().__init__()
        assert sink in ("learned", "zero", "none")
        self.heads, self.kv_heads, self.dim, self.vdim, self.scale, self.eps = heads, kv_heads, dim, vdim, scale, eps
        self.mask_kind, self.mask, self.rotary = self.MASKS[mask_kind], mask, rotary
        self.softcap, self.keep_first, self.v_heads, self.own_cache = softcap, keep_first, v_heads or kv_heads, own_cache
        f32 = dict(dtype=torch.float32)
        self.sink = nn.Parameter(torch.zeros(heads, **f32), requires_grad=False) if sink != "none" else None
        mk = lambda n, one: nn.Parameter((torch.ones if one else torch.zeros)(n, **f32), requires_grad=False)
        self.q_bias = mk(heads * dim, False) if bias else None
        self.k_bias = mk(kv_heads * dim, False) if bias else None
        self.v_bias = mk(kv_heads * vdim, False) if bias else None
        self.q_norm = mk(heads * dim, True) if qk_norm else None
        self.k_norm = mk(kv_heads * dim, True) if qk_norm else None
        self.k_cache = self.v_cache = torch.tensor([])

    def prepare(self, u: torch.Tensor, q_off: int, k_off: int, v_off: int) -> torch.Tensor:
        lay = get_context().step_layout
        q = torch.empty(u.shape[0], self.heads * self.dim, dtype=u.dtype, device=u.device)
        rot = self.rotary
        own = self.own_cache
        nat.attn_prep(u, q_off, k_off, v_off, self.q_bias, self.k_bias, self.v_bias if v_off >= 0 else None, self.q_norm,
                      self.k_norm, rot.freq if rot is not None else None, rot.dims if rot is not None else 0, lay, q,
                      self.k_cache if own else None, self.v_cache if own else None, self.heads, self.kv_heads, self.dim,
                      self.vdim, self.eps, interleaved=rot is not None and rot.interleaved, v_heads=self.v_heads)
        return q

    def forward(self, q: torch.Tensor, gate: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """``out_dtype`` float32 beside bfloat16 inputs: the heads' outputs are returned unrounded."""
        lay = get_context().step_layout
        out = torch.empty(q.shape[0], self.heads * self.vdim, dtype=out_dtype or q.dtype, device=q.device)
        nat.sink_attn(q, self.k_cache, self.v_cache, out, lay, self.sink, gate, self.heads, self.kv_heads, self.dim, self.vdim,
                      self.k_cache.shape[1], self.mask_kind, self.mask, self.scale, v_heads=self.v_heads,
                      keep_first=self.keep_first, softcap=self.softcap)
        return out


class DifferentialAttention(SinkSoftmaxAttention):
    """Two softmax maps per head over the same values, combined as map 1 - lambda * map 2, each head's result divided by
    its root mean square and multiplied by ``1 - diff``; lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff is one number per
    layer.  The maps run as ``2 * heads`` query heads over ``2 * kv_heads`` key heads that share ``kv_heads`` value heads;
    queries and keys are expected MAP-MAJOR (all heads of map 1, then all heads of map 2), which makes the grouping of
    query heads over key heads the ordinary one: a model permutes the projection's rows once when it loads them
    (``map_major``).  No positions enter; the mask is causal, a sliding window, optionally with kept first keys."""

    def __init__(self, heads: int, kv_heads: int, dim: int, vdim: int, window: int, keep_first: int, scale: float, diff: float,
                 eps: float = 1e-6, own_cache: bool = True):
        super().__init__(2 * heads, 2 * kv_heads, dim, vdim, "window", window, scale, eps=eps, sink="none", keep_first=keep_first,
                         v_heads=kv_heads, own_cache=own_cache)
        self.out_heads, self.diff = heads, diff
        f32 = dict(dtype=torch.float32)
        for name in ("lq1", "lk1", "lq2", "lk2"):
            setattr(self, name, nn.Parameter(torch.zeros(dim, **f32), requires_grad=False))
        self._lam = None

    @staticmethod
    def map_major(w: torch.Tensor, heads: int, dim: int) -> torch.Tensor:
        """Rows [head][map][dim] of a q or k projection -> [map][head][dim]."""
        return w.reshape(heads, 2, dim, -1).transpose(0, 1).reshape(w.shape)

    def lam(self) -> float:
        """lambda in float, computed once from the loaded vectors."""
        if self._lam is None:
            a = torch.exp((self.lq1.float() * self.lk1.float()).sum()) - torch.exp((self.lq2.float() * self.lk2.float()).sum())
            self._lam = float(a.item() + self.diff)
        return self._lam

    def forward(self, q: torch.Tensor) -> torch.Tensor:
        maps = super().forward(q, out_dtype=torch.float32)       # the difference is taken before anything is rounded
        out = torch.empty(q.shape[0], self.out_heads * self.vdim, dtype=q.dtype, device=q.device)
        return nat.diff_combine(maps, out, self.lam(), 1.0 - self.diff, self.out_heads, self.vdim, self.eps)
