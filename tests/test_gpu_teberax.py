"""Teberax on the GPU against the plain float64 restatement in ``oracle/teberax.py`` (no code shared with the package).

Kernel level: every new or extended mechanism alone, with inputs built so that a fault shows (one key that takes the whole
softmax, placed just inside / just outside a window, among the kept first keys and just behind them, at a page border,
far back among hundreds; a zero sink that must take half of a head; a score cap that must bite; recurrent state carried
over portions of 1, 2, 3 tokens through slots another sequence used; identity experts with all of a token's weight).
Engine level, through ``CausalLMEngine`` and its scheduler: whole prompts, token-by-token decoding, portions, mixed
batches, reuse of pages and state slots, long decoding across pages and windows, borrowed keys and values, odd sizes,
greedy generation, CUDA graphs against eager.  The float32 engine is the sharp comparison; bfloat16 is checked against its
rounding noise."""
import json

import pytest
import torch

from oracle import teberax as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def nat():
    import nano_qwen3tts_vllm_b200._native as n
    n.lib()
    return n


class Lay:
    """A hand-made step layout for kernel tests: sequences [(pos0, n_new, slot, block_table)]."""

    def __init__(self, seqs, page, max_blocks):
        tok_seq, pos, slots, start = [], [], [], []
        o = 0
        for b, (p0, n, _, bt) in enumerate(seqs):
            start.append(o)
            for t in range(n):
                p = p0 + t
                tok_seq.append(b), pos.append(p), slots.append(bt[p // page] * page + p % page if bt else 0)
            o += n
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.tok_seq, self.positions, self.slot_mapping = i32(tok_seq), i32(pos), i32(slots)
        self.seq_start, self.seq_pos0 = i32(start), i32([s[0] for s in seqs])
        self.seq_len, self.seq_slot = i32([s[1] for s in seqs]), i32([s[2] for s in seqs])
        bt = torch.zeros(len(seqs), max_blocks, dtype=torch.int32)
        for b, s in enumerate(seqs):
            bt[b, :len(s[3])] = torch.tensor(s[3], dtype=torch.int32)
        self.block_tables = bt.to(DEV)
        self.n_tokens, self.n_seqs, self.max_new = o, len(seqs), max(s[1] for s in seqs)


def rel(a, b):
    return ((a.double().cpu() - b.double().cpu()).abs().max() / b.double().abs().max().clamp_min(1e-30)).item()


TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


# ------------------------------------------------------------------------------------------------ per-row kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [24, 257, 1000])
def test_in_and_out_norms_around_a_sublayer(nat, dtype, cols):
    g = torch.Generator().manual_seed(cols)
    n, eps, tol = 6, 1e-3, TOL[dtype]
    x0 = torch.randn(n, cols, generator=g)
    a, b = (torch.randn(n, cols, generator=g) * 3).to(dtype), torch.randn(n, cols, generator=g).to(dtype)
    wa, wb = torch.rand(cols, generator=g) + 0.5, torch.rand(cols, generator=g) + 0.5
    g_out, g_in = torch.tensor([0.7]), torch.tensor([1.3])
    d = lambda t: t.to(DEV)
    # a dense output, with and without the next input norm
    x = d(x0.clone())
    h = nat.sandwich_residual(x, d(g_out), a=d(a), g_in=d(g_in), eps=eps)
    want_x = x0.double() + O.rms_norm(a.double(), g_out.double(), eps)
    assert rel(x, want_x) < 1e-5 and rel(h, O.rms_norm(want_x, g_in.double(), eps)) < tol
    x = d(x0.clone())
    assert nat.sandwich_residual(x, d(g_out), a=d(a), eps=eps) is None and rel(x, want_x) < 1e-5
    # two branches, each normed over the row with its weight vector, half their sum
    x = d(x0.clone())
    h = nat.sandwich_residual(x, d(g_out), a=d(a), b=d(b), wa=d(wa), wb=d(wb), branch_scale=0.5, g_in=d(g_in), eps=eps)
    y = 0.5 * (O.rms_norm(a.double(), wa.double(), eps) + O.rms_norm(b.double(), wb.double(), eps))
    want_x = x0.double() + O.rms_norm(y, g_out.double(), eps)
    assert rel(x, want_x) < 1e-5 and rel(h, O.rms_norm(want_x, g_in.double(), eps)) < tol
    # expert outputs per choice; choices >= n_real return the sublayer's input
    top, n_real = 3, 4
    z = torch.randn(n * top, cols, generator=g).to(dtype)
    zw = torch.rand(n, top, generator=g)
    idx = torch.randint(0, 6, (n, top), generator=g)
    idx[0] = torch.tensor([5, 4, 4])                         # a token all of whose choices are identity experts
    hin = torch.randn(n, cols, generator=g).to(dtype)
    x = d(x0.clone())
    nat.sandwich_residual(x, d(g_out), z=d(z), zw=d(zw), z_idx=d(idx.int()), n_real=n_real, hin=d(hin), eps=eps)
    zz = torch.where((idx < n_real)[:, :, None], z.double().view(n, top, cols), hin.double()[:, None, :].expand(n, top, cols))
    want_x = x0.double() + O.rms_norm((zw.double()[:, :, None] * zz).sum(1), g_out.double(), eps)
    assert rel(x, want_x) < 1e-5
    # a table row per token, the stream starting from zero whatever it held
    table = torch.randn(11, cols, generator=g).to(dtype)
    ids = torch.randint(0, 11, (n,), generator=g)
    x = d(torch.full((n, cols), 1e9))
    h = nat.sandwich_residual(x, d(g_out), a=d(table), a_index=d(ids.int()), init=True, g_in=d(g_in), eps=eps)
    want_x = O.rms_norm(table.double()[ids], g_out.double(), eps)
    assert rel(x, want_x) < 1e-5 and rel(h, O.rms_norm(want_x, g_in.double(), eps)) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [20, 333, 2048])
def test_polynorm_and_logit_cap(nat, dtype, cols):
    g = torch.Generator().manual_seed(cols)
    z = (torch.randn(5, cols, generator=g) * 2).to(dtype)
    coef = torch.tensor([0.9, -0.4, 0.25, 0.1])
    got = nat.polynorm_(z.clone().to(DEV), coef.to(DEV), 1e-4)
    assert rel(got, O.polynorm(z.double(), coef.double(), 1e-4)) < TOL[dtype]
    y = torch.randn(7, cols, generator=g) * 30
    assert rel(nat.tanh_cap_(y.clone().to(DEV), 12.5), 12.5 * torch.tanh(y.double() / 12.5)) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dv", [(3, 10), (4, 64), (1, 200)])
def test_combination_of_two_attention_maps(nat, dtype, H, dv):
    g = torch.Generator().manual_seed(H * dv)
    maps = torch.randn(9, 2, H, dv, generator=g).to(dtype)
    out = torch.empty(9, H * dv, dtype=dtype, device=DEV)
    nat.diff_combine(maps.reshape(9, -1).to(DEV), out, 0.37, 0.8, H, dv, 1e-4)
    want = O.rms_norm(maps[:, 0].double() - 0.37 * maps[:, 1].double(), None, 1e-4) * 0.8
    assert rel(out, want.reshape(9, -1)) < TOL[dtype]
    # float maps beside an output of the activation type: nothing is rounded before the difference
    fmaps = torch.randn(9, 2, H, dv, generator=g)
    nat.diff_combine(fmaps.reshape(9, -1).to(DEV), out, 0.37, 0.8, H, dv, 1e-4)
    want = O.rms_norm(fmaps[:, 0].double() - 0.37 * fmaps[:, 1].double(), None, 1e-4) * 0.8
    assert rel(out, want.reshape(9, -1)) < (2e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("H,G,Gv,d,dv,rot_dims", [(4, 2, 2, 12, 6, 8), (6, 2, 1, 10, 7, 0), (2, 1, 1, 8, 8, 8)])
def test_attention_preparation_interleaved_rotation_shared_values_and_query_only(nat, interleaved, H, G, Gv, d, dv, rot_dims):
    g = torch.Generator().manual_seed(H + d)
    page, base, factor = 16, 77.0, 3.0
    seqs = [(5, 9, 0, [2, 0]), (0, 3, 1, [1])]
    lay = Lay(seqs, page, 2)
    n = lay.n_tokens
    nq, nk, nv = H * d, G * d, Gv * dv
    u = torch.randn(n, nq + nk + nv + 5, generator=g)
    qb, kb, vb = torch.randn(nq, generator=g), torch.randn(nk, generator=g), torch.randn(nv, generator=g)
    freq = (base ** (-2.0 * torch.arange(max(rot_dims // 2, 1), dtype=F64) / max(rot_dims, 1)) / factor).float()
    kc, vc = torch.zeros(3, page, nk, device=DEV), torch.zeros(3, page, nv, device=DEV)
    q = torch.empty(n, nq, device=DEV)
    nat.attn_prep(u.to(DEV), 3, 3 + nq, 3 + nq + nk, qb.to(DEV), kb.to(DEV), vb.to(DEV), None, None, freq.to(DEV), rot_dims, lay, q, kc, vc,
                  H, G, d, dv, 1e-5, interleaved=interleaved, v_heads=Gv)
    pos = lay.positions.cpu()
    uq = (u[:, 3:3 + nq].double() + qb.double()).view(n, H, d)
    uk = (u[:, 3 + nq:3 + nq + nk].double() + kb.double()).view(n, G, d)
    uv = u[:, 3 + nq + nk:3 + nq + nk + nv].double() + vb.double()

    def rotate(v):
        if rot_dims == 0:
            return v
        if interleaved:
            return O.rotate_pairs(v, pos, rot_dims, base, factor)
        half = rot_dims // 2
        ang = pos.double()[:, None] * freq.double()[None, :half]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = v[..., :half], v[..., half:rot_dims]
        return torch.cat([a * c - b * s, b * c + a * s, v[..., rot_dims:]], -1)

    assert rel(q, rotate(uq).reshape(n, nq)) < 1e-5
    slots = lay.slot_mapping.cpu().long()
    assert rel(kc.view(-1, nk)[slots], rotate(uk).reshape(n, nk)) < 1e-5
    assert rel(vc.view(-1, nv)[slots], uv) < 1e-6
    # without caches only the queries are made
    q2 = torch.empty(n, nq, device=DEV)
    nat.attn_prep(u.to(DEV), 3, 0, 0, qb.to(DEV), None, None, None, None, freq.to(DEV), rot_dims, lay, q2, None, None, H, G, d, dv, 1e-5,
                  interleaved=interleaved, v_heads=Gv)
    assert torch.equal(q2, q)


# ------------------------------------------------------------------------------------------------ attention
def _attn_case(nat, H, G, d, dv, page, seqs, *, window=0, keep_first=0, softcap=0.0, sink=None, two_maps=False, dtype=torch.float32,
               spike=None, seed=0, path=0, scale=0.3, float_out=False):
    """``seqs`` = [(cached, new)]: the first ``cached`` tokens are in the cache, the last ``new`` run now.  ``two_maps``: H
    and G count heads that each carry two maps over shared values (the kernel sees 2H query heads over 2G key heads and G
    value heads, map-major).  ``spike`` = (sequence, query position, key position, map): that key takes that query's
    softmax in head 0 of that map.  Returns (kernel output, plain model's output) for the new tokens."""
    g = torch.Generator().manual_seed(seed)
    M = 2 if two_maps else 1
    n_pages = sum((c + n + page - 1) // page for c, n in seqs)
    perm = torch.randperm(n_pages + 3, generator=g).tolist()
    kc = torch.zeros(n_pages + 3, page, M * G * d)
    vc = torch.zeros(n_pages + 3, page, G * dv)
    lay_seqs, qs, refs = [], [], []
    at = 0
    for si, (c, n) in enumerate(seqs):
        T = c + n
        q, k, v = torch.randn(T, M, H, d, generator=g), torch.randn(T, M, G, d, generator=g), torch.randn(T, G, dv, generator=g)
        if spike is not None and spike[0] == si:
            _, qi, kj, mp = spike
            k[kj, mp, 0] = 6.0 * q[qi, mp, 0] / q[qi, mp, 0].norm()
            q[qi, mp, 0] *= 4.0
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        nb = (T + page - 1) // page
        bt = perm[at:at + nb]
        at += nb
        for t in range(T):
            kc[bt[t // page], t % page] = k[t].reshape(-1).float()
            vc[bt[t // page], t % page] = v[t].reshape(-1).float()
        mask = O.visible(T, window or None, keep_first)
        ref = torch.stack([O.softmax_attention(q[:, m].double(), k[:, m].double(), v.double(), scale, mask, softcap or None,
                                               zero_sink=sink == "zero") for m in range(M)], 1)           # [T, M, H, dv]
        lay_seqs.append((c, n, si, bt))
        qs.append(q[c:].reshape(n, M * H * d)), refs.append(ref[c:].reshape(n, M * H * dv))
    lay = Lay(lay_seqs, page, max(len(s[3]) for s in lay_seqs))
    out = torch.empty(lay.n_tokens, M * H * dv, dtype=torch.float32 if float_out else dtype, device=DEV)
    sk = torch.zeros(M * H, device=DEV) if sink == "zero" else None
    nat.sink_attn(torch.cat(qs).to(DEV), kc.to(dtype).to(DEV), vc.to(dtype).to(DEV), out, lay, sk, None, M * H, M * G, d, dv, page,
                  nat.MASK_WINDOW, window, scale, path, v_heads=G, keep_first=keep_first, softcap=softcap)
    return out, torch.cat(refs)


MIXED = [(0, 1), (0, 70), (3, 2), (64, 1), (40, 31), (129, 1), (65, 66)]


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 12, 12), (3, 1, 10, 6), (8, 2, 32, 64), (2, 2, 33, 200)])
@pytest.mark.parametrize("window,keep", [(0, 0), (1, 0), (7, 3), (64, 1), (65, 64), (20, 70), (200, 5)])
def test_two_maps_over_shared_values_with_window_and_kept_first_keys(nat, H, G, d, dv, window, keep):
    out, ref = _attn_case(nat, H, G, d, dv, 16, MIXED, window=window, keep_first=keep, two_maps=True, seed=window + keep)
    assert rel(out, ref) < 2e-5


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 12, 12), (6, 2, 64, 64), (2, 1, 16, 40), (4, 4, 128, 128)])
@pytest.mark.parametrize("softcap", [0.0, 0.8])
def test_capped_scores_and_a_zero_sink(nat, H, G, d, dv, softcap):
    out, ref = _attn_case(nat, H, G, d, dv, 16, MIXED, softcap=softcap, sink="zero", seed=3, scale=1.0)
    assert rel(out, ref) < 2e-5
    plain, ref2 = _attn_case(nat, H, G, d, dv, 16, MIXED, softcap=softcap, sink="zero", seed=3, scale=1.0, path=1)
    assert rel(plain, ref2) < 2e-5
    if softcap:                                             # the cap matters: without it the same inputs give something else
        loose, _ = _attn_case(nat, H, G, d, dv, 16, MIXED, softcap=0.0, sink="zero", seed=3, scale=1.0)
        assert rel(loose, ref) > 1e-2
    none, ref3 = _attn_case(nat, H, G, d, dv, 16, MIXED, softcap=softcap, sink=None, seed=3, scale=1.0)
    assert rel(none, ref3) < 2e-5 and rel(none, ref) > 1e-3


@pytest.mark.parametrize("H,G,d,dv,two", [(8, 2, 32, 64, True), (2, 1, 64, 64, True), (4, 2, 128, 128, False), (2, 2, 96, 64, False),
                                          (3, 1, 48, 128, True)])
@pytest.mark.parametrize("window,keep", [(0, 0), (1, 0), (7, 3), (64, 4), (65, 64), (20, 70), (130, 2)])
def test_tensor_core_prompt_kernel_with_the_new_switches(nat, H, G, d, dv, two, window, keep):
    seqs = [(0, 150), (3, 2), (64, 70), (0, 64), (129, 67), (10, 1)]
    kw = dict(window=window, keep_first=keep, two_maps=two, softcap=0.0 if two else 1.5, sink=None if two else "zero", dtype=torch.bfloat16,
              seed=window + keep)
    out, ref = _attn_case(nat, H, G, d, dv, 64, seqs, path=2, **kw)
    plain, _ = _attn_case(nat, H, G, d, dv, 64, seqs, path=1, **kw)
    assert rel(out, ref) < 1.5e-2 and rel(out, plain) < 1.5e-2
    # unrounded outputs (floats beside bfloat16 inputs): every kernel of the launch, closer to the model than bfloat16 can be
    fout, _ = _attn_case(nat, H, G, d, dv, 64, seqs, path=0, float_out=True, **kw)
    assert fout.dtype == torch.float32 and rel(fout, ref) < 2e-3
    fplain, _ = _attn_case(nat, H, G, d, dv, 64, seqs, path=1, float_out=True, **kw)
    assert rel(fplain, ref) < 2e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,two", [(8, 2, 32, True), (4, 1, 64, True), (4, 2, 128, False), (3, 3, 16, False)])
@pytest.mark.parametrize("window,keep", [(0, 0), (1, 0), (37, 5), (37, 60), (300, 2)])
def test_one_token_rows_with_the_new_switches(nat, dtype, H, G, d, two, window, keep):
    seqs = [(0, 1), (36, 1), (37, 1), (64, 1), (255, 1), (700, 1), (5, 1)]
    out, ref = _attn_case(nat, H, G, d, d, 16, seqs, window=window, keep_first=keep, two_maps=two, softcap=0.0 if two else 2.0,
                          sink=None if two else "zero", dtype=dtype, seed=window)
    assert rel(out, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("window,keep", [(33, 0), (64, 3), (200, 1), (20, 16)])
def test_one_key_that_takes_the_softmax_at_window_kept_first_and_page_edges(nat, dtype, page, window, keep):
    """The dominating key sits just inside the window, just outside it (then the query must not see it), on the last kept
    first position and on the first position behind the kept ones, in a prompt portion and for a decoded token, in both
    maps; 32 x 64 is a head size all three kernels take in bfloat16."""
    T = 260
    for q_pos in (T - 1, 129, window + keep + 1):
        for k_pos in {q_pos - window + 1, q_pos - window, keep - 1, keep, (q_pos // page) * page, (q_pos // page) * page - 1}:
            if not 0 <= k_pos <= q_pos:
                continue
            for cached, mp in ((q_pos, 0), (max(q_pos - 40, 0), 1)):              # decoded alone / inside a portion
                out, ref = _attn_case(nat, 2, 1, 32, 64, page, [(3, 4), (cached, q_pos + 1 - cached)], window=window, keep_first=keep,
                                      two_maps=True, dtype=dtype, spike=(1, q_pos, k_pos, mp), seed=k_pos)
                assert rel(out, ref) < TOL[dtype], (q_pos, k_pos, cached)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_far_key_among_hundreds_and_the_zero_sink_that_halves_a_head(nat, dtype):
    # causal, 700 keys back, prompt portion (tensor cores in bfloat16), plain kernel and a decoded token
    for cached, path in ((0, 0), (0, 1), (759, 0), (650, 0)):
        out, ref = _attn_case(nat, 2, 1, 128, 128, 64, [(cached, 760 - cached)], sink="zero", dtype=dtype, spike=(0, 759, 59, 0), seed=1,
                              path=path, scale=0.1)
        assert rel(out, ref) < TOL[dtype], (cached, path)
    # all scores far below zero: the sink takes nearly everything, outputs shrink accordingly
    out, ref = _attn_case(nat, 2, 1, 16, 16, 16, [(0, 40), (39, 1)], sink="zero", dtype=dtype, seed=2, scale=1e-6)
    assert rel(out, ref) < TOL[dtype]
    none, _ = _attn_case(nat, 2, 1, 16, 16, 16, [(0, 40), (39, 1)], sink=None, dtype=dtype, seed=2, scale=1e-6)
    assert none[0].float().abs().max() > 1.9 * out[0].float().abs().max()     # one key: weight 1/2 with the sink, 1 without


def _latent_case(nat, H, r, dr, window, page, seqs, dtype=torch.float32, spike=None, seed=0, path=0):
    """Latent attention WITHOUT a sink: cached rows [c | kr] (kr stored turned), queries [absorbed | not yet turned]; the
    plain model is multi-query softmax attention with key [c | kr] and value c.  ``spike`` = (sequence, key position)."""
    from nano_qwen3tts_vllm_b200.layers.rotary_embedding import PairRotary
    g = torch.Generator().manual_seed(seed)
    base, scale = 50.0, 0.3
    rot = PairRotary(dr, base, None).to(DEV)
    nb = [(c + n + page - 1) // page for c, n in seqs]
    perm = torch.randperm(sum(nb) + 3, generator=g).tolist()
    cache = torch.zeros(sum(nb) + 3, page, r + dr, dtype=dtype, device=DEV)
    flat = cache.view(-1, r + dr)
    lay_seqs, QL, QR, refs, at = [], [], [], [], 0
    for s, (c, n) in enumerate(seqs):
        T = c + n
        lat, kr = torch.randn(T, r, generator=g).to(dtype), torch.randn(T, dr, generator=g).to(dtype)
        ql, qr = torch.randn(T, H, r, generator=g).to(dtype), torch.randn(T, H, dr, generator=g).to(dtype)
        if spike is not None and spike[0] == s:
            ql[:, :, 0] = 6.0                                   # every query looks along coordinate 0 ...
            lat[:, 0] = 0.0
            lat[spike[1], 0] = 40.0                             # ... where only the spiked key has anything
            lat[spike[1], 1:] *= 5.0
        bt = perm[at:at + nb[s]]
        at += nb[s]
        slots = torch.tensor([bt[p // page] * page + p % page for p in range(T)])
        flat[slots.to(DEV)] = torch.cat([lat, kr], 1).to(DEV)
        q = torch.cat([ql.double(), O.rotate_pairs(qr.double(), torch.arange(T), dr, base)], -1)
        k = torch.cat([lat.double(), kr.double()], -1)[:, None, :]
        refs.append(O.softmax_attention(q, k, lat.double()[:, None, :], scale, O.visible(T, window or None))[c:])
        lay_seqs.append((c, n, 0, bt)), QL.append(ql[c:]), QR.append(qr[c:])
    lay = Lay(lay_seqs, page, max(nb))
    n_new = lay.n_tokens
    ql = torch.cat(QL).transpose(0, 1).contiguous().to(DEV)                  # [H, n, r]
    qr = torch.cat(QR).contiguous().to(DEV)                                  # [n, H, dr]
    out = torch.full((H, n_new, r), 7.0, dtype=dtype, device=DEV)
    nat.latent_attn(ql, (r, n_new * r), qr, (H * dr, dr), cache, out, (r, n_new * r), None, rot.freq, 1.0, dr, lay, H, r, dr, page, window,
                    scale, path)
    return rel(out.transpose(0, 1), torch.cat(refs))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,r,dr", [(3, 24, 6), (4, 32, 16), (16, 128, 32)])
def test_latent_attention_without_a_sink_at_window_edges_page_borders_and_far_back(nat, dtype, H, r, dr):
    tol = TOL[dtype]
    for window in (0, 1, 7, 65):
        assert _latent_case(nat, H, r, dr, window, 16, [(0, 1), (0, 70), (3, 2), (64, 1), (40, 31), (129, 1)], dtype=dtype, seed=window) < tol
    page, window = 16, 33
    for p in (page - 1, page, 2 * page + 5):                    # the spiked key is seen by queries p .. p + window - 1 only
        seqs = [(p + window - 3, 6), (p + window - 1, 1), (p + window, 1), (p, 1), (0, p + 2)]
        for sp in range(len(seqs)):
            assert _latent_case(nat, H, r, dr, window, page, seqs, dtype=dtype, spike=(sp, p), seed=p) < tol, (p, sp)
    for window, back in [(0, 699), (600, 599), (600, 600)]:
        assert _latent_case(nat, H, r, dr, window, 64, [(700, 1), (680, 21)], dtype=dtype, spike=(0, 700 - back), seed=back) < tol
        assert _latent_case(nat, H, r, dr, window, 64, [(700, 1), (680, 21)], dtype=dtype, spike=(1, 700 - back), seed=back) < tol
    if dtype == torch.bfloat16 and r % 32 == 0:                 # the tensor-core kernel against the plain one
        a = _latent_case(nat, H, r, dr, 65, 16, [(0, 150), (64, 70), (129, 1)], dtype=dtype, seed=5, path=nat.LATENT_ATTN_PLAIN)
        assert a < tol


# ------------------------------------------------------------------------------------------------ recurrence, router
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,dv", [(2, 5, 7), (3, 32, 32), (1, 40, 100), (2, 130, 16)])
def test_gated_linear_recurrence_in_portions_through_reused_slots(nat, dtype, H, d, dv):
    """Two sequences advance in portions of 1, 2, 3, ... tokens, side by side and alone, through state slots that hold
    another owner's values at the start; the result equals the token-by-token recurrence from a zero state."""
    g = torch.Generator().manual_seed(d)
    tau, T = 3.0, [23, 9]
    bias = torch.randn(H * d, generator=g)
    ins, refs = [], []
    for n in T:
        q, k, z = (torch.randn(n, H * d, generator=g).to(dtype) for _ in range(3))
        v = torch.randn(n, H * dv, generator=g).to(dtype)
        ins.append((q, k, v, z))
        alpha = torch.exp(torch.nn.functional.logsigmoid(z.double() + bias.double()) / tau).view(n, H, d)
        S, o = torch.zeros(H, d, dv, dtype=F64), []
        for t in range(n):
            S = alpha[t][:, :, None] * S + k[t].double().view(H, d)[:, :, None] * v[t].double().view(H, dv)[:, None, :]
            o.append(torch.einsum("hdv,hd->hv", S, q[t].double().view(H, d) * d ** -0.5).reshape(-1))
        refs.append(torch.stack(o))
    state = torch.full((3, H, d, dv), 7.0, device=DEV)                       # dirty slots
    got, at = [[], []], [0, 0]
    for cuts in [(1, 2), (2, 1), (3, 0), (17, 6)]:
        seqs, parts = [], []
        for s, n in enumerate(cuts):
            if n:
                seqs.append((at[s], n, 2 - s, []))
                parts.append(tuple(t[at[s]:at[s] + n] for t in ins[s]))
        lay = Lay(seqs, 16, 1)
        u = torch.cat([torch.cat(p, 1) for p in parts]).to(DEV)                 # [q | k | v | z] as slices of one tensor
        q, k, v, z = u[:, :H * d], u[:, H * d:2 * H * d], u[:, 2 * H * d:2 * H * d + H * dv], u[:, 2 * H * d + H * dv:]
        out = torch.empty(lay.n_tokens, H * dv, device=DEV)
        nat.gated_linear_scan(q, k, v, z, bias.to(DEV), tau, state, out, lay, H, d, dv)
        o = 0
        for s, n in enumerate(cuts):
            if n:
                got[s].append(out[o:o + n].cpu())
                o += n
                at[s] += n
    for s in range(2):
        assert rel(torch.cat(got[s]), refs[s]) < TOL[dtype], s


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,I,top,ff,width", [(5, 2, 3, 10, 24), (4, 0, 4, 16, 64), (3, 3, 1, 8, 40), (16, 2, 4, 96, 128)])
def test_softmax_router_with_choice_correction_and_identity_experts(nat, dtype, E, I, top, ff, width):
    from nano_qwen3tts_vllm_b200.layers.moe import SoftmaxIdentityMoE
    g = torch.Generator().manual_seed(E * 10 + I)
    n = 37
    torch.set_default_dtype(dtype)
    try:
        moe = SoftmaxIdentityMoE(width, ff, E, top, I).to(DEV)
    finally:
        torch.set_default_dtype(torch.float32)
    w = {"router": torch.randn(E + I, width, generator=g).bfloat16().double() * 0.5,
         "correction": torch.randn(E + I, generator=g).bfloat16().double() * 0.3}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = (torch.randn(ff, width, generator=g).bfloat16().double() * width ** -0.5 for _ in range(2))
        w[f"e{e}.down"] = torch.randn(width, ff, generator=g).bfloat16().double() * ff ** -0.5
        moe.up[e, :ff].copy_(w[f"e{e}.gate"]), moe.up[e, ff:].copy_(w[f"e{e}.up"]), moe.down[e].copy_(w[f"e{e}.down"])
    moe.router.copy_(w["router"]), moe.router_bias.copy_(w["correction"])
    h = torch.randn(n, width, generator=g).to(dtype)
    if I:                                                   # one token whose choices are all identity experts when top <= I
        h[0] = (w["router"][E:].sum(0) * 4).to(dtype)
    idx_ref, wt_ref = O.route(h.double(), w["router"], w["correction"], top)
    z, zw = moe(h.to(DEV))
    idx = moe.last_choice.cpu().long()
    assert torch.equal(idx.sort(1).values, idx_ref.sort(1).values)
    order = idx_ref.argsort(1).gather(1, idx.argsort(1).argsort(1))           # reference columns in the kernel's order
    assert rel(zw, wt_ref.gather(1, order)) < 1e-5
    x = torch.zeros(n, width, device=DEV)
    nat.sandwich_residual(x, torch.ones(1, device=DEV), z=z, zw=zw, z_idx=moe.last_choice, n_real=E, hin=h.to(DEV), eps=0.0)
    want = O.rms_norm(O.moe_ff(h.double(), w, {"router": {"experts": E, "top": top}}), None, 0.0)
    assert rel(x, want) < (1e-4 if dtype == torch.float32 else 3e-2)


# ------------------------------------------------------------------------------------------------ the engine
def make_engine(cfg: dict, sd: dict, dtype="float32", pages=12, page=64, seqs=4, slots=None, eager=True, budget=None, max_len=256):
    from nano_qwen3tts_vllm_b200.config import TeberaxConfig
    from nano_qwen3tts_vllm_b200.engine.llm_engine.lm_engine import CausalLMEngine
    c = TeberaxConfig.from_dict(cfg)
    return CausalLMEngine(c, state_dict={k: v.to(torch.bfloat16) for k, v in sd.items()}, dtype=dtype, kvcache_block_size=page,
                          num_kvcache_blocks=pages, max_num_seqs=seqs, max_state_slots=slots or seqs, max_model_len=max_len,
                          max_num_batched_tokens=budget or seqs * max_len, enforce_eager=eager, device=DEV)


def replay(engine, requests: dict, schedule: list):
    """Feed ``schedule`` = [[(id, count), ...], ...] through engine.step as held sequences; logits of every position."""
    at = {i: 0 for i in requests}
    live, got = set(), {i: [] for i in requests}
    for step in schedule:
        want = {}
        for i, n in step:
            toks = requests[i][at[i]:at[i] + n]
            if i in live:
                engine.feed(i, toks)
            else:
                engine.add_request(toks, request_id=i, hold=True)
                live.add(i)
            want[i] = list(range(n))
            at[i] += n
        out = engine.step(want=want)
        assert out.scheduled == {i: n for i, n in step}
        o = 0
        for i, n in step:
            got[i].append(out.logits[o:o + n].double().cpu())
            o += n
        for i, _ in step:
            if at[i] == len(requests[i]):
                engine.clear_request(i)
                live.discard(i)
    return {i: torch.cat(v) for i, v in got.items() if v}


def nerr_rows(got, ref):
    """Per-position error: rms over the vocabulary of the mean-free difference, relative to the rms of the logits."""
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.pow(2).mean().sqrt()


def nerr(got, ref):
    return nerr_rows(got, ref).max().item()


def tokens_for(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def cuts_of(T, sizes=(2, 3, 1, 17, 2, 1, 1, 30, 2)):
    cuts, left = [], T
    for n in sizes:
        n = min(n, left)
        if n:
            cuts.append(n)
            left -= n
    return cuts + [1] * left


CONFIGS = {
    "all_mixers_borrowed_keys": dict(kv_from={3: 2}),
    "borrowing_twice_attention_first": dict(types=("attention", "parallel", "attention", "latent_attention", "attention"), kv_from={2: 0, 4: 0},
                                            ff=("moe", None, "dense", "moe", "dense")),
    "no_feed_forward_no_cap": dict(ff=(None,), logit_softcap=0, types=("latent_attention", "parallel")),
    "equal_heads_windows_of_one_top_of_one": dict(attention=dict(heads=2, kv_heads=2, dim=4, vdim=4, diff=0.5, mask={"size": 1, "keep_first": 1}),
                                                  left=dict(heads=1, kv_heads=1, dim=6, vdim=6, softcap=1.0, rot={"dims": 6, "base": 20.0}),
                                                  right=dict(heads=1, dim=4, vdim=4, tau=1.0, decay_rank=1),
                                                  latent=dict(heads=1, dim=4, rot_dim=2, vdim=4, kv_rank=4, mask={"size": 1},
                                                              rot={"dims": 2, "base": 5.0}),
                                                  moe=dict(expert={"ff": 4}, router={"experts": 1, "identity": 1, "top": 1})),
    "causal_everywhere_all_experts_chosen": dict(attention=dict(mask=None), latent=dict(mask=None), left=dict(rot=None, softcap=0),
                                                 moe=dict(router={"experts": 3, "identity": 0, "top": 3})),
    "masks_that_span_pages_kept_block": dict(attention=dict(mask={"size": 70, "keep_first": 20}), latent=dict(mask={"size": 65})),
    "only_identity_experts_can_win": dict(moe=dict(router={"experts": 2, "identity": 4, "top": 2}), types=("attention", "latent_attention"),
                                          ff=("moe",)),
    "vector_width_shapes": dict(width=128, vocab=128, dense_ff=256,
                                attention=dict(heads=6, kv_heads=2, dim=32, vdim=64, diff=0.2, scale=0.2, mask={"size": 40, "keep_first": 3}),
                                left=dict(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.15, softcap=20.0,
                                          rot={"dims": 16, "base": 1e4, "scaling": {"factor": 2.0}}),
                                right=dict(heads=2, dim=32, vdim=64, tau=8.0, decay_rank=8),
                                latent=dict(heads=4, dim=16, rot_dim=8, vdim=32, kv_rank=64, scale=0.2, mask={"size": 33},
                                            rot={"dims": 8, "base": 1e3}),
                                moe=dict(expert={"ff": 64}, router={"experts": 8, "identity": 1, "top": 2})),
}


def _config(name):
    over = dict(CONFIGS[name])
    for key in ("attention", "latent"):                      # mask=None: drop the mask from the default
        if key in over and "mask" in over[key] and over[key]["mask"] is None:
            base = O.random_config()["layers"][2 if key == "attention" else 1]["mixer"]
            over[key] = {**{k: v for k, v in base.items() if k != "mask"}, **{k: v for k, v in over[key].items() if k != "mask"}}
    cfg = O.random_config(**over)
    for layer in cfg["layers"]:                              # rot=None / softcap=0: drop the keys, as a checkpoint would
        m = layer["mixer"]
        if layer["type"] in ("attention", "latent_attention") and m.get("mask") is None:
            m.pop("mask", None)
        if layer["type"] == "parallel":
            if m["left"].get("rot") is None:
                m["left"].pop("rot", None)
            if not m["left"].get("softcap"):
                m["left"].pop("softcap", None)
    return cfg


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_decode_and_portions_match_plain_model(name):
    cfg = _config(name)
    sd = O.random_weights(cfg, seed=len(name))
    toks = tokens_for(cfg, 90, 1)
    ref = O.forward(cfg, sd, toks)
    eng = make_engine(cfg, sd, page=16, pages=20, max_len=96)
    try:
        whole = replay(eng, {"a": toks}, [[("a", 90)]])["a"]
        decode = replay(eng, {"b": toks}, [[("b", 5)]] + [[("b", 1)] for _ in range(85)])["b"]
        parts = replay(eng, {"c": toks}, [[("c", n)] for n in cuts_of(90)])["c"]
        pairs = replay(eng, {"d": toks}, [[("d", 2)] for _ in range(45)])["d"]
    finally:
        eng.exit()
    for got in (whole, decode, parts, pairs):
        assert nerr(got, ref) < 5e-5


def test_residual_stream_after_every_layer():
    cfg = _config("all_mixers_borrowed_keys")
    sd = O.random_weights(cfg, seed=3)
    toks = tokens_for(cfg, 40, 2)
    trace = []
    O.forward(cfg, sd, toks, trace)
    eng = make_engine(cfg, sd, page=16, pages=8, max_len=64)
    try:
        eng.model_runner.model.trace_layers = got = []
        replay(eng, {"a": toks}, [[("a", 40)]])
    finally:
        eng.exit()
    assert len(got) == len(trace) == len(cfg["layers"])
    for i, (g, t) in enumerate(zip(got, trace)):
        assert rel(g, t) < 2e-5, i


def test_unequal_batch_matches_each_alone_and_reuses_pages_and_slots():
    """Five requests over four live slots and a pool smaller than their sum: portions of some beside single tokens of
    others; the fifth request takes over the pages and the slot of the first one that ends."""
    cfg = _config("all_mixers_borrowed_keys")
    sd = O.random_weights(cfg, seed=7)
    reqs = {i: tokens_for(cfg, n, 10 + k) for k, (i, n) in enumerate([("a", 70), ("b", 33), ("c", 100), ("d", 17), ("e", 64)])}
    refs = {i: O.forward(cfg, sd, t) for i, t in reqs.items()}
    sched = [[("a", 40), ("b", 2)], [("a", 1), ("b", 20), ("c", 64)], [("b", 1), ("c", 3), ("d", 17)], [("a", 29), ("b", 10), ("c", 1)],
             [("e", 5), ("c", 32)], [("e", 1)], [("e", 58)]]
    eng = make_engine(cfg, sd, pages=18, page=16, seqs=4, slots=4, max_len=128)
    try:
        got = replay(eng, reqs, sched)
        for i in reqs:
            assert nerr(got[i], refs[i]) < 5e-5, i
        alone = replay(eng, {"c2": reqs["c"]}, [[("c2", 100)]])["c2"]
        assert nerr(alone, got["c"]) < 2e-5
    finally:
        eng.exit()


def test_long_decode_over_pages_and_windows_graph_equals_eager():
    cfg = _config("masks_that_span_pages_kept_block")
    sd = O.random_weights(cfg, seed=11)
    toks = tokens_for(cfg, 150, 2)
    ref = O.forward(cfg, sd, toks)
    sched = [[("a", 9)]] + [[("a", 1)] for _ in range(141)]
    outs = []
    for eager in (True, False):
        eng = make_engine(cfg, sd, page=16, pages=12, eager=eager, max_len=160)
        try:
            outs.append(replay(eng, {"a": toks}, sched)["a"])
        finally:
            eng.exit()
    assert nerr(outs[0], ref) < 5e-5
    assert nerr(outs[1], ref) < 5e-5
    assert nerr(outs[1], outs[0]) < 1e-6


def bf16_close(got, want):
    # a small random model amplifies bfloat16 rounding at a few positions; everywhere else the error is rounding noise
    e = nerr_rows(got, want)
    return e.median().item() < 0.04 and (e > 0.2).float().mean().item() < 0.05


@pytest.mark.parametrize("name", ["all_mixers_borrowed_keys", "vector_width_shapes"])
def test_bfloat16_serving_precision_and_cut_independence(name):
    cfg = _config(name)
    sd = O.random_weights(cfg, seed=13)
    toks = tokens_for(cfg, 80, 3)
    ref = O.forward(cfg, sd, toks)
    eng = make_engine(cfg, sd, dtype="bfloat16", page=16, pages=16, max_len=96)
    try:
        whole = replay(eng, {"a": toks}, [[("a", 80)]])["a"]
        parts = replay(eng, {"b": toks}, [[("b", n)] for n in cuts_of(80)])["b"]
        other = tokens_for(cfg, 50, 4)
        mixed = replay(eng, {"c": toks, "x": other}, [[("c", 30), ("x", 1)]] + [[("c", 1), ("x", 1)] for _ in range(49)] + [[("c", 1)]])["c"]
    finally:
        eng.exit()
    assert bf16_close(whole, ref) and bf16_close(parts, ref) and bf16_close(mixed, ref)
    assert nerr(parts, whole) < 0.08 and nerr(mixed, whole) < 0.08


def test_greedy_generation_through_the_scheduler():
    """``generate``: chunked prompts beside decoding sequences under a small token budget, greedy sampling by the
    package's sampler; the completions are the plain model's greedy continuations (ties aside: margins are checked)."""
    from nano_qwen3tts_vllm_b200.sampling_params import SamplingParams
    cfg = _config("all_mixers_borrowed_keys")
    sd = O.random_weights(cfg, seed=17)
    prompts = [tokens_for(cfg, n, 20 + n) for n in (5, 37, 18)]
    eng = make_engine(cfg, sd, page=16, pages=16, seqs=3, budget=64, max_len=64)
    try:
        outs = eng.generate(prompts, SamplingParams(temperature=1.0, max_tokens=12, ignore_eos=True, top_k=1))
    finally:
        eng.exit()
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o["token_ids"]:
            lg = O.forward(cfg, sd, seq)[-1]
            top = torch.topk(lg, 2).values
            if (top[0] - top[1]).item() > 1e-3:
                assert tok == int(lg.argmax()), (len(seq), tok)
            seq.append(tok)
        assert len(o["token_ids"]) == 12


def test_checkpoint_loading_is_strict_and_sizes_come_from_tensor_shapes(tmp_path):
    from safetensors.torch import save_file
    from nano_qwen3tts_vllm_b200.config import TeberaxConfig, load_model_config
    from nano_qwen3tts_vllm_b200.llm import LLM
    from nano_qwen3tts_vllm_b200.models.teberax import TeberaxForCausalLM, random_state_dict
    cfg = _config("all_mixers_borrowed_keys")
    sd = {k: v.to(torch.bfloat16) for k, v in O.random_weights(cfg, seed=19).items()}
    c = TeberaxConfig.from_dict(cfg)
    assert c.to_dict() == cfg
    assert sorted(random_state_dict(c, 0)) == sorted(sd)
    model = TeberaxForCausalLM(c)
    assert sorted(model.checkpoint_names()) == sorted(sd)
    assert "l3.mix.k" not in sd and "l2.mix.k" in sd          # the borrowing layer has no key/value projections
    with pytest.raises(KeyError, match="missing"):
        model.load_state_dict({k: v for k, v in sd.items() if k != "l0.mix.left.out"})
    with pytest.raises(KeyError, match="unexpected"):
        model.load_state_dict({**sd, "l3.mix.k": sd["l2.mix.k"]})
    with pytest.raises(ValueError):
        TeberaxConfig.from_dict({**cfg, "layers": [{**cfg["layers"][0], "type": "other"}]})
    with pytest.raises(ValueError, match="kv_from"):
        TeberaxConfig.from_dict(O.random_config(kv_from={2: 1}))
    # a file's configuration does not give the inner size of the decay projection: it is read from the tensor's shape
    bare = json.loads(json.dumps(cfg))
    del bare["layers"][0]["mixer"]["right"]["decay_rank"]
    (tmp_path / "config.json").write_text(json.dumps(bare))
    save_file(sd, str(tmp_path / "model.safetensors"))
    loaded = load_model_config(str(tmp_path))
    assert isinstance(loaded, TeberaxConfig) and loaded.layers[0].mixer.right.decay_rank == cfg["layers"][0]["mixer"]["right"]["decay_rank"]
    toks = tokens_for(cfg, 20, 1)
    eng = LLM(str(tmp_path), dtype="float32", kvcache_block_size=16, num_kvcache_blocks=4, max_num_seqs=2, max_model_len=64,
              max_num_batched_tokens=128, enforce_eager=True, device=DEV)
    try:
        got = replay(eng, {"a": toks}, [[("a", 20)]])["a"]
    finally:
        eng.exit()
    assert nerr(got, O.forward(cfg, {k: v.double() for k, v in sd.items()}, toks)) < 5e-5
