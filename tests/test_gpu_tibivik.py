"""Tibivik on the GPU against the plain float64 restatement in ``oracle/tibivik.py`` (no code shared with the package).

Kernel level: every mechanism alone, with inputs built so that a fault shows (one key that takes the whole softmax, placed
just inside / just outside a window or a chunk, at a page border, far back among hundreds; a sink that swallows a head;
convolution rows and recurrent state carried over portions of 1, 2, 3 tokens through slots another sequence used).
Engine level, through ``CausalLMEngine`` and its scheduler: whole prompts, token-by-token decoding, portions, mixed
batches, reuse of pages and state slots, long decoding across pages, windows and chunks, looped layers, odd sizes, greedy
generation, CUDA graphs against eager.  The float32 engine is the sharp comparison; bfloat16 is checked against its
rounding noise."""
import math

import pytest
import torch

from oracle import tibivik as O

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


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols,streams", [(40, 1), (40, 3), (257, 2), (1000, 8)])
def test_bigram_embedding_stream_update_and_normed_read_out(nat, dtype, cols, streams):
    g = torch.Generator().manual_seed(cols + streams)
    n, vocab, buckets, mp, mc, eps = 7, 23, 11, 5, 3, 1e-3
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    emb = torch.randn(vocab, cols, generator=g).to(dtype)
    big = torch.randn(buckets + 1, cols, generator=g).to(dtype)
    tok = torch.randint(0, vocab, (n,), generator=g)
    prev = torch.randint(0, vocab, (n,), generator=g)
    prev[0] = prev[4] = -1                                      # first tokens of two sequences: the table's last row
    xs = torch.empty(n, streams, cols, device=DEV)
    nat.embed_bigram_streams(tok.int().to(DEV), prev.int().to(DEV), emb.to(DEV), big.to(DEV), xs, buckets, mp, mc)
    rows = torch.where(prev < 0, torch.full_like(tok, buckets), (prev * mp + tok * mc) % buckets)
    x0 = emb.double()[tok] + big.double()[rows]
    assert rel(xs, x0[:, None, :].expand(n, streams, cols)) < 1e-6
    xs2 = torch.empty_like(xs)
    nat.embed_bigram_streams(tok.int().to(DEV), prev.int().to(DEV), emb.to(DEV), None, xs2, 0, 0, 0)
    assert rel(xs2, emb.double()[tok][:, None, :].expand(n, streams, cols)) < 1e-6
    # distinct streams, then one update + read-out
    x = torch.randn(n, streams, cols, generator=g)
    mix, out_w, in_w = torch.randn(streams, streams, generator=g), torch.randn(streams, generator=g), torch.randn(streams, generator=g)
    w = torch.rand(cols, generator=g) + 0.5
    y1, y2 = torch.randn(n, cols, generator=g).to(dtype), torch.randn(n, cols, generator=g).to(dtype)
    for two in (False, True):
        xd = x.clone().to(DEV)
        h = torch.empty(n, cols, dtype=dtype, device=DEV)
        nat.stream_mix_norm(xd, y1.to(DEV), y2.to(DEV) if two else None, 0.7, 1.3, mix.to(DEV), out_w.to(DEV), in_w.to(DEV), w.to(DEV),
                            h, eps, dtype)
        y = 0.7 * y1.double() + (1.3 * y2.double() if two else 0)
        new = torch.einsum("st,nsc->ntc", mix.double(), x.double()) + out_w.double()[None, :, None] * y[:, None, :]
        assert rel(xd, new) < 1e-5
        u = (in_w.double()[None, :, None] * new).sum(1)
        assert rel(h, O.rms_norm(u, w.double(), eps)) < tol
    # read-out alone, and the update alone
    xd = x.clone().to(DEV)
    h = torch.empty(n, cols, dtype=dtype, device=DEV)
    nat.stream_mix_norm(xd, None, None, 1.0, 0.0, None, None, in_w.to(DEV), w.to(DEV), h, eps, dtype)
    assert torch.equal(xd.cpu(), x) and rel(h, O.rms_norm((in_w.double()[None, :, None] * x.double()).sum(1), w.double(), eps)) < tol
    pick = torch.tensor([5, 0, 5], dtype=torch.int32)
    out = nat.stream_gather_norm(x.to(DEV), pick.to(DEV), None, w.to(DEV), eps, dtype)
    assert rel(out, O.rms_norm(x.double()[pick.long()].sum(1), w.double(), eps)) < tol


@pytest.mark.parametrize("H,G,d,dv,rot_dims,tied,bias,norm", [(4, 2, 12, 12, 8, True, False, True), (3, 1, 10, 6, 0, False, True, False),
                                                             (6, 3, 64, 64, 64, True, False, True), (2, 2, 33, 7, 2, False, True, True)])
def test_attention_preparation_bias_whole_norm_rotation_and_cache_rows(nat, H, G, d, dv, rot_dims, tied, bias, norm):
    g = torch.Generator().manual_seed(H * d)
    page, eps, extra = 16, 1e-4, 3
    seqs = [(37, 11, 0, [4, 1, 6]), (0, 3, 1, [2]), (1000, 1, 2, [0] * 62 + [5])]
    lay = Lay(seqs, page, 63)
    n = lay.n_tokens
    nq, nk, nv = H * d, G * d, G * dv
    u = torch.randn(n, extra + nq + nk + (0 if tied else nv) + 2, generator=g)
    bq, bk, bv = (torch.randn(nq, generator=g), torch.randn(nk, generator=g), torch.randn(nv, generator=g)) if bias else (None,) * 3
    wq, wk = (torch.rand(nq, generator=g) + 0.5, torch.rand(nk, generator=g) + 0.5) if norm else (None, None)
    from nano_qwen3tts_vllm_b200.layers.rotary_embedding import HalfRotary
    rot = HalfRotary(rot_dims, 300.0).to(DEV) if rot_dims else None
    kc, vc = torch.zeros(7, page, nk, device=DEV), torch.zeros(7, page, nv, device=DEV)
    q = torch.empty(n, nq, device=DEV)
    dv_ = lambda t: None if t is None else t.to(DEV)
    nat.attn_prep(u.to(DEV), extra, extra + nq, -1 if tied else extra + nq + nk, dv_(bq), dv_(bk), dv_(bv), dv_(wq), dv_(wk),
                  rot.freq if rot else None, rot_dims, lay, q, kc, vc, H, G, d, dv, eps)
    ud = u.double()
    qr = ud[:, extra:extra + nq] + (bq.double() if bias else 0)
    kr = ud[:, extra + nq:extra + nq + nk] + (bk.double() if bias else 0)
    vr = kr if tied else ud[:, extra + nq + nk:extra + nq + nk + nv] + (bv.double() if bias else 0)
    if norm:
        qr, kr = O.rms_norm(qr, wq.double(), eps), O.rms_norm(kr, wk.double(), eps)
    pos = lay.positions.cpu().long()
    qr, kr = qr.reshape(n, H, d), kr.reshape(n, G, d)
    if rot_dims:
        qr, kr = O.rotate_half(qr, pos, rot_dims, 300.0), O.rotate_half(kr, pos, rot_dims, 300.0)
    assert rel(q, qr.reshape(n, nq)) < 2e-5                     # float angles at position 1000
    slots = lay.slot_mapping.cpu().long()
    assert rel(kc.view(-1, nk)[slots], kr.reshape(n, nk)) < 2e-5
    assert rel(vc.view(-1, nv)[slots], vr) < 1e-6
    untouched = torch.ones(7 * page, dtype=torch.bool)
    untouched[slots] = False
    assert not kc.view(-1, nk).cpu()[untouched].any() and not vc.view(-1, nv).cpu()[untouched].any()


def _attn_case(nat, H, G, d, dv, kind, mask, page, seqs, dtype=torch.float32, spike=None, sink_big=None, gate=False, seed=0, path=0):
    """``seqs`` = [(cached, new)]: sequences whose first ``cached`` tokens are in the cache and whose last ``new`` run now.
    ``spike`` = (sequence, query position, key position): that key is made to take that query's softmax in head 0."""
    g = torch.Generator().manual_seed(seed)
    scale = 0.3
    n_pages = sum((c + n + page - 1) // page for c, n in seqs)
    perm = torch.randperm(n_pages + 3, generator=g).tolist()
    kc = torch.zeros(n_pages + 3, page, G * d)
    vc = torch.zeros(n_pages + 3, page, G * dv)
    sink = torch.randn(H, generator=g)
    if sink_big is not None:
        sink[sink_big] = 40.0
    lay_seqs, qs, refs, gates = [], [], [], []
    at = 0
    for si, (c, n) in enumerate(seqs):
        T = c + n
        q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, dv, generator=g)
        if spike is not None and spike[0] == si:
            _, qi, kj = spike
            k[kj, 0] = 6.0 * q[qi, 0] / q[qi, 0].norm()
            q[qi, 0] *= 4.0
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        nb = (T + page - 1) // page
        bt = perm[at:at + nb]
        at += nb
        for t in range(T):
            kc[bt[t // page], t % page] = k[t].reshape(-1).float()
            vc[bt[t // page], t % page] = v[t].reshape(-1).float()
        ref = O.sink_softmax_attention(q.double(), k.double(), v.double(), scale, kind, mask, sink.double())
        gt = torch.randn(T, H, generator=g).to(dtype)
        if gate:
            ref = ref * torch.sigmoid(gt.double())[:, :, None]
        lay_seqs.append((c, n, si, bt))
        qs.append(q[c:].reshape(n, H * d)), refs.append(ref[c:].reshape(n, H * dv)), gates.append(gt[c:])
    lay = Lay(lay_seqs, page, max(len(s[3]) for s in lay_seqs))
    qd = torch.cat(qs).to(DEV)
    gd = torch.cat(gates).to(DEV) if gate else None
    out = torch.empty(lay.n_tokens, H * dv, dtype=dtype, device=DEV)
    nat.sink_attn(qd, kc.to(dtype).to(DEV), vc.to(dtype).to(DEV), out, lay, sink.to(DEV), gd, H, G, d, dv, page,
                  nat.MASK_WINDOW if kind == "window" else nat.MASK_CHUNK, mask, scale, path)
    return out, torch.cat(refs)


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 12, 12), (3, 1, 10, 6), (6, 3, 64, 64), (8, 8, 48, 40), (2, 1, 33, 200)])
@pytest.mark.parametrize("kind,mask", [("window", 1), ("window", 7), ("window", 64), ("window", 65), ("chunk", 1), ("chunk", 5),
                                       ("chunk", 64), ("chunk", 100)])
def test_sink_attention_prompts_portions_and_decoded_tokens_in_one_launch(nat, H, G, d, dv, kind, mask):
    seqs = [(0, 70), (130, 1), (33, 40), (64, 1), (0, 1), (199, 3)]
    out, ref = _attn_case(nat, H, G, d, dv, kind, mask, 16, seqs, gate=(H % 2 == 0), seed=mask)
    assert rel(out, ref) < 2e-5


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 64, 64), (2, 1, 48, 64), (4, 4, 128, 128), (3, 1, 32, 128), (2, 2, 96, 64), (2, 1, 128, 64)])
@pytest.mark.parametrize("kind,mask", [("window", 1), ("window", 7), ("window", 64), ("window", 65), ("window", 130), ("chunk", 1),
                                       ("chunk", 5), ("chunk", 64), ("chunk", 100)])
def test_tensor_core_sink_attention_against_plain_model_and_plain_kernel(nat, H, G, d, dv, kind, mask):
    """bfloat16 prompt portions on the tensor cores (decoded tokens of the same launch in the plain kernel): the error
    against the float64 model is that of the plain bfloat16 kernel."""
    seqs = [(0, 70), (130, 1), (33, 140), (64, 2), (0, 1), (199, 3), (5, 64)]
    tc, ref = _attn_case(nat, H, G, d, dv, kind, mask, 16, seqs, torch.bfloat16, gate=(H % 2 == 0), seed=mask, path=nat.SINK_ATTN_TENSOR)
    plain, _ = _attn_case(nat, H, G, d, dv, kind, mask, 16, seqs, torch.bfloat16, gate=(H % 2 == 0), seed=mask, path=nat.SINK_ATTN_PLAIN)
    assert rel(plain, ref) < 1.5e-2 and rel(tc, ref) < 1.5e-2


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("H,G,d", [(16, 8, 128), (8, 2, 32), (4, 1, 256), (3, 3, 64), (6, 1, 16), (2, 1, 64)])
@pytest.mark.parametrize("kind,mask", [("window", 1), ("window", 37), ("window", 300), ("chunk", 1), ("chunk", 64), ("chunk", 129)])
def test_one_token_rows_where_lanes_split_a_cached_row(nat, dtype, tol, H, G, d, kind, mask):
    """Sequences with ONE new token at contexts from 0 to several hundred keys (head sizes the row-splitting kernel takes,
    1 / 2 / 4 heads of a group per CTA), beside a prompt portion in the same launch; against the model and the plain kernel."""
    seqs = [(0, 1), (1, 1), (63, 1), (64, 1), (300, 1), (20, 5), (511, 1), (128, 1)]
    out, ref = _attn_case(nat, H, G, d, d, kind, mask, 16, seqs, dtype, gate=(H % 3 == 0), seed=mask + d)
    plain, _ = _attn_case(nat, H, G, d, d, kind, mask, 16, seqs, dtype, gate=(H % 3 == 0), seed=mask + d, path=nat.SINK_ATTN_PLAIN)
    assert rel(out, ref) < tol and rel(plain, ref) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("kind,mask", [("window", 33), ("window", 64), ("window", 200), ("chunk", 33), ("chunk", 64), ("chunk", 200)])
def test_one_key_that_takes_the_softmax_at_mask_edges_and_page_borders(nat, dtype, tol, page, kind, mask):
    """The query at position i, in a prompt portion and as a decoded token; the dominant key at the first position the
    mask lets through and at the one before it (which must NOT be seen), and at the query itself.  In bfloat16 the
    head size is one the tensor-core kernel takes, so prompt portions run there and decoded tokens in the plain kernel."""
    hd = 64 if dtype == torch.bfloat16 else 16
    for i in (mask - 1, mask, 2 * mask - 1, 2 * mask, 256):
        lo = max(0, i - mask + 1) if kind == "window" else (i // mask) * mask
        for kj in {lo, max(lo - 1, 0), i, (i // page) * page, max((i // page) * page - 1, 0)}:
            for cached, new in ((i, 1), (max(i - 9, 0), 14)):
                out, ref = _attn_case(nat, 4, 2, hd, hd, kind, mask, page, [(3, 2), (cached, new)], dtype, spike=(1, i, kj), seed=i + kj)
                assert rel(out, ref) < tol, (i, kj, cached, new)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_far_key_among_hundreds_and_a_sink_that_swallows_a_head(nat, dtype, tol):
    out, ref = _attn_case(nat, 4, 1, 32, 24, "window", 700, 64, [(0, 650), (649, 1)], dtype, spike=(0, 640, 3), seed=1)
    assert rel(out, ref) < tol
    if dtype == torch.bfloat16:                                           # the same through the tensor-core kernel
        out, ref = _attn_case(nat, 4, 1, 32, 64, "window", 700, 64, [(0, 650), (649, 1)], dtype, spike=(0, 640, 3), seed=1)
        assert rel(out, ref) < tol
        out, ref = _attn_case(nat, 4, 2, 64, 64, "window", 50, 16, [(0, 80), (79, 1)], dtype, sink_big=2, seed=3)
        assert rel(out, ref) < tol and out.view(-1, 4, 64)[:, 2].abs().max().item() < 1e-9
    out, ref = _attn_case(nat, 4, 1, 32, 24, "chunk", 1000, 64, [(645, 1)], dtype, spike=(0, 645, 2), seed=2)
    assert rel(out, ref) < tol
    out, ref = _attn_case(nat, 4, 2, 16, 16, "window", 50, 16, [(0, 80), (79, 1)], dtype, sink_big=2, seed=3)
    assert rel(out, ref) < tol
    assert out.view(-1, 4, 16)[:, 2].abs().max().item() < 1e-9           # the sink took the whole head


def _run_portions(mixer, hs, cuts, slots, dtype, page=16):
    """Run sequences ``hs`` (list of [T, D]) through ``mixer`` in portions ``cuts`` (the same cut for all), sequence b in
    state slot slots[b] with pages of its own; returns per sequence the list of the mixer's outputs."""
    from nano_qwen3tts_vllm_b200.utils.context import reset_context, set_context
    T = hs[0].shape[0]
    nb = (T + page - 1) // page
    outs = [[] for _ in hs]
    at = 0
    for n in cuts:
        lay = Lay([(at, n, slots[b], list(range(b * nb, (b + 1) * nb))) for b in range(len(hs))], page, nb)
        set_context(False, step_layout=lay)
        h = torch.cat([x[at:at + n] for x in hs]).to(dtype).to(DEV)
        with torch.inference_mode():
            y = mixer(h)
        reset_context()
        for b in range(len(hs)):
            outs[b].append(tuple(None if t is None or isinstance(t, float) else t[b * n:(b + 1) * n].double().cpu() for t in y))
        at += n
    assert at == T
    return outs


def _bind_dirty(mixer, slots, pages, page, dtype):
    """Caches and state filled with another owner's leftovers: position 0 must start from zero all the same."""
    plan = mixer.cache_plan()
    paged = [torch.full((pages, page, w), 3.0, dtype=dtype, device=DEV) for w in plan["paged"]]
    state = [torch.full((slots, *shape), 7.0, dtype=dt or dtype, device=DEV) for shape, dt in plan["state"]]
    mixer.bind(paged, state)
    return state


CUTS = [1, 2, 3, 7, 1, 1, 12, 2, 4]          # 33 tokens


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("ssm", [dict(), dict(heads=4, groups=2, norm_groups=4, conv=2, state=5, vdim=3),
                                 dict(heads=2, groups=2, norm_groups=2, conv=1, state=16, vdim=130),
                                 dict(heads=2, groups=1, norm_groups=1, conv=4, state=100, vdim=40),     # four lanes per column
                                 dict(heads=2, groups=2, norm_groups=1, conv=3, state=200, vdim=24)])    # eight lanes per column
def test_state_space_mixer_in_portions_through_reused_slots(dtype, tol, ssm):
    from nano_qwen3tts_vllm_b200.config import TibivikConfig
    from nano_qwen3tts_vllm_b200.models.tibivik import StateSpaceMixer
    cfg = O.random_config(types=("mamba2",), ssm=ssm, width=24)
    sd = O.random_weights(cfg, seed=2)
    c = TibivikConfig.from_dict(cfg)
    torch.set_default_dtype(dtype)
    try:
        with torch.device(DEV):
            mixer = StateSpaceMixer(c.width, c.layers[0].mixer, c.norm_eps)
    finally:
        torch.set_default_dtype(torch.float32)
    p = O._sub(sd, "l0.mix.")
    core = mixer.core
    with torch.no_grad():
        for name, prm in (("in", mixer.in_proj.weight), ("conv", core.conv.weight), ("conv.b", core.conv.bias), ("dt_bias", core.dt_bias),
                          ("A_log", core.A_log), ("D", core.D), ("norm", core.norm), ("o", mixer.o_proj.weight)):
            prm.copy_(p[name])
    g = torch.Generator().manual_seed(1)
    hs = [torch.randn(33, c.width, generator=g).to(dtype).float() for _ in range(2)]
    state = _bind_dirty(mixer, 3, 1, 16, dtype)
    outs = _run_portions(mixer, hs, CUTS, [2, 0], dtype)
    for b in range(2):
        ref = O.state_space(hs[b].double(), {k: v.double() for k, v in p.items()}, cfg["layers"][0]["mixer"], c.norm_eps)
        assert rel(torch.cat([o[0] for o in outs[b]]), ref) < tol
    assert bool((state[1][1] == 7.0).all())                         # the slot nobody owned is untouched


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("kind,over", [("parallel", dict()), ("parallel_2", dict()),
                                       ("parallel", dict(memory=dict(heads=1, dim=40, vdim=3, gate_cap=2.5),
                                                         window=dict(heads=2, kv_heads=2, dim=6, vdim=6, mask={"size": 4}, scale=0.5,
                                                                     rot={"dims": 6, "base": 17.0}))),
                                       ("parallel_2", dict(delta=dict(heads=3, kv_heads=3, dim=5, vdim=140, conv=2),
                                                           chunk=dict(heads=2, kv_heads=2, dim=7, vdim=9, mask={"size": 16}, scale=0.4))),
                                       # key sizes that put four and eight lanes on a value column of the recurrences
                                       ("parallel", dict(memory=dict(heads=2, dim=96, vdim=40, gate_cap=6.0))),
                                       ("parallel", dict(memory=dict(heads=1, dim=256, vdim=20, gate_cap=6.0))),
                                       ("parallel_2", dict(delta=dict(heads=4, kv_heads=2, dim=128, vdim=36, conv=3))),
                                       ("parallel_2", dict(delta=dict(heads=2, kv_heads=1, dim=130, vdim=33, conv=4)))])
def test_parallel_mixers_each_branch_in_portions_through_reused_slots(dtype, tol, kind, over):
    from nano_qwen3tts_vllm_b200.config import TibivikConfig
    from nano_qwen3tts_vllm_b200.models.tibivik import TibivikForCausalLM
    cfg = O.random_config(types=(kind,), width=24, ff=(None,), **over)
    sd = O.random_weights(cfg, seed=4)
    c = TibivikConfig.from_dict(cfg)
    torch.set_default_dtype(dtype)
    try:
        with torch.device(DEV):
            model = TibivikForCausalLM(c)
    finally:
        torch.set_default_dtype(torch.float32)
    model.load_state_dict({k: v.to(torch.bfloat16) for k, v in sd.items()})
    mixer = model.layers[0].mix
    g = torch.Generator().manual_seed(1)
    hs = [torch.randn(33, c.width, generator=g).to(dtype).float() for _ in range(2)]
    _bind_dirty(mixer, 3, 6, 16, dtype)
    outs = _run_portions(mixer, hs, CUTS, [2, 0], dtype)
    m = cfg["layers"][0]["mixer"]
    left, right = ({k: v.double() for k, v in O._sub(sd, f"l0.mix.{s}.").items()} for s in ("left", "right"))
    for b in range(2):
        h = hs[b].double()
        if kind == "parallel":
            ra, rb = O.window_attention_branch(h, left, m["left"], c.norm_eps), O.matrix_memory(h, right, m["right"], c.norm_eps)
        else:
            ra, rb = O.chunk_attention_branch(h, left, m["left"]), O.gated_delta(h, right, m["right"], c.norm_eps)
        assert rel(torch.cat([o[0] for o in outs[b]]), ra) < tol
        assert rel(torch.cat([o[1] for o in outs[b]]), rb) < tol


def test_matrix_memory_gates_stay_finite_when_the_running_maximum_moves_far(nat):
    """Large positive input gates and strongly negative forget gates: the maximum carries the scale, nothing overflows."""
    from nano_qwen3tts_vllm_b200.config import TibivikConfig
    from nano_qwen3tts_vllm_b200.models.tibivik import TibivikForCausalLM
    cfg = O.random_config(types=("parallel",), width=24, ff=(None,), memory=dict(heads=2, dim=8, vdim=8, gate_cap=60.0))
    sd = O.random_weights(cfg, seed=9)
    sd["l0.mix.right.i"] *= 40.0
    sd["l0.mix.right.f"] *= 40.0
    c = TibivikConfig.from_dict(cfg)
    with torch.device(DEV):
        model = TibivikForCausalLM(c)
    model.load_state_dict({k: v.to(torch.bfloat16) for k, v in sd.items()})
    sd = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    mixer = model.layers[0].mix
    hs = [torch.randn(33, c.width, generator=torch.Generator().manual_seed(3))]
    _bind_dirty(mixer, 1, 3, 16, torch.float32)
    outs = _run_portions(mixer, hs, CUTS, [0], torch.float32)
    ref = O.matrix_memory(hs[0].double(), {k: v.double() for k, v in O._sub(sd, "l0.mix.right.").items()}, cfg["layers"][0]["mixer"]["right"],
                          c.norm_eps)
    got = torch.cat([o[1] for o in outs[0]])
    assert torch.isfinite(got).all() and rel(got, ref) < 1e-4


# ------------------------------------------------------------------------------------------------ through the engine
def make_engine(cfg: dict, sd: dict, dtype="float32", pages=12, page=64, seqs=4, slots=None, eager=True, budget=None, max_len=256):
    from nano_qwen3tts_vllm_b200.config import TibivikConfig
    from nano_qwen3tts_vllm_b200.engine.llm_engine.lm_engine import CausalLMEngine
    c = TibivikConfig.from_dict(cfg)
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
    "all_three_mixers_looped": dict(loop=(1, 3, 2)),
    "plain_residual_no_bigram": dict(streams=0, bigram=None),
    "one_stream_loop_of_one_pass": dict(streams=1, loop=(0, 2, 1), types=("parallel", "mamba2")),
    "three_streams_whole_stack_looped": dict(streams=3, loop=(0, 3, 3), ff=(None, 16, None)),
    "empty_loop_attention_first": dict(loop=(1, 1, 4), types=("parallel_2", "parallel", "mamba2", "parallel_2")),
    "groups_and_norm_groups": dict(ssm=dict(heads=6, vdim=4, state=7, groups=3, conv=2, norm_groups=2), types=("mamba2", "mamba2")),
    "equal_heads_masks_of_one_no_taps": dict(window=dict(heads=2, kv_heads=2, dim=6, vdim=6, mask={"size": 1}, scale=1.0,
                                                         rot={"dims": 6, "base": 50.0}),
                                             chunk=dict(heads=1, kv_heads=1, dim=4, vdim=9, mask={"size": 1}, scale=1.0),
                                             delta=dict(heads=2, kv_heads=2, dim=4, vdim=4, conv=1),
                                             memory=dict(heads=1, dim=5, vdim=5, gate_cap=3.0), ssm=dict(conv=1, heads=1, vdim=5, state=3),
                                             scales=(1.0, 1.0)),
    "masks_that_span_pages": dict(window=dict(mask={"size": 70}), chunk=dict(mask={"size": 65}), types=("parallel", "parallel_2")),
    "rotation_of_two_coordinates": dict(window=dict(rot={"dims": 2, "base": 3.0}), types=("parallel",)),
    "vector_width_shapes": dict(width=128, vocab=128, ff=(128, 256), window=dict(heads=4, kv_heads=2, dim=32, vdim=32, rot={"dims": 16, "base": 1e4}),
                                chunk=dict(heads=4, kv_heads=4, dim=16, vdim=32), memory=dict(heads=2, dim=32, vdim=64),
                                delta=dict(heads=4, kv_heads=2, dim=16, vdim=16), ssm=dict(heads=4, vdim=32, state=16)),
}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_decode_and_portions_match_plain_model(name):
    cfg = O.random_config(**CONFIGS[name])
    sd = O.random_weights(cfg, seed=3)
    T = 90
    toks = tokens_for(cfg, T, 5)
    ref = O.forward(sd, cfg, toks)
    eng = make_engine(cfg, sd)
    try:
        whole = replay(eng, {"a": toks}, [[("a", T)]])["a"]
        assert nerr(whole, ref) < 5e-5
        one_by_one = replay(eng, {"b": toks}, [[("b", 1)] for _ in range(T)])["b"]
        assert nerr(one_by_one, ref) < 5e-5
        portions = replay(eng, {"c": toks}, [[("c", n)] for n in cuts_of(T)])["c"]
        assert nerr(portions, ref) < 5e-5
    finally:
        eng.exit()


def test_residual_stream_after_every_layer_run():
    cfg = O.random_config(loop=(1, 3, 2))
    sd = O.random_weights(cfg, seed=5)
    toks = tokens_for(cfg, 21, 1)
    want = []
    O.forward(sd, cfg, toks, layers_out=want)
    eng = make_engine(cfg, sd)
    try:
        eng.model_runner.model.trace_layers = got = []
        replay(eng, {"a": toks}, [[("a", 21)]])
    finally:
        eng.exit()
    assert len(got) == len(want) == 5
    for a, b in zip(got, want):
        assert rel(a, b) < 2e-5


def test_unequal_batch_matches_each_alone_and_reuses_pages_and_slots():
    """Five requests over four live slots and a pool smaller than their sum: portions of some beside single tokens of
    others; the fifth request takes over the pages and the slot of the first one that ends."""
    cfg = O.random_config(loop=(1, 3, 2), window=dict(mask={"size": 20}), chunk=dict(mask={"size": 18}))
    sd = O.random_weights(cfg, seed=7)
    reqs = {i: tokens_for(cfg, n, 10 + k) for k, (i, n) in enumerate([("a", 70), ("b", 33), ("c", 100), ("d", 17), ("e", 64)])}
    refs = {i: O.forward(sd, cfg, t) for i, t in reqs.items()}
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


def test_long_decode_over_pages_windows_and_chunks_graph_equals_eager():
    cfg = O.random_config(window=dict(mask={"size": 40}), chunk=dict(mask={"size": 33}))
    sd = O.random_weights(cfg, seed=11)
    toks = tokens_for(cfg, 150, 2)
    ref = O.forward(sd, cfg, toks)
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
    # a small random model amplifies bfloat16 rounding at a few positions (its recurrences' decays are random); everywhere
    # else the error is rounding noise
    e = nerr_rows(got, want)
    return e.median().item() < 0.04 and (e > 0.2).float().mean().item() < 0.05


def test_bfloat16_serving_precision_and_cut_independence():
    cfg = O.random_config(loop=(1, 3, 2), window=dict(mask={"size": 20}), chunk=dict(mask={"size": 18}))
    sd = O.random_weights(cfg, seed=13)
    toks = tokens_for(cfg, 80, 3)
    ref = O.forward(sd, cfg, toks)
    eng = make_engine(cfg, sd, dtype="bfloat16", page=16, pages=16, max_len=96)
    try:
        whole = replay(eng, {"a": toks}, [[("a", 80)]])["a"]
        parts = replay(eng, {"b": toks}, [[("b", n)] for n in cuts_of(80)])["b"]
        other = tokens_for(cfg, 50, 4)
        mixed = replay(eng, {"c": toks, "x": other}, [[("c", 30), ("x", 1)]] + [[("c", 1), ("x", 1)] for _ in range(49)] + [[("c", 1)]])["c"]
    finally:
        eng.exit()
    assert bf16_close(whole, ref) and bf16_close(parts, ref) and bf16_close(mixed, ref)
    assert nerr(parts, whole) < 0.05 and nerr(mixed, whole) < 0.05


def test_greedy_generation_through_the_scheduler():
    """``generate``: chunked prompts beside decoding sequences under a small token budget, greedy sampling by the
    package's sampler; the completions are the plain model's greedy continuations (ties aside: margins are checked)."""
    from nano_qwen3tts_vllm_b200.sampling_params import SamplingParams
    cfg = O.random_config()
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
            lg = O.forward(sd, cfg, seq)[-1]
            top = torch.topk(lg, 2).values
            if (top[0] - top[1]).item() > 1e-3:
                assert tok == int(lg.argmax()), (len(seq), tok)
            seq.append(tok)
        assert len(o["token_ids"]) == 12


def test_checkpoint_loading_is_strict_and_the_registry_finds_the_design(tmp_path):
    import json
    from safetensors.torch import save_file
    from nano_qwen3tts_vllm_b200.config import TibivikConfig, load_model_config
    from nano_qwen3tts_vllm_b200.llm import LLM
    from nano_qwen3tts_vllm_b200.models.tibivik import TibivikForCausalLM, random_state_dict
    cfg = O.random_config(loop=(0, 1, 2))
    sd = {k: v.to(torch.bfloat16) for k, v in O.random_weights(cfg, seed=19).items()}
    c = TibivikConfig.from_dict(cfg)
    assert c.to_dict() == cfg and c.runs() == [0, 0, 1, 2]
    assert sorted(random_state_dict(c, 0)) == sorted(sd)
    model = TibivikForCausalLM(c)
    assert sorted(model.checkpoint_names()) == sorted(sd)
    with pytest.raises(KeyError, match="missing"):
        model.load_state_dict({k: v for k, v in sd.items() if k != "l1.mix.left.sink"})
    with pytest.raises(KeyError, match="unexpected"):
        model.load_state_dict({**sd, "l0.mix.left.q": sd["embed"]})
    with pytest.raises(ValueError):
        TibivikConfig.from_dict({**cfg, "layers": [{**cfg["layers"][0], "type": "other"}]})
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file(sd, str(tmp_path / "model.safetensors"))
    assert isinstance(load_model_config(str(tmp_path)), TibivikConfig)
    toks = tokens_for(cfg, 20, 1)
    eng = LLM(str(tmp_path), dtype="float32", kvcache_block_size=16, num_kvcache_blocks=4, max_num_seqs=2, max_model_len=64,
              max_num_batched_tokens=128, enforce_eager=True, device=DEV)
    try:
        got = replay(eng, {"a": toks}, [[("a", 20)]])["a"]
    finally:
        eng.exit()
    assert nerr(got, O.forward({k: v.float() for k, v in sd.items()}, cfg, toks)) < 5e-5
