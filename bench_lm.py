"""``bench.py --lm``: prefill and decode throughput of the Bokenex decoder at layer sizes of a real model (random
weights), beside the package's closest existing model - the Qwen3-TTS talker stack (GQA softmax attention + gated MLP)
- with the same width, head layout, layer count and parameter count per layer.

Per size and model:
  prefill   tokens/s of one engine step over ``PREFILL_SEQS`` new prompts of ``PREFILL_LEN`` tokens (CUDA events around
            the engine's own ``step()``: layout upload, all layers, last-token logits, sampling);
  decode    tokens/s of the captured decode step for ``DECODE_SEQS`` sequences at a context of ``DECODE_CTX`` tokens
            (CUDA-graph replays back to back: the device time of one step, no host in it).
and, for the kernels that exist only in the new design, time and fraction of the measured roofline next to the like
kernel of the talker (``kernels``).  Timing: 3+ warm-up runs, CUDA events on the launching stream; the working sets
(weights + K/V of 64 sequences) are far above the 126 MB L2 for the decode steps, and an L2 flush precedes every timed
kernel launch of the ``kernels`` section."""
from __future__ import annotations

import json
import os
import time

PREFILL_SEQS, PREFILL_LEN = 4, 2048
DECODE_SEQS, DECODE_CTX = 64, 1100
WINDOW, TAPS, LAYERS = 1024, 4, 4
PAGE = 256

SIZES = {
    # name: width, heads, kv_heads, head size, talker intermediate (gated: 3 matrices) -> dense ff with the same parameters
    "w1024": dict(width=1024, heads=16, kv_heads=8, dim=128, inter=3072),
    "w2048": dict(width=2048, heads=16, kv_heads=8, dim=128, inter=6144),
}


def _peaks():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def bokenex_config(s: dict, moe: bool):
    from nano_qwen3tts_vllm_b200.config import BokenexConfig
    ff = s["inter"] * 3 // 2
    mlp = {"kind": "dense", "ff": ff} if not moe else \
        {"kind": "moe", "expert": {"ff": ff // 2}, "router": {"experts": 16, "top": 2, "scale": 1.0}}
    layer = {"type": "attention", "mlp": mlp,
             "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "conv": TAPS,
                       "mask": {"size": WINDOW}, "scale": s["dim"] ** -0.5}}
    return BokenexConfig.from_dict({"architecture": "Bokenex", "vocab": 3072, "width": s["width"], "max_positions": 4096,
                                    "norm": {"eps": 1e-6}, "residual_mult": 0.5, "layers": [layer] * LAYERS})


def _events(fn, iters, warm=3):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def bench_bokenex(s: dict, moe: bool, device: str, design: str = "bokenex") -> dict:
    import torch
    from nano_qwen3tts_vllm_b200.engine.llm_engine.lm_engine import CausalLMEngine
    from nano_qwen3tts_vllm_b200.sampling_params import SamplingParams
    cfg = {"bokenex": bokenex_config, "ridevik": ridevik_config, "tibivik": tibivik_config, "teberax": teberax_config}[design](s, moe)
    pages = DECODE_SEQS * ((DECODE_CTX + 64 + PAGE - 1) // PAGE) + PREFILL_SEQS * (PREFILL_LEN // PAGE + 1)
    eng = CausalLMEngine(cfg, state_dict="random:7", kvcache_block_size=PAGE, num_kvcache_blocks=pages,
                         max_num_seqs=DECODE_SEQS + PREFILL_SEQS, max_model_len=4096, max_num_batched_tokens=16384,
                         graph_batch_sizes=[DECODE_SEQS], device=device)
    g = torch.Generator().manual_seed(0)
    sp = SamplingParams(temperature=1.0, max_tokens=1 << 20, ignore_eos=True)
    prompt = lambda n: torch.randint(0, cfg.vocab, (n,), generator=g).tolist()
    out = {}
    # prefill: new prompts every run, given back afterwards
    times = []
    for it in range(6):
        ids = [f"p{it}_{i}" for i in range(PREFILL_SEQS)]
        for i in ids:
            eng.add_request(prompt(PREFILL_LEN), sp, request_id=i, hold=True)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step(want={i: [PREFILL_LEN - 1] for i in ids})
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        for i in ids:
            eng.clear_request(i)
    ms = sorted(times[3:])[len(times[3:]) // 2]
    out["prefill_ms"] = round(ms, 3)
    out["prefill_tok_s"] = round(PREFILL_SEQS * PREFILL_LEN / ms * 1e3)
    # decode: fill the contexts, one real decode step, then the captured step back to back
    for i in range(DECODE_SEQS):
        eng.add_request(prompt(DECODE_CTX), sp, request_id=f"d{i}")
    while any(s_.num_pending_tokens > 1 for s_ in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()
    eng.step()
    r = eng.model_runner
    assert DECODE_SEQS in r.graphs
    r.layout.set_decode_shape(DECODE_SEQS)
    ms = _events(r.graphs[DECODE_SEQS].replay, 30)
    out["decode_ms"] = round(ms, 4)
    out["decode_tok_s"] = round(DECODE_SEQS / ms * 1e3)
    eng.exit()
    return out


def ridevik_config(s: dict, moe: bool):
    """Layers of a real latent-attention model's shape: 16 heads of 128 + 64 (w2048) over a latent of 512, alternating
    the causal direct-query variant with the windowed, gated, query-latent one; feed-forwards with Bokenex's parameter
    count (dense: two matrices; experts: three matrices of a third less width)."""
    from nano_qwen3tts_vllm_b200.config import RidevikConfig
    d = s["dim"]
    ff = s["inter"] * 3 // 2
    mlp = {"kind": "dense", "ff": ff} if not moe else \
        {"kind": "moe", "expert": {"ff": ff // 3}, "router": {"experts": 16, "top": 2}}
    base = {"heads": s["heads"], "dim": d, "rot_dim": d // 2, "vdim": d, "kv_rank": 4 * d, "scale": (d + d // 2) ** -0.5}
    causal = {"type": "latent_attention_2", "mlp": mlp, "mixer": dict(base, rot={"base": 5e5, "dims": d // 2})}
    window = {"type": "latent_attention", "mlp": mlp,
              "mixer": dict(base, q_rank=s["width"] // 2, mask={"size": WINDOW},
                            rot={"base": 1e4, "dims": d // 2, "scaling": {"factor": 8.0, "original": 2048, "fast": 16.0, "slow": 2.0}})}
    return RidevikConfig.from_dict({"architecture": "Ridevik", "vocab": 3072, "width": s["width"], "embedding": {"scale": 1.0},
                                    "norm": {"eps": 1e-6, "groups": 4}, "layers": [causal, window] * (LAYERS // 2)})


def bench_talker(s: dict, device: str) -> dict:
    import torch
    from nano_qwen3tts_vllm_b200.config import ModelConfig, StackConfig
    from nano_qwen3tts_vllm_b200.llm import TalkerLLM
    from nano_qwen3tts_vllm_b200.sampling_params import SamplingParams
    stack = StackConfig(hidden_size=s["width"], intermediate_size=s["inter"], num_hidden_layers=LAYERS,
                        num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"], head_dim=s["dim"], vocab_size=3072,
                        rope_scaling={"mrope_section": [24, 20, 20], "interleaved": True})
    mc = ModelConfig(stack, StackConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=1, vocab_size=2048))
    pages = DECODE_SEQS * ((DECODE_CTX + 64 + PAGE - 1) // PAGE) + PREFILL_SEQS * (PREFILL_LEN // PAGE + 1)
    eng = TalkerLLM(mc, state_dict="random:7", num_kvcache_blocks=pages, max_num_seqs=DECODE_SEQS + PREFILL_SEQS,
                    max_model_len=4096, max_num_batched_tokens=16384, graph_batch_sizes=[DECODE_SEQS], device=device)
    sp = SamplingParams(temperature=1.0, max_tokens=1 << 20, ignore_eos=True)
    g = torch.Generator().manual_seed(0)
    emb = lambda n: (torch.randn(1, n, s["width"], generator=g) * 0.5).to(torch.bfloat16)
    out, times = {}, []
    for it in range(6):
        ids = [f"p{it}_{i}" for i in range(PREFILL_SEQS)]
        for i in ids:
            eng.add_request([emb(PREFILL_LEN)], sp, request_id=i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        for i in ids:
            eng.clear_request(i)
    ms = sorted(times[3:])[len(times[3:]) // 2]
    out["prefill_ms"] = round(ms, 3)
    out["prefill_tok_s"] = round(PREFILL_SEQS * PREFILL_LEN / ms * 1e3)
    ids = [f"d{i}" for i in range(DECODE_SEQS)]
    for i in ids:
        eng.add_request([emb(DECODE_CTX)], sp, request_id=i)
    eng.step()
    eng.add_requests(torch.randn(DECODE_SEQS, 1, s["width"], generator=g).to(torch.bfloat16), sp, ids)
    eng.step()
    r = eng.model_runner
    assert DECODE_SEQS in r.graphs
    r.set_decode_context(DECODE_SEQS)
    ms = _events(r.graphs[DECODE_SEQS].replay, 30)
    out["decode_ms"] = round(ms, 4)
    out["decode_tok_s"] = round(DECODE_SEQS / ms * 1e3)
    eng.exit()
    return out


def bench_kernels(device: str) -> dict:
    """The new design's own kernels at the w2048 layer shape, each after an L2 flush, with the fraction of the measured
    roofline (HBM copy bandwidth for the streaming kernels, cuBLAS bf16 for the contractions) and the like kernel of
    the talker measured the same way."""
    import torch
    import nano_qwen3tts_vllm_b200._native as nat
    hbm, tflops, how = _peaks()
    dev = torch.device(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    BF = torch.bfloat16

    def timed(fn, iters=5):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]

    class Lay:
        pass

    def layout(n_seqs, cached, new, pages_per_seq):
        lay = Lay()
        i32 = dict(dtype=torch.int32, device=dev)
        lay.n_seqs, lay.max_new, lay.n_tokens = n_seqs, new, n_seqs * new
        lay.seq_start = torch.arange(n_seqs, **i32) * new
        lay.seq_pos0 = torch.full((n_seqs,), cached, **i32)
        lay.seq_len = torch.full((n_seqs,), new, **i32)
        lay.seq_slot = torch.arange(n_seqs, **i32)
        lay.block_tables = torch.arange(n_seqs * pages_per_seq, **i32).view(n_seqs, pages_per_seq).contiguous()
        pos = (torch.arange(new, **i32) + cached).repeat(n_seqs)
        lay.positions = pos
        lay.tok_seq = torch.arange(n_seqs, **i32).repeat_interleave(new)
        lay.slot_mapping = (lay.tok_seq * pages_per_seq * PAGE + pos).to(torch.int32)
        return lay

    H, G, d, D = 16, 8, 128, 2048
    res = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": how}}
    r1 = torch.full((H,), 0.5, device=dev)
    r2 = torch.full((H,), 0.5, device=dev)
    pb = torch.full((H,), -3.0, device=dev)

    def entry(ms, bytes_=None, flops=None):
        e = {"us": round(ms * 1e3, 1)}
        if bytes_ is not None:
            e["gbs"] = round(bytes_ / ms / 1e6, 1)
            e["frac_hbm"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops is not None:
            e["tflops"] = round(flops / ms / 1e9, 1)
            e["frac_tensor"] = round(flops / ms / 1e9 / tflops, 4)
        return e

    # ---- attention, decode: 64 sequences at context 1100 (window 1024)
    pps = (DECODE_CTX + PAGE) // PAGE + 1
    lay = layout(DECODE_SEQS, DECODE_CTX, 1, pps)
    kc = torch.randn(DECODE_SEQS * pps, PAGE, G * d, device=dev).to(BF)
    vc = torch.randn(DECODE_SEQS * pps, PAGE, G * d, device=dev).to(BF)
    q = torch.randn(DECODE_SEQS, H * d, device=dev).to(BF)
    o = torch.empty_like(q)
    ms = timed(lambda: nat.window_sigmoid_attn(q, kc, vc, o, lay, r1, r2, pb, H, G, d, d, PAGE, WINDOW, d ** -0.5))
    res["window_sigmoid_attn decode 64x1100"] = entry(ms, bytes_=DECODE_SEQS * WINDOW * G * d * 2 * 2)
    ctx = torch.full((DECODE_SEQS,), DECODE_CTX + 1, dtype=torch.int32, device=dev)
    ws = torch.empty(nat.paged_attn_decode_workspace_bytes(DECODE_SEQS, H, d, pps * PAGE), dtype=torch.uint8, device=dev)
    kc4, vc4 = kc.view(-1, PAGE, G, d), vc.view(-1, PAGE, G, d)
    ms = timed(lambda: nat.paged_attn_decode(q.view(-1, H, d), kc4, vc4, lay.block_tables, ctx, d ** -0.5, pps * PAGE, workspace=ws))
    res["paged_attn_decode (talker) 64x1100"] = entry(ms, bytes_=DECODE_SEQS * (DECODE_CTX + 1) * G * d * 2 * 2)
    # ---- attention, prefill: 4 x 2048 tokens
    pps = PREFILL_LEN // PAGE
    lay = layout(PREFILL_SEQS, 0, PREFILL_LEN, pps)
    n = PREFILL_SEQS * PREFILL_LEN
    q = torch.randn(n, H * d, device=dev).to(BF)
    o = torch.empty_like(q)
    ms = timed(lambda: nat.window_sigmoid_attn(q, kc, vc, o, lay, r1, r2, pb, H, G, d, d, PAGE, WINDOW, d ** -0.5))
    pairs = PREFILL_SEQS * sum(min(i + 1, WINDOW) for i in range(PREFILL_LEN))
    res["window_sigmoid_attn prefill 4x2048"] = entry(ms, flops=pairs * H * d * 4)
    k = torch.randn(n, G, d, device=dev).to(BF)
    v = torch.randn(n, G, d, device=dev).to(BF)
    cu = (torch.arange(PREFILL_SEQS + 1, dtype=torch.int32, device=dev) * PREFILL_LEN).contiguous()
    ms = timed(lambda: nat.varlen_attn_prefill(q.view(n, H, d), k, v, cu, cu, PREFILL_LEN, PREFILL_LEN, d ** -0.5))
    res["prefill_attn_tc (talker, full causal) 4x2048"] = entry(ms, flops=PREFILL_SEQS * PREFILL_LEN * (PREFILL_LEN + 1) / 2 * H * d * 4)
    # ---- convolution + head norm + K/V write against head norm + rotation + K/V write
    C = H * d + 2 * G * d
    u = torch.randn(n, C, device=dev).to(BF)
    cw = torch.randn(C, TAPS, device=dev)
    st = torch.zeros(PREFILL_SEQS, TAPS - 1, C, dtype=BF, device=dev)
    nw = torch.ones(d, device=dev)
    qo = torch.empty(n, H * d, dtype=BF, device=dev)
    ms = timed(lambda: nat.conv_headnorm_kvwrite(u, cw, st, lay, nw, nw, qo, kc, vc, H, G, d, d, TAPS, 1e-6))
    res["conv_headnorm_kvwrite 8192 tokens"] = entry(ms, bytes_=n * (C + C) * 2)
    pos64 = lay.positions.to(torch.int64)
    inv = (1e6 ** (-torch.arange(0, d, 2, device=dev).float() / d)).contiguous()
    nwb = nw.to(BF)
    ms = timed(lambda: nat.qknorm_rope_kvwrite(u[:, :H * d].view(n, H, d), u[:, H * d:H * d + G * d].view(n, G, d),
                                               u[:, H * d + G * d:].view(n, G, d), nwb, nwb, 1e-6, pos64, inv,
                                               slot_mapping=lay.slot_mapping, k_cache=kc4, v_cache=vc4, want_k_out=False))
    res["qknorm_rope_kvwrite (talker) 8192 tokens"] = entry(ms, bytes_=n * (C + C) * 2)
    # ---- residual update + next norm against add + RMS norm
    x = torch.randn(n, D, device=dev)
    a_, b_ = torch.randn(n, D, device=dev).to(BF), torch.randn(n, D, device=dev).to(BF)
    h = torch.empty(n, D, dtype=BF, device=dev)
    gain = torch.ones(1, device=dev)
    ms = timed(lambda: nat.residual_norm(x, a_, b_, None, None, 0.5, h, gain, 1e-6, BF))
    res["residual_norm 8192x2048"] = entry(ms, bytes_=n * D * (4 + 4 + 2 + 2 + 2))
    wv = torch.ones(D, dtype=BF, device=dev)
    ms = timed(lambda: nat.add_rmsnorm(a_, b_, wv, 1e-6, 0, round_sum_first=False))
    res["add_rmsnorm (talker) 8192x2048"] = entry(ms, bytes_=n * D * 2 * 4)
    # ---- experts: grouped GEMM against the dense library GEMM of the same FLOPs
    E, top, ff = 16, 2, 4608
    from nano_qwen3tts_vllm_b200.layers.moe import SigmoidTopKMoE
    moe = SigmoidTopKMoE(D, ff, E, top, 1.0).to(dev)
    moe.router.normal_(0, D ** -0.5)
    moe.up.data = (torch.randn(E, ff, D, device=dev) * D ** -0.5).to(BF)
    moe.down.data = (torch.randn(E, D, ff, device=dev) * ff ** -0.5).to(BF)
    hh = torch.randn(n, D, device=dev).to(BF)
    ms = timed(lambda: moe(hh), iters=3)
    res["moe (route + 2 grouped GEMMs) 8192 tokens"] = entry(ms, flops=n * top * ff * D * 4)
    wd = (torch.randn(top * ff, D, device=dev) * 0.02).to(BF)
    ms = timed(lambda: torch.nn.functional.linear(hh, wd))
    res["dense GEMM of one projection's FLOPs (cuBLAS)"] = entry(ms, flops=n * top * ff * D * 2)
    return res


def bench_latent_kernels(device: str) -> dict:
    """Ridevik's own kernels at the w2048 layer shape (16 heads, latent 512 + 64 rotated), each after an L2 flush, with
    the fraction of the measured roofline; the like kernels of Bokenex come from ``bench_kernels`` in the same run."""
    import torch
    import nano_qwen3tts_vllm_b200._native as nat
    from nano_qwen3tts_vllm_b200.layers.rotary_embedding import PairRotary
    hbm, tflops, how = _peaks()
    dev = torch.device(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    BF = torch.bfloat16

    def timed(fn, iters=5):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]

    class Lay:
        pass

    def layout(n_seqs, cached, new, pages_per_seq):
        lay = Lay()
        i32 = dict(dtype=torch.int32, device=dev)
        lay.n_seqs, lay.max_new, lay.n_tokens = n_seqs, new, n_seqs * new
        lay.seq_start = torch.arange(n_seqs, **i32) * new
        lay.seq_pos0 = torch.full((n_seqs,), cached, **i32)
        lay.seq_len = torch.full((n_seqs,), new, **i32)
        lay.seq_slot = torch.arange(n_seqs, **i32)
        lay.block_tables = torch.arange(n_seqs * pages_per_seq, **i32).view(n_seqs, pages_per_seq).contiguous()
        pos = (torch.arange(new, **i32) + cached).repeat(n_seqs)
        lay.positions = pos
        lay.tok_seq = torch.arange(n_seqs, **i32).repeat_interleave(new)
        lay.slot_mapping = (lay.tok_seq * pages_per_seq * PAGE + pos).to(torch.int32)
        return lay

    def entry(ms, bytes_=None, flops=None):
        e = {"us": round(ms * 1e3, 1)}
        if bytes_ is not None:
            e["gbs"] = round(bytes_ / ms / 1e6, 1)
            e["frac_hbm"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops is not None:
            e["tflops"] = round(flops / ms / 1e9, 1)
            e["frac_tensor"] = round(flops / ms / 1e9 / tflops, 4)
        return e

    H, r, dr, dv, D, qrank = 16, 512, 64, 128, 2048, 1024
    Dk = r + dr
    res = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": how}}
    rot = PairRotary(dr, 1e4, None).to(dev)
    sink = torch.zeros(H, device=dev)
    scale = 192 ** -0.5

    def attn(lay, cache, window):
        n = lay.n_tokens
        ql = torch.randn(H, n, r, device=dev).to(BF)
        qr = torch.randn(n, H * dr, device=dev).to(BF)
        out = torch.empty_like(ql)
        return lambda: nat.latent_attn(ql, (r, n * r), qr, (H * dr, dr), cache, out, (r, n * r), sink, rot.freq, 1.0, dr, lay, H, r, dr,
                                       PAGE, window, scale)

    pps = (DECODE_CTX + PAGE) // PAGE + 1
    cache = torch.randn(DECODE_SEQS * pps, PAGE, Dk, device=dev).to(BF)
    lay = layout(DECODE_SEQS, DECODE_CTX, 1, pps)
    res["latent_attn decode 64x1100 causal"] = entry(timed(attn(lay, cache, 0)), bytes_=DECODE_SEQS * (DECODE_CTX + 1) * Dk * 2)
    res["latent_attn decode 64x1100 window 1024"] = entry(timed(attn(lay, cache, WINDOW)), bytes_=DECODE_SEQS * WINDOW * Dk * 2)
    pps = PREFILL_LEN // PAGE
    lay = layout(PREFILL_SEQS, 0, PREFILL_LEN, pps)
    n = PREFILL_SEQS * PREFILL_LEN
    pairs = PREFILL_SEQS * PREFILL_LEN * (PREFILL_LEN + 1) // 2
    res["latent_attn prefill 4x2048 causal"] = entry(timed(attn(lay, cache, 0), iters=3), flops=pairs * H * (Dk + r) * 2)
    pairs_w = PREFILL_SEQS * sum(min(i + 1, WINDOW) for i in range(PREFILL_LEN))
    res["latent_attn prefill 4x2048 window 1024"] = entry(timed(attn(lay, cache, WINDOW), iters=3), flops=pairs_w * H * (Dk + r) * 2)
    # ---- latent preparation: norms, key rotation, cache write
    C = qrank + Dk + H * dv
    u = torch.randn(n, C, device=dev).to(BF)
    cq = torch.empty(n, qrank, dtype=BF, device=dev)
    wq, wkv = torch.ones(qrank, device=dev), torch.ones(r, device=dev)
    ms = timed(lambda: nat.latent_prep(u, 0, qrank, cq, wq, wkv, rot.freq, 1.0, lay, cache, qrank, r, dr, dr, 1e-6))
    res["latent_prep 8192 tokens"] = entry(ms, bytes_=n * (qrank + Dk) * 2 * 2)
    # ---- token shift, residual + group norm, gate
    x = torch.randn(n, D, device=dev)
    mu = torch.rand(D, device=dev)
    st = torch.zeros(PREFILL_SEQS, D, device=dev)
    hs = torch.empty(n, D, dtype=BF, device=dev)
    ms = timed(lambda: nat.token_shift(x, mu, st, lay, hs))
    res["token_shift 8192x2048"] = entry(ms, bytes_=n * D * (4 + 2))
    a_ = torch.randn(n, D, device=dev).to(BF)
    w = torch.ones(D, device=dev)
    cp = torch.empty(n, D, dtype=BF, device=dev)
    ms = timed(lambda: nat.group_norm_residual(x, a_, None, None, w, 2, 1e-6, cp, BF))
    res["group_norm_residual 8192x2048"] = entry(ms, bytes_=n * D * (4 + 4 + 2 + 2))
    v = torch.randn(H, n, dv, device=dev).to(BF)
    ho = torch.empty(n, H * dv, dtype=BF, device=dev)
    ms = timed(lambda: nat.gate_heads(v, (dv, n * dv), u[:, qrank + Dk:], ho, H, dv))
    res["gate_heads 8192 tokens"] = entry(ms, bytes_=n * H * dv * 2 * 3)
    return res


def tibivik_config(s: dict, moe: bool = False):
    """Layers of real hybrid models' shapes at the size's width: a state-space layer (2 x width inner channels in heads of
    64, 128 state numbers, 4 taps), a chunked attention of the size's head layout beside a delta rule (as many value
    heads of the same size, half as many key heads), and a windowed attention with values tied to the keys beside a matrix
    memory of half as many heads; two residual streams, a hashed bigram table, SiLU-gated feed-forwards with the
    talker's three matrices."""
    from nano_qwen3tts_vllm_b200.config import TibivikConfig
    d, H, G, W = s["dim"], s["heads"], s["kv_heads"], s["width"]
    mlp = {"kind": "dense", "ff": s["inter"]}
    ssm = {"type": "mamba2", "mlp": mlp, "mixer": {"heads": 2 * W // 64, "vdim": 64, "state": 128, "groups": 1, "conv": TAPS, "norm_groups": 1}}
    chunk = {"type": "parallel_2", "mlp": mlp,
             "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "mask": {"size": WINDOW}, "scale": d ** -0.5},
                       "right": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "conv": TAPS}, "left_scale": 0.5, "right_scale": 1.0}}
    window = {"type": "parallel", "mlp": mlp,
              "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "mask": {"size": WINDOW}, "scale": d ** -0.5,
                                 "rot": {"dims": d // 2, "base": 1e4}},
                        "right": {"heads": H // 2, "dim": d, "vdim": d, "gate_cap": 10.0}, "left_scale": 0.5, "right_scale": 1.0}}
    return TibivikConfig.from_dict({"architecture": "Tibivik", "vocab": 3072, "width": W, "norm": {"eps": 1e-6}, "streams": 2,
                                    "embedding": {"bigram": {"buckets": 100003, "mul_prev": 31, "mul_cur": 17}},
                                    "layers": [ssm, chunk, window, chunk][:LAYERS]})


def bench_hybrid_kernels(device: str) -> dict:
    """Tibivik's own kernels at the w2048 layer shapes, each after an L2 flush, with the fraction of the measured roofline;
    the like kernels of Bokenex come from ``bench_kernels`` in the same run."""
    import torch
    import nano_qwen3tts_vllm_b200._native as nat
    hbm, tflops, how = _peaks()
    dev = torch.device(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    BF = torch.bfloat16

    def timed(fn, iters=5):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]

    class Lay:
        pass

    def layout(n_seqs, cached, new, pages_per_seq):
        lay = Lay()
        i32 = dict(dtype=torch.int32, device=dev)
        lay.n_seqs, lay.max_new, lay.n_tokens = n_seqs, new, n_seqs * new
        lay.seq_start = torch.arange(n_seqs, **i32) * new
        lay.seq_pos0 = torch.full((n_seqs,), cached, **i32)
        lay.seq_len = torch.full((n_seqs,), new, **i32)
        lay.seq_slot = torch.arange(n_seqs, **i32)
        lay.block_tables = torch.arange(n_seqs * pages_per_seq, **i32).view(n_seqs, pages_per_seq).contiguous()
        pos = (torch.arange(new, **i32) + cached).repeat(n_seqs)
        lay.positions = pos
        lay.tok_seq = torch.arange(n_seqs, **i32).repeat_interleave(new)
        lay.slot_mapping = (lay.tok_seq * pages_per_seq * PAGE + pos).to(torch.int32)
        return lay

    def entry(ms, bytes_=None, flops=None):
        e = {"us": round(ms * 1e3, 1)}
        if bytes_ is not None:
            e["gbs"] = round(bytes_ / ms / 1e6, 1)
            e["frac_hbm"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops is not None:
            e["tflops"] = round(flops / ms / 1e9, 1)
            e["frac_tensor"] = round(flops / ms / 1e9 / tflops, 4)
        return e

    H, G, d, D = 16, 8, 128, 2048
    res = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": how}}
    sink = torch.zeros(H, device=dev)
    scale = d ** -0.5

    def attn(lay, kc, vc, kind):
        n = lay.n_tokens
        q = torch.randn(n, H * d, device=dev).to(BF)
        out = torch.empty(n, H * d, dtype=BF, device=dev)
        return lambda: nat.sink_attn(q, kc, vc, out, lay, sink, None, H, G, d, d, PAGE, kind, WINDOW, scale)

    pps = (DECODE_CTX + PAGE) // PAGE + 1
    kc = torch.randn(DECODE_SEQS * pps, PAGE, G * d, device=dev).to(BF)
    vc = torch.randn(DECODE_SEQS * pps, PAGE, G * d, device=dev).to(BF)
    lay = layout(DECODE_SEQS, DECODE_CTX, 1, pps)
    res["sink_attn decode 64x1100 window 1024"] = entry(timed(attn(lay, kc, vc, nat.MASK_WINDOW)), bytes_=DECODE_SEQS * WINDOW * G * d * 2 * 2)
    res["sink_attn decode 64x1100 chunk 1024"] = entry(timed(attn(lay, kc, vc, nat.MASK_CHUNK)),
                                                        bytes_=DECODE_SEQS * (DECODE_CTX % WINDOW + 1) * G * d * 2 * 2)
    lay = layout(PREFILL_SEQS, 0, PREFILL_LEN, PREFILL_LEN // PAGE)
    n = PREFILL_SEQS * PREFILL_LEN
    pairs_w = PREFILL_SEQS * sum(min(i + 1, WINDOW) for i in range(PREFILL_LEN))
    res["sink_attn prefill 4x2048 window 1024"] = entry(timed(attn(lay, kc, vc, nat.MASK_WINDOW), iters=3), flops=pairs_w * H * 2 * d * 2)
    pairs_c = PREFILL_SEQS * sum(i % WINDOW + 1 for i in range(PREFILL_LEN))
    res["sink_attn prefill 4x2048 chunk 1024"] = entry(timed(attn(lay, kc, vc, nat.MASK_CHUNK), iters=3), flops=pairs_c * H * 2 * d * 2)
    # ---- attention preparation: whole-projection norm, rotation, cache write (values = raw keys)
    from nano_qwen3tts_vllm_b200.layers.rotary_embedding import HalfRotary
    rot = HalfRotary(d // 2, 1e4).to(dev)
    u = torch.randn(n, H * d + G * d, device=dev).to(BF)
    qo = torch.empty(n, H * d, dtype=BF, device=dev)
    wq, wk = torch.ones(H * d, device=dev), torch.ones(G * d, device=dev)
    ms = timed(lambda: nat.attn_prep(u, 0, H * d, -1, None, None, None, wq, wk, rot.freq, d // 2, lay, qo, kc, vc, H, G, d, d, 1e-6))
    res["attn_prep 8192 tokens"] = entry(ms, bytes_=n * (H * d * 2 + G * d * 3) * 2)
    # ---- residual streams: update + read-out + norm
    xs = torch.randn(n, 2, D, device=dev)
    y1, y2 = torch.randn(n, D, device=dev).to(BF), torch.randn(n, D, device=dev).to(BF)
    mix, ow, iw, w = torch.eye(2, device=dev), torch.ones(2, device=dev), torch.ones(2, device=dev), torch.ones(D, device=dev)
    h = torch.empty(n, D, dtype=BF, device=dev)
    ms = timed(lambda: nat.stream_mix_norm(xs, y1, y2, 0.7, 1.3, mix, ow, iw, w, h, 1e-6, BF))
    res["stream_mix_norm 8192x2x2048"] = entry(ms, bytes_=n * D * (2 * 4 * 2 + 2 * 2 + 2))
    # ---- short convolution + SiLU over the state-space layer's channels
    C = 2 * D + 256
    uc = torch.randn(n, C, device=dev).to(BF)
    cw = torch.randn(C, TAPS, device=dev)
    cst = torch.zeros(DECODE_SEQS, TAPS - 1, C, dtype=BF, device=dev)
    co = torch.empty(n, C, dtype=BF, device=dev)
    ms = timed(lambda: nat.short_conv_act(uc, 0, C, cw, None, cst, lay, co, TAPS, 1))
    res["short_conv_act 8192 tokens x 4352 channels"] = entry(ms, bytes_=n * C * 2 * 2)
    # ---- recurrences: prompt portions (4 x 2048 tokens) and decode steps (64 sequences)
    dlay = layout(DECODE_SEQS, DECODE_CTX, 1, 1)
    Hs, dvs, N = 2 * D // 64, 64, 128
    hz = torch.zeros(Hs, device=dev)
    for name, ly, nn in (("prefill 4x2048", lay, n), ("decode 64", dlay, DECODE_SEQS)):
        seqs = ly.n_seqs
        xbc = torch.randn(nn, Hs * dvs + 2 * N, device=dev).to(BF)
        dt = torch.randn(nn, Hs, device=dev).to(BF)
        st = torch.zeros(seqs, Hs, N, dvs, device=dev)
        yo = torch.empty(nn, Hs * dvs, device=dev)
        ms = timed(lambda: nat.ssm_scan(xbc, dt, hz, hz, hz, st, yo, ly, Hs, 1, dvs, N), iters=3)
        res[f"ssm_scan {name} (64 heads x 64, state 128)"] = entry(ms, bytes_=seqs * Hs * N * dvs * 4 * 2 + nn * (Hs * dvs * 6 + 2 * N * 2),
                                                                  flops=nn * Hs * N * dvs * 4)
        qkv = torch.randn(nn, 2 * G * d + H * d, device=dev).to(BF)
        ba = torch.randn(nn, 2 * H, device=dev).to(BF)
        st2 = torch.zeros(seqs, H, d, d, device=dev)
        o2 = torch.empty(nn, H * d, device=dev)
        hz2 = torch.zeros(H, device=dev)
        ms = timed(lambda: nat.delta_rule_scan(qkv, ba[:, :H], ba[:, H:], hz2, hz2, st2, o2, ly, H, G, d, d), iters=3)
        res[f"delta_rule_scan {name} (16 heads, 128 x 128)"] = entry(ms, bytes_=seqs * H * d * d * 4 * 2 + nn * (2 * G * d * 2 + H * d * 6),
                                                                    flops=nn * H * d * d * 8)
        Hm = H // 2
        um = torch.randn(nn, 3 * Hm * d + 2 * Hm, device=dev).to(BF)
        st3 = torch.zeros(seqs, Hm, d, d, device=dev)
        nm = torch.zeros(seqs, Hm, d + 1, device=dev)
        gs = torch.empty(nn, Hm, 3, device=dev)
        o3 = torch.empty(nn, Hm * d, device=dev)
        hz3 = torch.zeros(Hm, device=dev)
        cut = lambda a, w_: um[:, a:a + w_]
        ms = timed(lambda: nat.matrix_memory_scan(cut(0, Hm * d), cut(Hm * d, Hm * d), cut(2 * Hm * d, Hm * d), cut(3 * Hm * d, Hm),
                                                  cut(3 * Hm * d + Hm, Hm), hz3, hz3, 10.0, st3, nm, gs, o3, ly, Hm, d, d), iters=3)
        res[f"matrix_memory_scan {name} (8 heads, 128 x 128)"] = entry(ms, bytes_=seqs * Hm * d * d * 4 * 2 + nn * Hm * d * (6 + 4),
                                                                      flops=nn * Hm * d * d * 4)
    yy = torch.randn(n, H * d, device=dev)
    gg = torch.randn(n, H * d, device=dev).to(BF)
    oo = torch.empty(n, H * d, dtype=BF, device=dev)
    wn = torch.ones(d, device=dev)
    ms = timed(lambda: nat.gated_group_norm(yy, gg, wn, H, nat.GATE_SILU, False, 1e-6, oo))
    res["gated_group_norm 8192x2048 (16 heads)"] = entry(ms, bytes_=n * H * d * (4 + 2 + 2))
    return res


def teberax_config(s: dict, moe: bool = True):
    """Layers of real models' shapes at the size's width: biased rotary attention of the size's head layout (causal, capped
    scores, zero sink) beside gated linear attention of half as many heads of 128 x 128; windowed latent attention over a
    latent of 4 head sizes; differential attention whose two maps of half a head size share values of a full head size,
    window with four kept first keys, the second such layer on the first one's keys and values.  Feed-forwards: dense
    PolyNorm with two matrices of the talker's parameter count, or 16 SiLU-gated experts (top 2) and one identity expert."""
    from nano_qwen3tts_vllm_b200.config import TeberaxConfig
    d, H, G, W = s["dim"], s["heads"], s["kv_heads"], s["width"]
    ff = s["inter"] * 3 // 2
    dense = {"kind": "dense", "ff": ff}
    experts = {"kind": "moe", "expert": {"ff": ff // 3}, "router": {"experts": 16, "identity": 1, "top": 2}} if moe else dense
    par = {"type": "parallel", "mlp": dense,
           "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "softcap": 50.0,
                              "rot": {"dims": d // 2, "base": 1e4, "scaling": {"factor": 2.0}}},
                     "right": {"heads": H // 2, "dim": d, "vdim": d, "tau": 16.0, "decay_rank": 16}}}
    lat = {"type": "latent_attention", "mlp": experts,
           "mixer": {"heads": H, "dim": d, "rot_dim": d // 2, "vdim": d, "kv_rank": 4 * d, "scale": (d + d // 2) ** -0.5,
                     "mask": {"size": WINDOW}, "rot": {"dims": d // 2, "base": 1e4}}}
    att = {"heads": H, "kv_heads": G, "dim": d // 2, "vdim": d, "scale": (d // 2) ** -0.5, "diff": 0.5, "mask": {"size": WINDOW, "keep_first": 4}}
    own = {"type": "attention", "mlp": experts, "mixer": att}
    borrowed = {"type": "attention", "mlp": dense, "mixer": dict(att, kv_from=2)}
    return TeberaxConfig.from_dict({"architecture": "Teberax", "vocab": 3072, "width": W, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
                                    "layers": [par, lat, own, borrowed][:LAYERS]})


def bench_teberax_kernels(device: str) -> dict:
    """The kernels Teberax added or extended at the w2048 layer shapes, each after an L2 flush, with the fraction of the
    measured roofline; the like kernels of Tibivik come from ``bench_hybrid_kernels`` in the same run."""
    import torch
    import nano_qwen3tts_vllm_b200._native as nat
    hbm, tflops, how = _peaks()
    dev = torch.device(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    BF = torch.bfloat16

    def timed(fn, iters=5):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]

    class Lay:
        pass

    def layout(n_seqs, cached, new, pages_per_seq):
        lay = Lay()
        i32 = dict(dtype=torch.int32, device=dev)
        lay.n_seqs, lay.max_new, lay.n_tokens = n_seqs, new, n_seqs * new
        lay.seq_start = torch.arange(n_seqs, **i32) * new
        lay.seq_pos0 = torch.full((n_seqs,), cached, **i32)
        lay.seq_len = torch.full((n_seqs,), new, **i32)
        lay.seq_slot = torch.arange(n_seqs, **i32)
        lay.block_tables = torch.arange(n_seqs * pages_per_seq, **i32).view(n_seqs, pages_per_seq).contiguous()
        pos = (torch.arange(new, **i32) + cached).repeat(n_seqs)
        lay.positions = pos
        lay.tok_seq = torch.arange(n_seqs, **i32).repeat_interleave(new)
        lay.slot_mapping = (lay.tok_seq * pages_per_seq * PAGE + pos).to(torch.int32)
        return lay

    def entry(ms, bytes_=None, flops=None):
        e = {"us": round(ms * 1e3, 1)}
        if bytes_ is not None:
            e["gbs"] = round(bytes_ / ms / 1e6, 1)
            e["frac_hbm"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops is not None:
            e["tflops"] = round(flops / ms / 1e9, 1)
            e["frac_tensor"] = round(flops / ms / 1e9 / tflops, 4)
        return e

    H, G, d, D = 16, 8, 128, 2048
    res = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": how}}
    pps = (DECODE_CTX + PAGE) // PAGE + 1
    dlay = layout(DECODE_SEQS, DECODE_CTX, 1, pps)
    play = layout(PREFILL_SEQS, 0, PREFILL_LEN, PREFILL_LEN // PAGE)
    n = PREFILL_SEQS * PREFILL_LEN
    # ---- biased rotary branch: causal, capped scores, zero sink (heads 16 over 8, 128 x 128)
    kc = torch.randn(DECODE_SEQS * pps, PAGE, G * d, device=dev).to(BF)
    vc = torch.randn(DECODE_SEQS * pps, PAGE, G * d, device=dev).to(BF)
    zero = torch.zeros(H, device=dev)

    def left(lay):
        q = torch.randn(lay.n_tokens, H * d, device=dev).to(BF)
        out = torch.empty(lay.n_tokens, H * d, dtype=BF, device=dev)
        return lambda: nat.sink_attn(q, kc, vc, out, lay, zero, None, H, G, d, d, PAGE, nat.MASK_WINDOW, 0, d ** -0.5, softcap=50.0)

    res["sink_attn decode 64x1100 causal, cap, zero sink"] = entry(timed(left(dlay)), bytes_=DECODE_SEQS * (DECODE_CTX + 1) * G * d * 2 * 2)
    pairs = PREFILL_SEQS * sum(i + 1 for i in range(PREFILL_LEN))
    res["sink_attn prefill 4x2048 causal, cap, zero sink"] = entry(timed(left(play), iters=3), flops=pairs * H * 2 * d * 2)
    # ---- differential attention: 2 x 16 query heads of 64 over 2 x 8 key heads, 8 value heads of 128, window 1024 + 4 kept
    dq = d // 2
    kc2 = torch.randn(DECODE_SEQS * pps, PAGE, 2 * G * dq, device=dev).to(BF)

    def diff(lay):
        q = torch.randn(lay.n_tokens, 2 * H * dq, device=dev).to(BF)
        maps = torch.empty(lay.n_tokens, 2 * H * d, dtype=torch.float32, device=dev)     # unrounded, as the model asks for them
        return maps, (lambda: nat.sink_attn(q, kc2, vc, maps, lay, None, None, 2 * H, 2 * G, dq, d, PAGE, nat.MASK_WINDOW, WINDOW, dq ** -0.5,
                                            v_heads=G, keep_first=4))

    res["sink_attn decode 64x1100 two maps, window 1024 + 4 kept"] = entry(timed(diff(dlay)[1]),
                                                                          bytes_=DECODE_SEQS * (WINDOW + 4) * (2 * G * dq + G * d) * 2)
    pairs_w = PREFILL_SEQS * sum(min(i + 1, WINDOW + 4) for i in range(PREFILL_LEN))
    maps, fn = diff(play)
    res["sink_attn prefill 4x2048 two maps, window 1024 + 4 kept"] = entry(timed(fn, iters=3), flops=pairs_w * 2 * H * 2 * (dq + d))
    oc = torch.empty(n, H * d, dtype=BF, device=dev)
    res["diff_combine 8192 tokens x 16 heads x 128"] = entry(timed(lambda: nat.diff_combine(maps, oc, 0.3, 0.5, H, d, 1e-6)),
                                                            bytes_=n * H * d * (2 * 4 + 2))
    # ---- attention preparation: biases, interleaved rotation, cache write
    from nano_qwen3tts_vllm_b200.layers.rotary_embedding import PairRotary
    rot = PairRotary(d // 2, 1e4, {"factor": 2.0}).to(dev)
    u = torch.randn(n, H * d + 2 * G * d, device=dev).to(BF)
    qo = torch.empty(n, H * d, dtype=BF, device=dev)
    bq, bk = torch.zeros(H * d, device=dev), torch.zeros(G * d, device=dev)
    ms = timed(lambda: nat.attn_prep(u, 0, H * d, H * d + G * d, bq, bk, bk, None, None, rot.freq, d // 2, play, qo, kc, vc, H, G, d, d, 1e-6,
                                     interleaved=True))
    res["attn_prep 8192 tokens (biases, pair rotation)"] = entry(ms, bytes_=n * (H * d * 2 + G * d * 4) * 2)
    # ---- the in-and-out norms around a sublayer: dense, two branches, experts
    x = torch.randn(n, D, device=dev)
    a, b = torch.randn(n, D, device=dev).to(BF), torch.randn(n, D, device=dev).to(BF)
    wv, g1 = torch.ones(D, device=dev), torch.ones(1, device=dev)
    ms = timed(lambda: nat.sandwich_residual(x, g1, a=a, g_in=g1))
    res["sandwich_residual 8192x2048 dense"] = entry(ms, bytes_=n * D * (4 * 2 + 2 + 2))
    ms = timed(lambda: nat.sandwich_residual(x, g1, a=a, b=b, wa=wv, wb=wv, branch_scale=0.5, g_in=g1))
    res["sandwich_residual 8192x2048 two branches"] = entry(ms, bytes_=n * D * (4 * 2 + 2 * 2 + 2))
    z = torch.randn(n * 2, D, device=dev).to(BF)
    zw = torch.rand(n, 2, device=dev)
    zi = torch.randint(0, 17, (n, 2), device=dev, dtype=torch.int32)
    ms = timed(lambda: nat.sandwich_residual(x, g1, z=z, zw=zw, z_idx=zi, n_real=16, hin=a, g_in=g1))
    res["sandwich_residual 8192x2048 two experts of 16 + 1"] = entry(ms, bytes_=n * D * (4 * 2 + 3 * 2 + 2))
    ffw = 9216
    y = torch.randn(n, ffw, device=dev).to(BF)
    coef = torch.tensor([1.0, 0.3, 0.1, 0.0], device=dev)
    res["polynorm 8192x9216"] = entry(timed(lambda: nat.polynorm_(y, coef, 1e-6)), bytes_=n * ffw * 2 * 2)
    # ---- gated linear attention: 8 heads of 128 x 128
    Hr = H // 2
    for name, ly, nn in (("prefill 4x2048", play, n), ("decode 64", layout(DECODE_SEQS, DECODE_CTX, 1, 1), DECODE_SEQS)):
        uu = torch.randn(nn, 3 * Hr * d, device=dev).to(BF)
        zz = torch.randn(nn, Hr * d, device=dev).to(BF)
        st = torch.zeros(ly.n_seqs, Hr, d, d, device=dev)
        oo = torch.empty(nn, Hr * d, device=dev)
        bz = torch.zeros(Hr * d, device=dev)
        ms = timed(lambda: nat.gated_linear_scan(uu[:, :Hr * d], uu[:, Hr * d:2 * Hr * d], uu[:, 2 * Hr * d:], zz, bz, 16.0, st, oo, ly, Hr, d, d),
                   iters=3)
        res[f"gated_linear_scan {name} (8 heads, 128 x 128)"] = entry(ms, bytes_=ly.n_seqs * Hr * d * d * 4 * 2 + nn * Hr * d * (4 * 2 + 4 + 4 * 2),
                                                                     flops=nn * Hr * d * d * 6)
    # ---- router: softmax over 17 outputs, correction, top 2
    hh = torch.randn(n, D, device=dev).to(BF)
    rw, rb = torch.randn(17, D, device=dev), torch.zeros(17, device=dev)
    ti, tw = torch.empty(n, 2, dtype=torch.int32, device=dev), torch.empty(n, 2, device=dev)
    off, sp = torch.empty(18, dtype=torch.int32, device=dev), torch.empty(n * 2, dtype=torch.int32, device=dev)
    ms = timed(lambda: nat.moe_route(hh, rw, ti, tw, off, sp, 2, 1.0, bias=rb, mode=nat.ROUTE_SOFTMAX_ALL))
    res["moe_route 8192 tokens, 16 + 1 outputs"] = entry(ms, bytes_=n * D * 2)
    return res


def main_teberax(device: str = "cuda:0") -> dict:
    """``bench.py --lm-teberax``: Teberax beside Tibivik (the package's closest model: attention beside a recurrence behind
    one projection, the same attention and recurrence kernels, over the same engine) at equal width, head layout and layer
    count, then the kernels of both against their rooflines."""
    import torch
    t0 = time.time()
    out = {"metric": "lm_prefill_decode_throughput", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights)",
           "config": {"prefill": f"{PREFILL_SEQS}x{PREFILL_LEN} tokens per step", "decode": f"{DECODE_SEQS} sequences at context {DECODE_CTX}",
                      "layers": LAYERS, "window": WINDOW, "page": PAGE}, "sizes": {}}
    for name, s in SIZES.items():
        row = {"teberax_moe16top2": bench_bokenex(s, True, device, "teberax"), "teberax_dense": bench_bokenex(s, False, device, "teberax"),
               "tibivik": bench_bokenex(s, False, device, "tibivik")}
        out["sizes"][name] = row
        torch.cuda.empty_cache()
    out["kernels"] = bench_teberax_kernels(device)
    out["like_kernels"] = bench_hybrid_kernels(device)
    out["seconds"] = round(time.time() - t0, 1)
    return out


def main_hybrid(device: str = "cuda:0") -> dict:
    """``bench.py --lm-hybrid``: Tibivik beside Bokenex (the package's closest model: a token-id decoder with a short
    convolution and windowed attention over the same engine) at equal width, layer count and feed-forward parameters, then
    the kernels of both against their rooflines."""
    import torch
    t0 = time.time()
    out = {"metric": "lm_prefill_decode_throughput", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights)",
           "config": {"prefill": f"{PREFILL_SEQS}x{PREFILL_LEN} tokens per step", "decode": f"{DECODE_SEQS} sequences at context {DECODE_CTX}",
                      "layers": LAYERS, "window": WINDOW, "conv_taps": TAPS, "page": PAGE}, "sizes": {}}
    for name, s in SIZES.items():
        row = {"tibivik": bench_bokenex(s, False, device, "tibivik"), "bokenex_dense": bench_bokenex(s, False, device)}
        out["sizes"][name] = row
        torch.cuda.empty_cache()
    out["kernels"] = bench_hybrid_kernels(device)
    out["like_kernels"] = bench_kernels(device)
    out["seconds"] = round(time.time() - t0, 1)
    return out


def main_latent(device: str = "cuda:0") -> dict:
    """``bench.py --lm-latent``: Ridevik beside Bokenex (the package's closest model: a token-id decoder over the same
    engine) at equal width, layer count and feed-forward parameters, then the kernels of both against their rooflines."""
    import torch
    t0 = time.time()
    out = {"metric": "lm_prefill_decode_throughput", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights)",
           "config": {"prefill": f"{PREFILL_SEQS}x{PREFILL_LEN} tokens per step", "decode": f"{DECODE_SEQS} sequences at context {DECODE_CTX}",
                      "layers": LAYERS, "window": WINDOW, "page": PAGE}, "sizes": {}}
    for name, s in SIZES.items():
        row = {"ridevik_dense": bench_bokenex(s, False, device, "ridevik"), "ridevik_moe16top2": bench_bokenex(s, True, device, "ridevik"),
               "bokenex_dense": bench_bokenex(s, False, device), "bokenex_moe16top2": bench_bokenex(s, True, device)}
        out["sizes"][name] = row
        torch.cuda.empty_cache()
    out["kernels"] = bench_latent_kernels(device)
    out["like_kernels"] = bench_kernels(device)
    out["seconds"] = round(time.time() - t0, 1)
    return out


def main(device: str = "cuda:0") -> dict:
    import torch
    t0 = time.time()
    out = {"metric": "lm_prefill_decode_throughput", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights)",
           "config": {"prefill": f"{PREFILL_SEQS}x{PREFILL_LEN} tokens per step", "decode": f"{DECODE_SEQS} sequences at context {DECODE_CTX}",
                      "layers": LAYERS, "window": WINDOW, "conv_taps": TAPS, "page": PAGE}, "sizes": {}}
    for name, s in SIZES.items():
        row = {"bokenex_dense": bench_bokenex(s, False, device), "bokenex_moe16top2": bench_bokenex(s, True, device),
               "talker_stack": bench_talker(s, device)}
        out["sizes"][name] = row
        torch.cuda.empty_cache()
    out["kernels"] = bench_kernels(device)
    out["seconds"] = round(time.time() - t0, 1)
    return out


if __name__ == "__main__":
    print(json.dumps(main()))
