"""Plain, slow restatement of the Tibivik decoder (test infrastructure only: nothing in the package imports it).

One function per mechanism, whole sequences at a time, no cache, no carried state and no batching: attention looks at
the full prefix under its mask, every recurrence starts at zero and walks the sequence token by token, so the engine's
paged K/V, state slots, portions and mixed batches have something independent to be compared with.  Arithmetic is done
in the dtype of the tensors handed in (float64 in the tests).

Notation: x [T, D] one residual stream, s streams, H query heads over G key/value heads, d / dv the key and value size
per head, N the state size of the state-space layer, W a mask size (window length or chunk length).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------ small pieces
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis (``weight`` None: no multiplication)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def causal_conv(u, taps_w, bias=None):
    """u [T, C]; taps_w [C, K]: y_t = sum_j taps_w[:, K-1-j] * u_(t-j), zeros before the start."""
    T, C = u.shape
    K = taps_w.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + pad[j:j + T] * taps_w[:, j]
    return y if bias is None else y + bias


def rotate_half(v, positions, dims, base):
    """v [T, heads, d]: coordinate i < dims/2 of every head is paired with i + dims/2 and the pair turned by the
    angle position * base^(-2i/dims); coordinates from ``dims`` on pass."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    ang = positions.to(v.dtype)[:, None] * base ** (-2.0 * i / dims)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], -1)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every position: a hash of (previous token, token); the first position reads the
    extra last row."""
    rows = [buckets]
    for t in range(1, len(tokens)):
        rows.append((tokens[t - 1] * mul_prev + tokens[t] * mul_cur) % buckets)
    return torch.tensor(rows, dtype=torch.long)


# ------------------------------------------------------------------------------------------------ attention
def sink_softmax_attention(q, k, v, scale, mask_kind, W, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  ``mask_kind`` "window": i sees j with 0 <= i - j < W;
    "chunk": i sees j <= i with i // W == j // W.  ``sink`` [H]: exp(sink_h) joins the denominator and nothing else."""
    T, H, _ = q.shape
    G = k.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    if mask_kind == "window":
        seen = (j <= i) & (i - j < W)
    elif mask_kind == "chunk":
        seen = (j <= i) & (i // W == j // W)
    else:
        raise ValueError(mask_kind)
    out = []
    for h in range(H):
        g = h // (H // G)
        sc = (q[:, h] @ k[:, g].T) * scale
        sc = sc.masked_fill(~seen, -math.inf)
        m = torch.maximum(sc.max(-1, keepdim=True).values, sink[h])
        e = torch.exp(sc - m)
        den = e.sum(-1, keepdim=True) + torch.exp(sink[h] - m)
        out.append((e / den) @ v[:, g])
    return torch.stack(out, 1)


def window_attention_branch(h, p, m, eps):
    """The sliding-window branch: values are the raw key projections; q and k are RMS-normed over their whole
    projection, then rotated."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = h @ p["q"].T
    k = h @ p["k"].T
    v = k.reshape(T, G, d)
    q = rms_norm(q, p["q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k, p["k.norm"], eps).reshape(T, G, d)
    pos = torch.arange(T)
    r = m["rot"]
    q, k = rotate_half(q, pos, r["dims"], r["base"]), rotate_half(k, pos, r["dims"], r["base"])
    o = sink_softmax_attention(q, k, v, m["scale"], "window", m["mask"]["size"], p["sink"])
    return o.reshape(T, -1) @ p["o"].T


def chunk_attention_branch(h, p, m):
    """The chunked branch: biased projections, no positions, a sigmoid gate per head on the output."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T + p["q.b"]).reshape(T, H, d)
    k = (h @ p["k"].T + p["k.b"]).reshape(T, G, d)
    v = (h @ p["v"].T + p["v.b"]).reshape(T, G, dv)
    o = sink_softmax_attention(q, k, v, m["scale"], "chunk", m["mask"]["size"], p["sink"])
    o = o * torch.sigmoid(h @ p["g"].T)[:, :, None]
    return o.reshape(T, -1) @ p["o"].T


# ------------------------------------------------------------------------------------------------ recurrences
def matrix_memory(h, p, m, eps):
    """Matrix memory with exponential gates kept stable by a running maximum that starts at 0."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ p["q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ p["k"].T).reshape(T, H, d)
    v = (h @ p["v"].T).reshape(T, H, dv)
    li = cap * torch.tanh((h @ p["i"].T + p["i.b"]) / cap)
    lf = F.logsigmoid(cap * torch.tanh((h @ p["f"].T + p["f.b"]) / cap))
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    n = torch.zeros(H, d, dtype=h.dtype)
    mx = torch.zeros(H, dtype=h.dtype)
    out = []
    for t in range(T):
        m_new = torch.maximum(lf[t] + mx, li[t])
        a = torch.exp(lf[t] + mx - m_new)
        b = torch.exp(li[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out.append(num / den[:, None])
    o = torch.stack(out)                                           # [T, H, dv]
    o = rms_norm(o, None, eps).reshape(T, H * dv) * p["norm"]
    return (o * torch.sigmoid(h @ p["g"].T)) @ p["o"].T


def gated_delta(h, p, m, eps):
    """Delta-rule memory with one decay per head; q and k are shared by the value heads of a group."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = F.silu(causal_conv(h @ p["q"].T, p["q.conv"])).reshape(T, G, d)
    k = F.silu(causal_conv(h @ p["k"].T, p["k.conv"])).reshape(T, G, d)
    v = F.silu(causal_conv(h @ p["v"].T, p["v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ p["b"].T)
    decay = torch.exp(-torch.exp(p["A_log"]) * F.softplus(h @ p["a"].T + p["dt_bias"]))
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    out = []
    for t in range(T):
        o_t = []
        for hh in range(H):
            g = hh // (H // G)
            Sh = decay[t, hh] * S[hh]
            u = beta[t, hh] * (v[t, hh] - Sh.T @ k[t, g])
            Sh = Sh + k[t, g][:, None] * u[None, :]
            S[hh] = Sh
            o_t.append(Sh.T @ q[t, g])
        out.append(torch.stack(o_t))
    o = torch.stack(out)                                           # [T, H, dv]
    o = rms_norm(o, p["norm"], eps).reshape(T, H * dv)
    return (o * F.silu(h @ p["g"].T)) @ p["o"].T


def state_space(h, p, m, eps):
    """Selective state space with a scalar decay per head."""
    T = h.shape[0]
    H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * dv
    u = h @ p["in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = F.silu(causal_conv(xbc, p["conv"], p["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = F.softplus(dt + p["dt_bias"])
    decay = torch.exp(-torch.exp(p["A_log"]) * dt)
    S = torch.zeros(H, N, dv, dtype=h.dtype)
    ys = []
    for t in range(T):
        y_t = []
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = decay[t, hh] * S[hh] + dt[t, hh] * B[t, g][:, None] * x[t, hh][None, :]
            y_t.append(S[hh].T @ C[t, g] + p["D"][hh] * x[t, hh])
        ys.append(torch.stack(y_t))
    y = torch.stack(ys).reshape(T, inner) * F.silu(z)
    ng = m["norm_groups"]
    y = rms_norm(y.reshape(T, ng, inner // ng), None, eps).reshape(T, inner) * p["norm"]
    return y @ p["o"].T


def gated_ff(h, p):
    return (F.silu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


# ------------------------------------------------------------------------------------------------ the model
def _sub(sd, prefix):
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


def mixer(h, sd, i, spec, eps):
    kind, m = spec["type"], spec["mixer"]
    if kind == "mamba2":
        return state_space(h, _sub(sd, f"l{i}.mix."), m, eps)
    left, right = _sub(sd, f"l{i}.mix.left."), _sub(sd, f"l{i}.mix.right.")
    if kind == "parallel":
        a, b = window_attention_branch(h, left, m["left"], eps), matrix_memory(h, right, m["right"], eps)
    elif kind == "parallel_2":
        a, b = chunk_attention_branch(h, left, m["left"]), gated_delta(h, right, m["right"], eps)
    else:
        raise ValueError(kind)
    return m["left_scale"] * a + m["right_scale"] * b


def layer_order(config):
    """Layer indices in the order they run: the looped range is repeated in a row."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(sd: dict, config: dict, tokens, dtype=torch.float64, layers_out: list | None = None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` collects the sum of the streams after every layer run."""
    sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
    eps = config["norm"]["eps"]
    tok = torch.tensor(list(tokens), dtype=torch.long)
    x = sd["embed"][tok]
    bg = config.get("embedding", {}).get("bigram")
    if bg:
        x = x + sd["bigram"][bigram_rows(list(tokens), bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    s = config.get("streams")
    xs = [x.clone() for _ in range(s or 1)]
    for i in layer_order(config):
        spec = config["layers"][i]
        for q, fn in ((1, lambda hh: mixer(hh, sd, i, spec, eps)),
                      (2, (lambda hh: gated_ff(hh, _sub(sd, f"l{i}.mlp."))) if spec.get("mlp") else None)):
            if fn is None:
                continue
            if s:
                w_in, w_out, w_mix = sd[f"l{i}.hc{q}.in"], sd[f"l{i}.hc{q}.out"], sd[f"l{i}.hc{q}.mix"]
                u = sum(w_in[a] * xs[a] for a in range(s))
                y = fn(rms_norm(u, sd[f"l{i}.norm{q}"], eps))
                xs = [sum(w_mix[a, t] * xs[a] for a in range(s)) + w_out[t] * y for t in range(s)]
            else:
                xs = [xs[0] + fn(rms_norm(xs[0], sd[f"l{i}.norm{q}"], eps))]
        if layers_out is not None:
            layers_out.append(sum(xs))
    return rms_norm(sum(xs), sd["final.norm"], eps) @ sd["embed"].T


# ------------------------------------------------------------------------------------------------ random models for tests
def random_config(*, width=40, vocab=53, streams=2, bigram=(31, 5, 3), types=("mamba2", "parallel_2", "parallel"), loop=None,
                  ff=(24, None, 56), eps=1e-5, ssm=None, window=None, chunk=None, memory=None, delta=None,
                  scales=(0.7, 1.2)) -> dict:
    """A small configuration; ``ssm`` / ``window`` / ``chunk`` / ``memory`` / ``delta`` override the default sizes of
    the state-space mixer, the two attention branches and the two recurrent branches; ``ff`` cycles over the layers
    (None: no feed-forward); ``bigram`` = (buckets, mul_prev, mul_cur) or None; ``streams`` 0: one plain residual."""
    s = dict(heads=3, vdim=8, state=6, groups=1, conv=3, norm_groups=1)
    s.update(ssm or {})
    w = dict(heads=4, kv_heads=2, dim=12, vdim=12, mask={"size": 7}, scale=0.3, rot={"dims": 8, "base": 100.0})
    w.update(window or {})
    c = dict(heads=3, kv_heads=1, dim=10, vdim=6, mask={"size": 5}, scale=0.25)
    c.update(chunk or {})
    m = dict(heads=2, dim=6, vdim=10, gate_cap=8.0)
    m.update(memory or {})
    d = dict(heads=4, kv_heads=2, dim=6, vdim=5, conv=4)
    d.update(delta or {})
    layers = []
    for i, kind in enumerate(types):
        f = ff[i % len(ff)]
        mlp = {"kind": "dense", "ff": f} if f else None
        if kind == "mamba2":
            mixer = dict(s)
        elif kind == "parallel":
            mixer = {"left": dict(w), "right": dict(m), "left_scale": scales[0], "right_scale": scales[1]}
        else:
            mixer = {"left": dict(c), "right": dict(d), "left_scale": scales[0], "right_scale": scales[1]}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Tibivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams:
        cfg["streams"] = streams
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(config: dict, seed: int = 0) -> dict:
    """Random tensors (rounded to bfloat16, as a checkpoint stores them) under the checkpoint's names."""
    g = torch.Generator().manual_seed(seed)
    D = config["width"]
    sd = {}

    def put(name, *shape, std=1.0, mean=0.0):
        sd[name] = (mean + std * torch.randn(shape, generator=g)).to(torch.bfloat16).to(torch.float32)

    put("embed", config["vocab"], D)
    bg = config.get("embedding", {}).get("bigram")
    if bg:
        put("bigram", bg["buckets"] + 1, D, std=0.5)
    put("final.norm", D, mean=1.0, std=0.1)
    s = config.get("streams")
    for i, spec in enumerate(config["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        subs = [1] + ([2] if spec.get("mlp") else [])
        for q in subs:
            put(f"{p}norm{q}", D, mean=1.0, std=0.1)
            if s:
                put(f"{p}hc{q}.in", s, mean=0.7, std=0.3)
                put(f"{p}hc{q}.out", s, mean=0.8, std=0.3)
                sd[f"{p}hc{q}.mix"] = (torch.eye(s) + 0.25 * torch.randn(s, s, generator=g)).to(torch.bfloat16).to(torch.float32)
        if spec.get("mlp"):
            f = spec["mlp"]["ff"]
            put(p + "mlp.gate", f, D, std=D ** -0.5)
            put(p + "mlp.up", f, D, std=D ** -0.5)
            put(p + "mlp.down", D, f, std=f ** -0.5)
        if spec["type"] == "mamba2":
            inner, ch = m["heads"] * m["vdim"], m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
            put(p + "mix.in", inner + ch + m["heads"], D, std=D ** -0.5)
            put(p + "mix.conv", ch, m["conv"], std=0.5)
            put(p + "mix.conv.b", ch, std=0.2)
            put(p + "mix.dt_bias", m["heads"], std=0.5)
            put(p + "mix.A_log", m["heads"], std=0.5, mean=-0.5)
            put(p + "mix.D", m["heads"], std=0.5)
            put(p + "mix.norm", inner, mean=1.0, std=0.1)
            put(p + "mix.o", D, inner, std=inner ** -0.5)
            continue
        l, r = m["left"], m["right"]
        L, R = p + "mix.left.", p + "mix.right."
        put(L + "q", l["heads"] * l["dim"], D, std=D ** -0.5)
        put(L + "k", l["kv_heads"] * l["dim"], D, std=D ** -0.5)
        put(L + "sink", l["heads"], std=1.0)
        put(L + "o", D, l["heads"] * l["vdim"], std=(l["heads"] * l["vdim"]) ** -0.5)
        if spec["type"] == "parallel":
            put(L + "q.norm", l["heads"] * l["dim"], mean=1.0, std=0.1)
            put(L + "k.norm", l["kv_heads"] * l["dim"], mean=1.0, std=0.1)
            hd, hv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            for n, rows in (("q", hd), ("k", hd), ("v", hv), ("g", hv), ("i", r["heads"]), ("f", r["heads"])):
                put(R + n, rows, D, std=D ** -0.5)
            put(R + "i.b", r["heads"], std=0.5)
            put(R + "f.b", r["heads"], std=0.5, mean=1.0)
            put(R + "norm", hv, mean=1.0, std=0.1)
            put(R + "o", D, hv, std=hv ** -0.5)
        else:
            put(L + "v", l["kv_heads"] * l["vdim"], D, std=D ** -0.5)
            put(L + "g", l["heads"], D, std=D ** -0.5)
            for n, rows in (("q.b", l["heads"] * l["dim"]), ("k.b", l["kv_heads"] * l["dim"]), ("v.b", l["kv_heads"] * l["vdim"])):
                put(L + n, rows, std=0.3)
            gd, hv = r["kv_heads"] * r["dim"], r["heads"] * r["vdim"]
            for n, rows in (("q", gd), ("k", gd), ("v", hv)):
                put(R + n, rows, D, std=D ** -0.5)
                put(R + n + ".conv", rows, r["conv"], std=0.5)
            put(R + "g", hv, D, std=D ** -0.5)
            put(R + "b", r["heads"], D, std=D ** -0.5)
            put(R + "a", r["heads"], D, std=D ** -0.5)
            put(R + "A_log", r["heads"], std=0.5, mean=-0.5)
            put(R + "dt_bias", r["heads"], std=0.5)
            put(R + "norm", r["vdim"], mean=1.0, std=0.1)
            put(R + "o", D, hv, std=hv ** -0.5)
    return sd
