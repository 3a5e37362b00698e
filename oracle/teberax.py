"""Plain, slow restatement of the Teberax decoder (test infrastructure only: nothing in the package imports it).

One function per mechanism, whole sequences at a time, no cache, no carried state and no batching: attention looks at
the full prefix under its mask, the recurrence starts at zero and walks the sequence token by token, so the engine's
paged K/V, state slots, portions and mixed batches have something independent to be compared with.  Arithmetic is done
in the dtype of the tensors handed in (float64 in the tests).

Notation: x [T, D] the residual stream, H query heads over G key/value heads, d / dv the key and value size per head,
W a window length, F kept first tokens.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F_


# ------------------------------------------------------------------------------------------------ small pieces
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis (``weight`` a vector, one number, or None)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def rotate_pairs(v, positions, dims, base, factor=1.0):
    """v [T, heads, d]: coordinates 2i and 2i+1 (i < dims/2) of every head are turned by the angle
    position * base^(-2i/dims) / factor; coordinates from ``dims`` on pass."""
    i = torch.arange(dims // 2, dtype=v.dtype)
    ang = positions.to(v.dtype)[:, None] * (base ** (-2.0 * i / dims) / factor)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    rot = torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2)
    return torch.cat([rot, v[..., dims:]], -1)


def visible(T, window=None, keep_first=0):
    """[T, T] bool: i sees j when j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


# ------------------------------------------------------------------------------------------------ attention
def softmax_attention(q, k, v, scale, mask, softcap=None, zero_sink=False):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  ``softcap`` c: scores become c tanh(score / c).
    ``zero_sink``: the denominator gets one more term exp(0) that has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, float("-inf"))
        if zero_sink:
            s = torch.cat([s, torch.zeros(T, 1, dtype=s.dtype)], 1)
            p = torch.softmax(s, -1)[:, :T]
        else:
            p = torch.softmax(s, -1)
        out.append(p @ v[:, g])
    return torch.stack(out, 1)


def differential_attention(q, k, v, scale, mask, lam, diff, eps):
    """q [T, H, 2, d], k [T, G, 2, d], v [T, G, dv]: two softmax maps over the same values,
    o = a1 - lam * a2, each head's o divided by its root mean square, times (1 - diff)."""
    a1 = softmax_attention(q[:, :, 0], k[:, :, 0], v, scale, mask)
    a2 = softmax_attention(q[:, :, 1], k[:, :, 1], v, scale, mask)
    return rms_norm(a1 - lam * a2, None, eps) * (1.0 - diff)


def differential_lambda(lq1, lk1, lq2, lk2, diff):
    return torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + diff


def attention_mixer(h, w, m, eps, kv=None):
    """The 'attention' mixer.  ``w``: tensors by their short names; ``m``: the mixer's entry of the configuration.
    ``kv``: (k, v) of the layer whose keys and values this one borrows.  Returns (output, (k, v))."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, 2, d)
    if kv is None:
        kv = ((h @ w["k"].T).view(T, G, 2, d), (h @ w["v"].T).view(T, G, dv))
    mask_cfg = m.get("mask") or {}
    mask = visible(T, mask_cfg.get("size"), mask_cfg.get("keep_first", 0))
    lam = differential_lambda(w["lq1"], w["lk1"], w["lq2"], w["lk2"], m["diff"])
    o = differential_attention(q, kv[0], kv[1], m["scale"], mask, lam, m["diff"], eps)
    return o.reshape(T, H * dv) @ w["o"].T, kv


def biased_rotary_attention(h, w, m):
    """The left branch of a 'parallel' mixer: biased projections, pair rotation of the first rot.dims coordinates with
    linearly scaled frequencies, soft-capped scores, causal, a zero sink in the denominator."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w["q"].T + w["q.b"]).view(T, H, d)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, d)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, dv)
    r = m.get("rot")
    if r:
        factor = (r.get("scaling") or {}).get("factor", 1.0)
        q = rotate_pairs(q, pos, r["dims"], r["base"], factor)
        k = rotate_pairs(k, pos, r["dims"], r["base"], factor)
    o = softmax_attention(q, k, v, m["scale"], visible(T), m.get("softcap"), zero_sink=True)
    return o.reshape(T, H * dv) @ w["o"].T + w["o.b"]


def latent_attention_mixer(h, w, m, eps):
    """Keys and values expanded per head from one normed latent per token; one rotated key part shared by the heads."""
    T = h.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w["q"].T).view(T, H, d + dr)
    ckr = h @ w["dkv"].T
    c = rms_norm(ckr[:, :R], w["dkv.norm"], eps)
    r = m["rot"]
    factor = (r.get("scaling") or {}).get("factor", 1.0)
    kr = rotate_pairs(ckr[:, None, R:], pos, r["dims"], r["base"], factor)            # [T, 1, dr]
    qr = rotate_pairs(q[..., d:], pos, r["dims"], r["base"], factor)
    kn = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    qq = torch.cat([q[..., :d], qr], -1)
    kk = torch.cat([kn, kr.expand(T, H, dr)], -1)
    mask_cfg = m.get("mask") or {}
    o = softmax_attention(qq, kk, v, m["scale"], visible(T, mask_cfg.get("size"), 0))
    return o.reshape(T, H * dv) @ w["o"].T


# ------------------------------------------------------------------------------------------------ recurrence
def gated_linear_attention(h, w, m, eps):
    """The right branch of a 'parallel' mixer: S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, with a
    decay per key channel alpha = sigmoid(z)^(1/tau); head norm, SiLU gate, output projection."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.exp(F_.logsigmoid(z) / m["tau"]).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = []
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o.append(torch.einsum("hdv,hd->hv", S, q[t]))
    o = rms_norm(torch.stack(o), w["norm"], eps).reshape(T, H * dv)
    g = h @ w["g"].T
    return (o * g * torch.sigmoid(g)) @ w["o"].T


def parallel_mixer(h, w, m, eps):
    """Half the sum of the two branches, each RMS-normed over the model width with its own weight."""
    left = {k[5:]: t for k, t in w.items() if k.startswith("left.") and k != "left.out"}
    right = {k[6:]: t for k, t in w.items() if k.startswith("right.") and k != "right.out"}
    a = biased_rotary_attention(h, left, m["left"])
    b = gated_linear_attention(h, right, m["right"], eps)
    return 0.5 * (rms_norm(a, w["left.out"], eps) + rms_norm(b, w["right.out"], eps))


# ------------------------------------------------------------------------------------------------ feed-forwards
def polynorm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e with N = division by the root mean square over the last axis."""
    a, b, c, e = coef
    return a * rms_norm(z, None, eps) + b * rms_norm(z * z, None, eps) + c * rms_norm(z ** 3, None, eps) + e


def dense_ff(h, w, eps):
    return polynorm(h @ w["up"].T, w["act"], eps) @ w["down"].T


def route(h, router, correction, top):
    """Softmax over all router outputs; the ``top`` largest of score + correction are chosen; weights are the scores."""
    s = torch.softmax(h @ router.T, -1)
    idx = torch.topk(s + correction, top, dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def moe_ff(h, w, f):
    """Mixture of SiLU-gated experts; the last ``identity`` router outputs stand for experts that return their input."""
    E, top = f["router"]["experts"], f["router"]["top"]
    idx, wt = route(h, w["router"], w["correction"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(idx[t].tolist(), wt[t]):
            if e >= E:
                out[t] += p * h[t]
            else:
                g = h[t] @ w[f"e{e}.gate"].T
                out[t] += p * ((g * torch.sigmoid(g) * (h[t] @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T)
    return out


# ------------------------------------------------------------------------------------------------ the model
def sub(sd, prefix):
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


def forward(cfg: dict, sd: dict, tokens, trace=None):
    """tokens: a list of ids -> logits [T, vocab].  ``sd``: checkpoint names -> tensors (already in the working dtype).
    ``trace``: a list that receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = rms_norm(sd["embed"][torch.tensor(tokens)], sd["embed.norm"], eps)
    kvs = {}
    for i, layer in enumerate(cfg["layers"]):
        w = sub(sd, f"l{i}.")
        h = rms_norm(x, w["norm1"], eps)
        m, mw = layer["mixer"], sub(w, "mix.")
        if layer["type"] == "attention":
            y, kvs[i] = attention_mixer(h, mw, m, eps, kvs[m["kv_from"]] if m.get("kv_from") is not None else None)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, mw, m, eps)
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(h, mw, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w["norm1b"], eps)
        f = layer.get("mlp")
        if f is not None:
            h = rms_norm(x, w["norm2"], eps)
            y = dense_ff(h, sub(w, "mlp."), eps) if f["kind"] == "dense" else moe_ff(h, sub(w, "mlp."), f)
            x = x + rms_norm(y, w["norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    logits = rms_norm(x, sd["final.norm"], eps) @ sd["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
