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


# ------------------------------------------------------------------------------------------------ small random models
def random_config(vocab=61, width=24, types=("parallel", "latent_attention", "attention", "attention"), kv_from=None,
                  ff=("dense", "moe", "moe", None), logit_softcap=9.0, eps=1e-5, attention=None, left=None, right=None,
                  latent=None, moe=None, dense_ff=20) -> dict:
    """A small configuration in the checkpoint's format.  ``types``: the mixers in order; ``kv_from``: {layer: source};
    ``ff``: per layer "dense", "moe" or None; the dicts override fields of the matching mixer / feed-forward."""
    att = dict(heads=4, kv_heads=2, dim=6, vdim=10, diff=0.3, scale=0.5, mask={"size": 9, "keep_first": 2})
    att.update(attention or {})
    lf = dict(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.4, softcap=3.0, rot={"dims": 4, "base": 100.0, "scaling": {"factor": 4.0}})
    lf.update(left or {})
    rt = dict(heads=2, dim=5, vdim=7, tau=4.0, decay_rank=3)
    rt.update(right or {})
    lat = dict(heads=3, dim=6, rot_dim=4, vdim=5, kv_rank=12, scale=0.35, mask={"size": 11}, rot={"dims": 4, "base": 50.0})
    lat.update(latent or {})
    me = dict(kind="moe", expert={"ff": 10}, router={"experts": 5, "identity": 2, "top": 3})
    me.update(moe or {})
    layers = []
    for i, kind in enumerate(types):
        if kind == "attention":
            m = dict(att)
            if kv_from and i in kv_from:
                m["kv_from"] = kv_from[i]
        elif kind == "parallel":
            m = {"left": dict(lf), "right": dict(rt)}
        else:
            m = dict(lat)
        f = ff[i % len(ff)]
        mlp = None if f is None else ({"kind": "dense", "ff": dense_ff} if f == "dense" else dict(me))
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    out = {"architecture": "Teberax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if logit_softcap:
        out["logit_softcap"] = logit_softcap
    return out


def tensor_shapes(cfg: dict) -> dict:
    D, sh = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "embed.norm": (), "final.norm": (), "head": (cfg["vocab"], cfg["width"])}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        sh[p + "norm1"] = sh[p + "norm1b"] = ()
        if layer["type"] == "attention":
            sh[p + "mix.q"] = (m["heads"] * 2 * m["dim"], D)
            if m.get("kv_from") is None:
                sh[p + "mix.k"], sh[p + "mix.v"] = (m["kv_heads"] * 2 * m["dim"], D), (m["kv_heads"] * m["vdim"], D)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                sh[p + "mix." + n] = (m["dim"],)
            sh[p + "mix.o"] = (D, m["heads"] * m["vdim"])
        elif layer["type"] == "parallel":
            a, r = m["left"], m["right"]
            for n, rows in (("q", a["heads"] * a["dim"]), ("k", a["kv_heads"] * a["dim"]), ("v", a["kv_heads"] * a["vdim"])):
                sh[f"{p}mix.left.{n}"], sh[f"{p}mix.left.{n}.b"] = (rows, D), (rows,)
            sh[p + "mix.left.o"], sh[p + "mix.left.o.b"], sh[p + "mix.left.out"] = (D, a["heads"] * a["vdim"]), (D,), (D,)
            hd, hv, rk = r["heads"] * r["dim"], r["heads"] * r["vdim"], r["decay_rank"]
            for n, rows in (("q", hd), ("k", hd), ("v", hv), ("g", hv), ("a1", rk)):
                sh[f"{p}mix.right.{n}"] = (rows, D)
            sh[p + "mix.right.a2"], sh[p + "mix.right.a2.b"], sh[p + "mix.right.norm"] = (hd, rk), (hd,), (r["vdim"],)
            sh[p + "mix.right.o"], sh[p + "mix.right.out"] = (D, hv), (D,)
        else:
            sh[p + "mix.q"], sh[p + "mix.dkv"] = (m["heads"] * (m["dim"] + m["rot_dim"]), D), (m["kv_rank"] + m["rot_dim"], D)
            sh[p + "mix.dkv.norm"] = (m["kv_rank"],)
            sh[p + "mix.uk"], sh[p + "mix.uv"] = (m["heads"] * m["dim"], m["kv_rank"]), (m["heads"] * m["vdim"], m["kv_rank"])
            sh[p + "mix.o"] = (D, m["heads"] * m["vdim"])
        f = layer.get("mlp")
        if f is None:
            continue
        sh[p + "norm2"] = sh[p + "norm2b"] = ()
        if f["kind"] == "dense":
            sh[p + "mlp.up"], sh[p + "mlp.down"], sh[p + "mlp.act"] = (f["ff"], D), (D, f["ff"]), (4,)
        else:
            n_out = f["router"]["experts"] + f["router"].get("identity", 0)
            sh[p + "mlp.router"], sh[p + "mlp.correction"] = (n_out, D), (n_out,)
            for e in range(f["router"]["experts"]):
                sh[f"{p}mlp.e{e}.gate"] = sh[f"{p}mlp.e{e}.up"] = (f["expert"]["ff"], D)
                sh[f"{p}mlp.e{e}.down"] = (D, f["expert"]["ff"])
    return sh


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """Random tensors under the checkpoint's names, rounded to bfloat16 (what a file would hold), returned as float64."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        leaf = name.rsplit(".", 1)[-1]
        t = torch.randn(shape, generator=g)
        if len(shape) == 0:
            t = 1.0 + 0.2 * t
        elif len(shape) == 2:
            t = t * (1.5 if leaf == "router" else 1.0) * shape[1] ** -0.5
        elif leaf in ("norm", "out"):
            t = 1.0 + 0.2 * t
        elif leaf == "act":
            t = torch.tensor([1.0, 0.4, 0.2, 0.1]) + 0.1 * t
        elif leaf == "correction":
            t = 0.05 * t
        else:
            t = 0.4 * t
        sd[name] = t.to(torch.bfloat16).double()
    return sd
