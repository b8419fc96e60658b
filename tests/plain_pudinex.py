"""A plain, slow Pudinex in 64-bit numpy: one function per mechanism, whole sequences only.

It shares nothing with the engine: no kernels, no cache, no step function. A sequence goes in whole and the logits
of every position come out; the recurrence is a Python loop over the tokens, every attention row is worked out by itself
from the keys it may see. `w` maps tensor names to 64-bit arrays, `cfg` is the parsed config.json.

Notation. T tokens, E the model's width. n_g(v): v cut into `groups` equal consecutive parts, each divided by its own
sqrt(mean(part^2) + eps), the whole times a weight. A layer is x <- x + mixer(h) + ff(h) with the one h = n_g(x);
the stream starts as embed[token] * embedding.scale; the logits are head n_g(x).
"""
from __future__ import annotations

import math

import numpy as np

ROUND = None  # a function that rounds an array to the engine's 16-bit format, or None: exact


def mm(a, W):
    """a W^T; with `ROUND` set, `a` is rounded first, as a 16-bit engine rounds what enters a contraction."""
    return (ROUND(a) if ROUND is not None else a) @ W.T


def rms(v, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def silu(v):
    return v * sigmoid(v)


def group_norm(x, weight, groups, eps):
    T, E = x.shape
    return rms(x.reshape(T, groups, E // groups), eps).reshape(T, E) * weight


# ----------------------------------------------------------------------------------------------- rotation
def yarn_frequencies(rot):
    """The dims/2 angular frequencies: base^(-2i/dims), the slow ones divided by `factor` along a ramp between the
    pair numbers at which `original` positions make `fast` and `slow` turns. Returns (frequencies, the factor on cos
    and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(v, positions, rot):
    """Entry i of the first `dims` entries turns together with entry i + dims/2; the rest pass. v: [T, heads, d]."""
    dims = int(rot["dims"])
    f, mag = yarn_frequencies(rot)
    out = v.copy()
    half = dims // 2
    for t, p in enumerate(positions):
        for i in range(half):
            a = p * f[i]
            c, s = math.cos(a) * mag, math.sin(a) * mag
            lo, hi = v[t, :, i].copy(), v[t, :, i + half].copy()
            out[t, :, i] = lo * c - hi * s
            out[t, :, i + half] = hi * c + lo * s
    return out


# ----------------------------------------------------------------------------------------------- mixers
def sink_attention(h, w, p, m, eps):
    """Causal softmax attention whose denominator holds one more term, exp(0), that no value belongs to. Queries and
    keys are normed per head (with a weight) before they turn; values are normed per head (no weight) before they are
    kept; a score is capped smoothly: cap tanh(s / cap)."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    G = m.get("kv_heads") or H
    dv = m.get("vdim") or d
    q = rms(mm(h, w[p + "q"]).reshape(T, H, d), eps) * w[p + "q.norm"]
    k = rms(mm(h, w[p + "k"]).reshape(T, G, d), eps) * w[p + "k.norm"]
    v = rms(mm(h, w[p + "v"]).reshape(T, G, dv), eps)
    if m.get("rot"):
        q = rotate_half(q, range(T), m["rot"])
        k = rotate_half(k, range(T), m["rot"])
    if ROUND is not None:
        k, v = ROUND(k), ROUND(v)  # the cache holds 16-bit keys and values
    scale = m["scale"] if m.get("scale") is not None else d ** -0.5
    cap = m.get("softcap")
    out = np.zeros((T, H, dv))
    for t in range(T):
        for a in range(H):
            kv = a // (H // G)
            s = (k[:t + 1, kv] @ q[t, a]) * scale  # the keys 0..t of this row's key head
            if cap:
                s = cap * np.tanh(s / cap)
            top = max(s.max(), 0.0)
            e = np.exp(s - top)
            pr = e / (math.exp(-top) + e.sum())
            out[t, a] = pr @ v[:t + 1, kv]
    return mm(out.reshape(T, H * dv), w[p + "o"])


def hgrn2(h, w, p, m, eps):
    """Linear attention whose forget gate is also one minus its write strength. Per head S [dim, vdim], token by token:
    S <- f[:, None] * S + (1 - f)[:, None] * v[None, :];  o = S^T q. f = l + (1 - l) sigmoid(W_f h + b) with a lower
    bound l per head and channel."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(mm(h, w[p + "q"])).reshape(T, H, d)
    v = mm(h, w[p + "v"]).reshape(T, H, dv)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * sigmoid(mm(h, w[p + "f"]) + w[p + "f.b"])).reshape(T, H, d)
    out = np.zeros((T, H, dv))
    for a in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = f[t, a][:, None] * S + np.outer(1.0 - f[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    out = rms(out, eps) * w[p + "norm"]
    return mm(out.reshape(T, H * dv), w[p + "o"])


# ----------------------------------------------------------------------------------------------- feed-forwards
def capped_glu(f, w, p, limit):
    """down(g sigmoid(1.702 g) (u + 1)) with g = min(gate f, limit) and u = clamp(up f, -limit, limit)."""
    g = np.minimum(mm(f, w[p + "gate"]), limit)
    u = np.clip(mm(f, w[p + "up"]), -limit, limit)
    return mm(g * sigmoid(1.702 * g) * (u + 1.0), w[p + "down"])


def silu_glu(f, w, p):
    return mm(silu(mm(f, w[p + "gate"])) * mm(f, w[p + "up"]), w[p + "down"])


def routed_ff(f, w, p, mlp):
    """Scores are a softmax over all router outputs; the `top` largest of score + correction are chosen; a chosen one's
    weight is its score (without the correction) over the sum of the chosen scores. The last `identity` router outputs
    stand for experts that return their input. A shared expert, if the layer has one, is added for every token."""
    r = mlp["router"]
    n, ident, top = int(r["experts"]), int(r.get("identity") or 0), int(r["top"])
    z = mm(f, w[p + "router"])
    out = np.zeros_like(f)
    inp = ROUND(f) if ROUND is not None else f
    for t in range(f.shape[0]):
        s = np.exp(z[t] - z[t].max())
        s = s / s.sum()
        choice = s + w[p + "correction"]
        chosen = sorted(range(n + ident), key=lambda e: (-choice[e], e))[:top]
        total = sum(s[e] for e in chosen) + 1e-20
        for e in sorted(chosen):
            g = s[e] / total
            out[t] += g * (inp[t] if e >= n else silu_glu(f[t:t + 1], w, f"{p}e{e}.")[0])
    if mlp.get("shared"):
        out += silu_glu(f, w, p + "shared.")
    return out


# ----------------------------------------------------------------------------------------------- the model
def mixer(h, w, i, layer, eps):
    p = f"l{i}.mix."
    if layer["type"] == "attention":
        return sink_attention(h, w, p, layer["mixer"], eps)
    if layer["type"] == "hgrn2":
        return hgrn2(h, w, p, layer["mixer"], eps)
    raise ValueError(layer["type"])


def feed_forward(f, w, i, layer):
    mlp, p = layer["mlp"], f"l{i}.mlp."
    if mlp.get("kind", "dense") == "moe":
        return routed_ff(f, w, p, mlp)
    return capped_glu(f, w, p, float(mlp["limit"]))


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence. `layers_out`: a list that receives the stream after every layer."""
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups") or 1)
    x = w["embed"][np.asarray(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(cfg["layers"]):
        h = group_norm(x, w[f"l{i}.norm1"], groups, eps)
        y = mixer(h, w, i, layer, eps)
        if layer.get("mlp"):
            y = y + feed_forward(h, w, i, layer)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    return mm(group_norm(x, w["final.norm"], groups, eps), w["head"])
