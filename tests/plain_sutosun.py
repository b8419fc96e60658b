"""A plain, slow Sutosun in 64-bit numpy: one function per mechanism, whole sequences only.

It shares nothing with the engine: no kernels, no cache, no step function. A sequence goes in whole and the logits of
every position come out; recurrences are Python loops over the tokens, every attention row is worked out by itself from
the keys it may see. `w` maps tensor names to 64-bit arrays, `cfg` is the parsed config.json.

Notation. T tokens, E the model's width, n(v) = v / sqrt(mean(v^2) + eps). The stream starts as n(embed[token]) times
`embed.norm`; a layer is x <- x + mixer(n(x) w1), then x <- x + ff(n(x) w2) where the layer has a feed-forward; the
logits are c tanh(head (n(x) w_final) / c). A layer entry with `weights_of`: j runs with layer j's tensors.
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


def gelu_tanh(v):
    return 0.5 * v * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (v + 0.044715 * v ** 3)))


# ----------------------------------------------------------------------------------------------- rotation
def frequencies(rot):
    """The dims/2 angular frequencies base^(-2i/dims); with `scaling` (YaRN) the slow ones are divided by `factor` along
    a ramp between the pair numbers at which `original` positions make `fast` and `slow` turns. Returns (frequencies,
    the factor on cos and sin)."""
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
    f, mag = frequencies(rot)
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


def sink_softmax(s, sink):
    """Weights of the scores s when the denominator holds one more term exp(sink) that no value belongs to."""
    top = max(float(s.max()), sink)
    e = np.exp(s - top)
    return e / (math.exp(sink - top) + e.sum())


# ----------------------------------------------------------------------------------------------- mixers
def gated_attention(h, w, p, m, eps):
    """Causal softmax attention without rotation. Queries and keys (with biases) are normed over the whole projection,
    all heads at once, with a weight of that size; the query at position t is multiplied by
    1 + coef ln(floor((t + 1) / every) + 1); the denominator holds exp(sink) of the head; a head's output is
    multiplied by the sigmoid of one number per head."""
    T = h.shape[0]
    H, d = int(m["heads"]), int(m["dim"])
    G = int(m.get("kv_heads") or H)
    dv = int(m.get("vdim") or d)
    q = rms(mm(h, w[p + "q"]) + w[p + "q.b"], eps) * w[p + "q.norm"]
    k = rms(mm(h, w[p + "k"]) + w[p + "k.b"], eps) * w[p + "k.norm"]
    v = mm(h, w[p + "v"]) + w[p + "v.b"]
    qt = m.get("q_temp")
    if qt:
        temp = np.array([1.0 + float(qt["coef"]) * math.log((t + 1) // int(qt["every"]) + 1) for t in range(T)])
        q = q * temp[:, None]
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    if ROUND is not None:
        k, v = ROUND(k), ROUND(v)  # the cache holds 16-bit keys and values
    gate = sigmoid(mm(h, w[p + "g"]))  # [T, H]
    out = np.zeros((T, H, dv))
    for t in range(T):
        for a in range(H):
            kv = a // (H // G)
            pr = sink_softmax((k[:t + 1, kv] @ q[t, a]) * float(m["scale"]), float(w[p + "sink"][a]))
            out[t, a] = (pr @ v[:t + 1, kv]) * gate[t, a]
    return mm(out.reshape(T, H * dv), w[p + "o"])


def retention(h, w, p, m, eps):
    """Linear attention with one fixed decay per head, no softmax and no denominator. Per head S [dim, vdim] from zero:
    S <- decay S + k v^T, o = S^T q, with q and k turned by position and k times dim^(-1/2) after that; o is divided
    by its root mean square per head, and the concatenated heads are multiplied by silu(W_g h)."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = mm(h, w[p + "q"]).reshape(T, H, d)
    k = mm(h, w[p + "k"]).reshape(T, H, d)
    v = mm(h, w[p + "v"]).reshape(T, H, dv)
    if m.get("rot"):
        q = rotate_half(q, range(T), m["rot"])
        k = rotate_half(k, range(T), m["rot"])
    k = k * d ** -0.5
    out = np.zeros((T, H, dv))
    for a in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = float(m["decay"][a]) * S + np.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    out = rms(out, eps).reshape(T, H * dv) * silu(mm(h, w[p + "g"]))
    return mm(out, w[p + "o"])


def latent_attention(h, w, p, m, eps):
    """Causal softmax attention whose keys and values are made from a small normed latent c per position, plus one
    turned key part that all heads share. Head a: key [U_a c | turned part], value V_a c, query [plain | turned]."""
    T = h.shape[0]
    H, d, dr, dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = mm(h, w[p + "q"]).reshape(T, H, d + dr)
    down = mm(h, w[p + "dkv"])
    c = rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = down[:, rank:].reshape(T, 1, dr)
    q_plain, q_rot = q[:, :, :d], q[:, :, d:]
    if m.get("rot"):
        q_rot = rotate_half(q_rot, range(T), m["rot"])
        k_rot = rotate_half(k_rot, range(T), m["rot"])
    if ROUND is not None:
        c, k_rot = ROUND(c), ROUND(k_rot)  # what the cache holds
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, d)
    val = (c @ w[p + "uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for t in range(T):
        for a in range(H):
            s = (k_plain[:t + 1, a] @ q_plain[t, a] + k_rot[:t + 1, 0] @ q_rot[t, a]) * float(m["scale"])
            out[t, a] = sink_softmax(s, float(w[p + "sink"][a])) @ val[:t + 1, a]
    return mm(out.reshape(T, H * dv), w[p + "o"])


# ----------------------------------------------------------------------------------------------- feed-forwards
def gated_unit(f, w, p, act):
    return mm(act(mm(f, w[p + "gate"])) * mm(f, w[p + "up"]), w[p + "down"])


def chosen_experts(z, top):
    """The `top` largest logits (the lower number on a tie) and the softmax over just those."""
    chosen = sorted(range(len(z)), key=lambda e: (-z[e], e))[:top]
    e = np.exp(np.array([z[c] for c in chosen]) - z[chosen[0]])
    return chosen, e / e.sum()


def routed_ff(f, w, p, mlp):
    """Router logits W_r f + b; each token's `top` experts, weighted by the softmax over the chosen logits."""
    top = int(mlp["router"]["top"])
    z = mm(f, w[p + "router"]) + w[p + "router.b"]
    out = np.zeros_like(f)
    for t in range(f.shape[0]):
        chosen, weights = chosen_experts(z[t], top)
        for e, g in sorted(zip(chosen, weights)):
            out[t] += g * gated_unit(f[t:t + 1], w, f"{p}e{e}.", silu)[0]
    return out


# ----------------------------------------------------------------------------------------------- the model
MIXERS = {"attention": gated_attention, "retention": retention, "latent_attention": latent_attention}


def feed_forward(f, w, p, mlp):
    if mlp.get("kind", "dense") == "moe":
        return routed_ff(f, w, p, mlp)
    return gated_unit(f, w, p, gelu_tanh)


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence. `layers_out`: a list that receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = rms(w["embed"][np.asarray(tokens)], eps) * w["embed.norm"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer['weights_of'] if layer.get('weights_of') is not None else i}."
        x = x + MIXERS[layer["type"]](rms(x, eps) * w[p + "norm1"], w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            x = x + feed_forward(rms(x, eps) * w[p + "norm2"], w, p + "mlp.", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.copy())
    logits = mm(rms(x, eps) * w["final.norm"], w["head"])
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(logits / cap) if cap else logits
