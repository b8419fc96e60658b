"""Recurrent mixers: a state of fixed size per request, carried from token to token in 32-bit.

Each mixer declares its state (`StateNeeds`, by name) and gets it per slot in the cache view; a step's kernels walk
every request's rows in order from that state and leave the new one behind, so a request may be cut into steps
anywhere. Projections run in the compute dtype with 32-bit results; whatever enters a recurrence (gates, decays,
step sizes) is computed in 32-bit from them.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from . import rope  # noqa: F401  (registers the rotary tables the retention mixer asks for)
from .base import POSITIONS, CacheNeeds, Mixer, PartSpec, StateNeeds, TensorNeed, register_mixer


@register_mixer("mingru")
class MinGRU(Mixer):
    """A gated recurrence whose gates read only the current token:
        z = sigmoid(W_z h + b_z), u = W_x h + b_x, c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0),
        S_t = (1 - z) S_(t-1) + z c (element by element), out = W_o (S_t * silu(W_g h)).
    params: width (the model's), inner (the recurrence's). tensors: z, z_bias, x, x_bias, g, o."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.inner = int(spec.params["inner"])
        self.w_zxg = self.b_zxg = self.w_o = None

    def cache_needs(self):
        return CacheNeeds(state={"mingru": StateNeeds((self.inner,))})

    def tensors(self):
        t, W, E = self.spec.tensors, self.inner, self.width
        return {t["z"]: TensorNeed((W, E)), t["z_bias"]: TensorNeed((W,)), t["x"]: TensorNeed((W, E)),
                t["x_bias"]: TensorNeed((W,)), t["g"]: TensorNeed((W, E)), t["o"]: TensorNeed((E, W))}

    def load(self, get):
        t = self.spec.tensors
        self.w_zxg = torch.cat([get(t["z"]), get(t["x"]), get(t["g"])], dim=0).contiguous()
        bz, bx = get(t["z_bias"]), get(t["x_bias"])
        self.b_zxg = torch.cat([bz, bx, torch.zeros_like(bz)]).contiguous()
        self.w_o = get(t["o"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_zxg, self.b_zxg, self.w_o))

    def forward(self, h, stream, step, cache) -> None:
        zxg = self.rt.linear(h, self.w_zxg, bias=self.b_zxg, out_dtype=torch.float32)
        out = self.rt.empty(h.shape[0], self.inner)
        ops.mingru_scan(zxg, cache.state["mingru"], out, step)
        self.rt.stream(stream).add_linear(out, self.w_o)


@register_mixer("mamba2")
class Mamba2(Mixer):
    """A selective state space with one scalar decay per head. W_in h = [z | x | B | C | dt] (inner, inner, G N,
    G N, heads; inner = heads * vdim); x, B, C pass a causal convolution per channel (bias, silu);
    dt = softplus(dt + dt_bias); per head (group = head // (heads / G)), with S of N x vdim,
        S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T,   y_t = S_t^T C_t + D x_t;
    y * silu(z) is RMS-normed in `norm_groups` equal parts, times `norm`, then W_o.
    The state is S and the convolution's last taps - 1 inputs.
    params: width, heads, vdim, state, groups, conv (taps), norm_groups, eps.
    tensors: in, conv, conv_bias, dt_bias, A_log, D, norm, o."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width = int(p["width"])
        self.heads, self.vdim, self.n_state = int(p["heads"]), int(p["vdim"]), int(p["state"])
        self.groups, self.taps, self.norm_groups = int(p["groups"]), int(p["conv"]), int(p["norm_groups"])
        self.eps = float(p["eps"])
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n_state
        if self.heads % self.groups:
            raise ValueError(f"mamba2: {self.groups} groups must divide {self.heads} heads")
        if self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.norm_groups} norm groups must divide the inner size {self.inner}")
        if self.taps < 1:
            raise ValueError("mamba2: the convolution needs at least one tap")
        self.w_in = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d = self.norm_w = self.w_o = None

    def cache_needs(self):
        return CacheNeeds(state={"conv": StateNeeds((self.taps - 1, self.channels)),
                                 "ssm": StateNeeds((self.heads, self.vdim, self.n_state))})

    def tensors(self):
        t = self.spec.tensors
        H = self.heads
        return {t["in"]: TensorNeed((self.inner + self.channels + H, self.width)),
                t["conv"]: TensorNeed((self.channels, self.taps)), t["conv_bias"]: TensorNeed((self.channels,)),
                t["dt_bias"]: TensorNeed((H,), keep_fp32=True), t["A_log"]: TensorNeed((H,), keep_fp32=True),
                t["D"]: TensorNeed((H,), keep_fp32=True),
                t["norm"]: TensorNeed((self.inner,), keep_fp32=True, init="ones"),
                t["o"]: TensorNeed((self.width, self.inner))}

    def load(self, get):
        t = self.spec.tensors
        self.w_in, self.conv_w, self.conv_b = get(t["in"]), get(t["conv"]), get(t["conv_bias"])
        self.dt_bias, self.a_log, self.d = get(t["dt_bias"]), get(t["A_log"]), get(t["D"])
        self.norm_w, self.w_o = get(t["norm"]), get(t["o"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.conv_w, self.conv_b, self.dt_bias,
                                                          self.a_log, self.d, self.norm_w, self.w_o))

    def forward(self, h, stream, step, cache) -> None:
        rt, rows = self.rt, h.shape[0]
        proj = rt.linear(h, self.w_in, out_dtype=torch.float32)  # [z | x B C | dt]
        xbc = rt.empty(rows, self.channels, dtype=torch.float32)
        ops.causal_conv(proj, self.inner, self.conv_w, self.conv_b, cache.state["conv"], xbc, step)
        y = rt.empty(rows, self.inner, dtype=torch.float32)
        ops.ssm_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.d, cache.state["ssm"], y,
                     step, self.heads, self.vdim, self.n_state, self.groups)
        out = rt.empty(rows, self.inner)
        ops.gated_group_norm(y, proj, self.norm_w, out, self.norm_groups, self.eps)
        rt.stream(stream).add_linear(out, self.w_o)


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    """The delta rule with a gate on the write and a decay per head and key channel. q, k (`kv_heads` heads of
    `dim`) and v (`heads` heads of `vdim`) pass a short causal convolution per channel (no bias) and silu; q and k
    become unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q times dim^(-1/2); head a reads q/k head
    a // (heads / kv_heads). beta = sigmoid(W_b h) per head;
    g = exp(-exp(A_log[a]) * softplus(W_a2 (W_a1 h) + dt_bias)) per head and key channel. Per head, S of dim x vdim:
        S <- g[:, None] * S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   (q reads S after the token's own update).
    o / rms(o) per head, times `norm` [vdim], times sigmoid(W_g2 (W_g1 h)), then W_o. The ranks of the two low-rank
    pairs are the stored tensors' (`decay_rank`, `gate_rank` only size random weights).
    The state is S (32-bit) and the convolution's last taps - 1 inputs.
    params: width, heads, kv_heads, dim, vdim, conv (taps), eps, decay_rank, gate_rank.
    tensors: q, k, v, q_conv, k_conv, v_conv, b, A_log, dt_bias, a1, a2, g1, g2, norm, o."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width = int(p["width"])
        self.heads, self.kv_heads = int(p["heads"]), int(p.get("kv_heads") or p["heads"])
        self.dim, self.vdim, self.taps = int(p["dim"]), int(p["vdim"]), int(p["conv"])
        self.eps = float(p["eps"])
        self.decay_rank = int(p.get("decay_rank") or max(8, self.dim // 4))
        self.gate_rank = int(p.get("gate_rank") or max(8, self.vdim // 4))
        if self.heads % self.kv_heads:
            raise ValueError(f"gated_delta: {self.kv_heads} key heads must divide {self.heads} heads")
        if self.taps < 1:
            raise ValueError("gated_delta: the convolution needs at least one tap")
        if self.dim > ops.MATRIX_STATE_MAX_DIM:
            raise ValueError(f"gated_delta: {self.dim} key channels exceed {ops.MATRIX_STATE_MAX_DIM}")
        self.qk = self.kv_heads * self.dim
        self.channels = 2 * self.qk + self.heads * self.vdim
        self.w_in = self.w_low = self.w_2 = self.w_a2 = self.w_g2 = self.conv_w = self.dt_bias = self.a_log = None
        self.norm_w = self.w_o = None

    def cache_needs(self):
        return CacheNeeds(state={"conv": StateNeeds((self.taps - 1, self.channels)),
                                 "delta": StateNeeds((self.heads, self.vdim, self.dim))})

    def tensors(self):
        t, E, H = self.spec.tensors, self.width, self.heads
        inner = H * self.vdim
        return {t["q"]: TensorNeed((self.qk, E)), t["k"]: TensorNeed((self.qk, E)), t["v"]: TensorNeed((inner, E)),
                t["q_conv"]: TensorNeed((self.qk, self.taps)), t["k_conv"]: TensorNeed((self.qk, self.taps)),
                t["v_conv"]: TensorNeed((inner, self.taps)), t["b"]: TensorNeed((H, E)),
                t["A_log"]: TensorNeed((H,), keep_fp32=True), t["dt_bias"]: TensorNeed((H * self.dim,), keep_fp32=True),
                t["a1"]: TensorNeed((self.decay_rank, E), free=(0,)),
                t["a2"]: TensorNeed((H * self.dim, self.decay_rank), free=(1,)),
                t["g1"]: TensorNeed((self.gate_rank, E), free=(0,)),
                t["g2"]: TensorNeed((inner, self.gate_rank), free=(1,)),
                t["norm"]: TensorNeed((self.vdim,), keep_fp32=True, init="ones"), t["o"]: TensorNeed((E, inner))}

    def load(self, get):
        t = self.spec.tensors
        self.w_in = torch.cat([get(t["q"]), get(t["k"]), get(t["v"]), get(t["b"])], dim=0).contiguous()
        a1, g1 = get(t["a1"]), get(t["g1"])
        self.w_a2, self.w_g2 = get(t["a2"]), get(t["g2"])
        self.decay_rank, self.gate_rank = a1.shape[0], g1.shape[0]
        if self.w_a2.shape[1] != self.decay_rank or self.w_g2.shape[1] != self.gate_rank:
            raise ValueError(f"gated_delta: `{t['a2']}` / `{t['g2']}` do not continue `{t['a1']}` / `{t['g1']}`: ranks "
                             f"{self.w_a2.shape[1]}, {self.w_g2.shape[1]} against {self.decay_rank}, {self.gate_rank}")
        self.w_low = torch.cat([a1, g1], dim=0).contiguous()
        # the two second factors as one block-diagonal matrix: [a | gate] = [a1 h | g1 h] W2^T in one contraction
        w2 = torch.zeros(self.w_a2.shape[0] + self.w_g2.shape[0], self.decay_rank + self.gate_rank,
                         dtype=self.w_a2.dtype, device=self.w_a2.device)
        w2[:self.w_a2.shape[0], :self.decay_rank] = self.w_a2
        w2[self.w_a2.shape[0]:, self.decay_rank:] = self.w_g2
        self.w_2 = w2
        self.conv_w = torch.cat([get(t["q_conv"]), get(t["k_conv"]), get(t["v_conv"])], dim=0).contiguous()
        self.dt_bias, self.a_log, self.norm_w, self.w_o = get(t["dt_bias"]), get(t["A_log"]), get(t["norm"]), get(t["o"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_low, self.w_2, self.conv_w,
                                                          self.dt_bias, self.a_log, self.norm_w, self.w_o))

    def forward(self, h, stream, step, cache) -> None:
        rt, rows = self.rt, h.shape[0]
        H, G, d, dv, C = self.heads, self.kv_heads, self.dim, self.vdim, self.channels
        proj = rt.linear(h, self.w_in, out_dtype=torch.float32)  # [q | k | v | b]
        low = rt.linear(h, self.w_low)  # [a1 h | g1 h], rounded as everything is that enters a contraction
        second = rt.linear(low, self.w_2, out_dtype=torch.float32)  # [decay pre-activations | gate pre-activations]
        a_raw, gate = second[:, :H * d], second[:, H * d:]
        qkv = rt.empty(rows, C, dtype=torch.float32)
        ops.causal_conv(proj, 0, self.conv_w, None, cache.state["conv"], qkv, step)
        o = rt.empty(rows, H * dv, dtype=torch.float32)
        ops.delta_scan(qkv, a_raw, self.dt_bias, self.a_log, proj, C, cache.state["delta"], o, step, H, G, d, dv)
        out = rt.empty(rows, H * dv)
        ops.head_norm_gate(o, self.norm_w, False, gate, out, H, dv, self.eps)
        rt.stream(stream).add_linear(out, self.w_o)


@register_mixer("mlstm")
class MatrixLSTM(Mixer):
    """A matrix memory with exponential gates. q = W_q h * dim^(-1/2), k = W_k h (heads x dim), v = W_v h (heads x
    vdim); per head i = cap tanh((W_i h + b_i) / cap), f = logsigmoid(cap tanh((W_f h + b_f) / cap)); with a running
    maximum m (0 at the start, like S and n):
        m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n <- e^(f + m - m') n + e^(i - m') k;
        o = S^T q / (max(|n . q|, e^(-m')) + 1e-6).
    o / rms(o) per head, times `norm` [heads * vdim], times sigmoid(W_g h), then W_o. State: S, n, m in 32-bit.
    params: width, heads, dim, vdim, gate_cap, eps. tensors: q, k, v, g, i, i_bias, f, f_bias, norm, o."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width, self.heads = int(p["width"]), int(p["heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.cap, self.eps = float(p["gate_cap"]), float(p["eps"])
        if self.cap <= 0:
            raise ValueError("mlstm: gate_cap must be positive")
        if self.dim > ops.MATRIX_STATE_MAX_DIM:
            raise ValueError(f"mlstm: {self.dim} key channels exceed {ops.MATRIX_STATE_MAX_DIM}")
        self.w_in = self.i_bias = self.f_bias = self.norm_w = self.w_o = None

    def cache_needs(self):
        H = self.heads
        return CacheNeeds(state={"mem": StateNeeds((H, self.vdim, self.dim)), "norm": StateNeeds((H, self.dim)),
                                 "max": StateNeeds((H,))})

    def tensors(self):
        t, E, H = self.spec.tensors, self.width, self.heads
        inner = H * self.vdim
        return {t["q"]: TensorNeed((H * self.dim, E)), t["k"]: TensorNeed((H * self.dim, E)),
                t["v"]: TensorNeed((inner, E)), t["g"]: TensorNeed((inner, E)), t["i"]: TensorNeed((H, E)),
                t["i_bias"]: TensorNeed((H,), keep_fp32=True), t["f"]: TensorNeed((H, E)),
                t["f_bias"]: TensorNeed((H,), keep_fp32=True),
                t["norm"]: TensorNeed((inner,), keep_fp32=True, init="ones"), t["o"]: TensorNeed((E, inner))}

    def load(self, get):
        t = self.spec.tensors
        self.w_in = torch.cat([get(t[r]) for r in ("q", "k", "v", "g", "i", "f")], dim=0).contiguous()
        self.i_bias, self.f_bias = get(t["i_bias"]), get(t["f_bias"])
        self.norm_w, self.w_o = get(t["norm"]), get(t["o"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.i_bias, self.f_bias, self.norm_w, self.w_o))

    def forward(self, h, stream, step, cache) -> None:
        rt, rows = self.rt, h.shape[0]
        H, d, dv = self.heads, self.dim, self.vdim
        proj = rt.linear(h, self.w_in, out_dtype=torch.float32)  # [q | k | v | g | i | f]
        k_col, v_col, g_col = H * d, 2 * H * d, 2 * H * d + H * dv
        i_col = g_col + H * dv
        o = rt.empty(rows, H * dv, dtype=torch.float32)
        st = cache.state
        ops.mlstm_scan(proj, 0, k_col, v_col, i_col, i_col + H, self.i_bias, self.f_bias, self.cap, st["mem"],
                       st["norm"], st["max"], o, step, H, d, dv)
        out = rt.empty(rows, H * dv)
        ops.head_norm_gate(o, self.norm_w, True, proj[:, g_col:i_col], out, H, dv, self.eps)
        rt.stream(stream).add_linear(out, self.w_o)


@register_mixer("hgrn2")
class ForgetGateAttention(Mixer):
    """HGRN2: linear attention whose forget gate also decides what is written. q = silu(W_q h) (heads x dim),
    v = W_v h (heads x vdim), f = l + (1 - l) sigmoid(W_f h + b_f) per head and key channel with a lower bound l in
    [0, 1] per channel (a stored vector); per head, S of dim x vdim (zero at the start):
        S <- f[:, None] * S + (1 - f)[:, None] * v[None, :];   o = S^T q     (there is no key and no scale);
    o / rms(o) per head, times `norm` [vdim] (shared by the heads), then W_o. State: S in 32-bit.
    params: width, heads, dim, vdim, eps. tensors: q, f, f_bias, lower, v, norm, o."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width, self.heads = int(p["width"]), int(p["heads"])
        self.dim, self.vdim, self.eps = int(p["dim"]), int(p["vdim"]), float(p["eps"])
        if self.dim > ops.MATRIX_STATE_MAX_DIM:
            raise ValueError(f"hgrn2: {self.dim} key channels exceed {ops.MATRIX_STATE_MAX_DIM}")
        self.w_in = self.f_bias = self.lower = self.norm_w = self.w_o = None

    def cache_needs(self):
        return CacheNeeds(state={"memory": StateNeeds((self.heads, self.vdim, self.dim))})

    def tensors(self):
        t, E, H = self.spec.tensors, self.width, self.heads
        return {t["q"]: TensorNeed((H * self.dim, E)), t["f"]: TensorNeed((H * self.dim, E)),
                t["f_bias"]: TensorNeed((H * self.dim,), keep_fp32=True),
                t["lower"]: TensorNeed((H * self.dim,), keep_fp32=True),
                t["v"]: TensorNeed((H * self.vdim, E)),
                t["norm"]: TensorNeed((self.vdim,), keep_fp32=True, init="ones"), t["o"]: TensorNeed((E, H * self.vdim))}

    def load(self, get):
        t = self.spec.tensors
        self.w_in = torch.cat([get(t[r]) for r in ("q", "f", "v")], dim=0).contiguous()
        self.f_bias, self.lower = get(t["f_bias"]), get(t["lower"])
        self.norm_w, self.w_o = get(t["norm"]), get(t["o"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.f_bias, self.lower, self.norm_w, self.w_o))

    def forward(self, h, stream, step, cache) -> None:
        rt, rows = self.rt, h.shape[0]
        H, d, dv = self.heads, self.dim, self.vdim
        proj = rt.linear(h, self.w_in, out_dtype=torch.float32)  # [q | f | v]
        o = rt.empty(rows, H * dv, dtype=torch.float32)
        ops.forget_scan(proj, 0, H * d, 2 * H * d, self.f_bias, self.lower, cache.state["memory"], o, step, H, d, dv)
        out = rt.empty(rows, H * dv)
        ops.head_norm_gate(o, self.norm_w, False, None, out, H, dv, self.eps)
        rt.stream(stream).add_linear(out, self.w_o)


@register_mixer("retention")
class Retention(Mixer):
    """Retention: linear attention with one fixed decay per head, no softmax and no denominator. q = W_q h, k = W_k h
    (heads x dim), v = W_v h (heads x vdim); the first rotated dimensions of every q and k head turn by the position
    (the position part's tables, pairs (i, i + n/2)), then k is multiplied by dim^(-1/2); per head, S of dim x vdim
    (zero at the start):
        S <- decay_a S + k v^T;   o = S^T q;
    o / rms(o) per head (no weight), the concatenated heads times silu(W_g h), then W_o. State: S in 32-bit.
    params: width, heads, dim, vdim, decay (one number per head), eps, position (a rotary PartSpec or None).
    tensors: q, k, v, g, o."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width, self.heads = int(p["width"]), int(p["heads"])
        self.dim, self.vdim, self.eps = int(p["dim"]), int(p["vdim"]), float(p["eps"])
        self.decay_values = [float(v) for v in p["decay"]]
        if len(self.decay_values) != self.heads:
            raise ValueError(f"retention: {len(self.decay_values)} decays for {self.heads} heads")
        if self.dim > ops.MATRIX_STATE_MAX_DIM:
            raise ValueError(f"retention: {self.dim} key channels exceed {ops.MATRIX_STATE_MAX_DIM}")
        pos = p.get("position")
        self.position = POSITIONS.get(pos.kind)(pos, runtime) if isinstance(pos, PartSpec) else None
        if self.position is not None and self.position.pairs != "half":
            raise ValueError("retention: rotated dimensions pair as (i, i + n/2)")
        self.w_in = self.w_o = self.decay = None

    def cache_needs(self):
        return CacheNeeds(state={"memory": StateNeeds((self.heads, self.vdim, self.dim))})

    def tensors(self):
        t, E, H = self.spec.tensors, self.width, self.heads
        return {t["q"]: TensorNeed((H * self.dim, E)), t["k"]: TensorNeed((H * self.dim, E)),
                t["v"]: TensorNeed((H * self.vdim, E)), t["g"]: TensorNeed((H * self.vdim, E)),
                t["o"]: TensorNeed((E, H * self.vdim))}

    def load(self, get):
        t = self.spec.tensors
        self.w_in = torch.cat([get(t[r]) for r in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_o = get(t["o"])
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.rt.device)

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def prepare(self, context_length: int) -> None:
        if self.position is not None:
            self.position.prepare(context_length)

    def forward(self, h, stream, step, cache) -> None:
        rt, rows = self.rt, h.shape[0]
        H, d, dv = self.heads, self.dim, self.vdim
        proj = rt.linear(h, self.w_in, out_dtype=torch.float32)  # [q | k | v | g]
        cos, sin, rot = (self.position.cos, self.position.sin, self.position.rotary_dim) \
            if self.position is not None else (None, None, 0)
        o = rt.empty(rows, H * dv, dtype=torch.float32)
        ops.retention_scan(proj, 0, H * d, 2 * H * d, self.decay, cos, sin, rot, d ** -0.5, cache.state["memory"], o,
                           step, H, d, dv, rt.err)
        out = rt.empty(rows, H * dv)
        ops.head_norm_gate(o, None, False, proj[:, 2 * H * d + H * dv:], out, H, dv, self.eps, gate_act="silu")
        rt.stream(stream).add_linear(out, self.w_o)
