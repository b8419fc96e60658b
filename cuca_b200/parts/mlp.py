"""Dense SwiGLU feed-forward: y = down(silu(gate f) * (up f))
(src/provider/local/model/cpu.rs:3554-3565). gate and up are stacked into one
weight at load so one contraction with a SwiGLU epilogue yields the activation
(the reference accepts the stacked form too: model/cpu.rs:3131-3136)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, TensorNeed, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """params: width, inner. tensors: gate [inner, width], up [inner, width], down [width, inner]."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.inner = int(spec.params["inner"])
        self.w_gate_up = self.w_down = None

    def tensors(self):
        t = self.spec.tensors
        return {t["gate"]: TensorNeed((self.inner, self.width)), t["up"]: TensorNeed((self.inner, self.width)),
                t["down"]: TensorNeed((self.width, self.inner))}

    def load(self, get):
        t = self.spec.tensors
        self.w_gate_up = torch.cat([get(t["gate"]), get(t["up"])], dim=0).contiguous()
        self.w_down = get(t["down"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, h, stream, step) -> None:
        act = self.rt.linear(h, self.w_gate_up, epilogue=ops.EPI_SWIGLU)
        self.rt.stream(stream).add_linear(act, self.w_down)


@register_feed_forward("glu_capped")
class CappedGLU(FeedForward):
    """y = down(g sigmoid(alpha g) (u + 1)) with g = min(gate f, limit) and u = clamp(up f, -limit, limit).
    params: width, inner, limit, alpha (default 1.702). tensors: gate [inner, width], up [inner, width],
    down [width, inner]."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width, self.inner = int(spec.params["width"]), int(spec.params["inner"])
        self.limit, self.alpha = float(spec.params["limit"]), float(spec.params.get("alpha", 1.702))
        if not self.limit > 0:
            raise ValueError(f"capped feed-forward: the cap {self.limit} must be positive")
        self.w_gate_up = self.w_down = None

    def tensors(self):
        t = self.spec.tensors
        return {t["gate"]: TensorNeed((self.inner, self.width)), t["up"]: TensorNeed((self.inner, self.width)),
                t["down"]: TensorNeed((self.width, self.inner))}

    def load(self, get):
        t = self.spec.tensors
        self.w_gate_up = torch.cat([get(t["gate"]), get(t["up"])], dim=0).contiguous()
        self.w_down = get(t["down"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, h, stream, step) -> None:
        act = self.rt.empty(h.shape[0], self.inner)
        if h.dtype == torch.bfloat16 and ops.gemm_tc_supported(h, self.w_gate_up):
            # the unit is the contraction's epilogue, from the 32-bit sums (as SwiGLU is in the `swiglu` part)
            ops.gemm_tc_glu(h, self.w_gate_up, act, self.limit, self.alpha, self.rt.err)
        else:
            gu = self.rt.linear(h, self.w_gate_up)
            ops.glu_capped(gu, act, self.limit, self.alpha)
        self.rt.stream(stream).add_linear(act, self.w_down)


@register_feed_forward("glu")
class GatedUnit(FeedForward):
    """y = down(act(gate f) * (up f)) with act the silu or the tanh form of gelu,
    0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))). gate and up are stacked into one weight at load.
    params: width, inner, act ("silu" | "gelu_tanh"). tensors: gate [inner, width], up [inner, width],
    down [width, inner]."""

    graph_safe = True
    ACTS = {"silu": ops.GLU_SILU, "gelu_tanh": ops.GLU_GELU_TANH}

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width, self.inner = int(spec.params["width"]), int(spec.params["inner"])
        act = str(spec.params.get("act", "silu"))
        if act not in self.ACTS:
            raise ValueError(f"gated feed-forward: activation `{act}` is unknown; known: {', '.join(sorted(self.ACTS))}")
        self.act = self.ACTS[act]
        self.w_gate_up = self.w_down = None

    def tensors(self):
        t = self.spec.tensors
        return {t["gate"]: TensorNeed((self.inner, self.width)), t["up"]: TensorNeed((self.inner, self.width)),
                t["down"]: TensorNeed((self.width, self.inner))}

    def load(self, get):
        t = self.spec.tensors
        self.w_gate_up = torch.cat([get(t["gate"]), get(t["up"])], dim=0).contiguous()
        self.w_down = get(t["down"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, h, stream, step) -> None:
        if self.act == ops.GLU_SILU:  # the contraction's own epilogue
            act = self.rt.linear(h, self.w_gate_up, epilogue=ops.EPI_SWIGLU)
        elif h.dtype == torch.bfloat16 and ops.gemm_tc_supported(h, self.w_gate_up):
            # the unit is the contraction's epilogue, from the 32-bit sums (as SwiGLU is in the `swiglu` part)
            act = self.rt.empty(h.shape[0], self.inner)
            ops.gemm_tc_glu_act(h, self.w_gate_up, act, self.act, self.rt.err)
        else:
            gu = self.rt.linear(h, self.w_gate_up)
            act = self.rt.empty(h.shape[0], self.inner)
            ops.glu_act(gu, act, self.act)
        self.rt.stream(stream).add_linear(act, self.w_down)


@register_feed_forward("dense_act")
class DenseActivation(FeedForward):
    """y = down(act(up f + b_up)) + b_down with act the exact (erf) GELU or its tanh form.
    params: width, inner, act ("gelu" | "gelu_tanh"), bias (bool). tensors: up [inner, width], down [width, inner]
    and, with bias, up_bias [inner], down_bias [width]."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.inner = int(spec.params["inner"])
        self.act = str(spec.params.get("act", "gelu"))
        if self.act not in ("gelu", "gelu_tanh"):
            raise ValueError(f"dense feed-forward: activation `{self.act}` is unknown; known: gelu, gelu_tanh")
        self.bias = bool(spec.params.get("bias", True))
        self.w_up = self.w_down = self.b_up = self.b_down = None

    def tensors(self):
        t = self.spec.tensors
        out = {t["up"]: TensorNeed((self.inner, self.width)), t["down"]: TensorNeed((self.width, self.inner))}
        if self.bias:
            out[t["up_bias"]] = TensorNeed((self.inner,))
            out[t["down_bias"]] = TensorNeed((self.width,))
        return out

    def load(self, get):
        t = self.spec.tensors
        self.w_up, self.w_down = get(t["up"]), get(t["down"])
        if self.bias:
            self.b_up, self.b_down = get(t["up_bias"]), get(t["down_bias"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_up, self.w_down, self.b_up, self.b_down)
                   if w is not None)

    def forward(self, h, stream, step) -> None:
        a = self.rt.linear(h, self.w_up, bias=self.b_up)
        ops.gelu_(a, tanh_form=self.act == "gelu_tanh")
        self.rt.stream(stream).add_linear(a, self.w_down, bias=self.b_down)


@register_feed_forward("routed")
class RoutedExperts(FeedForward):
    """Every token goes to the `top` of `experts` small feed-forwards with the largest router logits z = W_r f
    (32-bit), with weights p = softmax of just those `top` logits: y = sum_e p_e down_e(act(up_e f)), act the
    square of relu. The experts' weights are stacked at load (`up` [experts * inner, width], `down` [width,
    experts * inner]). Many tokens: all experts' up-projections in one contraction, the activation weighted per
    expert (0 for the ones a token did not choose), one contraction over (expert, inner) down. Few tokens: only the
    chosen experts' rows are read, a warp per output. Both sum a token's experts in a fixed order.
    With act "swiglu" the experts are gated, down_e(silu(gate_e f) * (up_e f)): the gates and ups are stacked as
    `up` [2 experts * inner, width] (every expert's gate rows, then every expert's up rows). With `router_bias` the
    logits are z = W_r f + b.

    params: width, inner, experts, top, act ("relu2" | "swiglu"), router_bias (bool). tensors: router [experts, width],
    router_bias [experts], `up{e}` [inner, width] and `down{e}` [width, inner] for every expert e, and with "swiglu"
    `gate{e}` [inner, width]."""

    graph_safe = True
    SPARSE_MAX_TOKENS = 32  # up to this many tokens only the chosen experts are read

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width, self.inner = int(p["width"]), int(p["inner"])
        self.experts, self.top = int(p["experts"]), int(p["top"])
        act = str(p.get("act", "relu2"))
        if act not in ("relu2", "swiglu"):
            raise ValueError(f"routed feed-forward: activation `{act}` is unknown; known: relu2, swiglu")
        self.glu = act == "swiglu"
        self.router_bias = bool(p.get("router_bias", False))
        if not 1 <= self.top <= min(self.experts, ops.MOE_MAX_TOP) or self.experts > ops.MOE_MAX_EXPERTS:
            raise ValueError(f"routed feed-forward: {self.top} of {self.experts} experts is outside what the kernels "
                             f"take (experts <= {ops.MOE_MAX_EXPERTS}, chosen <= {ops.MOE_MAX_TOP})")
        self.w_router = self.b_router = self.w_up = self.w_down = None

    def tensors(self):
        t = self.spec.tensors
        out = {t["router"]: TensorNeed((self.experts, self.width))}
        if self.router_bias:
            out[t["router_bias"]] = TensorNeed((self.experts,))
        for e in range(self.experts):
            if self.glu:
                out[t[f"gate{e}"]] = TensorNeed((self.inner, self.width))
            out[t[f"up{e}"]] = TensorNeed((self.inner, self.width))
            out[t[f"down{e}"]] = TensorNeed((self.width, self.inner))
        return out

    def load(self, get):
        t = self.spec.tensors
        self.w_router = get(t["router"])
        if self.router_bias:
            self.b_router = get(t["router_bias"])
        gates = [get(t[f"gate{e}"]) for e in range(self.experts)] if self.glu else []
        self.w_up = torch.cat(gates + [get(t[f"up{e}"]) for e in range(self.experts)], dim=0).contiguous()
        self.w_down = torch.cat([get(t[f"down{e}"]) for e in range(self.experts)], dim=1).contiguous()

    def weight_bytes(self):
        """What a step of several tokens reads at most: the router and every expert once."""
        return sum(w.numel() * w.element_size() for w in (self.w_router, self.b_router, self.w_up, self.w_down)
                   if w is not None)

    def forward(self, h, stream, step) -> None:
        rt, T = self.rt, h.shape[0]
        logits = rt.linear(h, self.w_router, bias=self.b_router, out_dtype=torch.float32)
        idx = torch.empty(T, self.top, dtype=torch.int32, device=rt.device)
        wts = torch.empty(T, self.top, dtype=torch.float32, device=rt.device)
        if T <= self.SPARSE_MAX_TOKENS:
            ops.moe_route(logits, self.top, idx, wts)
            a = rt.empty(T * self.top, self.inner)
            y, fresh = rt.stream(stream).claim()
            ops.moe_sparse(h, self.w_up, self.w_down, idx, wts, a, y, fresh, self.top, self.experts, self.inner,
                           glu=self.glu)
            return
        spread = torch.empty(T, self.experts, dtype=torch.float32, device=rt.device)
        ops.moe_route(logits, self.top, idx, wts, spread)
        u = rt.linear(h, self.w_up)
        if self.glu:
            a = rt.empty(T, self.experts * self.inner)
            ops.moe_glu_dense(u, spread, a, self.experts * self.inner, self.inner)
        else:
            a = torch.empty_like(u)
            ops.moe_act_dense(u, spread, a, self.experts, self.inner)
        rt.stream(stream).add_linear(a, self.w_down)


@register_feed_forward("routed_scored")
class ScoredExperts(FeedForward):
    """Routed experts whose scores are a softmax over ALL router outputs, z = W_r f in 32-bit. The `top` outputs with
    the largest score + correction (a stored vector; only the choice sees it) are chosen, and a chosen one's weight is
    its score over the sum of the chosen scores (+ 1e-20). The first `experts` outputs are gated feed-forwards,
    down_e(silu(gate_e f) * (up_e f)); the last `identity` outputs are experts that return their input f. With
    `shared` > 0 one more gated feed-forward of that inner size runs for every token and is added.

    The experts' weights are stacked at load: `w_gu` [2 C, width] holds every expert's gate rows, the shared expert's
    behind them, then the up rows in the same order (C = experts * inner + shared); `w_down` [width, C]. Many tokens:
    one contraction gives all gates and ups, the activation is weighted per expert (0 for the ones a token did not
    choose, 1 for the shared one), one contraction over C goes down. Few tokens: only the chosen experts' rows are read,
    a warp per output, and the shared expert runs as a dense gated unit. Both sum a token's experts in a fixed order.

    params: width, inner, experts, identity, top, shared (0: none), correction (bool). tensors: router
    [experts + identity, width], correction [experts + identity], `gate{e}`, `up{e}` [inner, width], `down{e}`
    [width, inner] per expert e, and shared_gate, shared_up [shared, width], shared_down [width, shared]."""

    graph_safe = True
    SPARSE_MAX_TOKENS = 32  # up to this many tokens only the chosen experts are read

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width, self.inner = int(p["width"]), int(p["inner"])
        self.experts, self.identity, self.top = int(p["experts"]), int(p.get("identity") or 0), int(p["top"])
        self.shared = int(p.get("shared") or 0)
        self.corrected = bool(p.get("correction", True))
        self.outputs = self.experts + self.identity
        if (not 1 <= self.top <= min(self.outputs, ops.MOE_MAX_TOP) or self.outputs > ops.MOE_MAX_EXPERTS
                or self.experts < 0 or self.identity < 0):
            raise ValueError(f"routed feed-forward: {self.top} of {self.experts} + {self.identity} experts is outside "
                             f"what the kernels take (experts <= {ops.MOE_MAX_EXPERTS}, chosen <= {ops.MOE_MAX_TOP})")
        self.w_router = self.correction = self.w_gu = self.w_down = self.w_shared_gu = self.w_shared_down = None

    def tensors(self):
        t = self.spec.tensors
        out = {t["router"]: TensorNeed((self.outputs, self.width))}
        if self.corrected:
            out[t["correction"]] = TensorNeed((self.outputs,), keep_fp32=True)
        for e in range(self.experts):
            out[t[f"gate{e}"]] = TensorNeed((self.inner, self.width))
            out[t[f"up{e}"]] = TensorNeed((self.inner, self.width))
            out[t[f"down{e}"]] = TensorNeed((self.width, self.inner))
        if self.shared:
            out[t["shared_gate"]] = TensorNeed((self.shared, self.width))
            out[t["shared_up"]] = TensorNeed((self.shared, self.width))
            out[t["shared_down"]] = TensorNeed((self.width, self.shared))
        return out

    def load(self, get):
        t = self.spec.tensors
        self.w_router = get(t["router"])
        self.correction = get(t["correction"]) if self.corrected else None
        gates = [get(t[f"gate{e}"]) for e in range(self.experts)]
        ups = [get(t[f"up{e}"]) for e in range(self.experts)]
        downs = [get(t[f"down{e}"]) for e in range(self.experts)]
        if self.shared:
            gates.append(get(t["shared_gate"]))
            ups.append(get(t["shared_up"]))
            downs.append(get(t["shared_down"]))
        if gates:
            self.w_gu = torch.cat(gates + ups, dim=0).contiguous()
            self.w_down = torch.cat(downs, dim=1).contiguous()
        if self.shared:  # the shared expert alone, for steps of few tokens (views of the stacked weights will not do:
            # the dense gated unit wants [gate; up] in one piece)
            self.w_shared_gu = torch.cat([gates[-1], ups[-1]], dim=0).contiguous()
            self.w_shared_down = downs[-1].contiguous()

    def weight_bytes(self):
        """What a step of several tokens reads at most: the router and every expert once."""
        return sum(w.numel() * w.element_size() for w in (self.w_router, self.correction, self.w_gu, self.w_down)
                   if w is not None)

    def forward(self, h, stream, step) -> None:
        rt, T = self.rt, h.shape[0]
        stream = rt.stream(stream)
        logits = rt.linear(h, self.w_router, out_dtype=torch.float32)
        idx = torch.empty(T, self.top, dtype=torch.int32, device=rt.device)
        wts = torch.empty(T, self.top, dtype=torch.float32, device=rt.device)
        ident = torch.empty(T, dtype=torch.float32, device=rt.device) if self.identity else None
        sparse = T <= self.SPARSE_MAX_TOKENS or self.w_gu is None
        spread = None if sparse else torch.empty(T, self.outputs, dtype=torch.float32, device=rt.device)
        ops.moe_route_scored(logits, self.correction, self.experts, self.top, idx, wts, spread, ident)
        if ident is not None:
            y, fresh = stream.claim()
            ops.moe_identity_add(y, h, ident, fresh)
        if self.w_gu is None:
            return
        if sparse:
            if self.experts:
                a = rt.empty(T * self.top, self.inner)
                y, fresh = stream.claim()
                ops.moe_sparse(h, self.w_gu, self.w_down, idx, wts, a, y, fresh, self.top, self.experts, self.inner,
                               glu=True)
            if self.shared:
                act = rt.linear(h, self.w_shared_gu, epilogue=ops.EPI_SWIGLU)
                stream.add_linear(act, self.w_shared_down)
            return
        gu = rt.linear(h, self.w_gu)
        a = rt.empty(T, self.w_down.shape[1])
        ops.moe_glu_dense(gu, spread, a, self.experts * self.inner, self.inner)
        stream.add_linear(a, self.w_down)
