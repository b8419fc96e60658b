"""Block arrangements. `pre_norm`: x += mixer(norm(x)); x += ffn(norm(x))
(src/provider/local/model/cpu.rs:2650-2704 with pre_norms on, post_norms off).
`sandwich_shift`: a norm before and after each sublayer, and the mixer reads its input mixed with the previous
token's: x += n1b(mixer(shift(n1(x)))); x += n2b(ffn(n2(x))).
`hyper_connections`: several copies of the stream; a sublayer reads a weighted sum of them and writes into all.
`parallel_residual`: one norm, both sublayers read its output: x += mixer(h) + ffn(h) with h = norm(x)."""
from __future__ import annotations

from ..kernels import ops
from ..runtime import ResidualStream
from .base import Block, CacheNeeds, StateNeeds, TensorNeed, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def forward(self, stream, step, cache) -> None:
        h = self.mixer_norm.forward(stream)
        self.mixer.forward(h, stream, step, cache)
        if self.feed_forward is not None:
            f = self.ffn_norm.forward(stream)
            self.feed_forward.forward(f, stream, step)


@register_block("parallel_residual")
class ParallelResidualBlock(Block):
    """x += mixer(h) + ffn(h) with the one h = norm(x): the layer's `mixer_norm` is its only norm (an `ffn_norm` is
    not used). Both sublayers add into the stream; neither reads it, so their order does not matter."""

    def forward(self, stream, step, cache) -> None:
        h = self.mixer_norm.forward(stream)
        self.mixer.forward(h, stream, step, cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(h, stream, step)


@register_block("sandwich_shift")
class SandwichShiftBlock(Block):
    """x += post1(mixer(shift(pre1(x)))); x += post2(ffn(pre2(x))), with shift(h)_t = h_t + (h_(t-1) - h_t) * mix
    (h_(-1) = 0) and every norm an RMSNorm. The pre-norms are the layer's `mixer_norm` / `ffn_norm` parts; the
    post-norms' gains and `mix` are this block's own tensors. The previous token's h is kept per request in the
    layer run's state `shift`, beside whatever the mixer keeps.

    params: width, eps, post_gain ("scalar": one number, "vector": [width]). tensors: mix [width],
    mixer_post, ffn_post (absent without a feed-forward).

    Three passes over the stream per layer: pre-norm with the shift; the mixer's post-norm added and the
    feed-forward's pre-norm of the new row; the feed-forward's post-norm added. A sublayer's output is gathered in a
    stream of its own (`ResidualStream.unwritten`), since it is normed before it is added."""

    def __init__(self, spec, runtime, mixer, feed_forward, mixer_norm, ffn_norm):
        super().__init__(spec, runtime, mixer, feed_forward, mixer_norm, ffn_norm)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.gain_shape = () if spec.params.get("post_gain", "scalar") == "scalar" else (self.width,)
        self.mix = self.post1 = self.post2 = None

    def tensors(self):
        t = self.spec.tensors
        out = {t["mix"]: TensorNeed((self.width,), keep_fp32=True),
               t["mixer_post"]: TensorNeed(self.gain_shape, keep_fp32=True, init="ones")}
        if self.feed_forward is not None:
            out[t["ffn_post"]] = TensorNeed(self.gain_shape, keep_fp32=True, init="ones")
        return out

    def load(self, get):
        t = self.spec.tensors
        self.mix = get(t["mix"])
        self.post1 = get(t["mixer_post"]).reshape(-1).contiguous()
        if self.feed_forward is not None:
            self.post2 = get(t["ffn_post"]).reshape(-1).contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.mix, self.post1, self.post2) if w is not None)

    def cache_needs(self):
        needs = self.mixer.cache_needs()
        state = needs.state if isinstance(needs.state, dict) else ({} if needs.state is None else {"mixer": needs.state})
        if "shift" in state:
            raise ValueError("the mixer names a state `shift`, which is this block's")
        return CacheNeeds(kv=needs.kv, state={"shift": StateNeeds((self.width,)), **state})

    def forward(self, stream, step, cache) -> None:
        rt = self.rt
        x = rt.stream(stream).data
        rows = x.shape[0]
        h = rt.empty(rows, self.width)
        ops.norm_shift(x, self.mixer_norm.gain, self.mixer_norm.eps, self.mix, cache.state["shift"], h, step)
        y = ResidualStream.unwritten(rt, rows, self.width)
        self.mixer.forward(h, y, step, cache)
        if self.feed_forward is None:
            ops.post_norm_add(x, y.data, self.post1, self.eps)
            return
        f = rt.empty(rows, self.width)
        ops.post_norm_add(x, y.data, self.post1, self.eps, gain2=self.ffn_norm.gain, out=f)
        y = ResidualStream.unwritten(rt, rows, self.width)
        self.feed_forward.forward(f, y, step)
        ops.post_norm_add(x, y.data, self.post2, self.eps)


@register_block("hyper_connections")
class HyperConnectionsBlock(Block):
    """The stream is `streams` copies X[0..s-1] side by side (`[rows, s * width]`). Sublayer c (1: mixer, 2:
    feed-forward) has a read vector r [s], a write vector o [s] and a matrix M [s, s] (rows: from, columns: to):
        y = sublayer(norm_c(sum_a r[a] X[a]));   X'[b] = sum_a M[a, b] X[a] + o[b] y   for every b, from the old copies.
    The norms are the layer's `mixer_norm` / `ffn_norm` parts (their weights are used by this block's kernels, which
    read the copies, norm and round in one pass). Three passes over the copies per layer: the mixer's read; the
    mixer's write with the feed-forward's read of the new copies; the feed-forward's write.

    params: width, streams, eps. tensors: read1, write1, mix1 and, with a feed-forward, read2, write2, mix2."""

    def __init__(self, spec, runtime, mixer, feed_forward, mixer_norm, ffn_norm):
        super().__init__(spec, runtime, mixer, feed_forward, mixer_norm, ffn_norm)
        self.width = int(spec.params["width"])
        self.streams = int(spec.params["streams"])
        self.eps = float(spec.params["eps"])
        if not 1 <= self.streams <= ops.STREAMS_MAX:
            raise ValueError(f"hyper-connections: {self.streams} copies of the stream are outside 1..{ops.STREAMS_MAX}")
        self.hc = {}

    def _subs(self):
        return ("1",) if self.feed_forward is None else ("1", "2")

    def tensors(self):
        t, s = self.spec.tensors, self.streams
        out = {}
        for c in self._subs():
            out[t["read" + c]] = TensorNeed((s,), keep_fp32=True)
            out[t["write" + c]] = TensorNeed((s,), keep_fp32=True)
            out[t["mix" + c]] = TensorNeed((s, s), keep_fp32=True)
        return out

    def load(self, get):
        t = self.spec.tensors
        for c in self._subs():
            self.hc[c] = tuple(get(t[k + c]) for k in ("read", "write", "mix"))

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for ws in self.hc.values() for w in ws)

    def forward(self, stream, step, cache) -> None:
        rt, S, E = self.rt, self.streams, self.width
        X = rt.stream(stream).data
        rows = X.shape[0]
        read1, write1, mix1 = self.hc["1"]
        h = rt.empty(rows, E)
        ops.streams_read(X, read1, self.mixer_norm.weight, h, S, self.mixer_norm.eps)
        y = ResidualStream.unwritten(rt, rows, E)
        self.mixer.forward(h, y, step, cache)
        if self.feed_forward is None:
            ops.streams_write(X, y.data, mix1, write1, S, self.eps)
            return
        read2, write2, mix2 = self.hc["2"]
        f = rt.empty(rows, E)
        ops.streams_write(X, y.data, mix1, write1, S, self.eps, read2=read2, weight2=self.ffn_norm.weight, out2=f)
        y = ResidualStream.unwritten(rt, rows, E)
        self.feed_forward.forward(f, y, step)
        ops.streams_write(X, y.data, mix2, write2, S, self.eps)
