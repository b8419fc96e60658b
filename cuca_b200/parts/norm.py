"""RMSNorm: h = x * rsqrt(mean(x^2) + eps) * w, the weight multiplies directly
(src/provider/local/model/cpu.rs:3651-3654; formula in model/gpu.rs:5883-5896)."""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, TensorNeed, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: width, eps, groups (default 1: the whole row; g: the row is cut into g equal consecutive parts and each
    is divided by its own root mean square before the weight multiplies the whole). tensors: weight [width]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.groups = int(spec.params.get("groups") or 1)
        if self.groups < 1 or self.width % self.groups:
            raise ValueError(f"rmsnorm: {self.groups} parts do not divide the width {self.width}")
        self.weight = self.gain = None

    def tensors(self):
        return {self.spec.tensors["weight"]: TensorNeed((self.width,), keep_fp32=True, init="ones")}

    def load(self, get):
        self.weight = get(self.spec.tensors["weight"])
        self.gain = self.weight  # what kernels that take "a gain" get: the vector

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, stream, rows=None):
        # this kernel adds the K slices a contraction left on the stream while it reads the stream
        x, pending = self.rt.stream(stream).take()
        n = x.shape[0] if rows is None else rows.shape[0]
        out = self.rt.empty(n, self.width)
        if pending is not None:
            ops.add_partials_rmsnorm(x, pending, self.weight, out, self.eps, rows, groups=self.groups)
        else:
            ops.rmsnorm(x, self.weight, out, self.eps, rows, groups=self.groups)
        return out


@register_norm("rmsnorm_scalar")
class ScalarRMSNorm(RMSNorm):
    """RMSNorm whose gain is one number for every coordinate: h = x * rsqrt(mean(x^2) + eps) * g.
    params: width, eps. tensors: weight [] (a single number). `gain` is that number as a 32-bit tensor of one
    element (kernels that take a gain take it with stride 0); `weight` is it spread over the width for the kernels
    that want a vector."""

    def tensors(self):
        return {self.spec.tensors["weight"]: TensorNeed((), keep_fp32=True, init="ones")}

    def load(self, get):
        self.gain = get(self.spec.tensors["weight"]).reshape(1).contiguous()
        self.weight = self.gain.expand(self.width).contiguous()

    def weight_bytes(self):
        return self.gain.element_size()


@register_norm("rmsnorm_streams")
class StreamsRMSNorm(RMSNorm):
    """RMSNorm of the sum of the stream's copies: h = n(sum_s X[:, s]) * w, for a stream `[rows, streams * width]`.
    params: width, eps, streams. tensors: weight [width]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.streams = int(spec.params["streams"])

    def forward(self, stream, rows=None):
        X = self.rt.stream(stream).data
        n = X.shape[0] if rows is None else rows.shape[0]
        out = self.rt.empty(n, self.width)
        ops.streams_read(X, None, self.weight, out, self.streams, self.eps, rows)
        return out
