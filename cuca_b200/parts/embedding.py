"""Token embedding and output head.

x[r] = E[token[r]] into the 32-bit stream (src/provider/local/model/cpu.rs:2193-2198);
logits = n W_head^T in 32-bit, W_head = lm_head or the embedding table when tied
(src/provider/local/model/cpu.rs:1614-1622,2586-2621).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, TensorNeed


class TokenEmbedding(Part):
    """params: vocab, width, scale (a factor on every embedding row, default 1), norm_eps (None: none; a number: the
    row is RMS-normed, e / sqrt(mean(e^2) + norm_eps) times the tensor `norm`, before it becomes the stream).
    tensors: weight [vocab, width], norm [width] (with norm_eps)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.scale = float(spec.params.get("scale", 1.0))
        eps = spec.params.get("norm_eps")
        self.norm_eps = float(eps) if eps is not None else None
        self.weight = self.norm_weight = None

    def tensors(self):
        out = {self.spec.tensors["weight"]: TensorNeed((self.vocab, self.width))}
        if self.norm_eps is not None:
            out[self.spec.tensors["norm"]] = TensorNeed((self.width,), keep_fp32=True, init="ones")
        return out

    def load(self, get):
        self.weight = get(self.spec.tensors["weight"])
        if self.norm_eps is not None:
            self.norm_weight = get(self.spec.tensors["norm"])

    def forward(self, tokens, out) -> None:
        if self.norm_eps is not None:
            ops.embed_norm(self.weight, tokens, out, self.norm_weight, self.norm_eps, self.rt.err, self.scale)
        else:
            ops.embed(self.weight, tokens, out, self.rt.err, self.scale)


class OutputHead(Part):
    """params: vocab, width, scale (a factor on the logits, default 1), softcap (None or 0: none; c > 0: the logits
    become c tanh(logits / c), after the scale). tensors: weight [vocab, width] (the embedding's name when tied)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.scale = float(spec.params.get("scale", 1.0))
        self.softcap = float(spec.params.get("softcap") or 0.0)
        if self.softcap < 0:
            raise ValueError(f"output head: a cap of {self.softcap} on the logits is not positive")
        self.weight = None

    def tensors(self):
        return {self.spec.tensors["weight"]: TensorNeed((self.vocab, self.width))}

    def load(self, get):
        self.weight = get(self.spec.tensors["weight"])

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, h) -> torch.Tensor:
        logits = self.rt.linear(h, self.weight, out_dtype=torch.float32)
        if self.scale != 1.0:
            ops.scale_(logits, self.scale)
        if self.softcap > 0:
            ops.softcap_(logits, self.softcap)
        return logits
