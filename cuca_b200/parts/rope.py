"""Rotary position encoding: tables of cos/sin per position and pair.

theta(pos, i) = pos * base^(-2i/n) / factor_i * freq_scale, computed in 64-bit
and stored as 32-bit tables [positions, n/2] (src/provider/local/model/rope.rs:
118-152). `llama3` scaling gives per-pair divisors computed as the reference's
converter does, with the frequency in 32-bit
(src/provider/local/convert/config.rs:525-565); `linear` scales every frequency
by 1/factor (src/provider/local/model/params.rs:535-572). Pairs are (i, i + n/2)
in Hugging Face row order, which equals the reference's adjacent pairs on its
permuted rows (src/provider/local/model/cpu.rs:4247-4275).
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding, register_position


def llama3_factors(n_dims: int, base: float, factor: float, low: float, high: float, original: int) -> np.ndarray:
    out = np.empty(n_dims // 2, dtype=np.float32)
    low_wavelen, high_wavelen = original / low, original / high
    for i in range(n_dims // 2):
        freq = np.float32(1.0) / np.power(np.float32(base), np.float32(2 * i) / np.float32(n_dims), dtype=np.float32)
        wavelen = 2.0 * math.pi / float(freq)
        if wavelen < high_wavelen:
            r = 1.0
        elif wavelen > low_wavelen:
            r = factor
        else:
            smooth = (original / wavelen - low) / (high - low)
            r = 1.0 / ((1.0 - smooth) / factor + smooth)
        out[i] = np.float32(r)
    return out


def yarn_factors(n_dims: int, base: float, factor: float, original: float, fast: float, slow: float) -> np.ndarray:
    """Per-pair divisors of the frequencies for YaRN scaling. pair(t) = n ln(original / (2 pi t)) / (2 ln base) is the
    pair number whose wave makes t turns over `original` positions; from lo = max(floor(pair(fast)), 0) to
    hi = min(ceil(pair(slow)), n - 1) a ramp r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) goes from 0 to 1, and
    pair i turns at f_i (r_i / factor + 1 - r_i): fast pairs as they are, slow pairs `factor` times slower."""
    def pair(turns):
        return n_dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair(fast)), 0)
    hi = min(math.ceil(pair(slow)), n_dims - 1)
    ramp = np.clip((np.arange(n_dims // 2, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return 1.0 / (ramp / factor + (1.0 - ramp))


def rope_tables(positions: int, n_dims: int, base: float, factors=None, freq_scale: float = 1.0, magnitude: float = 1.0):
    """cos, sin (times `magnitude`) as float32 CPU tensors [positions, n_dims // 2], angles in float64."""
    i = np.arange(n_dims // 2, dtype=np.float64)
    inv = np.power(np.float64(base), -(2.0 * i) / n_dims)
    if factors is not None:
        inv = inv / np.asarray(factors, dtype=np.float64)
    inv = inv * freq_scale
    theta = np.arange(positions, dtype=np.float64)[:, None] * inv[None, :]
    return (torch.from_numpy((np.cos(theta) * magnitude).astype(np.float32)),
            torch.from_numpy((np.sin(theta) * magnitude).astype(np.float32)))


@register_position("rope")
class RotaryEncoding(PositionEncoding):
    """params: head_dim, rotary_dim, theta, pairs ("half" | "adjacent"), scaling {kind, factor, low_freq_factor, high_freq_factor,
    original_max_position_embeddings}, or scaling {kind: "yarn", factor, original, fast, slow, magnitude}: the
    frequencies of `yarn_factors`, and cos and sin times magnitude * ln(factor) + 1 (magnitude 0.1 by default)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.head_dim = int(p["head_dim"])
        self.rotary_dim = int(p.get("rotary_dim", self.head_dim))
        self.theta = float(p["theta"])
        self.scaling = dict(p.get("scaling") or {"kind": "default"})
        # which dimensions turn together: "half" pairs i with i + n/2, "adjacent" pairs 2i with 2i + 1. The tables
        # are the same; the kernel that applies them must pair as the model does
        self.pairs = str(p.get("pairs", "half"))
        if self.pairs not in ("half", "adjacent"):
            raise ValueError(f"rotary pairs `{self.pairs}` are unknown; known: half, adjacent")
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} must be even and at most the head size {self.head_dim}")
        self.cos = self.sin = None

    def host_tables(self, context_length: int):
        kind = self.scaling.get("kind", "default")
        factors, freq_scale, magnitude = None, 1.0, 1.0
        if kind == "yarn":
            sc = self.scaling
            factors = yarn_factors(self.rotary_dim, self.theta, float(sc["factor"]), float(sc["original"]),
                                   float(sc["fast"]), float(sc["slow"]))
            magnitude = float(sc.get("magnitude", 0.1)) * math.log(float(sc["factor"])) + 1.0
        elif kind == "llama3":
            factors = llama3_factors(self.rotary_dim, self.theta, float(self.scaling["factor"]),
                                     float(self.scaling["low_freq_factor"]), float(self.scaling["high_freq_factor"]),
                                     int(self.scaling["original_max_position_embeddings"]))
        elif kind == "linear":
            freq_scale = 1.0 / float(self.scaling["factor"])
        elif kind != "default":
            raise ValueError(f"rope scaling `{kind}` is unknown; known: default, llama3, linear, yarn")
        return rope_tables(context_length, self.rotary_dim, self.theta, factors, freq_scale, magnitude)

    def prepare(self, context_length: int) -> None:
        cos, sin = self.host_tables(context_length)
        self.cos = cos.to(self.rt.device)
        self.sin = sin.to(self.rt.device)

    def tables(self):
        """(cos, sin, rotary_dim, adjacent) for a kernel that pairs either way."""
        return self.cos, self.sin, self.rotary_dim, self.pairs == "adjacent"

    def fused_tables(self):
        if self.pairs != "half":
            raise ValueError("the fused rotate-and-store kernel pairs dimension i with i + n/2")
        return self.cos, self.sin, self.rotary_dim
