"""Attention whose keys and values come from a cached low-rank latent.

Per token the down-projection W_dkv h gives `kv_rank` values, RMS-normed with a weight into the latent c, and
`rot_dim` more that are rotated into a key part k_rot shared by all heads. Head a has k_a = U_a c (its unrotated
key) and v_a = V_a c; a query is [q_plain (dim) | q_rot (rot_dim, rotated)] per head, and
    score = (q_plain . k_a + q_rot . k_rot) * scale
over the keys the window allows, an ordinary softmax, the heads' outputs times sigmoid(W_g h), then W_o.
Only [c | k_rot] is cached, one row per position in the request's pages (a group with one key head and no value
slab). The kernels never form k_a or v_a: U_a^T carries the query into the latent space once per row
((U_a^T q_plain) . c = q_plain . (U_a c)) and V_a is applied to the softmax-weighted sum of latents.
Rotation turns pair i at position p by p times the position part's frequency i; which two dimensions are a pair,
(2i, 2i + 1) or (i, i + dims/2), is the position part's `pairs`.
Options: `gate` False leaves the output gate out (no tensor g); `sink` True puts one more term exp(sink_a), a stored
number per head with no key and no value, neither scaled nor normed, into head a's softmax denominator.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from . import rope  # noqa: F401  (registers the rotary tables this mixer asks for)
from .base import POSITIONS, CacheNeeds, KvNeeds, Mixer, PartSpec, TensorNeed, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """params: width, heads, dim, rot_dim, vdim, kv_rank, window (None: all keys), scale (None:
    1/sqrt(dim + rot_dim)), eps (of the latent's norm), position (a rotary PartSpec over rot_dim), gate (default
    True), sink (default False). tensors: q, dkv, dkv_norm, uk, uv, o, g (with the gate), sink [heads] (with the sink)."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width, self.heads = int(p["width"]), int(p["heads"])
        self.dim, self.rot_dim, self.vdim, self.rank = int(p["dim"]), int(p["rot_dim"]), int(p["vdim"]), int(p["kv_rank"])
        self.window = p.get("window")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dim + self.rot_dim)
        self.eps = float(p["eps"])
        self.gated, self.sink = bool(p.get("gate", True)), bool(p.get("sink", False))
        if not 1 <= self.rank <= ops.LATENT_MAX_RANK:
            raise ValueError(f"latent attention: latent size {self.rank} is outside what the kernels take "
                             f"(1..{ops.LATENT_MAX_RANK})")
        if self.dim < 1:
            raise ValueError("latent attention: a head needs at least one unrotated dimension")
        pos = p.get("position")
        self.position = POSITIONS.get(pos.kind)(pos, runtime) if isinstance(pos, PartSpec) else None
        self.rot_dims = self.position.rotary_dim if self.position is not None else 0
        if self.rot_dims > self.rot_dim:
            raise ValueError(f"latent attention: {self.rot_dims} rotated dimensions do not fit rot_dim {self.rot_dim}")
        self.key_dim = self.rank + self.rot_dim
        self.half_pairs = self.position is not None and self.position.pairs == "half"
        self.w_qkg = self.c_gain = self.w_ukt = self.w_uv = self.w_o = self.sink_values = None
        self._no_rot = None

    def cache_needs(self):
        return CacheNeeds(kv=KvNeeds(1, self.key_dim, self.window, v_head_dim=0))

    def tensors(self):
        t, H, E = self.spec.tensors, self.heads, self.width
        out = {t["q"]: TensorNeed((H * (self.dim + self.rot_dim), E)),
               t["dkv"]: TensorNeed((self.key_dim, E)),
               t["dkv_norm"]: TensorNeed((self.rank,), keep_fp32=True, init="ones"),
               t["uk"]: TensorNeed((H * self.dim, self.rank)), t["uv"]: TensorNeed((H * self.vdim, self.rank)),
               t["o"]: TensorNeed((E, H * self.vdim))}
        if self.gated:
            out[t["g"]] = TensorNeed((H * self.vdim, E))
        if self.sink:
            out[t["sink"]] = TensorNeed((H,), keep_fp32=True)
        return out

    def load(self, get):
        t, H = self.spec.tensors, self.heads
        self.w_qkg = torch.cat([get(t["q"]), get(t["dkv"])] + ([get(t["g"])] if self.gated else []), dim=0).contiguous()
        if self.sink:
            self.sink_values = get(t["sink"]).contiguous()
        self.c_gain = get(t["dkv_norm"])
        self.w_ukt = get(t["uk"]).view(H, self.dim, self.rank).transpose(1, 2).contiguous()  # [H, rank, dim]
        self.w_uv = get(t["uv"]).view(H, self.vdim, self.rank).contiguous()
        self.w_o = get(t["o"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_qkg, self.c_gain, self.w_ukt, self.w_uv, self.w_o,
                                                          self.sink_values) if w is not None)

    def prepare(self, context_length: int) -> None:
        if self.position is not None:
            self.position.prepare(context_length)
        else:  # nothing is rotated: one table row of no pairs per position is all the kernel looks at
            self._no_rot = torch.zeros(context_length, 0, dtype=torch.float32, device=self.rt.device)

    def forward(self, h, stream, step, cache) -> None:
        rt, rows, H = self.rt, h.shape[0], self.heads
        qd = self.dim + self.rot_dim
        qkg = rt.linear(h, self.w_qkg, out_dtype=torch.float32)  # [H x (q_plain | q_rot) | c, k_rot | gate]
        qk = rt.empty(rows, H, self.key_dim, dtype=torch.float32)  # per head [U^T q_plain | rotated q_rot]
        cos, sin = (self.position.cos, self.position.sin) if self.position is not None else (self._no_rot, self._no_rot)
        ops.latent_prepare(qkg, H, self.dim, self.rot_dim, self.rank, self.c_gain, self.eps, cos, sin, self.rot_dims,
                           qk, cache, step, rt.err, half_pairs=self.half_pairs)
        ops.head_linear(qkg, qkg.stride(0), qd, self.w_ukt, qk, H * self.key_dim, self.key_dim, rows)
        mixed = rt.empty(rows, H, self.rank, dtype=torch.float32)  # softmax-weighted sums of latents
        ops.latent_attention(qk, mixed, cache, step, H, self.rank, self.key_dim, self.scale, self.window, rt.err,
                             sink_values=self.sink_values)
        att = rt.empty(rows, H * self.vdim)
        ops.head_linear(mixed, H * self.rank, self.rank, self.w_uv, att, H * self.vdim, self.vdim, rows,
                        gate=qkg[:, H * qd + self.key_dim:] if self.gated else None, ldg=qkg.stride(0))
        rt.stream(stream).add_linear(att, self.w_o)
