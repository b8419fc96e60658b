"""Grouped-query attention over the paged cache.

q = h Wq^T, k = h Wk^T, v = h Wv^T (+ biases when the tensors exist); q and k
are rotated, k and v written to the request's pages, and each row attends to
keys lo..P of its request with scale 1/sqrt(head_dim) applied before the mask;
query head h reads key head h // (n_heads / n_kv_heads); then the output
projection is added to the stream (src/provider/local/model/cpu.rs:2822-2991,
3490-3521, model/cpu/paged_attn.rs:115-175, model/params.rs:704). The three
projections are stacked into one weight at load (the reference accepts the
stacked form: model/cpu.rs:3296-3301).

A layer that reads another layer's pages (`shares_cache`) has only q and o.

Values may have a size of their own (`v_head_dim`), the concatenated heads may pass an output gate
sigmoid(W_g h) before the output projection (`gate`), and the rotation may pair adjacent dimensions: any of these
takes the general path (one stacked projection q | k | v | gate, a rotate-and-store kernel that knows the columns,
the plain attention kernel with value rows of their own size).

Further options of the general path: an RMS norm per head on queries and keys with a weight of the head's size shared
by the heads (`qk_norm`, before the rotation) and on values without a weight (`v_norm`, before they are kept), a
smooth cap on the scaled score, c tanh(s / c) (`softcap`), and a sink: one more term exp(0), with no value, in the
softmax's denominator (`sink`).

Values of a size that is no multiple of the keys' are kept padded with zeros to the next multiple where the
tensor-core kernels take the rest of the shape (bfloat16, key sizes in steps of 16 up to 128, no output gate): the pool's
rows, the attention output and the output projection's input columns (zero columns, added at load) are that wide, and
the layer runs slab by slab like one whose values are a multiple. The norm on values is over the stored ones.

Three more options of the general path. `qk_norm` "whole": the RMS norm of q (and of k) is taken over the whole
projection, all heads at once, with a weight of that size (`q_norm` [heads * head_dim], `k_norm` [kv heads * head_dim]).
`q_temp` {coef, every}: the query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1) (after norm
and rotation). `sink` "learned": the sink's score is a stored number per query head (`sink` [heads], neither scaled nor
capped) instead of 0. `gate` "head": one gate per head, sigmoid(W_g h)_a with `g` [heads, width], multiplies head a's
output.
"""
from __future__ import annotations

import dataclasses
import math

import torch

from ..kernels import ops
from .base import POSITIONS, CacheNeeds, KvNeeds, Mixer, PartSpec, TensorNeed, register_mixer


@register_mixer("attention")
class PagedAttention(Mixer):
    """params: width, n_heads, n_kv_heads, head_dim, window (None: all keys), scale (None: 1/sqrt(head_dim)),
    position (PartSpec or None), shares_cache (bool), v_head_dim (None: head_dim), gate (bool, or "head"), qk_norm
    (bool, or "whole"), v_norm (bool), eps (of those norms), softcap (None or 0: none), sink (bool, or "learned"),
    q_temp ({coef, every} or None). tensors: q, k, v, o, g (with `gate`), q_norm and k_norm (with `qk_norm`), sink
    (with a learned sink) and optional q_bias, k_bias, v_bias, o_bias."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width = int(p["width"])
        self.n_heads = int(p["n_heads"])
        self.n_kv_heads = int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.window = p.get("window")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        self.shares_cache = bool(p.get("shares_cache", False))
        self.v_head_dim = int(p["v_head_dim"]) if p.get("v_head_dim") else self.head_dim
        self.head_gate = p.get("gate") == "head"  # one gate per head instead of one per value
        self.gated = bool(p.get("gate", False)) and not self.head_gate
        self.qk_norm, self.v_norm = bool(p.get("qk_norm", False)), bool(p.get("v_norm", False))
        self.norm_whole = p.get("qk_norm") == "whole"  # over the whole projection instead of per head
        self.eps = float(p.get("eps", 1e-6))
        self.softcap = float(p.get("softcap") or 0.0)
        self.sink = bool(p.get("sink", False))
        self.sink_learned = p.get("sink") == "learned"
        qt = p.get("q_temp")
        self.q_temp = (float(qt["coef"]), int(qt["every"])) if qt else None
        if self.q_temp is not None and self.q_temp[1] < 1:
            raise ValueError(f"attention: a query temperature every {self.q_temp[1]} positions is not positive")
        if self.norm_whole and self.v_norm:
            raise ValueError("attention: a norm over the whole projection is not combined with a norm on values")
        if self.softcap < 0:
            raise ValueError(f"attention: a score cap of {self.softcap} is not positive")
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_kv_heads} key heads must divide {self.n_heads} query heads")
        if not 1 <= self.head_dim <= ops.ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"attention: head size {self.head_dim} is outside what the kernels take "
                             f"(1..{ops.ATTENTION_MAX_HEAD_DIM})")
        pos = p.get("position")
        self.position = POSITIONS.get(pos.kind)(pos, runtime) if isinstance(pos, PartSpec) else None
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.w_qn = self.w_kn = self.sink_values = None
        # what the stacked-projection kernels of the usual path do not take
        self.normed = self.qk_norm or self.v_norm or self.q_temp is not None
        self.general = (self.v_head_dim != self.head_dim or self.gated or self.head_gate or self.normed
                        or self.softcap > 0 or self.sink or getattr(self.position, "pairs", "half") != "half")
        if self.general and self.shares_cache:
            raise ValueError("attention: a layer that reads another layer's pages takes neither a value size of its "
                             "own, an output gate, head norms, a score cap, a sink nor adjacent rotation pairs")
        # the width of a value row in the pool: padded to a multiple of the key size for the tensor-core kernels
        self.v_pool_dim = self.v_head_dim
        d, dv = self.head_dim, self.v_head_dim
        if (self.general and not self.gated and runtime is not None and runtime.dtype == torch.bfloat16 and dv % d
                and d % 16 == 0 and d <= 128 and -(-dv // d) * d <= 2 * ops.ATTENTION_MAX_HEAD_DIM):
            self.v_pool_dim = -(-dv // d) * d
        if self.general and not 1 <= self.v_head_dim <= 2 * ops.ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"attention: value size {self.v_head_dim} is outside what the kernels take "
                             f"(1..{2 * ops.ATTENTION_MAX_HEAD_DIM})")

    # ------------------------------------------------------------ description
    def cache_needs(self):
        return CacheNeeds(kv=KvNeeds(self.n_kv_heads, self.head_dim, self.window,
                                     None if self.v_pool_dim == self.head_dim else self.v_pool_dim))

    def tensors(self):
        t, d, dv = self.spec.tensors, self.head_dim, self.v_head_dim
        out = {t["q"]: TensorNeed((self.n_heads * d, self.width)),
               t["o"]: TensorNeed((self.width, self.n_heads * dv))}
        if self.gated:
            out[t["g"]] = TensorNeed((self.n_heads * dv, self.width))
        if self.head_gate:
            out[t["g"]] = TensorNeed((self.n_heads, self.width))
        if self.qk_norm:
            whole = self.norm_whole
            out[t["q_norm"]] = TensorNeed((self.n_heads * d if whole else d,), keep_fp32=True, init="ones")
            out[t["k_norm"]] = TensorNeed((self.n_kv_heads * d if whole else d,), keep_fp32=True, init="ones")
        if self.sink_learned:
            out[t["sink"]] = TensorNeed((self.n_heads,), keep_fp32=True)
        if not self.shares_cache:
            out[t["k"]] = TensorNeed((self.n_kv_heads * d, self.width))
            out[t["v"]] = TensorNeed((self.n_kv_heads * dv, self.width))
        for role, rows in (("q_bias", self.n_heads * d), ("k_bias", self.n_kv_heads * d),
                           ("v_bias", self.n_kv_heads * dv), ("o_bias", self.width)):
            if role in t and not (self.shares_cache and role in ("k_bias", "v_bias")):
                out[t[role]] = TensorNeed((rows,), optional=True)
        return out

    def load(self, get):
        t = self.spec.tensors
        roles = ["q"] if self.shares_cache else ["q", "k", "v"] + (["g"] if self.gated or self.head_gate else [])
        stacked = [get(t[r]) for r in roles]
        biases = [get(t[r + "_bias"]) if r + "_bias" in t else None for r in roles]
        rows = sum(w.shape[0] for w in stacked)
        if self.head_gate and rows % 8:  # rows of no weight, so that a projected row stays a multiple of 16 bytes
            stacked.append(stacked[0].new_zeros(8 - rows % 8, self.width))
            biases.append(None)
        self.w_qkv = torch.cat(stacked, dim=0).contiguous()
        if any(b is not None for b in biases):
            if any(b is None for b in biases[:3]):
                raise ValueError("attention biases must be given for q, k and v together")
            biases = [b if b is not None else biases[0].new_zeros(w.shape[0]) for b, w in zip(biases, stacked)]
            self.b_qkv = torch.cat(biases).contiguous()
        self.w_o = get(t["o"])
        if self.v_pool_dim != self.v_head_dim:  # zero columns where the padded attention output holds zeros
            w = self.w_o.view(self.width, self.n_heads, self.v_head_dim)
            wide = w.new_zeros(self.width, self.n_heads, self.v_pool_dim)
            wide[:, :, :self.v_head_dim] = w
            self.w_o = wide.view(self.width, self.n_heads * self.v_pool_dim).contiguous()
        self.b_o = get(t["o_bias"]) if "o_bias" in t else None
        if self.qk_norm:
            self.w_qn, self.w_kn = get(t["q_norm"]), get(t["k_norm"])
        if self.sink_learned:
            self.sink_values = get(t["sink"]).contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.w_o, self.b_qkv, self.b_o, self.w_qn, self.w_kn,
                                                          self.sink_values) if w is not None)

    def prepare(self, context_length: int) -> None:
        if self.position is not None:
            self.position.prepare(context_length)

    # ------------------------------------------------------------ step
    def plan(self, step):
        """How this step's rows go to the attention kernels: made once per step from the per-request description
        (`StepBatch.req_row0/req_count/req_start`) and shared by the attention layers of the step."""
        return ops.attention_plan(step)

    def value_split(self, cache) -> int:
        """How this layer's value pool is laid out. r >= 1: for the tensor-core kernels, which want values as wide
        as keys: values are r times as wide, the pool is r slabs of heads as wide as the keys, and the kernels run
        once per slab against the same keys. 0: value rows as they are, for the plain kernel. The answer depends on
        the layer's sizes, the compute dtype and the page size alone, so every step lays the pool out alike."""
        d, dv, bs = self.head_dim, self.v_pool_dim, cache.block_size
        if (self.rt.dtype == torch.bfloat16 and dv % d == 0 and bs & (bs - 1) == 0
                and ops.attention_mma_supported(self.n_heads, self.n_kv_heads, d, self.w_qkv.shape[0], self.n_heads * d)):
            return dv // d
        return 0

    def forward_general(self, h, stream, step, cache) -> None:
        """q | k | v | gate in one projection; rotation (either pairing, part of a head) and the page write; attention
        on the tensor cores, once per slab of the values, where the shape allows it, else the plain kernel over value
        rows of their own size; the gate; the output projection."""
        nh, nkv, d, dv = self.n_heads, self.n_kv_heads, self.head_dim, self.v_pool_dim  # (dv: of pool and output)
        dv_row = self.v_head_dim if dv != self.v_head_dim else 0  # the projection's value heads, where narrower
        rows = h.shape[0]
        proj = self.rt.linear(h, self.w_qkv, bias=self.b_qkv)
        cos, sin, rot, adjacent = self.position.tables() if self.position is not None else (None, None, 0, False)
        split = self.value_split(cache)
        plan = self.plan(step) if split else None
        if split > 1 and plan is None:
            raise ValueError("attention: this layer's value pool is laid out for the tensor-core kernels, which need "
                             "the step's per-request description")
        tensor_cores = split >= 1 and plan is not None
        split = max(split, 1)
        if self.normed:
            ops.norm_rope_store(proj, nh * d, (nh + nkv) * d, step.positions, step.seq_of_row, cache.tables, cos, sin,
                                rot, adjacent, self.w_qn, self.w_kn, self.v_norm, self.eps, cache.k, cache.v,
                                cache.block_size, nh, nkv, d, dv, self.rt.err, v_split=split, v_row_dim=dv_row,
                                whole=self.norm_whole, q_temp=self.q_temp)
        else:
            ops.rope_store_general(proj, nh * d, (nh + nkv) * d, step.positions, step.seq_of_row, cache.tables, cos, sin,
                                   rot, adjacent, cache.k, cache.v, cache.block_size, nh, nkv, d, dv, self.rt.err,
                                   v_split=split, v_row_dim=dv_row)
        g_col = (nh + nkv) * d + nkv * self.v_head_dim
        gate = proj[:, g_col:] if self.gated else None  # (a layer with a gate per value is never padded)
        attn = self.rt.empty(rows, nh * dv)
        if tensor_cores:
            slabs = cache.v.view(split, *cache.k.shape)
            parts = self.rt.empty(split, rows, nh * d) if (split > 1 or gate is not None) else attn.view(1, rows, nh * d)
            for j in range(split):
                ops.attention(proj, parts[j], dataclasses.replace(cache, v=slabs[j]), step, plan, nh, nkv, d, self.scale,
                              self.window, self.rt.err, softcap=self.softcap, sink=self.sink,
                              sink_values=self.sink_values)
            if parts.data_ptr() != attn.data_ptr():
                ops.gate_merge(parts, gate, attn, nh, dv)
        else:
            ops.attention_generic_v(proj, proj.stride(0), attn, cache.k, cache.v, step.positions, step.seq_of_row,
                                    cache.tables, nh, nkv, d, dv, self.scale, self.window, self.rt.err,
                                    softcap=self.softcap, sink=self.sink, sink_values=self.sink_values)
            if gate is not None:
                ops.sigmoid_gate_(attn, gate)
        if self.head_gate:
            ops.head_gate_(attn, proj[:, g_col:g_col + nh], nh, dv)
        stream.add_linear(attn, self.w_o, bias=self.b_o)

    def forward(self, h, stream, step, cache) -> None:
        stream = self.rt.stream(stream)
        if self.general:
            return self.forward_general(h, stream, step, cache)
        nh, d = self.n_heads, self.head_dim
        nkv = 0 if self.shares_cache else self.n_kv_heads
        fused = self.position.fused_tables() if self.position is not None else None
        kpool, vpool = (None, None) if nkv == 0 else (cache.k, cache.v)
        plan = self.plan(step)
        if (fused is not None and self.rt.use_partials and h.shape[0] <= ops.ROPE_PARTIAL_MAX_ROWS
                and ops.gemm_partial_supported(h, self.w_qkv)):
            # few tokens: the projection leaves its K slices unadded; rotate-and-store adds them in 32-bit
            cos, sin, rot = fused
            parts = ops.gemm_partial(h, self.w_qkv, self.rt.err)
            if ops.attention_decode_fused_supported(plan, cache, h.dtype, h.shape[0], nh, self.n_kv_heads, d):
                # single tokens only: adding the slices, rotation, the page write and attention are one launch
                attn = self.rt.empty(h.shape[0], nh * d)
                chunk, n_splits = plan.chunk(self.n_kv_heads, d)
                ops.attention_decode_fused(parts, self.b_qkv, cos, sin, rot, nkv > 0, attn, cache.k, cache.v,
                                           step.positions, step.seq_of_row, cache.tables, None,
                                           plan.n_decode, nh, self.n_kv_heads, d, self.scale, self.window, chunk,
                                           n_splits, self.rt.err)
                stream.add_linear(attn, self.w_o, bias=self.b_o)
                return
            q = self.rt.empty(h.shape[0], nh * d)
            ops.rope_store_partial(parts, self.b_qkv, q, step.positions, step.seq_of_row, cache.tables, cos, sin, rot,
                                   kpool, vpool, cache.block_size, nh, nkv, d, self.rt.err)
        else:
            q = self.rt.linear(h, self.w_qkv, bias=self.b_qkv)  # [rows, (nh + 2 nkv) d]; q is the head of each row
            if fused is None:
                if self.position is not None:
                    self.position.apply(q, nh, nkv, d, step.positions)
                cos = sin = None
                rot = 0
            else:
                cos, sin, rot = fused
            ops.rope_store(q, step.positions, step.seq_of_row, cache.tables, cos, sin, rot, kpool, vpool,
                           cache.block_size, nh, nkv, d, self.rt.err)
        attn = self.rt.empty(h.shape[0], nh * d)
        ops.attention(q, attn, cache, step, plan, nh, self.n_kv_heads, d, self.scale, self.window, self.rt.err)
        stream.add_linear(attn, self.w_o, bias=self.b_o)
