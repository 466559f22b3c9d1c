"""Two-map differential attention (`DifferentialAttentionSpec`):

    [q | k | v | g] = h Wfused^T;   cache <- k, v
    a_m = softmax(q_m k_m^T * scale + mask) v            (m = 1, 2: two maps, one set of values)
    o = a_1 - lam a_2;   o <- o / sqrt(mean(o^2) + eps) * (1 - diff);   out = Wo [o * sigmoid(g)]

with lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, one number a layer, worked out in float64
when the weights are bound. No rotation. The mask is causal, and with `chunk` c a query sees
only the keys of its own run of c positions counted from the sequence's start. Queries lie
head by head as [map 1 | map 2]; a key/value head's cached key row holds both maps' keys, so
the kernel reads it once for all the query heads and maps that share it. Scores, softmax
weights, the weighted sums, the combination and the unit norm are fp32 in both modes
(`csrc/attention_distance.cu`).
"""

from __future__ import annotations

import math

import torch

from .. import ops
from ..cache.needs import KVNeed
from ..weights.decl import TensorDecl
from .base import Part, register_part

MAPS = 2


class DifferentialAttention(Part):
    kernel_libraries = ("attention_distance", "gemm_f32", "gemm_tc")

    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        s = spec
        if s.heads % s.kv_heads:
            raise ValueError(f"{s.heads} heads are not a multiple of {s.kv_heads} kv heads")
        if s.head_dim > 256 or s.value_dim > 512:
            raise ValueError("the attention kernel takes head_dim up to 256 and value_dim up to 512")
        self.q_cols = s.heads * MAPS * s.head_dim
        self.k_cols = s.kv_heads * MAPS * s.head_dim
        self.v_cols = s.kv_heads * s.value_dim
        self.g_cols = s.heads * s.value_dim if s.gate else 0
        self.lam = None

    def _fused(self):
        names = [("q", self.q_cols), ("k", self.k_cols), ("v", self.v_cols)]
        if self.spec.gate:
            names.append(("g", self.g_cols))
        return names

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        decls = [TensorDecl(p + n, (rows, s.hidden), group=p + "fused") for n, rows in self._fused()]
        decls += [TensorDecl(p + n, (s.head_dim,)) for n in ("lq1", "lk1", "lq2", "lk2")]
        decls.append(TensorDecl(p + "o", (s.hidden, s.heads * s.value_dim)))
        return decls

    def bind(self, arena):
        s, p = self.spec, self.prefix
        self.w_in = arena.group_view(p + "fused")
        if self.w_in is None:
            self.w_in = torch.cat([arena.view(p + n) for n, _ in self._fused()])
        lq1, lk1, lq2, lk2 = (arena.view(p + n).double().cpu() for n in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = (math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum()))
                    + s.diff)
        self.w_o = arena.view(p + "o")

    def cache_need(self):
        s = self.spec
        return KVNeed(s.kv_heads, MAPS * s.head_dim, None, value_dim=s.value_dim)

    def produce(self, h, step, view, write_cache=True):
        """The mixer's output, fp32 [T, hidden]."""
        s = self.spec
        fused = ops.linear(h, self.w_in, out_dtype=self.act_dtype)
        if write_cache:
            ops.kv_store(fused, self.q_cols, self.q_cols + self.k_cols, step.positions,
                         step.token_seq, view.block_table, view.keys, view.values)
        queries = fused[:, :self.q_cols].view(fused.shape[0], s.heads * MAPS, s.head_dim)
        gated = ops.cached_attention(
            queries, view.keys, view.values, step.positions, step.token_seq, view.block_table,
            s.heads, s.head_dim, s.value_dim, s.scale, maps=MAPS, chunk=s.chunk, lam=self.lam,
            out_scale=1.0 - s.diff, eps=s.eps,
            gate_elem_off=self.q_cols + self.k_cols + self.v_cols if s.gate else None,
            **self._decode_form(step, fused))
        return ops.linear(gated, self.w_o, out_dtype=torch.float32)

    def _decode_form(self, step, fused) -> dict:
        """See `LatentAttention._decode_form`; a token sees at most its chunk."""
        if fused.dtype == torch.float32 or not step.is_decode:
            return {}
        s = self.spec
        keys = step.max_len_bound or step.max_len
        if s.chunk:
            keys = min(keys, s.chunk)
        return {"heads_first": True,
                "key_splits": ops.plan_token_blocks(keys, step.tokens * s.kv_heads)}

    def forward(self, h, step, view, residual, write_cache=True):
        ops.add_into(residual, self.produce(h, step, view, write_cache))


register_part("differential_attention", DifferentialAttention)
