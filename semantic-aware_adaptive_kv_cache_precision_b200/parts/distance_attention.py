"""Windowed grouped-query attention with a logarithmic distance penalty
(`LogDistanceAttentionSpec`):

    s_ij = q_i . k_j * scale - slope[h] * ln(1 + rate[h] * (i - j)),   0 <= i - j < window
    out = Wo [ softmax(s) v * sigmoid(Wg x)[h] ] (+ bo)

No rotation: the distance enters through the penalty alone, so keys go to the cache as the
projection made them. Queries, keys, values and the gates' rows are one product over [Wq; Wk;
Wv; Wg]; values may have a width of their own (`KVNeed.value_dim`). Scores, penalty, softmax
and the weighted sum are fp32 in both modes (`csrc/attention_distance.cu`).
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.needs import KVNeed
from ..weights.decl import TensorDecl
from .base import Part, register_part


class LogDistanceAttention(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        s = spec
        if s.heads % s.kv_heads:
            raise ValueError(f"{s.heads} heads are not a multiple of {s.kv_heads} kv heads")
        if max(s.head_dim, s.value_dim) > 512:
            raise ValueError("the attention kernel takes key and value widths up to 512")
        self.q_cols = s.heads * s.head_dim
        self.k_cols = s.kv_heads * s.head_dim
        self.v_cols = s.kv_heads * s.value_dim

    def _fused(self):
        names = [("q", self.q_cols), ("k", self.k_cols), ("v", self.v_cols)]
        if self.spec.head_gate:
            names.append(("g", self.spec.heads))
        return names

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        decls = [TensorDecl(p + n, (rows, s.hidden), group=p + "fused") for n, rows in self._fused()]
        if s.qkv_bias:
            decls += [TensorDecl(f"{p}{n}.b", (rows,), group=p + "fused.b")
                      for n, rows in self._fused() if n != "g"]
        decls += [TensorDecl(p + "r1", (s.heads,), init="uniform", span=(0.0, 2.0)),
                  TensorDecl(p + "r2", (s.heads,), init="uniform", span=(0.1, 0.5)),
                  TensorDecl(p + "o", (s.hidden, s.heads * s.value_dim))]
        if s.out_bias:
            decls.append(TensorDecl(p + "o.b", (s.hidden,)))
        return decls

    def bind(self, arena):
        s, p = self.spec, self.prefix
        names = [n for n, _ in self._fused()]
        self.w_in = arena.group_view(p + "fused")
        if self.w_in is None:
            self.w_in = torch.cat([arena.view(p + n) for n in names])
        self.b_in = None
        if s.qkv_bias:
            b = arena.group_view(p + "fused.b")
            if b is None:
                b = torch.cat([arena.view(f"{p}{n}.b") for n in names if n != "g"])
            if s.head_gate:          # the gates' rows have no bias: zeros complete the vector
                b = torch.cat([b, torch.zeros(s.heads, dtype=b.dtype, device=b.device)])
            self.b_in = b
        self.slope = arena.view(p + "r1").float().contiguous()
        self.rate = arena.view(p + "r2").float().contiguous()
        self.w_o = arena.view(p + "o")
        self.b_o = arena.view(p + "o.b") if s.out_bias else None

    def cache_need(self):
        s = self.spec
        return KVNeed(s.kv_heads, s.head_dim, s.window, value_dim=s.value_dim)

    def produce(self, h, step, view, write_cache=True):
        """The mixer's output, fp32 [T, hidden]."""
        s = self.spec
        qkv = ops.linear(h, self.w_in, self.b_in, out_dtype=self.act_dtype)
        if write_cache:
            ops.kv_store(qkv, self.q_cols, self.q_cols + self.k_cols, step.positions,
                         step.token_seq, view.block_table, view.keys, view.values)
        attended = ops.distance_attention(
            qkv, view.keys, view.values, step.positions, step.token_seq, view.block_table,
            s.heads, s.scale, s.window, self.slope, self.rate,
            gate_off=self.q_cols + self.k_cols + self.v_cols if s.head_gate else None,
            splits=self._splits(step, qkv))
        return ops.linear(attended, self.w_o, self.b_o, out_dtype=torch.float32)

    def _splits(self, step, qkv) -> int:
        """How many warps share a token's keys. One in the 32-bit mode and for prompts (the
        sums then have one order however the tokens are cut); for decode steps in bfloat16 one
        warp for every two chunks of 32 keys that a token can see, up to 16. (A decode
        step's graph is keyed by the width of the block lists, which bounds the length.)"""
        if qkv.dtype == torch.float32 or not step.is_decode:
            return 1
        keys = step.max_len_bound or step.max_len
        if self.spec.window:
            keys = min(keys, self.spec.window + 31)
        splits = 1
        while splits < 16 and splits * 64 < keys:
            splits *= 2
        return splits

    def forward(self, h, step, view, residual, write_cache=True):
        ops.add_into(residual, self.produce(h, step, view, write_cache))


register_part("log_distance_attention", LogDistanceAttention)
