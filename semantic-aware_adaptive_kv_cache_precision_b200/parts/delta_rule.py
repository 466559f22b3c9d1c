"""The delta-rule recurrent mixer (`DeltaRuleSpec`): one matrix of state a head, decayed
channel by channel, with the part along the current unit key partly removed before the new
key-value pair is written:

    S <- diag(w) S - (a * u)(u^T S) + k v^T;    o = S^T r
    out = Wo [ o / rms(o) * norm * sigmoid(Wg x) ]

The six projections that read the mixer's input (r, k, v, g, the removal rate's and the
decay's first, narrow matrix) are one product over their rows laid back to back, with an
fp32 result: everything after it (the decay's second matrix and its exponentials, the
sigmoids, the unit key, the recurrence, the per-head norm and the gate) is one kernel in
fp32 (`csrc/delta_rule.cu`). The state lives in the cache as fixed-size per-sequence state.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.needs import StateNeed
from ..weights.decl import TensorDecl
from .base import Part, register_part

_FUSED = ("r", "k", "v", "g", "a", "w1")


class DeltaRuleMixer(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        if spec.head_dim > 256:
            raise ValueError(f"head_dim {spec.head_dim}: the recurrence kernel takes up to 256")

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        hd = s.heads * s.head_dim
        decls = [TensorDecl(p + n, (s.decay_rank if n == "w1" else hd, s.hidden),
                            group=p + "fused") for n in _FUSED]
        return decls + [
            TensorDecl(p + "a.b", (hd,)),
            TensorDecl(p + "w2", (hd, s.decay_rank)),
            TensorDecl(p + "w0", (hd,), init="uniform", span=(-6.0, 0.0)),
            TensorDecl(p + "norm", (hd,), init="ones_normal"),
            TensorDecl(p + "o", (s.hidden, hd)),
        ]

    def bind(self, arena):
        p = self.prefix
        self.w_in = arena.group_view(p + "fused")
        if self.w_in is None:
            self.w_in = torch.cat([arena.view(p + n) for n in _FUSED])
        self.a_bias, self.w2, self.w0 = (arena.view(p + n) for n in ("a.b", "w2", "w0"))
        self.norm_w, self.w_o = arena.view(p + "norm"), arena.view(p + "o")
        hd = self.spec.heads * self.spec.head_dim
        self.offsets = tuple(i * hd for i in range(6))       # r, k, v, g, a, then the narrow one

    def cache_need(self):
        s = self.spec
        return StateNeed((s.heads, s.head_dim, s.head_dim), "float32")

    def produce(self, h, step, view, write_cache=True):
        """The mixer's output, fp32 [T, hidden]."""
        s = self.spec
        proj = ops.linear(h, self.w_in, out_dtype=torch.float32)
        mixed = ops.delta_rule(proj, self.offsets, self.w2, self.w0, self.a_bias, self.norm_w,
                               view.state, step, s.heads, s.head_dim, s.decay_scale, s.key_eps,
                               s.eps, self.act_dtype, keep_state=write_cache)
        return ops.linear(mixed, self.w_o, out_dtype=torch.float32)

    def forward(self, h, step, view, residual, write_cache=True):
        ops.add_into(residual, self.produce(h, step, view, write_cache))


register_part("general_delta", DeltaRuleMixer)
