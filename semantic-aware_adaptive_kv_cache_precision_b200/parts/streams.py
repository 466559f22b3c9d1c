"""A pre-norm layer over several copies of the residual stream (`StreamBlockSpec`).

Each sublayer q (the mixer, then the feed-forward) reads a weighted sum of the streams and
writes its output back to all of them,

    u = sum_s in_q[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + out_q[t] y

and the mixer's input is first blended with the previous token's (token shift), whose value
is per-sequence state beside whatever the mixer itself caches. A sublayer's write-back and
the next sublayer's read and norm are one pass over the streams (`ops.streams_step`); the
write-back of a layer's last sublayer is handed to the next layer as `pending`, which does it
on its first pass. Without `connections` there is one stream and the plain `x += y`, through
the same kernels. Mixers and feed-forwards give their output through `produce(...)` (fp32 [T,
hidden]); a part that only has `forward(..., residual)` is given a zeroed tensor to add into.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.needs import MultiNeed, StateNeed
from ..weights.decl import TensorDecl
from .base import Part, build_part, register_part


class StreamUpdate:
    """A sublayer's output that still has to be written back to the streams."""

    __slots__ = ("y", "mix", "out_w")

    def __init__(self, y, mix, out_w):
        self.y, self.mix, self.out_w = y, mix, out_w

    def apply(self, xs) -> None:
        ops.streams_step(_as_streams(xs), y=self.y, mix=self.mix, out_w=self.out_w, reduce=False)


def _as_streams(x):
    return x if x.dim() == 3 else x.unsqueeze(0)


class StreamBlock(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        p = spec.prefix
        if not spec.connections and spec.streams != 1:
            raise ValueError("several streams need their connections")
        self.mixer_norm = build_part(spec.mixer_norm, p + spec.mixer_norm_name, mode)
        self.mixer = build_part(spec.mixer, p + spec.mixer_name + ".", mode)
        self.ffn = self.ffn_norm = None
        if spec.ffn is not None:
            self.ffn_norm = build_part(spec.ffn_norm, p + spec.ffn_norm_name, mode)
            self.ffn = build_part(spec.ffn, p + spec.ffn_name + ".", mode)
        self.parts = tuple(x for x in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)
                           if x is not None)
        self.graph_safe = all(getattr(part, "graph_safe", True) for part in self.parts)
        self.hc = {}
        self.shift = None

    def _sublayers(self):
        return (1, 2) if self.ffn is not None else (1,)

    def tensor_decls(self):
        s, p = self.spec, self.spec.prefix
        decls = [d for part in self.parts for d in part.tensor_decls()]
        if s.connections:
            n = s.streams
            for q in self._sublayers():
                decls += [TensorDecl(f"{p}hc{q}.in", (n,), init="uniform", span=(0.2, 0.8)),
                          TensorDecl(f"{p}hc{q}.out", (n,), init="ones_normal"),
                          TensorDecl(f"{p}hc{q}.mix", (n, n), init="eye_normal")]
        if s.token_shift:
            decls.append(TensorDecl(p + "shift", (s.mixer_norm.size,), init="uniform",
                                    span=(0.0, 0.8)))
        return decls

    def bind(self, arena):
        s, p = self.spec, self.spec.prefix
        for part in self.parts:
            part.bind(arena)
        for q in self._sublayers():
            self.hc[q] = tuple(arena.view(f"{p}hc{q}.{n}") for n in ("in", "mix", "out")) \
                if s.connections else (None, None, None)
        if s.token_shift:
            self.shift = arena.view(p + "shift")
            # the norm's weight and the connections' constants go to one kernel: one type
            self._same_type(self.shift, self.mixer_norm.weight)

    @staticmethod
    def _same_type(*tensors):
        if len({t.dtype for t in tensors}) > 1:
            raise TypeError("a stream block's constants must be stored in one type")

    def prepare(self, device, max_positions):
        for part in self.parts:
            part.prepare(device, max_positions)

    def cache_need(self):
        need = self.mixer.cache_need()
        if not self.spec.token_shift:
            return need
        return MultiNeed((need, StateNeed((self.spec.mixer_norm.size,), "float32")))

    carries_pending = True

    def forward(self, x, step, view, write_cache=True, pending=None, leave_pending=True):
        s = self.spec
        xs = _as_streams(x)
        if pending is not None and not isinstance(pending, StreamUpdate):
            pending = StreamUpdate(pending if pending.dim() == 2 else pending.sum(0), None, None)
        mixer_view, shift_view = (view.parts if s.token_shift else (view, None))
        w_in, w_mix, w_out = self.hc[1]
        norm = self.mixer_norm
        # one token a sequence: the blend with the token before is part of the same kernel
        inside = s.token_shift and step.is_decode
        h = ops.streams_step(
            xs, y=None if pending is None else pending.y,
            mix=None if pending is None else pending.mix,
            out_w=None if pending is None else pending.out_w, in_w=w_in, norm_w=norm.weight,
            eps=norm.spec.eps,
            out_dtype=torch.float32 if s.token_shift and not inside else self.act_dtype,
            shift=(shift_view.state, self.shift, step) if inside else None,
            keep_state=write_cache)
        if s.token_shift and not inside:
            h = ops.token_shift(h, shift_view.state, self.shift, step, self.act_dtype,
                                keep_state=write_cache)
        update = StreamUpdate(self._run(self.mixer, h, step, mixer_view, write_cache),
                              w_mix, w_out)
        if self.ffn is not None:
            w_in, w_mix, w_out = self.hc[2]
            norm = self.ffn_norm
            h = ops.streams_step(xs, y=update.y, mix=update.mix, out_w=update.out_w, in_w=w_in,
                                 norm_w=norm.weight, eps=norm.spec.eps, out_dtype=self.act_dtype)
            update = StreamUpdate(self._run(self.ffn, h, step), w_mix, w_out)
        if leave_pending:
            return update
        update.apply(xs)
        return None

    @staticmethod
    def _run(part, h, step, *cache):
        if hasattr(part, "produce"):
            return part.produce(h, step, *cache)
        y = torch.zeros((h.shape[0], part.spec.hidden), dtype=torch.float32, device=h.device)
        if cache:
            part.forward(h, step, cache[0], y, cache[1])
        else:
            part.forward(h, step, y)
        return y


register_part("stream_block", StreamBlock)
