"""A layer with a norm before and after each sublayer (`SandwichBlockSpec`):

    x += norm1b(mixer(norm1(x)));   x += norm2b(ffn(norm2(x)))

on the fp32 residual stream. A sublayer's output is normed and added in the same pass over
the stream that norms the next sublayer's input (`LayerNorm.forward(x, add=, add_norm=)`);
what the layer's last sublayer produced leaves the block as `pending` (a `NormedUpdate`), so
that the next layer's first norm does it on its way. Mixers and feed-forwards give their output
through `produce(...)` (fp32 [T, hidden]); a part that only has `forward(..., residual)` is
given a zeroed tensor to add into.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, build_part, register_part


class NormedUpdate:
    """A sublayer's output that still has to be normed and added to the stream."""

    __slots__ = ("y", "norm")

    def __init__(self, y, norm):
        self.y, self.norm = y, norm

    def apply(self, x) -> None:
        _complete(x, self.y, self.norm)


def _complete(x, y, norm) -> None:
    if hasattr(norm, "complete"):
        norm.complete(x, y)
    else:
        ops.add_into(x, norm.forward(y, out_dtype=torch.float32))


def _normed(norm, x, pending):
    """norm(x) after the stream has taken up what is pending."""
    if pending is None:
        return norm.forward(x)
    if isinstance(pending, NormedUpdate):
        if getattr(norm, "folds_normed", False) and getattr(pending.norm, "folds_normed", False):
            return norm.forward(x, add=pending.y, add_norm=pending.norm)
        pending.apply(x)
    elif hasattr(pending, "apply"):
        pending.apply(x)
    else:
        ops.add_into(x, pending)
    return norm.forward(x)


class SandwichBlock(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        p = spec.prefix
        pre1, post1, pre2, post2 = spec.norm_names
        self.mixer_norm = build_part(spec.norm, p + pre1, mode)
        self.mixer_after = build_part(spec.norm, p + post1, mode)
        self.mixer = build_part(spec.mixer, p + spec.mixer_name + ".", mode)
        self.ffn = self.ffn_norm = self.ffn_after = None
        if spec.ffn is not None:
            self.ffn_norm = build_part(spec.norm, p + pre2, mode)
            self.ffn_after = build_part(spec.norm, p + post2, mode)
            self.ffn = build_part(spec.ffn, p + spec.ffn_name + ".", mode)
        self.parts = tuple(x for x in (self.mixer_norm, self.mixer_after, self.mixer,
                                       self.ffn_norm, self.ffn_after, self.ffn) if x is not None)
        self.graph_safe = all(getattr(part, "graph_safe", True) for part in self.parts)
        self.kernel_libraries = tuple(n for part in self.parts
                                      for n in getattr(part, "kernel_libraries", ()))

    def tensor_decls(self):
        return [d for part in self.parts for d in part.tensor_decls()]

    def bind(self, arena):
        for part in self.parts:
            part.bind(arena)

    def prepare(self, device, max_positions):
        for part in self.parts:
            part.prepare(device, max_positions)

    def cache_need(self):
        return self.mixer.cache_need()

    carries_pending = True

    def forward(self, x, step, view, write_cache=True, pending=None, leave_pending=True):
        h = _normed(self.mixer_norm, x, pending)
        update = NormedUpdate(_run(self.mixer, h, step, view, write_cache), self.mixer_after)
        if self.ffn is not None:
            h = _normed(self.ffn_norm, x, update)
            update = NormedUpdate(_run(self.ffn, h, step), self.ffn_after)
        if leave_pending:
            return update
        update.apply(x)
        return None


def _run(part, h, step, *cache):
    if hasattr(part, "produce"):
        return part.produce(h, step, *cache)
    y = torch.zeros((h.shape[0], part.spec.hidden), dtype=torch.float32, device=h.device)
    if cache:
        part.forward(h, step, cache[0], y, cache[1])
    else:
        part.forward(h, step, y)
    return y


register_part("sandwich_block", SandwichBlock)
