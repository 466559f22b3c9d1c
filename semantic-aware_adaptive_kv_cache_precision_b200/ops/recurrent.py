"""The delta-rule recurrence over a step's tokens (`csrc/delta_rule.cu`)."""

from __future__ import annotations

import torch

from ._lib import KernelError, call, dtype_code, ptr, require_cuda


def delta_rule(proj: torch.Tensor, offsets: tuple, w2: torch.Tensor, w0: torch.Tensor,
               a_bias: torch.Tensor, norm_w: torch.Tensor, state: torch.Tensor, step, heads: int,
               dim: int, decay_scale: float, key_eps: float, eps: float,
               out_dtype: torch.dtype, keep_state: bool = True) -> torch.Tensor:
    """`proj`: fp32 [T, P], whose columns from `offsets` = (r, k, v, g, a, l) on are the
    receptance, key, value, gate and removal-rate pre-activations (heads * dim each) and the
    decay's low-rank output (rank = w2.shape[1]). `state`: fp32 [slots, heads, dim, dim], read
    and left for each of the step's sequences. Returns the normed, gated output [T, heads *
    dim] of `out_dtype`."""
    require_cuda(proj, w2, w0, a_bias, norm_w, state)
    tokens = proj.shape[0]
    hd = heads * dim
    rank = w2.shape[1]

    def check(cond, message):
        if not cond:
            raise KernelError(message)

    check(proj.dtype == torch.float32 and proj.dim() == 2 and proj.stride(1) == 1,
          "proj: fp32 [T, P] with contiguous rows")
    check(len(offsets) == 6 and max(offsets[:5]) + hd <= proj.shape[1]
          and offsets[5] + rank <= proj.shape[1], "offsets reach beyond proj's columns")
    check(w2.shape == (hd, rank) and w2.is_contiguous(), "w2: [heads * dim, rank]")
    for t, name in ((w0, "w0"), (a_bias, "a_bias"), (norm_w, "norm_w")):
        check(t.shape == (hd,) and t.is_contiguous() and t.dtype == w2.dtype,
              f"{name}: [heads * dim] of w2's type")
    check(state.dtype == torch.float32 and state.is_contiguous()
          and tuple(state.shape[1:]) == (heads, dim, dim), "state: fp32 [slots, heads, dim, dim]")
    out = torch.empty((tokens, hd), dtype=out_dtype, device=proj.device)
    prepared = torch.empty((tokens, 3, hd), dtype=torch.float32, device=proj.device)
    raw = torch.empty((tokens, hd), dtype=torch.float32, device=proj.device)
    call("sakv_delta_rule", ptr(proj), proj.stride(0), *[int(o) for o in offsets], ptr(w2),
         ptr(w0), ptr(a_bias), ptr(norm_w), dtype_code(w2.dtype), ptr(prepared), ptr(raw), ptr(state),
         ptr(step.cu_seqlens), ptr(step.slots), ptr(out), dtype_code(out_dtype), tokens,
         step.sequences, heads, dim, rank,
         int(max(1, min(16, getattr(step, "max_new", 0) or tokens))),
         float(decay_scale), float(key_eps), float(eps), int(keep_state))
    return out
