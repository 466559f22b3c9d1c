"""Several copies of the residual stream, and the blend of a row with the row before it
(`csrc/streams.cu`)."""

from __future__ import annotations

import torch

from ._lib import KernelError, call, dtype_code, ptr, require_cuda


def _check(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


def _constants(*tensors):
    given = [t for t in tensors if t is not None]
    require_cuda(*given)
    kinds = {t.dtype for t in given}
    _check(len(kinds) <= 1 and all(t.is_contiguous() for t in given),
           "the constants of a streams step must be contiguous and of one type")
    return dtype_code(kinds.pop()) if kinds else 0


def streams_step(xs: torch.Tensor, *, y: torch.Tensor | None = None,
                 mix: torch.Tensor | None = None, out_w: torch.Tensor | None = None,
                 reduce: bool = True, in_w: torch.Tensor | None = None,
                 norm_w: torch.Tensor | None = None, eps: float = 0.0,
                 out_dtype: torch.dtype = torch.float32, shift: tuple | None = None,
                 keep_state: bool = True) -> torch.Tensor | None:
    """On `xs` (fp32 [streams, T, width], updated in place): with `y` (fp32 [T, width]) first
    `xs[t] <- sum_s mix[s, t] xs[s] + out_w[t] y` (`mix` None: the identity, `out_w` None:
    ones); then, with `reduce`, returns `norm(sum_s in_w[s] xs[s])` as [T, width] of
    `out_dtype` (`in_w` None: ones; `norm_w` None: the sum itself, fp32).

    `shift` = (state, shift_w, step), only for a step in which every sequence brings ONE token:
    the result is blended with the sequence's row before as `token_shift` does, in the same
    kernel, and `state` receives the unblended rows."""
    require_cuda(xs, y)
    _check(xs.dtype == torch.float32 and xs.dim() == 3 and xs[0].is_contiguous(),
           "xs: fp32 [streams, T, width] with contiguous streams")
    streams, tokens, width = xs.shape
    _check(y is not None or reduce, "a streams step without y and without a result does nothing")
    if y is not None:
        _check(y.dtype == torch.float32 and y.shape == (tokens, width) and y.is_contiguous(),
               "y: contiguous fp32 [T, width]")
        _check(mix is None or mix.shape == (streams, streams), "mix: [streams, streams]")
        _check(out_w is None or out_w.shape == (streams,), "out_w: [streams]")
    _check(in_w is None or in_w.shape == (streams,), "in_w: [streams]")
    _check(norm_w is None or norm_w.shape == (width,), "norm_w: [width]")
    state = shift_w = step = None
    if shift is not None:
        state, shift_w, step = shift
        require_cuda(state, shift_w)
        _check(reduce and norm_w is not None, "a shift needs the normed result")
        _check(state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == width
               and state.is_contiguous(), "state: contiguous fp32 [slots, width]")
        _check(shift_w.shape == (width,) and step.sequences == tokens,
               "shift_w: [width]; a shift inside the step needs one token a sequence")
    code = _constants(mix, out_w, in_w, norm_w, shift_w)
    out = None
    if reduce:
        if norm_w is None:
            out_dtype = torch.float32
        out = torch.empty((tokens, width), dtype=out_dtype, device=xs.device)
    call("sakv_streams_step", ptr(xs), xs.stride(0), streams, tokens, width, ptr(y), ptr(mix),
         ptr(out_w), int(reduce), ptr(in_w), ptr(norm_w), code, float(eps), ptr(out),
         dtype_code(out.dtype) if out is not None else 0, ptr(state), ptr(shift_w),
         ptr(step.token_seq) if step is not None else None,
         ptr(step.slots) if step is not None else None, int(keep_state))
    return out


def streams_spread(xs: torch.Tensor) -> torch.Tensor:
    """Every stream of `xs` (fp32 [streams, T, width]) becomes a copy of the first."""
    require_cuda(xs)
    _check(xs.dtype == torch.float32 and xs.dim() == 3 and xs[0].is_contiguous(),
           "xs: fp32 [streams, T, width] with contiguous streams")
    call("sakv_streams_spread", ptr(xs), xs.stride(0), xs.shape[0], xs[0].numel())
    return xs


def token_shift(h: torch.Tensor, state: torch.Tensor, shift: torch.Tensor, step,
                out_dtype: torch.dtype, keep_state: bool = True) -> torch.Tensor:
    """`h + (h_prev - h) * shift` for fp32 `h` [T, width], with `h_prev` the row of the token
    before in the same sequence; a sequence's first row of this step takes it from
    `state[slot]` (fp32 [slots, width]), which then receives the sequence's last row."""
    require_cuda(h, state, shift)
    tokens, width = h.shape
    _check(h.dtype == torch.float32 and h.is_contiguous(), "h: contiguous fp32 [T, width]")
    _check(state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == width
           and state.is_contiguous(), "state: contiguous fp32 [slots, width]")
    _check(shift.shape == (width,) and shift.is_contiguous(), "shift: [width]")
    out = torch.empty((tokens, width), dtype=out_dtype, device=h.device)
    call("sakv_token_shift", ptr(h), ptr(state), ptr(shift), dtype_code(shift.dtype),
         ptr(step.token_seq), ptr(step.cu_seqlens), ptr(step.slots), ptr(out),
         dtype_code(out_dtype), tokens, width, int(keep_state))
    return out
