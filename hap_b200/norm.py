"""``torch.nn.functional.layer_norm`` over the last dimension on this package's kernels.

Same call shape as the function the planner's programs name (``hap.rs:1637-1660``): the fx target
can be swapped without touching the arguments.  Rows of up to 2048 float32 / bfloat16 elements
(a multiple of 8) with an elementwise weight take the fused kernels (one read of ``x`` forward; one
read of ``x`` and ``dy`` backward, deterministic parameter gradients); any other call is handed to
torch's own CUDA implementation unchanged.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _native as N

_DTYPES = {torch.float32: N.F32, torch.bfloat16: N.BF16}


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        E = x.shape[-1]
        xc = x.contiguous()
        rows = xc.numel() // E
        y = torch.empty_like(xc)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        w = weight.contiguous()
        b = None if bias is None else bias.contiguous()
        with torch.cuda.device(x.device):
            N.check(N.lib.hapx_layer_norm_forward(xc.data_ptr(), w.data_ptr(), 0 if b is None else b.data_ptr(), y.data_ptr(),
                                                  mean.data_ptr(), rstd.data_ptr(), _DTYPES[x.dtype], rows, E, float(eps),
                                                  torch.cuda.current_stream().cuda_stream))
        ctx.save_for_backward(xc, w, mean, rstd)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, w, mean, rstd = ctx.saved_tensors
        E = xc.shape[-1]
        rows = xc.numel() // E
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        need_w, need_b = ctx.needs_input_grad[1], ctx.has_bias and ctx.needs_input_grad[2]
        dw = torch.empty_like(w) if need_w else None
        db = torch.empty_like(w) if need_b else None
        blocks = N.lib.hapx_layer_norm_backward_blocks(rows, E)
        partial = torch.empty(2 * E * blocks, dtype=torch.float32, device=xc.device)
        with torch.cuda.device(xc.device):
            N.check(N.lib.hapx_layer_norm_backward(xc.data_ptr(), dyc.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                                   dx.data_ptr(), 0 if dw is None else dw.data_ptr(), 0 if db is None else db.data_ptr(),
                                                   partial.data_ptr(), _DTYPES[xc.dtype], rows, E,
                                                   torch.cuda.current_stream().cuda_stream))
        return dx, dw, db, None


class _LayerNormFork(torch.autograd.Function):
    """(x, layer_norm(x)): the input handed through next to its normalised form, so that the gradient arriving
    through the residual connection and the gradient of the normalised branch meet in ONE backward kernel
    (``dx = layer_norm_backward(dy) + d_residual``) instead of in an addition kernel of autograd's."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        y = _LayerNorm.forward(ctx, x, weight, bias, eps)
        return x.view_as(x), y

    @staticmethod
    def backward(ctx, d_residual, dy):
        xc, w, mean, rstd = ctx.saved_tensors
        if dy is None:                       # the normalised branch took no part in the loss
            return d_residual, None, None, None
        E = xc.shape[-1]
        rows = xc.numel() // E
        dyc = dy.contiguous()
        add = None if d_residual is None else d_residual.contiguous()
        dx = torch.empty_like(xc)
        need_w, need_b = ctx.needs_input_grad[1], ctx.has_bias and ctx.needs_input_grad[2]
        dw = torch.empty_like(w) if need_w else None
        db = torch.empty_like(w) if need_b else None
        blocks = N.lib.hapx_layer_norm_backward_blocks(rows, E)
        partial = torch.empty(2 * E * blocks, dtype=torch.float32, device=xc.device)
        with torch.cuda.device(xc.device):
            N.check(N.lib.hapx_layer_norm_backward_add(xc.data_ptr(), dyc.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                                       0 if add is None else add.data_ptr(), dx.data_ptr(),
                                                       0 if dw is None else dw.data_ptr(), 0 if db is None else db.data_ptr(),
                                                       partial.data_ptr(), _DTYPES[xc.dtype], rows, E,
                                                       torch.cuda.current_stream().cuda_stream))
        return dx.view(ctx.x_shape), dw, db, None


def _fusable(input, shape, weight, bias) -> bool:
    E = input.shape[-1] if input.dim() else 0
    return (input.is_cuda and len(shape) == 1 and shape[0] == E and weight is not None and input.dtype in _DTYPES
            and weight.dtype == input.dtype and (bias is None or bias.dtype == input.dtype)
            and E % 8 == 0 and 8 <= E <= 2048 and input.numel() > 0)


def layer_norm(input: torch.Tensor, normalized_shape, weight=None, bias=None, eps: float = 1e-5) -> torch.Tensor:
    shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
    if not _fusable(input, shape, weight, bias):
        return F.layer_norm(input, shape, weight, bias, eps)
    return _LayerNorm.apply(input, weight, bias, eps)


def layer_norm_fork(input: torch.Tensor, normalized_shape, weight=None, bias=None, eps: float = 1e-5):
    """``(input, layer_norm(input, ...))`` for the pre-LN residual pattern ``x + f(layer_norm(x))``: use the first
    result where the program used ``x`` on the residual path.  Same values as :func:`layer_norm`; the backward pass
    adds the residual path's gradient inside the normalisation's backward kernel."""
    shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
    if not _fusable(input, shape, weight, bias) or not input.is_contiguous():
        return input, layer_norm(input, shape, weight, bias, eps)
    return _LayerNormFork.apply(input, weight, bias, eps)
