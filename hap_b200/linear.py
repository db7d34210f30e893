"""``F.linear`` on ratio-sharded tensors, through the C ABI into the tcgen05 GEMM kernels.

Stands in for the ``torch.nn.functional.linear`` nodes of the synthesized program
(``hap.rs:1030-1037``, sharding variants ``hap.rs:2787-2816``): same signature, same autograd
results (``dx = g W``, ``dW = g^T x``, ``db = sum g``).  bfloat16 operands run on the tensor cores
with fp32 accumulation; float32 operands (the 1e-5 parity configuration) run an fp32 FFMA kernel.
There is no fallback to cuBLAS: unsupported inputs raise.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _native as N
from .comm import _on_device, _stream

_EPILOGUES = {"none": 0, "relu": 1, "gelu": 2, "sigmoid": 3}


def _check(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what}: hap_b200 has no CPU path; tensor is on {t.device}")
    if t.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"{what}: operands must be bfloat16 or float32, got {t.dtype}")


def _same(ref: torch.Tensor, *others) -> None:
    for t in others:
        if t is not None and t.dtype != ref.dtype:
            raise TypeError(f"linear: mixed operand dtypes {ref.dtype} and {t.dtype}")


def _default_out(t: torch.Tensor, out_dtype):
    return out_dtype if out_dtype is not None else t.dtype


def _out_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return N.BF16
    if dtype == torch.float32:
        return N.F32
    raise TypeError(f"linear: output dtype must be bfloat16 or float32, got {dtype}")


def linear_forward(x2: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], epilogue: str = "none",
                   out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y[m,n] = act(x2[m,k] @ w[n,k]^T + b[n]) for contiguous 2-D operands (bf16 or fp32)."""
    _check(x2, "linear"), _check(w, "linear"), _same(x2, w, b)
    out_dtype = _default_out(x2, out_dtype)
    m, k = x2.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError(f"linear: input features {k} != weight in_features {w.shape[1]}")
    if b is not None:
        _check(b, "linear")
        if b.numel() != n:
            raise ValueError("linear: bias size does not match out_features")
    if x2.dtype == torch.bfloat16 and k % 8:
        raise ValueError(f"linear: bfloat16 in_features must be a multiple of 8 (got {k})")
    y = torch.empty((m, n), dtype=out_dtype, device=x2.device)
    with _on_device(x2.device):
        N.check(N.lib.hapx_linear_forward(y.data_ptr(), x2.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
                                          _out_code(x2.dtype), _out_code(out_dtype), m, n, k, _EPILOGUES[epilogue],
                                          _stream(x2.device)))
    return y


def _pad_dim(t: torch.Tensor, dim: int, to: int) -> torch.Tensor:
    """Zero-extend ``t`` on ``dim`` to extent ``to`` with the package's own re-sharding kernel
    (the backward of dynamic_slice writes a shard into a zeroed larger tensor)."""
    from .comm import dynamic_slice_backward
    return dynamic_slice_backward(t, dim, [t.shape[dim], to - t.shape[dim]], 0)


def _round8(n: int) -> int:
    return (n + 7) // 8 * 8


def linear_dgrad(g2: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    _check(g2, "linear backward"), _check(w, "linear backward"), _same(g2, w)
    out_dtype = _default_out(g2, out_dtype)
    m, n = g2.shape
    k = w.shape[1]
    if g2.dtype == torch.bfloat16 and n % 8 and k % 8 == 0:
        # a column-parallel shard whose width is not a multiple of 8 (e.g. 2458 of 4096): the tensor
        # maps need 16-byte row pitches, so contract over a zero-extended copy of g and w
        n8 = _round8(n)
        return linear_dgrad(_pad_dim(g2, 1, n8), _pad_dim(w, 0, n8), out_dtype)
    if g2.dtype == torch.bfloat16 and (n % 8 or k % 8):
        raise ValueError(f"linear backward: bfloat16 features must be multiples of 8 (got n={n}, k={k})")
    dx = torch.empty((m, k), dtype=out_dtype, device=g2.device)
    with _on_device(g2.device):
        N.check(N.lib.hapx_linear_dgrad(dx.data_ptr(), g2.data_ptr(), w.data_ptr(), _out_code(g2.dtype), _out_code(out_dtype),
                                        m, n, k, _stream(g2.device)))
    return dx


def linear_wgrad(g2: torch.Tensor, x2: torch.Tensor, need_weight: bool = True, need_bias: bool = True,
                 out_dtype: Optional[torch.dtype] = None):
    _check(g2, "linear backward"), _check(x2, "linear backward"), _same(g2, x2)
    out_dtype = _default_out(g2, out_dtype)
    m, n = g2.shape
    k = x2.shape[1]
    if g2.dtype == torch.bfloat16 and n % 8 and k % 8 == 0:
        # see linear_dgrad: compute the gradient of the zero-extended shard, then cut the extension off
        from .comm import dynamic_slice
        n8 = _round8(n)
        dw8, db8 = linear_wgrad(_pad_dim(g2, 1, n8), x2, need_weight, need_bias, out_dtype)
        cut = lambda t: dynamic_slice(t, 0, [n, n8 - n], 0) if t is not None else None
        return cut(dw8), cut(db8)
    if g2.dtype == torch.bfloat16 and (n % 8 or k % 8):
        raise ValueError(f"linear backward: bfloat16 features must be multiples of 8 (got n={n}, k={k})")
    dw = torch.empty((n, k), dtype=out_dtype, device=g2.device) if need_weight else None
    db = torch.empty((n,), dtype=out_dtype, device=g2.device) if need_bias else None
    with _on_device(g2.device):
        N.check(N.lib.hapx_linear_wgrad(dw.data_ptr() if need_weight else None, db.data_ptr() if need_bias else None,
                                        g2.data_ptr(), x2.data_ptr(), _out_code(g2.dtype), _out_code(out_dtype), m, n, k,
                                        _stream(g2.device)))
    return dw, db


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        wc = w.contiguous()
        ctx.save_for_backward(x2, wc)
        ctx.has_bias = b is not None
        ctx.x_shape = x.shape
        y = linear_forward(x2, wc, b.contiguous() if b is not None else None)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, g):
        x2, w = ctx.saved_tensors
        g2 = g.reshape(-1, g.shape[-1]).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = linear_dgrad(g2, w).view(ctx.x_shape)
        need_w, need_b = ctx.needs_input_grad[1], ctx.has_bias and ctx.needs_input_grad[2]
        if need_w or need_b:
            dw, db = linear_wgrad(g2, x2, need_w, need_b)
        return dx, dw, db


def linear(input: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Drop-in for ``torch.nn.functional.linear`` on CUDA bfloat16 or float32 tensors."""
    return _Linear.apply(input, weight, bias)


def gemm_status() -> None:
    """Synchronise and raise if a GEMM kernel reported a barrier wait that ran out."""
    N.check(N.lib.hapx_gemm_status())
