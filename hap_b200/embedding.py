"""``torch.nn.functional.embedding`` whose backward runs on this package's kernel.

The programs look tokens up with ``F.embedding(tokens, weight)`` (``models.py:66-71``).  The forward pass is
torch's row gather; the gradient of the table - ``dweight[v] = sum of grad rows at the positions holding v`` -
comes from one sort-free kernel that adds the rows in ascending order of position (bit-reproducible, no
atomics) instead of torch's radix sort + segmented reduction.  Calls the kernel does not cover (a padding index,
``max_norm``, ``scale_grad_by_freq``, ``sparse``, other dtypes, rows that are not a multiple of 8 wide, CPU tensors)
go to torch unchanged.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _native as N

_DTYPES = {torch.float32: N.F32, torch.bfloat16: N.BF16}
_MAX_POSITIONS = 1 << 16      # the kernel compares every position with every other one


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, indices, weight):
        ctx.save_for_backward(indices)
        ctx.table = (weight.shape[0], weight.shape[1], weight.dtype)
        return F.embedding(indices, weight)

    @staticmethod
    def backward(ctx, grad):
        (indices,) = ctx.saved_tensors
        V, E, dtype = ctx.table
        idx = indices.reshape(-1).contiguous()
        g = grad.reshape(-1, E).contiguous()
        dweight = torch.empty((V, E), dtype=dtype, device=g.device)
        with torch.cuda.device(g.device):
            N.check(N.lib.hapx_embedding_backward(dweight.data_ptr(), g.data_ptr(), idx.data_ptr(), _DTYPES[dtype], idx.numel(), V, E,
                                                  torch.cuda.current_stream().cuda_stream))
        return None, dweight


def embedding(input: torch.Tensor, weight: torch.Tensor, padding_idx=None, max_norm=None, norm_type: float = 2.0,
              scale_grad_by_freq: bool = False, sparse: bool = False) -> torch.Tensor:
    covered = (weight.is_cuda and input.is_cuda and input.dtype == torch.int64 and weight.dim() == 2 and weight.dtype in _DTYPES
               and weight.shape[1] % 8 == 0 and 8 <= weight.shape[1] <= 2048 and padding_idx is None and max_norm is None
               and not scale_grad_by_freq and not sparse and input.numel() <= _MAX_POSITIONS and weight.requires_grad)
    if not covered:
        return F.embedding(input, weight, padding_idx, max_norm, norm_type, scale_grad_by_freq, sparse)
    return _Embedding.apply(input, weight)
