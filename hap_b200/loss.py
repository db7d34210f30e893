"""``log_softmax`` + ``nll_loss(reduction='sum')`` as one GPU pass in each direction.

The planner emits the two ops separately (``hap.rs:1808, 1858``; the models end in
``torch.log_softmax`` + ``NLLLoss(reduction='sum')``, ``models.py:116-117``); on bf16 logits that
moves a float copy of the logits, the log-probabilities and their gradients through HBM.  This
function reads the logits once per direction and keeps one float per row.
"""
from __future__ import annotations

import torch

from . import _native as N

_DTYPES = {torch.float32: N.F32, torch.bfloat16: N.BF16}


class _NllLogSoftmaxSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        if logits.dtype not in _DTYPES:
            raise TypeError(f"nll_log_softmax_sum: unsupported dtype {logits.dtype}")
        if not logits.is_cuda:
            raise ValueError("nll_log_softmax_sum runs on CUDA tensors only (there is no CPU path)")
        V = logits.shape[-1]
        x = logits.reshape(-1, V)
        if x.stride(-1) != 1 or (x.shape[0] > 1 and x.stride(0) < V):
            x = x.contiguous()
        t = targets.reshape(-1)
        if t.dtype != torch.int64 or not t.is_contiguous():
            t = t.to(torch.int64).contiguous()
        if t.numel() != x.shape[0]:
            raise ValueError("nll_log_softmax_sum: one target per row of logits expected")
        rows = x.shape[0]
        row_loss = torch.empty(rows, dtype=torch.float32, device=x.device)
        row_lse = torch.empty(rows, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            N.check(N.lib.hapx_nll_logsoftmax_forward(x.data_ptr(), t.data_ptr(), row_loss.data_ptr(), row_lse.data_ptr(),
                                                      _DTYPES[x.dtype], rows, V, x.stride(0) if rows > 1 else V,
                                                      torch.cuda.current_stream().cuda_stream))
        ctx.save_for_backward(x, t, row_lse)
        ctx.shape = logits.shape
        return row_loss.sum()

    @staticmethod
    def backward(ctx, grad_out):
        x, t, row_lse = ctx.saved_tensors
        rows, V = x.shape
        grad = torch.empty((rows, V), dtype=x.dtype, device=x.device)
        go = grad_out.to(torch.float32).contiguous()
        with torch.cuda.device(x.device):
            N.check(N.lib.hapx_nll_logsoftmax_backward(x.data_ptr(), t.data_ptr(), row_lse.data_ptr(), go.data_ptr(), grad.data_ptr(),
                                                       _DTYPES[x.dtype], rows, V, x.stride(0) if rows > 1 else V, V,
                                                       torch.cuda.current_stream().cuda_stream))
        return grad.view(ctx.shape), None


def nll_log_softmax_sum(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """``F.nll_loss(F.log_softmax(logits.float(), -1).reshape(-1, V), targets.reshape(-1), reduction='sum')``
    for float32 or bfloat16 ``logits`` of shape (..., V) and integer ``targets`` of shape (...).
    Returns a float32 scalar; the gradient has the logits' dtype."""
    return _NllLogSoftmaxSum.apply(logits, targets)
