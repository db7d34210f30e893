"""``F.dropout`` for the synthesized programs, and the generator state behind every dropout of the
package (this one and the dropout on the attention probabilities).

The planner emits ``torch.nn.functional.dropout(input, p)`` (``hap.rs:1446-1464``); the reference trains
with ``dropout = 0.1`` (``config.py:33``).  :func:`dropout` has the same signature.  Masks come from a
counter-based generator: a pure function of (seed, iteration counter, call id, element index), so the
backward pass regenerates the mask instead of saving it.  Seed and iteration counter live in device
memory: :func:`manual_seed` sets them, :func:`advance` steps the counter with a one-thread kernel - the
step driver calls it once per iteration, and because it is a kernel, a step replayed from a CUDA graph
draws fresh masks on every replay.  Call ids number the dropout sites in program order; they restart at
:func:`advance`, so a replayed graph and the eager step it was recorded from use the same ids.
"""
from __future__ import annotations

import torch

from . import _native as N
from .comm import _on_device, _stream

_next_call_id = 0


def new_call_id() -> int:
    """Id for one dropout site of the current iteration (shared with the attention kernels)."""
    global _next_call_id
    _next_call_id += 1
    return _next_call_id


def manual_seed(seed: int, device=None) -> None:
    """Seed the device's generator and reset its iteration counter."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with _on_device(device):
        N.check(N.lib.hapx_rng_seed(int(seed) & 0xFFFFFFFFFFFFFFFF, _stream(device)))


def advance(device=None) -> None:
    """Step the iteration counter (device side) and restart the call ids (host side)."""
    global _next_call_id
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with _on_device(device):
        N.check(N.lib.hapx_rng_advance(_stream(device)))
    _next_call_id = 0


def _dense(*tensors):
    """The tensors as they are when they share one dense, non-overlapping layout (a permuted view of contiguous
    memory counts: an elementwise kernel can then walk the storage, and ``empty_like`` keeps the strides, so the
    layout of, say, expert-major activations survives the op); contiguous copies otherwise."""
    first = tensors[0]
    span = sum((n - 1) * st for n, st in zip(first.shape, first.stride())) + 1 if first.numel() else 0
    if span == first.numel() and all(t.stride() == first.stride() and t.shape == first.shape for t in tensors[1:]) \
            and torch.empty_like(first).stride() == first.stride():
        return tensors
    return tuple(t.contiguous() for t in tensors)


def _in_layout(t: torch.Tensor, strides) -> torch.Tensor:
    """``t`` with exactly these strides (a copy when it has others).  The mask of an element is looked up by
    its position in memory, so a backward pass must see the gradient in the layout the forward pass used."""
    if t.stride() == tuple(strides):
        return t
    return torch.empty_strided(t.shape, strides, dtype=t.dtype, device=t.device).copy_(t)


def _apply(x: torch.Tensor, p: float, call_id: int, out: torch.Tensor = None) -> torch.Tensor:
    (x,) = _dense(x)
    y = torch.empty_like(x) if out is None else out
    code = N.BF16 if x.dtype == torch.bfloat16 else N.F32
    with _on_device(x.device):
        N.check(N.lib.hapx_dropout(y.data_ptr(), x.data_ptr(), code, x.numel(), float(p), call_id, _stream(x.device)))
    return y


class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, call_id):
        y = _apply(x, p, call_id)
        ctx.meta = (p, call_id, y.stride())
        return y

    @staticmethod
    def backward(ctx, grad):
        p, call_id, strides = ctx.meta
        return _apply(_in_layout(grad, strides), p, call_id), None, None


def dropout(input: torch.Tensor, p: float = 0.5, training: bool = True, inplace: bool = False) -> torch.Tensor:
    """Drop-in for ``torch.nn.functional.dropout`` on CUDA bfloat16 / float32 tensors."""
    if not input.is_cuda:
        raise RuntimeError(f"dropout: hap_b200 has no CPU path; tensor is on {input.device}")
    if input.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"dropout: bfloat16 or float32 only, got {input.dtype}")
    if not 0.0 <= p < 1.0:
        raise ValueError(f"dropout: p must be in [0, 1), got {p}")
    if inplace:
        raise NotImplementedError("dropout: the planner never emits inplace=True (hap.rs:1450)")
    if not training or p == 0.0:
        return input
    return _Dropout.apply(input, float(p), new_call_id())


_ACTS = {"relu": 1, "gelu": 2}


class _DropoutAdd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, p, call_id):
        x, residual = _dense(x, residual)
        y = torch.empty_like(x)
        ctx.meta = (p, call_id, y.stride())
        with _on_device(x.device):
            N.check(N.lib.hapx_dropout_add(y.data_ptr(), x.data_ptr(), residual.data_ptr(), _code(x), x.numel(), float(p), call_id,
                                           _stream(x.device)))
        return y

    @staticmethod
    def backward(ctx, grad):
        p, call_id, strides = ctx.meta
        gx = _apply(_in_layout(grad, strides), p, call_id) if ctx.needs_input_grad[0] else None
        return gx, (grad if ctx.needs_input_grad[1] else None), None, None


class _ActDropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, act, p, call_id):
        (x,) = _dense(x)
        y = torch.empty_like(x)
        with _on_device(x.device):
            N.check(N.lib.hapx_act_dropout(y.data_ptr(), x.data_ptr(), _code(x), x.numel(), act, float(p), call_id, _stream(x.device)))
        ctx.save_for_backward(y if act == 1 else x)     # relu: the output tells active-and-kept; gelu: needs its input
        ctx.meta = (act, p, call_id)
        return y

    @staticmethod
    def backward(ctx, grad):
        (saved,) = ctx.saved_tensors
        act, p, call_id = ctx.meta
        grad = _in_layout(grad, saved.stride())       # the layout the forward pass walked
        dx = torch.empty_like(grad)
        with _on_device(grad.device):
            N.check(N.lib.hapx_act_dropout_backward(dx.data_ptr(), grad.data_ptr(), saved.data_ptr(), _code(grad), grad.numel(), act,
                                                    float(p), call_id, _stream(grad.device)))
        return dx, None, None, None


def _code(t: torch.Tensor) -> int:
    return N.BF16 if t.dtype == torch.bfloat16 else N.F32


def _check(t: torch.Tensor, what: str, p: float) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what}: hap_b200 has no CPU path; tensor is on {t.device}")
    if t.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"{what}: bfloat16 or float32 only, got {t.dtype}")
    if not 0.0 <= p < 1.0:
        raise ValueError(f"{what}: p must be in [0, 1), got {p}")


def dropout_add(x: torch.Tensor, residual: torch.Tensor, p: float, training: bool = True) -> torch.Tensor:
    """``residual + dropout(x, p)`` in one pass: the two residual connections of an encoder layer
    (``x + dropout1(sa(x))``, ``x + dropout2(ff(x))``)."""
    _check(x, "dropout_add", p)
    if residual.shape != x.shape or residual.dtype != x.dtype or residual.device != x.device:
        raise ValueError("dropout_add: x and residual must agree in shape, dtype and device")
    p = float(p) if training else 0.0
    return _DropoutAdd.apply(x, residual, p, new_call_id() if p > 0.0 else 0)


def act_dropout(x: torch.Tensor, act: str, p: float, training: bool = True) -> torch.Tensor:
    """``dropout(act(x), p)`` in one pass (``act``: ``"relu"`` or ``"gelu"``): the FFN's
    ``dropout(activation(linear1(x)))``.  With p == 0 it is the bare activation."""
    _check(x, "act_dropout", p)
    p = float(p) if training else 0.0
    return _ActDropout.apply(x, _ACTS[act], p, new_call_id() if p > 0.0 else 0)


def keep_mask(n: int, p: float, call_id: int, device=None) -> torch.Tensor:
    """The keep mask (uint8, n elements) that call ``call_id`` draws in the current iteration."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    mask = torch.empty(n, dtype=torch.uint8, device=device)
    with _on_device(device):
        N.check(N.lib.hapx_dropout_mask(mask.data_ptr(), n, float(p), call_id, _stream(device)))
    return mask
