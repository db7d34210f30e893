"""Step tail of the SPMD iteration on the GPU: clip by the local-shard gradient norm, then Adam.

Stands in for ``torch.nn.utils.clip_grad_norm_(dmodel.parameters(), 0.5)`` followed by
``optimizer.step()`` (``worker.py:74, 76`` of the reference, optimizer built at ``worker.py:47``)
with two kinds of multi-tensor kernels (``hapx_grad_sqnorm``, ``hapx_clip_adam_apply``) that never
synchronise with the host, so the whole iteration can be recorded into a CUDA graph.

Differences from the torch pair it replaces: the update is computed in fp32 and rounded once
(torch rounds after every elementwise op for bf16 parameters), and ``.grad`` is left unscaled.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable, Optional, Sequence

import torch

from . import _native as N

_DTYPES = {torch.float32: N.F32, torch.bfloat16: N.BF16}


class ClipAdam:
    """``torch.optim.Adam`` (no amsgrad) fused with gradient-norm clipping.

    ``max_norm=None`` disables clipping.  State tensors ``exp_avg[i]`` / ``exp_avg_sq[i]`` have the
    dtype of their parameter, as in torch.  All parameters must live on one CUDA device and be
    contiguous; float32 and bfloat16 parameters may be mixed (the norm covers both).
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-3, betas: Sequence[float] = (0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0, max_norm: Optional[float] = None):
        self.params = [p for p in params]
        if not self.params:
            raise ValueError("optimizer got an empty parameter list")
        dev = self.params[0].device
        if dev.type != "cuda":
            raise ValueError("ClipAdam runs on CUDA tensors only (there is no CPU path)")
        for p in self.params:
            if p.device != dev:
                raise ValueError("all parameters must be on the same device")
            if p.dtype not in _DTYPES:
                raise TypeError(f"unsupported parameter dtype {p.dtype}")
            if not p.is_contiguous():
                raise ValueError("parameters must be contiguous")
        self.lr, self.betas, self.eps, self.weight_decay = float(lr), (float(betas[0]), float(betas[1])), float(eps), float(weight_decay)
        self.max_norm = None if max_norm is None else float(max_norm)
        self.device = dev
        self.exp_avg = [torch.zeros_like(p, memory_format=torch.contiguous_format) for p in self.params]
        self.exp_avg_sq = [torch.zeros_like(p, memory_format=torch.contiguous_format) for p in self.params]
        self.state = torch.zeros(N.OPTIM_STATE_FLOATS, dtype=torch.float32, device=dev)
        # torch.optim-compatible view for code that reads the learning rate
        self.param_groups = [{"params": self.params, "lr": self.lr, "betas": self.betas, "eps": self.eps,
                              "weight_decay": self.weight_decay}]
        self._groups = {}
        self._fixed = {}
        for i, p in enumerate(self.params):
            self._groups.setdefault(_DTYPES[p.dtype], []).append(i)

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            if p.grad is None:
                continue
            if set_to_none:
                p.grad = None
            else:
                p.grad.detach_()
                p.grad.zero_()

    @property
    def grad_norm(self) -> torch.Tensor:
        """Device scalar: the gradient norm the last clipped step saw."""
        return self.state[1]

    @property
    def steps(self) -> torch.Tensor:
        return self.state[0]

    @torch.no_grad()
    def step(self) -> None:
        self.lr = float(self.param_groups[0]["lr"])
        stream = torch.cuda.current_stream(self.device).cuda_stream
        live = {}
        for code, idx in self._groups.items():
            keep = []
            for i in idx:
                g = self.params[i].grad
                if g is None:
                    continue
                if g.dtype != self.params[i].dtype or not g.is_contiguous():
                    g = g.to(self.params[i].dtype).contiguous()
                    self.params[i].grad = g
                keep.append(i)
            if keep:
                live[code] = keep
        if not live:
            return
        with torch.cuda.device(self.device):
            state = self.state.data_ptr()
            packed = {}
            for code, idx in live.items():
                key = (code, tuple(idx))
                where = [self.params[i].data_ptr() for i in idx]
                cached = self._fixed.get(key)
                if cached is None or cached[0] != where:       # parameter addresses normally stay put between steps
                    cached = self._fixed[key] = (where, (
                        N.ptr_array(where), N.ptr_array([self.exp_avg[i].data_ptr() for i in idx]),
                        N.ptr_array([self.exp_avg_sq[i].data_ptr() for i in idx]), N.i64_array([self.params[i].numel() for i in idx])))
                fixed = cached[1]
                grads = (C.c_void_p * len(idx))(*[self.params[i].grad.data_ptr() for i in idx])
                packed[code] = (len(idx), grads) + fixed
            if self.max_norm is not None:
                first = True
                for code, (n, grads, _, _, _, numel) in packed.items():
                    N.check(N.lib.hapx_grad_sqnorm(n, grads, numel, code, state, 1 if first else 0, stream))
                    first = False
            codes = list(packed)
            for k, code in enumerate(codes):
                n, grads, ps, ms, vs, numel = packed[code]
                N.check(N.lib.hapx_clip_adam_apply(
                    n, ps, grads, ms, vs, numel, code, self.lr, self.betas[0], self.betas[1], self.eps, self.weight_decay,
                    self.max_norm if self.max_norm is not None else 0.0, state, 1 if k == len(codes) - 1 else 0, stream))
