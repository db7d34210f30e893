"""CPU variants of the package's two step executors, for checking emitted programs without a GPU.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

``hap_b200.spmd.LockstepWorld`` / ``ProcessWorker`` run an fx program with the package's CUDA
kernels and have no host path.  The subclasses here keep their control flow (``worker.py:58-83``:
zero_grad, forward, summed partial losses, backward, clip, Adam) and swap in the reference's own
host-side pair for the step tail - ``torch.nn.utils.clip_grad_norm_(params, 0.5)`` over the local
shards (``worker.py:74``) and ``torch.optim.Adam`` (``worker.py:47, 76``) - and accept collective
nodes bound to ``oracle.gloo_port`` next to ``collectives``.
"""
from __future__ import annotations

import torch

from hap_b200.spmd import LockstepWorld, ProcessWorker


class CpuLockstepWorld(LockstepWorld):
    collective_modules = ("collectives", "gloo_port")

    def _make_optimizer(self, params, lr, clip):
        return torch.optim.Adam(params, lr=lr)

    def _optimizer_step(self, module, optimizer) -> None:
        torch.nn.utils.clip_grad_norm_(module.parameters(), self.clip)
        optimizer.step()

    def _new_iteration(self) -> None:
        pass            # torch's CPU generator advances by itself


class CpuProcessWorker(ProcessWorker):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.uses_dropout = False       # torch's CPU dropout keeps its own generator state

    def _make_optimizer(self, params, lr, clip):
        return torch.optim.Adam(params, lr=lr)

    def _optimizer_step(self) -> None:
        torch.nn.utils.clip_grad_norm_(self.module.parameters(), self.clip)
        self.optimizer.step()
