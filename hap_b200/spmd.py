"""Run a synthesized SPMD program: the training step of the reference's ``worker.py``.

Two executors for the same ``torch.fx`` programs:

* :class:`ProcessWorker` - one rank per process (``worker.py:44, 58-83``): the program is an
  ordinary ``torch.fx.GraphModule`` whose collective nodes call :mod:`hap_b200.collectives`.
* :class:`LockstepWorld` - all ``world`` ranks of the program inside one process on one device.
  The ranks' graphs are walked node by node in lockstep; at a collective node the inputs of
  all ranks go to the list-based backend (:class:`hap_b200.LocalCollectives`, i.e. one
  cooperative kernel over all virtual ranks), every other node runs per rank.  This is how the
  whole step is exercised on a single GPU.

Both follow the reference's step: ``zero_grad`` -> forward -> partial losses summed
(``dist.reduce`` at ``worker.py:63-64``) -> backward -> ``clip_grad_norm_(params, 0.5)`` over the
LOCAL shards only (``worker.py:74``) -> Adam (``worker.py:47, 76``).
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import torch
from torch.fx.node import map_arg

from . import dropout as _dropout
from .collectives import NAMES as _COLLECTIVE_NAMES


def _is_collective(target, modules=("collectives",)) -> bool:
    module = (getattr(target, "__module__", "") or "").split(".")[-1]
    return getattr(target, "__name__", None) in _COLLECTIVE_NAMES and module in modules


def _program_has_dropout(module) -> bool:
    """True when the fx program holds a dropout node or an attention node with dropout_p > 0."""
    for n in getattr(module, "graph", torch.fx.Graph()).nodes:
        if n.op != "call_function":
            continue
        name = getattr(n.target, "__name__", "")
        if name == "dropout" or (name == "multi_head_attention_forward" and float(n.kwargs.get("dropout_p", 0.0) or 0.0) > 0.0):
            return True
        if name in ("dropout_add", "act_dropout") and float(n.args[2]) > 0.0:
            return True
    return False


def _fused_step_tail(params, lr, clip):
    """clip by the local-shard norm + Adam as multi-tensor kernels (``worker.py:74, 76``); GPU only."""
    from .optim import ClipAdam
    if not params or not all(p.is_cuda and p.dtype in (torch.float32, torch.bfloat16) for p in params):
        raise RuntimeError("hap_b200.spmd: parameters must be float32 / bfloat16 CUDA tensors (there is no CPU path)")
    return ClipAdam(params, lr=lr, max_norm=clip)


class LockstepWorld:
    collective_modules = ("collectives",)      # modules whose eight functions are collective nodes

    def __init__(self, modules: Sequence[torch.fx.GraphModule], backend, lr: float = 5e-4, clip: float = 0.5):
        self.modules = list(modules)
        self.world = len(self.modules)
        self.backend = backend
        self.clip = clip
        self.optimizers = [self._make_optimizer(list(m.parameters()), lr, clip) for m in self.modules]
        self._nodes = [list(m.graph.nodes) for m in self.modules]
        if len({len(n) for n in self._nodes}) != 1:
            raise ValueError("SPMD ranks must run the same node sequence")

    def _make_optimizer(self, params, lr, clip):
        return _fused_step_tail(params, lr, clip)

    def _optimizer_step(self, module, optimizer) -> None:
        optimizer.step()       # the fused tail clips by the local-shard norm itself

    def _new_iteration(self) -> None:
        if any(_program_has_dropout(m) for m in self.modules):
            _dropout.advance()

    def forward(self, inputs_per_rank: Sequence[Sequence[torch.Tensor]]) -> List[torch.Tensor]:
        envs = [dict() for _ in range(self.world)]
        feeds = [iter(inp) for inp in inputs_per_rank]
        results = [None] * self.world
        load = lambda r: (lambda n: envs[r][n])
        for step in zip(*self._nodes):
            n0 = step[0]
            if n0.op == "placeholder":
                for r, n in enumerate(step):
                    envs[r][n] = next(feeds[r])
            elif n0.op == "get_attr":
                for r, n in enumerate(step):
                    obj = self.modules[r]
                    for part in n.target.split("."):
                        obj = getattr(obj, part)
                    envs[r][n] = obj
            elif n0.op == "call_function" and _is_collective(n0.target, self.collective_modules):
                name = n0.target.__name__
                per_rank = [map_arg(n.args, load(r)) for r, n in enumerate(step)]
                tensors = [a[0] for a in per_rank]
                if name in ("all_reduce", "replicate"):
                    outs = getattr(self.backend, name)(tensors)
                elif name == "all_to_all":
                    outs = self.backend.all_to_all(tensors, *per_rank[0][1:5])
                else:  # (tensor, dim, sharding_lengths, rank)
                    outs = getattr(self.backend, name)(tensors, per_rank[0][1], per_rank[0][2])
                for r, n in enumerate(step):
                    envs[r][n] = outs[r]
            elif n0.op == "call_function":
                for r, n in enumerate(step):
                    envs[r][n] = n.target(*map_arg(n.args, load(r)), **map_arg(n.kwargs, load(r)))
            elif n0.op == "call_method":
                for r, n in enumerate(step):
                    args = map_arg(n.args, load(r))
                    envs[r][n] = getattr(args[0], n.target)(*args[1:], **map_arg(n.kwargs, load(r)))
            elif n0.op == "output":
                for r, n in enumerate(step):
                    results[r] = map_arg(n.args[0], load(r))
            else:
                raise NotImplementedError(n0.op)
        return results

    def step(self, inputs_per_rank) -> float:
        """One training iteration for all ranks; returns the global loss (sum of the partial losses)."""
        self._new_iteration()
        for opt in self.optimizers:
            opt.zero_grad()
        losses = self.forward(inputs_per_rank)
        total = torch.stack([l.detach() for l in losses]).sum()
        torch.stack(losses).sum().backward()
        for m, opt in zip(self.modules, self.optimizers):
            self._optimizer_step(m, opt)
        return total


class ProcessWorker:
    """One rank of the program in its own process (``worker.py:44-83``).

    With ``comm`` given, the gradients of all parameters that enter the program through
    ``collectives.replicate`` are reduced by ONE in-place all_reduce over a flat buffer that lives
    in the peer-visible heap (the parameters' ``.grad`` are views of it, so autograd accumulates
    straight into it and nothing is staged), instead of one all_reduce per parameter as in the
    reference.  The sum each parameter receives is the same.
    """

    def __init__(self, module: torch.fx.GraphModule, lr: float = 5e-4, clip: float = 0.5,
                 reduce_loss: Callable[[torch.Tensor], torch.Tensor] = None, comm=None):
        self.module = module
        self.clip = clip
        self.lr = lr
        self.reduce_loss = reduce_loss
        self.comm = comm
        if comm is not None and comm.world > 1:
            self._move_gathered_parameters_into_heap()
        # clip by the local-shard norm + Adam as multi-tensor kernels without a host round trip
        self.optimizer = self._make_optimizer(list(module.parameters()), lr, clip)
        self.uses_dropout = _program_has_dropout(module)
        self._buckets = []          # (flat tensor in the heap, [parameters])
        if comm is not None and comm.world > 1:       # a world of one reduces nothing: gradients stay where autograd leaves them
            self._build_buckets()

    def _make_optimizer(self, params, lr, clip):
        return _fused_step_tail(params, lr, clip)

    def _optimizer_step(self) -> None:
        self.optimizer.step()

    def _join_side_stream(self) -> None:
        """Gradients of parameters whose gather ran on the communicator's side stream are produced there
        (autograd runs a backward node on its forward's stream): the step tail waits for that stream."""
        from . import collectives
        comm = self.comm if self.comm is not None else (collectives.get_default_comm() if collectives.has_default_comm() else None)
        if comm is not None and comm._side_stream is not None:
            torch.cuda.current_stream(comm.device).wait_stream(comm._side_stream)

    def _move_gathered_parameters_into_heap(self) -> None:
        """Parameters that the program all-gathers (ZeRO-style shards, ``hap.rs:2527-2555``) are re-homed in
        the peer-visible heap, so the gather kernels read them in place on every step instead of copying
        them into the staging area first."""
        names = []
        for n in self.module.graph.nodes:
            if n.op == "call_function" and getattr(n.target, "__name__", "") in ("all_gather", "all_gather_by_group_call", "all_gather_start") \
                    and isinstance(n.args[0], torch.fx.Node) and n.args[0].op == "get_attr":
                names.append(n.args[0].target)
        params = dict(self.module.named_parameters())
        for name in dict.fromkeys(names):
            p = params.get(name)
            if p is None or not p.is_cuda:
                continue
            try:
                home = self.comm.symm_empty(tuple(p.shape), p.dtype)
            except MemoryError:
                return                  # the heap is full: the remaining parameters are staged as before
            home.copy_(p.data)
            p.data = home

    def _build_buckets(self) -> None:
        names = [n.args[0].target for n in self.module.graph.nodes
                 if n.op == "call_function" and getattr(n.target, "__name__", "") == "replicate"
                 and isinstance(n.args[0], torch.fx.Node) and n.args[0].op == "get_attr"]
        params = dict(self.module.named_parameters())
        by_dtype = {}
        for name in dict.fromkeys(names):
            p = params[name]
            if p.requires_grad:
                by_dtype.setdefault(p.dtype, []).append(p)
        for dtype, ps in by_dtype.items():
            total = sum((p.numel() + 7) // 8 * 8 for p in ps)
            flat = self.comm.symm_empty((total,), dtype)
            flat.zero_()                  # the gaps between parameters stay zero: only parameter regions are ever written
            off, views = 0, []
            for p in ps:
                views.append(flat[off:off + p.numel()].view_as(p))
                off += (p.numel() + 7) // 8 * 8
            self._buckets.append((flat, ps, views))

    def zero_grad(self) -> None:
        # gradients are left where autograd puts them (no accumulation kernels into preset buffers); the replicated
        # parameters' gradients are packed into their bucket after the backward pass, see _fill_buckets
        for p in self.module.parameters():
            p.grad = None

    def _fill_buckets(self) -> None:
        """Copy the replicated parameters' gradients into their flat, peer-visible buckets (one multi-tensor copy per
        bucket instead of one accumulation kernel per parameter) and make the bucket slices the gradients the
        optimizer reads: the all_reduce that follows works in place on the bucket."""
        for flat, ps, views in self._buckets:
            dst = [v for p, v in zip(ps, views) if p.grad is not None]
            src = [p.grad for p in ps if p.grad is not None]
            if dst:
                torch._foreach_copy_(dst, src)
            for p, v in zip(ps, views):
                if p.grad is None:
                    v.zero_()             # a parameter the program did not use
                p.grad = v

    def capture(self, *example_inputs, warmup: int = 3):
        """Record one whole iteration (zero_grad ... optimizer step) into a CUDA graph and return a
        callable ``replay(*inputs) -> total loss`` that copies the inputs into the graph's static
        buffers and launches the graph: the per-node Python dispatch of the eager step (the
        reference's hot loop (i), ``worker.py:58-83``) disappears.  The flag words of the
        collectives carry call numbers that are baked into the graph, so an iteration must hold at
        least two collectives of this library (then no flag of one replay can satisfy a wait of the
        next; checked here) and all ranks must replay the same number of times."""
        from . import _native as N
        from . import collectives
        comm = self.comm if self.comm is not None else (collectives.get_default_comm() if collectives.has_default_comm() else None)
        static_in = [t.clone() for t in example_inputs]
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(warmup):
                    self.step(*static_in)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            if comm is not None:
                # calls on different streams stay ordered by an event inside the capture; forget the event of the
                # eager calls so far, which must not be waited on from a capturing stream
                comm.set_stream_ordering(True)
            graph = torch.cuda.CUDAGraph()
            before = N.lib.hapx_launch_count()
            calls_before = comm.calls_issued() if comm is not None else 0
            with torch.cuda.graph(graph):
                static_out = self.step(*static_in)
            calls = (comm.calls_issued() - calls_before) if comm is not None else 0
        finally:
            if comm is not None:
                comm.set_stream_ordering(True)      # and forget the captured event: eager calls must not wait on it
        if comm is not None and comm.world > 1 and calls < 2:
            raise RuntimeError("ProcessWorker.capture: an iteration with fewer than two collectives cannot be replayed safely "
                               "(its flag words would repeat from one replay to the next)")
        self._graph = graph
        self.captured_launches = int(N.lib.hapx_launch_count() - before)    # kernels of this library in one replay

        def replay(*inputs):
            if comm is not None:
                comm.poll()
            for dst, src in zip(static_in, inputs):
                dst.copy_(src, non_blocking=True)
            graph.replay()
            return static_out

        return replay

    def step(self, *inputs) -> torch.Tensor:
        from . import collectives
        if self.comm is not None:
            self.comm.poll()        # a collective of an earlier step that gave up on a peer raises here
        if self.uses_dropout:
            _dropout.advance()      # new masks for this iteration (a kernel: also on every graph replay)
        self.zero_grad()
        loss = self.module(*inputs)
        total = loss.detach().clone()
        if self.reduce_loss is not None:
            total = self.reduce_loss(total)
        if self._buckets:
            collectives.defer_replicate(True)
            try:
                loss.backward()
            finally:
                collectives.defer_replicate(False)
            self._join_side_stream()
            self._fill_buckets()
            for flat, _, _ in self._buckets:
                self.comm.all_reduce([flat], inplace=True)
        else:
            loss.backward()
        self._join_side_stream()
        self._optimizer_step()
        return total
