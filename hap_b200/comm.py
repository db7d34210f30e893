"""Communicators and the tensor-level operations on them (no autograd here).

A :class:`Comm` wraps one ``hapx_comm``:

* :func:`init_process_comm` - one process per GPU (what ``worker.py:14-18`` of the
  reference sets up with ``init_process_group('nccl')``): every rank allocates a
  peer-visible heap, the CUDA IPC handles travel through the already initialised
  ``torch.distributed`` group, every rank maps every peer's heap.
* :func:`local_comm` - ``world`` virtual ranks on one device in one process.  Every
  collective is then a single cooperative launch over all ranks' data; the kernels and
  the flag protocol are the ones the multi-GPU path runs.  Meant for single-GPU tests.

All methods take and return LISTS with one tensor per local rank (length 1 for a
process communicator).  PyTorch supplies device memory and the current stream; all
data movement and arithmetic happens in the library's kernels.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence

import torch

from . import _native as N

_DTYPES = {
    torch.float32: N.F32, torch.bfloat16: N.BF16, torch.float16: N.F16, torch.float64: N.F64,
    torch.int8: N.B8, torch.uint8: N.B8, torch.bool: N.B8, torch.int16: N.B16,
    torch.int32: N.B32, torch.int64: N.B64,
}
_REDUCIBLE = (torch.float32, torch.bfloat16, torch.float16)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"hap_b200: unsupported dtype {dtype}") from None


def _prod(xs) -> int:
    out = 1
    for x in xs:
        out *= int(x)
    return out


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptrs1(t: torch.Tensor):
    """Pointer array of one tensor (the one-rank-per-process case) without a list in between."""
    arr = (C.c_void_p * 1)()
    arr[0] = t.data_ptr()
    return arr


class _on_device:
    """``with torch.cuda.device(d)`` costs several microseconds per use; switch only when the
    tensor's device is not the current one (never, with one process per GPU)."""

    def __init__(self, device):
        self._ctx = None
        if device.index is not None and device.index != torch.cuda.current_device():
            self._ctx = torch.cuda.device(device)

    def __enter__(self):
        if self._ctx is not None:
            self._ctx.__enter__()

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)


class _RawDeviceMemory:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2, "strides": None,
        }


class Comm:
    def __init__(self, handle: int, device: torch.device):
        self._h = C.c_void_p(handle)
        self.device = device
        w, nl, fr = C.c_int(), C.c_int(), C.c_int()
        N.check(N.lib.hapx_comm_world(self._h, C.byref(w), C.byref(nl), C.byref(fr)))
        self.world, self.n_local, self.first_rank = w.value, nl.value, fr.value
        # A world of ONE rank: all_gather, reduce_scatter (unscaled), all_reduce (unscaled) and all_to_all are the
        # identity, so the tensor-level methods hand the input back instead of launching a copy.
        self._alone = self.world == 1
        self._heap_views: List[Optional[torch.Tensor]] = [None] * self.n_local
        self._heap_cursor = [0] * self.n_local
        self.debug_sync = os.environ.get("HAPX_DEBUG_SYNC", "0") == "1"
        self._side_stream: Optional[torch.cuda.Stream] = None

    # ---- lifecycle -------------------------------------------------------------------
    def destroy(self, group=None) -> None:
        """Release the communicator.  Ranks that are separate processes tear down in two phases -
        close the mappings of the peers' heaps, meet at a barrier, free the own heap - because a
        heap must not be freed while a peer still has it mapped.  The barrier runs on ``group`` (or
        the default ``torch.distributed`` group) when this is a multi-process communicator and
        ``torch.distributed`` is still initialised; call ``destroy`` on all ranks."""
        if not self._h:
            return
        self._heap_views = [None] * self.n_local
        if self.n_local == 1 and self.world > 1:
            import torch.distributed as dist
            N.check(N.lib.hapx_comm_close_peers(self._h))
            if dist.is_available() and dist.is_initialized():
                with torch.cuda.device(self.device):
                    dist.barrier(group=group)
        N.check(N.lib.hapx_comm_destroy(self._h))
        self._h = None

    def check(self) -> None:
        """Synchronise and raise if a kernel recorded an error (e.g. a peer that never arrived)."""
        N.check(N.lib.hapx_comm_check(self._h))

    def poll(self) -> None:
        """Raise if a kernel that has already run gave up waiting for a peer.  No synchronisation:
        one read of pinned host memory.  Every collective call makes the same test on entry."""
        N.check(N.lib.hapx_comm_poll(self._h))

    def calls_issued(self) -> int:
        n = C.c_int64()
        N.check(N.lib.hapx_comm_calls_issued(self._h, C.byref(n)))
        return n.value

    def set_timeout_ms(self, ms: int) -> None:
        N.check(N.lib.hapx_comm_set_timeout_ms(self._h, int(ms)))

    def set_stream_ordering(self, on: bool) -> None:
        N.check(N.lib.hapx_comm_set_stream_ordering(self._h, int(bool(on))))

    def side_stream(self) -> torch.cuda.Stream:
        """A second stream for collectives that should overlap with the current stream's work (calls on
        different streams are ordered against each other by the library with an event)."""
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(self.device)
        return self._side_stream

    def set_fused_all_reduce(self, mode) -> None:
        """Form of large all_reduces: False = two launches, True = one launch, ``"push"`` = one launch that writes the
        sums straight into the peers' outputs when all of them lie in the heap; None = the default (``"push"``
        between processes, two launches in the single-device emulation).  Same setting on every rank."""
        code = {None: -1, False: 0, True: 1, "push": 2}[mode]
        N.check(N.lib.hapx_comm_set_fused_all_reduce(self._h, code))

    def set_max_ctas(self, ctas: int) -> None:
        N.check(N.lib.hapx_comm_set_max_ctas(self._h, int(ctas)))

    def ranks(self) -> List[int]:
        return list(range(self.first_rank, self.first_rank + self.n_local))

    # ---- peer-visible tensors --------------------------------------------------------
    def _heap(self, i: int) -> torch.Tensor:
        if self._heap_views[i] is None:
            base, nbytes = C.c_void_p(), C.c_size_t()
            N.check(N.lib.hapx_comm_heap(self._h, i, C.byref(base), C.byref(nbytes)))
            self._heap_views[i] = torch.as_tensor(_RawDeviceMemory(base.value, nbytes.value), device=self.device)
        return self._heap_views[i]

    def symm_empty(self, shape, dtype=torch.float32, local_index: int = 0) -> torch.Tensor:
        """A tensor inside local rank ``local_index``'s peer-visible heap (bump allocation, 256-byte
        aligned, never freed individually; :meth:`symm_reset` releases everything).  Collectives
        read such inputs in place instead of staging them."""
        heap = self._heap(local_index)
        nbytes = _prod(shape) * torch.empty((), dtype=dtype).element_size()
        start = (self._heap_cursor[local_index] + 255) // 256 * 256
        if start + nbytes > heap.numel():
            raise MemoryError(f"hap_b200: heap exhausted ({start + nbytes} > {heap.numel()} bytes)")
        self._heap_cursor[local_index] = start + nbytes
        return heap[start:start + nbytes].view(dtype).view(*shape)

    def symm_reset(self) -> None:
        self._heap_cursor = [0] * self.n_local

    def get(self, peer: int, peer_tensor_like: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One-sided read of the peer's copy of a heap tensor: ``peer_tensor_like`` is THIS rank's
        tensor from :meth:`symm_empty`; ranks that allocate from their heaps in the same order hold
        their counterpart at the same offset, and that counterpart on ``peer`` is what is read.
        No handshake: order it against the peer's writes yourself (e.g. a barrier)."""
        heap = self._heap(0)
        off = peer_tensor_like.data_ptr() - heap.data_ptr()
        nbytes = peer_tensor_like.numel() * peer_tensor_like.element_size()
        if off < 0 or off + nbytes > heap.numel():
            raise ValueError("get: the tensor does not live in this communicator's heap")
        out = torch.empty_like(peer_tensor_like, memory_format=torch.contiguous_format) if out is None else out
        if not out.is_cuda or not out.is_contiguous():
            raise RuntimeError("get: the destination must be a contiguous CUDA tensor")
        N.check(N.lib.hapx_comm_get(self._h, int(peer), off, out.data_ptr(), nbytes, _stream(self.device)))
        return out

    # ---- helpers ---------------------------------------------------------------------------
    def _lists(self, tensors: Sequence[torch.Tensor], what: str) -> List[torch.Tensor]:
        if len(tensors) != self.n_local:
            raise ValueError(f"{what}: expected {self.n_local} tensor(s), one per local rank, got {len(tensors)}")
        out = []
        for t in tensors:
            if not t.is_cuda:
                raise RuntimeError(f"{what}: hap_b200 has no CPU path; tensor is on {t.device}")
            out.append(t.contiguous())
        return out

    def _lengths(self, lengths: Sequence[int], what: str) -> List[int]:
        lengths = [int(x) for x in lengths]
        if len(lengths) != self.world:
            raise ValueError(f"{what}: {len(lengths)} sharding lengths for world size {self.world}")
        return lengths

    def _after(self) -> None:
        if self.debug_sync:
            self.check()

    # ---- collectives ----------------------------------------------------------------------------
    def all_gather(self, shards: Sequence[torch.Tensor], dim: int, lengths: Sequence[int],
                   mode: int = N.MODE_PADDING, out: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
        shards = self._lists(shards, "all_gather")
        lengths = self._lengths(lengths, "all_gather")
        ref = shards[0]
        dim = dim % ref.dim()
        for i, (r, t) in enumerate(zip(self.ranks(), shards)):
            if t.shape[dim] != lengths[r]:
                raise ValueError(f"all_gather: rank {r} holds extent {t.shape[dim]} on dim {dim}, sharding length is {lengths[r]}")
            if t.dtype != ref.dtype or t.shape[:dim] != ref.shape[:dim] or t.shape[dim + 1:] != ref.shape[dim + 1:]:
                raise ValueError("all_gather: shards disagree in dtype or non-sharded extents")
        if self._alone and out is None:
            return shards                      # a world of one: the shard is the whole tensor
        full = list(ref.shape)
        full[dim] = sum(lengths)
        outs = list(out) if out is not None else [torch.empty(full, dtype=ref.dtype, device=t.device) for t in shards]
        one = self.n_local == 1
        N.check(N.lib.hapx_all_gather(self._h, _ptrs1(outs[0]) if one else N.ptr_array([o.data_ptr() for o in outs]),
                                      _ptrs1(shards[0]) if one else N.ptr_array([t.data_ptr() for t in shards]), dtype_code(ref.dtype),
                                      _prod(ref.shape[:dim]), _prod(ref.shape[dim + 1:]), N.i64_array(lengths),
                                      mode, _stream(self.device)))
        self._after()
        return outs

    def reduce_scatter(self, inputs: Sequence[torch.Tensor], dim: int, lengths: Sequence[int],
                       mode: int = N.MODE_PADDING, scale: float = 1.0,
                       out_dtype: Optional[torch.dtype] = None) -> List[torch.Tensor]:
        inputs = self._lists(inputs, "reduce_scatter")
        lengths = self._lengths(lengths, "reduce_scatter")
        ref = inputs[0]
        dim = dim % ref.dim()
        if ref.dtype not in _REDUCIBLE:
            raise TypeError(f"reduce_scatter: unsupported dtype {ref.dtype}")
        if ref.shape[dim] != sum(lengths):
            raise ValueError(f"reduce_scatter: extent {ref.shape[dim]} on dim {dim} != sum of sharding lengths {sum(lengths)}")
        for t in inputs:
            if t.shape != ref.shape or t.dtype != ref.dtype:
                raise ValueError("reduce_scatter: inputs disagree in shape or dtype")
        out_dtype = out_dtype or ref.dtype
        if self._alone and scale == 1.0 and out_dtype == ref.dtype:
            return inputs                      # a world of one: nothing to add, nothing to cut
        outs = []
        for r in self.ranks():
            shape = list(ref.shape)
            shape[dim] = lengths[r]
            outs.append(torch.empty(shape, dtype=out_dtype, device=ref.device))
        one = self.n_local == 1
        N.check(N.lib.hapx_reduce_scatter(self._h, _ptrs1(outs[0]) if one else N.ptr_array([o.data_ptr() for o in outs]),
                                          _ptrs1(inputs[0]) if one else N.ptr_array([t.data_ptr() for t in inputs]), dtype_code(ref.dtype),
                                          dtype_code(out_dtype), float(scale), _prod(ref.shape[:dim]),
                                          _prod(ref.shape[dim + 1:]), N.i64_array(lengths), mode, _stream(self.device)))
        self._after()
        return outs

    def all_reduce(self, inputs: Sequence[torch.Tensor], scale: float = 1.0, out_dtype: Optional[torch.dtype] = None,
                   inplace: bool = False, out: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
        inputs = self._lists(inputs, "all_reduce")
        ref = inputs[0]
        if ref.dtype not in _REDUCIBLE:
            raise TypeError(f"all_reduce: unsupported dtype {ref.dtype}")
        for t in inputs:
            if t.shape != ref.shape or t.dtype != ref.dtype:
                raise ValueError("all_reduce: inputs disagree in shape or dtype")
        out_dtype = out_dtype or ref.dtype
        if self._alone and scale == 1.0 and out_dtype == ref.dtype and out is None:
            return inputs
        if inplace:
            if out_dtype != ref.dtype:
                raise ValueError("all_reduce: in-place needs out_dtype == input dtype")
            outs = inputs
        elif out is not None:
            outs = self._lists(out, "all_reduce")
            for o, t in zip(outs, inputs):
                if o.shape != t.shape or o.dtype != out_dtype or not o.is_contiguous():
                    raise ValueError("all_reduce: out must be contiguous tensors of the inputs' shape and the output dtype")
        else:
            outs = [torch.empty(t.shape, dtype=out_dtype, device=t.device) for t in inputs]
        one = self.n_local == 1
        N.check(N.lib.hapx_all_reduce(self._h, _ptrs1(outs[0]) if one else N.ptr_array([o.data_ptr() for o in outs]),
                                      _ptrs1(inputs[0]) if one else N.ptr_array([t.data_ptr() for t in inputs]), dtype_code(ref.dtype),
                                      dtype_code(out_dtype), float(scale), ref.numel(), _stream(self.device)))
        self._after()
        return outs

    def all_to_all(self, inputs: Sequence[torch.Tensor], split_dim: int, cat_dim: int,
                   split_lengths: Sequence[int], cat_lengths: Sequence[int]) -> List[torch.Tensor]:
        split_lengths = self._lengths(split_lengths, "all_to_all")
        cat_lengths = self._lengths(cat_lengths, "all_to_all")
        nd = inputs[0].dim()
        split_dim, cat_dim = split_dim % nd, cat_dim % nd
        if split_dim == cat_dim:
            raise ValueError("all_to_all: split_dim and cat_dim must differ")
        if self._alone and len(inputs) == 1 and inputs[0].is_cuda and \
                inputs[0].shape[split_dim] == split_lengths[0] and inputs[0].shape[cat_dim] == cat_lengths[0]:
            return list(inputs)                # a world of one: the tensor as it is, whatever its memory layout
        inputs = self._lists(inputs, "all_to_all")
        ref = inputs[0]
        d1, d2 = min(split_dim, cat_dim), max(split_dim, cat_dim)
        outs = []
        for r, t in zip(self.ranks(), inputs):
            if t.shape[split_dim] != sum(split_lengths):
                raise ValueError(f"all_to_all: extent {t.shape[split_dim]} on split dim != sum of split lengths {sum(split_lengths)}")
            if t.shape[cat_dim] != cat_lengths[r]:
                raise ValueError(f"all_to_all: rank {r} holds extent {t.shape[cat_dim]} on cat dim, sharding length is {cat_lengths[r]}")
            shape = list(t.shape)
            shape[split_dim] = split_lengths[r]
            shape[cat_dim] = sum(cat_lengths)
            outs.append(torch.empty(shape, dtype=t.dtype, device=t.device))
        a, b, c = _prod(ref.shape[:d1]), _prod(ref.shape[d1 + 1:d2]), _prod(ref.shape[d2 + 1:])
        N.check(N.lib.hapx_all_to_all(self._h, N.ptr_array([o.data_ptr() for o in outs]),
                                      N.ptr_array([t.data_ptr() for t in inputs]), dtype_code(ref.dtype),
                                      a, b, c, 1 if split_dim < cat_dim else 0, N.i64_array(split_lengths),
                                      N.i64_array(cat_lengths), _stream(self.device)))
        self._after()
        return outs


# ---- purely local re-sharding (no communicator needed) ------------------------------------------
def dynamic_slice(tensor: torch.Tensor, dim: int, lengths: Sequence[int], rank: int) -> torch.Tensor:
    if not tensor.is_cuda:
        raise RuntimeError(f"dynamic_slice: hap_b200 has no CPU path; tensor is on {tensor.device}")
    t = tensor.contiguous()
    dim = dim % t.dim()
    lengths = [int(x) for x in lengths]
    if t.shape[dim] != sum(lengths):
        raise ValueError(f"dynamic_slice: extent {t.shape[dim]} on dim {dim} != sum of sharding lengths {sum(lengths)}")
    shape = list(t.shape)
    shape[dim] = lengths[rank]
    out = torch.empty(shape, dtype=t.dtype, device=t.device)
    with _on_device(t.device):
        N.check(N.lib.hapx_dynamic_slice(out.data_ptr(), t.data_ptr(), dtype_code(t.dtype), _prod(t.shape[:dim]),
                                         _prod(t.shape[dim + 1:]), N.i64_array(lengths), len(lengths), int(rank),
                                         _stream(t.device)))
    return out


def dynamic_slice_backward(grad: torch.Tensor, dim: int, lengths: Sequence[int], rank: int) -> torch.Tensor:
    g = grad.contiguous()
    dim = dim % g.dim()
    lengths = [int(x) for x in lengths]
    shape = list(g.shape)
    shape[dim] = sum(lengths)
    out = torch.empty(shape, dtype=g.dtype, device=g.device)
    with _on_device(g.device):
        N.check(N.lib.hapx_dynamic_slice_backward(out.data_ptr(), g.data_ptr(), dtype_code(g.dtype), _prod(g.shape[:dim]),
                                                  _prod(g.shape[dim + 1:]), N.i64_array(lengths), len(lengths), int(rank),
                                                  _stream(g.device)))
    return out


# ---- construction ---------------------------------------------------------------------------------
def _sizes(heap_bytes: Optional[int], stage_bytes: Optional[int]):
    stage = int(stage_bytes if stage_bytes is not None else os.environ.get("HAPX_STAGE_BYTES", 512 << 20))
    stage = (stage + 255) // 256 * 256
    heap = int(heap_bytes if heap_bytes is not None else os.environ.get("HAPX_HEAP_BYTES", 0)) or (stage + (64 << 20))
    heap = max(heap, stage + (1 << 20))
    return heap, stage


def local_comm(world: int, device=None, heap_bytes: Optional[int] = None, stage_bytes: Optional[int] = None) -> Comm:
    """``world`` virtual ranks on one device (single-GPU emulation of the multi-GPU path)."""
    if not torch.cuda.is_available():
        raise RuntimeError("hap_b200 needs a CUDA device (there is no CPU fallback)")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    heap, stage = _sizes(heap_bytes, stage_bytes)
    h = C.c_void_p()
    torch.cuda.init()
    N.check(N.lib.hapx_comm_create_local(C.byref(h), int(world), device.index or 0, heap, stage))
    return Comm(h.value, device)


def single_comm(device=None, heap_bytes: Optional[int] = None, stage_bytes: Optional[int] = None) -> Comm:
    """A one-rank-per-process communicator for a world of ONE process: no peers, no
    ``torch.distributed``.  Every collective degenerates to local kernels (the 1-GPU point of the
    scaling curve) while the program still runs through the same drop-in functions."""
    if not torch.cuda.is_available():
        raise RuntimeError("hap_b200 needs a CUDA device (there is no CPU fallback)")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    heap, stage = _sizes(heap_bytes, stage_bytes)
    torch.cuda.init()
    h = C.c_void_p()
    N.check(N.lib.hapx_comm_create(C.byref(h), 1, 0, device.index or 0, heap, stage))
    return Comm(h.value, device)


def init_process_comm(group=None, device=None, heap_bytes: Optional[int] = None,
                      stage_bytes: Optional[int] = None) -> Comm:
    """One rank per process.  ``torch.distributed`` must be initialised; it only carries the
    64-byte IPC handles and a barrier."""
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise RuntimeError("hap_b200 needs a CUDA device (there is no CPU fallback)")
    if not dist.is_initialized():
        raise RuntimeError("hap_b200: call torch.distributed.init_process_group first")
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    heap, stage = _sizes(heap_bytes, stage_bytes)
    torch.cuda.init()
    h = C.c_void_p()
    N.check(N.lib.hapx_comm_create(C.byref(h), world, rank, device.index or 0, heap, stage))
    mine = C.create_string_buffer(N.IPC_HANDLE_BYTES)
    N.check(N.lib.hapx_comm_ipc_handle(h, mine))
    handles = [None] * world
    with torch.cuda.device(device):
        dist.all_gather_object(handles, bytes(mine.raw), group=group)
        N.check(N.lib.hapx_comm_open_peers(h, b"".join(handles)))
        dist.barrier(group=group)  # nobody launches before every rank has mapped everyone
    return Comm(h.value, device)


def local_all_reduce_noalloc(inputs: Sequence[torch.Tensor], outputs: Sequence[torch.Tensor], scale: float = 1.0) -> None:
    """Sum ``inputs`` (one tensor per virtual rank, all on the current device) into every tensor of
    ``outputs`` without allocating anything: no communicator, no ``cudaMalloc``, no torch allocation.

    For callers that cannot obtain device memory at the moment the collective is due - the whole
    card already belongs to another allocator, or the calling thread must not take the device-wide
    synchronisation an allocation implies.  The caller provides inputs AND outputs (contiguous;
    ``outputs[r]`` may be ``inputs[r]``); all scratch is a fixed 16 MiB array inside the library,
    which limits the call to 8 ranks and roughly 460 000 float32 elements at 8 ranks (a larger call
    raises ``HapxError`` with code ``ERR_STAGING``).  The first call on a device should happen
    outside stream capture and while device memory is still available (the driver reserves the
    array when it first loads the library's code on that device).  Calls share the scratch: do not
    let two of them overlap on the GPU.  :func:`local_all_reduce_noalloc_status` reports a bounded
    wait that ran out inside the kernels.
    """
    if len(inputs) != len(outputs) or not inputs:
        raise ValueError("local_all_reduce_noalloc: need one output per input")
    ref = inputs[0]
    for t in list(inputs) + list(outputs):
        if not t.is_cuda:
            raise RuntimeError(f"local_all_reduce_noalloc: hap_b200 has no CPU path; tensor is on {t.device}")
        if not t.is_contiguous() or t.numel() != ref.numel() or t.device != ref.device:
            raise ValueError("local_all_reduce_noalloc: tensors must be contiguous, equally sized and on one device")
    if any(t.dtype != ref.dtype for t in inputs) or any(o.dtype != outputs[0].dtype for o in outputs):
        raise ValueError("local_all_reduce_noalloc: mixed dtypes")
    with _on_device(ref.device):
        N.check(N.lib.hapx_local_all_reduce_noalloc(len(inputs), N.ptr_array([o.data_ptr() for o in outputs]),
                                                    N.ptr_array([t.data_ptr() for t in inputs]), dtype_code(ref.dtype),
                                                    dtype_code(outputs[0].dtype), float(scale), ref.numel(),
                                                    _stream(ref.device)))


def local_all_reduce_noalloc_status() -> None:
    """Synchronise the current device and raise if a kernel of an earlier
    :func:`local_all_reduce_noalloc` gave up on a bounded wait (its outputs are then unwritten)."""
    N.check(N.lib.hapx_local_all_reduce_noalloc_status())
