"""hap_b200 - B200-native (sm_100a) executor for the hot path of HAP's synthesized SPMD programs.

The package holds the uneven collectives (drop-in for the reference's ``collectives.py``),
the shard-extent rounding, and the CUDA sources behind them (``csrc/``, C ABI in
``include/hapx.h``).  Importing it requires the built ``libhapx.so``; there is no CPU path.
"""
from . import _native
from .sharding import sharding_round, sharding_round_
from .comm import Comm, init_process_comm, local_comm, single_comm
from . import collectives
from .local import LocalCollectives
from . import linear as linear_ops
from .linear import linear
from . import plan, spmd, attention, fxpass, profiler, dropout
from .einsum import einsum
from .loss import nll_log_softmax_sum
from .norm import layer_norm
from .optim import ClipAdam

__all__ = ["Comm", "init_process_comm", "local_comm", "single_comm", "collectives", "LocalCollectives",
           "sharding_round", "sharding_round_", "linear", "linear_ops", "plan", "spmd", "attention", "einsum"]
