"""qkan_b200 — the QKANLayer forward/backward of Jim137/qkan as hand-written sm_100a CUDA kernels.

``QKAN`` / ``QKANLayer`` keep the reference's public interface; ``solver="b200"`` is the one
solver of this package. The kernels sit behind a C ABI (``include/qkan_b200.h``,
``qkan_b200/lib/libqkan_b200.so``); build it with ``python -m qkan_b200.build``.
"""
from .layer import QKANLayer, SOLVER_NAME
from .model import QKAN
from .hqkan import FusedHQKAN
from .solver import B200Solver, get_registry, get_solver, register, register_with_reference
from .parallel import GradBucket, bind_host_thread_near_gpu, get_dist_info, print0, shard_rows

__version__ = "0.1.0"
__all__ = ["QKAN", "QKANLayer", "FusedHQKAN", "B200Solver", "GradBucket", "SOLVER_NAME", "bind_host_thread_near_gpu", "get_dist_info",
           "get_registry", "get_solver", "print0", "register", "register_with_reference", "shard_rows"]
