"""B200-native configurable hierarchical collectives.

Allreduce, reduce-scatter and allgather whose schedules are configurable by a
radix ``k`` and a group size ``b`` (plus the MPICH-style algorithms they are
compared against), compiled into step programs and executed by persistent
sm_100a kernels that read peer GPUs' memory over NVLink / NVSwitch.

Typical use, one process per GPU::

    import torch.distributed as dist
    import configurable_hierarchical_allreduce_algorithms_b200 as chb
    dist.init_process_group("nccl")
    comm = chb.Communicator.from_process_group()
    y = chb.all_reduce(comm, x)                                # tuned choice
    y = chb.all_reduce(comm, x, algo="radix_batch", k=4, b=2)  # explicit schedule
"""
from . import _native
from .parallel.program import Program, ProgramError, list_algorithms, cached_program

__all__ = ["Program", "ProgramError", "list_algorithms", "cached_program", "Communicator", "CollectiveError",
           "all_reduce", "reduce_scatter", "all_gather", "all_to_all", "gather",
           "allgather_radix_batch", "reduce_scatter_radix_batch", "all_reduce_radix_batch",
           "all_reduce_host", "HostAllReduce", "TwoLevel", "DeviceLevel", "LibraryLevel", "GlooLevel", "split_world"]

_LAZY = {
    "Communicator": ("parallel.comm", "Communicator"),
    "CollectiveError": ("parallel.comm", "CollectiveError"),
    "all_reduce": ("ops.collectives", "all_reduce"),
    "reduce_scatter": ("ops.collectives", "reduce_scatter"),
    "all_gather": ("ops.collectives", "all_gather"),
    "all_to_all": ("ops.collectives", "all_to_all"),
    "gather": ("ops.collectives", "gather"),
    "allgather_radix_batch": ("ops.collectives", "allgather_radix_batch"),
    "reduce_scatter_radix_batch": ("ops.collectives", "reduce_scatter_radix_batch"),
    "all_reduce_radix_batch": ("ops.collectives", "all_reduce_radix_batch"),
    "all_reduce_host": ("ops.host", "all_reduce_host"),
    "HostAllReduce": ("ops.host", "HostAllReduce"),
    "TwoLevel": ("parallel.hierarchy", "TwoLevel"),
    "DeviceLevel": ("parallel.hierarchy", "DeviceLevel"),
    "LibraryLevel": ("parallel.hierarchy", "LibraryLevel"),
    "GlooLevel": ("parallel.hierarchy", "GlooLevel"),
    "split_world": ("parallel.hierarchy", "split_world"),
}


def __getattr__(name):
    # torch-dependent parts are imported on first use so that the schedule
    # compiler stays importable in environments without torch
    if name in _LAZY:
        import importlib

        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
    raise AttributeError(name)
