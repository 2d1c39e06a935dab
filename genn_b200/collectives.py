"""Cross-process reductions of custom-update targets.

A data-parallel run gives every process a share of the batch.  A batch-reduce
custom update then needs the reduced value over ALL shares: each process
reduces its own (``b200_custom_update_reduce``), the targets are combined here
with one all-reduce per target over ``torch.distributed`` (NCCL on the device
arrays, gloo on host arrays in the CPU tests), and every process writes the
combined value back (``b200_custom_update_broadcast``).  The reference emits one
NCCL reduction per such group (backends/cuda/backend.cc, genNCCLReduction;
backendBase.h:127-486 lists it among the backend's duties)."""
from typing import Iterable, Sequence


class CudaArrayView:
    """Lets torch adopt a device array of the runner (``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, shape: Sequence[int], typestr: str = "<f4"):
        self.__cuda_array_interface__ = {"shape": tuple(int(x) for x in shape), "typestr": typestr,
                                         "data": (int(ptr), False), "version": 2}


def device_tensor(ptr: int, shape: Sequence[int], device: int):
    import torch
    return torch.as_tensor(CudaArrayView(ptr, shape), device=f"cuda:{device}")


def all_reduce_targets(tensors: Iterable, operations: Iterable[str]):
    """In-place all-reduce of each tensor over the default process group; operation "SUM" or "MAX"."""
    import torch.distributed as dist
    ops = {"SUM": dist.ReduceOp.SUM, "MAX": dist.ReduceOp.MAX}
    for t, op in zip(tensors, operations):
        dist.all_reduce(t, op=ops[op])
