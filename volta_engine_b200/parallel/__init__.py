"""Tensor / expert / context parallelism over NVLink 5 + NVSwitch (one process per GPU)."""
from .comm import LocalComm


def make_comm(kind: str, device, **kw):
    """``symm`` = the engine's own NVLink kernels over symmetric memory; ``nccl`` = library baseline."""
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return LocalComm()
    if kind == "nccl":
        from .symm import NcclComm
        return NcclComm(device)
    from .symm import SymmComm
    return SymmComm(device, **kw)
