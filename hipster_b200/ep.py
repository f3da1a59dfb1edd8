"""Expert parallelism plumbing for the MoE configuration: which GPU owns which routed experts, and distribution of the
NCCL unique id through torch.distributed. The exchange itself runs inside the engine (C++/NCCL)."""
import ctypes

from ._lib import lib, check


def expert_range(rank, world, n_expert):
    """Routed experts [lo, hi) held by `rank`: contiguous blocks, expert e lives on GPU e // (E / G)."""
    return rank * n_expert // world, (rank + 1) * n_expert // world


def owner_of(expert, world, n_expert):
    for r in range(world):
        lo, hi = expert_range(r, world, n_expert)
        if lo <= expert < hi:
            return r
    raise ValueError(expert)


def unique_id():
    buf = (ctypes.c_char * 128)()
    check(lib().hp_ep_unique_id(buf))
    return bytes(buf)


def broadcast_unique_id(dist, rank):
    """Rank 0 creates the NCCL id; every rank receives it through the existing torch.distributed group."""
    import torch
    t = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        t = torch.tensor(list(unique_id()), dtype=torch.uint8)
    dev = torch.device("cuda") if dist.get_backend() == "nccl" else torch.device("cpu")
    t = t.to(dev)
    dist.broadcast(t, src=0)
    return bytes(t.cpu().tolist())
