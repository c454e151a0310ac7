"""One-process-per-GPU plumbing (torchrun-style launches) over torch.distributed.

The library itself only needs 64 opaque bytes from every peer
(b200opt_ipc_export / b200opt_ipc_attach) and, for the NCCL fallback, 128
bytes from rank 0; how they travel is the launcher's business.  Here they
travel through the default process group (gloo on CPU, NCCL's object
collectives on GPU)."""
import os


def env_rank():
    """(rank, world_size, local_rank) from the torchrun environment."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def all_gather_bytes(payload, group=None):
    """Every rank's bytes, in rank order."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    out = [None] * world
    dist.all_gather_object(out, bytes(payload), group=group)
    return out


def broadcast_bytes(payload, src=0, group=None):
    import torch.distributed as dist
    box = [bytes(payload) if dist.get_rank(group) == src else None]
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]


def wire_process_group(adam_group, group=None, with_nccl=False):
    """Attaches every peer rank's memory to `adam_group` (an AdamGroup created with
    this process's rank) and optionally creates the NCCL fallback communicator."""
    import torch.distributed as dist
    if adam_group.nranks == 1:
        return
    assert dist.get_world_size(group) == adam_group.nranks
    assert dist.get_rank(group) == adam_group.rank
    handles = all_gather_bytes(adam_group.ipc_export(), group)
    for q, hb in enumerate(handles):
        if q != adam_group.rank:
            adam_group.ipc_attach(q, hb)
    if with_nccl:
        uid = adam_group.nccl_unique_id() if adam_group.rank == 0 else b""
        adam_group.nccl_init(broadcast_bytes(uid, 0, group))
    dist.barrier(group)  # nobody steps before every rank has wired its peers


def max_over_ranks(values, device=None, group=None):
    """Element-wise maximum of a list of floats over all ranks (timing rule)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device or "cpu")
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return [float(x) for x in t]
