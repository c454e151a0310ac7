"""One-process-per-GPU plumbing (torchrun-style launches) over torch.distributed.

The library itself only needs 64 opaque bytes from every peer
(b200opt_ipc_export / b200opt_ipc_attach) and, for the NCCL fallback, 128
bytes from rank 0; how they travel is the launcher's business.  Here they
travel through the default process group (gloo on CPU, NCCL's object
collectives on GPU).  Arenas created with capi.CREATE_FABRIC are shared as
file descriptors instead, which travel between the processes of one machine
as SCM_RIGHTS messages over Unix datagram sockets (FdExchange)."""
import array
import os
import socket
import struct
import uuid


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


class FdExchange:
    """File descriptors between the ranks of one machine: every rank binds a Unix
    datagram socket in the abstract namespace under a name all ranks can derive,
    and descriptors travel as SCM_RIGHTS ancillary data."""

    def __init__(self, rank, world, group=None, timeout_s=120.0):
        import torch.distributed as dist
        self.rank, self.world = rank, world
        token = broadcast_bytes(uuid.uuid4().hex.encode() if rank == 0 else b"", 0, group).decode()
        self._name = lambda r: ("\0b200opt-%s-%d" % (token, r)).encode()
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
        self.sock.settimeout(timeout_s)
        self.sock.bind(self._name(rank))
        dist.barrier(group)  # every socket is bound before anyone sends

    def send(self, dest, fd, tag):
        self.sock.sendmsg([struct.pack("<ii", self.rank, tag)],
                          [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [fd]))],
                          0, self._name(dest))

    def recv(self, count):
        """`count` messages as (source rank, tag, fd); the caller closes the fds."""
        out = []
        for _ in range(count):
            data, fds, _flags, _addr = socket.recv_fds(self.sock, 8, 1)
            if len(fds) != 1:
                raise RuntimeError("a descriptor message arrived without its descriptor")
            src, tag = struct.unpack("<ii", data)
            out.append((src, tag, fds[0]))
        return out

    def close(self):
        self.sock.close()


def wire_process_group(adam_group, group=None, with_nccl=False):
    """Attaches every peer rank's memory to `adam_group` (an AdamGroup created with
    this process's rank) and optionally creates the NCCL fallback communicator.

    A group created with capi.CREATE_MULTICAST also gets its NVSwitch multicast
    object when every rank's GPU supports one.  Returns {"multicast": bool}."""
    import torch.distributed as dist
    from . import capi
    info = {"multicast": False}
    if adam_group.nranks == 1:
        return info
    assert dist.get_world_size(group) == adam_group.nranks
    assert dist.get_rank(group) == adam_group.rank
    rank, world = adam_group.rank, adam_group.nranks
    if getattr(adam_group, "flags_created", 0):
        want_mc = bool(adam_group.flags_created & capi.CREATE_MULTICAST)
        if want_mc:
            votes = [None] * world
            dist.all_gather_object(votes, adam_group.multicast_supported(adam_group.device),
                                   group=group)
            want_mc = all(votes)
        ex = FdExchange(rank, world, group)
        try:
            fd = adam_group.fd_export()
            for q in range(world):
                if q != rank:
                    ex.send(q, fd, 0)
            os.close(fd)
            mc_ok = False
            if want_mc:
                # rank 0 creates the object and says whether that worked before
                # anyone waits for its descriptor
                mfd, box = -1, [None]
                if rank == 0:
                    try:
                        mfd = adam_group.mc_create()
                        box = [True]
                    except capi.B200OptError:
                        box = [False]
                dist.broadcast_object_list(box, src=0, group=group)
                mc_ok = bool(box[0])
                if rank == 0 and mc_ok:
                    for q in range(1, world):
                        ex.send(q, mfd, 1)
                    os.close(mfd)
            got = ex.recv(world - 1 + (1 if mc_ok and rank != 0 else 0))
            for src, tag, pfd in got:
                try:
                    if tag == 0:
                        adam_group.fd_attach(src, pfd)
                    else:
                        adam_group.mc_join(pfd)
                finally:
                    os.close(pfd)
            if mc_ok:
                dist.barrier(group)  # every GPU has joined the object before anyone binds
                adam_group.mc_bind()
                info["multicast"] = True
        finally:
            ex.close()
    else:
        handles = all_gather_bytes(adam_group.ipc_export(), group)
        for q, hb in enumerate(handles):
            if q != rank:
                adam_group.ipc_attach(q, hb)
    if with_nccl:
        uid = adam_group.nccl_unique_id() if rank == 0 else b""
        adam_group.nccl_init(broadcast_bytes(uid, 0, group))
    dist.barrier(group)  # nobody steps before every rank has wired its peers
    return info


def max_over_ranks(values, device=None, group=None):
    """Element-wise maximum of a list of floats over all ranks (timing rule)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device or "cpu")
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return [float(x) for x in t]
