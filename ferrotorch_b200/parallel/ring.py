"""Ring all-reduce, binary-tree broadcast and the two-lap ring barrier written against the plain
``send`` / ``recv`` of any :class:`~.backend.Group`, so they run over in-process simulated ranks as
well as over sockets -- the reference keeps them behind a ``RingTransport`` trait for the same
reason (ferrotorch-distributed/src/gloo_native/collectives.rs:50-320).  ``TcpGroup`` has native
versions of the same algorithms (``csrc/host/tcp_comm.cpp``); these are the portable ones."""
from __future__ import annotations

import threading

import torch

from .backend import Group, InvalidRank


def _exchange(group: Group, send_t: torch.Tensor, dst: int, recv_t: torch.Tensor, src: int) -> None:
    """Send to the right neighbour on a helper thread while receiving from the left one, so that no
    two neighbours wait on each other."""
    err: list = []

    def run():
        try:
            group.send(send_t, dst)
        except BaseException as e:  # noqa: BLE001
            err.append(e)

    t = threading.Thread(target=run, daemon=True)
    t.start()
    group.recv(recv_t, src)
    t.join()
    if err:
        raise err[0]


def ring_all_reduce(group: Group, tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
    """In place.  W - 1 reduce-scatter steps then W - 1 all-gather steps; chunk i covers elements
    ``[i * n / W, (i + 1) * n / W)``; every rank sends ``2 (W - 1) / W`` of the data in total.  The
    order of additions differs from rank to rank, so results agree to rounding, not bitwise (the
    star all-reduce is the bitwise one)."""
    assert op in ("sum", "mean")
    W, r = group.world_size, group.rank
    if W == 1:
        return tensor
    flat = tensor.contiguous().view(-1)
    n = flat.numel()
    lo = [i * n // W for i in range(W + 1)]
    chunk = lambda i: flat[lo[i % W]:lo[i % W + 1]]  # noqa: E731
    right, left = (r + 1) % W, (r - 1) % W
    for s in range(W - 1):                                    # reduce-scatter lap
        send_c, recv_c = chunk(r - s), chunk(r - s - 1)
        tmp = torch.empty_like(recv_c)
        _exchange(group, send_c.clone(), right, tmp, left)
        recv_c += tmp
    own = chunk(r + 1)
    if op == "mean":
        own /= W
    for s in range(W - 1):                                    # all-gather lap
        send_c, recv_c = chunk(r + 1 - s), chunk(r - s)
        tmp = torch.empty_like(recv_c)
        _exchange(group, send_c.clone(), right, tmp, left)
        recv_c.copy_(tmp)
    if flat.data_ptr() != tensor.data_ptr():
        tensor.copy_(flat.view(tensor.shape))
    return tensor


def tree_broadcast(group: Group, tensor: torch.Tensor, root: int = 0) -> torch.Tensor:
    """Rank ``v = (rank - root) mod W`` receives from ``(v - 1) / 2`` and forwards to ``2v + 1`` and
    ``2v + 2``: ``ceil(log2 W)`` hops instead of W - 1 sends from the root."""
    W = group.world_size
    if not 0 <= root < W:
        raise InvalidRank("broadcast root %d outside a world of %d" % (root, W))
    if W == 1:
        return tensor
    v = (group.rank - root) % W
    buf = tensor if tensor.is_contiguous() else tensor.contiguous()
    if v:
        group.recv(buf, ((v - 1) // 2 + root) % W)
    for child in (2 * v + 1, 2 * v + 2):
        if child < W:
            group.send(buf, (child + root) % W)
    if buf.data_ptr() != tensor.data_ptr():
        tensor.copy_(buf)
    return tensor


def ring_barrier(group: Group) -> None:
    """A token goes round the ring twice: after the first lap everybody has arrived, the second
    releases them."""
    W, r = group.world_size, group.rank
    if W == 1:
        return
    token = torch.zeros(1, dtype=torch.uint8)
    for _ in range(2):
        if r == 0:
            group.send(token, 1 % W)
            group.recv(token, W - 1)
        else:
            group.recv(token, r - 1)
            group.send(token, (r + 1) % W)
