"""Process-group back-ends and the collectives layered on them.

The verbs mirror the reference's ``Backend`` trait -- ``rank, world_size, send, recv,
recv_timeout, barrier`` (ferrotorch-distributed/src/backend.rs:42-89) -- and the collectives
its ``collective.rs`` builds on top: ``allreduce`` (Sum / Mean, accumulated at rank 0 in rank
order so every rank ends bitwise identical, collective.rs:80-148), ``broadcast`` (:158-196),
``all_gather`` (:225-298), ``reduce_scatter`` (:328-426), ``all_to_all`` (+ uneven, :464-667).

Back-ends:

* :class:`TcpGroup` -- the native C++ transport (``csrc/host/tcp_comm.cpp``): TCP star
  rendezvous from ``MASTER_ADDR / MASTER_PORT / RANK / WORLD_SIZE``, framed messages with
  timeouts, star and ring all-reduce.
* :class:`SimulatedGroup` -- in-process ranks as threads with a ``world x world`` queue matrix
  (the reference's ``SimulatedBackend``, backend.rs:401-582); unit tests need no sockets.
* :class:`SubGroup` -- a view of a parent group restricted to some ranks (backend.rs:608-766).
* :class:`TorchGroup` -- ``torch.distributed`` (gloo on CPU, NCCL on GPU).
"""
from __future__ import annotations

import ctypes
import os
import queue
import threading
from dataclasses import dataclass
from typing import Sequence

import torch

from .. import _native


# --------------------------------------------------------------------------- errors (error.rs:21-66)
class DistributedError(RuntimeError):
    pass


class InvalidRank(DistributedError):
    pass


class InvalidWorldSize(DistributedError):
    pass


class SelfSend(DistributedError):
    pass


class NoConnection(DistributedError):
    pass


class SizeMismatch(DistributedError):
    pass


class IoError(DistributedError):
    pass


class Timeout(DistributedError):
    pass


class UnsupportedOp(DistributedError):
    pass


class BackendUnavailable(DistributedError):
    pass


_CODES = {-1: InvalidRank, -2: InvalidWorldSize, -3: SelfSend, -4: NoConnection, -5: SizeMismatch, -6: IoError,
          -7: Timeout, -8: UnsupportedOp}

DEFAULT_COLLECTIVE_TIMEOUT_S = 60.0  # collective.rs:35


def _raise(code: int, what: str):
    if code != 0:
        raise _CODES.get(code, DistributedError)("%s failed (code %d)" % (what, code))


class PendingOp:
    """Handle of a posted send or receive: ``wait()`` blocks until it has completed and re-raises
    what it raised (async collectives of the reference: ferrotorch-distributed/src/async_collective.rs)."""

    def __init__(self):
        self._done = threading.Event()
        self._error: BaseException | None = None

    def _finish(self, error: BaseException | None = None) -> None:
        self._error = error
        self._done.set()

    def is_done(self) -> bool:
        return self._done.is_set()

    def wait(self, timeout: float | None = None) -> None:
        if not self._done.wait(timeout):
            raise Timeout("posted operation did not complete in %.1f s" % timeout)
        if self._error is not None:
            raise self._error


class _Lane:
    """One worker thread executing posted operations in order."""

    def __init__(self):
        self._q: queue.Queue = queue.Queue()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def post(self, fn, *args) -> PendingOp:
        op = PendingOp()
        self._q.put((op, fn, args))
        return op

    def _run(self) -> None:
        while True:
            op, fn, args = self._q.get()
            try:
                fn(*args)
                op._finish()
            except BaseException as e:  # noqa: BLE001  (handed to the waiter)
                op._finish(e)


class _TorchWork(PendingOp):
    def __init__(self, work, keep):
        super().__init__()
        self._work, self._keep = work, keep

    def is_done(self) -> bool:
        return self._work.is_completed()

    def wait(self, timeout: float | None = None) -> None:
        self._work.wait()
        self._keep = None


class Group:
    """Common collective implementations over ``send`` / ``recv`` (bytes-oriented)."""

    rank: int
    world_size: int

    # --- point to point (to be provided)
    def send(self, t: torch.Tensor, dst: int) -> None:
        raise NotImplementedError

    def recv(self, t: torch.Tensor, src: int, timeout: float | None = None) -> None:
        raise NotImplementedError

    def _check_peer(self, peer: int) -> None:
        if peer == self.rank:
            raise SelfSend("rank %d cannot send to / receive from itself" % peer)
        if not 0 <= peer < self.world_size:
            raise InvalidRank("rank %d outside world of %d" % (peer, self.world_size))

    # --- non-blocking point to point.  Messages to one peer leave in the order they were posted
    # and receives from one peer complete in the order they were posted: each (peer, direction)
    # has one worker thread with a FIFO of requests.  Back-ends with native asynchronous
    # operations (``TorchGroup``) override both.
    def isend(self, t: torch.Tensor, dst: int) -> "PendingOp":
        self._check_peer(dst)
        return self._lane(dst, "send").post(self.send, t, dst)

    def irecv(self, t: torch.Tensor, src: int, timeout: float | None = None) -> "PendingOp":
        self._check_peer(src)
        return self._lane(src, "recv").post(self.recv, t, src, timeout)

    def _lane(self, peer: int, direction: str) -> "_Lane":
        lanes = self.__dict__.setdefault("_lanes", {})
        lock = self.__dict__.setdefault("_lanes_lock", threading.Lock())
        with lock:
            lane = lanes.get((peer, direction))
            if lane is None:
                lane = lanes[(peer, direction)] = _Lane()
            return lane

    def sendrecv(self, send_t: torch.Tensor, recv_t: torch.Tensor, peer: int) -> None:
        """Deadlock-free exchange: the lower rank sends first (p2p.rs:30-160)."""
        if self.rank < peer:
            self.send(send_t, peer)
            self.recv(recv_t, peer)
        else:
            self.recv(recv_t, peer)
            self.send(send_t, peer)

    # --- collectives
    def barrier(self) -> None:
        t = torch.zeros(1)
        self.all_reduce(t)

    def all_reduce(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """In place; accumulation happens at rank 0 in rank order."""
        assert op in ("sum", "mean")
        if self.world_size == 1:
            return t
        flat = t.contiguous().view(-1)
        if self.rank == 0:
            tmp = torch.empty_like(flat)
            for r in range(1, self.world_size):
                self.recv(tmp, r)
                flat += tmp
            if op == "mean":
                flat /= self.world_size
            for r in range(1, self.world_size):
                self.send(flat, r)
        else:
            self.send(flat, 0)
            self.recv(flat, 0)
        if flat.data_ptr() != t.data_ptr():
            t.copy_(flat.view_as(t))
        return t

    def broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        if not 0 <= root < self.world_size:
            raise InvalidRank("broadcast root %d" % root)
        if self.world_size == 1:
            return t
        buf = t.contiguous()
        if self.rank == root:
            for r in range(self.world_size):
                if r != root:
                    self.send(buf, r)
        else:
            self.recv(buf, root)
            if buf.data_ptr() != t.data_ptr():
                t.copy_(buf)
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """Concatenate every rank's tensor on dim 0."""
        parts = [torch.empty_like(t) for _ in range(self.world_size)]
        parts[self.rank] = t.contiguous()
        for r in range(self.world_size):
            self.broadcast(parts[r], r)
        return torch.cat(parts, dim=0)

    def reduce_scatter(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """All-reduce then keep slice ``rank`` of dim 0 (dim 0 must divide by the world size)."""
        if t.shape[0] % self.world_size:
            raise SizeMismatch("reduce_scatter: dim 0 (%d) not divisible by world size %d" % (t.shape[0], self.world_size))
        full = self.all_reduce(t.clone(), op)
        n = t.shape[0] // self.world_size
        return full[self.rank * n:(self.rank + 1) * n].clone()

    def all_to_all(self, t: torch.Tensor, send_counts: Sequence[int] | None = None,
                   recv_counts: Sequence[int] | None = None) -> torch.Tensor:
        """Rank r sends chunk p of dim 0 to rank p; pairwise ordered exchange
        (collective.rs:519-547).  ``send_counts`` / ``recv_counts`` give the uneven variant."""
        W = self.world_size
        if send_counts is None:
            if t.shape[0] % W:
                raise SizeMismatch("all_to_all: dim 0 (%d) not divisible by world size %d" % (t.shape[0], W))
            send_counts = recv_counts = [t.shape[0] // W] * W
        assert recv_counts is not None and len(send_counts) == W and len(recv_counts) == W
        offs = [0]
        for c in send_counts:
            offs.append(offs[-1] + c)
        outs = [torch.empty((recv_counts[p],) + tuple(t.shape[1:]), dtype=t.dtype) for p in range(W)]
        outs[self.rank].copy_(t[offs[self.rank]:offs[self.rank + 1]])
        for p in range(W):
            if p != self.rank:
                self.sendrecv(t[offs[p]:offs[p + 1]].contiguous(), outs[p], p)
        return torch.cat(outs, dim=0)


# --------------------------------------------------------------------------- TCP (native)
_host_ready = False


def _host_lib():
    global _host_ready
    lib = _native.host()
    if not _host_ready:
        vp, ci, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.ftc_create.restype = vp
        lib.ftc_create.argtypes = [ctypes.c_char_p, ci, ci, ci, ll]
        lib.ftc_destroy.argtypes = [vp]
        lib.ftc_last_error_code.restype = ci
        lib.ftc_set_timeout.argtypes = [vp, ll]
        for name, args in (("ftc_send", [vp, vp, ll, ci]), ("ftc_recv", [vp, vp, ll, ci, ll]),
                           ("ftc_barrier", [vp]), ("ftc_broadcast", [vp, vp, ll, ci]),
                           ("ftc_allreduce_f32", [vp, vp, ll, ci]), ("ftc_allreduce_f64", [vp, vp, ll, ci]),
                           ("ftc_allgather", [vp, vp, vp, ll]), ("ftc_connect_mesh", [vp]),
                           ("ftc_ring_allreduce_f32", [vp, vp, ll, ci]),
                           ("ftc_tree_broadcast", [vp, vp, ll, ci]), ("ftc_ring_barrier", [vp])):
            fn = getattr(lib, name)
            fn.restype = ci
            fn.argtypes = args
        _host_ready = True
    return lib


class TcpGroup(Group):
    """CPU ranks over loopback / LAN TCP through the native transport."""

    def __init__(self, rank: int | None = None, world_size: int | None = None, master_addr: str | None = None,
                 master_port: int | None = None, timeout: float = DEFAULT_COLLECTIVE_TIMEOUT_S):
        env = os.environ
        self.rank = int(env["RANK"]) if rank is None else rank
        self.world_size = int(env["WORLD_SIZE"]) if world_size is None else world_size
        addr = master_addr or env.get("MASTER_ADDR", "127.0.0.1")
        port = int(master_port or env.get("MASTER_PORT", "29500"))
        self._lib = _host_lib()
        self.timeout = float(timeout)
        self._h = self._lib.ftc_create(addr.encode(), port, self.rank, self.world_size, int(timeout * 1000))
        if not self._h:
            _raise(self._lib.ftc_last_error_code() or -6, "rendezvous")

    @classmethod
    def from_env(cls, **kw) -> "TcpGroup":
        return cls(**kw)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ftc_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_timeout(self, seconds: float) -> None:
        self.timeout = float(seconds)
        self._lib.ftc_set_timeout(self._h, int(seconds * 1000))

    def send(self, t: torch.Tensor, dst: int) -> None:
        self._check_peer(dst)
        t = t.contiguous()
        _raise(self._lib.ftc_send(self._h, t.data_ptr(), t.numel() * t.element_size(), dst), "send")

    def recv(self, t: torch.Tensor, src: int, timeout: float | None = None) -> None:
        self._check_peer(src)
        assert t.is_contiguous()
        ms = -1 if timeout is None else int(timeout * 1000)
        _raise(self._lib.ftc_recv(self._h, t.data_ptr(), t.numel() * t.element_size(), src, ms), "recv")

    def barrier(self, algorithm: str = "star") -> None:
        """``"star"``: gather at rank 0, then release; ``"ring"``: a token goes round the ring of
        the full mesh twice, no coordinator."""
        assert algorithm in ("star", "ring")
        _raise((self._lib.ftc_ring_barrier if algorithm == "ring" else self._lib.ftc_barrier)(self._h), "barrier")

    def broadcast(self, t: torch.Tensor, root: int = 0, algorithm: str = "star") -> torch.Tensor:
        """``"star"`` relays through rank 0; ``"tree"`` forwards down a binary tree rooted at
        ``root`` over the full mesh (log2 W hops)."""
        assert algorithm in ("star", "tree")
        if not 0 <= root < self.world_size:
            raise InvalidRank("root %d outside a world of %d" % (root, self.world_size))
        buf = t if t.is_contiguous() else t.contiguous()
        fn = self._lib.ftc_tree_broadcast if algorithm == "tree" else self._lib.ftc_broadcast
        _raise(fn(self._h, buf.data_ptr(), buf.numel() * buf.element_size(), root), "broadcast")
        if buf.data_ptr() != t.data_ptr():
            t.copy_(buf)
        return t

    def all_reduce(self, t: torch.Tensor, op: str = "sum", algorithm: str = "star") -> torch.Tensor:
        """``algorithm="star"`` reduces at rank 0 in rank order (bitwise identical on every rank);
        ``"ring"`` is the bandwidth-optimal ring over the full mesh (fp32 only)."""
        assert op in ("sum", "mean")
        if t.dtype not in (torch.float32, torch.float64):
            return super().all_reduce(t, op)
        buf = t if t.is_contiguous() else t.contiguous()
        if algorithm == "ring" and t.dtype == torch.float32:
            rc = self._lib.ftc_ring_allreduce_f32(self._h, buf.data_ptr(), buf.numel(), int(op == "mean"))
        elif t.dtype == torch.float32:
            rc = self._lib.ftc_allreduce_f32(self._h, buf.data_ptr(), buf.numel(), int(op == "mean"))
        else:
            rc = self._lib.ftc_allreduce_f64(self._h, buf.data_ptr(), buf.numel(), int(op == "mean"))
        _raise(rc, "all_reduce")
        if buf.data_ptr() != t.data_ptr():
            t.copy_(buf)
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        out = torch.empty((self.world_size * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype)
        _raise(self._lib.ftc_allgather(self._h, t.data_ptr(), out.data_ptr(), t.numel() * t.element_size()), "all_gather")
        return out

    def connect_mesh(self) -> None:
        """Collective: build the full mesh.  The rendezvous only creates the star through rank 0
        (like the reference's ``TcpBackend``); point-to-point traffic between two non-zero ranks
        needs this first."""
        _raise(self._lib.ftc_connect_mesh(self._h), "connect_mesh")

    def all_to_all(self, t, send_counts=None, recv_counts=None):
        if self.world_size > 2:
            self.connect_mesh()
        return super().all_to_all(t, send_counts, recv_counts)


# --------------------------------------------------------------------------- simulated (threads)
class _SimWorld:
    def __init__(self, n: int):
        self.n = n
        self.q = [[queue.Queue() for _ in range(n)] for _ in range(n)]  # q[src][dst]


class SimulatedGroup(Group):
    """One object per rank, used from one thread per rank (backend.rs:401-582)."""

    def __init__(self, world: _SimWorld, rank: int, timeout: float = DEFAULT_COLLECTIVE_TIMEOUT_S):
        self._w, self.rank, self.world_size, self.timeout = world, rank, world.n, timeout

    @staticmethod
    def create_group(n: int, timeout: float = DEFAULT_COLLECTIVE_TIMEOUT_S) -> list["SimulatedGroup"]:
        if n < 1:
            raise InvalidWorldSize("world size %d" % n)
        w = _SimWorld(n)
        return [SimulatedGroup(w, r, timeout) for r in range(n)]

    def send(self, t: torch.Tensor, dst: int) -> None:
        self._check_peer(dst)
        self._w.q[self.rank][dst].put(t.detach().clone())

    def recv(self, t: torch.Tensor, src: int, timeout: float | None = None) -> None:
        self._check_peer(src)
        try:
            got = self._w.q[src][self.rank].get(timeout=self.timeout if timeout is None else timeout)
        except queue.Empty:
            raise Timeout("recv from rank %d timed out" % src) from None
        if got.numel() * got.element_size() != t.numel() * t.element_size():
            raise SizeMismatch("expected %d bytes, got %d" % (t.numel() * t.element_size(),
                                                              got.numel() * got.element_size()))
        t.copy_(got.view_as(t))


def run_simulated(n: int, fn, *args, timeout: float = 30.0):
    """Run ``fn(group, *args)`` on ``n`` simulated ranks (one thread each); returns the results
    in rank order and re-raises the first exception."""
    groups = SimulatedGroup.create_group(n, timeout)
    results, errors = [None] * n, [None] * n

    def work(r):
        try:
            results[r] = fn(groups[r], *args)
        except BaseException as e:  # noqa: BLE001
            errors[r] = e

    threads = [threading.Thread(target=work, args=(r,), daemon=True) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout + 30)
    for e in errors:
        if e is not None:
            raise e
    return results


class SubGroup(Group):
    """A group restricted to a sorted, de-duplicated subset of the parent's ranks; local ranks
    are positions in that list and every call forwards to the parent (backend.rs:608-766)."""

    def __init__(self, parent: Group, members: Sequence[int]):
        self.members = sorted(set(members))
        for m in self.members:
            if not 0 <= m < parent.world_size:
                raise InvalidRank("member %d outside parent world %d" % (m, parent.world_size))
        if parent.rank not in self.members:
            raise InvalidRank("rank %d is not a member of %s" % (parent.rank, self.members))
        self.parent = parent
        self.rank = self.members.index(parent.rank)
        self.world_size = len(self.members)

    def global_rank(self, local: int) -> int:
        return self.members[local]

    # backend.rs ``SubBackend::{to_global, to_local}``
    to_global = global_rank

    def to_local(self, global_rank: int) -> int:
        if global_rank not in self.members:
            raise InvalidRank("rank %d is not a member of this sub-group %s" % (global_rank, self.members))
        return self.members.index(global_rank)

    def send(self, t, dst):
        self._check_peer(dst)
        self.parent.send(t, self.members[dst])

    def recv(self, t, src, timeout=None):
        self._check_peer(src)
        self.parent.recv(t, self.members[src], timeout)


class TorchGroup(Group):
    """``torch.distributed`` process group (gloo on CPU tensors, NCCL on CUDA tensors)."""

    def __init__(self, pg=None):
        import torch.distributed as dist

        self._dist, self.pg = dist, pg if pg is not None else dist.group.WORLD
        self.rank, self.world_size = dist.get_rank(self.pg), dist.get_world_size(self.pg)

    def _g(self, r):
        return self._dist.get_global_rank(self.pg, r)

    def send(self, t, dst):
        self._check_peer(dst)
        self._dist.send(t.contiguous(), self._g(dst), group=self.pg)

    def recv(self, t, src, timeout=None):
        self._check_peer(src)
        self._dist.recv(t, self._g(src), group=self.pg)

    def isend(self, t, dst):
        self._check_peer(dst)
        t = t.contiguous()
        return _TorchWork(self._dist.isend(t, self._g(dst), group=self.pg), t)   # keeps the buffer alive

    def irecv(self, t, src, timeout=None):
        self._check_peer(src)
        return _TorchWork(self._dist.irecv(t, self._g(src), group=self.pg), t)

    def barrier(self):
        self._dist.barrier(self.pg)

    def all_reduce(self, t, op="sum"):
        d = self._dist
        if op == "mean" and not t.is_cuda:
            d.all_reduce(t, d.ReduceOp.SUM, group=self.pg)
            t /= self.world_size
        else:
            d.all_reduce(t, d.ReduceOp.AVG if op == "mean" else d.ReduceOp.SUM, group=self.pg)
        return t

    def broadcast(self, t, root=0):
        self._dist.broadcast(t, self._g(root), group=self.pg)
        return t

    def all_gather(self, t):
        t = t.contiguous()
        out = torch.empty((self.world_size * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        self._dist.all_gather_into_tensor(out, t, group=self.pg)
        return out

    def reduce_scatter(self, t, op="sum"):
        if t.shape[0] % self.world_size:
            raise SizeMismatch("reduce_scatter: dim 0 (%d) not divisible by world size %d" % (t.shape[0], self.world_size))
        if not t.is_cuda:
            return super().reduce_scatter(t, op)
        d = self._dist
        out = torch.empty((t.shape[0] // self.world_size,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        d.reduce_scatter_tensor(out, t.contiguous(), d.ReduceOp.AVG if op == "mean" else d.ReduceOp.SUM, group=self.pg)
        return out


class HybridGroup(Group):
    """Two transports under one group (ferrotorch-distributed/src/hybrid_backend.rs:49-120): a
    ``control`` group (TCP) carries point-to-point messages, barriers and collectives on host
    tensors, a ``data`` group (NCCL) carries collectives on device tensors.  The control group is
    built first, so a rank that cannot rendezvous fails before any NCCL communicator exists."""

    def __init__(self, control: Group, data: Group):
        if (control.rank, control.world_size) != (data.rank, data.world_size):
            raise InvalidRank("HybridGroup: control is rank %d of %d but data is rank %d of %d"
                              % (control.rank, control.world_size, data.rank, data.world_size))
        self.control, self.data = control, data
        self.rank, self.world_size = control.rank, control.world_size

    def synchronize_nccl(self) -> None:
        """Wait for the data group's device work (hybrid_backend.rs): collectives here are stream-ordered, so
        this is only needed before the host reads a result."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def tcp(self) -> Group:
        return self.control

    def nccl(self) -> Group:
        return self.data

    def _for(self, t: torch.Tensor) -> Group:
        return self.data if t.is_cuda else self.control

    def send(self, t, dst):
        self.control.send(t, dst)

    def recv(self, t, src, timeout=None):
        self.control.recv(t, src, timeout)

    def barrier(self):
        self.control.barrier()

    def all_reduce(self, t, op="sum"):
        return self._for(t).all_reduce(t, op)

    def broadcast(self, t, root=0):
        return self._for(t).broadcast(t, root)

    def all_gather(self, t):
        return self._for(t).all_gather(t)

    def reduce_scatter(self, t, op="sum"):
        return self._for(t).reduce_scatter(t, op)

    def all_to_all(self, t, send_counts=None, recv_counts=None):
        return self._for(t).all_to_all(t, send_counts, recv_counts)

    def synchronize_data(self) -> None:
        """Wait for the data transport's device work (the reference's ``synchronize_nccl``)."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def close(self) -> None:
        if hasattr(self.control, "close"):
            self.control.close()


@dataclass
class RendezvousConfig:
    """Where and who: read from the launcher's environment (gloo_native/connect.rs:116
    ``RendezvousConfig::from_env``).  ``RANK`` / ``WORLD_SIZE`` are what ``torchrun`` sets; the Open
    MPI and PMI names are accepted as well, so a job started by ``mpirun`` or a PMI launcher needs
    no wrapper (mpi_backend.rs reads the same variables)."""
    master_addr: str
    master_port: int
    rank: int
    world_size: int

    @classmethod
    def from_env(cls, env=None) -> "RendezvousConfig":
        env = os.environ if env is None else env

        def first(names, what):
            for n in names:
                v = env.get(n)
                if v not in (None, ""):
                    try:
                        return int(v)
                    except ValueError:
                        raise InvalidRank("%s=%r is not an integer" % (n, v))
            raise NoConnection("none of %s is set: cannot tell the %s" % (", ".join(names), what))

        rank = first(("RANK", "OMPI_COMM_WORLD_RANK", "PMI_RANK"), "rank")
        world = first(("WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "PMI_SIZE"), "world size")
        if world < 1:
            raise InvalidWorldSize("world size %d" % world)
        if not 0 <= rank < world:
            raise InvalidRank("rank %d outside a world of %d" % (rank, world))
        try:
            port = int(env.get("MASTER_PORT", "29500"))
        except ValueError:
            raise NoConnection("MASTER_PORT=%r is not a port number" % env.get("MASTER_PORT"))
        return cls(env.get("MASTER_ADDR", "127.0.0.1"), port, rank, world)


def init_group(backend: str = "tcp", **kw) -> Group:
    """``backend``: "tcp" (native), "gloo" / "nccl" (torch.distributed, initialised here when
    needed), "simulated" is created with :func:`SimulatedGroup.create_group`."""
    if backend == "tcp":
        if "rank" not in kw and "world_size" not in kw:
            rc = RendezvousConfig.from_env()
            kw = dict(rank=rc.rank, world_size=rc.world_size, master_addr=rc.master_addr, master_port=rc.master_port, **kw)
        return TcpGroup(**kw)
    if backend in ("gloo", "nccl"):
        import torch.distributed as dist

        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group(backend, **kw)
        return TorchGroup()
    if backend == "hybrid":
        tcp_kw = {k: kw.pop(k) for k in ("rank", "world_size", "master_addr", "master_port", "timeout") if k in kw}
        control = init_group("tcp", **tcp_kw)                    # first: fails fast on a bad rendezvous
        return HybridGroup(control, init_group(kw.pop("data_backend", "nccl"), **kw))
    raise BackendUnavailable("unknown backend %r (tcp, gloo, nccl, hybrid)" % backend)
