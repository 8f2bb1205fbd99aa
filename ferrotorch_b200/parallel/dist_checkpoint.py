"""Sharded (per-rank) checkpoints with resharding and an asynchronous writer, plus async
collective handles and a small RPC layer.

Reference: ``save_distributed`` writes one SafeTensors file per rank (``rank_{r}.safetensors``)
and a rank-0 ``metadata.json`` = ``{num_ranks, tensor_specs: {name: {full_shape, shard_dim,
shard_sizes}}}``; ``load_distributed`` reshards when the world size changed, giving the first
``total % world`` ranks one row more (ferrotorch-distributed/src/checkpoint.rs:107-140, 359-573).
This module writes ``shard_{r}.safetensors`` and a richer ``metadata.json`` (replicated tensors,
dtypes, free-form extras) and reads both layouts.  ``AsyncCheckpointer``
(:686-910); ``PendingCollective`` (async_collective.rs:59-145); ``RpcAgent`` with a name ->
handler registry, length-prefixed frames capped at 1 GiB, ``rpc_sync`` / ``rpc_async``
(rpc.rs:44-607).
"""
from __future__ import annotations

import json
import os
import pickle
import socket
import struct
import threading
from concurrent.futures import Future

import torch

from ..serialize.state import load_safetensors, save_safetensors
from .backend import Group, SizeMismatch


# --------------------------------------------------------------------------- sharded checkpoints
def save_distributed(directory: str, local_state: dict[str, torch.Tensor], shard_dims: dict[str, int | None],
                     group: Group | None = None, rank: int | None = None, world_size: int | None = None,
                     extra: dict | None = None) -> None:
    """``shard_dims[name]`` = dimension along which ``local_state[name]`` is this rank's shard, or
    ``None`` for a replicated tensor (saved by rank 0 only)."""
    rank = group.rank if group is not None else (rank or 0)
    world = group.world_size if group is not None else (world_size or 1)
    os.makedirs(directory, exist_ok=True)
    mine = {k: v for k, v in local_state.items() if shard_dims.get(k) is not None or rank == 0}
    save_safetensors(mine, os.path.join(directory, "shard_%d.safetensors" % rank))
    if rank == 0:
        specs = {}
        for k, v in local_state.items():
            d = shard_dims.get(k)
            gs = list(v.shape)
            if d is not None:
                gs[d] *= world
            specs[k] = {"global_shape": gs, "shard_dim": d, "dtype": str(v.dtype)}
        with open(os.path.join(directory, "metadata.json"), "w") as f:
            json.dump({"world_size": world, "tensors": specs, "extra": extra or {}}, f, indent=1)
    if group is not None:
        group.barrier()


def shard_sizes(total: int, parts: int) -> list[int]:
    """Sizes of ``parts`` contiguous shards of ``total`` rows: the first ``total % parts`` get one
    more (checkpoint.rs ``compute_shard_sizes``)."""
    base, rem = divmod(total, parts)
    return [base + (1 if i < rem else 0) for i in range(parts)]


def _take(full: torch.Tensor, d: int, rank: int, world_size: int, name: str, uneven: bool) -> torch.Tensor:
    if full.shape[d] % world_size and not uneven:
        raise SizeMismatch("%s: dim %d (%d) not divisible by new world size %d" % (name, d, full.shape[d], world_size))
    sizes = shard_sizes(full.shape[d], world_size)
    return full.narrow(d, sum(sizes[:rank]), sizes[rank]).contiguous()


def load_distributed(directory: str, rank: int, world_size: int, device="cpu", uneven: bool = False) -> tuple[dict, dict]:
    """Load this rank's shards, resharding when ``world_size`` differs from the saved one.
    Returns ``(state, extra)``.  A dimension that does not divide by the new world size is an
    error unless ``uneven`` (then the split follows :func:`shard_sizes`).  A directory written by
    the reference (``num_ranks`` / ``tensor_specs`` metadata, ``rank_{r}.safetensors``) loads too;
    its rule is the uneven one."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank %d outside a world of %d" % (rank, world_size))
    with open(os.path.join(directory, "metadata.json")) as f:
        meta = json.load(f)
    if "tensor_specs" in meta:                        # the reference's layout
        saved, specs, extra, pattern, uneven = meta["num_ranks"], meta["tensor_specs"], {}, "rank_%d.safetensors", True
    else:
        saved, specs, extra, pattern = meta["world_size"], meta["tensors"], meta["extra"], "shard_%d.safetensors"

    def shard_file(r):
        path = os.path.join(directory, pattern % r)
        if not os.path.exists(path):
            raise FileNotFoundError("missing shard %s" % path)
        return path

    if saved == world_size:
        if not specs and not os.path.exists(os.path.join(directory, pattern % rank)):
            return {}, extra
        st = load_safetensors(shard_file(rank), device)
        if rank != 0:
            rep = {k for k, s in specs.items() if s["shard_dim"] is None}
            if rep:
                st.update(load_safetensors(shard_file(0), device, key_filter=lambda k: k in rep))
        return st, extra
    shards = [load_safetensors(shard_file(r), "cpu") for r in range(saved)]
    out = {}
    for name, spec in specs.items():
        d = spec["shard_dim"]
        if d is None:
            out[name] = shards[0][name].to(device)
            continue
        for r, sh in enumerate(shards):
            if name not in sh:
                raise KeyError("tensor %r missing from the shard of rank %d" % (name, r))
        full = torch.cat([sh[name] for sh in shards], dim=d)
        want = spec.get("full_shape") or spec.get("global_shape")
        if want is not None and list(full.shape) != list(want):
            raise SizeMismatch("%s: shards add up to %s, metadata says %s" % (name, list(full.shape), list(want)))
        out[name] = _take(full, d, rank, world_size, name, uneven).to(device)
    return out, extra


def save_reference_distributed(directory: str, local_state: dict[str, torch.Tensor], shard_dim: dict[str, int],
                               sizes: dict[str, list[int]], rank: int, world_size: int) -> None:
    """Write this rank's part of a checkpoint in the reference's layout (every tensor sharded;
    ``sizes[name]`` = size along ``shard_dim[name]`` on every rank)."""
    os.makedirs(directory, exist_ok=True)
    save_safetensors(local_state, os.path.join(directory, "rank_%d.safetensors" % rank))
    if rank == 0:
        specs = {}
        for k, v in local_state.items():
            full = list(v.shape)
            full[shard_dim[k]] = sum(sizes[k])
            specs[k] = {"full_shape": full, "shard_dim": shard_dim[k], "shard_sizes": list(sizes[k])}
        with open(os.path.join(directory, "metadata.json"), "w") as f:
            json.dump({"num_ranks": world_size, "tensor_specs": specs}, f, indent=2)


class AsyncDistributedCheckpointer:
    def __init__(self):
        self._thread: threading.Thread | None = None
        self._err: list = []

    def save_async(self, directory, local_state, shard_dims, rank, world_size, extra=None) -> "AsyncDistributedCheckpointer":
        self.wait()
        snap = {k: v.detach().to("cpu", copy=True) for k, v in local_state.items()}

        def work():
            try:
                save_distributed(directory, snap, shard_dims, None, rank, world_size, extra)
            except BaseException as e:  # noqa: BLE001
                self._err.append(e)

        self._thread = threading.Thread(target=work, daemon=True)
        self._thread.start()
        return self

    def is_done(self) -> bool:
        return self._thread is None or not self._thread.is_alive()

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._err:
            raise self._err.pop()


# --------------------------------------------------------------------------- async collectives
class PendingCollective:
    """A collective running on a helper thread; ``wait()`` returns its result or re-raises."""

    def __init__(self, fn, *args):
        self._fut: Future = Future()

        def run():
            try:
                self._fut.set_result(fn(*args))
            except BaseException as e:  # noqa: BLE001
                self._fut.set_exception(e)

        threading.Thread(target=run, daemon=True).start()

    def is_done(self) -> bool:
        return self._fut.done()

    def wait(self, timeout: float | None = None):
        return self._fut.result(timeout)


def all_reduce_async(group: Group, t: torch.Tensor, op: str = "sum") -> PendingCollective:
    return PendingCollective(group.all_reduce, t, op)


def all_gather_async(group: Group, t: torch.Tensor) -> PendingCollective:
    return PendingCollective(group.all_gather, t)


# --------------------------------------------------------------------------- RPC
MAX_RPC_MSG_SIZE = 1 << 30


def _send_msg(sock: socket.socket, payload: bytes) -> None:
    if len(payload) > MAX_RPC_MSG_SIZE:
        raise SizeMismatch("RPC message of %d bytes exceeds the 1 GiB cap" % len(payload))
    sock.sendall(struct.pack("<Q", len(payload)) + payload)


def _recv_msg(sock: socket.socket) -> bytes:
    hdr = b""
    while len(hdr) < 8:
        c = sock.recv(8 - len(hdr))
        if not c:
            raise ConnectionError("peer closed")
        hdr += c
    (n,) = struct.unpack("<Q", hdr)
    if n > MAX_RPC_MSG_SIZE:
        raise SizeMismatch("RPC frame of %d bytes exceeds the 1 GiB cap" % n)
    buf = bytearray()
    while len(buf) < n:
        c = sock.recv(min(1 << 20, n - len(buf)))
        if not c:
            raise ConnectionError("peer closed")
        buf += c
    return bytes(buf)


class RpcAgent:
    """Serve registered handlers on a TCP port and call handlers of other agents by name."""

    def __init__(self, name: str, host: str = "127.0.0.1", port: int = 0):
        self.name, self.handlers = name, {}
        self._srv = socket.socket()
        self._srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._srv.bind((host, port))
        self._srv.listen(16)
        self.address = self._srv.getsockname()
        self._stop = False
        threading.Thread(target=self._serve, daemon=True).start()

    def register(self, fn_name: str, fn) -> None:
        self.handlers[fn_name] = fn

    def _serve(self):
        while not self._stop:
            try:
                conn, _ = self._srv.accept()
            except OSError:
                return
            threading.Thread(target=self._handle, args=(conn,), daemon=True).start()

    def _handle(self, conn):
        with conn:
            try:
                fn_name, args, kwargs = pickle.loads(_recv_msg(conn))
                if fn_name not in self.handlers:
                    res = ("err", "no handler %r on %s" % (fn_name, self.name))
                else:
                    res = ("ok", self.handlers[fn_name](*args, **kwargs))
            except BaseException as e:  # noqa: BLE001
                res = ("err", repr(e))
            try:
                _send_msg(conn, pickle.dumps(res))
            except OSError:
                pass

    @staticmethod
    def rpc_sync(address, fn_name: str, *args, timeout: float = 60.0, **kwargs):
        with socket.create_connection(address, timeout=timeout) as s:
            _send_msg(s, pickle.dumps((fn_name, args, kwargs)))
            status, val = pickle.loads(_recv_msg(s))
        if status != "ok":
            raise RuntimeError("remote call %s failed: %s" % (fn_name, val))
        return val

    @staticmethod
    def rpc_async(address, fn_name: str, *args, **kwargs) -> PendingCollective:
        return PendingCollective(lambda: RpcAgent.rpc_sync(address, fn_name, *args, **kwargs))

    def shutdown(self):
        self._stop = True
        self._srv.close()
