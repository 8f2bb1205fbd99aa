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
import socket
import struct
import threading
from concurrent.futures import Future

import torch

from ..serialize.state import load_safetensors, save_safetensors
from .backend import Group, InvalidRank, SizeMismatch


# --------------------------------------------------------------------------- sharded checkpoints
def save_distributed(directory: str, local_state: dict[str, torch.Tensor], shard_dims: dict[str, int | None],
                     group: Group | None = None, rank: int | None = None, world_size: int | None = None,
                     extra: dict | None = None, sizes: dict[str, list[int]] | None = None) -> None:
    """``shard_dims[name]`` = dimension along which ``local_state[name]`` is this rank's shard, or
    ``None`` for a replicated tensor (saved by rank 0 only).

    Shards may be uneven (after an elastic reload on a world size that does not divide the
    tensor).  The metadata records every rank's size along the shard dimension
    (``shard_sizes``, as the reference does: checkpoint.rs:107-140): gathered through ``group``,
    or given as ``sizes[name]`` when there is no group; with neither, shards are taken to be even.
    Every rank also writes its own sizes next to its shard (``shard_{r}.sizes.json``), which the
    loader prefers, so a directory written without a group still reshards correctly."""
    rank = group.rank if group is not None else (rank or 0)
    world = group.world_size if group is not None else (world_size or 1)
    os.makedirs(directory, exist_ok=True)
    mine = {k: v for k, v in local_state.items() if shard_dims.get(k) is not None or rank == 0}
    save_safetensors(mine, os.path.join(directory, "shard_%d.safetensors" % rank))
    sharded = sorted(k for k in local_state if shard_dims.get(k) is not None)
    local_sizes = {k: int(local_state[k].shape[shard_dims[k]]) for k in sharded}
    with open(os.path.join(directory, "shard_%d.sizes.json" % rank), "w") as f:
        json.dump(local_sizes, f)
    all_sizes: dict[str, list[int]] | None = None
    if sizes is not None:
        all_sizes = {k: [int(x) for x in sizes[k]] for k in sharded}
    elif group is not None and world > 1 and sharded:
        mine_t = torch.tensor([local_sizes[k] for k in sharded], dtype=torch.int64,
                              device=local_state[sharded[0]].device)
        gathered = group.all_gather(mine_t)
        rows = gathered.view(world, len(sharded)) if isinstance(gathered, torch.Tensor) else torch.stack(list(gathered))
        rows = rows.cpu()
        all_sizes = {k: [int(rows[r, i]) for r in range(world)] for i, k in enumerate(sharded)}
    if rank == 0:
        specs = {}
        for k, v in local_state.items():
            d = shard_dims.get(k)
            gs = list(v.shape)
            spec = {"shard_dim": d, "dtype": str(v.dtype)}
            if d is not None:
                per_rank = all_sizes[k] if all_sizes is not None else [gs[d]] * world
                if len(per_rank) != world:
                    raise SizeMismatch("%s: %d shard sizes for a world of %d" % (k, len(per_rank), world))
                gs[d] = sum(per_rank)
                spec["shard_sizes"] = per_rank
            spec["global_shape"] = gs
            specs[k] = spec
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
    side = None
    side_paths = [os.path.join(directory, "shard_%d.sizes.json" % r) for r in range(saved)]
    if all(os.path.exists(pth) for pth in side_paths):
        side = []
        for pth in side_paths:
            with open(pth) as f:
                side.append(json.load(f))
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
        if side is not None and want is not None:
            # sizes written by the ranks themselves win over what rank 0 could know at save time
            want = list(want)
            want[d] = sum(int(sz[name]) for sz in side)
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
    """Sharded saves on a helper thread from a host snapshot of the tensors.  Built empty (every
    ``save_async`` names its directory and rank) or, as the reference's ``AsyncCheckpointer::new``
    (ferrotorch-distributed/src/checkpoint.rs:757), bound to ``(directory, rank, world_size)`` so that
    ``save(state, shard_dims)`` needs nothing else."""

    def __init__(self, directory: str | None = None, rank: int = 0, world_size: int = 1):
        self._thread: threading.Thread | None = None
        self._err: list = []
        self._dir, self._rank, self._world = directory, rank, world_size

    def dir(self) -> str | None:
        return self._dir

    def rank(self) -> int:
        return self._rank

    def world_size(self) -> int:
        return self._world

    def save(self, local_state, shard_dims, extra=None) -> "AsyncDistributedCheckpointer":
        if self._dir is None:
            raise ValueError("AsyncDistributedCheckpointer.save: built without a directory; use save_async")
        return self.save_async(self._dir, local_state, shard_dims, self._rank, self._world, extra)

    def is_saving(self) -> bool:
        return not self.is_done()

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

    def __init__(self, fn, *args, op_name: str | None = None):
        self._fut: Future = Future()
        self._op_name = op_name or getattr(fn, "__name__", "collective")

        def run():
            try:
                self._fut.set_result(fn(*args))
            except BaseException as e:  # noqa: BLE001
                self._fut.set_exception(e)

        threading.Thread(target=run, daemon=True).start()

    def is_done(self) -> bool:
        return self._fut.done()

    def op_name(self) -> str:
        return self._op_name

    def wait(self, timeout: float | None = None):
        return self._fut.result(timeout)


def all_reduce_async(group: Group, t: torch.Tensor, op: str = "sum") -> PendingCollective:
    return PendingCollective(group.all_reduce, t, op)


def all_gather_async(group: Group, t: torch.Tensor) -> PendingCollective:
    return PendingCollective(group.all_gather, t)


# --------------------------------------------------------------------------- RPC
MAX_RPC_MSG_SIZE = 1 << 30

# Wire format (little endian), following the reference's frames (rpc.rs:141-234):
#   request : u64 request id | u32 name length | name (utf-8) | u64 payload length | payload
#   response: u64 request id | u8 status (0 ok, 1 error) | u64 payload length | payload
# The payload is data only: a JSON document for the structure (None, bool, int, float, str, list,
# tuple, dict with string keys) in which tensors and byte strings are references to raw blobs
# appended after it.  Nothing on the wire can name code, so a peer cannot make the agent run
# anything but its registered handlers.
_DTYPES = {str(d): d for d in (torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int8,
                               torch.uint8, torch.int16, torch.int32, torch.int64, torch.bool)}


def _encode(obj) -> bytes:
    blobs: list[bytes] = []

    def enc(o):
        if o is None or isinstance(o, (bool, int, float, str)):
            return o
        if isinstance(o, torch.Tensor):
            t = o.detach().cpu().contiguous()
            if str(t.dtype) not in _DTYPES:
                raise TypeError("RPC cannot carry a tensor of dtype %s" % t.dtype)
            blobs.append(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
            return {"__t": len(blobs) - 1, "dtype": str(t.dtype), "shape": list(t.shape)}
        if isinstance(o, (bytes, bytearray, memoryview)):
            blobs.append(bytes(o))
            return {"__b": len(blobs) - 1}
        if isinstance(o, tuple):
            return {"__tuple": [enc(x) for x in o]}
        if isinstance(o, list):
            return [enc(x) for x in o]
        if isinstance(o, dict):
            if not all(isinstance(k, str) for k in o):
                raise TypeError("RPC dictionaries need string keys")
            return {"__d": {k: enc(v) for k, v in o.items()}}
        raise TypeError("RPC cannot carry a value of type %s" % type(o).__name__)

    doc = json.dumps(enc(obj)).encode()
    out = [struct.pack("<QI", len(doc), len(blobs)), doc]
    for bl in blobs:
        out.append(struct.pack("<Q", len(bl)))
        out.append(bl)
    return b"".join(out)


def _decode(buf: bytes):
    if len(buf) < 12:
        raise SizeMismatch("RPC payload of %d bytes is too short" % len(buf))
    n_doc, n_blobs = struct.unpack_from("<QI", buf, 0)
    pos = 12
    if n_doc > len(buf) - pos:
        raise SizeMismatch("RPC payload: document length %d exceeds the frame" % n_doc)
    doc = json.loads(buf[pos:pos + n_doc].decode())
    pos += n_doc
    blobs = []
    for _ in range(n_blobs):
        if pos + 8 > len(buf):
            raise SizeMismatch("RPC payload: truncated blob table")
        (n,) = struct.unpack_from("<Q", buf, pos)
        pos += 8
        if n > len(buf) - pos:
            raise SizeMismatch("RPC payload: blob of %d bytes exceeds the frame" % n)
        blobs.append(buf[pos:pos + n])
        pos += n

    def blob(i):
        if not isinstance(i, int) or not 0 <= i < len(blobs):
            raise SizeMismatch("RPC payload: blob index %r out of range" % (i,))
        return blobs[i]

    def dec(o):
        if isinstance(o, list):
            return [dec(x) for x in o]
        if isinstance(o, dict):
            if "__t" in o:
                dt = _DTYPES.get(o.get("dtype"))
                if dt is None:
                    raise TypeError("RPC payload: unknown dtype %r" % (o.get("dtype"),))
                raw = blob(o["__t"])
                shape = [int(x) for x in o["shape"]]
                t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dt) if raw else torch.empty(0, dtype=dt)
                return t.reshape(shape)
            if "__b" in o:
                return blob(o["__b"])
            if "__tuple" in o:
                return tuple(dec(x) for x in o["__tuple"])
            if "__d" in o:
                return {k: dec(v) for k, v in o["__d"].items()}
            raise TypeError("RPC payload: unknown node %r" % (sorted(o),))
        return o

    return dec(doc)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        c = sock.recv(min(1 << 20, n - len(buf)))
        if not c:
            raise ConnectionError("peer closed")
        buf += c
    return bytes(buf)


def _recv_len(sock: socket.socket) -> int:
    (n,) = struct.unpack("<Q", _recv_exact(sock, 8))
    if n > MAX_RPC_MSG_SIZE:
        raise SizeMismatch("RPC frame of %d bytes exceeds the 1 GiB cap" % n)
    return n


def _send_request(sock: socket.socket, req_id: int, name: str, payload: bytes) -> None:
    if len(payload) > MAX_RPC_MSG_SIZE:
        raise SizeMismatch("RPC message of %d bytes exceeds the 1 GiB cap" % len(payload))
    nm = name.encode()
    sock.sendall(struct.pack("<QI", req_id, len(nm)) + nm + struct.pack("<Q", len(payload)) + payload)


def _recv_request(sock: socket.socket):
    req_id, n_name = struct.unpack("<QI", _recv_exact(sock, 12))
    if n_name > 4096:
        raise SizeMismatch("RPC handler name of %d bytes" % n_name)
    name = _recv_exact(sock, n_name).decode()
    return req_id, name, _recv_exact(sock, _recv_len(sock))


def _send_response(sock: socket.socket, req_id: int, ok: bool, payload: bytes) -> None:
    if len(payload) > MAX_RPC_MSG_SIZE:
        raise SizeMismatch("RPC message of %d bytes exceeds the 1 GiB cap" % len(payload))
    sock.sendall(struct.pack("<QBQ", req_id, 0 if ok else 1, len(payload)) + payload)


def _recv_response(sock: socket.socket):
    req_id, status = struct.unpack("<QB", _recv_exact(sock, 9))
    return req_id, status == 0, _recv_exact(sock, _recv_len(sock))


class _ByteSource:
    """``recv`` over a bytes object, so that the frame parsers also read frames held in memory."""

    def __init__(self, data: bytes):
        self._data, self._pos = bytes(data), 0

    def recv(self, n: int) -> bytes:
        out = self._data[self._pos:self._pos + n]
        self._pos += len(out)
        return out


class _ByteSink:
    def __init__(self):
        self.data = bytearray()

    def sendall(self, b: bytes) -> None:
        self.data += b


def encode_rpc_request(req_id: int, fn_name: str, *args, **kwargs) -> bytes:
    """One request frame (what ``rpc_sync`` puts on the wire) as bytes."""
    sink = _ByteSink()
    _send_request(sink, req_id, fn_name, _encode((list(args), kwargs)))
    return bytes(sink.data)


def decode_rpc_response(frame: bytes):
    """``(request id, ok, value)`` of a response frame."""
    req_id, ok, body = _recv_response(_ByteSource(frame))
    return req_id, ok, _decode(body)


class RpcAgent:
    """Serve registered handlers on a TCP port and call handlers of other agents by name.  ``rank`` /
    ``world_size`` label the agent inside a job (the reference's agent sits on a rank-addressed
    back-end, ferrotorch-distributed/src/rpc.rs:372-610; this one is addressed by ``(host, port)``)."""

    def __init__(self, name: str, host: str = "127.0.0.1", port: int = 0, rank: int = 0, world_size: int = 1):
        if not 0 <= rank < world_size:
            raise InvalidRank("rank %d outside a world of %d" % (rank, world_size))
        self._rank, self._world = rank, world_size
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

    def rank(self) -> int:
        return self._rank

    def world_size(self) -> int:
        return self._world

    def handle_request(self, src_rank: int, request_data: bytes) -> bytes:
        """Server-side dispatch of one request frame held in memory (rpc.rs:561): looks the handler up,
        runs it, and returns the response frame that would go back to ``src_rank``.  Failures (unknown
        handler, handler exception, malformed frame) come back as an error response, not as an exception."""
        req_id = 0
        try:
            req_id, fn_name, payload = _recv_request(_ByteSource(request_data))
            if fn_name not in self.handlers:
                ok, res = False, "no handler %r on %s (request from rank %d)" % (fn_name, self.name, src_rank)
            else:
                args, kwargs = _decode(payload)
                ok, res = True, self.handlers[fn_name](*args, **kwargs)
        except BaseException as e:  # noqa: BLE001 - reported to the caller in the response
            ok, res = False, repr(e)
        sink = _ByteSink()
        try:
            body = _encode(res)
        except TypeError as e:
            ok, body = False, _encode("handler result cannot be sent: %s" % e)
        _send_response(sink, req_id, ok, body)
        return bytes(sink.data)

    def _serve(self):
        while not self._stop:
            try:
                conn, _ = self._srv.accept()
            except OSError:
                return
            threading.Thread(target=self._handle, args=(conn,), daemon=True).start()

    def _handle(self, conn):
        with conn:
            req_id = 0
            try:
                req_id, fn_name, payload = _recv_request(conn)
                if fn_name not in self.handlers:
                    ok, res = False, "no handler %r on %s" % (fn_name, self.name)
                else:
                    args, kwargs = _decode(payload)
                    ok, res = True, self.handlers[fn_name](*args, **kwargs)
            except BaseException as e:  # noqa: BLE001
                ok, res = False, repr(e)
            try:
                try:
                    body = _encode(res)
                except TypeError as e:
                    ok, body = False, _encode("handler result cannot be sent: %s" % e)
                _send_response(conn, req_id, ok, body)
            except OSError:
                pass

    _next_id = [0]
    _id_lock = threading.Lock()

    @staticmethod
    def rpc_sync(address, fn_name: str, *args, timeout: float = 60.0, **kwargs):
        with RpcAgent._id_lock:
            RpcAgent._next_id[0] += 1
            req_id = RpcAgent._next_id[0]
        with socket.create_connection(address, timeout=timeout) as s:
            _send_request(s, req_id, fn_name, _encode((list(args), kwargs)))
            got_id, ok, body = _recv_response(s)
        if got_id != req_id:
            raise RuntimeError("remote call %s: response for request %d, expected %d" % (fn_name, got_id, req_id))
        val = _decode(body)
        if not ok:
            raise RuntimeError("remote call %s failed: %s" % (fn_name, val))
        return val

    @staticmethod
    def rpc_async(address, fn_name: str, *args, **kwargs) -> PendingCollective:
        return PendingCollective(lambda: RpcAgent.rpc_sync(address, fn_name, *args, **kwargs))

    def shutdown(self):
        self._stop = True
        self._srv.close()


class TcpRpcBackend:
    """Rank-addressed byte messages over a :class:`~.backend.Group` (ferrotorch-distributed/src/rpc.rs:282-350):
    what the reference's RPC agent sits on.  ``send`` frames nothing itself -- the receiver asks for exactly
    the bytes it expects, as the group's tensor transport does."""

    def __init__(self, group: Group):
        self.group = group

    def rank(self) -> int:
        return self.group.rank

    def world_size(self) -> int:
        return self.group.world_size

    def send(self, data: bytes, dst_rank: int) -> None:
        if not 0 <= dst_rank < self.group.world_size or dst_rank == self.group.rank:
            raise InvalidRank("cannot send to rank %d from rank %d of %d" % (dst_rank, self.group.rank, self.group.world_size))
        self.group.send(torch.frombuffer(bytearray(data), dtype=torch.uint8), dst_rank)

    def recv(self, nbytes: int, src_rank: int, timeout: float | None = None) -> bytes:
        if not 0 <= src_rank < self.group.world_size or src_rank == self.group.rank:
            raise InvalidRank("cannot receive from rank %d on rank %d of %d" % (src_rank, self.group.rank, self.group.world_size))
        buf = torch.empty(nbytes, dtype=torch.uint8)
        self.group.recv(buf, src_rank, timeout) if timeout is not None else self.group.recv(buf, src_rank)
        return bytes(buf.numpy())


class GroupRpcAgent:
    """Remote calls between the ranks of a :class:`~.backend.Group` (the reference's agent sits on its rank-addressed
    back-end the same way, ferrotorch-distributed/src/rpc.rs:372-610).  Every message is one frame
    ``kind (1 byte: 0 request, 1 response) + length + body`` sent with the group's point-to-point transport.

    Calls are correlated by request id: several threads of one rank may call the same peer at once, the
    responses may come back in any order (``serve(..., concurrent=True)`` answers every request on its own thread),
    and a response that arrives while another call is receiving is kept for its owner.  A request that arrives
    while this rank waits for a response is served on the spot, so two ranks may call each other at the same time."""

    def __init__(self, group: Group, name: str | None = None):
        self.group, self.name = group, name or "rank%d" % group.rank
        self.transport = TcpRpcBackend(group)
        self.handlers: dict = {}
        self._counter = 0
        self._id_lock = threading.Lock()
        self._buffered: dict = {}
        self._buf_lock = threading.Lock()
        self._send_locks = {r: threading.Lock() for r in range(group.world_size)}
        self._recv_locks = {r: threading.Lock() for r in range(group.world_size)}

    def rank(self) -> int:
        return self.group.rank

    def world_size(self) -> int:
        return self.group.world_size

    def register(self, fn_name: str, fn) -> None:
        self.handlers[fn_name] = fn

    # ---- frames
    def _send(self, dst: int, kind: int, body: bytes) -> None:
        if len(body) > MAX_RPC_MSG_SIZE:
            raise SizeMismatch("RPC message of %d bytes exceeds the 1 GiB cap" % len(body))
        with self._send_locks[dst]:
            self.transport.send(bytes([kind]) + struct.pack("<Q", len(body)), dst)
            self.transport.send(body, dst)

    def _recv(self, src: int, timeout: float | None):
        head = self.transport.recv(9, src, timeout)
        (n,) = struct.unpack("<Q", head[1:])
        if n > MAX_RPC_MSG_SIZE:
            raise SizeMismatch("RPC frame of %d bytes exceeds the 1 GiB cap" % n)
        return head[0], self.transport.recv(n, src, timeout)

    def _answer(self, src: int, request: bytes) -> None:
        helper = RpcAgent.__new__(RpcAgent)
        helper.handlers, helper.name = self.handlers, self.name
        self._send(src, 1, RpcAgent.handle_request(helper, src, request))

    # ---- client side
    def rpc_sync(self, dst_rank: int, fn_name: str, *args, timeout: float | None = 60.0, **kwargs):
        if not 0 <= dst_rank < self.group.world_size or dst_rank == self.group.rank:
            raise InvalidRank("rpc_sync: cannot call rank %d from rank %d of %d" % (dst_rank, self.group.rank, self.group.world_size))
        with self._id_lock:
            self._counter += 1
            req_id = (self.group.rank << 40) | self._counter
        self._send(dst_rank, 0, encode_rpc_request(req_id, fn_name, *args, **kwargs))
        ok, val = self._await(dst_rank, req_id, timeout)
        if not ok:
            raise RuntimeError("remote call %s on rank %d failed: %s" % (fn_name, dst_rank, val))
        return val

    def rpc_async(self, dst_rank: int, fn_name: str, *args, **kwargs) -> PendingCollective:
        return PendingCollective(lambda: self.rpc_sync(dst_rank, fn_name, *args, **kwargs), op_name="rpc:" + fn_name)

    def _take_buffered(self, req_id: int):
        with self._buf_lock:
            return self._buffered.pop(req_id, None)

    def _await(self, src: int, req_id: int, timeout: float | None):
        import time

        deadline = None if timeout is None else time.time() + timeout
        while True:
            got = self._take_buffered(req_id)
            if got is not None:
                return got
            if not self._recv_locks[src].acquire(timeout=0.01):
                if deadline is not None and time.time() > deadline:
                    raise TimeoutError("rpc: no response from rank %d within %.1f s" % (src, timeout))
                continue                               # another call of this rank is receiving; it will file our response
            try:
                got = self._take_buffered(req_id)
                if got is not None:
                    return got
                kind, body = self._recv(src, None if deadline is None else max(0.01, deadline - time.time()))
            finally:
                self._recv_locks[src].release()
            if kind == 0:
                self._answer(src, body)                # the peer is calling us while we wait for it
                continue
            rid, ok, val = decode_rpc_response(body)
            if rid == req_id:
                return ok, val
            with self._buf_lock:
                self._buffered[rid] = (ok, val)

    # ---- server side
    def serve(self, src_rank: int, count: int = 1, concurrent: bool = False, timeout: float | None = 60.0) -> None:
        """Answer ``count`` requests from ``src_rank``; ``concurrent`` runs every handler on its own thread, so a
        slow call does not hold back the ones behind it."""
        threads = []
        served = 0
        while served < count:
            with self._recv_locks[src_rank]:
                kind, body = self._recv(src_rank, timeout)
            if kind == 1:                              # a response for one of this rank's own calls
                rid, ok, val = decode_rpc_response(body)
                with self._buf_lock:
                    self._buffered[rid] = (ok, val)
                continue
            served += 1
            if concurrent:
                t = threading.Thread(target=self._answer, args=(src_rank, body), daemon=True)
                t.start()
                threads.append(t)
            else:
                self._answer(src_rank, body)
        for t in threads:
            t.join()
