"""State-dict and checkpoint formats.

Covers the reference's ``ferrotorch-serialize``:

* SafeTensors single / sharded (``model.safetensors.index.json``) / filtered load and save,
  optional down-cast on load (safetensors_io.rs:129-916);
* PyTorch ``.pt`` / ``.bin`` import and export (pytorch_import.rs:938, pytorch_export.rs:235) --
  ``torch.load(weights_only=True)`` is the pickle VM here;
* the native state-dict format: JSON-lines header, ``\\n---\\n``, raw little-endian bytes
  (state_dict.rs:1-17, 74, 176);
* training checkpoints: three length-prefixed sections -- metadata JSON, optimizer-state JSON,
  binary state dict (checkpoint.rs:1-17, 59-123) -- plus an asynchronous writer that snapshots
  to pinned host memory and writes on a thread (checkpoint.rs:575).
"""
from __future__ import annotations

from dataclasses import dataclass
import json
import os
import struct
import threading
from typing import Callable

import torch

_DT = {"F32": torch.float32, "F64": torch.float64, "F16": torch.float16, "BF16": torch.bfloat16,
       "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
       "BOOL": torch.bool}
_DT_INV = {v: k for k, v in _DT.items()}


# --------------------------------------------------------------------------- SafeTensors
def save_safetensors(state: dict[str, torch.Tensor], path: str, metadata: dict | None = None) -> None:
    from safetensors.torch import save_file

    save_file({k: v.detach().contiguous().cpu() for k, v in state.items()}, path, metadata=metadata)


def load_safetensors(path: str, device="cpu", dtype: torch.dtype | None = None,
                     key_filter: Callable[[str], bool] | None = None) -> dict[str, torch.Tensor]:
    """Memory-mapped load; ``key_filter`` selects tensors, ``dtype`` down-casts floating tensors."""
    from safetensors import safe_open

    out = {}
    with safe_open(path, framework="pt", device=str(device)) as f:
        for k in f.keys():
            if key_filter is not None and not key_filter(k):
                continue
            t = f.get_tensor(k)
            if dtype is not None and t.is_floating_point():
                t = t.to(dtype)
            out[k] = t
    return out


_ST_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
              "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}


def read_safetensors_header(path: str) -> tuple[dict, int]:
    """``(header, data_offset)`` of a SafeTensors file: 8 bytes little-endian header length, the
    JSON header (``name -> {dtype, shape, data_offsets}`` plus ``__metadata__``), then the data."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError("safetensors: %s is shorter than its length field" % path)
        n = int.from_bytes(raw, "little")
        if n <= 0 or 8 + n > size:
            raise ValueError("safetensors: header length %d in a %d-byte file" % (n, size))
        header = json.loads(f.read(n))
    return header, 8 + n


def load_safetensors_parallel(path: str, device="cpu", dtype: torch.dtype | None = None,
                              key_filter: Callable[[str], bool] | None = None, threads: int = 8) -> dict[str, torch.Tensor]:
    """The eager counterpart of :func:`load_safetensors` for checkpoints that go to a GPU anyway:
    the span of the file that holds the selected tensors is read by ``threads`` positional reads
    into one (page-locked) buffer, the tensors are views into it, and their copies to ``device`` are
    asynchronous.  Offsets, sizes and dtypes of the header are validated before anything is read."""
    header, base = read_safetensors_header(path)
    size = os.path.getsize(path)
    want = {}
    for k, e in header.items():
        if k == "__metadata__" or (key_filter is not None and not key_filter(k)):
            continue
        dt = _ST_DTYPES.get(e.get("dtype"))
        if dt is None:
            raise ValueError("safetensors: dtype %r of %s is not supported" % (e.get("dtype"), k))
        lo, hi = (int(v) for v in e["data_offsets"])
        numel = 1
        for d in e["shape"]:
            numel *= int(d)
        if lo < 0 or hi < lo or base + hi > size or numel * torch.empty(0, dtype=dt).element_size() != hi - lo:
            raise ValueError("safetensors: tensor %s: offsets [%d, %d) do not fit shape %s / file size" % (k, lo, hi, e["shape"]))
        want[k] = (dt, [int(d) for d in e["shape"]], lo, hi)
    if not want:
        return {}
    first, last = min(v[2] for v in want.values()), max(v[3] for v in want.values())
    dev = torch.device(device)
    buf = read_file_parallel(path, base + first, last - first, threads=threads, pin=dev.type == "cuda")
    out = {}
    for k, (dt, shape, lo, hi) in want.items():
        if hi == lo:
            t = torch.empty(shape, dtype=dt)
        else:
            t8 = buf[lo - first:hi - first]
            item = torch.empty(0, dtype=dt).element_size()
            t = (t8 if t8.data_ptr() % item == 0 else t8.clone()).view(dt).reshape(shape)
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        out[k] = t.to(dev, non_blocking=True) if dev.type != "cpu" else t
    if dev.type == "cuda":
        torch.cuda.current_stream(dev).synchronize()      # the page-locked buffer is released after this call
    return out


def save_safetensors_sharded(state: dict[str, torch.Tensor], directory: str, max_shard_bytes: int = 5 << 30,
                             prefix: str = "model") -> str:
    """Write ``prefix-0000i-of-0000n.safetensors`` + ``prefix.safetensors.index.json``."""
    os.makedirs(directory, exist_ok=True)
    shards, cur, cur_bytes = [], {}, 0
    for k, v in state.items():
        nb = v.numel() * v.element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = v
        cur_bytes += nb
    if cur:
        shards.append(cur)
    weight_map, total = {}, 0
    for i, sh in enumerate(shards):
        name = "%s-%05d-of-%05d.safetensors" % (prefix, i + 1, len(shards))
        save_safetensors(sh, os.path.join(directory, name))
        for k, v in sh.items():
            weight_map[k] = name
            total += v.numel() * v.element_size()
    index = os.path.join(directory, prefix + ".safetensors.index.json")
    with open(index, "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1)
    return index


def load_safetensors_sharded(index_path: str, device="cpu", dtype: torch.dtype | None = None,
                             key_filter: Callable[[str], bool] | None = None,
                             progress: Callable[[int, int], None] | None = None) -> dict[str, torch.Tensor]:
    with open(index_path) as f:
        index = json.load(f)
    by_file: dict[str, list[str]] = {}
    for k, fn in index["weight_map"].items():
        if key_filter is None or key_filter(k):
            by_file.setdefault(fn, []).append(k)
    out, base = {}, os.path.dirname(index_path)
    for i, (fn, keys) in enumerate(sorted(by_file.items())):
        ks = set(keys)
        out.update(load_safetensors(os.path.join(base, fn), device, dtype, lambda k: k in ks))
        if progress is not None:
            progress(i + 1, len(by_file))
    return out


@dataclass
class ShardProgress:
    """Passed to the progress callback of :func:`load_safetensors_sharded_with_progress`."""
    shard_index: int
    shard_count: int
    shard_file: str
    tensors_loaded: int


def load_safetensors_mmap(path: str, device="cpu", **kw) -> dict[str, torch.Tensor]:
    """Same as :func:`load_safetensors`: the file is always memory-mapped (safetensors_io.rs)."""
    return load_safetensors(path, device, **kw)


def load_safetensors_sharded_filtered(index_path: str, key_filter: Callable[[str], bool], device="cpu",
                                      dtype: torch.dtype | None = None) -> dict[str, torch.Tensor]:
    """Only the tensors ``key_filter`` accepts; shards without any of them are not opened."""
    return load_safetensors_sharded(index_path, device, dtype, key_filter)


load_safetensors_sharded_mmap = load_safetensors_sharded


def load_safetensors_sharded_with_progress(index_path: str, on_progress: Callable[[ShardProgress], None],
                                           device="cpu", dtype: torch.dtype | None = None) -> dict[str, torch.Tensor]:
    with open(index_path) as f:
        files = sorted(set(json.load(f)["weight_map"].values()))
    out, base = {}, os.path.dirname(index_path)
    for i, fn in enumerate(files):
        out.update(load_safetensors(os.path.join(base, fn), device, dtype))
        on_progress(ShardProgress(i, len(files), fn, len(out)))
    return out


def load_safetensors_auto(path: str, device="cpu", dtype: torch.dtype | None = None) -> dict[str, torch.Tensor]:
    """A ``.safetensors`` file, a ``*.index.json`` of a sharded checkpoint, or a directory that
    holds ``model.safetensors`` or ``model.safetensors.index.json``."""
    if os.path.isdir(path):
        for cand in ("model.safetensors.index.json", "model.safetensors"):
            if os.path.exists(os.path.join(path, cand)):
                return load_safetensors_auto(os.path.join(path, cand), device, dtype)
        raise FileNotFoundError("no model.safetensors[.index.json] under %s" % path)
    if path.endswith(".json"):
        return load_safetensors_sharded(path, device, dtype)
    return load_safetensors(path, device, dtype)


def validate_checkpoint(path: str) -> dict:
    """Check that a ``.pt`` / ``.bin`` file is a plain state dict a safe loader accepts (tensors
    only, no arbitrary pickled objects); returns ``{"tensors", "parameters", "dtypes"}``
    (pytorch_export.rs ``validate_checkpoint``)."""
    sd = load_pytorch_state_dict(path)
    if not sd:
        raise ValueError("%s holds no tensors" % path)
    return {"tensors": len(sd), "parameters": sum(v.numel() for v in sd.values()),
            "dtypes": sorted({str(v.dtype) for v in sd.values()})}


# --------------------------------------------------------------------------- PyTorch .pt
def load_pytorch_state_dict(path: str, device="cpu") -> dict[str, torch.Tensor]:
    sd = torch.load(path, map_location=device, weights_only=True)
    if isinstance(sd, dict) and "state_dict" in sd and isinstance(sd["state_dict"], dict):
        sd = sd["state_dict"]
    return {k: v for k, v in sd.items() if isinstance(v, torch.Tensor)}


def load_pytorch_state_dict_mmap(path: str) -> dict[str, torch.Tensor]:
    """The same with the tensor data memory-mapped from the file instead of read into memory
    (zip-format checkpoints only; pytorch_import.rs ``load_pytorch_state_dict_mmap``)."""
    sd = torch.load(path, map_location="cpu", weights_only=True, mmap=True)
    if isinstance(sd, dict) and "state_dict" in sd and isinstance(sd["state_dict"], dict):
        sd = sd["state_dict"]
    return {k: v for k, v in sd.items() if isinstance(v, torch.Tensor)}


def parse_pickle(data: bytes) -> list[tuple[str, object]]:
    """The opcodes of a pickle stream as ``(name, argument)`` pairs, without executing anything:
    for inspecting what a checkpoint would import before loading it (the reference walks the same
    stream with its own pickle machine, pytorch_import.rs:154)."""
    import pickletools

    try:
        return [(op.name, arg) for op, arg, _ in pickletools.genops(data)]
    except Exception as e:  # noqa: BLE001
        raise ValueError("not a well-formed pickle stream: %s" % e)


def pickle_imports(path: str) -> list[str]:
    """``module.name`` of every global a ``.pt`` file's pickle refers to (zip or legacy format)."""
    import zipfile

    if zipfile.is_zipfile(path):
        with zipfile.ZipFile(path) as z:
            name = next(n for n in z.namelist() if n.endswith("data.pkl"))
            data = z.read(name)
    else:
        with open(path, "rb") as f:
            data = f.read()
    out, strings = [], []
    for op, arg in parse_pickle(data):
        if op == "GLOBAL":
            out.append(str(arg).replace(" ", "."))
        elif op in ("SHORT_BINUNICODE", "BINUNICODE", "UNICODE"):
            strings.append(str(arg))
        elif op == "STACK_GLOBAL" and len(strings) >= 2:
            out.append("%s.%s" % (strings[-2], strings[-1]))
    return sorted(set(out))


def save_pytorch(state: dict[str, torch.Tensor], path: str) -> None:
    torch.save({k: v.detach().cpu() for k, v in state.items()}, path)


# --------------------------------------------------------------------------- native state dict
def _to_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu().reshape(-1)
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


_TAG = {torch.float32: "f32", torch.float64: "f64", torch.float16: "f16", torch.bfloat16: "bf16",
        torch.int64: "i64", torch.int32: "i32", torch.int16: "i16", torch.int8: "i8", torch.uint8: "u8",
        torch.bool: "bool"}
_TAG_INV = {v: k for k, v in _TAG.items()}


def dumps_state_dict(state: dict[str, torch.Tensor]) -> bytes:
    """The reference's layout byte for byte (state_dict.rs:74-165): one JSON line per tensor, keys
    sorted, fields ``name, shape, dtype, byte_offset, byte_length`` without spaces, every line
    ended by a newline, then the separator, then the raw little-endian bytes.  An f32 / f64 file
    written here loads in the reference; the other dtype tags (bf16, f16, i64 ...) extend it."""
    header, blobs, off = [], [], 0
    for k in sorted(state):
        v = state[k]
        b = _to_bytes(v)
        header.append('{"name":%s,"shape":[%s],"dtype":"%s","byte_offset":%d,"byte_length":%d}\n'
                      % (json.dumps(k), ",".join(str(int(d)) for d in v.shape), _TAG[v.dtype], off, len(b)))
        blobs.append(b)
        off += len(b)
    return "".join(header).encode() + b"\n---\n" + b"".join(blobs)


def loads_state_dict(buf: bytes, device="cpu") -> dict[str, torch.Tensor]:
    """Reads the layout above, files the reference wrote, and the first layout of this package
    (fields ``offset`` / ``nbytes``, upper-case dtype names)."""
    base = None
    if isinstance(buf, torch.Tensor):           # a uint8 tensor (read_file_parallel): views come straight from it
        base = buf
        raw = memoryview(buf.numpy())
        window = 1 << 16                                    # the header is at the front: copy only as much as holds it
        while True:
            probe = bytes(raw[:min(len(raw), window)])
            if probe.startswith(b"---\n") or b"\n---\n" in probe or window >= len(raw):
                break
            window <<= 2
    else:
        if not isinstance(buf, bytearray):
            buf = bytearray(buf)                # one copy; the tensors below are views into it
        raw, probe = memoryview(buf), buf
    head_end = 0 if probe.startswith(b"---\n") else probe.find(b"\n---\n") + 1
    if head_end == 0 and not probe.startswith(b"---\n"):
        raise ValueError("state dict: no separator line")
    body_start = head_end + 4
    body = raw[body_start:]
    out = {}
    for line in bytes(probe[:head_end]).decode().splitlines():
        if not line.strip():
            continue
        e = json.loads(line)
        off = e["byte_offset"] if "byte_offset" in e else e["offset"]
        n = e["byte_length"] if "byte_length" in e else e["nbytes"]
        tag = e["dtype"]
        dt = _TAG_INV.get(tag) or _DT.get(tag)
        if dt is None:
            raise ValueError("state dict: unknown dtype %r for %s" % (tag, e["name"]))
        if off < 0 or n < 0 or off + n > len(body):
            raise ValueError("state dict: tensor %r needs bytes [%d, %d) of a %d-byte body"
                             % (e["name"], off, off + n, len(body)))
        numel = 1
        for d in e["shape"]:
            numel *= int(d)
        if numel * torch.empty(0, dtype=dt).element_size() != n:
            raise ValueError("state dict: shape %s of %r does not match %d bytes" % (e["shape"], e["name"], n))
        if n:
            t8 = (base[body_start + off:body_start + off + n] if base is not None
                  else torch.frombuffer(buf, dtype=torch.uint8, count=n, offset=body_start + off))
            item = torch.empty(0, dtype=dt).element_size()
            t = (t8 if t8.data_ptr() % item == 0 else t8.clone()).view(dt)     # views need aligned storage
        else:
            t = torch.empty(0, dtype=dt)
        out[e["name"]] = t.reshape(e["shape"]).to(device)
    return out


def save_state_dict(state: dict[str, torch.Tensor], path: str, align: int = 64) -> None:
    """Streams: the header first, then every tensor's bytes straight from its storage (no
    concatenated copy of the whole checkpoint in memory).  With ``align`` the last header line is
    padded with spaces (insignificant JSON white space, also for the reference's reader) so that
    the tensor bytes start on an ``align``-byte file offset, and every tensor is placed on a
    multiple of 8 bytes: a loader can then hand out views of one buffer or of a memory map without
    copying.  ``align=0`` writes the dense layout of :func:`dumps_state_dict`."""
    keys = sorted(state)
    header, off, views = [], 0, []
    for k in keys:
        v = state[k].detach().contiguous().cpu()
        nbytes = v.numel() * v.element_size()
        if align and off % 8:
            views.append(torch.zeros(8 - off % 8, dtype=torch.uint8))           # gap: no header entry points at it
            off += 8 - off % 8
        header.append('{"name":%s,"shape":[%s],"dtype":"%s","byte_offset":%d,"byte_length":%d}\n'
                      % (json.dumps(k), ",".join(str(int(d)) for d in v.shape), _TAG[v.dtype], off, nbytes))
        views.append(v)
        off += nbytes
    head = "".join(header).encode()
    if align and header:
        pad = -(len(head) + 5) % align                                         # + len("\n---\n")
        head = head[:-1] + b" " * pad + b"\n"
    # one streaming writer: positional writes from several threads were measured slower than this
    # on a memory-backed file system (2.4 GB/s streamed against 0.4-1.0 GB/s with eight writers)
    with open(path, "wb") as f:
        f.write(head + b"\n---\n")
        for v in views:
            if v.numel():
                f.write(memoryview(v.reshape(-1).view(torch.uint8).numpy()))


def read_file_parallel(path: str, offset: int = 0, nbytes: int | None = None, threads: int = 8, pin: bool = False) -> torch.Tensor:
    """``nbytes`` of ``path`` from ``offset`` as one uint8 tensor, filled by ``threads`` positional
    reads of the native host library (``csrc/host/io_parallel.cpp``); ``pin`` allocates page-locked
    memory so that a following copy to a GPU is asynchronous.  Falls back to one ``readinto``
    when the library is not available."""
    import ctypes

    from .. import _native

    size = os.path.getsize(path)
    nbytes = size - offset if nbytes is None else nbytes
    if offset < 0 or nbytes < 0 or offset + nbytes > size:
        raise ValueError("read_file_parallel: bytes [%d, %d) of a %d-byte file" % (offset, offset + nbytes, size))
    out = torch.empty(nbytes, dtype=torch.uint8, pin_memory=pin and torch.cuda.is_available())
    if nbytes == 0:
        return out
    lib = _native.host(required=False)
    if lib is None or not hasattr(lib, "ftio_read"):
        with open(path, "rb") as f:
            f.seek(offset)
            f.readinto(memoryview(out.numpy()))
        return out
    lib.ftio_read.restype = ctypes.c_int
    lib.ftio_read.argtypes = [ctypes.c_char_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int]
    rc = lib.ftio_read(os.fsencode(path), offset, nbytes, out.data_ptr(), int(threads))
    if rc != 0:
        raise OSError(-rc if rc < -1 else 5, "reading %s failed (%d)" % (path, rc))
    return out


def load_state_dict(path: str, device="cpu", threads: int = 8, mmap: bool = False) -> dict[str, torch.Tensor]:
    """The file is read once, in parallel, into one buffer (page-locked when ``device`` is a GPU);
    the tensors are views into it (``device='cpu'``) or asynchronous copies from it.  ``mmap=True``
    maps the file instead (private, copy-on-write): nothing is read until a tensor is touched, and
    the tensors stay valid only while the file does."""
    if mmap and os.path.getsize(path) > 0:
        buf = torch.from_file(path, shared=False, size=os.path.getsize(path), dtype=torch.uint8)
    else:
        buf = read_file_parallel(path, threads=threads, pin=torch.device(device).type == "cuda")
    return loads_state_dict(buf, device)


# --------------------------------------------------------------------------- training checkpoint
MAGIC = b"FTCK1\n"


def _flatten_opt(obj, prefix=""):
    """Split an optimizer state into JSON-able scalars and a tensor dict."""
    tensors, meta = {}, None
    if isinstance(obj, torch.Tensor):
        tensors[prefix] = obj
        meta = {"__tensor__": prefix}
    elif isinstance(obj, dict):
        meta = {}
        for k, v in obj.items():
            t, m = _flatten_opt(v, "%s/%s" % (prefix, k) if prefix else str(k))
            tensors.update(t)
            meta[str(k)] = m
    elif isinstance(obj, (list, tuple)):
        meta = []
        for i, v in enumerate(obj):
            t, m = _flatten_opt(v, "%s/%d" % (prefix, i))
            tensors.update(t)
            meta.append(m)
    else:
        meta = obj
    return tensors, meta


def _unflatten_opt(meta, tensors):
    if isinstance(meta, dict):
        if "__tensor__" in meta and len(meta) == 1:
            return tensors[meta["__tensor__"]]
        return {(int(k) if k.lstrip("-").isdigit() else k): _unflatten_opt(v, tensors) for k, v in meta.items()}
    if isinstance(meta, list):
        return [_unflatten_opt(v, tensors) for v in meta]
    return meta


def save_checkpoint(path: str, model_state: dict[str, torch.Tensor], optimizer_state: dict | None = None,
                    epoch: int = 0, step: int = 0, extra: dict | None = None) -> None:
    """``TrainingCheckpoint`` (model + optimizer + epoch + step + extra such as scaler / RNG state)."""
    opt_tensors, opt_meta = _flatten_opt(optimizer_state or {})
    sections = [json.dumps({"epoch": epoch, "step": step, "extra": extra or {}}).encode(),
                json.dumps(opt_meta).encode(),
                dumps_state_dict({**{"model/" + k: v for k, v in model_state.items()},
                                  **{"optim/" + k: v for k, v in opt_tensors.items()}})]
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(MAGIC)
        for s in sections:
            f.write(struct.pack("<Q", len(s)))
            f.write(s)
    os.replace(tmp, path)


def _read_sections(f, path: str, n_sections: int = 3) -> list[bytes]:
    size = os.fstat(f.fileno()).st_size
    secs = []
    for _ in range(n_sections):
        head = f.read(8)
        if len(head) != 8:
            raise ValueError("%s: truncated checkpoint (section length)" % path)
        (n,) = struct.unpack("<Q", head)
        if n > size - f.tell():
            raise ValueError("%s: a section claims %d bytes, the file has %d left" % (path, n, size - f.tell()))
        secs.append(f.read(n))
    return secs


def save_reference_checkpoint(path: str, model_state: dict[str, torch.Tensor],
                              optimizer_state: dict[str, dict[str, list[float]]] | None = None,
                              epoch: int = 0, step: int = 0) -> None:
    """A checkpoint in the reference's own ``.ftc`` layout (checkpoint.rs:1-17, 86-123): three
    sections with 8-byte little-endian lengths -- ``{"epoch":E,"step":S}``, the optimizer state
    as ``{param: {slot: [floats]}}`` with sorted keys, and the state-dict bytes.  No magic, no
    extras: use it to hand a model back to the reference."""
    opt = optimizer_state or {}
    opt_json = "{%s}" % ",".join(
        '%s:{%s}' % (json.dumps(k), ",".join('%s:[%s]' % (json.dumps(ik), ",".join(repr(float(x)) for x in opt[k][ik]))
                                             for ik in sorted(opt[k]))) for k in sorted(opt))
    sections = [('{"epoch":%d,"step":%d}' % (epoch, step)).encode(), opt_json.encode(), dumps_state_dict(model_state)]
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        for sec in sections:
            f.write(struct.pack("<Q", len(sec)))
            f.write(sec)
    os.replace(tmp, path)


def load_checkpoint(path: str, device="cpu") -> dict:
    """Loads a checkpoint of this package (magic ``FTCK1``) or one the reference wrote (no magic:
    the file starts with the length of its metadata JSON)."""
    with open(path, "rb") as f:
        if f.read(len(MAGIC)) != MAGIC:
            f.seek(0)
            meta_b, opt_b, sd_b = _read_sections(f, path)
            try:
                meta, opt = json.loads(meta_b), json.loads(opt_b)
            except ValueError as e:
                raise ValueError("%s is neither a ferrotorch_b200 nor a ferrotorch checkpoint: %s" % (path, e))
            return {"model": loads_state_dict(sd_b, device), "optimizer": opt, "epoch": int(meta["epoch"]),
                    "step": int(meta["step"]), "extra": {}}
        secs = []
        for _ in range(3):
            (n,) = struct.unpack("<Q", f.read(8))
            secs.append(f.read(n))
    meta, opt_meta = json.loads(secs[0]), json.loads(secs[1])
    tensors = loads_state_dict(secs[2], device)
    model = {k[6:]: v for k, v in tensors.items() if k.startswith("model/")}
    opt_t = {k[6:]: v for k, v in tensors.items() if k.startswith("optim/")}
    return {"model": model, "optimizer": _unflatten_opt(opt_meta, opt_t), "epoch": meta["epoch"],
            "step": meta["step"], "extra": meta["extra"]}


@dataclass
class TrainingCheckpoint:
    """Model + optimizer + progress in one object (ferrotorch-serialize/src/checkpoint.rs:59);
    ``save`` / ``load`` are :func:`save_checkpoint` / :func:`load_checkpoint`."""
    model_state: dict
    optimizer_state: dict | None = None
    epoch: int = 0
    step: int = 0
    extra: dict | None = None

    def save(self, path: str) -> None:
        save_checkpoint(path, self.model_state, self.optimizer_state, self.epoch, self.step, self.extra)

    @classmethod
    def load(cls, path: str, device="cpu") -> "TrainingCheckpoint":
        d = load_checkpoint(path, device)
        return cls(d["model"], d["optimizer"], int(d["epoch"]), int(d["step"]), d.get("extra") or {})


PickleValue = object      # what ``parse_pickle`` yields as values: plain Python objects and tensor stubs


class CheckpointFuture:
    def __init__(self, thread: threading.Thread, box: list):
        self._t, self._box = thread, box

    def is_done(self) -> bool:
        return not self._t.is_alive()

    def wait(self) -> None:
        self._t.join()
        if self._box:
            raise self._box[0]


class AsyncCheckpointer:
    """Snapshot tensors to (pinned) host memory on the caller's thread, write the file on a
    background thread (checkpoint.rs:575; distributed variant checkpoint.rs:686-910)."""

    def __init__(self):
        self._last: CheckpointFuture | None = None

    def save_async(self, path: str, model_state: dict, optimizer_state: dict | None = None, **kw) -> CheckpointFuture:
        if self._last is not None:
            self._last.wait()

        def snap(o):
            if isinstance(o, torch.Tensor):
                h = torch.empty(o.shape, dtype=o.dtype, device="cpu", pin_memory=o.is_cuda)
                h.copy_(o.detach(), non_blocking=o.is_cuda)
                return h
            if isinstance(o, dict):
                return {k: snap(v) for k, v in o.items()}
            if isinstance(o, (list, tuple)):
                return [snap(v) for v in o]
            return o

        m, opt = snap(model_state), snap(optimizer_state)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        box: list = []

        def work():
            try:
                save_checkpoint(path, m, opt, **kw)
            except BaseException as e:  # noqa: BLE001
                box.append(e)

        t = threading.Thread(target=work, daemon=True)
        t.start()
        self._last = CheckpointFuture(t, box)
        return self._last

    # checkpoint.rs:575-680 names
    save = save_async

    def is_saving(self) -> bool:
        return self._last is not None and not self._last.is_done()

    def wait(self) -> None:
        """Block until the last save has been written (re-raises its error, if any)."""
        if self._last is not None:
            self._last.wait()
