"""GGUF checkpoints: native mmap reader (``csrc/host/gguf.cpp``), dequantisation, the
GGUF -> HF key map for Llama, and a small writer / Q4_0 quantiser used by tests and benchmarks.

Reference: ferrotorch-serialize/src/gguf.rs:56-927 (types, block layouts, ``load_gguf_state_dict``)
and ferrotorch-llama/src/gguf_remap.rs:23-52 (``token_embd -> model.embed_tokens``, ``blk.{i}.attn_q
-> model.layers.{i}.self_attn.q_proj`` ...).

Element order of the 4- and 5-bit block formats: the default (``nibble_order="ggml"``) is the file
format's, as llama.cpp writes it -- byte j of a block carries element j (low nibble) and element
j + 16 (high nibble).  The reference's decoders emit the nibbles of byte j as elements 2j, 2j + 1
(gguf.rs:543-577; ferrotorch-cubecl/src/quant.rs:348); ``nibble_order="interleaved"`` reproduces
that for bit-for-bit agreement with tensors the reference decoded.
"""
from __future__ import annotations

import ctypes
import json
import os
import re
import struct

import numpy as np
import torch

from .. import _native

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q5_0, GGML_Q5_1, GGML_Q8_0, GGML_Q8_1, GGML_BF16 = 0, 1, 2, 3, 6, 7, 8, 9, 30
_BLOCK = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2), GGML_Q4_0: (32, 18), GGML_Q4_1: (32, 20),
          GGML_Q5_0: (32, 22), GGML_Q5_1: (32, 24), GGML_Q8_0: (32, 34), GGML_Q8_1: (32, 36)}
_ready = False


def _lib():
    global _ready
    lib = _native.host()
    if not _ready:
        vp, ll, cp = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_char_p
        lib.ftg_open.restype, lib.ftg_open.argtypes = vp, [cp]
        lib.ftg_error.restype, lib.ftg_error.argtypes = cp, [vp]
        lib.ftg_close.argtypes = [vp]
        lib.ftg_version.argtypes = [vp]
        lib.ftg_n_tensors.restype, lib.ftg_n_tensors.argtypes = ll, [vp]
        lib.ftg_metadata_json.restype, lib.ftg_metadata_json.argtypes = cp, [vp]
        lib.ftg_tensor_name.restype, lib.ftg_tensor_name.argtypes = cp, [vp, ll]
        lib.ftg_tensor_info.argtypes = [vp, ll, vp]
        lib.ftg_tensor_data.restype, lib.ftg_tensor_data.argtypes = vp, [vp, ll]
        lib.ftg_dequantize.argtypes = [ctypes.c_uint, vp, vp, ll]
        lib.ftg_split_q4_0.argtypes = [vp, ll, ll, vp, vp]
        lib.ftg_dequantize_ex.argtypes = [ctypes.c_uint, vp, vp, ll, ctypes.c_int]
        lib.ftg_repack_nibbles.argtypes = [ctypes.c_uint, vp, ll, ctypes.c_int]
        lib.ftg_dequantize_pairwise.argtypes = [ctypes.c_uint, vp, vp, ll]
        _ready = True
    return lib


class GgufFile:
    """An open GGUF file.  ``tensors`` maps name -> (ggml_type, shape (outermost first), nbytes)."""

    def __init__(self, path: str):
        self._lib = _lib()
        self._h = self._lib.ftg_open(path.encode())
        err = self._lib.ftg_error(self._h)
        if err:
            msg = err.decode()
            self.close()
            raise ValueError("GGUF %s: %s" % (path, msg))
        self.version = self._lib.ftg_version(self._h)
        self.metadata = json.loads(self._lib.ftg_metadata_json(self._h).decode(errors="replace"))
        self.tensors, self._index = {}, {}
        info = (ctypes.c_ulonglong * 8)()
        for i in range(self._lib.ftg_n_tensors(self._h)):
            name = self._lib.ftg_tensor_name(self._h, i).decode()
            self._lib.ftg_tensor_info(self._h, i, info)
            nd = int(info[1])
            shape = tuple(int(info[2 + d]) for d in range(nd))[::-1]  # GGUF stores innermost first
            self.tensors[name] = (int(info[0]), shape, int(info[6]))
            self._index[name] = i

    def close(self):
        if getattr(self, "_h", None):
            self._lib.ftg_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def raw(self, name: str) -> torch.Tensor:
        """The tensor's bytes as a uint8 tensor (copied out of the mapping)."""
        t, shape, nbytes = self.tensors[name]
        ptr = self._lib.ftg_tensor_data(self._h, self._index[name])
        buf = (ctypes.c_ubyte * nbytes).from_address(ptr)
        return torch.frombuffer(bytearray(buf), dtype=torch.uint8)

    def data(self, name: str) -> memoryview:
        """The tensor's bytes as a read-only view of the file mapping (no copy; valid until ``close``)."""
        _t, _shape, nbytes = self.tensors[name]
        ptr = self._lib.ftg_tensor_data(self._h, self._index[name])
        return memoryview((ctypes.c_ubyte * nbytes).from_address(ptr)).toreadonly()

    def dequantize(self, name: str, dtype=torch.float32, nibble_order: str = "ggml") -> torch.Tensor:
        t, shape, nbytes = self.tensors[name]
        n = int(np.prod(shape)) if shape else 1
        out = torch.empty(n, dtype=torch.float32)
        rc = self._lib.ftg_dequantize_ex(t, self._lib.ftg_tensor_data(self._h, self._index[name]), out.data_ptr(), n,
                                         _order_flag(nibble_order))
        if rc != 0:
            raise ValueError("unsupported ggml type %d for %s" % (t, name))
        return out.view(shape).to(dtype)

    def q4_0_planes(self, name: str, nibble_order: str = "ggml"):
        """``(scales fp16 [rows, cols/32], nibbles uint8 [rows, cols/2])`` of a Q4_0 matrix, in the
        layout the dequant-GEMM kernel reads.  With ``nibble_order="interleaved"`` the file's bytes
        are taken to mean elements (2j, 2j+1) and are re-packed on the host first."""
        t, shape, _ = self.tensors[name]
        assert t == GGML_Q4_0 and len(shape) == 2, "%s is not a Q4_0 matrix" % name
        rows, cols = shape
        scales = torch.empty((rows, cols // 32), dtype=torch.float16)
        nib = torch.empty((rows, cols // 2), dtype=torch.uint8)
        if _order_flag(nibble_order):
            blocks = self.raw(name)
            repack_nibbles(blocks, GGML_Q4_0, to_interleaved=False)
            src = blocks.data_ptr()
        else:
            src = self._lib.ftg_tensor_data(self._h, self._index[name])
        rc = self._lib.ftg_split_q4_0(src, rows, cols, scales.data_ptr(), nib.data_ptr())
        assert rc == 0
        return scales, nib


def _order_flag(nibble_order: str) -> int:
    if nibble_order not in ("ggml", "interleaved"):
        raise ValueError("nibble_order must be 'ggml' or 'interleaved', got %r" % (nibble_order,))
    return int(nibble_order == "interleaved")


def repack_nibbles(blocks: torch.Tensor, ggml_type: int = GGML_Q4_0, to_interleaved: bool = False) -> torch.Tensor:
    """Re-pack, in place, the nibble bytes of raw Q4_0 / Q4_1 blocks (a contiguous uint8 tensor)
    between the interleaved element order and the file format's order; returns ``blocks``."""
    assert blocks.dtype == torch.uint8 and blocks.is_contiguous() and blocks.device.type == "cpu"
    bb = _BLOCK[ggml_type][1]
    assert ggml_type in (GGML_Q4_0, GGML_Q4_1) and blocks.numel() % bb == 0
    rc = _lib().ftg_repack_nibbles(ggml_type, blocks.data_ptr(), blocks.numel() // bb, int(to_interleaved))
    assert rc == 0
    return blocks


def dequantize_blocks(raw: torch.Tensor, ggml_type: int, n: int, nibble_order: str = "ggml") -> torch.Tensor:
    """Dequantise ``n`` elements from raw block bytes (uint8, CPU) to float32."""
    raw = raw.contiguous()
    be, bb = _BLOCK[ggml_type]
    if n % be or raw.numel() < n // be * bb:
        raise ValueError("%d elements of ggml type %d need %d bytes, got %d" % (n, ggml_type, n // be * bb, raw.numel()))
    out = torch.empty(n, dtype=torch.float32)
    rc = _lib().ftg_dequantize_ex(ggml_type, raw.data_ptr(), out.data_ptr(), n, _order_flag(nibble_order))
    if rc != 0:
        raise ValueError("unsupported ggml type %d" % ggml_type)
    return out


_LAYER_MAP = {"attn_norm": "input_layernorm", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj",
              "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj", "ffn_norm": "post_attention_layernorm",
              "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}
_TOP_MAP = {"token_embd": "model.embed_tokens", "output_norm": "model.norm", "output": "lm_head"}


def gguf_key_to_hf(key: str) -> str | None:
    """``blk.3.attn_q.weight`` -> ``model.layers.3.self_attn.q_proj.weight`` (None if unknown)."""
    m = re.fullmatch(r"blk\.(\d+)\.([a-z_]+)\.(weight|bias)", key)
    if m and m.group(2) in _LAYER_MAP:
        return "model.layers.%s.%s.%s" % (m.group(1), _LAYER_MAP[m.group(2)], m.group(3))
    m = re.fullmatch(r"([a-z_]+)\.(weight|bias)", key)
    if m and m.group(1) in _TOP_MAP:
        return "%s.%s" % (_TOP_MAP[m.group(1)], m.group(2))
    return None


def gguf_to_hf_state_dict(state: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Rename the keys of an already loaded GGUF state dict to the HF names; keys without a mapping
    are kept (ferrotorch-llama/src/gguf_remap.rs ``gguf_to_hf_state_dict``)."""
    return {(gguf_key_to_hf(k) or k): v for k, v in state.items()}


def load_gguf_state_dict(path: str, dtype=torch.bfloat16, remap: bool = True,
                         nibble_order: str = "ggml") -> dict[str, torch.Tensor]:
    """Dequantise every tensor to ``dtype`` (HF key names when ``remap``)."""
    out = {}
    with GgufFile(path) as f:
        for name in f.tensors:
            key = gguf_key_to_hf(name) if remap else name
            out[key or name] = f.dequantize(name, dtype, nibble_order)
    return out


# --------------------------------------------------------------------------- writer / quantiser
def quantize_q4_0(w: torch.Tensor) -> torch.Tensor:
    """Quantise a float matrix ``[rows, cols]`` (cols % 32 == 0) to Q4_0 blocks, returned as a
    uint8 tensor ``[rows * cols / 32, 18]``.  ggml rule: ``d = max_abs_signed / -8``,
    ``q = clamp(round(x / d) + 8, 0, 15)``."""
    x = w.detach().float().cpu().reshape(-1, 32)
    idx = x.abs().argmax(dim=1, keepdim=True)
    mx = x.gather(1, idx)
    d = mx / -8.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = (x * inv + 8.5).floor().clamp(0, 15).to(torch.uint8)
    packed = q[:, :16] | (q[:, 16:] << 4)
    dh = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    return torch.cat([dh, packed], dim=1).contiguous()


def _kv_bytes(key: str, value) -> bytes:
    kb = key.encode()
    out = struct.pack("<Q", len(kb)) + kb
    if isinstance(value, bool):
        return out + struct.pack("<IB", 7, int(value))
    if isinstance(value, int):
        return out + struct.pack("<II", 4, value) if 0 <= value < 2 ** 32 else out + struct.pack("<Iq", 11, value)
    if isinstance(value, float):
        return out + struct.pack("<If", 6, value)
    if isinstance(value, str):
        vb = value.encode()
        return out + struct.pack("<IQ", 8, len(vb)) + vb
    raise TypeError("unsupported metadata value %r" % (value,))


def write_gguf(path: str, tensors: dict[str, tuple[int, tuple, bytes]], metadata: dict | None = None,
               alignment: int = 32) -> None:
    """``tensors``: name -> (ggml_type, shape (outermost first), raw bytes)."""
    metadata = dict(metadata or {})
    metadata.setdefault("general.alignment", alignment)
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata))
    for k, v in metadata.items():
        head += _kv_bytes(k, v)
    off, blobs = 0, []
    for name, (t, shape, raw) in tensors.items():
        nb = name.encode()
        head += struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(shape))
        for d in reversed(shape):
            head += struct.pack("<Q", d)
        head += struct.pack("<IQ", t, off)
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad + b"".join(blobs))


# --------------------------------------------------------------------------- the reference's type and function names
import enum as _enum  # noqa: E402
from dataclasses import dataclass as _dataclass  # noqa: E402


class GgmlType(_enum.IntEnum):
    """Tensor encodings this reader understands (ferrotorch-serialize/src/gguf.rs:56)."""
    F32 = GGML_F32
    F16 = GGML_F16
    Q4_0 = GGML_Q4_0
    Q4_1 = GGML_Q4_1
    Q5_0 = GGML_Q5_0
    Q5_1 = GGML_Q5_1
    Q8_0 = GGML_Q8_0
    Q8_1 = GGML_Q8_1
    BF16 = GGML_BF16

    @property
    def block_size(self) -> int:
        """Elements per block."""
        return _BLOCK[int(self)][0]

    @property
    def type_size(self) -> int:
        """Bytes per block."""
        return _BLOCK[int(self)][1]

    def nbytes(self, n_elements: int) -> int:
        if n_elements % self.block_size:
            raise ValueError("%d elements are not a whole number of %s blocks" % (n_elements, self.name))
        return n_elements // self.block_size * self.type_size


GgufValue = object           # metadata values arrive as plain Python (int / float / bool / str / list)
GgufMetadata = dict


@_dataclass(frozen=True)
class GgufTensorInfo:
    name: str
    ggml_type: GgmlType
    shape: tuple             # outermost dimension first
    nbytes: int

    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


def tensor_infos(f: GgufFile) -> list:
    return [GgufTensorInfo(k, GgmlType(t), shape, nb) for k, (t, shape, nb) in f.tensors.items()]


def load_gguf(path: str) -> GgufFile:
    """Open a GGUF file: header, metadata and tensor directory parsed, tensor data memory-mapped."""
    return GgufFile(path)


load_gguf_mmap = load_gguf   # the reader always maps the file; the name exists for the reference's callers


def parse_gguf_bytes(data: bytes) -> GgufFile:
    """Parse a GGUF image held in memory (written to an anonymous temporary file and mapped)."""
    import tempfile

    with tempfile.NamedTemporaryFile(suffix=".gguf", delete=False) as tmp:
        tmp.write(data)
        path = tmp.name
    try:
        return GgufFile(path)
    finally:
        os.unlink(path)      # the mapping keeps the pages alive


def dequantize_gguf_tensor(f: GgufFile, name: str, dtype=torch.float32, nibble_order: str = "ggml") -> torch.Tensor:
    return f.dequantize(name, dtype, nibble_order)


def load_gguf_state_dict_mmap(path: str, dtype=torch.bfloat16, remap: bool = True, **kw) -> dict:
    return load_gguf_state_dict(path, dtype, remap, **kw)


# --------------------------------------------------------------------------- device-side dequantisation
_QUANT_TYPES = (GGML_Q4_0, GGML_Q4_1, GGML_Q5_0, GGML_Q5_1, GGML_Q8_0, GGML_Q8_1)
_native.register_protos({"ft_gguf_dequantize": (_native._i, [_native._vp, _native._vp, _native._ll, _native._i, _native._i,
                                                              _native._i, _native._vp])})


def dequantize_pairwise_host(raw: torch.Tensor, ggml_type: int, n: int) -> torch.Tensor:
    """The device kernel's decoder (``csrc/gguf_blocks.h``) run on the host: fp32 ``[n]``."""
    out = torch.empty(n, dtype=torch.float32)
    raw = raw.contiguous()
    if _lib().ftg_dequantize_pairwise(int(ggml_type), raw.data_ptr(), out.data_ptr(), n) != 0:
        raise ValueError("dequantize_pairwise_host: type %d is not a 32-element quantised block type" % ggml_type)
    return out


def dequantize_on_device(raw: torch.Tensor, ggml_type: int, shape, dtype=torch.bfloat16) -> torch.Tensor:
    """Expand raw blocks (uint8, on a CUDA device) to ``dtype`` (bf16 or fp32) on that device with
    ``ft_gguf_dequantize`` -- the quantised bytes are what crosses PCIe, not the expanded tensor."""
    if ggml_type not in _QUANT_TYPES or dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("dequantize_on_device: quantised block types to bf16 / fp32 only")
    n = 1
    for d in shape:
        n *= int(d)
    be, bb = _BLOCK[ggml_type]
    if not raw.is_cuda or raw.dtype != torch.uint8 or n % be or raw.numel() != n // be * bb:
        raise ValueError("dequantize_on_device: need %d bytes of uint8 on a CUDA device for shape %s" % (n // be * bb, tuple(shape)))
    raw = raw.contiguous()
    out = torch.empty(n, dtype=dtype, device=raw.device)
    rc = _native.kernels().ft_gguf_dequantize(raw.data_ptr(), out.data_ptr(), n // be, int(ggml_type), int(dtype == torch.float32),
                                              raw.device.index or 0, torch.cuda.current_stream().cuda_stream)
    _native.check(rc, "ft_gguf_dequantize")
    return out.view(tuple(shape))


def load_gguf_state_dict_gpu(path: str, device="cuda", dtype=torch.bfloat16, remap: bool = True) -> dict:
    """Read a GGUF file with the quantised tensors expanded on the device (the reference's
    ``from_gguf_gpu_dequant``, ferrotorch-llama/src/gpu_gguf.rs:336): raw blocks are uploaded and
    dequantised there; F32 / F16 / BF16 tensors are converted with torch."""
    out = {}
    with GgufFile(path) as f:
        for name, (t, shape, _) in f.tensors.items():
            if t in _QUANT_TYPES:
                out[name] = dequantize_on_device(f.raw(name).to(device, non_blocking=True), t, shape, dtype)
            else:
                out[name] = f.dequantize(name, torch.float32).to(device=device, dtype=dtype)
    return gguf_to_hf_state_dict(out) if remap else out
