"""Every ctypes prototype of the kernel library against the C signature it binds: same number of
parameters, pointers / 64-bit / 32-bit / float in the same places.  A mismatch would otherwise
only show on the first call on a GPU."""
import ctypes
import glob
import importlib
import os
import re

import pytest

from ferrotorch_b200 import _native

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ferrotorch_b200")


def _c_signatures() -> dict:
    sigs = {}
    for path in glob.glob(os.path.join(ROOT, "csrc", "*.cu")):
        text = re.sub(r"//[^\n]*", "", open(path).read())
        for m in re.finditer(r"FT_API\s+([\w\s\*]+?)\s*\b(ft_\w+)\s*\(([^)]*)\)\s*\{", text):
            params = [p.strip() for p in m.group(3).split(",") if p.strip() and p.strip() != "void"]
            sigs[m.group(2)] = (m.group(1).strip(), params)
    return sigs


def _kind(c_param: str) -> str:
    t = re.sub(r"\b\w+$", "", c_param).strip() if not c_param.endswith("*") else c_param     # drop the parameter name
    if "*" in t or "cudaStream_t" in t:
        return "ptr"
    if "long long" in t or "int64_t" in t or "size_t" in t or "uint64_t" in t:
        return "i64"
    if "double" in t:
        return "f64"
    if "float" in t:
        return "f32"
    return "i32"


_CT = {ctypes.c_void_p: "ptr", ctypes.c_char_p: "ptr", ctypes.c_longlong: "i64", ctypes.c_ulonglong: "i64", ctypes.c_size_t: "i64",
       ctypes.c_int: "i32", ctypes.c_uint: "i32", ctypes.c_float: "f32", ctypes.c_double: "f64"}


def _registered() -> dict:
    for mod in ("nn.paged", "ops.attention", "ops.batchnorm", "ops.conv", "ops.functional", "ops.quant", "parallel.ddp",
                "parallel.peer_collectives", "parallel.tensor_parallel", "utils.grammar", "serialize.gguf", "ops.pool"):
        importlib.import_module("ferrotorch_b200." + mod)
    importlib.import_module("ferrotorch_b200.utils.grammar")._register_token_mask_proto()
    return dict(_native._KERNEL_PROTOS)


def test_every_prototype_matches_its_c_signature():
    sigs, protos = _c_signatures(), _registered()
    assert len(sigs) > 40 and len(protos) > 40
    problems = []
    for name, (_, argtypes) in protos.items():
        if name not in sigs:
            problems.append("%s: bound in Python but not defined with FT_API in csrc/*.cu" % name)
            continue
        c_params = sigs[name][1]
        if len(c_params) != len(argtypes):
            problems.append("%s: C takes %d parameters, the prototype lists %d" % (name, len(c_params), len(argtypes)))
            continue
        for k, (cp, at) in enumerate(zip(c_params, argtypes)):
            want, have = _kind(cp), _CT.get(at, getattr(at, "_type_", None) and "ptr" or str(at))
            if issubclass(at, ctypes._Pointer) if isinstance(at, type) else False:
                have = "ptr"
            if want != have:
                problems.append("%s: parameter %d is `%s` in C but %s in the prototype" % (name, k, cp, have))
    assert not problems, "\n".join(problems)
