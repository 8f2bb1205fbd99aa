"""Name-level parity with the reference: every name that one of its crates re-exports from
``lib.rs`` (``tests/conformance/reference_exports.json``, the export lists read as text) resolves in
the namespace of this package that plays that crate's role, except the names listed with a reason."""
import json
import os

import pytest

import ferrotorch_b200 as ft

NAMESPACES = {
    "ferrotorch": ["", "prelude"], "ferrotorch-core": ["", "autograd", "core", "tensor_ops"], "ferrotorch-nn": ["nn"],
    "ferrotorch-optim": ["optim"], "ferrotorch-data": ["data"], "ferrotorch-train": ["train"], "ferrotorch-vision": ["vision"],
    "ferrotorch-jit": ["jit"], "ferrotorch-serialize": ["serialize"], "ferrotorch-distributed": ["distributed"],
    "ferrotorch-gpu": ["gpu"], "ferrotorch-llama": ["llama"], "ferrotorch-bert": ["bert"], "ferrotorch-whisper": ["whisper"],
    "ferrotorch-graph": ["graph"], "ferrotorch-rl": ["rl"], "ferrotorch-diffusion": ["diffusion"],
    "ferrotorch-distributions": ["distributions"], "ferrotorch-profiler": ["profiler"], "ferrotorch-hub": ["hub"],
    "ferrotorch-tokenize": ["tokenize"], "ferrotorch-grammar": ["grammar"], "ferrotorch-cubecl": ["cubecl"], "ferrotorch-mps": [],
}
WITHOUT_COUNTERPART = {
    # run-time plumbing of a portable-GPU layer that this package does not have: tensors and torch.device play these roles
    "ferrotorch-cubecl": {"CubeClient", "CubeDevice", "CubeRuntime", "CubeclStorageHandle", "cubecl_handle_of", "upload_f32",
                          "wrap_kernel_output"},
    "ferrotorch-llama": {"cubecl_cuda_client"},
    "ferrotorch-mps": {"MtlBackend"},                 # Metal back-end: dropped
    "ferrotorch-nn": {"DeriveModule"},                # derive macro: nn.Module registers parameters on assignment
}

with open(os.path.join(os.path.dirname(__file__), "conformance", "reference_exports.json")) as _f:
    EXPORTS = json.load(_f)


def _namespace(path: str):
    obj = ft
    for part in filter(None, path.split(".")):
        obj = getattr(obj, part)
    return obj


@pytest.mark.parametrize("crate", sorted(EXPORTS))
def test_exported_names_resolve(crate):
    spaces = [_namespace(p) for p in NAMESPACES[crate]]
    skip = WITHOUT_COUNTERPART.get(crate, set())
    missing = [n for n in EXPORTS[crate] if n not in skip and not any(hasattr(s, n) for s in spaces)]
    assert not missing, "%s: %s" % (crate, missing)
    assert not [n for n in skip if any(hasattr(s, n) for s in spaces)], "a name listed as missing now exists: drop it from the list"


def test_the_fixture_is_the_size_it_should_be():
    assert sum(len(v) for v in EXPORTS.values()) > 1300 and len(EXPORTS) == len(NAMESPACES)
    assert sum(len(v) for v in WITHOUT_COUNTERPART.values()) <= 10
