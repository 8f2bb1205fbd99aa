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


# --------------------------------------------------------------------------- method level
# ``reference_methods.json``: for every reference type whose name resolves to a class of this package,
# the ``pub fn`` names of its ``impl`` blocks (read as text).  A class answers a name when it has the
# attribute or assigns ``self.<name>``.  The names below are the ones it does not answer, with the reason;
# the gate fails when a new name goes missing and when a listed name has since been added.
with open(os.path.join(os.path.dirname(__file__), "conformance", "reference_methods.json")) as _f:
    METHODS = json.load(_f)

NOT_ANSWERED = {
    # parser-state probes of the reference's hand-written JSON automaton; the grammar here is a schema -> NFA
    # compiler whose states are sets, with no per-kind emission stage to report
    ("ferrotorch-grammar", "JsonGrammar"): {"boolean_emission_stage", "boolean_emission_stage_top", "integer_emission_stage",
                                            "integer_emission_stage_top", "is_array_at_start_top", "is_object_at_start_top",
                                            "null_emission_stage", "null_emission_stage_top", "nullable_emission_stage",
                                            "number_emission_stage", "number_emission_stage_top", "object_key_emission_stage",
                                            "step_str", "string_emission_stage", "string_emission_stage_top",
                                            "string_enum_emission_stage", "string_enum_emission_stage_top",
                                            "top_frame_parent_terminators"},
    # the two halves of the VAE are plain conv stacks here; scaling, sampling and checkpoint loading live on
    # ``AutoencoderKL``, which owns the quantisation convolutions they need
    ("ferrotorch-diffusion", "VaeEncoder"): {"encode", "encode_with_scaling", "load_hf_state_dict"},
    ("ferrotorch-diffusion", "VaeDecoder"): {"decode_with_scaling", "load_hf_state_dict"},
    # the status is a plain enum here; the compiled graph travels in ``InductorCompileOutcome``
    ("ferrotorch-jit", "InductorCompileStatus"): {"compiled_graph", "into_compiled_graph"},
    # instance attributes that torch's base classes set (``nn.Linear.__init__``, ``register_buffer``)
    ("ferrotorch-nn", "Linear"): {"in_features", "out_features"},
    ("ferrotorch-optim", "AveragedModel"): {"n_averaged"},
    # ``BertOutput`` names the model's output record here; the reference's module of that name (dense + residual +
    # layer norm) is ``BertSelfOutput``, reused for both places
    ("ferrotorch-bert", "BertOutput"): {"forward_residual"},
    # torch's L-BFGS has no ``maximize``
    ("ferrotorch-optim", "LbfgsConfig"): {"with_maximize"},
}
KNOWN_METHOD_GAPS = 0


def _answers(cls, name: str) -> bool:
    import inspect
    import re

    if hasattr(cls, name):
        return True
    try:
        return re.search(r"self\.%s\b" % re.escape(name), inspect.getsource(cls)) is not None
    except (OSError, TypeError):
        return False


def test_own_classes_answer_the_reference_method_names():
    import inspect

    missing, stale = {}, []
    for crate, types in METHODS.items():
        spaces = [_namespace(p) for p in NAMESPACES[crate]]
        for ty, names in types.items():
            cls = next((getattr(s, ty) for s in spaces if hasattr(s, ty)), None)
            if cls is None or not inspect.isclass(cls):
                continue
            allowed = NOT_ANSWERED.get((crate, ty), set())
            gone = [n for n in names if not _answers(cls, n)]
            extra = [n for n in gone if n not in allowed]
            if extra:
                missing[(crate, ty)] = extra
            stale += [(crate, ty, n) for n in allowed if n not in gone]
    total = sum(len(v) for v in missing.values())
    assert total <= KNOWN_METHOD_GAPS, "method names answered by fewer classes than before (%d > %d): %s" % (
        total, KNOWN_METHOD_GAPS, {k: v for k, v in list(missing.items())[:12]})
    assert not stale, "listed as unanswered but present: %s" % stale[:10]
