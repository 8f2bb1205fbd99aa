"""Static gates over the source tree (the reference keeps comparable gates in ``tooling/``:
``anti-pattern-gate.py``): patterns that must never appear in committed code are searched for
as text.  The needles are assembled at run time so that this file does not contain them."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CODE_EXT = (".py", ".cu", ".cuh", ".cpp", ".h", ".hpp")


def _files(exts, skip_dirs=("_work", "gpurun_out", ".git", "baseline", "__pycache__", "_C", "build")):
    for base, dirs, names in os.walk(ROOT):
        dirs[:] = [d for d in dirs if d not in skip_dirs]
        for n in names:
            if n.endswith(exts):
                yield os.path.join(base, n)


def _read(path):
    with open(path, errors="replace") as f:
        return f.read()


def test_no_batched_memcpy_entry_points_are_named():
    # four driver / runtime entry points that must not be used: one async copy per transfer instead
    stems = ["cudaMemcpy", "cudaMemcpy3D", "cuMemcpy", "cuMemcpy3D"]
    needles = [s + "Batch" + "Async" for s in stems]
    bad = [(p, n) for p in _files(CODE_EXT + (".sh",)) for n in needles if n in _read(p)]
    assert not bad, bad


def test_no_cluster_multicast_on_bulk_or_tensor_loads():
    # a TMA / bulk *load* with cluster multicast is never issued (tcgen05.commit may carry the qualifier)
    qual = ".multicast" + "::cluster"
    bad = []
    for p in _files((".cu", ".cuh", ".h", ".py")):
        for i, line in enumerate(_read(p).splitlines(), 1):
            if qual in line and "cp.async.bulk" in line:
                bad.append((os.path.relpath(p, ROOT), i))
    assert not bad, bad


def test_device_code_has_no_trap_and_no_unbounded_flag_spin():
    trap = "__" + "trap" + "()"
    bad = []
    for p in _files((".cu", ".cuh")):
        src = _read(p)
        if trap in src:
            bad.append((os.path.relpath(p, ROOT), trap))
        # every `while (...)` that polls memory written by another agent sits in a helper that
        # also reads the clock: a polling loop without a time limit is a hang waiting to happen
        for m in re.finditer(r"while\s*\(([^;{]*?(ld_acquire|try_wait|volatile)[^;{]*?)\)\s*\{", src):
            body = src[m.end():m.end() + 600]
            if "globaltimer" not in body and "limit" not in body and "tries" not in body and "spins" not in body:
                bad.append((os.path.relpath(p, ROOT), src[:m.start()].count("\n") + 1))
    assert not bad, bad


def test_profiler_commands_in_profiles_leave_the_clocks_alone():
    flag = "--clock-control none"
    bad = []
    for p in _files((".md", ".txt")):
        if os.sep + "profiles" + os.sep not in p:
            continue
        for i, line in enumerate(_read(p).splitlines(), 1):
            if re.search(r"(^|\s)ncu\s+(-|\$)", line) and " -i " not in line:
                ctx = "\n".join(_read(p).splitlines()[max(0, i - 6):i + 3])
                if flag not in ctx and "$S" not in line:
                    bad.append((os.path.relpath(p, ROOT), i))
    assert not bad, bad


def test_no_gpu_setting_is_changed_anywhere():
    # clocks, power limits, persistence / compute / ECC mode, MIG, resets: never from this tree
    smi = "nvidia-smi"
    flags = [" -lgc", " -rgc", " -ac ", " -rac", " -pl ", " -pm ", " -c ", " -e ", " -mig", " --gpu-reset", " -r "]
    calls = ["nvmlDeviceSet", "nvmlDeviceReset"]
    bad = []
    for p in _files(CODE_EXT + (".sh",)):
        if p.endswith("test_static_gates_cpu.py"):
            continue
        for i, line in enumerate(_read(p).splitlines(), 1):
            if smi in line and any(f in line + " " for f in flags):
                bad.append((os.path.relpath(p, ROOT), i))
            if any(c in line for c in calls):
                bad.append((os.path.relpath(p, ROOT), i))
    assert not bad, bad


def test_comments_do_not_point_at_working_notes_or_machine_paths():
    docs = ["".join(parts) + ".md" for parts in (("SUR", "VEY"), ("DES", "IGN"), ("VER", "DICT"), ("AD", "VICE"), ("BASE", "LINE"))]
    others = ["gpu" + "run", "/" + "root" + "/"]
    bad = []
    for p in _files(CODE_EXT):
        rel = os.path.relpath(p, ROOT)
        if rel.startswith("tests" + os.sep + "test_static_gates"):
            continue
        src = _read(p)
        for n in docs + others:
            if n in src:
                bad.append((rel, n))
    assert not bad, bad


def test_committed_code_does_not_reach_into_the_scratch_folder():
    scratch = "_" + "work"
    bad = []
    for p in _files(CODE_EXT):
        if p.endswith("test_static_gates_cpu.py"):
            continue
        for i, line in enumerate(_read(p).splitlines(), 1):
            if re.search(r"(import|open|from|path|run)\b.*\b" + scratch + r"\b", line):
                bad.append((os.path.relpath(p, ROOT), i))
    assert not bad, bad


def test_every_cuda_source_is_part_of_the_build():
    from ferrotorch_b200 import _native

    listed = _read(_native.__file__)
    missing = [n for n in os.listdir(os.path.join(ROOT, "ferrotorch_b200", "csrc")) if n.endswith(".cu") and n not in listed]
    if missing:      # sources may be discovered by a glob instead of being listed
        assert "glob" in listed or "listdir" in listed, missing


@pytest.mark.parametrize("name", ["bench.py", "__graft_entry__.py"])
def test_entry_points_exist_and_define_their_contract(name):
    src = _read(os.path.join(ROOT, name))
    if name == "bench.py":
        for key in ('"metric"', '"value"', '"n_gpus"', '"ms_per_step"', '"vs_baseline"', '"e2e"', '"gpu_launches"', '"clocks"',
                    "--impl", "--gpus", "--steps", "--warmup"):
            assert key in src, key
    else:
        assert "def build()" in src and "def smoke()" in src


def test_every_exported_native_function_has_a_python_caller():
    # an export nobody binds is dead weight or a forgotten prototype
    import glob

    exported = set()
    for f in glob.glob(os.path.join(ROOT, "ferrotorch_b200", "csrc", "*.cu")) + glob.glob(os.path.join(ROOT, "ferrotorch_b200", "csrc", "host", "*.cpp")):
        for m in re.finditer(r"(?:FT_API|FTC_API|FTD_API|FTIO_API)\s+[\w\s\*]+?\b(ft\w*_\w+)\s*\(", _read(f)):
            exported.add(m.group(1))
    assert len(exported) > 60
    python = "".join(_read(p) for p in _files((".py",)))
    accessors = {"ftc_rank", "ftc_world"}          # plain getters of the TCP group handle, kept for embedders
    missing = sorted(n for n in exported - accessors if n not in python)
    assert not missing, missing


def test_citations_of_the_reference_point_at_existing_files_and_lines():
    """Docstrings cite the reference as ``crate/src/file.rs:line``.  With the reference's tree at
    ``$FERROTORCH_REFERENCE_DIR`` every cited file must exist and be at least that long (the reference
    keeps a comparable gate, ``tooling/fix-cite-drift.py``); without the tree the gate is skipped."""
    tree = os.environ.get("FERROTORCH_REFERENCE_DIR", "")
    if not tree or not os.path.isdir(tree):
        pytest.skip("FERROTORCH_REFERENCE_DIR is not set")
    pat = re.compile(r"(ferrotorch(?:-[a-z\-]+)?/(?:src|tests|examples|benches)/[A-Za-z0-9_/.\-]+\.(?:rs|metal|py|toml))(?::(\d+))?")
    seen, bad = 0, []
    for p in _files(CODE_EXT):
        for m in pat.finditer(_read(p)):
            seen += 1
            target = os.path.join(tree, m.group(1))
            if not os.path.exists(target):
                bad.append((os.path.relpath(p, ROOT), m.group(0), "no such file"))
            elif m.group(2):
                with open(target, errors="replace") as f:
                    if sum(1 for _ in f) < int(m.group(2)):
                        bad.append((os.path.relpath(p, ROOT), m.group(0), "file is shorter"))
    assert seen > 100 and not bad, bad
