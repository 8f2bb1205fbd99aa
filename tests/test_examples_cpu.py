"""The scripts under examples/ run to completion on CPU."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script,args", [
    ("train_tiny_llama.py", ["--steps", "8", "--device", "cpu"]),
    ("generate_text.py", []),
    ("compile_and_checkpoint.py", ["--device", "cpu"]),
    ("ddp_over_tcp.py", []),
    ("constrained_json.py", []),
    ("tiny_text_to_image.py", ["--steps", "3", "--size", "32"]),
    ("coming_from_ferrotorch.py", []),
    ("detect_objects.py", ["--model", "fcos"]),
    ("pipeline_and_context_parallel.py", []),
    ("fsdp_flat_units.py", []),
    ("serve_many_requests.py", []),
    ("train_mnist_synthetic.py", ["--epochs", "2", "--samples", "600"]),
])
def test_example_runs(script, args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script), *args], env=env,
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
