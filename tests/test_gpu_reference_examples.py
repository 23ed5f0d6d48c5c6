"""The reference's own cpp_examples, compiled without any change to their source against this repository's
include/mirage/** and libmugraph.so (oracle/Makefile, target `examples`; only the search they end with is a
stand-in), and run on the GPU.  Each example builds the un-fused computation graph and its hand-written muGraph,
fingerprints both, asserts DTensor::has_same_fingerprint between their outputs and profiles every operator: the
reference's integration test, with this library underneath.  Skipped where the binaries have not been built (they
need the reference checkout at build time)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXDIR = os.path.join(ROOT, "oracle", "_ref", "examples")
NAMES = sorted(os.listdir(EXDIR)) if os.path.isdir(EXDIR) else []

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not NAMES, reason="oracle/_ref/examples not built")]


@pytest.mark.parametrize("name", NAMES or ["none"])
def test_reference_example_runs_on_this_library(name):
    r = subprocess.run([os.path.join(EXDIR, name)], capture_output=True, text=True, timeout=600)
    tail = (r.stdout + r.stderr)[-2000:]
    # exit status 0 means the example's own `assert(... has_same_fingerprint ...)` held (a failed assert aborts)
    assert r.returncode == 0, tail
    assert "Total runtime" in r.stdout, tail
    # examples that go on to the search hand the computation graph to the generator by value
    assert "no search is run" in r.stdout or "Search time" not in r.stdout, tail
