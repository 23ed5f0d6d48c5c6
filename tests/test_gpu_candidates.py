"""The reference's search found 69 muGraphs equivalent to the un-fused speculative-decode attention graph, with
its own fingerprint kernels (tests/golden/spec_decode_candidates.json.gz, written by make_candidates.py from the
reference's demo checkpoint).  An executor with the reference's fingerprint semantics must agree: every candidate,
loaded through the JSON wire format and evaluated on the GPU, has the computation graph's fingerprint."""
import gzip
import json
import os

import numpy as np
import pytest

import attention_superoptimizer_b200 as mg
from oracle import mugraph_oracle as mo
from tests.helpers import assert_close, from_bits, to_bits

pytestmark = pytest.mark.gpu
FIXTURE = os.path.join(os.path.dirname(__file__), "golden", "spec_decode_candidates.json.gz")
BIG = 227 * 1024


def load_fixture():
    with gzip.open(FIXTURE) as f:
        return json.loads(f.read().decode())


def inputs_of(g):
    return [g.operator(i)[1][0] for i in range(g.num_operators) if g.operator(i)[0] == 1001]


@pytest.mark.parametrize("fill", ["reference", "uniform"])
def test_every_candidate_verifies(runtime, fill):
    runtime.set_max_smem(BIG)
    fx = load_fixture()
    rng = np.random.default_rng(5)
    with mg.PyGraph.from_json(fx["computation_graph"], runtime) as ref:
        ref_in = inputs_of(ref)
        if fill == "reference":  # KNInputOp::fingerprint: fp[i] = i mod 25651
            ref.fingerprint(refill_inputs=True)
            x = [t.download_fingerprint() for t in ref_in]
        else:
            x = [rng.integers(0, mo.FP_PQ, size=t.shape).astype(np.uint16) for t in ref_in]
            for t, a in zip(ref_in, x):
                t.upload_fingerprint(a)
            ref.fingerprint()
        ref_out = ref.operator(ref.num_operators - 1)[1][0]
        want = ref_out.download_fingerprint()
        # the un-fused graph itself against the oracle's kernel-level operators
        assert np.array_equal(want, mo.unfused_attention_fp(*x))
        assert len(np.unique(want)) > 200  # results are multiples of 113: 227 possible values
        for n, doc in enumerate(fx["generated_graphs"]):
            with mg.PyGraph.from_json(doc, runtime) as g:
                for t, a in zip(inputs_of(g), x):
                    t.upload_fingerprint(a)
                g.fingerprint()
                out = g.operator(g.num_operators - 1)[1][0]
                assert out.shape == want.shape
                assert out.has_same_fingerprint(ref_out), "candidate %d" % n   # compared on the device
                assert np.array_equal(out.download_fingerprint(), want), "candidate %d" % n


def test_candidates_in_float_mode(runtime):
    """One candidate of each structure, float mode, against exp(Q K) V / rowsum in fp64."""
    runtime.set_max_smem(BIG)
    fx = load_fixture()
    rng = np.random.default_rng(6)
    rnd = lambda a: from_bits(to_bits(a, mg.float16), mg.float16)
    q = rnd(rng.standard_normal((2, 256, 64)) / 8.0)
    k = rnd(rng.standard_normal((2, 64, 4096)))
    v = rnd(rng.standard_normal((2, 4096, 64)))
    e = np.exp(q.astype(np.float64) @ k.astype(np.float64))
    want = (e / e.sum(axis=-1, keepdims=True)) @ v.astype(np.float64)
    mem = [q, np.ascontiguousarray(k.transpose(0, 2, 1)), np.ascontiguousarray(v.transpose(0, 2, 1))]  # K, V column-major
    seen = set()
    for doc in fx["generated_graphs"]:
        shape = tuple((op["op_type"], json.dumps(op.get("plan", {}).get("ops")), json.dumps(op.get("plan", {}).get("grid_dim")),
                       op.get("plan", {}).get("forloop_range")) for op in doc)
        if shape in seen:
            continue
        seen.add(shape)
        with mg.PyGraph.from_json(doc, runtime) as g:
            for t, a in zip(inputs_of(g), mem):
                t.upload_data(to_bits(a, mg.float16))
            g.run()
            out = g.operator(g.num_operators - 1)[1][0]
            got = from_bits(out.download_data(), mg.float16).reshape(out.shape)
        assert_close(got, want, mg.float16, "candidate structure %d" % len(seen))
    assert len(seen) >= 9


def test_batched_verification(runtime):
    """mg_verify_candidates: every candidate resident at once, fingerprint kernels and on-device comparisons enqueued
    back to back, one synchronisation.  One candidate gets different inputs and must be reported as different."""
    import contextlib
    runtime.set_max_smem(BIG)
    fx = load_fixture()
    rng = np.random.default_rng(8)
    with contextlib.ExitStack() as stack:  # graphs are released in reverse order of creation (LIFO arena)
        ref = stack.enter_context(mg.PyGraph.from_json(fx["computation_graph"], runtime))
        ref_in = inputs_of(ref)
        x = [rng.integers(0, mo.FP_PQ, size=t.shape).astype(np.uint16) for t in ref_in]
        for t, a in zip(ref_in, x):
            t.upload_fingerprint(a)
        ref.fingerprint()
        ref_out = ref.operator(ref.num_operators - 1)[1][0]
        batch = []
        odd = 17
        for n, doc in enumerate(fx["generated_graphs"]):
            g = stack.enter_context(mg.PyGraph.from_json(doc, runtime))
            for i, (t, a) in enumerate(zip(inputs_of(g), x)):
                t.upload_fingerprint((a + 1) % mo.FP_PQ if (n == odd and i == 0) else a)
            batch.append((g, g.operator(g.num_operators - 1)[1][0]))
        verdict = mg.verify_candidates(ref_out, batch)
        assert len(verdict) == 69
        assert verdict == [n != odd for n in range(69)]
        assert mg.verify_candidates(ref_out, []) == []
