"""The reference's own GPU fingerprint kernel (compute_customizedop_fingerprint, built for sm_100a into
oracle/_ref/libref_gpu.so) against this library's kernels and against the CPU oracle: all three must produce the
same fingerprints, bit for bit.  Skipped where the reference-derived library has not been built."""
import json
import os

import numpy as np
import pytest

import attention_superoptimizer_b200 as mg
from oracle import mugraph_oracle as mo
from oracle import ref_gpu

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_gpu.available(), reason="oracle/_ref/libref_gpu.so not built")]
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "gqa_decode_reference_host.json")


def reference_pair(B, M, D, L, S, F):
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, S, F)
    op1 = ref_gpu.CustomizedOp(specs, p1)
    op2 = ref_gpu.CustomizedOp(None, p2, producer=op1)
    return specs, op1, op2


def ours(runtime, B, M, D, L, S, F, x=None):
    with mg.PyGraph(runtime) as g:
        Q = g.new_input((B, M, D)); K = g.new_input((B, D, L), layout=mg.DmemColumnMajor); V = g.new_input((B, L, D), layout=mg.DmemColumnMajor)
        p1, p2 = mg.gqa_decode_plans(B, M, D, L, S, F)
        parts = g.customized([Q, K, V], p1)
        out = g.customized(parts, p2)
        if x is None:
            g.fingerprint(refill_inputs=True)
        else:
            for t, a in zip((Q, K, V), x):
                t.upload_fingerprint(a)
            g.fingerprint()
        return parts[0].download_fingerprint(), parts[1].download_fingerprint(), out[0].download_fingerprint()


@pytest.mark.parametrize("name", ["reference_example_bs1", "baseline_c2"])
def test_reference_kernel_reproduces_the_golden_digests(runtime, name):
    """The reference's kernel on the reference's input fill: the digests the reference's host code produced for the
    example shape (Q[2,8,64], K[2,64,4096]) and for the benchmark's decode shape; this library's kernels agree."""
    with open(GOLDEN) as f:
        c = next(c for c in json.load(f)["cases"] if c["name"] == name)
    shape = (c["B"], c["M"], c["D"], c["L"], c["S"], c["F"])
    specs, op1, op2 = reference_pair(*shape)
    try:
        assert op1.info["num_ops"] == c["op1"]["num_ops"] and op1.info["smem_bytes"] == c["op1"]["smem_bytes"]
        for i in range(3):
            op1.fill_reference(i)
        op1.fingerprint()
        op2.fingerprint()
        o_part, r_part, final = op1.output(0), op1.output(1), op2.output(0)
    finally:
        op2.destroy()
        op1.destroy()
    assert str(mo.fnv1a64(np.concatenate([o_part.ravel(), r_part.ravel()]))) == c["op1_digest"]
    assert str(mo.fnv1a64(final)) == c["final_digest"]
    assert final.ravel()[:4].tolist() == c["final_head"]
    mine = ours(runtime, *shape)
    assert np.array_equal(mine[0], o_part) and np.array_equal(mine[1], r_part) and np.array_equal(mine[2], final)


def test_reference_kernel_equals_ours_and_the_oracle_on_sweep_sets(runtime):
    """Three seeded input sets of the verification sweep through the reference's kernel, this library's kernels and
    the numpy oracle; the committed digest of each set matches as well."""
    B, M, D, L, S, F = 8, 4, 128, 4096, 16, 4
    with open(os.path.join(os.path.dirname(__file__), "golden", "sweep_digests_gqa_decode.json")) as f:
        digests = json.load(f)["digests"]
    specs, op1, op2 = reference_pair(B, M, D, L, S, F)
    try:
        for s in (0, 1234, 4095):
            x = mo.sweep_inputs(s, specs)
            for i, a in enumerate(x):
                op1.set_input(i, a)
            op1.fingerprint()
            op2.fingerprint()
            final = op2.output(0)
            assert str(mo.fnv1a64(final)) == digests[s]
            assert np.array_equal(final, mo.unfused_attention_fp(*x))
            assert np.array_equal(final, ours(runtime, B, M, D, L, S, F, x)[2])
    finally:
        op2.destroy()
        op1.destroy()
