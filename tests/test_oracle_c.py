"""The plain-C restatement (timed CPU baseline) against the numpy oracle."""
import numpy as np
import pytest

from oracle import fp_oracle, mugraph_oracle as mo


@pytest.mark.parametrize("shape", [(2, 8, 64, 1024, 4, 4), (8, 4, 128, 4096, 16, 4), (3, 1, 8, 48, 3, 2)])
def test_c_oracle_equals_numpy_oracle(shape):
    B, M, D, L, S, F = shape
    rng = np.random.default_rng(sum(shape))
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, S, F)
    x = [rng.integers(0, mo.FP_PQ, size=s.dims).astype(np.uint16) for s in specs]
    g1 = mo.build_customized(specs, p1)
    o1 = mo.run_fingerprint(g1, x)
    c1, used = fp_oracle.run(g1, x)
    assert used >= 1 and all(np.array_equal(a, b) for a, b in zip(o1, c1))
    g2 = mo.build_customized(mo.output_specs(g1), p2)
    c2, _ = fp_oracle.run(g2, c1)
    assert np.array_equal(c2[0], mo.run_fingerprint(g2, o1)[0])
    assert np.array_equal(c2[0], mo.unfused_attention_fp(*x))


def test_c_oracle_sets_and_threads():
    B, M, D, L, S, F = 2, 4, 32, 128, 2, 2
    rng = np.random.default_rng(1)
    specs, p1, _ = mo.gqa_decode_plans(B, M, D, L, S, F)
    g1 = mo.build_customized(specs, p1)
    sets = [[rng.integers(0, mo.FP_P, size=s.dims).astype(np.uint16) for s in specs] for _ in range(3)]
    stacked = [np.stack([sets[s][i] for s in range(3)]) for i in range(3)]
    out1, _ = fp_oracle.run(g1, stacked, num_sets=3, threads=1)
    outn, _ = fp_oracle.run(g1, stacked, num_sets=3, threads=0)
    for s in range(3):
        want = mo.run_fingerprint(g1, sets[s])
        assert np.array_equal(out1[0][s], want[0]) and np.array_equal(outn[1][s], want[1])


@pytest.mark.parametrize("layouts", [(mo.DmemRowMajor, mo.DmemRowMajor), (mo.DmemColumnMajor, mo.DmemColumnMajor)])
def test_c_float_evaluator_equals_numpy_evaluator(layouts):
    B, M, D, L, S, F = 2, 4, 64, 512, 4, 2
    kl, vl = layouts
    rng = np.random.default_rng(4)
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, S, F, k_layout=kl, v_layout=vl)
    q = (rng.standard_normal((B, M, D)) / np.sqrt(D)).astype(np.float16).astype(np.float32)
    k = rng.standard_normal((B, D, L)).astype(np.float16).astype(np.float32)
    v = rng.standard_normal((B, L, D)).astype(np.float16).astype(np.float32)
    mem = [q, k if kl == mo.DmemRowMajor else np.ascontiguousarray(k.transpose(0, 2, 1)),
           v if vl == mo.DmemRowMajor else np.ascontiguousarray(v.transpose(0, 2, 1))]
    g1 = mo.build_customized(specs, p1)
    n1 = mo.run_float(g1, mem)
    c1, _ = fp_oracle.run_float(g1, mem)
    for a, b in zip(n1, c1):
        assert np.allclose(a, b, rtol=1e-5, atol=1e-4)  # fp32 summation order differs
    g2 = mo.build_customized(mo.output_specs(g1), p2)
    c2, _ = fp_oracle.run_float(g2, c1)
    assert np.allclose(c2[0], mo.attention_fp32(q, k, v), rtol=1e-4, atol=1e-5)
