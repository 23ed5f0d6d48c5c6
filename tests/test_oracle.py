"""CPU tests of the oracle itself: it must reproduce the reference's own results before it is
allowed to judge the CUDA path."""
import json
import os

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from oracle import mugraph_oracle as mo
from oracle import ref_host

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "gqa_decode_reference_host.json")


def golden_cases():
    with open(GOLDEN) as f:
        return json.load(f)["cases"]


def case_inputs(c, specs):
    if c["fill"] == "reference":
        return [mo.reference_fill(s.dims) for s in specs]
    return [np.array(v, np.uint16).reshape(s.dims) for v, s in zip(c["inputs_full"], specs)]


def test_constants_and_tables():
    # the relations asserted by the reference when it builds its tables
    # (src/kernel/device_memory_manager.cu:39-46, 63-65, 83-85)
    assert mo.FP_Q < mo.FP_P and (mo.FP_P - 1) % mo.FP_Q == 0 and mo.FP_P * mo.FP_Q == mo.FP_PQ
    assert mo.FP_Q_MUL_P_MOD_1 % mo.FP_Q == 0 and mo.FP_Q_MUL_P_MOD_1 % mo.FP_P == 1
    assert mo.FP_P_MUL_Q_MOD_1 % mo.FP_P == 0 and mo.FP_P_MUL_Q_MOD_1 % mo.FP_Q == 1
    e, p, q = mo.EXP_TBL, mo.DIV_P_TBL, mo.DIV_Q_TBL
    assert e[0] == 1 and (e[mo.FP_Q - 1] * mo.FP_EXP_BASE) % mo.FP_P == 1
    assert len(set(e.tolist())) == mo.FP_Q  # 3 has order Q modulo P
    assert p[0] == 1 and q[0] == 1
    for i in range(2, mo.FP_P):
        assert p[i] != 1 and (i * p[i]) % mo.FP_P == 1
    for i in range(2, mo.FP_Q):
        assert q[i] != 1 and (i * q[i]) % mo.FP_Q == 1


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c["name"])
def test_oracle_matches_reference_host_golden(case):
    """Known answers produced by the reference's own host builder and fingerprinter classes."""
    c = case
    specs, p1, p2 = mo.gqa_decode_plans(c["B"], c["M"], c["D"], c["L"], c["S"], c["F"])
    x = case_inputs(c, specs)
    g1 = mo.build_customized(specs, p1)
    assert len(g1.ops) == c["op1"]["num_ops"] and g1.smem_offset == c["op1"]["smem_bytes"]
    o1 = mo.run_fingerprint(g1, x)
    assert [list(o.shape) for o in o1] == c["op1_output_shapes"]
    assert o1[0].ravel()[:4].tolist() == c["o_part_head"] and o1[1].ravel()[:4].tolist() == c["r_part_head"]
    assert str(mo.fnv1a64(np.concatenate([o.ravel() for o in o1]))) == c["op1_digest"]
    g2 = mo.build_customized(mo.output_specs(g1), p2)
    assert len(g2.ops) == c["op2"]["num_ops"] and g2.smem_offset == c["op2"]["smem_bytes"]
    o2 = mo.run_fingerprint(g2, o1)
    assert list(o2[0].shape) == c["final_shape"] and o2[0].ravel()[:4].tolist() == c["final_head"]
    assert str(mo.fnv1a64(o2[0])) == c["final_digest"]
    if "final_full" in c:
        assert o2[0].ravel().tolist() == c["final_full"]
    # the reference's integration check: fused graph == un-fused graph
    # (cpp_examples/group_query_attn_inc_decode.cc:104-108)
    assert np.array_equal(o2[0], mo.unfused_attention_fp(*x))


@pytest.mark.skipif(not ref_host.available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_tables_match_reference_host():
    e, p, q = ref_host.tables()
    assert np.array_equal(e, mo.EXP_TBL) and np.array_equal(p, mo.DIV_P_TBL) and np.array_equal(q, mo.DIV_Q_TBL)


@pytest.mark.skipif(not ref_host.available(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("shape", [(2, 8, 64, 1024, 4, 4), (1, 4, 128, 512, 2, 4), (4, 16, 32, 256, 8, 1),
                                   (3, 1, 8, 48, 3, 2)])
def test_oracle_matches_reference_host_live(shape):
    """Random inputs in [0, PQ): the numpy restatement against the reference's own code, op by op."""
    B, M, D, L, S, F = shape
    rng = np.random.default_rng(sum(shape))
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, S, F)
    x = [rng.integers(0, mo.FP_PQ, size=s.dims).astype(np.uint16) for s in specs]
    ref1, info1 = ref_host.customized_fingerprint(specs, p1, x)
    g1 = mo.build_customized(specs, p1)
    o1 = mo.run_fingerprint(g1, x)
    assert g1.smem_offset == info1["smem_bytes"] and len(g1.ops) == info1["num_ops"]
    assert all(np.array_equal(a, b) for a, b in zip(ref1, o1))
    ref2, info2 = ref_host.customized_fingerprint(mo.output_specs(g1), p2, ref1)
    g2 = mo.build_customized(mo.output_specs(g1), p2)
    o2 = mo.run_fingerprint(g2, o1)
    assert g2.smem_offset == info2["smem_bytes"]
    assert np.array_equal(ref2[0], o2[0])


@pytest.mark.skipif(not ref_host.available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_oracle_matches_reference_host_other_graphs():
    """Graphs outside the attention pattern: matmul chain, concat, to_dimx on a middle dim, grid.z."""
    rng = np.random.default_rng(5)
    # matmul chain X[16,256] W1[256,128] W2[128,64]: grid over W1's columns / W2's rows, for-loop over K
    specs = [mo.DTensorSpec((16, 256)), mo.DTensorSpec((256, 128)), mo.DTensorSpec((128, 64))]
    plan = mo.ExecutionPlan(
        ops=[(mo.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mo.TB_MATMUL_OP, [(3, 0), (2, 0)])],
        input_map=[(-1, -1, -1), (1, -1, -1), (0, -1, -1)], forloop_dim=[1, 0, -1],
        input_smem_layouts=[mo.SmemRowMajor] * 3, output_map=(1, -1, -1), forloop_range=4, grid_dim=(4, 1, 1),
        reduction_dimx=64)
    x = [rng.integers(0, mo.FP_PQ, size=s.dims).astype(np.uint16) for s in specs]
    ref, _ = ref_host.customized_fingerprint(specs, plan, x)
    got = mo.run_fingerprint(mo.build_customized(specs, plan), x)
    assert len(ref) == len(got) == 1 and np.array_equal(ref[0], got[0])
    # linearity makes the block partials sum to the un-fused chain
    total = got[0].astype(np.int64).reshape(16, 4, 64).sum(axis=1) % mo.FP_PQ
    assert np.array_equal(total, mo.fp_matmul(mo.fp_matmul(x[0], x[1]), x[2]))
    # concat + exp + div with broadcasting, 3-D tensors split on grid x and z
    specs = [mo.DTensorSpec((4, 8, 32)), mo.DTensorSpec((4, 8, 32)), mo.DTensorSpec((4, 8, 64))]
    plan = mo.ExecutionPlan(
        ops=[(mo.TB_CONCAT_2_OP, [(0, 0), (1, 0)]), (mo.TB_EXP_OP, [(3, 0)]), (mo.TB_REDUCTION_2_OP, [(4, 0)]),
             (mo.TB_DIV_OP, [(2, 0), (5, 0)]), (mo.TB_REDUCTION_2_TO_DIMX_OP, [(6, 0)])],
        input_map=[(0, -1, 1), (0, -1, 1), (0, -1, 1)], forloop_dim=[-1, -1, -1],
        input_smem_layouts=[mo.SmemRowMajor] * 3, output_map=(0, -1, 1), forloop_range=1, grid_dim=(4, 1, 2),
        reduction_dimx=16)
    x = [rng.integers(0, mo.FP_PQ, size=s.dims).astype(np.uint16) for s in specs]
    ref, _ = ref_host.customized_fingerprint(specs, plan, x)
    got = mo.run_fingerprint(mo.build_customized(specs, plan), x)
    assert len(ref) == len(got) and all(np.array_equal(a, b) for a, b in zip(ref, got))


@settings(max_examples=25, deadline=None)
@given(B=st.integers(1, 3), M=st.sampled_from([1, 2, 4, 8]), D=st.sampled_from([8, 16, 32]),
       tile=st.sampled_from([8, 16]), S=st.sampled_from([1, 2, 4]), F=st.sampled_from([1, 2, 3]),
       seed=st.integers(0, 2 ** 16))
def test_fused_equals_unfused_property(B, M, D, tile, S, F, seed):
    """The reference's only integration check, as a property over shapes and inputs."""
    L = tile * S * F
    rng = np.random.default_rng(seed)
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, S, F)
    x = [rng.integers(0, mo.FP_PQ, size=s.dims).astype(np.uint16) for s in specs]
    g1 = mo.build_customized(specs, p1)
    o1 = mo.run_fingerprint(g1, x)
    o2 = mo.run_fingerprint(mo.build_customized(mo.output_specs(g1), p2), o1)
    assert np.array_equal(o2[0], mo.unfused_attention_fp(*x))


def test_float_evaluator_matches_unfused_attention():
    rng = np.random.default_rng(3)
    B, M, D, L, S, F = 2, 4, 32, 256, 4, 2
    for kl, vl in [(mo.DmemRowMajor, mo.DmemRowMajor), (mo.DmemColumnMajor, mo.DmemColumnMajor)]:
        specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, S, F, k_layout=kl, v_layout=vl)
        q = (rng.standard_normal((B, M, D)) / np.sqrt(D)).astype(np.float16).astype(np.float32)
        k = rng.standard_normal((B, D, L)).astype(np.float16).astype(np.float32)
        v = rng.standard_normal((B, L, D)).astype(np.float16).astype(np.float32)
        mem = [q, k if kl == mo.DmemRowMajor else np.ascontiguousarray(k.transpose(0, 2, 1)),
               v if vl == mo.DmemRowMajor else np.ascontiguousarray(v.transpose(0, 2, 1))]
        g1 = mo.build_customized(specs, p1)
        o1 = mo.run_float(g1, mem)
        o2 = mo.run_float(mo.build_customized(mo.output_specs(g1), p2), o1)
        ref = mo.attention_fp32(q, k, v)
        assert np.allclose(o2[0], ref, rtol=1e-4, atol=1e-5)


def test_invalid_plans_are_rejected():
    specs, p1, _ = mo.gqa_decode_plans(2, 4, 16, 64, 4, 2)
    bad = mo.ExecutionPlan(**{**p1.__dict__, "grid_dim": (2, 3, 1)})  # 64 not divisible by 3
    with pytest.raises(mo.InvalidGraph):
        mo.build_customized(specs, bad)
    bad = mo.ExecutionPlan(**{**p1.__dict__, "ops": [(mo.TB_MATMUL_OP, [(0, 0), (2, 0)])]})  # inner dims differ
    with pytest.raises(mo.InvalidGraph):
        mo.build_customized(specs, bad)
    with pytest.raises(mo.InvalidGraph):
        mo.build_customized(specs, p1, max_smem=512)


def test_oracle_matches_reference_sweep_digests():
    """The committed per-set digests of the verification sweep (produced by the reference's own host code) against
    the numpy restatement, on a few of the 4096 sets."""
    import json
    import os
    path = os.path.join(os.path.dirname(__file__), "golden", "sweep_digests_gqa_decode.json")
    with open(path) as f:
        golden = json.load(f)
    sh = golden["shape"]
    assert len(golden["digests"]) == 4096
    specs, _, _ = mo.gqa_decode_plans(sh["B"], sh["M"], sh["D"], sh["L"], sh["S"], sh["F"])
    for s in (0, 1, 2047, 4095):
        out = mo.unfused_attention_fp(*mo.sweep_inputs(s, specs))
        assert str(mo.fnv1a64(out)) == golden["digests"][s]
        if str(s) in golden["head_of_set"]:
            assert out.ravel()[:4].tolist() == golden["head_of_set"][str(s)]
