"""GPU parity tests: the CUDA executor, called through the C ABI, against the CPU oracle and the
reference-host golden vectors.  Fingerprint mode must be bit-exact; float mode within 2e-3 (fp16) /
1e-2 (bf16) relative of the fp32 evaluation (helpers.assert_close)."""
import json
import os

import numpy as np
import pytest

import attention_superoptimizer_b200 as mg
from oracle import mugraph_oracle as mo
from tests.helpers import assert_close, from_bits, spec_of, to_bits, to_oracle_plan, to_package_plan

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "gqa_decode_reference_host.json")
BIG = 227 * 1024


def golden_cases():
    with open(GOLDEN) as f:
        return json.load(f)["cases"]


def build_gqa(g, B, M, D, L, S, F, kl=mg.DmemColumnMajor, vl=mg.DmemColumnMajor, dtype=mg.float16):
    Q = g.new_input((B, M, D), dtype)
    K = g.new_input((B, D, L), dtype, kl)
    V = g.new_input((B, L, D), dtype, vl)
    p1, p2 = mg.gqa_decode_plans(B, M, D, L, S, F)
    o = g.customized([Q, K, V], p1)
    f = g.customized(o, p2)
    return (Q, K, V), o, f, (p1, p2)


def oracle_fp(ins, plans, x):
    g1 = mo.build_customized([spec_of(t) for t in ins], to_oracle_plan(plans[0]), max_smem=BIG)
    o1 = mo.run_fingerprint(g1, x)
    g2 = mo.build_customized(mo.output_specs(g1), to_oracle_plan(plans[1]), max_smem=BIG)
    return o1, mo.run_fingerprint(g2, o1)


@pytest.fixture(params=[2, 1, 0], ids=["fused", "specialised", "interpreter"])
def rt(request, runtime):
    runtime.set_max_smem(BIG)
    runtime.set_specialisation(request.param)
    yield runtime
    runtime.set_specialisation(2)


def test_lookup_tables_on_device(runtime):
    e, p, q = runtime.tables()
    assert np.array_equal(e, mo.EXP_TBL) and np.array_equal(p, mo.DIV_P_TBL) and np.array_equal(q, mo.DIV_Q_TBL)


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c["name"])
def test_fingerprint_golden(rt, case):
    """Known answers from the reference's own host code, including the reference's input fill."""
    c = case
    with mg.PyGraph(rt) as g:
        ins, o, f, plans = build_gqa(g, c["B"], c["M"], c["D"], c["L"], c["S"], c["F"])
        if c["fill"] == "reference":
            g.fingerprint(refill_inputs=True)  # KNInputOp::fingerprint: fp[i] = i % FP_PQ
        else:
            for t, v in zip(ins, c["inputs_full"]):
                t.upload_fingerprint(np.array(v, np.uint16))
            g.fingerprint()
        o_part, r_part, final = o[0].download_fingerprint(), o[1].download_fingerprint(), f[0].download_fingerprint()
        assert o_part.ravel()[:4].tolist() == c["o_part_head"] and r_part.ravel()[:4].tolist() == c["r_part_head"]
        assert str(mo.fnv1a64(np.concatenate([o_part.ravel(), r_part.ravel()]))) == c["op1_digest"]
        assert final.ravel()[:4].tolist() == c["final_head"]
        assert str(mo.fnv1a64(final)) == c["final_digest"]
        if "final_full" in c:
            assert final.ravel().tolist() == c["final_full"]


@pytest.mark.parametrize("shape", [(2, 8, 64, 1024, 4, 4), (1, 4, 128, 512, 2, 4), (4, 16, 32, 256, 8, 1),
                                   (3, 1, 8, 48, 3, 2), (2, 32, 128, 1024, 4, 4), (2, 5, 24, 96, 2, 3),
                                   (2, 4, 128, 2048, 2, 16), (3, 7, 64, 1024, 1, 16), (1, 1, 128, 64, 1, 1)])
@pytest.mark.parametrize("hi", [mo.FP_P, mo.FP_PQ, 65536], ids=["lt_P", "lt_PQ", "any_u16"])
def test_fingerprint_random_vs_oracle(rt, shape, hi):
    B, M, D, L, S, F = shape
    rng = np.random.default_rng(sum(shape) + hi)
    with mg.PyGraph(rt) as g:
        ins, o, f, plans = build_gqa(g, *shape)
        x = [rng.integers(0, hi, size=t.shape).astype(np.uint16) for t in ins]
        if hi == 65536:
            x[1].ravel()[:7] = 65535  # the largest storable value
        for t, v in zip(ins, x):
            t.upload_fingerprint(v)
        g.fingerprint()
        ref1, ref2 = oracle_fp(ins, plans, x)
        assert np.array_equal(o[0].download_fingerprint(), ref1[0])
        assert np.array_equal(o[1].download_fingerprint(), ref1[1])
        assert np.array_equal(f[0].download_fingerprint(), ref2[0])
        # second evaluation is identical (no state leaks between launches)
        g.fingerprint()
        assert np.array_equal(f[0].download_fingerprint(), ref2[0])


@pytest.mark.parametrize("shape", [(64, 4, 64, 512, 4, 2), (150, 4, 128, 256, 2, 2)], ids=["256_items", "300_items"])
def test_fingerprint_walking_blocks_keep_every_partial(rt, shape):
    """More (head, split) items than blocks that fit at once, evaluated by blocks that walk the items (forced: the
    default keeps one block per item when the partials are tensors of the graph): both outputs of the first
    operator and the result of the second equal the oracle's."""
    rng = np.random.default_rng(5 + sum(shape))
    rt.set_option(mg.OPT_ATTN_PERSISTENT, 2)
    try:
        with mg.PyGraph(rt) as g:
            ins, o, f, plans = build_gqa(g, *shape)
            x = [rng.integers(0, mo.FP_PQ, size=t.shape).astype(np.uint16) for t in ins]
            for t, v in zip(ins, x):
                t.upload_fingerprint(v)
            for _ in range(2):
                g.fingerprint()
                ref1, ref2 = oracle_fp(ins, plans, x)
                assert np.array_equal(o[0].download_fingerprint(), ref1[0])
                assert np.array_equal(o[1].download_fingerprint(), ref1[1])
                assert np.array_equal(f[0].download_fingerprint(), ref2[0])
    finally:
        rt.set_option(mg.OPT_ATTN_PERSISTENT, 0)


def test_fused_graph_matches_unfused_graph_on_device(rt):
    """The reference's integration check (cpp_examples/group_query_attn_inc_decode.cc:14-108): both
    graphs evaluated on the device from the reference fill, compared with has_same_fingerprint."""
    B, M, D, L = 2, 8, 64, 4096
    with mg.PyGraph(rt) as ref, mg.PyGraph(rt) as g:
        Q = ref.new_input((B, M, D))
        K = ref.new_input((B, D, L), layout=mg.DmemColumnMajor)
        V = ref.new_input((B, L, D), layout=mg.DmemColumnMajor)
        A = ref.matmul(Q, K)
        E = ref.exp(A)
        S = ref.reduction(E, 2)
        Dv = ref.div(E, S)
        O = ref.matmul(Dv, V)
        ref.fingerprint(refill_inputs=True)
        ins, o, f, plans = build_gqa(g, B, M, D, L, 16, 4)
        g.fingerprint(refill_inputs=True)
        assert O.has_same_fingerprint(f[0])
        assert not O.has_same_fingerprint(Dv) and not f[0].has_same_fingerprint(ins[0])
        x = [mo.reference_fill(t.shape) for t in ins]
        assert np.array_equal(O.download_fingerprint(), mo.unfused_attention_fp(*x))
        # un-fused intermediates against the oracle's kernel-level operators
        assert np.array_equal(A.download_fingerprint(), mo.kn_matmul_fp(x[0], x[1]))
        assert np.array_equal(S.download_fingerprint(), mo.kn_reduction_fp(mo.kn_exp_fp(mo.kn_matmul_fp(x[0], x[1])), 2))


def run_generic_fp(rt, specs, plan, seed):
    rng = np.random.default_rng(seed)
    with mg.PyGraph(rt) as g:
        ins = [g.new_input(s.dims, s.dtype, s.layout) for s in specs]
        x = [rng.integers(0, mo.FP_PQ, size=s.dims).astype(np.uint16) for s in specs]
        for t, v in zip(ins, x):
            t.upload_fingerprint(v)
        outs = g.customized(ins, to_package_plan(plan))
        g.fingerprint()
        got = [t.download_fingerprint() for t in outs]
    want = mo.run_fingerprint(mo.build_customized(specs, plan, max_smem=BIG), x)
    assert len(got) == len(want)
    for a, b in zip(got, want):
        assert np.array_equal(a, b)
    return x, got


def test_fingerprint_other_graphs(rt):
    """Graphs outside the attention pattern go through the generic interpreter."""
    # config-1 style matmul chain, grid over the intermediate columns, for-loop over K tiles of 64
    specs = [mo.DTensorSpec((16, 1024)), mo.DTensorSpec((1024, 1024)), mo.DTensorSpec((1024, 1024))]
    chain = mo.ExecutionPlan(
        ops=[(mo.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mo.TB_MATMUL_OP, [(3, 0), (2, 0)])],
        input_map=[(-1, -1, -1), (1, -1, -1), (0, -1, -1)], forloop_dim=[1, 0, -1],
        input_smem_layouts=[mo.SmemRowMajor] * 3, output_map=(1, -1, -1), forloop_range=16, grid_dim=(16, 1, 1),
        reduction_dimx=1024)
    x, got = run_generic_fp(rt, specs, chain, 1)
    total = got[0].astype(np.int64).reshape(16, 16, 1024).sum(axis=1) % mo.FP_PQ
    assert np.array_equal(total, mo.fp_matmul(mo.fp_matmul(x[0], x[1]), x[2]))
    # concat, exp, reduction, div with broadcasting, to_dimx; 3-D tensors split over grid x and z
    specs = [mo.DTensorSpec((4, 8, 32)), mo.DTensorSpec((4, 8, 32)), mo.DTensorSpec((4, 8, 64))]
    mixed = mo.ExecutionPlan(
        ops=[(mo.TB_CONCAT_2_OP, [(0, 0), (1, 0)]), (mo.TB_EXP_OP, [(3, 0)]), (mo.TB_REDUCTION_2_OP, [(4, 0)]),
             (mo.TB_DIV_OP, [(2, 0), (5, 0)]), (mo.TB_REDUCTION_2_TO_DIMX_OP, [(6, 0)])],
        input_map=[(0, -1, 1), (0, -1, 1), (0, -1, 1)], forloop_dim=[-1, -1, -1],
        input_smem_layouts=[mo.SmemRowMajor] * 3, output_map=(0, -1, 1), forloop_range=1, grid_dim=(4, 1, 2),
        reduction_dimx=16)
    run_generic_fp(rt, specs, mixed, 2)
    # identity: an input passed straight to an output keeps its raw values
    specs = [mo.DTensorSpec((6, 40))]
    ident = mo.ExecutionPlan(ops=[(mo.TB_REDUCTION_0_OP, [(0, 0)])], input_map=[(1, -1, -1)], forloop_dim=[0],
                             input_smem_layouts=[mo.SmemRowMajor], output_map=(1, -1, -1), forloop_range=3,
                             grid_dim=(5, 1, 1))
    run_generic_fp(rt, specs, ident, 3)


@pytest.mark.parametrize("mkn", [(1, 16, 16), (4, 16, 16), (5, 32, 48), (6, 48, 32), (16, 64, 1024), (33, 128, 64),
                                 (7, 24, 16), (8, 16, 24), (3, 5, 7)],
                         ids=lambda s: "x".join(map(str, s)))
def test_interpreter_matmul_shapes_and_full_range(runtime, mkn):
    """The interpreter's matmul - integer tensor cores where k and n are multiples of 16, scalar otherwise - on row
    counts that do not fill a 4-row group and on operands over the whole uint16 range (byte planes up to 255),
    for-loop accumulation included."""
    m, k, n = mkn
    F = 2
    runtime.set_max_smem(BIG)
    runtime.set_specialisation(0)
    try:
        rng = np.random.default_rng(m * 1000 + k * 10 + n)
        specs = [mo.DTensorSpec((m, F * k)), mo.DTensorSpec((F * k, n))]
        plan = mo.ExecutionPlan(ops=[(mo.TB_MATMUL_OP, [(0, 0), (1, 0)])], input_map=[(-1, -1, -1), (-1, -1, -1)],
                                forloop_dim=[1, 0], input_smem_layouts=[mo.SmemRowMajor] * 2, output_map=(-1, -1, -1),
                                forloop_range=F, grid_dim=(1, 1, 1))
        for hi in (mo.FP_PQ, 65536):
            x = [rng.integers(0, hi, size=s.dims).astype(np.uint16) for s in specs]
            with mg.PyGraph(runtime) as g:
                ins = [g.new_input(s.dims, s.dtype, s.layout) for s in specs]
                for t, v in zip(ins, x):
                    t.upload_fingerprint(v)
                outs = g.customized(ins, to_package_plan(plan))
                g.fingerprint()
                got = outs[0].download_fingerprint()
            want = (x[0].astype(np.int64) @ x[1].astype(np.int64)) % mo.FP_PQ
            assert np.array_equal(got.astype(np.int64), want), "operands below %d" % hi
    finally:
        runtime.set_specialisation(2)


@pytest.mark.parametrize("dtype", [mg.float16, mg.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("mkn", [(1, 16, 16), (4, 16, 8), (5, 32, 48), (16, 64, 1024), (33, 128, 64), (20, 48, 96),
                                 (7, 24, 16), (8, 16, 20), (3, 5, 7), (4, 64, 1600)],
                         ids=lambda s: "x".join(map(str, s)))
def test_float_interpreter_matmul_shapes(runtime, mkn, dtype):
    """The float interpreter's matmul: tensor cores (mma.sync, A staged as 16-bit rows, B rows padded when their
    dense pitch is a multiple of 128 bytes) when n % 8 == 0 and k % 16 == 0, for row counts that do not fill a
    16-row tile and for one or four n-tiles per warp; the CUDA cores otherwise, and when the staging room does not
    fit beside the tiles (the 64 x 1600 B tile); for-loop accumulation included.  A second plan feeds a computed
    (fp32) tile into the A side."""
    m, k, n = mkn
    F = 2
    runtime.set_max_smem(BIG)
    runtime.set_specialisation(0)
    try:
        rng = np.random.default_rng(m * 1000 + k * 10 + n)
        rnd = lambda a: from_bits(to_bits(a, dtype), dtype)
        specs = [mo.DTensorSpec((m, F * k), dtype), mo.DTensorSpec((F * k, n), dtype)]
        plan = mo.ExecutionPlan(ops=[(mo.TB_MATMUL_OP, [(0, 0), (1, 0)])], input_map=[(-1, -1, -1), (-1, -1, -1)],
                                forloop_dim=[1, 0], input_smem_layouts=[mo.SmemRowMajor] * 2, output_map=(-1, -1, -1),
                                forloop_range=F, grid_dim=(1, 1, 1))
        x = [rnd(rng.standard_normal(s.dims) * (1.0 if i == 0 else k ** -0.5)) for i, s in enumerate(specs)]
        with mg.PyGraph(runtime) as g:
            ins = [g.new_input(s.dims, s.dtype, s.layout) for s in specs]
            for t, a in zip(ins, x):
                t.upload_data(to_bits(a, dtype))
            outs = g.customized(ins, to_package_plan(plan))
            g.run()
            got = from_bits(outs[0].download_data(), dtype).reshape(outs[0].shape)
        assert_close(got, x[0].astype(np.float64) @ x[1].astype(np.float64), dtype, "A B")
        if m * n > 4096:  # the chained plan of the big shapes does not fit as fp32 tiles
            return
        # (A B) C with the computed product as the A operand of the second matmul; C is [n, 16]
        specs2 = specs + [mo.DTensorSpec((n, 16), dtype)]
        plan2 = mo.ExecutionPlan(ops=[(mo.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mo.TB_MATMUL_OP, [(3, 0), (2, 0)])],
                                 input_map=[(-1, -1, -1)] * 3, forloop_dim=[1, 0, -1],
                                 input_smem_layouts=[mo.SmemRowMajor] * 3, output_map=(-1, -1, -1), forloop_range=F,
                                 grid_dim=(1, 1, 1))
        x2 = x + [rnd(rng.standard_normal((n, 16)) * n ** -0.5)]
        with mg.PyGraph(runtime) as g:
            ins = [g.new_input(s.dims, s.dtype, s.layout) for s in specs2]
            for t, a in zip(ins, x2):
                t.upload_data(to_bits(a, dtype))
            outs = g.customized(ins, to_package_plan(plan2))
            g.run()
            got = from_bits(outs[0].download_data(), dtype).reshape(outs[0].shape)
        want = mo.run_float(mo.build_customized(specs2, plan2, max_smem=BIG), x2)[0]
        assert_close(got, want, dtype, "(A B) C")
    finally:
        runtime.set_specialisation(2)


def interpreter_corner_plans():
    """Plans that exercise the interpreters' own memory planning: operands stored with padded rows or not, tiles
    loaded once or every iteration, in-place exp on an input tile, a matmul adding straight into the accumulator."""
    P = mo.ExecutionPlan
    row = [mo.SmemRowMajor]
    return {
        # exp in place on an input tile that does not move with the for-loop (must be reloaded every iteration),
        # then used as the A operand; B (64 x 64: dense pitch 128 B) is padded
        "exp_on_invariant_input": ([(8, 64), (128, 64)],
                                   P(ops=[(mo.TB_EXP_OP, [(0, 0)]), (mo.TB_MATMUL_OP, [(2, 0), (1, 0)])],
                                     input_map=[(-1, -1, -1), (-1, -1, -1)], forloop_dim=[-1, 0], input_smem_layouts=row * 2,
                                     output_map=(-1, -1, -1), forloop_range=2, grid_dim=(1, 1, 1))),
        # the same loaded tile is B of one matmul and A of another: not padded
        "tile_as_a_and_b": ([(64, 64), (16, 64)],
                            P(ops=[(mo.TB_MATMUL_OP, [(1, 0), (0, 0)]), (mo.TB_MATMUL_OP, [(0, 0), (0, 0)]),
                                   (mo.TB_MATMUL_OP, [(2, 0), (3, 0)])],
                              input_map=[(-1, -1, -1), (-1, -1, -1)], forloop_dim=[-1, -1], input_smem_layouts=row * 2,
                              output_map=(-1, -1, -1), forloop_range=1, grid_dim=(1, 1, 1))),
        # a computed tile (matmul result) is the B operand of the next matmul; two outputs
        "computed_b_operand": ([(16, 32), (32, 64), (48, 16)],
                               P(ops=[(mo.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mo.TB_MATMUL_OP, [(2, 0), (3, 0)]),
                                      (mo.TB_REDUCTION_1_OP, [(3, 0)])],
                                 input_map=[(-1, -1, -1), (1, -1, -1), (-1, -1, -1)], forloop_dim=[-1, -1, -1],
                                 input_smem_layouts=row * 3, output_map=(1, -1, -1), forloop_range=1, grid_dim=(2, 1, 1))),
        # concat of two loaded tiles feeds a matmul as B; B rows of 64 elements; grid over y, for-loop over k
        "concat_into_matmul": ([(3, 8, 64), (3, 64, 32), (3, 64, 32)],
                               P(ops=[(mo.TB_CONCAT_2_OP, [(1, 0), (2, 0)]), (mo.TB_MATMUL_OP, [(0, 0), (3, 0)])],
                                 input_map=[(0, -1, -1), (0, -1, -1), (0, -1, -1)], forloop_dim=[2, 1, 1],
                                 input_smem_layouts=row * 3, output_map=(0, -1, -1), forloop_range=2, grid_dim=(3, 1, 1))),
        # wide padded B (16 x 256), loop-invariant, A moves with the for-loop; division by a loaded tile
        "invariant_wide_b": ([(4, 64), (16, 256), (4, 256)],
                             P(ops=[(mo.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mo.TB_DIV_OP, [(3, 0), (2, 0)])],
                               input_map=[(-1, -1, -1), (-1, -1, -1), (-1, -1, -1)], forloop_dim=[1, -1, -1],
                               input_smem_layouts=row * 3, output_map=(-1, -1, -1), forloop_range=4, grid_dim=(1, 1, 1))),
    }


@pytest.mark.parametrize("name", sorted(interpreter_corner_plans()))
def test_interpreter_corner_plans(runtime, name):
    dims, plan = interpreter_corner_plans()[name]
    runtime.set_max_smem(BIG)
    runtime.set_specialisation(0)
    try:
        specs = [mo.DTensorSpec(d) for d in dims]
        run_generic_fp(runtime, specs, plan, 5)
        rng = np.random.default_rng(6)
        # the third tensor (a divisor in one plan) stays away from zero
        x = [from_bits(to_bits(rng.standard_normal(s.dims) * 0.1 + (1.0 if i == 2 else 0.0), mg.float16), mg.float16)
             for i, s in enumerate(specs)]
        with mg.PyGraph(runtime) as g:
            ins = [g.new_input(s.dims, s.dtype, s.layout) for s in specs]
            for t, a in zip(ins, x):
                t.upload_data(to_bits(a, mg.float16))
            outs = g.customized(ins, to_package_plan(plan))
            g.run()
            got = [from_bits(t.download_data(), mg.float16).reshape(t.shape) for t in outs]
        want = mo.run_float(mo.build_customized(specs, plan, max_smem=BIG), x)
        assert len(got) == len(want)
        for a, b in zip(got, want):
            assert_close(a, b, mg.float16, name)
    finally:
        runtime.set_specialisation(2)


def float_inputs(rng, B, M, D, L, kl, vl, dtype):
    """Logical tensors rounded to storage precision, plus their memory images."""
    rnd = lambda a: from_bits(to_bits(a, dtype), dtype)
    q = rnd(rng.standard_normal((B, M, D)) / np.sqrt(D))  # 1/sqrt(d) folded into Q on the host
    k = rnd(rng.standard_normal((B, D, L)))
    v = rnd(rng.standard_normal((B, L, D)))
    mem = [q, k if kl == mg.DmemRowMajor else np.ascontiguousarray(k.transpose(0, 2, 1)),
           v if vl == mg.DmemRowMajor else np.ascontiguousarray(v.transpose(0, 2, 1))]
    return (q, k, v), mem


@pytest.mark.parametrize("dtype", [mg.float16, mg.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("layouts", [(mg.DmemColumnMajor, mg.DmemColumnMajor), (mg.DmemRowMajor, mg.DmemRowMajor),
                                     (mg.DmemColumnMajor, mg.DmemRowMajor)], ids=["kc_vc", "kr_vr", "kc_vr"])
@pytest.mark.parametrize("shape", [(2, 4, 128, 1024, 4, 4), (2, 8, 64, 512, 2, 4), (1, 32, 128, 1024, 4, 2),
                                   (3, 1, 32, 96, 3, 2), (2, 20, 128, 2048, 2, 16), (1, 7, 64, 1024, 2, 8),
                                   # 176 (head, split) work items of four 128-wide tiles: more items than SMs, so
                                   # the persistent tensor-memory kernel walks several items per block
                                   (11, 24, 128, 8192, 16, 8)])
def test_float_gqa_vs_fp32_oracle(rt, shape, layouts, dtype):
    B, M, D, L, S, F = shape
    kl, vl = layouts
    rng = np.random.default_rng(sum(shape))
    with mg.PyGraph(rt) as g:
        ins, o, f, plans = build_gqa(g, B, M, D, L, S, F, kl, vl, dtype)
        (q, k, v), mem = float_inputs(rng, B, M, D, L, kl, vl, dtype)
        for t, a in zip(ins, mem):
            t.upload_data(to_bits(a, dtype))
        g.run()
        og1 = mo.build_customized([spec_of(t) for t in ins], to_oracle_plan(plans[0]), max_smem=BIG)
        ref1 = mo.run_float(og1, mem)
        assert_close(from_bits(o[0].download_data(), dtype).reshape(o[0].shape), ref1[0], dtype, "O_part")
        assert_close(from_bits(o[1].download_data(), dtype).reshape(o[1].shape), ref1[1], dtype, "R_part")
        final = from_bits(f[0].download_data(), dtype).reshape(f[0].shape)
        assert_close(final, mo.attention_fp32(q, k, v), dtype, "O vs un-fused fp32 attention")


def test_float_causal_window_extension(runtime):
    """Speculative-decode mask (float-mode extension of the split-KV attention kernel): 8 draft tokens x
    group 4 = 32 query rows; fingerprint mode is unaffected by the mask."""
    B, M, D, L, S, F, W = 2, 32, 128, 2048, 8, 4, 8
    rng = np.random.default_rng(31)
    runtime.set_specialisation(True)
    with mg.PyGraph(runtime) as g:
        ins, o, f, plans = build_gqa(g, B, M, D, L, S, F)
        g.set_causal_window(3, W)
        assert g.customized_info(3)["kernel_float"] == mg.KERNEL_ATTN_SPLIT
        (q, k, v), mem = float_inputs(rng, B, M, D, L, mg.DmemColumnMajor, mg.DmemColumnMajor, mg.float16)
        for t, a in zip(ins, mem):
            t.upload_data(to_bits(a, mg.float16))
        g.run()
        final = from_bits(f[0].download_data(), mg.float16).reshape(f[0].shape)
        assert_close(final, mo.attention_fp32_causal_window(q, k, v, W), mg.float16, "masked output")
        unmasked = mo.attention_fp32(q, k, v)
        assert np.abs(final - unmasked).max() > 1e-3  # the mask does change the result
        x = [rng.integers(0, mo.FP_PQ, size=t.shape).astype(np.uint16) for t in ins]
        for t, a in zip(ins, x):
            t.upload_fingerprint(a)
        g.fingerprint()
        assert np.array_equal(f[0].download_fingerprint(), mo.unfused_attention_fp(*x))


def test_specialised_kernels_are_selected(runtime):
    runtime.set_specialisation(True)
    with mg.PyGraph(runtime) as g:
        build_gqa(g, 8, 4, 128, 4096, 16, 4)
        i1, i2 = g.customized_info(3), g.customized_info(4)
        assert i1["kernel_fingerprint"] == mg.KERNEL_ATTN_SPLIT and i1["kernel_float"] == mg.KERNEL_ATTN_SPLIT
        assert i2["kernel_fingerprint"] == mg.KERNEL_ATTN_MERGE and i2["kernel_float"] == mg.KERNEL_ATTN_MERGE
    runtime.set_specialisation(False)
    with mg.PyGraph(runtime) as g:
        build_gqa(g, 8, 4, 128, 4096, 16, 4)
        assert g.customized_info(3)["kernel_float"] == mg.KERNEL_INTERPRETER
    runtime.set_specialisation(True)


def test_float_baseline_c2_full_size(rt):
    """BASELINE config: 8 KV heads, group 4, head_dim 128, KV 4096, 16 splits, KV tiles of 64, fp16."""
    B, M, D, L, S, F = 8, 4, 128, 4096, 16, 4
    rng = np.random.default_rng(2024)
    with mg.PyGraph(rt) as g:
        ins, o, f, plans = build_gqa(g, B, M, D, L, S, F)
        (q, k, v), mem = float_inputs(rng, B, M, D, L, mg.DmemColumnMajor, mg.DmemColumnMajor, mg.float16)
        for t, a in zip(ins, mem):
            t.upload_data(to_bits(a, mg.float16))
        g.run()
        final = from_bits(f[0].download_data(), mg.float16).reshape(f[0].shape)
        assert_close(final, mo.attention_fp32(q, k, v), mg.float16, "C2 output")
        ms = g.profile_op(3, warmup=3, iters=5)
        assert 0 < ms < 1000


def test_float_spec_decode_c3_full_size(runtime):
    """BASELINE config 3 at full size: 32 (batch x KV head) units, 8 draft tokens x group 4 = 32 query rows, KV 8192,
    16 splits x for-loop 8, causal draft window, K column-major / V row-major as the benchmark runs it: 512 work items
    on the persistent tcgen05 kernel (3 or 4 per block) plus the merge kernel; the `mma.sync` engine on the same
    inputs must agree with the same oracle."""
    B, M, D, L, S, F, W = 32, 32, 128, 8192, 16, 8, 8
    rng = np.random.default_rng(33)
    runtime.set_max_smem(BIG)
    runtime.set_specialisation(True)
    kl, vl = mg.DmemColumnMajor, mg.DmemRowMajor
    with mg.PyGraph(runtime) as g:
        ins, o, f, plans = build_gqa(g, B, M, D, L, S, F, kl, vl)
        g.set_causal_window(3, W)
        (q, k, v), mem = float_inputs(rng, B, M, D, L, kl, vl, mg.float16)
        for t, a in zip(ins, mem):
            t.upload_data(to_bits(a, mg.float16))
        want = mo.attention_fp32_causal_window(q, k, v, W)
        for engine in (mg.ENGINE_TCGEN05, mg.ENGINE_MMA_SYNC):
            runtime.set_option(mg.OPT_ATTN_ENGINE, engine)
            try:
                g.run()
                g.run()  # again: barriers, tensor memory and the launch order are set up afresh by every launch
            finally:
                runtime.set_option(mg.OPT_ATTN_ENGINE, mg.ENGINE_AUTO)
            final = from_bits(f[0].download_data(), mg.float16).reshape(f[0].shape)
            assert_close(final, want, mg.float16, "masked output, engine %d" % engine)
        # The batched entry point on the same graph (two sets, the second one a permutation of the heads): its
        # partials are scratch, so the tcgen05 kernel deals single tiles to its blocks and sums what a block holds
        # of a head (13 or 14 tiles of 64; five or six partial sums per head), and the merge reads those slots only.
        import torch
        perm = rng.permutation(B)
        sets = [mem, [a[perm] for a in mem]]
        dev = [torch.from_numpy(np.stack([to_bits(sets[s][i], mg.float16) for s in range(2)]).astype(np.int16)).cuda() for i in range(3)]
        res = torch.zeros((2,) + tuple(f[0].shape), dtype=torch.int16, device="cuda")
        wbytes = g.run_batched_workspace(2)
        work = torch.empty(max(wbytes, 256), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        for _ in range(2):
            res.zero_()
            torch.cuda.synchronize()
            g.run_batched(2, [d.data_ptr() for d in dev], res.data_ptr(), work.data_ptr(), wbytes)
            mg.synchronize()
            got = from_bits(res.cpu().numpy().view(np.uint16), mg.float16)
            assert_close(got[0], want, mg.float16, "batched, set 0")
            assert_close(got[1], want[perm], mg.float16, "batched, set 1")


def build_prefill(g, H, SQ, D, L, dtype, kl=mg.DmemColumnMajor, vl=mg.DmemColumnMajor):
    Q = g.new_input((H, SQ, D), dtype)
    K = g.new_input((H, D, L), dtype, kl)
    V = g.new_input((H, L, D), dtype, vl)
    p1, p2 = mg.attention_prefill_plans(H, SQ, D, L)
    acc = g.customized([Q, K, V], p1)
    out = g.customized(acc, p2)
    return (Q, K, V), acc, out, (p1, p2)


@pytest.mark.parametrize("dtype", [mg.bfloat16, mg.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("layouts", [(mg.DmemColumnMajor, mg.DmemColumnMajor), (mg.DmemRowMajor, mg.DmemRowMajor),
                                     (mg.DmemColumnMajor, mg.DmemRowMajor), (mg.DmemRowMajor, mg.DmemColumnMajor)],
                         ids=["kc_vc", "kr_vr", "kc_vr", "kr_vc"])
@pytest.mark.parametrize("shape", [(2, 256, 512), (1, 128, 128), (3, 384, 1024), (2, 512, 1024)])
def test_float_prefill_tensor_core_kernel(runtime, shape, layouts, dtype):
    """Dense attention on tcgen05 / tensor memory (128 x 128 tiles) against the fp32 evaluation.  Query lengths that
    are multiples of 256 run on the two-tiles-per-block kernel (every K / V layout), the others on the one-tile kernel
    (K and V column-major only)."""
    H, SQ, L = shape
    D = 128
    kl, vl = layouts
    if SQ % 256 != 0 and layouts != (mg.DmemColumnMajor, mg.DmemColumnMajor):
        pytest.skip("the one-tile kernel takes K and V column-major only")
    runtime.set_max_smem(BIG)
    runtime.set_specialisation(2)
    rng = np.random.default_rng(H * 7 + SQ + L)
    with mg.PyGraph(runtime) as g:
        ins, acc, out, plans = build_prefill(g, H, SQ, D, L, dtype, kl, vl)
        assert g.customized_info(3)["kernel_float"] == mg.KERNEL_ATTN_ROWS
        (q, k, v), mem = float_inputs(rng, H, SQ, D, L, kl, vl, dtype)
        for t, a in zip(ins, mem):
            t.upload_data(to_bits(a, dtype))
        g.run()
        og1 = mo.build_customized([spec_of(t) for t in ins], to_oracle_plan(plans[0]), max_smem=BIG)
        ref1 = mo.run_float(og1, mem)
        assert_close(from_bits(acc[0].download_data(), dtype).reshape(acc[0].shape), ref1[0], dtype, "O_acc")
        assert_close(from_bits(acc[1].download_data(), dtype).reshape(acc[1].shape), ref1[1], dtype, "R")
        final = from_bits(out[0].download_data(), dtype).reshape(out[0].shape)
        assert_close(final, mo.attention_fp32(q, k, v), dtype, "O vs un-fused fp32 attention")
        # run again: tensor memory and barriers are set up afresh by every launch
        g.run()
        again = from_bits(out[0].download_data(), dtype).reshape(out[0].shape)
        assert np.array_equal(final, again)


def test_prefill_calls_back_to_back_on_one_stream(runtime):
    """Dense attention launches let the next kernel of the stream start while they drain, and read their inputs before
    the kernel in front has finished when the library knows that kernel did not write them.  A stream of calls - two
    graphs taking turns, each several times, nothing synchronised in between - leaves in every graph what one call
    alone leaves; and a call whose input is the output of the call in front waits for it."""
    import torch
    H, SQ, L, D = 4, 512, 1024, 128
    runtime.set_max_smem(BIG)
    runtime.set_specialisation(2)
    rng = np.random.default_rng(77)
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream
    with mg.PyGraph(runtime) as ga, mg.PyGraph(runtime) as gb:
        built = []
        for g in (ga, gb):
            ins, acc, out, plans = build_prefill(g, H, SQ, D, L, mg.bfloat16)
            (q, k, v), mem = float_inputs(rng, H, SQ, D, L, mg.DmemColumnMajor, mg.DmemColumnMajor, mg.bfloat16)
            for t, a in zip(ins, mem):
                t.upload_data(to_bits(a, mg.bfloat16))
            g.run()
            built.append((ins, out, from_bits(out[0].download_data(), mg.bfloat16).copy(), mem))
        for _ in range(6):
            ga.run(stream=sh, sync=False)
            gb.run(stream=sh, sync=False)
        stream.synchronize()
        mg.synchronize()
        for ins, out, alone, _ in built:
            assert np.array_equal(from_bits(out[0].download_data(), mg.bfloat16), alone)
        # graph B takes its Q from graph A's output: B's loads must wait for A although B is launched to overlap it
        (qa, _, _), out_a, _, mem_a = built[0]
        _, out_b, _, _ = built[1]
        gb.rebind_input(0, data_ptr=out_a[0].pod.data_ptr)
        ga.run()
        gb.run()
        stale = from_bits(out_b[0].download_data(), mg.bfloat16).copy()
        q2 = float_inputs(rng, H, SQ, D, L, mg.DmemColumnMajor, mg.DmemColumnMajor, mg.bfloat16)[1][0]
        qa.upload_data(to_bits(q2, mg.bfloat16))
        for _ in range(3):
            ga.run(stream=sh, sync=False)
            gb.run(stream=sh, sync=False)
        stream.synchronize()
        mg.synchronize()
        chained = from_bits(out_b[0].download_data(), mg.bfloat16).copy()
        ga.run()
        gb.run()
        assert np.array_equal(chained, from_bits(out_b[0].download_data(), mg.bfloat16))
        assert not np.array_equal(chained, stale)


def test_decode_calls_released_early_wait_for_an_older_producer(runtime):
    """A one-call decode launch (128 blocks) releases its successor as soon as it starts, so a call may run beside the
    TWO calls in front of it.  Three graphs on one stream, nothing synchronised: A writes a tensor, X has nothing to do
    with it, B takes its Q from A's output.  B must see what the A two launches in front of it wrote, every time."""
    import torch
    B_, M, D, L, S, F = 8, 4, 128, 4096, 16, 4
    runtime.set_max_smem(BIG)
    runtime.set_specialisation(2)
    rng = np.random.default_rng(4242)
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream
    with mg.PyGraph(runtime) as ga, mg.PyGraph(runtime) as gx, mg.PyGraph(runtime) as gb:
        built = []
        for g in (ga, gx, gb):
            ins, o, f, plans = build_gqa(g, B_, M, D, L, S, F)
            (q, k, v), mem = float_inputs(rng, B_, M, D, L, mg.DmemColumnMajor, mg.DmemColumnMajor, mg.float16)
            for t, a in zip(ins, mem):
                t.upload_data(to_bits(a, mg.float16))
            built.append((ins, f))
        (qa, _, _), fa = built[0]
        _, fb = built[2]
        gb.rebind_input(0, data_ptr=fa[0].pod.data_ptr)
        results = []
        for trial in range(4):
            q_new = float_inputs(rng, B_, M, D, L, mg.DmemColumnMajor, mg.DmemColumnMajor, mg.float16)[1][0]
            qa.upload_data(to_bits(q_new, mg.float16))
            for _ in range(3):  # A, X, B back to back; B's input is rewritten by every A
                ga.run(stream=sh, sync=False)
                gx.run(stream=sh, sync=False)
                gb.run(stream=sh, sync=False)
            stream.synchronize()
            mg.synchronize()
            chained = from_bits(fb[0].download_data(), mg.float16).copy()
            ga.run()
            gb.run()
            assert np.array_equal(chained, from_bits(fb[0].download_data(), mg.float16)), "trial %d" % trial
            results.append(chained)
        assert not np.array_equal(results[0], results[1])


def test_prefill_fingerprint_uses_interpreter(runtime):
    """The same dense graph in fingerprint mode (128 x 128 x 128 mod-PQ contractions) stays bit-exact."""
    H, SQ, D, L = 1, 128, 128, 256
    runtime.set_max_smem(BIG)
    rng = np.random.default_rng(12)
    with mg.PyGraph(runtime) as g:
        ins, acc, out, plans = build_prefill(g, H, SQ, D, L, mg.bfloat16)
        x = [rng.integers(0, mo.FP_PQ, size=t.shape).astype(np.uint16) for t in ins]
        for t, a in zip(ins, x):
            t.upload_fingerprint(a)
        g.fingerprint()
        assert np.array_equal(out[0].download_fingerprint(), mo.unfused_attention_fp(*x))


def test_float_other_graph_generic(rt):
    """Matmul chain in float mode through the generic interpreter."""
    rng = np.random.default_rng(9)
    specs = [mo.DTensorSpec((16, 256)), mo.DTensorSpec((256, 128)), mo.DTensorSpec((128, 64))]
    plan = mo.ExecutionPlan(
        ops=[(mo.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mo.TB_MATMUL_OP, [(3, 0), (2, 0)])],
        input_map=[(-1, -1, -1), (1, -1, -1), (0, -1, -1)], forloop_dim=[1, 0, -1],
        input_smem_layouts=[mo.SmemRowMajor] * 3, output_map=(1, -1, -1), forloop_range=4, grid_dim=(4, 1, 1),
        reduction_dimx=64)
    x = [from_bits(to_bits(rng.standard_normal(s.dims) * 0.05, mg.float16), mg.float16) for s in specs]
    with mg.PyGraph(rt) as g:
        ins = [g.new_input(s.dims, s.dtype, s.layout) for s in specs]
        for t, a in zip(ins, x):
            t.upload_data(to_bits(a, mg.float16))
        outs = g.customized(ins, to_package_plan(plan))
        g.run()
        got = from_bits(outs[0].download_data(), mg.float16).reshape(outs[0].shape)
    want = mo.run_float(mo.build_customized(specs, plan), x)[0]
    assert_close(got, want, mg.float16, "chain partials")


@pytest.mark.parametrize("dtype", [mg.float16, mg.bfloat16], ids=["fp16", "bf16"])
def test_float_matmul_chain_c1_full_size(rt, dtype):
    """BASELINE config 1 at full size in float mode: X[16,1024] W1[1024,1024] W2[1024,1024], grid over the
    intermediate columns, for-loop over K tiles of 64, then the cross-block reduction; both customized ops go
    through the generic float interpreter (16-bit input tiles, fp32 computed tiles, tensor-core matmuls: 211 KB of shared memory)."""
    rng = np.random.default_rng(31)
    specs = [mo.DTensorSpec((16, 1024), dtype), mo.DTensorSpec((1024, 1024), dtype), mo.DTensorSpec((1024, 1024), dtype)]
    chain = mo.ExecutionPlan(
        ops=[(mo.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mo.TB_MATMUL_OP, [(3, 0), (2, 0)])],
        input_map=[(-1, -1, -1), (1, -1, -1), (0, -1, -1)], forloop_dim=[1, 0, -1],
        input_smem_layouts=[mo.SmemRowMajor] * 3, output_map=(1, -1, -1), forloop_range=16, grid_dim=(16, 1, 1),
        reduction_dimx=1024)
    reduce_plan = mo.ExecutionPlan(ops=[(mo.TB_REDUCTION_1_TO_DIMX_OP, [(0, 0)])], input_map=[(0, -1, -1)],
                                   forloop_dim=[-1], input_smem_layouts=[mo.SmemRowMajor], output_map=(0, -1, -1),
                                   forloop_range=1, grid_dim=(16, 1, 1), reduction_dimx=1024)
    # N(0, 1/32) keeps X W1 W2 at unit scale (the named N(0, 0.02) would push the partial sums into fp16 subnormals)
    x = [from_bits(to_bits(rng.standard_normal(s.dims) / 32.0 * (32.0 if i == 0 else 1.0), dtype), dtype)
         for i, s in enumerate(specs)]
    with mg.PyGraph(rt) as g:
        ins = [g.new_input(s.dims, dtype, s.layout) for s in specs]
        for t, a in zip(ins, x):
            t.upload_data(to_bits(a, dtype))
        part = g.customized(ins, to_package_plan(chain))
        outs = g.customized(part, to_package_plan(reduce_plan))
        g.run()
        got_part = from_bits(part[0].download_data(), dtype).reshape(part[0].shape)
        got = from_bits(outs[0].download_data(), dtype).reshape(outs[0].shape)
    g1 = mo.build_customized(specs, chain, max_smem=BIG)
    want_part = mo.run_float(g1, x)[0]
    assert_close(got_part, want_part, dtype, "chain partials")
    # the second op reads the 16-bit partials the first one stored
    g2 = mo.build_customized(mo.output_specs(g1), reduce_plan, max_smem=BIG)
    want = mo.run_float(g2, [got_part])[0]
    assert_close(got, want, dtype, "chain result")
    exact = (x[0].astype(np.float64) @ x[1].astype(np.float64)) @ x[2].astype(np.float64)
    assert_close(got, exact, dtype, "chain result vs fp64 product")


@pytest.mark.parametrize("shape", [(2, 4, 64, 512, 4, 2, 5), (4, 4, 128, 512, 4, 2, 150), (3, 3, 64, 384, 3, 2, 97)],
                         ids=["few_sets", "whole_heads_per_block", "three_splits"])
def test_batched_fingerprint_sets(rt, shape):
    """Many independent input sets in one pass equal per-set evaluations by the oracle (with many sets a block of the
    fused kernel sums runs of consecutive splits of a head; modulo arithmetic makes that exact)."""
    import torch
    B, M, D, L, S, F, nsets = shape
    rng = np.random.default_rng(77)
    with mg.PyGraph(rt) as g:
        ins, o, f, plans = build_gqa(g, B, M, D, L, S, F)
        xs = [[rng.integers(0, mo.FP_P, size=t.shape).astype(np.uint16) for t in ins] for _ in range(nsets)]
        dev = [torch.from_numpy(np.stack([xs[s][i] for s in range(nsets)]).astype(np.int16)).cuda() for i in range(3)]
        out = torch.zeros((nsets,) + f[0].shape, dtype=torch.int16, device="cuda")
        wbytes = g.fingerprint_batched_workspace(nsets)
        work = torch.zeros(max(wbytes, 16), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        g.fingerprint_batched(nsets, [d.data_ptr() for d in dev], out.data_ptr(), work.data_ptr(), wbytes)
        mg.synchronize()
        got = out.cpu().numpy().view(np.uint16)
        for s in sorted(set(range(0, nsets, max(1, nsets // 12))) | {nsets - 1}):
            _, ref2 = oracle_fp(ins, plans, xs[s])
            assert np.array_equal(got[s], ref2[0]), "set %d" % s
        # every set: the same launch with one block per (set, head, split) item
        first = got.copy()
        rt.set_option(mg.OPT_ATTN_PERSISTENT, 1)
        try:
            out.zero_()
            torch.cuda.synchronize()
            g.fingerprint_batched(nsets, [d.data_ptr() for d in dev], out.data_ptr(), work.data_ptr(), wbytes)
            mg.synchronize()
        finally:
            rt.set_option(mg.OPT_ATTN_PERSISTENT, 0)
        assert np.array_equal(out.cpu().numpy().view(np.uint16), first)


def test_unsupported_is_an_error_not_a_fallback(rt):
    """A graph too large for the generic float interpreter is refused with a status code."""
    with mg.PyGraph(rt) as g:
        specs = [(1, 128, 128), (1, 128, 128)]
        A = g.new_input(specs[0])
        Bt = g.new_input(specs[1])
        plan = mg.ExecutionPlan(ops=[(mg.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mg.TB_EXP_OP, [(2, 0)]),
                                     (mg.TB_MATMUL_OP, [(3, 0), (1, 0)]), (mg.TB_MATMUL_OP, [(4, 0), (1, 0)])],
                                input_map=[(0, -1, -1), (0, -1, -1)], forloop_dim=[-1, -1],
                                input_smem_layouts=[mg.SmemRowMajor] * 2, output_map=(0, -1, -1), forloop_range=1,
                                grid_dim=(1, 1, 1))
        outs = g.customized([A, Bt], plan)  # two 16-bit input tiles of 32 KB + three fp32 tiles of 64 KB = 256 KB
        with pytest.raises(mg.MuGraphError) as e:
            g.run()
        assert e.value.status == 5
        A.upload_fingerprint(np.ones(A.shape, np.uint16))
        Bt.upload_fingerprint(np.ones(Bt.shape, np.uint16))
        g.fingerprint()  # fingerprint mode fits (2-byte tiles)
        assert outs[0].download_fingerprint().shape == (1, 128, 128)
