"""CPU tests of the host C++ (graph building, validation, shared-memory planning, lowering, kernel
selection) through the C ABI on a planning-only runtime, checked against the oracle's restatement of
the reference's host logic and against the reference-host golden metadata."""
import json
import os

import pytest

import attention_superoptimizer_b200 as mg
from oracle import mugraph_oracle as mo
from tests.helpers import spec_of, to_oracle_plan

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "gqa_decode_reference_host.json")


def build_gqa(g, B, M, D, L, S, F, kl=mg.DmemColumnMajor, vl=mg.DmemColumnMajor, dtype=mg.float16):
    Q = g.new_input((B, M, D), dtype)
    K = g.new_input((B, D, L), dtype, kl)
    V = g.new_input((B, L, D), dtype, vl)
    p1, p2 = mg.gqa_decode_plans(B, M, D, L, S, F)
    o = g.customized([Q, K, V], p1)
    f = g.customized(o, p2)
    return (Q, K, V), o, f, (p1, p2)


def check_program_against_oracle(prog, og):
    """Every stride / offset of the lowered program equals the oracle's (reference graph.cc:106-239)."""
    assert prog.num_ops == len(og.ops) and prog.smem_bytes == og.smem_offset
    assert list(prog.grid) == list(og.grid_dim) and prog.forloop_range == og.forloop_range
    for i, op in enumerate(og.ops):
        a = list(prog.ops[i].a)
        assert prog.ops[i].type == op.type
        if op.type == mo.TB_INPUT_OP:
            rbs, cbs, rfs, cfs, gbs, gfs = mo._input_offsets(og, op)
            st = op.outputs[0]
            assert a[0:3] == rbs and a[3:6] == cbs and a[6] == rfs and a[7] == cfs
            assert a[8:11] == gbs and a[11] == gfs
            assert a[12:14] == list(op.dtensor.dims[-2:]) and a[14:16] == st.dims[-2:]
            assert a[16] == op.dtensor.layout and a[17] == st.smem_offset
        elif op.type == mo.TB_OUTPUT_OP:
            rbs, cbs, gbs = mo._output_offsets(og, op)
            assert a[0:3] == rbs and a[3:6] == cbs and a[6:9] == gbs
            assert a[9:11] == list(op.out_dtensor.dims[-2:]) and a[11:13] == op.inputs[0].dims[-2:]
            assert a[13] == op.inputs[0].smem_offset and a[14] == op.outputs[0].smem_offset
        elif op.type == mo.TB_MATMUL_OP:
            A, B, C = op.inputs[0], op.inputs[1], op.outputs[0]
            assert a[0:6] == [A.dims[-2], B.dims[-1], A.dims[-1], A.smem_offset, B.smem_offset, C.smem_offset]
        elif op.type == mo.TB_EXP_OP:
            assert a[0:2] == [op.inputs[0].smem_offset, op.inputs[0].num_elements]
        elif op.type in (mo.TB_DIV_OP, mo.TB_ADD_OP):
            assert a[0:3] == mo._bcast3(op.inputs[0]) and a[3:6] == mo._bcast3(op.inputs[1])
            assert a[6:9] == [op.inputs[0].smem_offset, op.inputs[1].smem_offset, op.outputs[0].smem_offset]
        elif mo.TB_REDUCTION_0_OP <= op.type <= mo.TB_REDUCTION_2_TO_DIMX_OP:
            n, deg, inner = mo._reduction_params(op)
            assert a[0:5] == [n, deg, inner, op.inputs[0].smem_offset, op.outputs[0].smem_offset]


@pytest.mark.parametrize("shape", [(2, 8, 64, 4096, 16, 4), (8, 4, 128, 4096, 16, 4), (32, 32, 128, 8192, 16, 8),
                                   (3, 1, 8, 48, 3, 2)])
def test_gqa_graph_plan_matches_oracle_and_reference_golden(planning_runtime, shape):
    B, M, D, L, S, F = shape
    with mg.PyGraph(planning_runtime) as g:
        ins, o, f, (p1, p2) = build_gqa(g, *shape)
        assert [t.shape for t in o] == [(B, M, S * D), (B, M, S)] and f[0].shape == (B, M, D)
        og1 = mo.build_customized([spec_of(t) for t in ins], to_oracle_plan(p1), max_smem=227 * 1024)
        og2 = mo.build_customized([spec_of(t) for t in o], to_oracle_plan(p2), max_smem=227 * 1024)
        check_program_against_oracle(g.customized_program(3), og1)
        check_program_against_oracle(g.customized_program(4), og2)
        for c in json.load(open(GOLDEN))["cases"]:
            if (c["B"], c["M"], c["D"], c["L"], c["S"], c["F"]) == shape:
                i1, i2 = g.customized_info(3), g.customized_info(4)
                assert i1["num_tb_operators"] == c["op1"]["num_ops"] and i1["smem_bytes"] == c["op1"]["smem_bytes"]
                assert i2["num_tb_operators"] == c["op2"]["num_ops"] and i2["smem_bytes"] == c["op2"]["smem_bytes"]
    used, _ = planning_runtime.arena_usage()
    assert used <= 2048  # everything was released in LIFO order; only the tables remain


def test_invalid_plans_return_invalid_graph(planning_runtime):
    with mg.PyGraph(planning_runtime) as g:
        Q = g.new_input((2, 4, 16))
        K = g.new_input((2, 16, 64))
        V = g.new_input((2, 64, 16))
        p1, _ = mg.gqa_decode_plans(2, 4, 16, 64, 4, 2)
        cases = {
            "grid does not divide": dict(grid_dim=(2, 3, 1)),
            "for-loop does not divide": dict(forloop_range=5),
            "matmul inner dims differ": dict(ops=[(mg.TB_MATMUL_OP, [(0, 0), (2, 0)])]),
            "operand refers forward": dict(ops=[(mg.TB_EXP_OP, [(7, 0)])]),
            "unknown operator": dict(ops=[(2999, [(0, 0)])]),
            "leading tile dim > 1": dict(input_map=[(-1, -1, -1), (0, 2, -1), (0, 1, -1)]),
            "zero for-loop": dict(forloop_range=0),
        }
        for why, change in cases.items():
            bad = mg.ExecutionPlan(**{**p1.__dict__, **change})
            with pytest.raises(mg.MuGraphError) as e:
                g.customized([Q, K, V], bad)
            assert e.value.status == 2, why
        with pytest.raises(mg.MuGraphError) as e:
            g.customized([Q, K], p1)
        assert e.value.status == 2
        assert g.num_operators == 3  # nothing half-built was left behind
        # reduction needs a row-major tile: Q is loaded with a tensor-op layout tag
        bad = mg.ExecutionPlan(ops=[(mg.TB_REDUCTION_2_OP, [(0, 0)])], input_map=[(0, -1, -1)], forloop_dim=[-1],
                               input_smem_layouts=[mg.SmemRowMajorTensorOpMultiplicand_Crosswise64],
                               output_map=(0, -1, -1), forloop_range=1, grid_dim=(2, 1, 1))
        with pytest.raises(mg.MuGraphError):
            g.customized([Q], bad)


def test_shared_memory_budget_is_enforced(planning_runtime):
    planning_runtime.set_max_smem(96 * 1024)  # the reference's limit
    with mg.PyGraph(planning_runtime) as g:
        Q = g.new_input((1, 128, 128))
        K = g.new_input((1, 128, 2048))
        V = g.new_input((1, 2048, 128))
        p1, _ = mg.gqa_decode_plans(1, 128, 128, 2048, 1, 16)
        with pytest.raises(mg.MuGraphError) as e:
            g.customized([Q, K, V], p1)  # 128x128 tiles: needs ~200 KB in this plan
        assert e.value.status == 2
        planning_runtime.set_max_smem(227 * 1024)
        out = g.customized([Q, K, V], p1)
        assert out[0].shape == (1, 128, 128)


def test_arena_exhaustion_is_reported(planning_runtime):
    with mg.PyGraph(planning_runtime) as g:
        with pytest.raises(mg.MuGraphError) as e:
            g.new_input((1024, 1024, 1024))  # 2 GiB data + 2 GiB fingerprints > 1 GiB arena
        assert e.value.status == 3
        a = g.new_input((4, 4))
        assert a.shape == (4, 4)


def test_kernel_selection_and_launch_refusal(planning_runtime):
    with mg.PyGraph(planning_runtime) as g:
        build_gqa(g, 8, 4, 128, 4096, 16, 4)
        info = g.customized_info(3)
        assert info["kernel_fingerprint"] in (mg.KERNEL_INTERPRETER, mg.KERNEL_ATTN_SPLIT)
        with pytest.raises(mg.MuGraphError) as e:
            g.fingerprint()
        assert e.value.status == 7  # no device: refuses instead of computing on the CPU
        with pytest.raises(mg.MuGraphError) as e:
            g.run()
        assert e.value.status == 7


def test_matmul_chain_and_reduction_patterns_are_recognised(planning_runtime):
    """The lowered programs of the matmul-chain operator and of a single-reduction operator select their kernels;
    a chain whose second right operand moves with the for-loop does not (it stays on the interpreters)."""
    chain = mg.ExecutionPlan(ops=[(mg.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mg.TB_MATMUL_OP, [(3, 0), (2, 0)])],
                             input_map=[(-1, -1, -1), (1, -1, -1), (0, -1, -1)], forloop_dim=[1, 0, -1],
                             input_smem_layouts=[mg.SmemRowMajor] * 3, output_map=(1, -1, -1), forloop_range=16,
                             grid_dim=(16, 1, 1), reduction_dimx=1024)
    reduce_plan = mg.ExecutionPlan(ops=[(mg.TB_REDUCTION_1_TO_DIMX_OP, [(0, 0)])], input_map=[(0, -1, -1)],
                                   forloop_dim=[-1], input_smem_layouts=[mg.SmemRowMajor], output_map=(0, -1, -1),
                                   forloop_range=1, grid_dim=(16, 1, 1), reduction_dimx=1024)
    planning_runtime.set_max_smem(227 * 1024)
    with mg.PyGraph(planning_runtime) as g:
        X = g.new_input((16, 1024)); W1 = g.new_input((1024, 1024)); W2 = g.new_input((1024, 1024))
        part = g.customized([X, W1, W2], chain)
        g.customized(part, reduce_plan)
        i1, i2 = g.customized_info(3), g.customized_info(4)
        assert i1["kernel_float"] == mg.KERNEL_MATMUL_CHAIN and i1["kernel_fingerprint"] == mg.KERNEL_MATMUL_CHAIN
        assert i2["kernel_float"] == mg.KERNEL_TILE_REDUCE and i2["kernel_fingerprint"] == mg.KERNEL_TILE_REDUCE
    moving = mg.ExecutionPlan(ops=[(mg.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mg.TB_MATMUL_OP, [(3, 0), (2, 0)])],
                              input_map=[(-1, -1, -1), (1, -1, -1), (-1, -1, -1)], forloop_dim=[1, 0, 1],
                              input_smem_layouts=[mg.SmemRowMajor] * 3, output_map=(1, -1, -1), forloop_range=4,
                              grid_dim=(2, 1, 1), reduction_dimx=64)
    with mg.PyGraph(planning_runtime) as g:
        X = g.new_input((16, 256)); W1 = g.new_input((256, 128)); W2 = g.new_input((64, 256))
        g.customized([X, W1, W2], moving)
        assert g.customized_info(3)["kernel_float"] == mg.KERNEL_INTERPRETER


def test_unfused_graph_shapes(planning_runtime):
    with mg.PyGraph(planning_runtime) as g:
        Q = g.new_input((2, 8, 64))
        K = g.new_input((2, 64, 256))
        V = g.new_input((2, 256, 64))
        A = g.matmul(Q, K)
        E = g.exp(A)
        S = g.reduction(E, 2)
        D = g.div(E, S)
        O = g.matmul(D, V)
        assert A.shape == (2, 8, 256) and S.shape == (2, 8, 1) and D.shape == (2, 8, 256) and O.shape == (2, 8, 64)
        with pytest.raises(mg.MuGraphError):
            g.matmul(Q, V)
        with pytest.raises(mg.MuGraphError):
            g.reduction(E, 2, 7)
