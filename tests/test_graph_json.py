"""Graph JSON wire format (to_json / from_json of the reference, src/kernel/graph.cc:33-159), on a planning-only
runtime: documents the reference wrote load, and what this library writes back is the same document."""
import gzip
import json
import os

import pytest

import attention_superoptimizer_b200 as mg

FIXTURE = os.path.join(os.path.dirname(__file__), "golden", "spec_decode_candidates.json.gz")
BIG = 227 * 1024


def load_fixture():
    with gzip.open(FIXTURE) as f:
        return json.loads(f.read().decode())


def without(doc, keys=("guid", "reduction_dimx")):
    """guids are process-local counters; `reduction_dimx` postdates the checkpoint the fixture comes from."""
    if isinstance(doc, dict):
        return {k: without(v, keys) for k, v in doc.items() if k not in keys}
    if isinstance(doc, list):
        return [without(v, keys) for v in doc]
    return doc


def test_reference_candidates_round_trip(planning_runtime):
    """All 69 candidate muGraphs of the reference's search checkpoint load through from_json; dumping them again
    gives the reference's document: operator order, tensor shapes and layouts, plans and - for the candidates whose
    "bgraph" the fixture keeps - every tile shape and shared-memory offset the reference's planner chose."""
    planning_runtime.set_max_smem(BIG)
    base, _ = planning_runtime.arena_usage()  # the lookup tables sit at the arena base
    fx = load_fixture()
    assert len(fx["generated_graphs"]) == 69
    with_bgraph = 0
    for doc in fx["generated_graphs"]:
        with mg.PyGraph.from_json(doc, planning_runtime) as g:
            assert g.num_operators == len(doc)
            back = json.loads(g.to_json())
        for mine, ref in zip(back, doc):
            if "bgraph" in ref:
                with_bgraph += 1
            else:
                mine = {k: v for k, v in mine.items() if k != "bgraph"}
            assert without(mine) == without(ref)
    assert with_bgraph >= 4
    used, _ = planning_runtime.arena_usage()
    assert used == base  # every graph released its tensors


def test_computation_graph_round_trip(planning_runtime):
    fx = load_fixture()
    with mg.PyGraph.from_json(json.dumps(fx["computation_graph"]), planning_runtime) as g:
        back = json.loads(g.to_json())
        kinds = [g.operator(i)[0] for i in range(g.num_operators)]
    assert without(back) == without(fx["computation_graph"])
    assert kinds == [1001, 1001, 1001, 1003, 1007, 1006, 1010, 1003]
    # operand guids of the dump refer to earlier outputs of the same dump
    seen = set()
    for op in back:
        assert all(t["guid"] in seen for t in op["input_tensors"])
        seen.update(t["guid"] for t in op["output_tensors"])


def test_own_graph_round_trip(planning_runtime):
    """A graph built through the API dumps to a document that rebuilds the same graph."""
    planning_runtime.set_max_smem(BIG)
    with mg.PyGraph(planning_runtime) as g:
        Q = g.new_input((8, 4, 128))
        K = g.new_input((8, 128, 4096), layout=mg.DmemColumnMajor)
        V = g.new_input((8, 4096, 128))
        p1, p2 = mg.gqa_decode_plans(8, 4, 128, 4096, 16, 4)
        parts = g.customized([Q, K, V], p1)
        g.customized(parts, p2)
        first = g.to_json()
        info = g.customized_info(3)
    with mg.PyGraph.from_json(first, planning_runtime) as h:
        second = h.to_json()
        assert h.customized_info(3) == info  # same shared-memory plan, same kernel choice
        _, outs = h.operator(4)
        assert outs[0].shape == (8, 4, 128)
    assert without(json.loads(first), ("guid",)) == without(json.loads(second), ("guid",))
    plan = json.loads(first)[3]["plan"]
    assert plan["ops"][0] == ["tb_matmul_op", [[0, 0], [1, 0]]]
    assert plan["grid_dim"] == {"x": 8, "y": 16, "z": 1} and plan["forloop_range"] == 4


@pytest.mark.parametrize("text,needle", [
    ("{", "JSON"),
    ("{}", "not an array"),
    ('[{"op_type": "kn_nonsense_op", "input_tensors": [], "output_tensors": [{}]}]', "op_type"),
    ('[{"op_type": "kn_exp_op", "input_tensors": [{"guid": 7}], "output_tensors": [{"guid": 8}]}]', "guid 7"),
    ('[{"op_type": "kn_input_op", "input_tensors": [], "output_tensors": [{"data_type": 921, "dim": [4, 0, 0, 0], '
     '"guid": 1, "layout": "DmemDiagonal", "num_dims": 1}]}]', "layout"),
])
def test_malformed_documents_are_refused(planning_runtime, text, needle):
    base, _ = planning_runtime.arena_usage()
    with pytest.raises(mg.MuGraphError) as e:
        mg.PyGraph.from_json(text, planning_runtime)
    assert e.value.status == 2 and needle in str(e.value)
    used, _ = planning_runtime.arena_usage()
    assert used == base  # nothing of the half-built graph is left behind
