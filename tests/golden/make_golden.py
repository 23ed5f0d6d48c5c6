"""Generates tests/golden/gqa_decode_reference_host.json.

The expected values come from the reference's OWN code: its host graph builder / serialiser and its
fingerprinter classes, compiled for the CPU into oracle/_ref/libref_host.so (`make -C oracle ref`,
needs the reference checkout).  Inputs are the reference's deterministic fill fp[i] = i % 25651
(src/kernel/cuda/input_kernel.cu:56-62) and seeded uniform values; the file stores shapes, plan
metadata, the first outputs and FNV-1a digests, plus full outputs of the small cases.

    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import mugraph_oracle as mo  # noqa: E402
from oracle import ref_host  # noqa: E402

# (kv heads, query rows, head dim, kv length, splits, for-loop range)
CASES = [
    dict(name="reference_example_bs1", B=2, M=8, D=64, L=4096, S=16, F=4, fill="reference"),
    dict(name="baseline_c2", B=8, M=4, D=128, L=4096, S=16, F=4, fill="reference"),
    dict(name="small_uniform_pq", B=2, M=4, D=16, L=64, S=2, F=2, fill="uniform_pq", seed=7),
    dict(name="small_uniform_p", B=2, M=8, D=16, L=128, S=2, F=4, fill="uniform_p", seed=11),
]


def make_inputs(case, specs):
    if case["fill"] == "reference":
        return [mo.reference_fill(s.dims) for s in specs]
    rng = np.random.default_rng(case["seed"])
    hi = mo.FP_PQ if case["fill"] == "uniform_pq" else mo.FP_P
    return [rng.integers(0, hi, size=s.dims).astype(np.uint16) for s in specs]


def main():
    assert ref_host.available(), "build oracle/_ref first: make -C oracle ref"
    out = []
    for c in CASES:
        specs, p1, p2 = mo.gqa_decode_plans(c["B"], c["M"], c["D"], c["L"], c["S"], c["F"])
        x = make_inputs(c, specs)
        o1, info1 = ref_host.customized_fingerprint(specs, p1, x)
        specs2 = [mo.DTensorSpec(o.shape) for o in o1]
        o2, info2 = ref_host.customized_fingerprint(specs2, p2, o1)
        rec = dict(c)
        rec.update(op1=info1, op2=info2,
                   op1_output_shapes=[list(o.shape) for o in o1],
                   o_part_head=[int(v) for v in o1[0].ravel()[:4]],
                   r_part_head=[int(v) for v in o1[1].ravel()[:4]],
                   op1_digest=str(mo.fnv1a64(np.concatenate([o.ravel() for o in o1]))),
                   final_shape=list(o2[0].shape),
                   final_head=[int(v) for v in o2[0].ravel()[:4]],
                   final_digest=str(mo.fnv1a64(o2[0])))
        if o2[0].size <= 4096:
            rec["final_full"] = [int(v) for v in o2[0].ravel()]
            if c["fill"] != "reference":
                rec["inputs_full"] = [[int(v) for v in a.ravel()] for a in x]
        out.append(rec)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gqa_decode_reference_host.json")
    with open(path, "w") as f:
        json.dump(dict(generator="tests/golden/make_golden.py",
                       source="reference host serialiser + fingerprinter classes (oracle/_ref/libref_host.so)",
                       cases=out), f, separators=(",", ":"))
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
