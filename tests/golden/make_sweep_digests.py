"""Generates tests/golden/sweep_digests_gqa_decode.json: one FNV-1a-64 digest per input set of the
fingerprint verification sweep (4096 sets of the grouped-query decode muGraph: Q[8,4,128], K[8,128,4096],
V[8,4096,128], 16 KV splits x for-loop 4, then the cross-split merge).

The expected fingerprints come from the reference's OWN code - its host graph builder / serialiser and its
fingerprinter classes compiled for the CPU (oracle/_ref/libref_host.so, `make -C oracle ref`, needs the reference
checkout).  Input tensor i of set s is the seeded uniform fill with seed 3 * (2024 + s) + i over [0, 227)
(oracle.mugraph_oracle.sweep_inputs - the device fill mg_tensor_fill_fingerprint_seeded produces the same values).
About 11 core-minutes; the sets are spread over worker processes.

    python tests/golden/make_sweep_digests.py [--sets 4096] [--workers 8]
"""
import argparse
import json
import multiprocessing as mp
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import mugraph_oracle as mo  # noqa: E402
from oracle import ref_host  # noqa: E402

SHAPE = dict(B=8, M=4, D=128, L=4096, S=16, F=4)


def digests_of(sets):
    ref_host.set_threads(1)  # one worker process per core
    specs, p1, p2 = mo.gqa_decode_plans(SHAPE["B"], SHAPE["M"], SHAPE["D"], SHAPE["L"], SHAPE["S"], SHAPE["F"])
    out = []
    for s in sets:
        x = mo.sweep_inputs(s, specs)
        o1, _ = ref_host.customized_fingerprint(specs, p1, x)
        o2, _ = ref_host.customized_fingerprint([mo.DTensorSpec(o.shape) for o in o1], p2, o1)
        out.append((s, str(mo.fnv1a64(o2[0])), [int(v) for v in o2[0].ravel()[:4]]))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sets", type=int, default=4096)
    ap.add_argument("--workers", type=int, default=len(os.sched_getaffinity(0)))
    args = ap.parse_args()
    assert ref_host.available(), "build oracle/_ref first: make -C oracle ref"
    chunks = [list(range(w, args.sets, args.workers)) for w in range(args.workers)]
    with mp.get_context("fork").Pool(args.workers) as pool:
        parts = pool.map(digests_of, chunks)
    rows = sorted(r for part in parts for r in part)
    assert [r[0] for r in rows] == list(range(args.sets))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sweep_digests_gqa_decode.json")
    with open(path, "w") as f:
        json.dump(dict(generator="tests/golden/make_sweep_digests.py",
                       source="reference host serialiser + fingerprinter classes (oracle/_ref/libref_host.so)",
                       shape=SHAPE, seed_rule="tensor i of set s: seed 3 * (2024 + s) + i, uniform in [0, 227)",
                       digest="FNV-1a-64 over the uint16 values of the final fingerprint O[8,4,128]",
                       digests=[r[1] for r in rows], head_of_set={str(r[0]): r[2] for r in rows[:8]}),
                  f, separators=(",", ":"))
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
