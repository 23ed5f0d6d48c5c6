"""Writes tests/golden/spec_decode_candidates.json.gz from the reference's demo search checkpoint.

    python tests/golden/make_candidates.py /path/to/reference

The checkpoint (demo/checkpoint_group_query_attn_spec_decode.json) holds the un-fused computation graph of
grouped-query attention for speculative decoding and the 69 candidate muGraphs the reference's search found
equivalent to it with its own fingerprint kernels.  The fixture keeps, in the reference's JSON wire format:
  * "computation_graph": the un-fused graph, unchanged;
  * "generated_graphs": every candidate; the first four keep their "bgraph" entry (threadblock operators with
    tile shapes and shared-memory offsets as the reference planned them), the others only what from_json
    reads (operator types, tensor descriptors, plans).
The search statistics and configuration of the checkpoint are dropped."""
import gzip
import json
import os
import sys

KEEP_BGRAPH = 4


def main(reference_root):
    src = os.path.join(reference_root, "demo", "checkpoint_group_query_attn_spec_decode.json")
    with open(src) as f:
        ckpt = json.load(f)
    graphs = []
    for i, g in enumerate(ckpt["generated_graphs"]):
        graphs.append([{k: v for k, v in op.items() if k != "bgraph" or i < KEEP_BGRAPH} for op in g])
    out = {"source": "demo/checkpoint_group_query_attn_spec_decode.json of the reference",
           "computation_graph": ckpt["computation_graph"], "generated_graphs": graphs}
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "spec_decode_candidates.json.gz")
    with gzip.GzipFile(dst, "wb", mtime=0) as f:
        f.write(json.dumps(out, separators=(",", ":"), sort_keys=True).encode())
    print(dst, os.path.getsize(dst), "bytes,", len(graphs), "candidates")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
