"""CPU tests of the multi-GPU partitioning logic with world_size 2 over gloo.  The per-rank evaluation is done
by the CPU oracle here (stand-in for the GPU executor); what is under test is the sharding, the all-gather and
the de-duplication / comparison that follow."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from attention_superoptimizer_b200 import sharding  # noqa: E402
from oracle import fp_oracle, mugraph_oracle as mo  # noqa: E402

SHAPE = (2, 4, 16, 64, 2, 2)  # kv heads, rows, head dim, kv len, splits, for-loop
SETS = 6


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def evaluate_sets(first, count):
    """Fingerprints of input sets [first, first + count): seed = 100 + set index; sets 1 and 4 are given the
    same inputs on purpose (duplicates for the dedup step)."""
    B, M, D, L, S, F = SHAPE
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, S, F)
    g1 = mo.build_customized(specs, p1)
    g2 = mo.build_customized(mo.output_specs(g1), p2)
    out = []
    for s in range(first, first + count):
        seed = 100 + (1 if s == 4 else s)
        rng = np.random.default_rng(seed)
        x = [rng.integers(0, mo.FP_P, size=t.dims).astype(np.uint16) for t in specs]
        o1, _ = fp_oracle.run(g1, x)
        o2, _ = fp_oracle.run(g2, o1)
        out.append(o2[0].ravel())
    return np.stack(out)


def worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        first, count = sharding.shard_range(SETS, rank, world)
        local = torch.from_numpy(evaluate_sets(first, count).astype(np.int16))
        gathered = sharding.all_gather_fingerprints(local, world).numpy().view(np.uint16)
        np.save(os.path.join(result_dir, "rank%d.npy" % rank), gathered)
    finally:
        dist.destroy_process_group()


def test_shard_ranges_cover_everything_once():
    for total in (0, 1, 7, 4096):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                s, c = sharding.shard_range(total, r, world)
                seen += list(range(s, s + c))
            assert seen == list(range(total))
    assert sharding.kv_head_shard(8, 3, 4) == (6, 2)
    with pytest.raises(ValueError):
        sharding.kv_head_shard(8, 0, 3)


def test_two_rank_sweep_matches_single_process(tmp_path):
    world, port = 2, free_port()
    mp.spawn(worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    want = evaluate_sets(0, SETS)
    for r in range(world):
        got = np.load(os.path.join(str(tmp_path), "rank%d.npy" % r))
        assert np.array_equal(got, want)  # every rank holds all fingerprints, in set order
    groups = sharding.dedup(want)
    assert groups[1] == [1, 4] and sorted(groups) == [0, 1, 2, 3, 5]
    assert sharding.matches_reference(want, want[4]) == [False, True, False, False, True, False]
    import torch
    t = torch.from_numpy(want.astype(np.int32))
    assert sharding.matches_reference_on_device(t, t[4]).tolist() == [False, True, False, False, True, False]


def failing_worker(rank, world, port, result_dir):
    from datetime import timedelta
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=5))
    if rank == 1:
        os._exit(0)  # this rank leaves between steps, before the collective
    try:
        local = torch.zeros((3, 8), dtype=torch.int16)
        sharding.all_gather_fingerprints(local, world)
        outcome = "completed"
    except Exception as e:  # the survivor must get an error, not hang
        outcome = "error: " + type(e).__name__
    with open(os.path.join(result_dir, "outcome.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


def test_rank_that_leaves_is_detected_not_waited_for_forever(tmp_path):
    world, port = 2, free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=failing_worker, args=(r, world, port, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive()
    assert open(os.path.join(str(tmp_path), "outcome.txt")).read().startswith("error")


# ---- candidate graphs dealt round-robin, verdicts all-gathered ----------------------------------------------------
CANDIDATES = 7


def candidate_fingerprint(i):
    """Stand-in for candidate graph i: candidates 2 and 5 compute something else than the reference."""
    rng = np.random.default_rng(3 if i not in (2, 5) else 100 + i)
    return rng.integers(0, mo.FP_PQ, size=64).astype(np.uint16)


def verify_worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        reference = candidate_fingerprint(0)

        def verify_local(indices):
            seen.extend(indices)
            return [(bool(np.array_equal(candidate_fingerprint(i), reference)), mo.fnv1a64(candidate_fingerprint(i)))
                    for i in indices]

        seen = []
        flags, digests = sharding.verify_candidates_sharded(CANDIDATES, verify_local, world, rank)
        np.save(os.path.join(result_dir, "flags%d.npy" % rank), np.array(flags))
        np.save(os.path.join(result_dir, "digests%d.npy" % rank), np.array(digests, dtype=np.uint64))
        np.save(os.path.join(result_dir, "seen%d.npy" % rank), np.array(seen))
    finally:
        dist.destroy_process_group()


def test_candidate_shards_and_two_rank_verification(tmp_path):
    for n in (0, 1, 7, 69):
        for world in (1, 2, 3, 8):
            dealt = sorted(i for r in range(world) for i in sharding.candidate_shard(n, r, world))
            assert dealt == list(range(n))
    assert sharding.unit_shard(32, 3, 8) == (12, 4)
    with pytest.raises(ValueError):
        sharding.unit_shard(32, 0, 5)
    world, port = 2, free_port()
    mp.spawn(verify_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    want_flags = [i not in (2, 5) for i in range(CANDIDATES)]
    want_digests = [mo.fnv1a64(candidate_fingerprint(i)) for i in range(CANDIDATES)]
    for r in range(world):
        assert np.load(os.path.join(str(tmp_path), "flags%d.npy" % r)).tolist() == want_flags
        assert np.load(os.path.join(str(tmp_path), "digests%d.npy" % r)).tolist() == want_digests
        assert np.load(os.path.join(str(tmp_path), "seen%d.npy" % r)).tolist() == list(range(r, CANDIDATES, world))
    # single process: same interface, no collective
    flags, digests = sharding.verify_candidates_sharded(3, lambda idx: [i != 1 for i in idx], 1, 0)
    assert flags == [True, False, True] and digests is None
