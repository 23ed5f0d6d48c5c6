"""Multi-GPU partitioning of the two workloads that shard naturally (one process per GPU):

* decode: the KV heads of a grouped-query attention call are independent (they are already `grid.x` of the
  muGraph), so rank r evaluates heads [r*H/N, (r+1)*H/N) - no collective on the data path;
* speculative decode: the batch x KV-head units of a call are independent too; rank r evaluates a contiguous
  range of them, again without a collective;
* verification sweep: independent input sets are split evenly over the ranks; every rank evaluates its share
  and the resulting fingerprints are all-gathered so that each rank can compare and de-duplicate all of them;
* candidate graphs: the candidates a search wants verified are dealt round-robin to the ranks; every rank
  verifies its share against the computation graph's fingerprint and the pass / fail flags (and, on request,
  a digest of every candidate's fingerprint) are all-gathered, so every rank ends up with the verdict on every
  candidate (the reference verifies them one after the other on one GPU, src/search/search.cc:569-623).

The reference is single-GPU (it has no collective anywhere); `torch.distributed` is used as plumbing only:
NCCL over NVLink on GPUs, gloo in the CPU tests.
"""
from __future__ import annotations

import hashlib
from typing import Dict, List, Tuple


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous shard [start, start + count) of `total` items for `rank`; the first total % world ranks
    take one extra item."""
    if not (0 <= rank < world) or total < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def kv_head_shard(num_kv_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """Heads of this rank; head counts must divide evenly so that every rank runs the same plan."""
    if num_kv_heads % world != 0:
        raise ValueError("%d KV heads do not split evenly over %d ranks" % (num_kv_heads, world))
    per = num_kv_heads // world
    return rank * per, per


def all_gather_fingerprints(local, world: int, group=None, out=None):
    """All-gather of per-set fingerprints.  `local` is a [sets_per_rank, n] int16/uint16 tensor (CUDA with
    NCCL, CPU with gloo); every rank must pass the same shape.  Returns [world * sets_per_rank, n]; `out` is an
    optional preallocated tensor of that shape and dtype (keeps the allocator out of a timed region)."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return local
    if out is None:
        out = torch.empty((world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    # moved as bytes: 16-bit integer types are not accepted by every backend
    dist.all_gather_into_tensor(out.view(torch.uint8), local.contiguous().view(torch.uint8), group=group)
    return out


def matches_reference_on_device(fingerprints, reference):
    """The verify step on the device: `fingerprints` [n, m] and `reference` [m] are torch tensors on the same
    device; returns a bool tensor [n] (True where the whole fingerprint equals the reference's)."""
    return (fingerprints == reference.reshape(1, -1)).all(dim=1)


def fingerprint_digest(row) -> bytes:
    """128-bit digest of one fingerprint (host side, for grouping)."""
    return hashlib.blake2b(row.tobytes(), digest_size=16).digest()


def dedup(fingerprints) -> Dict[int, List[int]]:
    """Groups equal fingerprints: {first index: [all indices with the same fingerprint]}.  `fingerprints` is a
    [n, m] integer numpy array.  Digests pre-group, full rows confirm (no false merges)."""
    import numpy as np
    groups: Dict[bytes, List[int]] = {}
    for i in range(fingerprints.shape[0]):
        groups.setdefault(fingerprint_digest(np.ascontiguousarray(fingerprints[i])), []).append(i)
    out: Dict[int, List[int]] = {}
    for idxs in groups.values():
        reps: List[int] = []
        for i in idxs:
            for r in reps:
                if np.array_equal(fingerprints[r], fingerprints[i]):
                    out[r].append(i)
                    break
            else:
                reps.append(i)
                out[i] = [i]
    return out


def matches_reference(fingerprints, reference) -> List[bool]:
    """Per candidate: does its fingerprint equal the reference graph's? (the verify step of the search,
    reference src/search/search.cc:601-609)"""
    import numpy as np
    return [bool(np.array_equal(fingerprints[i], reference)) for i in range(fingerprints.shape[0])]


def unit_shard(num_units: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous range of the independent (batch, KV head) units of a decode call that `rank` evaluates; the
    count must divide evenly so that every rank runs the same plan."""
    if num_units % world != 0:
        raise ValueError("%d units do not split evenly over %d ranks" % (num_units, world))
    per = num_units // world
    return rank * per, per


def candidate_shard(num_candidates: int, rank: int, world: int) -> List[int]:
    """Indices of the candidates `rank` verifies: round-robin, so that candidates of similar cost (a search emits
    them in families) spread over the ranks."""
    if not (0 <= rank < world):
        raise ValueError("bad shard request")
    return list(range(rank, num_candidates, world))


def verify_candidates_sharded(num_candidates: int, verify_local, world: int, rank: int, device=None, group=None):
    """Distributed form of the search's verify step.  `verify_local(indices)` verifies the candidates with those
    indices on this rank's GPU and returns, per candidate, either a bool or a (bool, 64-bit digest of its
    fingerprint) pair - on the GPU path it wraps `verify_candidates` of this package.  The flags (and digests) of
    all ranks are all-gathered; returns (flags, digests) as lists of length num_candidates on every rank, digests
    None when the callable gives none.  One small collective per call: 16 bytes per candidate."""
    import torch
    import torch.distributed as dist
    mine = candidate_shard(num_candidates, rank, world)
    results = list(verify_local(mine)) if mine else []
    if len(results) != len(mine):
        raise ValueError("verify_local returned %d results for %d candidates" % (len(results), len(mine)))
    per_rank = -(-num_candidates // world) if num_candidates else 0
    # [per_rank, 2] int64 rows (flag, digest); ranks with fewer candidates pad with -1
    local = torch.full((max(per_rank, 1), 2), -1, dtype=torch.int64)
    with_digests = False
    for j, r in enumerate(results):
        if isinstance(r, tuple):
            flag, digest = r
            with_digests = True
            # digests are unsigned 64-bit values: carried as their two's-complement image
            local[j, 1] = int(digest) - (1 << 64) if int(digest) >= (1 << 63) else int(digest)
        else:
            flag = r
        local[j, 0] = 1 if flag else 0
    if world == 1:
        gathered = local.unsqueeze(0)
    else:
        if device is not None:
            local = local.to(device)
        flat = torch.empty((world * local.shape[0], 2), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(flat, local, group=group)
        gathered = flat.cpu().view(world, local.shape[0], 2)
    flags: List[bool] = [False] * num_candidates
    digests: List[int] = [0] * num_candidates
    any_digest = with_digests
    for r in range(world):
        for j, idx in enumerate(candidate_shard(num_candidates, r, world)):
            flags[idx] = bool(gathered[r, j, 0].item() == 1)
            d = int(gathered[r, j, 1].item())
            if d != -1 or with_digests:
                any_digest = any_digest or d != -1
            digests[idx] = d + (1 << 64) if d < 0 else d
    return flags, (digests if any_digest else None)
