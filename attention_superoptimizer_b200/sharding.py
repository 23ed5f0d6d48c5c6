"""Multi-GPU partitioning of the two workloads that shard naturally (one process per GPU):

* decode: the KV heads of a grouped-query attention call are independent (they are already `grid.x` of the
  muGraph), so rank r evaluates heads [r*H/N, (r+1)*H/N) - no collective on the data path;
* verification sweep: independent input sets (or candidate graphs) are split evenly over the ranks; every
  rank evaluates its share and the resulting fingerprints are all-gathered so that each rank can compare
  and de-duplicate all of them.

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
