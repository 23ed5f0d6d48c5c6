"""CPU oracle for muGraph execution.  TEST INFRASTRUCTURE ONLY.

This module restates, in numpy, the algorithm the reference uses to evaluate a
customized operator's threadblock graph.  It exists to check the CUDA executor;
nothing in the product imports it.  Only tests, the smoke check and the CPU leg
of the benchmark may call it.

Parity status: PINNED.  The restatement is checked (tests/test_oracle.py)
against (a) known-answer values computed by the reference's own host
serialiser and fingerprinter classes compiled for the CPU (the recipe is
oracle/Makefile -> oracle/_ref/), committed under tests/golden/, and (b) the
reference's own integration property "fused graph fingerprint == un-fused graph
fingerprint" (cpp_examples/group_query_attn_inc_decode.cc:104-108).

What each part follows in the reference (paths relative to the reference root):

  constants / tables      include/mirage/type.h:26-36,
                          src/kernel/device_memory_manager.cu:41-90
  tile shapes, smem plan  src/threadblock/input_loader.cc:33-140,
                          src/threadblock/output.cc:39-79,
                          src/threadblock/{matmul,element_unary,element_binary,
                          reduction,concat}.cc, src/threadblock/graph.cc:43-52
  plan -> op list         src/kernel/customized.cc:65-186
  block / forloop offsets src/threadblock/graph.cc:68-432
  interpreter loop        src/kernel/cuda/customized_kernel.cu:307-603
  per-op arithmetic       include/mirage/threadblock/cuda/{input_loader.h:444-478,
                          matmul.h:751-806, element_unary.h:46-72,
                          element_binary.h:62-111, reduction.h:128-156,
                          concat.h:78-103, output_saver.h:359-449}
  un-fused (kernel-level) src/kernel/cuda/{matmul_kernel.cu:145-173,
  operators               element_unary_kernel.cu:77-94,
                          element_binary_kernel.cu:97-143,
                          reduction_kernel.cu:80-108, input_kernel.cu:56-62}

Float mode has no usable reference implementation (the reference's fp16
interpreter is a timing proxy that does not store correct values), so
`run_float` evaluates the same graph semantics in fp32: per for-loop iteration
every operator is recomputed from freshly loaded tiles, output operators sum
over iterations, results land in the output tensor according to `output_map`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

# ---- include/mirage/type.h:26-36 -------------------------------------------
FP_P = 227
FP_Q = 113
FP_EXP_BASE = 3
FP_PQ = 25651
FP_P_MUL_Q_MOD_1 = 227
FP_Q_MUL_P_MOD_1 = 25425

# operator / dtype / layout codes: numeric values of the reference enums
TB_INPUT_OP, TB_OUTPUT_OP, TB_MATMUL_OP = 2001, 2002, 2003
TB_EXP_OP, TB_ADD_OP, TB_MUL_OP, TB_DIV_OP = 2007, 2008, 2009, 2010
TB_REDUCTION_0_OP, TB_REDUCTION_1_OP, TB_REDUCTION_2_OP = 2101, 2102, 2103
TB_REDUCTION_0_TO_DIMX_OP, TB_REDUCTION_1_TO_DIMX_OP, TB_REDUCTION_2_TO_DIMX_OP = 2104, 2105, 2106
TB_CONCAT_0_OP, TB_CONCAT_1_OP, TB_CONCAT_2_OP = 2200, 2201, 2202
DT_BFLOAT16, DT_FLOAT16, DT_FLOAT32 = 920, 921, 930
DmemRowMajor, DmemColumnMajor = 100, 101
SmemRowMajor, SmemColumnMajor = 200, 201
SmemRowMajorTensorOpMultiplicand_Crosswise64 = 204
SmemColumnMajorTensorOpMultiplicand_Crosswise64 = 207

DEFAULT_MAX_SMEM = 96 * 1024  # include/mirage/type.h:35


def lookup_tables():
    """exp / inverse tables, src/kernel/device_memory_manager.cu:41-90."""
    exp_tbl = np.ones(FP_Q, dtype=np.int64)
    for i in range(1, FP_Q):
        exp_tbl[i] = (exp_tbl[i - 1] * FP_EXP_BASE) % FP_P
    assert (exp_tbl[FP_Q - 1] * FP_EXP_BASE) % FP_P == 1

    def inverse_table(m):
        t = np.ones(m, dtype=np.int64)  # entry 0 (and 1) keep the initial 1
        for i in range(m):
            for j in range(1, m):
                if (i * j) % m == 1:
                    t[i] = j
        return t

    return exp_tbl, inverse_table(FP_P), inverse_table(FP_Q)


EXP_TBL, DIV_P_TBL, DIV_Q_TBL = lookup_tables()


def fp_exp(x):
    """element_unary.h:60-66 - only the mod-Q residue of the argument is used."""
    x = np.asarray(x, dtype=np.int64)
    return (EXP_TBL[x % FP_Q] * FP_Q_MUL_P_MOD_1) % FP_PQ


def fp_div(x, y):
    """element_binary.h:100-104 - CRT recombination of two table inverses."""
    x = np.asarray(x, dtype=np.int64)
    y = np.asarray(y, dtype=np.int64)
    z = (x % FP_P) * DIV_P_TBL[y % FP_P] * FP_Q_MUL_P_MOD_1 + \
        (x % FP_Q) * DIV_Q_TBL[y % FP_Q] * FP_P_MUL_Q_MOD_1
    return z % FP_PQ


def fp_matmul(a, b):
    """matmul.h:773-804: reduction after every MAC == one reduction at the end."""
    return (np.asarray(a, dtype=np.int64) @ np.asarray(b, dtype=np.int64)) % FP_PQ


def reference_fill(shape):
    """src/kernel/cuda/input_kernel.cu:56-62: fp[idx] = idx % FP_PQ."""
    n = int(np.prod(shape))
    return (np.arange(n, dtype=np.int64) % FP_PQ).astype(np.uint16).reshape(shape)


def seeded_uniform(seed, n, modulus):
    """Host twin of mg_rng_uniform (include/mugraph_rng.h): splitmix64 finaliser over (seed, index), upper 32 bits
    modulo `modulus`; the device fill of the same seed produces the same uint16 values."""
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64)
        z = np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15) + idx * np.uint64(0xD1B54A32D192ED03) + np.uint64(0x632BE59BD9B4E019)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return ((z >> np.uint64(32)) % np.uint64(modulus)).astype(np.uint16)


SWEEP_BASE_SEED = 2024


def sweep_inputs(set_index, specs, modulus=FP_P):
    """Input tensors of set `set_index` of the verification sweep: tensor i of set s is the seeded uniform fill
    with seed 3 * (2024 + s) + i, values in [0, modulus)."""
    return [seeded_uniform(3 * (SWEEP_BASE_SEED + set_index) + i, int(np.prod(sp.dims)), modulus).reshape(sp.dims)
            for i, sp in enumerate(specs)]


def fnv1a64(values) -> int:
    """Digest used by the known-answer tables: FNV-1a over the integer values."""
    h = 1469598103934665603
    for x in np.asarray(values).reshape(-1).tolist():
        h ^= int(x)
        h = (h * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


# ---------------------------------------------------------------------------
# plan and threadblock-graph construction (host logic)
# ---------------------------------------------------------------------------
@dataclass
class ExecutionPlan:
    """Mirror of threadblock::ExecutionPlan, include/mirage/threadblock/graph.h:28-42."""
    ops: List[Tuple[int, List[Tuple[int, int]]]]
    input_map: List[Tuple[int, int, int]]
    forloop_dim: List[int]
    input_smem_layouts: List[int]
    output_map: Tuple[int, int, int]
    forloop_range: int
    grid_dim: Tuple[int, int, int]
    block_dim: Tuple[int, int, int] = (128, 1, 1)
    reduction_dimx: int = 64


@dataclass
class DTensorSpec:
    dims: Tuple[int, ...]
    dtype: int = DT_FLOAT16
    layout: int = DmemRowMajor

    @property
    def num_elements(self):
        return int(np.prod(self.dims))


@dataclass
class STensor:
    dims: List[int]
    layout: int
    smem_offset: int  # bytes
    elem_size: int = 2

    @property
    def num_elements(self):
        return int(np.prod(self.dims))

    def size(self):
        return self.num_elements * self.elem_size


@dataclass
class TBOp:
    type: int
    inputs: List[STensor] = field(default_factory=list)
    inputs_src: List[Tuple[int, int]] = field(default_factory=list)
    outputs: List[STensor] = field(default_factory=list)
    # input op
    dtensor: Optional[DTensorSpec] = None
    imap: Tuple[int, int, int] = (-1, -1, -1)
    forloop_dim: int = -1
    # output op
    omap: Tuple[int, int, int] = (-1, -1, -1)
    out_dtensor: Optional[DTensorSpec] = None


class InvalidGraph(Exception):
    """Raised where the reference's create_*_op returns nullptr or asserts."""


def _elem_size(dtype):
    if dtype in (DT_FLOAT16, DT_BFLOAT16):
        return 2
    if dtype == DT_FLOAT32:
        return 4
    raise InvalidGraph("unsupported element type %d" % dtype)


class TBGraph:
    """Shape inference + shared-memory plan of one customized op."""

    def __init__(self, grid_dim, block_dim, forloop_range, reduction_dimx, max_smem=DEFAULT_MAX_SMEM):
        if reduction_dimx <= 0:
            raise InvalidGraph("reduction_dimx must be positive")
        self.grid_dim = tuple(int(g) for g in grid_dim)
        self.block_dim = tuple(int(b) for b in block_dim)
        self.forloop_range = int(forloop_range)
        self.reduction_dimx = int(reduction_dimx)
        self.max_smem = max_smem
        self.smem_offset = 0
        self.ops: List[TBOp] = []

    # src/threadblock/graph.cc:43-52
    def _allocate(self, t: STensor) -> int:
        ret = self.smem_offset
        self.smem_offset += (t.size() + 15) & ~15
        if self.smem_offset > self.max_smem:
            raise InvalidGraph("shared memory overflow")
        return ret

    def _partition(self, dims, imap):
        dims = list(dims)
        for axis in range(3):
            if self.grid_dim[axis] > 1 and imap[axis] >= 0:
                d = imap[axis]
                if dims[d] <= 0 or dims[d] % self.grid_dim[axis] != 0:
                    raise InvalidGraph("dimension not divisible by grid")
                dims[d] //= self.grid_dim[axis]
        return dims

    # src/threadblock/input_loader.cc:33-140
    def new_input(self, dt: DTensorSpec, imap, forloop_dim, layout):
        dims = self._partition(dt.dims, imap)
        if forloop_dim >= 0:
            if dims[forloop_dim] <= 0 or dims[forloop_dim] % self.forloop_range != 0:
                raise InvalidGraph("forloop dimension not divisible")
            dims[forloop_dim] //= self.forloop_range
        if any(d != 1 for d in dims[:-2]):
            raise InvalidGraph("leading tile dimensions must be 1")
        t = STensor(dims, layout, 0, _elem_size(dt.dtype))
        if self.smem_offset + t.size() > self.max_smem:
            raise InvalidGraph("shared memory overflow")
        t.smem_offset = self._allocate(t)
        op = TBOp(TB_INPUT_OP, outputs=[t], dtensor=dt, imap=tuple(imap), forloop_dim=forloop_dim)
        self.ops.append(op)
        return t

    # src/threadblock/matmul.cc:31-84
    def matmul(self, a: STensor, b: STensor, src=None):
        if len(a.dims) != len(b.dims) or a.dims[-1] != b.dims[-2]:
            raise InvalidGraph("matmul shape mismatch")
        if any(d != 1 for d in a.dims[:-2]) or any(d != 1 for d in b.dims[:-2]):
            raise InvalidGraph("threadblock matmul is 2-D only")
        c = STensor(list(a.dims[:-1]) + [b.dims[-1]], SmemRowMajor, 0, a.elem_size)
        c.smem_offset = self._allocate(c)
        self.ops.append(TBOp(TB_MATMUL_OP, [a, b], src or [], [c]))
        return c

    # src/threadblock/element_unary.cc:36-53 (in place)
    def exp(self, a: STensor, src=None):
        out = STensor(list(a.dims), a.layout, a.smem_offset, a.elem_size)
        self.ops.append(TBOp(TB_EXP_OP, [a], src or [], [out]))
        return out

    # src/threadblock/element_binary.cc:47-94
    def _binary(self, ty, a: STensor, b: STensor, src=None):
        if len(a.dims) != len(b.dims):
            raise InvalidGraph("rank mismatch")
        for x, y in zip(a.dims, b.dims):
            if x != y and x > 1 and y > 1:
                raise InvalidGraph("broadcast mismatch")
        out = STensor([max(x, y) for x, y in zip(a.dims, b.dims)], a.layout, 0, a.elem_size)
        out.smem_offset = self._allocate(out)
        self.ops.append(TBOp(ty, [a, b], src or [], [out]))
        return out

    def div(self, a, b, src=None):
        return self._binary(TB_DIV_OP, a, b, src)

    def add(self, a, b, src=None):
        return self._binary(TB_ADD_OP, a, b, src)

    # src/threadblock/reduction.cc:30-104
    def reduction(self, a: STensor, dim, src=None):
        if not (len(a.dims) > dim) or a.layout != SmemRowMajor:
            raise InvalidGraph("reduction needs a row-major input")
        if dim < len(a.dims) - 2:
            raise InvalidGraph("reduction over a leading dimension")
        dims = list(a.dims)
        dims[dim] = 1
        out = STensor(dims, a.layout, 0, a.elem_size)
        out.smem_offset = self._allocate(out)
        self.ops.append(TBOp(TB_REDUCTION_0_OP + dim, [a], src or [], [out]))
        return out

    def reduction_to_dimx(self, a: STensor, dim, src=None):
        if not (len(a.dims) > dim) or a.layout != SmemRowMajor:
            raise InvalidGraph("reduction needs a row-major input")
        dims = list(a.dims)
        dims[dim] = self.reduction_dimx
        out = STensor(dims, a.layout, 0, a.elem_size)
        out.smem_offset = self._allocate(out)
        self.ops.append(TBOp(TB_REDUCTION_0_TO_DIMX_OP + dim, [a], src or [], [out]))
        return out

    # src/threadblock/concat.cc:31-78
    def concat(self, a: STensor, b: STensor, dim, src=None):
        if len(a.dims) != len(b.dims) or len(a.dims) <= dim:
            raise InvalidGraph("concat rank mismatch")
        for i, (x, y) in enumerate(zip(a.dims, b.dims)):
            if i != dim and x != y:
                raise InvalidGraph("concat shape mismatch")
        if a.layout != b.layout:
            raise InvalidGraph("concat layout mismatch")
        dims = list(a.dims)
        dims[dim] = a.dims[dim] + b.dims[dim]
        out = STensor(dims, a.layout, 0, a.elem_size)
        out.smem_offset = self._allocate(out)
        self.ops.append(TBOp(TB_CONCAT_0_OP + dim, [a, b], src or [], [out]))
        return out

    # src/threadblock/output.cc:30-79
    def new_output(self, s: STensor, omap, dtype=DT_FLOAT16):
        if self.smem_offset + s.size() >= self.max_smem:
            raise InvalidGraph("shared memory overflow")
        acc = STensor(list(s.dims), s.layout, 0, s.elem_size)
        acc.smem_offset = self._allocate(acc)
        dims = list(acc.dims)
        for axis in range(3):
            if self.grid_dim[axis] > 1 and omap[axis] >= 0:
                dims[omap[axis]] *= self.grid_dim[axis]
        dt = DTensorSpec(tuple(dims), dtype, DmemRowMajor)
        self.ops.append(TBOp(TB_OUTPUT_OP, [s], [], [acc], omap=tuple(omap), out_dtensor=dt))
        return dt


def build_customized(inputs: Sequence[DTensorSpec], plan: ExecutionPlan, max_smem=DEFAULT_MAX_SMEM) -> TBGraph:
    """KNCustomizedOp(inputs, plan), src/kernel/customized.cc:65-186."""
    if not (len(inputs) == len(plan.input_map) == len(plan.forloop_dim) == len(plan.input_smem_layouts)):
        raise InvalidGraph("plan/input count mismatch")
    g = TBGraph(plan.grid_dim, plan.block_dim, plan.forloop_range, plan.reduction_dimx, max_smem)
    for dt, imap, fd, lay in zip(inputs, plan.input_map, plan.forloop_dim, plan.input_smem_layouts):
        g.new_input(dt, imap, fd, lay)
    for ty, srcs in plan.ops:
        ins = []
        for (oi, ti) in srcs:
            if not (0 <= oi < len(g.ops)) or not (0 <= ti < len(g.ops[oi].outputs)):
                raise InvalidGraph("operand index out of range")
            ins.append(g.ops[oi].outputs[ti])
        srcs = [tuple(s) for s in srcs]
        if ty == TB_MATMUL_OP:
            g.matmul(ins[0], ins[1], srcs)
        elif ty == TB_EXP_OP:
            g.exp(ins[0], srcs)
        elif ty == TB_ADD_OP:
            g.add(ins[0], ins[1], srcs)
        elif ty == TB_DIV_OP:
            g.div(ins[0], ins[1], srcs)
        elif TB_REDUCTION_0_OP <= ty <= TB_REDUCTION_2_OP:
            g.reduction(ins[0], ty - TB_REDUCTION_0_OP, srcs)
        elif TB_REDUCTION_0_TO_DIMX_OP <= ty <= TB_REDUCTION_2_TO_DIMX_OP:
            g.reduction_to_dimx(ins[0], ty - TB_REDUCTION_0_TO_DIMX_OP, srcs)
        elif TB_CONCAT_0_OP <= ty <= TB_CONCAT_2_OP:
            g.concat(ins[0], ins[1], ty - TB_CONCAT_0_OP, srcs)
        else:
            raise InvalidGraph("unsupported operator %d" % ty)
    # customized.cc:144-185: every op output nobody consumes later becomes an
    # output.  "Consumes" compares tensors by value (shape, owner and offset),
    # so an in-place exp result and its source are different tensors.
    n = len(g.ops)
    dtype = inputs[0].dtype if inputs else DT_FLOAT16
    for i in range(n):
        op = g.ops[i]
        if op.type == TB_INPUT_OP:
            continue
        for ts in range(len(op.outputs)):
            used = any((i, ts) in later.inputs_src for later in g.ops[i + 1:n])
            if not used:
                g.new_output(op.outputs[ts], plan.output_map, dtype)
    return g


def output_specs(g: TBGraph) -> List[DTensorSpec]:
    return [op.out_dtensor for op in g.ops if op.type == TB_OUTPUT_OP]


# ---------------------------------------------------------------------------
# block / forloop offsets, src/threadblock/graph.cc:106-166 and 214-239
# ---------------------------------------------------------------------------
def _input_offsets(g: TBGraph, op: TBOp):
    st = op.outputs[0]
    dt = op.dtensor
    nd = len(st.dims)
    fr = g.forloop_range
    row_bs = [(st.dims[nd - 2] if op.imap[a] == nd - 2 else 0) * (fr if op.forloop_dim == nd - 2 else 1) for a in range(3)]
    col_bs = [(st.dims[nd - 1] if op.imap[a] == nd - 1 else 0) * (fr if op.forloop_dim == nd - 1 else 1) for a in range(3)]
    row_fs = st.dims[nd - 2] if op.forloop_dim == nd - 2 else 0
    col_fs = st.dims[nd - 1] if op.forloop_dim == nd - 1 else 0
    glob_bs = [0, 0, 0]
    glob_fs = 0
    if nd > 2:
        strides = [0] * nd
        strides[nd - 3] = dt.dims[nd - 2] * dt.dims[nd - 1]
        for j in range(nd - 4, -1, -1):
            strides[j] = strides[j + 1] * dt.dims[j + 1]
        for a in range(3):
            if 0 <= op.imap[a] < nd - 2:
                glob_bs[a] = strides[op.imap[a]]
        if 0 <= op.forloop_dim < nd - 2:
            glob_fs = st.dims[op.forloop_dim] * strides[op.forloop_dim]
    return row_bs, col_bs, row_fs, col_fs, glob_bs, glob_fs


def _output_offsets(g: TBGraph, op: TBOp):
    st = op.inputs[0]
    dt = op.out_dtensor
    nd = len(st.dims)
    row_bs = [st.dims[nd - 2] if op.omap[a] == nd - 2 else 0 for a in range(3)]
    col_bs = [st.dims[nd - 1] if op.omap[a] == nd - 1 else 0 for a in range(3)]
    glob_bs = [0, 0, 0]
    if nd > 2:
        strides = [0] * nd
        strides[nd - 3] = dt.dims[nd - 2] * dt.dims[nd - 1]
        for j in range(nd - 4, -1, -1):
            strides[j] = strides[j + 1] * dt.dims[j + 1]
        for a in range(3):
            if 0 <= op.omap[a] < nd - 2:
                glob_bs[a] = strides[op.omap[a]]
    return row_bs, col_bs, glob_bs


def _reduction_params(op: TBOp):
    inp, out = op.inputs[0], op.outputs[0]
    ty = op.type
    rdim = ty - TB_REDUCTION_0_TO_DIMX_OP if ty >= TB_REDUCTION_0_TO_DIMX_OP else ty - TB_REDUCTION_0_OP
    degree = inp.num_elements // out.num_elements
    inner = int(np.prod(out.dims[rdim:]))
    return out.num_elements, degree, inner


def _bcast3(t: STensor):
    d = list(t.dims)
    if any(x != 1 for x in d[:-3]):
        raise InvalidGraph("only the last three dims may exceed 1")
    d = d[-3:]
    return [1] * (3 - len(d)) + d


# ---------------------------------------------------------------------------
# interpreters
# ---------------------------------------------------------------------------
def _run(g: TBGraph, inputs, out_dtype, mode, layouts_matter):
    """Walk blocks x iterations x ops exactly like customized_kernel.cu:323-602.

    Shared memory is modelled as one flat element array addressed by the
    planned byte offsets (all tiles are 2-byte elements), which reproduces the
    aliasing of the in-place exp.
    """
    in_ops = [op for op in g.ops if op.type == TB_INPUT_OP]
    out_ops = [op for op in g.ops if op.type == TB_OUTPUT_OP]
    assert len(inputs) == len(in_ops)
    work = np.int64 if mode == "fp" else np.float32
    flat_in = []
    for arr, op in zip(inputs, in_ops):
        a = np.asarray(arr)
        assert a.size == op.dtensor.num_elements
        if layouts_matter and op.dtensor.layout == DmemColumnMajor:
            # memory holds each [rows, cols] matrix column-major: present it as
            # the logical row-major array the graph semantics talk about
            dims = op.dtensor.dims
            lead = int(np.prod(dims[:-2]))
            a = a.reshape(lead, dims[-1], dims[-2]).transpose(0, 2, 1)
        flat_in.append(np.ascontiguousarray(a).reshape(-1).astype(work))
    outs = [np.zeros(op.out_dtensor.num_elements, dtype=work) for op in out_ops]
    smem = np.zeros(g.smem_offset // 2 + 8, dtype=work)

    def view(t: STensor):
        return smem[t.smem_offset // 2: t.smem_offset // 2 + t.num_elements]

    gx, gy, gz = g.grid_dim
    for bz in range(gz):
        for by in range(gy):
            for bx in range(gx):
                b = (bx, by, bz)
                for it in range(g.forloop_range):
                    oi = 0
                    for op in g.ops:
                        ty = op.type
                        if ty == TB_INPUT_OP:
                            st = op.outputs[0]
                            rbs, cbs, rfs, cfs, gbs, gfs = _input_offsets(g, op)
                            row = sum(b[a] * rbs[a] for a in range(3)) + it * rfs
                            col = sum(b[a] * cbs[a] for a in range(3)) + it * cfs
                            go = sum(b[a] * gbs[a] for a in range(3)) + it * gfs
                            R, C = st.dims[-2], st.dims[-1]
                            ld = op.dtensor.dims[-1]
                            src = flat_in[in_ops.index(op)]
                            idx = go + (row + np.arange(R))[:, None] * ld + col + np.arange(C)[None, :]
                            view(st)[:] = src[idx.reshape(-1)]
                        elif ty == TB_MATMUL_OP:
                            A, B, Cc = op.inputs[0], op.inputs[1], op.outputs[0]
                            m, k, n = A.dims[-2], A.dims[-1], B.dims[-1]
                            r = view(A).reshape(m, k) @ view(B).reshape(k, n)
                            view(Cc)[:] = (r % FP_PQ if mode == "fp" else r).reshape(-1)
                        elif ty == TB_EXP_OP:
                            v = view(op.outputs[0])
                            v[:] = fp_exp(v) if mode == "fp" else np.exp(v)
                        elif ty in (TB_DIV_OP, TB_ADD_OP):
                            d1, d2 = _bcast3(op.inputs[0]), _bcast3(op.inputs[1])
                            x = view(op.inputs[0]).reshape(d1)
                            y = view(op.inputs[1]).reshape(d2)
                            if ty == TB_DIV_OP:
                                z = fp_div(x, y) if mode == "fp" else x / y
                            else:
                                if mode == "fp":
                                    raise InvalidGraph("TB add has no fingerprint definition in the reference")
                                z = x + y
                            view(op.outputs[0])[:] = np.broadcast_to(z, [max(p, q) for p, q in zip(d1, d2)]).reshape(-1)
                        elif TB_REDUCTION_0_OP <= ty <= TB_REDUCTION_2_TO_DIMX_OP:
                            n_out, deg, inner = _reduction_params(op)
                            i = np.arange(n_out)
                            pos = (i // inner) * (inner * deg) + i % inner
                            gathered = view(op.inputs[0])[pos[:, None] + inner * np.arange(deg)[None, :]]
                            r = gathered.sum(axis=1)
                            view(op.outputs[0])[:] = r % FP_PQ if mode == "fp" else r
                        elif TB_CONCAT_0_OP <= ty <= TB_CONCAT_2_OP:
                            dim = ty - TB_CONCAT_0_OP
                            A, B = op.inputs
                            r = np.concatenate([view(A).reshape(A.dims), view(B).reshape(B.dims)], axis=dim)
                            view(op.outputs[0])[:] = r.reshape(-1)
                        elif ty == TB_OUTPUT_OP:
                            x, acc = view(op.inputs[0]), view(op.outputs[0])
                            if it == 0:
                                acc[:] = x
                            else:
                                acc[:] = (x + acc) % FP_PQ if mode == "fp" else x + acc
                            if it == g.forloop_range - 1:
                                st = op.inputs[0]
                                rbs, cbs, gbs = _output_offsets(g, op)
                                row = sum(b[a] * rbs[a] for a in range(3))
                                col = sum(b[a] * cbs[a] for a in range(3))
                                go = sum(b[a] * gbs[a] for a in range(3))
                                R, C = st.dims[-2], st.dims[-1]
                                ld = op.out_dtensor.dims[-1]
                                idx = go + (row + np.arange(R))[:, None] * ld + col + np.arange(C)[None, :]
                                outs[oi][idx.reshape(-1)] = acc
                            oi += 1
                        else:
                            raise InvalidGraph("unsupported operator %d" % ty)
    return [o.astype(out_dtype).reshape(op.out_dtensor.dims) for o, op in zip(outs, out_ops)]


def run_fingerprint(g: TBGraph, inputs):
    """Fingerprint-mode evaluation: uint16 in, uint16 out, layout flags ignored
    (input_loader.h:457-467 indexes row-major whatever the declared layout)."""
    return _run(g, inputs, np.uint16, "fp", layouts_matter=False)


def run_float(g: TBGraph, inputs):
    """fp32 evaluation of the graph semantics.  `inputs` hold the values as
    they sit in device memory (so a DmemColumnMajor tensor is passed as its
    memory image, shape ignored) already rounded to the 16-bit storage type."""
    return _run(g, inputs, np.float32, "float", layouts_matter=True)


# ---------------------------------------------------------------------------
# un-fused kernel-level operators (fingerprint domain)
# ---------------------------------------------------------------------------
def kn_matmul_fp(a, b):
    """matmul_kernel.cu:145-173, batched over leading dims."""
    return ((np.asarray(a, np.int64) @ np.asarray(b, np.int64)) % FP_PQ).astype(np.uint16)


def kn_exp_fp(x):
    return fp_exp(x).astype(np.uint16)


def kn_reduction_fp(x, dim, size=1):
    """reduction_kernel.cu:80-133: out[i] sums `factor` entries strided by the
    output's inner extent."""
    x = np.asarray(x, np.int64)
    factor = x.shape[dim] // size
    shp = list(x.shape)
    shp[dim:dim + 1] = [factor, size]
    return (x.reshape(shp).sum(axis=dim) % FP_PQ).astype(np.uint16)


def kn_div_fp(x, y):
    return fp_div(x, y).astype(np.uint16)


def kn_add_fp(x, y):
    return ((np.asarray(x, np.int64) + np.asarray(y, np.int64)) % FP_PQ).astype(np.uint16)


def kn_mul_fp(x, y):
    return ((np.asarray(x, np.int64) * np.asarray(y, np.int64)) % FP_PQ).astype(np.uint16)


# ---------------------------------------------------------------------------
# the benchmark configurations expressed as plans
# ---------------------------------------------------------------------------
def gqa_decode_plans(num_kv_heads, group, head_dim, kv_len, splits, forloop_range,
                     k_layout=DmemColumnMajor, v_layout=DmemColumnMajor, dtype=DT_FLOAT16):
    """The two customized ops of the grouped-query decode muGraph, pattern of
    cpp_examples/group_query_attn_inc_decode.cc:46-103 with free sizes.
    Returns (input specs, plan1, plan2)."""
    B, M, D, L = num_kv_heads, group, head_dim, kv_len
    ins = [DTensorSpec((B, M, D), dtype, DmemRowMajor),
           DTensorSpec((B, D, L), dtype, k_layout),
           DTensorSpec((B, L, D), dtype, v_layout)]
    plan1 = ExecutionPlan(
        ops=[(TB_MATMUL_OP, [(0, 0), (1, 0)]), (TB_EXP_OP, [(3, 0)]),
             (TB_MATMUL_OP, [(4, 0), (2, 0)]), (TB_REDUCTION_2_OP, [(4, 0)])],
        input_map=[(0, -1, -1), (0, 2, -1), (0, 1, -1)],
        forloop_dim=[-1, 2, 1],
        input_smem_layouts=[SmemRowMajorTensorOpMultiplicand_Crosswise64,
                            SmemColumnMajorTensorOpMultiplicand_Crosswise64,
                            SmemColumnMajorTensorOpMultiplicand_Crosswise64],
        output_map=(0, 2, -1), forloop_range=forloop_range,
        grid_dim=(B, splits, 1), reduction_dimx=D)
    plan2 = ExecutionPlan(
        ops=[(TB_REDUCTION_2_TO_DIMX_OP, [(0, 0)]), (TB_REDUCTION_2_OP, [(1, 0)]),
             (TB_DIV_OP, [(2, 0), (3, 0)])],
        input_map=[(0, -1, -1), (0, -1, -1)], forloop_dim=[-1, -1],
        input_smem_layouts=[SmemRowMajor, SmemRowMajor],
        output_map=(0, -1, -1), forloop_range=1, grid_dim=(B, 1, 1), reduction_dimx=D)
    return ins, plan1, plan2


def unfused_attention_fp(q, k, v):
    """Fingerprint of the un-fused graph matmul -> exp -> reduction -> div ->
    matmul (cpp_examples/group_query_attn_inc_decode.cc:16-27)."""
    a = kn_matmul_fp(q, k)
    e = kn_exp_fp(a)
    s = kn_reduction_fp(e, 2)
    d = kn_div_fp(e, s)
    return kn_matmul_fp(d, v)


def attention_fp32(q, k, v):
    """fp32 evaluation of the same un-fused graph on logical [B,M,D],[B,D,L],[B,L,D]."""
    q, k, v = (np.asarray(t, np.float32) for t in (q, k, v))
    e = np.exp(q @ k)
    return (e / e.sum(axis=2, keepdims=True)) @ v


def attention_fp32_causal_window(q, k, v, window):
    """Float-mode extension (no counterpart in the reference): the last `window` KV positions are a
    draft window; query row r belongs to draft token r // (rows // window) and sees KV positions
    <= kv_len - window + token.  Masked positions contribute neither to the numerator nor to the
    row sum."""
    q, k, v = (np.asarray(t, np.float32) for t in (q, k, v))
    B, M, D = q.shape
    L = k.shape[2]
    e = np.exp(q @ k)
    token = np.arange(M) // (M // window)
    visible = np.arange(L)[None, :] <= (L - window + token)[:, None]
    e = e * visible[None, :, :]
    return (e / e.sum(axis=2, keepdims=True)) @ v
