"""B200-native muGraph executor - Python surface.

Mirrors the names of the reference's Python binding (python/mirage/__init__.py:7-9 and
python/mirage/_cython/core.pyx:135-236: `new_graph`, `PyGraph.new_input/matmul/reduction/exp/add/
mul/div`, `PyTensor.dim/num_dims/dtype`) and adds what the reference exposes only in C++:
`PyGraph.customized(inputs, plan)` with an `ExecutionPlan`, `fingerprint()`, `profile()`, `run()`,
and tensor upload / download.  Everything goes through the C ABI of include/mugraph.h; there is no
Python or CPU implementation of any operator here.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import numpy as np

from . import _abi
from ._abi import MuGraphError, check, mg_plan, mg_tensor

__version__ = "0.1.0"

# ---- enums (numeric values of the reference) -----------------------------------------------------
bfloat16, float16, float32 = 920, 921, 930
DmemRowMajor, DmemColumnMajor = 100, 101
SmemRowMajor, SmemColumnMajor = 200, 201
SmemRowMajorTensorOpMultiplicand_Crosswise64 = 204
SmemColumnMajorTensorOpMultiplicand_Crosswise64 = 207
TB_MATMUL_OP, TB_EXP_OP, TB_ADD_OP, TB_MUL_OP, TB_DIV_OP = 2003, 2007, 2008, 2009, 2010
TB_REDUCTION_0_OP, TB_REDUCTION_1_OP, TB_REDUCTION_2_OP = 2101, 2102, 2103
TB_REDUCTION_0_TO_DIMX_OP, TB_REDUCTION_1_TO_DIMX_OP, TB_REDUCTION_2_TO_DIMX_OP = 2104, 2105, 2106
TB_CONCAT_0_OP, TB_CONCAT_1_OP, TB_CONCAT_2_OP = 2200, 2201, 2202
FP_P, FP_Q, FP_PQ = 227, 113, 25651

POLICY_LATENCY, POLICY_THROUGHPUT = 0, 1
(OPT_ATTN_STAGES, OPT_ATTN_TILE_GROUPS, OPT_ATTN_ENGINE, OPT_ROWS_ENGINE, OPT_INTERP_THREADS, OPT_WAIT_LIMIT,
 OPT_ATTN_PERSISTENT, OPT_KN_MATMUL_ENGINE, OPT_ATTN_DEPENDENT_LAUNCH) = range(9)
ENGINE_AUTO, ENGINE_MMA_SYNC, ENGINE_TCGEN05 = 0, 1, 2
ROWS_AUTO, ROWS_ONE_TILE, ROWS_TWO_TILES = 0, 1, 2
KERNEL_INTERPRETER, KERNEL_ATTN_SPLIT, KERNEL_ATTN_MERGE, KERNEL_ATTN_ROWS, KERNEL_MATMUL_CHAIN, KERNEL_TILE_REDUCE = range(6)


class InputNotFoundError(Exception):
    """Raised when input tensors cannot be found (name kept from the reference package)."""


@dataclass
class ExecutionPlan:
    """threadblock::ExecutionPlan (include/mirage/threadblock/graph.h:28-42)."""
    ops: List[Tuple[int, List[Tuple[int, int]]]]
    input_map: List[Tuple[int, int, int]]
    forloop_dim: List[int]
    input_smem_layouts: List[int]
    output_map: Tuple[int, int, int]
    forloop_range: int
    grid_dim: Tuple[int, int, int]
    block_dim: Tuple[int, int, int] = (128, 1, 1)
    reduction_dimx: int = 64

    def to_c(self):
        """Returns (mg_plan, keepalive) - the arrays must outlive the call."""
        i32 = ctypes.c_int32
        types = (i32 * max(1, len(self.ops)))(*[t for t, _ in self.ops])
        nsrc = (i32 * max(1, len(self.ops)))(*[len(s) for _, s in self.ops])
        flat = [x for _, s in self.ops for pair in s for x in pair]
        srcs = (i32 * max(1, len(flat)))(*flat)
        n = len(self.input_map)
        imap = (i32 * max(1, 3 * n))(*[x for m in self.input_map for x in m])
        fdim = (i32 * max(1, n))(*self.forloop_dim)
        lay = (i32 * max(1, n))(*self.input_smem_layouts)
        p = mg_plan()
        p.num_ops = len(self.ops)
        p.op_types, p.op_num_srcs, p.op_srcs = types, nsrc, srcs
        p.num_inputs = n
        p.input_map, p.forloop_dim, p.input_smem_layouts = imap, fdim, lay
        p.output_map = (i32 * 3)(*self.output_map)
        p.forloop_range = int(self.forloop_range)
        p.reduction_dimx = int(self.reduction_dimx)
        p.grid_dim = (i32 * 3)(*self.grid_dim)
        p.block_dim = (i32 * 3)(*self.block_dim)
        return p, (types, nsrc, srcs, imap, fdim, lay)


class Runtime:
    """The process-wide device memory manager (reference: DeviceMemoryManager singleton)."""
    _instance = None

    def __init__(self, device=0, arena_bytes=0):
        self.lib = _abi.load()
        h = ctypes.c_void_p()
        check(self.lib.mg_runtime_create(device, arena_bytes, ctypes.byref(h)))
        self.handle = h
        self.device = device

    @classmethod
    def get(cls, device=0, arena_bytes=0):
        if cls._instance is None:
            cls._instance = Runtime(device, arena_bytes)
        return cls._instance

    @classmethod
    def shutdown(cls):
        if cls._instance is not None:
            check(cls._instance.lib.mg_runtime_destroy(cls._instance.handle))
            cls._instance = None

    def arena_usage(self):
        used, total = ctypes.c_size_t(), ctypes.c_size_t()
        check(self.lib.mg_runtime_arena_usage(self.handle, ctypes.byref(used), ctypes.byref(total)))
        return used.value, total.value

    def set_max_smem(self, nbytes):
        check(self.lib.mg_runtime_set_max_smem(self.handle, nbytes))

    def set_specialisation(self, level):
        """0 / False = generic interpreters only, 1 = specialised kernels, 2 / True = specialised kernels plus
        one-launch fusion of the split-KV attention operator with its merge operator."""
        level = 2 if level is True else (0 if level is False else int(level))
        check(self.lib.mg_runtime_set_specialisation(self.handle, level))

    def set_launch_policy(self, policy):
        """POLICY_LATENCY (one call at a time) or POLICY_THROUGHPUT (several independent calls in flight)."""
        check(self.lib.mg_runtime_set_launch_policy(self.handle, int(policy)))

    def set_option(self, key, value):
        """Tuning switch OPT_* (0 = automatic); read when a launch is configured."""
        check(self.lib.mg_runtime_set_option(self.handle, int(key), int(value)))

    def get_option(self, key):
        v = ctypes.c_int32()
        check(self.lib.mg_runtime_get_option(self.handle, int(key), ctypes.byref(v)))
        return v.value

    def selftest_bounded_wait(self, poll_limit=4096, stream=None):
        """Enqueue the failure-path self-test: a wait nobody satisfies gives up after `poll_limit` polls and sets
        the device status word; the next synchronising call raises MG_ERR_DEVICE_TIMEOUT once."""
        check(self.lib.mg_selftest_bounded_wait(self.handle, int(poll_limit), ctypes.c_void_p(stream or 0)))

    def tables(self):
        """Host copies of the arena's exp / div_p / div_q lookup tables."""
        e, p, q = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        check(self.lib.mg_runtime_tables(self.handle, ctypes.byref(e), ctypes.byref(p), ctypes.byref(q)))
        out = []
        for ptr, n in ((e, 113), (p, 227), (q, 113)):
            host = np.zeros(n, np.uint16)
            t = mg_tensor()
            t.data_type, t.num_dims, t.dim[0], t.fp_ptr = float16, 1, n, ptr.value
            check(self.lib.mg_tensor_download_fingerprint(self.handle, ctypes.byref(t), host.ctypes.data))
            out.append(host)
        return out


class PyTensor:
    """A device tensor of a graph (reference: PyTensor, core.pyx:135-177)."""

    def __init__(self, graph: "PyGraph", pod: mg_tensor):
        self.graph = graph
        self.pod = pod

    @property
    def num_dims(self):
        return self.pod.num_dims

    @property
    def dtype(self):
        return self.pod.data_type

    @property
    def layout(self):
        return self.pod.layout

    def dim(self, idx):
        assert idx < self.pod.num_dims, "Error: index out of range"
        return self.pod.dim[idx]

    @property
    def shape(self):
        return tuple(self.pod.dim[i] for i in range(self.pod.num_dims))

    @property
    def num_elements(self):
        return int(np.prod(self.shape))

    # -- contents ---------------------------------------------------------------------------------
    def upload_fingerprint(self, host):
        a = np.ascontiguousarray(host, dtype=np.uint16)
        assert a.size == self.num_elements
        g = self.graph
        check(g.lib.mg_tensor_upload_fingerprint(g.rt.handle, ctypes.byref(self.pod), a.ctypes.data))

    def download_fingerprint(self):
        out = np.zeros(self.shape, np.uint16)
        g = self.graph
        check(g.lib.mg_tensor_download_fingerprint(g.rt.handle, ctypes.byref(self.pod), out.ctypes.data))
        return out

    def upload_data(self, host_bits):
        """host_bits: uint16 array holding the fp16 / bf16 bit patterns in memory order."""
        a = np.ascontiguousarray(host_bits).view(np.uint16)
        assert a.size == self.num_elements
        g = self.graph
        check(g.lib.mg_tensor_upload_data(g.rt.handle, ctypes.byref(self.pod), a.ctypes.data))

    def download_data(self):
        """Bit patterns (uint16) in memory order."""
        out = np.zeros(self.num_elements, np.uint16)
        g = self.graph
        check(g.lib.mg_tensor_download_data(g.rt.handle, ctypes.byref(self.pod), out.ctypes.data))
        return out

    def fill_fingerprint_reference(self):
        g = self.graph
        check(g.lib.mg_tensor_fill_fingerprint_reference(g.rt.handle, ctypes.byref(self.pod)))

    def fill_fingerprint_seeded(self, seed, modulus=FP_P):
        g = self.graph
        check(g.lib.mg_tensor_fill_fingerprint_seeded(g.rt.handle, ctypes.byref(self.pod), seed, modulus))

    def fill_data_seeded(self, seed, sigma=1.0):
        g = self.graph
        check(g.lib.mg_tensor_fill_data_seeded(g.rt.handle, ctypes.byref(self.pod), seed, sigma))

    def has_same_fingerprint(self, other: "PyTensor"):
        same = ctypes.c_int32()
        g = self.graph
        check(g.lib.mg_tensor_has_same_fingerprint(g.rt.handle, ctypes.byref(self.pod), ctypes.byref(other.pod),
                                                   ctypes.byref(same)))
        return bool(same.value)


class PyGraph:
    """kernel::Graph (reference: PyGraph, core.pyx:180-236) plus the customized-operator API."""

    def __init__(self, runtime: Runtime = None, _handle=None):
        self.rt = runtime or Runtime.get()
        self.lib = self.rt.lib
        if _handle is None:
            _handle = ctypes.c_void_p()
            check(self.lib.mg_graph_create(self.rt.handle, ctypes.byref(_handle)))
        self.handle = _handle

    # -- graph JSON wire format (to_json / from_json, src/kernel/graph.cc:33-159) --------------------
    @classmethod
    def from_json(cls, document, runtime: Runtime = None):
        """Rebuild a graph from the reference's JSON form: a list of operators as `json(graph)` prints it, e.g.
        one entry of a search checkpoint's "generated_graphs".  `document` is the text or the parsed list."""
        import json as _json
        rt = runtime or Runtime.get()
        text = document if isinstance(document, str) else _json.dumps(document)
        h = ctypes.c_void_p()
        check(rt.lib.mg_graph_from_json(rt.handle, text.encode(), ctypes.byref(h)))
        return cls(rt, _handle=h)

    def to_json(self):
        """`json(graph).dump()` of the reference (keys in alphabetical order)."""
        need = ctypes.c_size_t()
        self.lib.mg_graph_to_json(self.handle, None, 0, ctypes.byref(need))
        buf = ctypes.create_string_buffer(need.value + 1)
        check(self.lib.mg_graph_to_json(self.handle, buf, need.value + 1, ctypes.byref(need)))
        return buf.value.decode()

    def operator(self, op_idx):
        """(KN operator type code, [output tensors]) of operator op_idx - the way to reach the tensors of a
        graph that was loaded from JSON."""
        t, n = ctypes.c_int32(), ctypes.c_int32()
        outs = (mg_tensor * 8)()
        check(self.lib.mg_graph_operator_info(self.handle, op_idx, ctypes.byref(t), outs, 8, ctypes.byref(n)))
        tensors = []
        for i in range(min(8, n.value)):
            pod = mg_tensor()
            ctypes.memmove(ctypes.byref(pod), ctypes.byref(outs[i]), ctypes.sizeof(mg_tensor))
            tensors.append(PyTensor(self, pod))
        return t.value, tensors

    def close(self):
        if self.handle is not None:
            check(self.lib.mg_graph_destroy(self.handle))
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- builders ---------------------------------------------------------------------------------
    def new_input(self, dims: tuple, dtype=float16, layout=DmemRowMajor):
        arr = (ctypes.c_int32 * len(dims))(*dims)
        t = mg_tensor()
        check(self.lib.mg_graph_new_input(self.handle, arr, len(dims), dtype, layout, ctypes.byref(t)))
        return PyTensor(self, t)

    def _binary(self, fn, A, B):
        t = mg_tensor()
        check(fn(self.handle, ctypes.byref(A.pod), ctypes.byref(B.pod), ctypes.byref(t)))
        return PyTensor(self, t)

    def matmul(self, A, B):
        return self._binary(self.lib.mg_graph_matmul, A, B)

    def add(self, A, B):
        return self._binary(self.lib.mg_graph_add, A, B)

    def mul(self, A, B):
        return self._binary(self.lib.mg_graph_mul, A, B)

    def div(self, A, B):
        return self._binary(self.lib.mg_graph_div, A, B)

    def exp(self, A):
        t = mg_tensor()
        check(self.lib.mg_graph_exp(self.handle, ctypes.byref(A.pod), ctypes.byref(t)))
        return PyTensor(self, t)

    def reduction(self, A, dim, size=1):
        t = mg_tensor()
        check(self.lib.mg_graph_reduction(self.handle, ctypes.byref(A.pod), dim, size, ctypes.byref(t)))
        return PyTensor(self, t)

    def customized(self, inputs: Sequence[PyTensor], plan: ExecutionPlan):
        """Graph::customized(inputs, plan) (src/kernel/customized.cc:32-44)."""
        n = len(inputs)
        ins = (mg_tensor * max(1, n))(*[t.pod for t in inputs])
        outs = (mg_tensor * 8)()
        nout = ctypes.c_int32()
        cplan, keep = plan.to_c()
        check(self.lib.mg_graph_customized(self.handle, ins, n, ctypes.byref(cplan), outs, 8, ctypes.byref(nout)))
        del keep
        res = []
        for i in range(nout.value):
            t = mg_tensor()
            ctypes.memmove(ctypes.byref(t), ctypes.byref(outs[i]), ctypes.sizeof(mg_tensor))
            res.append(PyTensor(self, t))
        return res

    # -- execution ----------------------------------------------------------------------------------
    @property
    def num_operators(self):
        n = ctypes.c_int32()
        check(self.lib.mg_graph_num_operators(self.handle, ctypes.byref(n)))
        return n.value

    def customized_info(self, op_idx):
        a, b, c, d = (ctypes.c_int32() for _ in range(4))
        check(self.lib.mg_graph_customized_info(self.handle, op_idx, ctypes.byref(a), ctypes.byref(b),
                                                ctypes.byref(c), ctypes.byref(d)))
        return dict(num_tb_operators=a.value, smem_bytes=b.value, kernel_fingerprint=c.value, kernel_float=d.value)

    def customized_program(self, op_idx):
        """The lowered kernel-level program (block / for-loop strides, tile offsets) of a customized op."""
        prog = _abi.mgd_program()
        check(self.lib.mg_graph_customized_program(self.handle, op_idx, ctypes.byref(prog), ctypes.sizeof(prog)))
        return prog

    def set_causal_window(self, op_idx, window):
        check(self.lib.mg_graph_customized_set_causal_window(self.handle, op_idx, window))

    def fingerprint(self, refill_inputs=False):
        """Evaluate every operator in fingerprint mode (`for op in graph.operators: op.fingerprint()`).
        refill_inputs=True also runs the input operators' fill fp[i] = i % FP_PQ, like the reference."""
        if refill_inputs:
            check(self.lib.mg_graph_fingerprint(self.handle))
        else:
            check(self.lib.mg_graph_fingerprint_compute(self.handle))

    def fingerprint_op(self, op_idx):
        check(self.lib.mg_op_fingerprint(self.handle, op_idx))

    def run(self, stream=None, sync=True):
        check(self.lib.mg_graph_run(self.handle, ctypes.c_void_p(stream or 0)))
        if sync:
            check(self.lib.mg_device_synchronize())

    def run_op(self, op_idx, stream=None):
        check(self.lib.mg_op_run(self.handle, op_idx, ctypes.c_void_p(stream or 0)))

    def profile_op(self, op_idx, warmup=0, iters=0):
        """KNOperator::profile: mean milliseconds per launch (0,0 = the reference's 1024 + 1024)."""
        ms = ctypes.c_float()
        check(self.lib.mg_op_profile(self.handle, op_idx, warmup, iters, ctypes.byref(ms)))
        return ms.value

    def rebind_input(self, op_idx, data_ptr=None, fp_ptr=None):
        check(self.lib.mg_graph_rebind_input(self.handle, op_idx, ctypes.c_void_p(data_ptr or 0),
                                             ctypes.c_void_p(fp_ptr or 0)))

    def fingerprint_batched(self, num_sets, in_ptrs, out_ptr, workspace_ptr, workspace_bytes, stream=None):
        arr = (ctypes.c_void_p * len(in_ptrs))(*in_ptrs)
        sz = ctypes.c_size_t(workspace_bytes)
        check(self.lib.mg_graph_fingerprint_batched(self.handle, num_sets, arr, ctypes.c_void_p(out_ptr),
                                                    ctypes.c_void_p(workspace_ptr), ctypes.byref(sz),
                                                    ctypes.c_void_p(stream or 0)))

    def run_batched(self, num_sets, in_ptrs, out_ptr, workspace_ptr, workspace_bytes, stream=None):
        """`num_sets` independent float-mode calls of this graph as one pass (device pointers to dense
        [set][tensor] arrays of 16-bit values); asynchronous on `stream`."""
        arr = (ctypes.c_void_p * len(in_ptrs))(*in_ptrs)
        sz = ctypes.c_size_t(workspace_bytes)
        check(self.lib.mg_graph_run_batched(self.handle, num_sets, arr, ctypes.c_void_p(out_ptr),
                                            ctypes.c_void_p(workspace_ptr), ctypes.byref(sz), ctypes.c_void_p(stream or 0)))

    def run_batched_workspace(self, num_sets):
        sz = ctypes.c_size_t(0)
        check(self.lib.mg_graph_run_batched(self.handle, num_sets, None, None, None, ctypes.byref(sz), None))
        return sz.value

    def fingerprint_batched_workspace(self, num_sets):
        sz = ctypes.c_size_t(0)
        check(self.lib.mg_graph_fingerprint_batched(self.handle, num_sets, None, None, None, ctypes.byref(sz), None))
        return sz.value


def verify_candidates(reference: "PyTensor", candidates, stream=None):
    """The search's verify step for a batch (src/search/search.cc:569-623): `candidates` is a list of
    (PyGraph, output PyTensor) whose inputs are already in place; every graph is evaluated in fingerprint mode and
    its output compared with `reference` on the device - one synchronisation for the whole batch.  Returns a list
    of bools."""
    n = len(candidates)
    if n == 0:
        return []
    rt = reference.graph.rt
    graphs = (ctypes.c_void_p * n)(*[g.handle for g, _ in candidates])
    outs = (mg_tensor * n)(*[t.pod for _, t in candidates])
    same = (ctypes.c_int32 * n)()
    check(rt.lib.mg_verify_candidates(rt.handle, ctypes.byref(reference.pod), graphs, outs, n, same,
                                      ctypes.c_void_p(stream or 0)))
    return [bool(v) for v in same]


class CapturedSequence:
    """A launch sequence captured into a CUDA graph on `stream` (a raw cudaStream_t value)."""

    def __init__(self, stream, record):
        self.lib = _abi.load()
        self.stream = ctypes.c_void_p(stream)
        before = launch_count()
        check(self.lib.mg_capture_begin(self.stream))
        try:
            record()
        finally:
            h = ctypes.c_void_p()
            st = self.lib.mg_capture_end(self.stream, ctypes.byref(h))
        check(st)
        self.handle = h
        self.kernels = launch_count() - before  # kernels one replay launches

    def launch(self):
        check(self.lib.mg_captured_launch(self.handle, self.stream))

    def close(self):
        if self.handle:
            check(self.lib.mg_captured_destroy(self.handle))
            self.handle = None


def compare_fingerprint_rows(runtime, a_ptr, b_ptr, rows, row_elements, flags_ptr, mismatch_count_ptr=None, stream=None):
    """Row-wise equality of two device arrays of fingerprints; flags_ptr -> int32[rows] (1 = equal),
    mismatch_count_ptr -> optional int32 (rows that differ).  Asynchronous on `stream`."""
    check(runtime.lib.mg_compare_fingerprint_rows(runtime.handle, ctypes.c_void_p(a_ptr), ctypes.c_void_p(b_ptr), int(rows),
                                                  int(row_elements), ctypes.c_void_p(flags_ptr),
                                                  ctypes.c_void_p(mismatch_count_ptr or 0), ctypes.c_void_p(stream or 0)))


def fill_data_seeded_raw(runtime, device_ptr, num_elements, seed, sigma, dtype=None):
    """Seeded N(0, sigma) fill of caller-owned device memory holding 16-bit floats."""
    pod = mg_tensor()
    pod.data_type, pod.num_dims, pod.dim[0] = dtype or float16, 1, int(num_elements)
    pod.data_ptr = int(device_ptr)
    check(runtime.lib.mg_tensor_fill_data_seeded(runtime.handle, ctypes.byref(pod), int(seed), float(sigma)))


def fill_fingerprint_seeded_raw(runtime, device_ptr, num_elements, seed, modulus=FP_P):
    """Seeded uniform fill of caller-owned device memory (uint16 fingerprints), same generator as
    PyTensor.fill_fingerprint_seeded."""
    pod = mg_tensor()
    pod.data_type, pod.num_dims, pod.dim[0] = float16, 1, int(num_elements)
    pod.fp_ptr = int(device_ptr)
    check(runtime.lib.mg_tensor_fill_fingerprint_seeded(runtime.handle, ctypes.byref(pod), int(seed), int(modulus)))


def stream_inputs_written(stream=None):
    """Tell the library that work of the caller's own on `stream` wrote input tensors of its graphs."""
    check(_abi.load().mg_stream_inputs_written(ctypes.c_void_p(stream or 0)))


def new_graph():
    return PyGraph()


def synchronize():
    check(_abi.load().mg_device_synchronize())


def launch_count():
    return int(_abi.load().mg_launch_count())


# ---- the benchmark muGraphs as plans --------------------------------------------------------------
def attention_prefill_plans(heads, seq_q, head_dim, kv_len, q_tile=128, kv_tile=128):
    """The two customized operators of the dense (prefill) attention muGraph (pattern of the reference's
    cpp_examples/multi_head_attn_prefill.cc:43-98): op1 accumulates E V and rowsum(E) over KV tiles for a tile of
    query rows, op2 divides.  Inputs Q[heads, seq_q, d], K[heads, d, kv_len], V[heads, kv_len, d]."""
    qt = seq_q // q_tile
    plan1 = ExecutionPlan(
        ops=[(TB_MATMUL_OP, [(0, 0), (1, 0)]), (TB_EXP_OP, [(3, 0)]),
             (TB_MATMUL_OP, [(4, 0), (2, 0)]), (TB_REDUCTION_2_OP, [(4, 0)])],
        input_map=[(0, 1, -1), (0, -1, -1), (0, -1, -1)], forloop_dim=[-1, 2, 1],
        input_smem_layouts=[SmemRowMajor, SmemColumnMajor, SmemColumnMajor],
        output_map=(0, 1, -1), forloop_range=kv_len // kv_tile, grid_dim=(heads, qt, 1), reduction_dimx=head_dim)
    plan2 = ExecutionPlan(
        ops=[(TB_DIV_OP, [(0, 0), (1, 0)])], input_map=[(0, 1, -1), (0, 1, -1)], forloop_dim=[-1, -1],
        input_smem_layouts=[SmemRowMajor, SmemRowMajor], output_map=(0, 1, -1), forloop_range=1,
        grid_dim=(heads, qt, 1), reduction_dimx=head_dim)
    return plan1, plan2


def gqa_decode_plans(num_kv_heads, group, head_dim, kv_len, splits, forloop_range):
    """The two customized operators of the grouped-query decode muGraph (pattern of the reference's
    cpp_examples/group_query_attn_inc_decode.cc:46-103).  Returns (plan1, plan2)."""
    plan1 = ExecutionPlan(
        ops=[(TB_MATMUL_OP, [(0, 0), (1, 0)]), (TB_EXP_OP, [(3, 0)]),
             (TB_MATMUL_OP, [(4, 0), (2, 0)]), (TB_REDUCTION_2_OP, [(4, 0)])],
        input_map=[(0, -1, -1), (0, 2, -1), (0, 1, -1)], forloop_dim=[-1, 2, 1],
        input_smem_layouts=[SmemRowMajorTensorOpMultiplicand_Crosswise64,
                            SmemColumnMajorTensorOpMultiplicand_Crosswise64,
                            SmemColumnMajorTensorOpMultiplicand_Crosswise64],
        output_map=(0, 2, -1), forloop_range=forloop_range, grid_dim=(num_kv_heads, splits, 1),
        reduction_dimx=head_dim)
    plan2 = ExecutionPlan(
        ops=[(TB_REDUCTION_2_TO_DIMX_OP, [(0, 0)]), (TB_REDUCTION_2_OP, [(1, 0)]), (TB_DIV_OP, [(2, 0), (3, 0)])],
        input_map=[(0, -1, -1), (0, -1, -1)], forloop_dim=[-1, -1], input_smem_layouts=[SmemRowMajor, SmemRowMajor],
        output_map=(0, -1, -1), forloop_range=1, grid_dim=(num_kv_heads, 1, 1), reduction_dimx=head_dim)
    return plan1, plan2
