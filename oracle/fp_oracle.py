"""ctypes wrapper over oracle/libfp_oracle.so (fp_oracle.c).  TEST INFRASTRUCTURE ONLY.

Flattens a graph built by mugraph_oracle.build_customized into the 20-int operator records the C
code reads: {type, a[0..18]} with
  input      a[0..2] row block strides, a[3..5] column block strides, a[6] row for-loop stride,
             a[7] column for-loop stride, a[8..10] leading-dim block strides, a[11] leading-dim
             for-loop stride, a[12..13] tensor rows, cols, a[14..15] tile rows, cols, a[17] tile offset,
             a[18] input slot
  output     a[0..2], a[3..5] row / column block strides, a[6..8] leading-dim block strides,
             a[9..10] tensor rows, cols, a[11..12] tile rows, cols, a[13] source offset,
             a[14] accumulator offset, a[15] output slot
  matmul     m, n, k, offsets A, B, C        exp   offset, elements
  div        shapes x, y (3 each), offsets x, y, out
  reduction  output elements, degree, inner, offsets in, out
  concat     output elements, extents A, B, inner, offsets A, B, out
"""
import ctypes
import os
import subprocess

import numpy as np

from . import mugraph_oracle as mo

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "libfp_oracle.so")
_lib = None


def available():
    return os.path.exists(_PATH)


def ensure_built():
    if not available():
        subprocess.run(["make", "-C", _HERE, "port"], check=True, capture_output=True)


def _load():
    global _lib
    if _lib is None:
        ensure_built()
        _lib = ctypes.CDLL(_PATH)
        _lib.fp_oracle_run.restype = ctypes.c_int
        _lib.f32_oracle_run.restype = ctypes.c_int
    return _lib


def flatten(g: mo.TBGraph):
    recs = []
    n_in = n_out = 0
    for op in g.ops:
        a = [0] * 19
        if op.type == mo.TB_INPUT_OP:
            rbs, cbs, rfs, cfs, gbs, gfs = mo._input_offsets(g, op)
            st = op.outputs[0]
            a[0:3], a[3:6], a[6], a[7], a[8:11], a[11] = rbs, cbs, rfs, cfs, gbs, gfs
            a[12], a[13] = op.dtensor.dims[-2], op.dtensor.dims[-1]
            a[14], a[15], a[16], a[17], a[18] = st.dims[-2], st.dims[-1], op.dtensor.layout, st.smem_offset, n_in
            n_in += 1
        elif op.type == mo.TB_OUTPUT_OP:
            rbs, cbs, gbs = mo._output_offsets(g, op)
            st = op.inputs[0]
            a[0:3], a[3:6], a[6:9] = rbs, cbs, gbs
            a[9], a[10] = op.out_dtensor.dims[-2], op.out_dtensor.dims[-1]
            a[11], a[12], a[13], a[14], a[15] = st.dims[-2], st.dims[-1], st.smem_offset, op.outputs[0].smem_offset, n_out
            n_out += 1
        elif op.type == mo.TB_MATMUL_OP:
            A, B, C = op.inputs[0], op.inputs[1], op.outputs[0]
            a[0:6] = [A.dims[-2], B.dims[-1], A.dims[-1], A.smem_offset, B.smem_offset, C.smem_offset]
        elif op.type == mo.TB_EXP_OP:
            a[0:2] = [op.inputs[0].smem_offset, op.inputs[0].num_elements]
        elif op.type in (mo.TB_DIV_OP, mo.TB_ADD_OP, mo.TB_MUL_OP):
            a[0:3], a[3:6] = mo._bcast3(op.inputs[0]), mo._bcast3(op.inputs[1])
            a[6:9] = [op.inputs[0].smem_offset, op.inputs[1].smem_offset, op.outputs[0].smem_offset]
        elif mo.TB_REDUCTION_0_OP <= op.type <= mo.TB_REDUCTION_2_TO_DIMX_OP:
            n, deg, inner = mo._reduction_params(op)
            a[0:5] = [n, deg, inner, op.inputs[0].smem_offset, op.outputs[0].smem_offset]
        elif mo.TB_CONCAT_0_OP <= op.type <= mo.TB_CONCAT_2_OP:
            dim = op.type - mo.TB_CONCAT_0_OP
            A, B, out = op.inputs[0], op.inputs[1], op.outputs[0]
            a[0:7] = [out.num_elements, A.dims[dim], B.dims[dim], int(np.prod(out.dims[dim + 1:])), A.smem_offset,
                      B.smem_offset, out.smem_offset]
        else:
            raise mo.InvalidGraph("operator %d has no fingerprint definition" % op.type)
        recs += [op.type] + [int(v) for v in a]
    return np.array(recs, dtype=np.int32), n_in, n_out


def run(g: mo.TBGraph, inputs, num_sets=1, threads=0):
    """inputs: uint16 arrays, each holding `num_sets` sets back to back.  Returns (outputs, threads used)."""
    lib = _load()
    recs, n_in, n_out = flatten(g)
    specs = mo.output_specs(g)
    ins = [np.ascontiguousarray(a, dtype=np.uint16) for a in inputs]
    outs = [np.zeros((num_sets,) + tuple(s.dims), np.uint16) for s in specs]
    in_ptr = (ctypes.c_void_p * 8)(*[a.ctypes.data for a in ins])
    out_ptr = (ctypes.c_void_p * 8)(*[a.ctypes.data for a in outs])
    in_stride = (ctypes.c_int64 * 8)(*[a.size // num_sets for a in ins])
    out_stride = (ctypes.c_int64 * 8)(*[s.num_elements for s in specs])
    grid = (ctypes.c_int32 * 3)(*g.grid_dim)
    used = lib.fp_oracle_run(recs.ctypes.data_as(ctypes.c_void_p), len(g.ops), grid, g.forloop_range, g.smem_offset,
                             n_in, in_ptr, in_stride, n_out, out_ptr, out_stride, num_sets, threads)
    if num_sets == 1:
        outs = [o[0] for o in outs]
    return outs, used


def run_float(g: mo.TBGraph, inputs, threads=0):
    """fp32 evaluation by f32_oracle.c.  inputs: float arrays in memory order (already rounded to the
    16-bit storage type).  Returns (outputs as float32 arrays, threads used)."""
    lib = _load()
    recs, n_in, n_out = flatten(g)
    specs = mo.output_specs(g)
    ins = [np.ascontiguousarray(a, dtype=np.float32) for a in inputs]
    outs = [np.zeros(tuple(s.dims), np.float32) for s in specs]
    in_ptr = (ctypes.c_void_p * 8)(*[a.ctypes.data for a in ins])
    out_ptr = (ctypes.c_void_p * 8)(*[a.ctypes.data for a in outs])
    grid = (ctypes.c_int32 * 3)(*g.grid_dim)
    used = lib.f32_oracle_run(recs.ctypes.data_as(ctypes.c_void_p), len(g.ops), grid, g.forloop_range, g.smem_offset,
                              n_in, in_ptr, n_out, out_ptr, threads)
    return outs, used
