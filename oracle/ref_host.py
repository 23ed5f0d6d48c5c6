"""ctypes wrapper over oracle/_ref/libref_host.so - the reference's own host
code for building and fingerprinting a customized operator, run on the CPU.
TEST INFRASTRUCTURE ONLY (see ref_host_driver.cc).  Available only where the
library has been built from a reference checkout (`make -C oracle ref`)."""
import ctypes
import os

import numpy as np

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libref_host.so")


def available() -> bool:
    return os.path.exists(_PATH)


_lib = None


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_PATH)
        _lib.ref_customized_create.restype = ctypes.c_void_p
    return _lib


def _ints(seq):
    arr = (ctypes.c_int * max(1, len(seq)))(*[int(x) for x in seq])
    return arr


def set_threads(n):
    """OpenMP threads for the block loop (n <= 0 leaves the setting); returns the count in effect."""
    return int(_load().ref_set_threads(int(n)))


def tables():
    lib = _load()
    e = np.zeros(113, np.uint16)
    p = np.zeros(227, np.uint16)
    q = np.zeros(113, np.uint16)
    lib.ref_tables(e.ctypes.data_as(ctypes.c_void_p), p.ctypes.data_as(ctypes.c_void_p),
                   q.ctypes.data_as(ctypes.c_void_p))
    return e, p, q


def customized_fingerprint(input_specs, plan, inputs):
    """input_specs: objects with .dims/.dtype/.layout; plan: object with the
    ExecutionPlan fields; inputs: uint16 arrays.  Returns (outputs, info) where
    info = dict(num_ops, num_params, smem_bytes)."""
    lib = _load()
    n = len(input_specs)
    ndims = [len(s.dims) for s in input_specs]
    dims = []
    for s in input_specs:
        dims += list(s.dims) + [0] * (4 - len(s.dims))
    srcs = []
    for _, ss in plan.ops:
        for (a, b) in ss:
            srcs += [a, b]
    imap = [x for m in plan.input_map for x in m]
    info = (ctypes.c_int * 4)()
    h = lib.ref_customized_create(
        n, _ints(ndims), _ints(dims), _ints([s.layout for s in input_specs]), _ints([s.dtype for s in input_specs]),
        len(plan.ops), _ints([t for t, _ in plan.ops]), _ints([len(ss) for _, ss in plan.ops]), _ints(srcs),
        _ints(imap), _ints(plan.forloop_dim), _ints(plan.input_smem_layouts), _ints(plan.output_map),
        int(plan.forloop_range), int(plan.reduction_dimx), _ints(plan.grid_dim), _ints(plan.block_dim), info)
    h = ctypes.c_void_p(h)
    try:
        for i, a in enumerate(inputs):
            a = np.ascontiguousarray(a, dtype=np.uint16)
            lib.ref_customized_set_input(h, i, a.ctypes.data_as(ctypes.c_void_p))
        lib.ref_customized_fingerprint(h)
        outs = []
        for i in range(info[3]):
            nd = ctypes.c_int()
            d = (ctypes.c_int * 4)()
            lib.ref_customized_output_dims(h, i, ctypes.byref(nd), d)
            shape = tuple(d[j] for j in range(nd.value))
            o = np.zeros(shape, np.uint16)
            lib.ref_customized_get_output(h, i, o.ctypes.data_as(ctypes.c_void_p))
            outs.append(o)
    finally:
        lib.ref_customized_destroy(h)
    return outs, dict(num_ops=info[0], num_params=info[1], smem_bytes=info[2])
