"""ctypes wrapper over oracle/_ref/libref_gpu.so - the reference's own GPU fingerprint kernel
(src/kernel/cuda/customized_kernel.cu, compute_customizedop_fingerprint), its arena and its input fill,
compiled for sm_100a by `make -C oracle refgpu`.  TEST INFRASTRUCTURE ONLY (see ref_gpu_driver.cu): the
same-box GPU comparator of the benchmark and a second source of golden fingerprints for the GPU tests.
Loading it needs a CUDA device; the first operator created allocates the reference's 10 GiB arena."""
import ctypes
import os

import numpy as np

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libref_gpu.so")
_lib = None


def available() -> bool:
    return os.path.exists(_PATH)


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_PATH)
        _lib.refgpu_customized_create.restype = ctypes.c_void_p
        _lib.refgpu_customized_output_ptr.restype = ctypes.c_void_p
        _lib.refgpu_time_pair.restype = ctypes.c_double
    return _lib


def _ints(seq):
    return (ctypes.c_int * max(1, len(seq)))(*[int(x) for x in seq])


class CustomizedOp:
    """One customized operator built by the reference's constructor.  `producer` = another CustomizedOp whose
    outputs are this operator's inputs (input_specs are then ignored)."""

    def __init__(self, input_specs, plan, producer=None):
        lib = _load()
        n = len(plan.input_map)
        ndims, dims, layouts, dtypes = [], [], [], []
        for s in (input_specs or []):
            ndims.append(len(s.dims))
            dims += list(s.dims) + [0] * (4 - len(s.dims))
            layouts.append(s.layout)
            dtypes.append(s.dtype)
        srcs = [x for _, ss in plan.ops for pair in ss for x in pair]
        info = (ctypes.c_int * 4)()
        h = lib.refgpu_customized_create(
            n, _ints(ndims), _ints(dims), _ints(layouts), _ints(dtypes), len(plan.ops), _ints([t for t, _ in plan.ops]),
            _ints([len(ss) for _, ss in plan.ops]), _ints(srcs), _ints([x for m in plan.input_map for x in m]),
            _ints(plan.forloop_dim), _ints(plan.input_smem_layouts), _ints(plan.output_map), int(plan.forloop_range),
            int(plan.reduction_dimx), _ints(plan.grid_dim), _ints(plan.block_dim),
            ctypes.c_void_p(producer.handle.value) if producer else None, info)
        self.handle = ctypes.c_void_p(h)
        self.info = dict(num_ops=info[0], num_params=info[1], smem_bytes=info[2], num_outputs=info[3])

    def fill_reference(self, idx):
        assert _load().refgpu_customized_fill_reference(self.handle, idx) == 0

    def set_input(self, idx, host_u16):
        a = np.ascontiguousarray(host_u16, dtype=np.uint16)
        assert _load().refgpu_customized_set_input(self.handle, idx, a.ctypes.data_as(ctypes.c_void_p)) == 0

    def set_input_from_device(self, idx, device_ptr):
        assert _load().refgpu_customized_set_input_from_device(self.handle, idx, ctypes.c_void_p(device_ptr)) == 0

    def fingerprint(self):
        assert _load().refgpu_customized_fingerprint(self.handle) == 0

    def output_shape(self, idx):
        nd = ctypes.c_int()
        d = (ctypes.c_int * 4)()
        _load().refgpu_customized_output_dims(self.handle, idx, ctypes.byref(nd), d)
        return tuple(d[j] for j in range(nd.value))

    def output(self, idx):
        o = np.zeros(self.output_shape(idx), np.uint16)
        assert _load().refgpu_customized_get_output(self.handle, idx, o.ctypes.data_as(ctypes.c_void_p)) == 0
        return o

    def output_ptr(self, idx):
        return _load().refgpu_customized_output_ptr(self.handle, idx)

    def destroy(self):
        if self.handle:
            _load().refgpu_customized_destroy(self.handle)
            self.handle = None


def has_same_fingerprint(a, a_idx, b, b_idx):
    """The reference's DTensor::has_same_fingerprint between two operators' outputs."""
    return bool(_load().refgpu_has_same_fingerprint(a.handle, a_idx, b.handle, b_idx))


def time_pair(op1, op2, iters):
    """Milliseconds per evaluation of a two-operator muGraph with the reference's protocol (one launch and one
    device synchronisation per operator)."""
    return float(_load().refgpu_time_pair(op1.handle, op2.handle, int(iters)))
