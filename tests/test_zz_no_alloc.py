"""The allocation-free decode entry point (`mgd_attn_decode_fused_noalloc`).

Some embedders cannot let this library allocate: a serving process whose own pool has already claimed the
GPU's memory, or a latency-critical loop where cudaMalloc / cudaFree would stall the device.  For them the
library offers one launch whose scratch (ticket counters + status word) sits in a static device array.  This
test calls it through the C ABI with caller-owned buffers, twice in a row, and compares each result with the
regular graph path on the same inputs.  The file name sorts last on purpose: a run that stops at the first
failure has by then executed every other test."""
import ctypes

import numpy as np
import pytest

import attention_superoptimizer_b200 as mg
from attention_superoptimizer_b200 import _abi
from oracle import mugraph_oracle as mo
from tests.helpers import assert_close, from_bits, to_bits

pytestmark = pytest.mark.gpu


class mgd_attn_split(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("heads", "m", "d", "kv_len", "splits", "forloop_range", "k_layout",
                                               "v_layout", "data_type", "causal_window", "num_sets", "reserved")] + \
               [(n, ctypes.c_int64) for n in ("q_set_stride", "k_set_stride", "v_set_stride", "o_set_stride",
                                               "r_set_stride")]


def noalloc_call(lib, desc, q, k, v, o_part, r_part, out, fp_mode):
    lib.mgd_last_error.restype = ctypes.c_char_p
    fn = lib.mgd_attn_decode_fused_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(mgd_attn_split)] + [ctypes.c_void_p] * 6 + [ctypes.c_int32, ctypes.c_int32,
                                                                                ctypes.c_void_p]
    st = fn(ctypes.byref(desc), q, k, v, o_part, r_part, out, fp_mode, 1, None)
    assert st == 0, lib.mgd_last_error()


def test_no_alloc_entry_matches_graph_path_twice(runtime):
    import torch
    B, M, D, L, S, F = 8, 4, 128, 4096, 16, 4
    runtime.set_max_smem(227 * 1024)
    runtime.set_specialisation(2)
    lib = _abi.load()
    rng = np.random.default_rng(123)
    with mg.PyGraph(runtime) as g:
        Q = g.new_input((B, M, D), mg.float16)
        K = g.new_input((B, D, L), mg.float16, mg.DmemColumnMajor)
        V = g.new_input((B, L, D), mg.float16, mg.DmemRowMajor)
        p1, p2 = mg.gqa_decode_plans(B, M, D, L, S, F)
        parts = g.customized([Q, K, V], p1)
        final = g.customized(parts, p2)
        desc = mgd_attn_split(heads=B, m=M, d=D, kv_len=L, splits=S, forloop_range=F, k_layout=mg.DmemColumnMajor,
                              v_layout=mg.DmemRowMajor, data_type=mg.float16, causal_window=0, num_sets=1)
        # caller-owned outputs (here: torch tensors; nothing is allocated inside the entry point)
        o_part = torch.zeros(B * M * S * D, dtype=torch.int16, device="cuda")
        r_part = torch.zeros(B * M * S, dtype=torch.int16, device="cuda")
        out = torch.zeros(B * M * D, dtype=torch.int16, device="cuda")
        for round_ in range(2):  # two calls in a row share the static scratch
            rnd = lambda a: from_bits(to_bits(a, mg.float16), mg.float16)
            q = rnd(rng.standard_normal((B, M, D)) / np.sqrt(D))
            k = rnd(rng.standard_normal((B, D, L)))
            v = rnd(rng.standard_normal((B, L, D)))
            Q.upload_data(to_bits(q, mg.float16))
            K.upload_data(to_bits(np.ascontiguousarray(k.transpose(0, 2, 1)), mg.float16))
            V.upload_data(to_bits(v, mg.float16))
            g.run()
            want = final[0].download_data()
            out.zero_()
            torch.cuda.synchronize()
            noalloc_call(lib, desc, Q.pod.data_ptr, K.pod.data_ptr, V.pod.data_ptr, o_part.data_ptr(), r_part.data_ptr(),
                         out.data_ptr(), 0)
            got = out.cpu().numpy().view(np.uint16)
            assert_close(from_bits(got, mg.float16), from_bits(want, mg.float16), mg.float16, "float round %d" % round_)
            assert_close(from_bits(got, mg.float16).reshape(B, M, D), mo.attention_fp32(q, k, v), mg.float16, "vs fp32")
            # fingerprint mode: bit-exact with the graph path
            x = [rng.integers(0, mo.FP_PQ, size=t.shape).astype(np.uint16) for t in (Q, K, V)]
            for t, a in zip((Q, K, V), x):
                t.upload_fingerprint(a)
            g.fingerprint()
            want_fp = final[0].download_fingerprint()
            out.zero_()
            torch.cuda.synchronize()
            noalloc_call(lib, desc, Q.pod.fp_ptr, K.pod.fp_ptr, V.pod.fp_ptr, o_part.data_ptr(), r_part.data_ptr(),
                         out.data_ptr(), 1)
            got_fp = out.cpu().numpy().view(np.uint16).reshape(B, M, D)
            assert np.array_equal(got_fp, want_fp)
            assert np.array_equal(got_fp, mo.unfused_attention_fp(*x))


def test_no_alloc_entry_rejects_oversized_requests(runtime):
    lib = _abi.load()
    lib.mgd_last_error.restype = ctypes.c_char_p
    desc = mgd_attn_split(heads=8, m=4, d=128, kv_len=4096, splits=16, forloop_range=4, k_layout=mg.DmemColumnMajor,
                          v_layout=mg.DmemRowMajor, data_type=mg.float16, causal_window=0, num_sets=1024)
    desc.k_set_stride = desc.v_set_stride = 8 * 128 * 4096
    fn = lib.mgd_attn_decode_fused_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(mgd_attn_split)] + [ctypes.c_void_p] * 6 + [ctypes.c_int32, ctypes.c_int32,
                                                                                ctypes.c_void_p]
    dummy = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    st = fn(ctypes.byref(desc), dummy, dummy, dummy, dummy, dummy, dummy, 0, 0, None)
    assert st == 1 and b"4096" in lib.mgd_last_error()
