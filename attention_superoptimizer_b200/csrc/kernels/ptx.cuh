// Inline-PTX primitives every sm_100a kernel of this library shares: shared-memory addresses, mbarriers with
// bounded waits, TMA tile loads, proxy fences and the programmatic-dependent-launch controls.  One definition, one
// poll limit: a wait that runs out never hangs the GPU - it reports failure to its caller, which records a code in
// the device status word and winds the block down.
#pragma once
#include <cstdint>
#include <cuda.h>

namespace mgk {
namespace ptx {

// Polls of one mbarrier before a wait gives up.  At roughly 20-40 ns per poll this is tens of milliseconds: far
// above any legitimate wait of these kernels, far below a watchdog.
constexpr int kWaitLimit = 2000000;

__device__ __forceinline__ uint32_t smem_u32(void const *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// makes freshly initialised barriers visible to the async proxy (TMA, tcgen05.commit)
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Non-blocking test of a phase.  `try_wait` may park the thread for a while when the phase is not complete, and a
// parked thread wakes hundreds of cycles after the phase completes; a thread on a kernel's critical path polls with
// this instead.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Three phases tested at once: bit n of the result says that phase n is complete.  The tests overlap, so the thread
// pays one round trip to shared memory instead of three.
__device__ __forceinline__ uint32_t mbar_test_wait3(uint32_t bar0, uint32_t parity0, uint32_t bar1, uint32_t parity1,
                                                    uint32_t bar2, uint32_t parity2) {
  uint32_t a, b, c;
  asm volatile("{\n\t.reg .pred p, q, r;\n\t"
               "mbarrier.test_wait.parity.shared::cta.b64 p, [%3], %4;\n\t"
               "mbarrier.test_wait.parity.shared::cta.b64 q, [%5], %6;\n\t"
               "mbarrier.test_wait.parity.shared::cta.b64 r, [%7], %8;\n\t"
               "selp.u32 %0, 1, 0, p;\n\tselp.u32 %1, 2, 0, q;\n\tselp.u32 %2, 4, 0, r;\n\t}"
               : "=r"(a), "=r"(b), "=r"(c)
               : "r"(bar0), "r"(parity0), "r"(bar1), "r"(parity1), "r"(bar2), "r"(parity2) : "memory");
  return a | b | c;
}
// Bounded wait: false after `limit` polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int limit = kWaitLimit) {
  for (int i = 0; i < limit; i++)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// Bounded wait of a kernel whose roles wait on one another: gives up at once when another role has raised the
// abort flag, raises it when the limit is hit.
__device__ __forceinline__ bool mbar_wait_or_abort(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                                   int limit = kWaitLimit) {
  for (int i = 0; i < limit; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// The same as a spin on `mbar_test_wait` (for one thread that must see the phase as soon as it completes).
__device__ __forceinline__ bool mbar_spin_or_abort(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                                   int limit = 16 * kWaitLimit) {
  for (int i = 0; i < limit; i++) {
    if (mbar_test_wait(bar, parity)) return true;
    if ((i & 4095) == 4095 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// TMA tile loads (no multicast anywhere in this library).  The innermost coordinate times the element size must be
// a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, CUtensorMap const *map, uint32_t bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, CUtensorMap const *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// TMA tile store from shared memory (same alignment rule; never at a negative coordinate), and the wait that lets the
// issuing thread reuse or give up the shared-memory source.
__device__ __forceinline__ void tma_store_3d(CUtensorMap const *map, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_commit_and_wait_read() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void prefetch_tensormap(CUtensorMap const *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// writes of the generic proxy (st.shared) become visible to the async proxy (TMA, tcgen05 operand reads)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Programmatic dependent launch: wait for the previous kernel of the stream (a no-op for a plain launch), and let
// the next kernel's blocks be scheduled.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

} // namespace ptx

// cuTensorMapEncodeTiled, looked up once through the runtime's driver entry point (the library does not link the
// driver); null where no driver is present.  Defined in runtime.cu.
using TensorMapEncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, cuuint64_t const *,
                                       cuuint64_t const *, cuuint32_t const *, cuuint32_t const *, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TensorMapEncodeFn tensor_map_encoder();
} // namespace mgk
