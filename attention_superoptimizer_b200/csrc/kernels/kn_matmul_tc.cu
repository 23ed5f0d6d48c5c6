// Kernel-level matmul (the reference's KNMatmulOp::run, src/kernel/cuda/matmul_kernel.cu:30-112, which calls
// cublasGemmStridedBatchedEx there) on the 5th-generation tensor cores, for un-fused graphs in float mode:
//     C[b] (m x n, row-major) = A[b] (m x k) B[b] (k x n),  fp16 or bf16 operands, fp32 accumulation in tensor memory.
// One block per 128 x 128 output tile and batch entry.  The contraction runs in steps of 64 through a four-stage
// TMA ring (128-byte swizzle); operands are used as they lie in memory - an operand whose output index is the
// contiguous one (column-major A, row-major B) is described as MN-major instead of being transposed.  Rows, columns
// and contraction steps past the tensors' extents are zeros of the TMA fill and are never stored.
//   warp 0, one lane   TMA producer
//   warp 1             allocates / frees tensor memory; one lane issues the MMAs (4 per stage, M = N = 128, K = 16)
//   warps 2-5          epilogue: one thread per output row, tcgen05.ld 32 columns at a time, pack to 16 bits, store
// Every wait is bounded; a role that gives up raises a block-wide flag, the block frees its tensor memory, records
// the failure in the device status word and returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace mgk {
namespace kmm {
using namespace t5;

constexpr int kBM = 128, kBN = 128, kBK = 64;
constexpr int kStages = 4;
constexpr int kOperand = 128 * kBK * 2; // one operand tile of a stage: 16 KB
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 128;

struct Params {
  void *c;
  int32_t *status;
  int m, n, k, batches;
};

struct Shared {
  uint64_t full[kStages], empty[kStages], acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

// A_MN: A lies in memory as [k][m] (column-major).  B_MN: B lies in memory as [k][n] (row-major).
template <bool BF16, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads)
kn_matmul_tc_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                    const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  uint32_t const ring = smem_u32(smem); // [stage][A 16 KB | B 16 KB]
  Shared *sh = reinterpret_cast<Shared *>(smem + kStages * 2 * kOperand);
  volatile int *abort_flag = &sh->abort_flag;
  int const tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int const n0 = blockIdx.x * kBN, m0 = blockIdx.y * kBM, batch = blockIdx.z;
  int const steps = (p.k + kBK - 1) / kBK;

  if (tid == 0) {
    sh->abort_flag = 0;
    asm volatile("prefetch.tensormap [%0];" ::"l"(&a_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&b_map) : "memory");
    for (int s = 0; s < kStages; s++) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    mbar_init(smem_u32(&sh->acc_full), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) tmem_alloc(smem_u32(&sh->tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t const tmem = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    bool ok = true;
    for (int i = 0; i < steps && ok; i++) {
      int const s = i % kStages, k0 = i * kBK;
      if (i >= kStages) ok = mbar_wait(smem_u32(&sh->empty[s]), (uint32_t)((i / kStages - 1) & 1), abort_flag);
      if (!ok) break;
      if (lane == 0) {
        uint32_t const full = smem_u32(&sh->full[s]), adst = ring + (uint32_t)(s * 2 * kOperand), bdst = adst + kOperand;
        mbar_expect_tx(full, 2 * kOperand);
        if (A_MN) { // rows = contraction steps, two boxes of 64 output rows
          tma_load_3d(adst, &a_map, full, m0, k0, batch);
          tma_load_3d(adst + kOperand / 2, &a_map, full, m0 + 64, k0, batch);
        } else {    // rows = output rows, one box of 64 contraction steps
          tma_load_3d(adst, &a_map, full, k0, m0, batch);
        }
        if (B_MN) {
          tma_load_3d(bdst, &b_map, full, n0, k0, batch);
          tma_load_3d(bdst + kOperand / 2, &b_map, full, n0 + 64, k0, batch);
        } else {
          tma_load_3d(bdst, &b_map, full, k0, n0, batch);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    uint32_t const idesc = instr_desc_f16(BF16 ? 1u : 0u, A_MN, B_MN, kBM, kBN);
    uint64_t const a_desc0 = A_MN ? smem_desc(ring, kOperand / 2, 1024, 2) : smem_desc(ring, 16, 1024, 2);
    uint64_t const b_desc0 = B_MN ? smem_desc(ring + kOperand, kOperand / 2, 1024, 2) : smem_desc(ring + kOperand, 16, 1024, 2);
    bool ok = true;
    for (int i = 0; i < steps && ok; i++) {
      int const s = i % kStages;
      ok = mbar_wait(smem_u32(&sh->full[s]), (uint32_t)((i / kStages) & 1), abort_flag);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        uint64_t const ad = a_desc0 + (uint64_t)((s * 2 * kOperand) >> 4), bd = b_desc0 + (uint64_t)((s * 2 * kOperand) >> 4);
#pragma unroll
        for (int ks = 0; ks < kBK / 16; ks++) {
          // one K step: 16 elements along a swizzled 128-byte row (K-major) or 16 rows of 128 bytes (MN-major)
          uint64_t const a = ad + (uint64_t)((A_MN ? ks * 16 * 128 : ks * 32) >> 4);
          uint64_t const b = bd + (uint64_t)((B_MN ? ks * 16 * 128 : ks * 32) >> 4);
          umma_f16(tmem, a, b, idesc, (i > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&sh->empty[s]));
        if (i == steps - 1) umma_commit(smem_u32(&sh->acc_full));
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    int const quarter = warp & 3; // the tensor-memory lanes this warp may touch: 32 * (warp % 4)
    int const row = m0 + quarter * 32 + lane;
    uint32_t const lane_base = (uint32_t)(quarter * 32) << 16;
    bool ok = mbar_wait(smem_u32(&sh->acc_full), 0u, abort_flag);
    if (ok) {
      tc_fence_after();
      uint16_t *c_row = static_cast<uint16_t *>(p.c) + ((size_t)batch * p.m + (size_t)(row < p.m ? row : 0)) * p.n;
      bool const vec = (p.n & 7) == 0 && (reinterpret_cast<uintptr_t>(p.c) & 15) == 0;
#pragma unroll 1
      for (int chunk = 0; chunk < kBN / 32; chunk++) {
        uint32_t v[32];
        tmem_ld32(tmem + lane_base + (uint32_t)(chunk * 32), v); // (every lane of the warp takes part)
        int const c0 = n0 + chunk * 32;
        if (row >= p.m || c0 >= p.n) continue;
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; j++) packed[j] = pack2<BF16>(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
        if (vec && c0 + 32 <= p.n) {
#pragma unroll
          for (int j = 0; j < 4; j++)
            *reinterpret_cast<uint4 *>(c_row + c0 + 8 * j) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (c0 + j < p.n) c_row[c0 + j] = (uint16_t)((j & 1) ? packed[j >> 1] >> 16 : packed[j >> 1] & 0xFFFFu);
        }
      }
    }
  }

  // ---- teardown: every role arrives here, failed or not --------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && tid == 0) {
    // copies this block issued may still be in flight: give them a bounded time to land before the block exits
    for (int s = 0; s < kStages; s++)
      for (int i = 0; i < 20000 && !mbar_try_wait(smem_u32(&sh->full[s]), 0) && !mbar_try_wait(smem_u32(&sh->full[s]), 1); i++) {
      }
    atomicExch(p.status, 4);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// [batch][rows][cols] 16-bit array, box [1][box_rows][64], 128-byte swizzle, zero fill outside the array
static bool make_map(CUtensorMap *map, void const *base, uint64_t batch, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  TensorMapEncodeFn fn = tensor_map_encoder();
  if (!fn) return false;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {cols * 2, rows * cols * 2};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Shapes the tensor-core kernel takes: 16-byte aligned operands whose rows in memory are multiples of 16 bytes (a
// tensor map needs both), and enough work to fill a 128-row MMA at all.
bool supported(void const *a, void const *b, int batches, int m, int n, int k, int a_col_major, int b_col_major) {
  if (batches <= 0 || batches > 65535 || m <= 0 || n <= 0 || k <= 0) return false;
  if (m < 32 || k < 16) return false;
  int const a_inner = a_col_major ? m : k, b_inner = b_col_major ? k : n;
  if ((a_inner & 7) || (b_inner & 7)) return false;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return false;
  if ((((int64_t)m * k) & 7) || (((int64_t)k * n) & 7)) return false; // batch entries stay 16-byte aligned
  if ((m + kBM - 1) / kBM > 65535) return false;
  return tensor_map_encoder() != nullptr;
}

int launch(void const *a, void const *b, void *c, int batches, int m, int n, int k, int dtype, int a_col_major,
           int b_col_major, void *stream) {
  CUtensorMap am, bm;
  bool ok = a_col_major ? make_map(&am, a, batches, k, m, kBK) : make_map(&am, a, batches, m, k, kBM);
  ok = ok && (b_col_major ? make_map(&bm, b, batches, n, k, kBN) : make_map(&bm, b, batches, k, n, kBK));
  if (!ok) return set_error(MG_ERR_CUDA, "kn matmul: cuTensorMapEncodeTiled failed");
  Params p;
  p.c = c;
  p.status = device_error_word();
  if (!p.status) return set_error(MG_ERR_CUDA, "cannot allocate the device status word");
  p.m = m; p.n = n; p.k = k; p.batches = batches;
  size_t const smem = 1024 + (size_t)kStages * 2 * kOperand + sizeof(Shared) + 64;
  using Kernel = void (*)(CUtensorMap, CUtensorMap, Params);
  static Kernel const kernels[8] = {
      kn_matmul_tc_kernel<false, false, false>, kn_matmul_tc_kernel<false, false, true>,
      kn_matmul_tc_kernel<false, true, false>,  kn_matmul_tc_kernel<false, true, true>,
      kn_matmul_tc_kernel<true, false, false>,  kn_matmul_tc_kernel<true, false, true>,
      kn_matmul_tc_kernel<true, true, false>,   kn_matmul_tc_kernel<true, true, true>};
  constexpr int kMaxDevices = 64;
  static bool configured[kMaxDevices][8] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  int const which = (dtype == MG_DT_BFLOAT16 ? 4 : 0) | (a_col_major ? 2 : 0) | (b_col_major ? 0 : 1);
  if (!configured[dev][which]) {
    if (cudaFuncSetAttribute(kernels[which], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return check_launch("cudaFuncSetAttribute(kn_matmul_tc_kernel)");
    configured[dev][which] = true;
  }
  dim3 const grid((unsigned)((n + kBN - 1) / kBN), (unsigned)((m + kBM - 1) / kBM), (unsigned)batches);
  kernels[which]<<<grid, kThreads, smem, (cudaStream_t)stream>>>(am, bm, p);
  return check_launch("kn_matmul_tc_kernel");
}

} // namespace kmm
} // namespace mgk
