// Generic float interpreter: evaluates any threadblock program on fp16 / bf16 tensors.
//
// Semantics (the ones the reference's fingerprint interpreter and its Triton generator define,
// src/kernel/cuda/customized_kernel.cu:307-603 and src/kernel/triton_code_gen.cc:222-268): per
// for-loop iteration every operator is recomputed from freshly loaded tiles; output operators add
// their operand into an accumulator across iterations and store it, row-major, after the last one.
// The reference's own float kernel (customized_kernel.cu:39-305) is a timing stand-in that never
// writes its accumulators; this kernel computes the values.
//
// Shared-memory plan (made on the host per launch, replan() below; the reference's plan counts two
// bytes per element for every tile):
//   * a tile that only an input loader writes keeps the tensor's 16-bit elements (they are exact);
//   * every computed tile is fp32, so chained operators do not round to 16 bits between steps;
//   * a matmul whose result feeds nothing but an output operator adds straight into that operator's
//     accumulator and the result tile is not allocated;
//   * an input tile that does not move with the for-loop is loaded in the first iteration only;
//   * 16-bit input tiles of row-major tensors are fetched by the TMA engine, the moving ones into a multi-stage ring
//     along the for-loop (interp_common.cuh); other input tiles use plain loads;
//   * a matmul by a loop-invariant tile whose result is only summed over the for-loop is taken once, after the loop,
//     on the sum of its left operands (interp_common.cuh);
//   * a matmul whose B operand is such a 16-bit tile (n % 8 == 0, k % 16 == 0) runs on the tensor cores
//     (mma.sync m16n8k16, fp32 accumulate): its A operand, 16-bit or computed fp32, is staged as 16-bit rows in a
//     region behind the tiles, B tiles that only such matmuls read get 16 bytes of row padding (both for
//     conflict-free ldmatrix); other matmuls run on the CUDA cores;
//   * the kernel's copy of the operator table and the bindings sits behind all of that.
// Loads honour the tensor's DmemLayout: a column-major tensor keeps each [rows, cols] matrix with the
// row index contiguous.  Outputs are rounded to nearest on store.
#include "common.cuh"
#include "interp_common.cuh"
#include <cstdio>
#include <cstring>
#include <cstdlib>

namespace mgk {
int validate_program(mgd_program const *p, mgd_bindings const *b);

// flag bits the host packs into operator arguments after replanning
constexpr int kIn16 = 1 << 8;         // input a[16]: the tile keeps 16-bit elements
constexpr int kInPadShift = 16;       // input a[16] bits 16-23: elements of padding after every tile row

template <typename T> __device__ __forceinline__ void cvt4(uint2 w, float *f);
template <> __device__ __forceinline__ void cvt4<__half>(uint2 w, float *f) {
  float2 a = __half22float2(*reinterpret_cast<__half2 const *>(&w.x)), b = __half22float2(*reinterpret_cast<__half2 const *>(&w.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <> __device__ __forceinline__ void cvt4<__nv_bfloat16>(uint2 w, float *f) {
  float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 const *>(&w.x));
  float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 const *>(&w.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// element i of a tile that is either 16-bit (T) or fp32
template <typename T> __device__ __forceinline__ float rd(unsigned char const *tile, bool is16, int i) {
  return is16 ? to_float<T>(reinterpret_cast<T const *>(tile)[i]) : reinterpret_cast<float const *>(tile)[i];
}

// C (fp32, m x n) = or += A (m x k) B (k x n), all row-major in shared memory; either operand 16-bit or fp32.
// Fallback for the shapes the tensor-core form below does not take.  One copy of the code with the operand
// widths as run-time flags: the interpreter is bound by instruction fetch (every operator jumps to code that has
// left the instruction cache), so a small footprint is worth more than the last FMA.
template <typename T>
__device__ __noinline__ void matmul_tiles(unsigned char const *Ap, unsigned char const *Bp, float *C, int m, int n, int k,
                                          bool a16, bool b16, bool add, int tid, int nt) {
  if ((n & 3) == 0) {
    int const nq = n >> 2;
    for (int i = tid; i < m * nq; i += nt) {
      int const r = i / nq, c = (i % nq) * 4;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int kk = 0; kk < k; kk++) {
        float b[4];
        if (b16) cvt4<T>(*reinterpret_cast<uint2 const *>(Bp + (size_t)(kk * n + c) * 2), b);
        else {
          float4 v = *reinterpret_cast<float4 const *>(Bp + (size_t)(kk * n + c) * 4);
          b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w;
        }
        float const av = rd<T>(Ap, a16, r * k + kk);
#pragma unroll
        for (int y = 0; y < 4; y++) acc[y] = fmaf(av, b[y], acc[y]);
      }
      float4 *dst = reinterpret_cast<float4 *>(C + r * n + c);
      float4 v = make_float4(acc[0], acc[1], acc[2], acc[3]);
      if (add) { float4 o = *dst; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
      *dst = v;
    }
  } else {
    for (int i = tid; i < m * n; i += nt) {
      int const r = i / n, c = i % n;
      float acc = 0.f;
      for (int kk = 0; kk < k; kk++) acc = fmaf(rd<T>(Ap, a16, r * k + kk), rd<T>(Bp, b16, kk * n + c), acc);
      C[i] = add ? C[i] + acc : acc;
    }
  }
}

// ---- the same product on the tensor cores (mma.sync m16n8k16, fp32 accumulate) -----------------------------------
// Taken when B keeps the tensor's 16-bit elements, n % 8 == 0 and k % 16 == 0.  A computed (fp32) A operand is
// rounded to the tensor's 16-bit type as its fragments are built, which is what the reference's shared-memory tiles
// hold anyway; rows of A past m enter as zeros and are not stored.  A warp owns a 16 x (8 NT) patch of C: the B
// fragments come from ldmatrix (transposed; `b_pitch` elements between B rows, padded by the host when the dense
// pitch would put the eight rows of a load on the same banks).
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&h);
}
template <typename T> __device__ __forceinline__ void mma16816(float (&c)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma16816<__half>(float (&c)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A is first written by the whole block as 16-bit rows of k + 8 elements into the staging room the host planned
// (rows past m as zeros), so that its fragments come from one conflict-free ldmatrix per step: A's dense rows are a
// multiple of 128 bytes apart for the usual k and four plain loads per step would share their banks.
// `residual`: stage what the 16-bit rounding of an fp32 operand left over, A - round(A), instead of round(A); a
// product taken once after the for-loop adds that second term so that the sum it multiplies keeps fp32 precision.
template <typename T>
__device__ __noinline__ void stage_a(unsigned char const *Ap, bool a16, unsigned char *staged, int m, int k, int tid, int nt,
                                     bool residual = false) {
  int const half_k = k >> 1, rows = ((m + 15) >> 4) << 4, pitch2 = (k + 8) >> 1;
  uint32_t *dst = reinterpret_cast<uint32_t *>(staged);
  for (int i = tid; i < rows * half_k; i += nt) {
    int const r = i / half_k, c2 = i % half_k;
    uint32_t v = 0u;
    if (r < m) {
      if (a16) v = reinterpret_cast<uint32_t const *>(Ap)[(size_t)r * half_k + c2];
      else {
        float2 const x = reinterpret_cast<float2 const *>(Ap)[(size_t)r * half_k + c2];
        v = pack_pair<T>(x.x, x.y);
        if (residual) {
          T const *h = reinterpret_cast<T const *>(&v);
          v = pack_pair<T>(x.x - to_float<T>(h[0]), x.y - to_float<T>(h[1]));
        }
      }
    }
    dst[r * pitch2 + c2] = v;
  }
}

// `b_swizzled`: B sits as 64-column boxes of k rows x 128 bytes with the 128-byte swizzle, as the TMA engine wrote it
// (16-byte unit u of row r at unit u ^ (r % 8)); dense or padded rows of `b_pitch` elements otherwise.
template <typename T, int NT>
__device__ __noinline__ void matmul_mma(unsigned char const *staged, unsigned char const *Bp, float *C, int m, int n, int k,
                                        int b_pitch, bool b_swizzled, bool add, int tid, int nt) {
  int const lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
  int const g = lane >> 2, t = lane & 3, mi = lane >> 3, rr = lane & 7;
  int const m_tiles = (m + 15) >> 4, n_units = n / (8 * NT);
  int const a_pitch = k + 8;
  uint32_t const a_base = (uint32_t)__cvta_generic_to_shared(staged), b_base = (uint32_t)__cvta_generic_to_shared(Bp);
  for (int u = warp; u < m_tiles * n_units; u += nwarps) {
    int const m0 = (u / n_units) * 16, n0 = (u % n_units) * 8 * NT;
    int const r0 = m0 + g, r1 = m0 + g + 8;
    bool const v0 = r0 < m, v1 = r1 < m;
    float acc[NT][4];
#pragma unroll
    for (int x = 0; x < NT; x++)
#pragma unroll
      for (int y = 0; y < 4; y++) acc[x][y] = 0.f;
    // ldmatrix addresses of this lane. A: row (mi % 2) * 8 + rr of the m-tile, k columns (mi / 2) * 8.  B
    // (transposed load): k-row (mi % 2) * 8 + rr of the 8 columns starting at (mi / 2) * 8; with one n-tile per
    // warp only lanes 0-15 supply addresses, the two k halves of the same 8 columns.
    uint32_t aaddr = a_base + (uint32_t)(((m0 + (mi & 1) * 8 + rr) * a_pitch + (mi >> 1) * 8) * 2);
    uint32_t baddr = b_base + (uint32_t)((((mi & 1) * 8 + rr) * b_pitch + n0 + (NT >= 2 ? (mi >> 1) * 8 : 0)) * 2);
    uint32_t bstep = (uint32_t)(16 * b_pitch * 2), bnext = 32u; // next 16 k-rows; next 16 columns (second x4 load)
    if (b_swizzled) {
      int const unit = (n0 >> 3) + (NT >= 2 ? (mi >> 1) : 0); // 16-byte unit of the row; 8 per box; NT = 4: + 2 for the second load
      uint32_t const rowpart = (uint32_t)((unit >> 3) * k * 128 + ((mi & 1) * 8 + rr) * 128);
      baddr = b_base + rowpart + (uint32_t)(((unit & 7) ^ rr) << 4);
      bnext = (uint32_t)((((unit + 2) & 7) ^ rr) << 4) - (uint32_t)(((unit & 7) ^ rr) << 4); // same box: n0 % 32 == 0
      bstep = 16u * 128u;
    }
#pragma unroll 2
    for (int k0 = 0; k0 < k; k0 += 16, baddr += bstep, aaddr += 32u) {
      uint32_t a[4];
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(aaddr));
      if (NT == 1) {
        uint32_t b0, b1;
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(baddr));
        mma16816<T>(acc[0], a, b0, b1);
      } else {
#pragma unroll
        for (int h = 0; h < NT / 2; h++) {
          uint32_t bf[4];
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(bf[0]), "=r"(bf[1]), "=r"(bf[2]), "=r"(bf[3]) : "r"(baddr + (uint32_t)h * bnext));
          mma16816<T>(acc[2 * h], a, bf[0], bf[1]);
          mma16816<T>(acc[2 * h + 1], a, bf[2], bf[3]);
        }
      }
    }
    // C rows are a multiple of 128 bytes apart for the usual n, so eight lanes storing the same columns of eight
    // rows would share their banks: in store j the lanes of row g take n-tile (j + g) % NT instead (the register
    // is picked with selects: indices must be static).
#pragma unroll
    for (int j = 0; j < NT; j++) {
      int const x = (j + g) & (NT - 1);
      float lo0 = acc[0][0], lo1 = acc[0][1], hi0 = acc[0][2], hi1 = acc[0][3];
#pragma unroll
      for (int y = 1; y < NT; y++)
        if (x == y) { lo0 = acc[y][0]; lo1 = acc[y][1]; hi0 = acc[y][2]; hi1 = acc[y][3]; }
      int const c = n0 + x * 8 + 2 * t;
      if (v0) {
        float2 *dst = reinterpret_cast<float2 *>(C + (size_t)r0 * n + c);
        float2 v = make_float2(lo0, lo1);
        if (add) { float2 o = *dst; v.x += o.x; v.y += o.y; }
        *dst = v;
      }
      if (v1) {
        float2 *dst = reinterpret_cast<float2 *>(C + (size_t)r1 * n + c);
        float2 v = make_float2(hi0, hi1);
        if (add) { float2 o = *dst; v.x += o.x; v.y += o.y; }
        *dst = v;
      }
    }
  }
}

// LEAN: an instance without the code of the element-wise operators, the reductions, concat, the plain loaders and
// the CUDA-core matmul, for programs of TMA-fetched inputs, tensor-core matmuls, accumulation and outputs only.  The
// interpreter's time goes into fetching the code of one operator after another; the small instance stays in the
// instruction cache.
template <typename T, bool LEAN>
__global__ void __launch_bounds__(1024) float_interp_kernel(const __grid_constant__ mgd_program prog,
                                                           const __grid_constant__ mgd_bindings bind,
                                                           const __grid_constant__ interp::TmaPlan tma,
                                                           const __grid_constant__ interp::TmaMaps maps, int32_t *status) {
  extern __shared__ __align__(16) unsigned char smem_dyn[];
  // swizzled boxes want their 1024-byte pattern aligned: the plan's offsets are relative to an aligned base
  // (the host leaves room for that only when a tensor-map form is in use)
  unsigned char *smem_b = (tma.tiled_mask | tma.swizzled_mask)
                              ? reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023)
                              : smem_dyn;
  __shared__ uint64_t bars[interp::kMaxStages + 1]; // [0 .. stages) ring stages, [kMaxStages] tiles fetched once
  int const tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5;
  int const gx = prog.grid[0], gy = prog.grid[1], gz = prog.grid[2];
  int64_t b = blockIdx.x;
  int const bx = (int)(b % gx), by = (int)((b / gx) % gy), bz = (int)((b / ((int64_t)gx * gy)) % gz);
  int64_t const set = b / ((int64_t)gx * gy * gz);
  int const last = prog.forloop_range - 1;
  // a tile of the ring lives in stage (iteration % stages); every other tile at its planned place
  int stage_offset = 0;
  auto tile = [&](int byte_offset) {
    int const extra = (unsigned)(byte_offset - tma.ring_lo) < (unsigned)tma.ring_bytes ? stage_offset : 0;
    return smem_b + byte_offset + extra;
  };
  auto ftile = [&](int byte_offset) { return reinterpret_cast<float *>(smem_b + byte_offset); }; // fp32 tiles are never in the ring
  uint32_t const tma_mask = tma.moving_mask | tma.once_mask;
  // The operator table and the bindings are read with computed indices all the time; out of the kernel parameters
  // such a read costs tens of cycles each (about 1200 cycles of address set-up per operator were measured), out of
  // shared memory a few.  The host puts the copy behind the tiles (prog.smem_bytes = its offset).
  mgd_op const *ops = reinterpret_cast<mgd_op const *>(smem_b + prog.smem_bytes);
  mgd_bindings const &bnd = *reinterpret_cast<mgd_bindings const *>(smem_b + prog.smem_bytes + prog.num_ops * (int)sizeof(mgd_op));
  {
    int32_t *dst = reinterpret_cast<int32_t *>(smem_b + prog.smem_bytes);
    int const op_words = prog.num_ops * (int)(sizeof(mgd_op) / 4), bind_words = (int)(sizeof(mgd_bindings) / 4);
    for (int i = tid; i < op_words; i += nt) dst[i] = reinterpret_cast<int32_t const *>(prog.ops)[i];
    for (int i = tid; i < bind_words; i += nt) dst[op_words + i] = reinterpret_cast<int32_t const *>(&bind)[i];
    if (tid == 0) {
      for (int s = 0; s <= interp::kMaxStages; s++) ptx::mbar_init(ptx::smem_u32(&bars[s]), 1);
      ptx::mbar_init_fence();
    }
    __syncthreads();
  }
  // the inputs the TMA engine fetches (16-bit tiles of row-major tensors), resolved once for this block
  __shared__ interp::TileFetch fetch[MGD_MAX_IO];
  int const n_fetch = __popc(tma_mask);
  if (tid < prog.num_ops && ((tma_mask >> tid) & 1u)) {
    int32_t const *a = ops[tid].a;
    interp::resolve_fetch(fetch[__popc(tma_mask & ((1u << tid) - 1u))], a, tma, maps, tid, bnd.in[a[18]],
                          set * bnd.in_set_stride[a[18]], bx, by, bz, a[15] + ((a[16] >> kInPadShift) & 0xff), smem_b);
  }
  __syncthreads();
  auto issue = [&](uint32_t mask, int it, int stage, uint32_t bar, int tx) {
    interp::issue_fetches(fetch, n_fetch, mask == tma.moving_mask ? 1 : 0, it, stage, bar, tx, lane);
  };
  int issued = 0; // iterations whose ring tiles have been requested
#ifdef MG_FI_TIMING
  long long const pro_t0 = clock64();
  long long pro_t1 = 0, pro_t2 = 0;
#endif
  if (warp == 0) {
    if (tma.once_mask) issue(tma.once_mask, 0, 0, ptx::smem_u32(&bars[interp::kMaxStages]), tma.once_tx);
#ifdef MG_FI_TIMING
    pro_t1 = clock64();
#endif
    if (tma.stages > 0)
      for (; issued < tma.stages && issued <= last; issued++)
        issue(tma.moving_mask, issued, issued, ptx::smem_u32(&bars[issued]), tma.moving_tx);
#ifdef MG_FI_TIMING
    pro_t2 = clock64();
#endif
  }
  // Bounded waits: when one runs out the block records it, waits (bounded again) for the copies still in flight so
  // that none lands in shared memory of a later block, and returns.
  auto give_up = [&]() {
    if (tid == 0) {
      atomicExch(status, 3);
      if (tma.once_mask) ptx::mbar_wait(ptx::smem_u32(&bars[interp::kMaxStages]), 0);
      for (int s = 0; s < tma.stages && s < issued; s++) {
        int const loads = (issued - s + tma.stages - 1) / tma.stages;
        ptx::mbar_wait(ptx::smem_u32(&bars[s]), (uint32_t)((loads - 1) & 1));
      }
    }
  };
  if (tma.once_mask) {
    bool ok = ptx::mbar_wait(ptx::smem_u32(&bars[interp::kMaxStages]), 0);
    if (!__syncthreads_and(ok)) { give_up(); return; }
  }
#ifdef MG_FI_TIMING
  if (blockIdx.x == 0 && tid == 0)
    printf("prologue: issue once %lld, issue ring %lld, once wait %lld cycles\n", pro_t1 - pro_t0, pro_t2 - pro_t1, clock64() - pro_t2);
#endif

#ifdef MG_FI_TIMING // cycles per operator (with its barrier), printed by one thread of block 0
  long long op_cycles[MGD_MAX_OPS] = {};
  long long ld_setup = 0, ld_copy = 0, wait_cycles = 0, issue_cycles = 0;
  long long const kernel_t0 = clock64();
#endif
  for (int it = 0; it <= last; it++) {
#ifdef MG_FI_TIMING
    long long const wait_t0 = clock64();
#endif
    if (tma.stages > 0) {
      int const s = it % tma.stages;
      stage_offset = s * tma.ring_bytes;
      bool ok = ptx::mbar_wait(ptx::smem_u32(&bars[s]), (uint32_t)((it / tma.stages) & 1));
      if (!__syncthreads_and(ok)) { give_up(); return; }
    }
#ifdef MG_FI_TIMING
    wait_cycles += clock64() - wait_t0;
#endif
    for (int oi = 0; oi < prog.num_ops; oi++) {
      mgd_op const &op = ops[oi];
      int32_t const *a = op.a;
      if (op.type == interp::kOpInput) {
        if ((tma_mask >> oi) & 1u) continue;                              // fetched by the TMA engine
        if (it > 0 && ((tma.plain_once_mask >> oi) & 1u)) continue;       // same tile as in the first iteration
      } else if (a[interp::kPhaseSlot] != 0 && it != last) {
        continue;                                                         // runs once, after the loop
      } else if (op.type == interp::kOpAccumulate && a[4] != 0) {
        continue;                                                         // the matmul before it did the adding
      }
      bool const first = it == 0 || (op.type != interp::kOpInput && a[interp::kPhaseSlot] != 0);
#ifdef MG_FI_TIMING
      long long const op_t0 = clock64();
#endif
      switch (op.type) {
        case 2001: if constexpr (!LEAN) {
          int row = bx * a[0] + by * a[1] + bz * a[2] + it * a[6];
          int col = bx * a[3] + by * a[4] + bz * a[5] + it * a[7];
          int64_t lead = (int64_t)bx * a[8] + (int64_t)by * a[9] + (int64_t)bz * a[10] + (int64_t)it * a[11];
          T const *src = static_cast<T const *>(bnd.in[a[18]]) + set * bnd.in_set_stride[a[18]] + lead;
          bool const keep16 = (a[16] & kIn16) != 0;
          T *dst16 = reinterpret_cast<T *>(tile(a[17]));
          float *dst32 = ftile(a[17]);
          int rows = a[14], cols = a[15], n = rows * cols;
          int const pitch = cols + ((a[16] >> kInPadShift) & 0xff); // padded only for 16-bit tiles
          if ((a[16] & 0xff) == MG_DMEM_COLUMN_MAJOR) {
            int ld = a[12]; // rows of the whole matrix: consecutive rows are adjacent in memory
            for (int i = tid; i < n; i += nt) {
              int c = i / rows, r = i % rows;
              T v = src[(size_t)(col + c) * ld + row + r];
              if (keep16) dst16[r * pitch + c] = v;
              else dst32[r * cols + c] = to_float<T>(v);
            }
          } else {
            int ld = a[13];
            T const *first = src + (size_t)row * ld + col;
            if (keep16 && (cols & 7) == 0 && (ld & 7) == 0 && (reinterpret_cast<uintptr_t>(first) & 15) == 0) {
              int const cv = cols >> 3; // 16-byte pieces per tile row
#ifdef MG_FI_TIMING
              ld_setup += clock64() - op_t0;
              long long const ld_t1 = clock64();
#endif
              for (int i = tid; i < rows * cv; i += nt) {
                int r = i / cv, c = i % cv;
                *reinterpret_cast<uint4 *>(dst16 + r * pitch + c * 8) = __ldg(reinterpret_cast<uint4 const *>(first + (size_t)r * ld) + c);
              }
#ifdef MG_FI_TIMING
              ld_copy += clock64() - ld_t1;
#endif
              // the tile of the next iteration: one prefetch per 128-byte line, so that its loads find it in L1
              // instead of paying an L2 round trip between two barriers
              if (it + 1 < prog.forloop_range && !((tma.plain_once_mask >> oi) & 1u)) {
                T const *next = first + (size_t)a[6] * ld + a[7] + a[11];
                int const lines = (cols * (int)sizeof(T) + 127) >> 7;
                for (int i = tid; i < rows * lines; i += nt) {
                  int r = i / lines, l = i % lines;
                  asm volatile("prefetch.global.L1 [%0];" ::"l"(next + (size_t)r * ld + l * (128 / (int)sizeof(T))));
                }
              }
            } else {
              for (int i = tid; i < n; i += nt) {
                int r = i / cols, c = i % cols;
                T v = first[(size_t)r * ld + c];
                if (keep16) dst16[r * pitch + c] = v;
                else dst32[i] = to_float<T>(v);
              }
            }
          }
          break;
        } else break;
        case MG_TB_MATMUL_OP: {
          int m = a[0], n = a[1], k = a[2];
          unsigned char const *A = tile(a[3]), *B = tile(a[4]);
          float *C = ftile(a[5]);
          bool const add = a[8] != 0 && !first;
          if (a[10] > 0) { // host-planned staging room: B in 16 bits, n % 8 == 0, k % 16 == 0 -> tensor cores
            unsigned char *staged = smem_b + a[10];
            stage_a<T>(A, a[6] != 0, staged, m, k, tid, nt);
            __syncthreads();
            int const bp = a[9] > 0 ? a[9] : n;
            // the wide warp patch when it still gives every warp one
            bool const wide = (n & 31) == 0 && ((m + 15) >> 4) * (n >> 5) >= (nt >> 5);
            bool const swz = a[11] != 0;
            if (wide) matmul_mma<T, 4>(staged, B, C, m, n, k, bp, swz, add, tid, nt);
            else matmul_mma<T, 1>(staged, B, C, m, n, k, bp, swz, add, tid, nt);
            if (a[interp::kPhaseSlot] != 0 && a[6] == 0) { // taken once on an fp32 sum: add the rounding residual's product
              __syncthreads();
              stage_a<T>(A, false, staged, m, k, tid, nt, true);
              __syncthreads();
              if (wide) matmul_mma<T, 4>(staged, B, C, m, n, k, bp, swz, true, tid, nt);
              else matmul_mma<T, 1>(staged, B, C, m, n, k, bp, swz, true, tid, nt);
            }
          } else if constexpr (!LEAN) {
            matmul_tiles<T>(A, B, C, m, n, k, a[6] != 0, a[7] != 0, add, tid, nt);
          }
          break;
        }
        case MG_TB_EXP_OP: if constexpr (!LEAN) {
          float *x = ftile(a[0]);
          for (int i = tid; i < a[1]; i += nt) x[i] = expf(x[i]);
          break;
        } else break;
        case MG_TB_DIV_OP:
        case MG_TB_ADD_OP:
        case MG_TB_MUL_OP: if constexpr (!LEAN) {
          int const xd[3] = {a[0], a[1], a[2]}, yd[3] = {a[3], a[4], a[5]};
          int const zd[3] = {max(xd[0], yd[0]), max(xd[1], yd[1]), max(xd[2], yd[2])};
          unsigned char const *x = tile(a[6]), *y = tile(a[7]);
          bool const x16 = a[9] != 0, y16 = a[10] != 0;
          float *z = ftile(a[8]);
          int n = zd[0] * zd[1] * zd[2];
          for (int i = tid; i < n; i += nt) {
            int rest = i, xs = 1, ys = 1, xi = 0, yi = 0;
            for (int d = 2; d >= 0; d--) {
              xi += (rest % xd[d]) * xs;
              yi += (rest % yd[d]) * ys;
              xs *= xd[d];
              ys *= yd[d];
              rest /= zd[d];
            }
            float xv = rd<T>(x, x16, xi), yv = rd<T>(y, y16, yi);
            z[i] = op.type == MG_TB_DIV_OP ? xv / yv : (op.type == MG_TB_ADD_OP ? xv + yv : xv * yv);
          }
          break;
        } else break;
        case MG_TB_REDUCTION_0_OP: case MG_TB_REDUCTION_1_OP: case MG_TB_REDUCTION_2_OP:
        case MG_TB_REDUCTION_0_TO_DIMX_OP: case MG_TB_REDUCTION_1_TO_DIMX_OP: case MG_TB_REDUCTION_2_TO_DIMX_OP: if constexpr (!LEAN) {
          int n_out = a[0], degree = a[1], inner = a[2];
          unsigned char const *x = tile(a[3]);
          bool const x16 = a[5] != 0;
          float *y = ftile(a[4]);
          if (n_out < nt && degree >= 8) { // fewer sums than threads: a warp per sum, lanes stride over the terms
            for (int i = tid >> 5; i < n_out; i += nt >> 5) {
              int const base = (i / inner) * (inner * degree) + i % inner;
              float acc = 0.f;
              for (int k = tid & 31; k < degree; k += 32) acc += rd<T>(x, x16, base + k * inner);
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
              if ((tid & 31) == 0) y[i] = acc;
            }
            break;
          }
          for (int i = tid; i < n_out; i += nt) {
            int pos = (i / inner) * (inner * degree) + i % inner;
            float acc = 0.f;
            for (int k = 0; k < degree; k++, pos += inner) acc += rd<T>(x, x16, pos);
            y[i] = acc;
          }
          break;
        } else break;
        case MG_TB_CONCAT_0_OP: case MG_TB_CONCAT_1_OP: case MG_TB_CONCAT_2_OP: if constexpr (!LEAN) {
          int n_out = a[0], ad = a[1], bd = a[2], inner = a[3];
          unsigned char const *A = tile(a[4]), *B = tile(a[5]);
          bool const a16 = a[7] != 0, b16 = a[8] != 0;
          float *y = ftile(a[6]);
          for (int i = tid; i < n_out; i += nt) {
            int in_idx = i % inner, along = (i / inner) % (ad + bd), outer = (i / inner) / (ad + bd);
            y[i] = along < ad ? rd<T>(A, a16, in_idx + along * inner + outer * inner * ad)
                              : rd<T>(B, b16, in_idx + (along - ad) * inner + outer * inner * bd);
          }
          break;
        } else break;
        case interp::kOpAccumulate: { // running sum of a tile over the for-loop (the hoisted matmul's left operand)
          unsigned char const *x = tile(a[1]);
          bool const x16 = a[3] != 0;
          float *acc = ftile(a[2]);
          if (first) {
            for (int i = tid; i < a[0]; i += nt) acc[i] = rd<T>(x, x16, i);
          } else {
            for (int i = tid; i < a[0]; i += nt) acc[i] += rd<T>(x, x16, i);
          }
          break;
        }
        case 2002: {
          int n = a[11] * a[12];
          float *acc = ftile(a[14]);
          if (!a[17]) { // a[17]: the producing matmul already added into the accumulator
            unsigned char const *x = tile(a[13]);
            bool const x16 = a[16] != 0;
            if (first) {
              for (int i = tid; i < n; i += nt) acc[i] = rd<T>(x, x16, i);
            } else {
              for (int i = tid; i < n; i += nt) acc[i] += rd<T>(x, x16, i);
            }
          }
          if (it == prog.forloop_range - 1) {
            __syncthreads();
            int row = bx * a[0] + by * a[1] + bz * a[2];
            int col = bx * a[3] + by * a[4] + bz * a[5];
            int64_t lead = (int64_t)bx * a[6] + (int64_t)by * a[7] + (int64_t)bz * a[8];
            T *dst = static_cast<T *>(bnd.out[a[15]]) + set * bnd.out_set_stride[a[15]] + lead;
            int cols = a[12], ld = a[10];
            for (int i = tid; i < n; i += nt) dst[(size_t)(row + i / cols) * ld + col + i % cols] = from_float<T>(acc[i]);
          }
          break;
        }
        default: break;
      }
      __syncthreads();
#ifdef MG_FI_TIMING
      op_cycles[oi] += clock64() - op_t0;
#endif
    }
    // every thread is past its last read of this iteration's stage: request the tiles of iteration it + stages into it
#ifdef MG_FI_TIMING
    long long const issue_t0 = clock64();
#endif
    if (warp == 0 && tma.stages > 0 && issued <= last) {
      ptx::fence_proxy_async_smem();
      int const s = it % tma.stages;
      issue(tma.moving_mask, issued, s, ptx::smem_u32(&bars[s]), tma.moving_tx);
      issued++;
    }
#ifdef MG_FI_TIMING
    issue_cycles += clock64() - issue_t0;
#endif
  }
#ifdef MG_FI_TIMING
  if (blockIdx.x == 0 && tid == 0)
  {
    printf("kernel %lld cycles; ring waits %lld; issue %lld; threads %d stages %d\n", clock64() - kernel_t0, wait_cycles, issue_cycles, nt, tma.stages);
    for (int oi = 0; oi < prog.num_ops; oi++) printf("op %d type %d: %lld cycles\n", oi, ops[oi].type, op_cycles[oi]);
    printf("loaders (vector path): setup %lld copy %lld\n", ld_setup, ld_copy);
  }
#endif
}

// ---- host: shared-memory replanning ------------------------------------------------------------------------------
namespace {
struct TileUse {
  int planned;    // byte offset in the reference's two-bytes-per-element plan (identifies the tile)
  int elems;
  bool loaded;    // written by an input loader
  bool computed;  // written by any other operator
  bool dropped;   // folded into an output accumulator
  int offset;     // byte offset in this kernel's plan
  int rows, cols; // shape the loader writes (loaded tiles)
  int pad;        // extra elements per row: a 16-bit matmul B operand whose dense pitch conflicts in ldmatrix
  bool ring;      // refilled by the TMA engine every iteration: lives in the multi-stage ring
  bool swizzled;  // stored as 64-column boxes with the 128-byte swizzle (instead of padded rows)
  bool boxed;     // fetched as one dense tensor-map box
  bool is16() const { return loaded && !computed; }
  size_t bytes() const { return pad ? (size_t)rows * (cols + pad) * 2 : (size_t)elems * (is16() ? 2 : 4); }
  // a tensor-map box must land on a 128-byte boundary; the swizzle pattern repeats every 1024 bytes
  size_t alignment() const { return swizzled ? 1024 : (boxed ? 128 : 16); }
  size_t room() const { return (bytes() + alignment() - 1) & ~(alignment() - 1); }
  size_t place(size_t at) const { return (at + alignment() - 1) & ~(alignment() - 1); }
};

struct Replanned {
  mgd_program prog;
  interp::TmaPlan tma;
  interp::TmaMaps maps;
  size_t smem_bytes;
};

struct TileTable {
  TileUse t[3 * MGD_MAX_OPS];
  int n = 0;
  int find(int planned) const {
    for (int i = 0; i < n; i++)
      if (t[i].planned == planned) return i;
    return -1;
  }
  int touch(int planned, int elems) {
    int i = find(planned);
    if (i < 0) {
      i = n++;
      t[i] = TileUse{planned, elems, false, false, false, 0, 0, 0, 0, false, false, false};
    } else if (elems > t[i].elems) {
      t[i].elems = elems;
    }
    return i;
  }
};

using interp::is_binary;
using interp::is_concat;
using interp::is_reduction;
using interp::reads_of;
using interp::written_by;

void replan(mgd_program const &in, mgd_bindings const *bind, Replanned *out) {
  TileTable tt;
  out->prog = in;
  std::memset(&out->tma, 0, sizeof(out->tma));
  mgd_program &p = out->prog;
  // pass 1: every tile with its size and who writes it
  for (int i = 0; i < in.num_ops; i++) {
    mgd_op const &op = in.ops[i];
    int32_t const *a = op.a;
    if (op.type == 2001) {
      TileUse &t = tt.t[tt.touch(a[17], a[14] * a[15])];
      t.loaded = true;
      t.rows = a[14];
      t.cols = a[15];
    } else if (op.type == MG_TB_MATMUL_OP) {
      tt.touch(a[3], a[0] * a[2]);
      tt.touch(a[4], a[2] * a[1]);
      tt.t[tt.touch(a[5], a[0] * a[1])].computed = true;
    } else if (op.type == MG_TB_EXP_OP) {
      tt.t[tt.touch(a[0], a[1])].computed = true;
    } else if (is_binary(op.type)) {
      int zx = a[0] > a[3] ? a[0] : a[3], zy = a[1] > a[4] ? a[1] : a[4], zz = a[2] > a[5] ? a[2] : a[5];
      tt.touch(a[6], a[0] * a[1] * a[2]);
      tt.touch(a[7], a[3] * a[4] * a[5]);
      tt.t[tt.touch(a[8], zx * zy * zz)].computed = true;
    } else if (is_reduction(op.type)) {
      tt.touch(a[3], a[0] * a[1]);
      tt.t[tt.touch(a[4], a[0])].computed = true;
    } else if (is_concat(op.type)) {
      int along = a[1] + a[2];
      tt.touch(a[4], along > 0 ? a[0] / along * a[1] : 0);
      tt.touch(a[5], along > 0 ? a[0] / along * a[2] : 0);
      tt.t[tt.touch(a[6], a[0])].computed = true;
    } else if (op.type == interp::kOpAccumulate) {
      tt.touch(a[1], a[0]);
      tt.t[tt.touch(a[2], a[0])].computed = true;
    } else if (op.type == 2002) {
      tt.touch(a[13], a[11] * a[12]);
      tt.t[tt.touch(a[14], a[11] * a[12])].computed = true;
    }
  }
  // pass 2: a matmul whose result only an output operator reads accumulates in place of that operator
  int fused_matmul[MGD_MAX_OPS];
  for (int i = 0; i < in.num_ops; i++) fused_matmul[i] = -1;
  for (int o = 0; o < in.num_ops; o++) {
    bool const is_acc = in.ops[o].type == interp::kOpAccumulate; // the running sum of a hoisted product's operand
    if (in.ops[o].type != 2002 && !is_acc) continue;
    int src = is_acc ? in.ops[o].a[1] : in.ops[o].a[13], writer = -1, writers = 0, reads = 0;
    for (int i = 0; i < in.num_ops; i++) {
      if (written_by(in.ops[i]) == src) { writers++; writer = i; }
      reads += reads_of(in.ops[i], src);
    }
    if (writers == 1 && reads == 1 && writer < o && in.ops[writer].type == MG_TB_MATMUL_OP) {
      fused_matmul[o] = writer;
      tt.t[tt.find(src)].dropped = true;
    }
  }
  // pass 3: offsets, 16-byte aligned.  A 16-bit tile that is read only as the B operand of tensor-core matmuls of
  // its own shape gets 8 elements of row padding when its dense pitch is a multiple of 128 bytes (the eight rows
  // of an ldmatrix would share their banks); without it if the padded plan does not fit.
  for (int i = 0; i < tt.n; i++) {
    TileUse &t = tt.t[i];
    if (!t.is16() || t.rows <= 0 || (t.cols * 2) % 128 != 0) continue;
    bool only_b = true, used = false;
    for (int o = 0; o < in.num_ops; o++) {
      mgd_op const &op = in.ops[o];
      int const reads = reads_of(op, t.planned);
      if (reads == 0) continue;
      if (op.type == MG_TB_MATMUL_OP && op.a[4] == t.planned && op.a[3] != t.planned && op.a[2] == t.rows &&
          op.a[1] == t.cols && (op.a[2] & 15) == 0)
        used = true;
      else
        only_b = false;
    }
    t.pad = (used && only_b) ? 8 : 0;
  }
  // staging room for the A operand of the tensor-core matmuls (16-bit rows of k + 8 elements, m rounded up to 16),
  // one region shared by all of them
  size_t staging = 0;
  for (int i = 0; i < in.num_ops; i++) {
    int32_t const *a = in.ops[i].a;
    if (in.ops[i].type != MG_TB_MATMUL_OP || !tt.t[tt.find(a[4])].is16() || (a[1] & 7) != 0 || (a[2] & 15) != 0) continue;
    size_t const need = (size_t)((a[0] + 15) / 16 * 16) * (a[2] + 8) * 2;
    if (need > staging) staging = need;
  }
  size_t const table = (size_t)in.num_ops * sizeof(mgd_op) + sizeof(mgd_bindings) + 32;
  size_t at = 0;
  int staging_offset = 0;
  interp::TmaPlan &tma = out->tma;
  for (int pass = 0; pass < 2; pass++) {
    // Which inputs the TMA engine fetches (needs the row pitches of this pass): 16-bit tiles of row-major tensors
    // whose rows are 16-byte aligned; the ones that move with the for-loop go through the ring.
    std::memset(&tma, 0, sizeof(tma));
    std::memset(&out->maps, 0, sizeof(out->maps));
    for (int i = 0; i < tt.n; i++) {
      tt.t[i].ring = false;
      tt.t[i].swizzled = tt.t[i].boxed = false; // a second pass starts over
    }
    for (int i = 0; i < in.num_ops; i++) {
      mgd_op const &op = in.ops[i];
      if (op.type != 2001) continue;
      TileUse &t = tt.t[tt.find(op.a[17])];
      int writers = 0;
      for (int j = 0; j < in.num_ops; j++) writers += written_by(in.ops[j]) == t.planned;
      bool const invariant = t.is16() && !interp::input_moves(op) && writers == 1;
      int const slot = op.a[18];
      bool const eligible = bind != nullptr && t.is16() && writers == 1 && t.elems == t.rows * t.cols &&
                            interp::tma_eligible(op, bind->in[slot], bind->in_set_stride[slot], bind->num_sets, t.cols + t.pad, true);
      if (eligible) {
        int form = interp::tiled_form(op, bind->in_set_stride[slot], bind->num_sets, t.pad > 0);
        if (form && !interp::make_tile_map(&out->maps.m[slot], bind->in[slot], (uint64_t)op.a[13], (uint64_t)op.a[12],
                                           interp::matrices_addressed(in, op, bind->in_set_stride[slot], bind->num_sets),
                                           form == 2 ? 64u : (uint32_t)t.cols, (uint32_t)t.rows, form == 2))
          form = 0;
        if (form == 2) {
          tma.swizzled_mask |= 1u << i;
          t.swizzled = true;
          t.pad = 0;
        } else if (form == 1) {
          tma.tiled_mask |= 1u << i;
          t.boxed = true;
        }
      }
      if (eligible && (invariant || in.forloop_range == 1)) {
        tma.once_mask |= 1u << i;
        tma.once_tx += t.rows * t.cols * 2;
      } else if (eligible) {
        tma.moving_mask |= 1u << i;
        tma.moving_tx += t.rows * t.cols * 2;
        t.ring = true;
      } else if (invariant) {
        tma.plain_once_mask |= 1u << i;
      }
    }
    size_t ring_bytes = 0, rest_bytes = 0;
    for (int i = 0; i < tt.n; i++) {
      if (tt.t[i].dropped) continue;
      if (tt.t[i].ring) ring_bytes = tt.t[i].place(ring_bytes) + tt.t[i].room();
      else rest_bytes += tt.t[i].room() + (tt.t[i].alignment() > 16 ? tt.t[i].alignment() : 0);
    }
    ring_bytes = (ring_bytes + 1023) & ~(size_t)1023;
    int stages = 0;
    if (ring_bytes > 0) {
      stages = in.forloop_range < 3 ? in.forloop_range : 3;
      while (stages > 1 && ring_bytes * stages + rest_bytes + staging + table + 1024 > (size_t)interp::kDynSmemLimit) stages--;
    }
    tma.stages = stages;
    tma.ring_lo = 0;
    tma.ring_bytes = (int32_t)ring_bytes;
    at = 0;
    for (int i = 0; i < tt.n; i++) { // the ring first
      if (tt.t[i].dropped || !tt.t[i].ring) continue;
      at = tt.t[i].place(at);
      tt.t[i].offset = (int)at;
      at += tt.t[i].room();
    }
    at = ring_bytes * (size_t)stages;
    for (int i = 0; i < tt.n; i++) {
      if (tt.t[i].dropped || tt.t[i].ring) continue;
      at = tt.t[i].place(at);
      tt.t[i].offset = (int)at;
      at += tt.t[i].room();
    }
    if (staging > 0 && at + staging + table + 1024 <= (size_t)interp::kDynSmemLimit) {
      staging_offset = (int)at;
      at += staging;
      break;
    }
    if (staging == 0) break;
    // no room for the staging area: those matmuls run on the CUDA cores, which read B densely
    for (int i = 0; i < tt.n; i++) tt.t[i].pad = 0;
  }
  // behind the tiles: the kernel's copy of the operator table and the bindings
  at = (at + 15) & ~(size_t)15;
  p.smem_bytes = (int32_t)at;
  at += (size_t)in.num_ops * sizeof(mgd_op) + sizeof(mgd_bindings);
  out->smem_bytes = at + 16 + ((out->tma.tiled_mask | out->tma.swizzled_mask) ? 1024 : 0); // + room to align the base
  // pass 4: rewrite operands
  auto off = [&](int planned) { return tt.t[tt.find(planned)].offset; };
  auto is16 = [&](int planned) { return tt.t[tt.find(planned)].is16() ? 1 : 0; };
  for (int i = 0; i < in.num_ops; i++) {
    int32_t const *a = in.ops[i].a;
    int32_t *w = p.ops[i].a;
    int type = in.ops[i].type;
    if (type == 2001) {
      w[17] = off(a[17]);
      w[16] = (a[16] & 0xff) | (is16(a[17]) ? kIn16 : 0) | (tt.t[tt.find(a[17])].pad << kInPadShift);
    } else if (type == MG_TB_MATMUL_OP) {
      w[3] = off(a[3]); w[4] = off(a[4]);
      w[6] = is16(a[3]); w[7] = is16(a[4]);
      w[8] = 0;
      w[9] = tt.t[tt.find(a[4])].pad ? a[1] + tt.t[tt.find(a[4])].pad : 0; // row pitch of B when it is padded
      w[10] = (is16(a[4]) && (a[1] & 7) == 0 && (a[2] & 15) == 0) ? staging_offset : 0;
      w[11] = tt.t[tt.find(a[4])].swizzled ? 1 : 0;
      w[5] = tt.t[tt.find(a[5])].dropped ? -1 : off(a[5]);
    } else if (type == MG_TB_EXP_OP) {
      w[0] = off(a[0]);
    } else if (is_binary(type)) {
      w[6] = off(a[6]); w[7] = off(a[7]); w[8] = off(a[8]);
      w[9] = is16(a[6]); w[10] = is16(a[7]);
    } else if (is_reduction(type)) {
      w[3] = off(a[3]); w[4] = off(a[4]);
      w[5] = is16(a[3]);
    } else if (is_concat(type)) {
      w[4] = off(a[4]); w[5] = off(a[5]); w[6] = off(a[6]);
      w[7] = is16(a[4]); w[8] = is16(a[5]);
    } else if (type == interp::kOpAccumulate) {
      w[2] = off(a[2]);
      w[4] = fused_matmul[i] >= 0 ? 1 : 0; // the producing matmul adds into the running sum itself
      w[1] = w[4] ? 0 : off(a[1]);
      w[3] = w[4] ? 0 : is16(a[1]);
      if (w[4]) {
        p.ops[fused_matmul[i]].a[5] = w[2];
        p.ops[fused_matmul[i]].a[8] = 1;
      }
    } else if (type == 2002) {
      w[14] = off(a[14]);
      w[17] = fused_matmul[i] >= 0 ? 1 : 0;
      w[13] = w[17] ? 0 : off(a[13]);
      w[16] = w[17] ? 0 : is16(a[13]);
      if (w[17]) {
        p.ops[fused_matmul[i]].a[5] = w[14];
        p.ops[fused_matmul[i]].a[8] = 1;
      }
    }
  }
}
} // namespace
} // namespace mgk

using namespace mgk;

extern "C" int mgd_float_interp_smem(const mgd_program *prog, size_t *bytes, int32_t *fits) {
  if (!prog || !bytes || !fits) return set_error(MG_ERR_INVALID_ARGUMENT, "null pointer");
  if (prog->num_ops <= 0 || prog->num_ops > MGD_MAX_OPS) return set_error(MG_ERR_INVALID_ARGUMENT, "operator count out of range");
  Replanned r;
  mgd_program rewritten = *prog;
  interp::hoist_invariant_products(rewritten);
  replan(rewritten, nullptr, &r);
  if (r.smem_bytes > (size_t)interp::kDynSmemLimit) replan(*prog, nullptr, &r);
  *bytes = r.smem_bytes;
  *fits = *bytes <= (size_t)interp::kDynSmemLimit;
  return MG_OK;
}

extern "C" int mgd_launch_float_interp(const mgd_program *prog, const mgd_bindings *bind, int32_t dt, void *stream) {
  int st = validate_program(prog, bind);
  if (st != MG_OK) return st;
  // Rewrite (hoisted products), then plan with the TMA ring; step back to the plain program and plain loads when
  // that does not fit.
  Replanned r;
  mgd_program rewritten = *prog;
  interp::hoist_invariant_products(rewritten);
  replan(rewritten, bind, &r);
  if (r.smem_bytes > (size_t)interp::kDynSmemLimit) replan(rewritten, nullptr, &r);
  if (r.smem_bytes > (size_t)interp::kDynSmemLimit) replan(*prog, nullptr, &r);
  size_t smem = r.smem_bytes;
  int32_t *status = device_error_word();
  if (!status) return set_error(MG_ERR_CUDA, "cannot allocate the device status word");
  if (smem > (size_t)interp::kDynSmemLimit)
    return set_error(MG_ERR_UNSUPPORTED,
                     "the generic float interpreter keeps computed tiles in fp32 and this graph needs more than 227 KB "
                     "that way; only graphs matched by a specialised kernel can run at this size");
  int64_t blocks = (int64_t)prog->grid[0] * prog->grid[1] * prog->grid[2] * bind->num_sets;
  if (blocks > 0x7fffffffLL) return set_error(MG_ERR_UNSUPPORTED, "too many blocks for one launch");
  // Blocks run one operator at a time with a barrier after each: big tiles get more warps to hide the latency of
  // the dependent instruction chains (the largest operator decides).  More warps also repeat every operator's
  // set-up code more often (32 warps share four schedulers), so loaders and tensor-core matmuls, which need few
  // warps, ask for less: the matmul chain of 16 x 64 x 1024 tiles ran 129 us on 512 threads, 144 on 1024, 148 on 256.
  int64_t largest = 0;
  for (int i = 0; i < r.prog.num_ops; i++) {
    int32_t const *a = r.prog.ops[i].a;
    // what runs once after the loop does not size the block when the loop is long: its few big operators finish
    // on fewer warps, every iteration's barriers are cheaper for it
    if (r.prog.ops[i].type != 2001 && a[interp::kPhaseSlot] != 0 && r.prog.forloop_range >= 4) continue;
    int64_t work = 0;
    switch (r.prog.ops[i].type) {
      case 2001: // plain loads; nothing for the threads to do when the TMA engine fetches the tile
        work = ((r.tma.moving_mask | r.tma.once_mask) >> i) & 1u ? 0 : (int64_t)a[14] * a[15] / 16;
        break;
      case interp::kOpAccumulate: work = a[0]; break;
      case 2002: work = (int64_t)a[11] * a[12] / ((a[17] || a[interp::kPhaseSlot]) ? 4 : 1); break; // stores once, at the end
      case MG_TB_MATMUL_OP:
        work = r.prog.ops[i].a[10] > 0 ? (int64_t)((a[0] + 15) / 16) * a[1] * 4 : (int64_t)a[0] * a[1] / 4;
        break;
      case MG_TB_EXP_OP: work = a[1]; break;
      default: work = a[0]; break;
    }
    if (work > largest) largest = work;
  }
  unsigned threads = largest >= 8192 ? 1024u : (largest >= 2048 ? 512u : (largest >= 512 ? 256u : 128u));
  if (int const v = option(MGD_OPT_INTERP_THREADS)) // 128 ... 1024: for measurements
    if (v == 128 || v == 256 || v == 512 || v == 1024) threads = (unsigned)v;
  // the lean instance: every input fetched by the TMA engine, every matmul on the tensor cores, nothing else but
  // accumulation and outputs
  bool lean = true;
  for (int i = 0; i < r.prog.num_ops && lean; i++) {
    mgd_op const &op = r.prog.ops[i];
    if (op.type == 2001) lean = ((r.tma.moving_mask | r.tma.once_mask) >> i) & 1u;
    else if (op.type == MG_TB_MATMUL_OP) lean = op.a[10] > 0;
    else lean = op.type == interp::kOpAccumulate || op.type == 2002;
  }
  if (lean) {
    static bool lean_h = false, lean_b = false;
    if (dt == MG_DT_FLOAT16) {
      if (smem > 48 * 1024 && !lean_h) {
        if (cudaFuncSetAttribute(float_interp_kernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, interp::kDynSmemLimit) != cudaSuccess)
          return check_launch("cudaFuncSetAttribute(float_interp_kernel)");
        lean_h = true;
      }
      float_interp_kernel<__half, true><<<(unsigned)blocks, threads, smem, (cudaStream_t)stream>>>(r.prog, *bind, r.tma, r.maps, status);
      return check_launch("float_interp_kernel");
    }
    if (dt == MG_DT_BFLOAT16) {
      if (smem > 48 * 1024 && !lean_b) {
        if (cudaFuncSetAttribute(float_interp_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, interp::kDynSmemLimit) != cudaSuccess)
          return check_launch("cudaFuncSetAttribute(float_interp_kernel)");
        lean_b = true;
      }
      float_interp_kernel<__nv_bfloat16, true><<<(unsigned)blocks, threads, smem, (cudaStream_t)stream>>>(r.prog, *bind, r.tma, r.maps, status);
      return check_launch("float_interp_kernel");
    }
  }
  static bool configured_h = false, configured_b = false;
  if (dt == MG_DT_FLOAT16) {
    if (smem > 48 * 1024 && !configured_h) {
      if (cudaFuncSetAttribute(float_interp_kernel<__half, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, interp::kDynSmemLimit) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(float_interp_kernel)");
      configured_h = true;
    }
    float_interp_kernel<__half, false><<<(unsigned)blocks, threads, smem, (cudaStream_t)stream>>>(r.prog, *bind, r.tma, r.maps, status);
  } else if (dt == MG_DT_BFLOAT16) {
    if (smem > 48 * 1024 && !configured_b) {
      if (cudaFuncSetAttribute(float_interp_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, interp::kDynSmemLimit) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(float_interp_kernel)");
      configured_b = true;
    }
    float_interp_kernel<__nv_bfloat16, false><<<(unsigned)blocks, threads, smem, (cudaStream_t)stream>>>(r.prog, *bind, r.tma, r.maps, status);
  } else {
    return set_error(MG_ERR_UNSUPPORTED, "float mode runs on fp16 or bf16 tensors");
  }
  return check_launch("float_interp_kernel");
}
