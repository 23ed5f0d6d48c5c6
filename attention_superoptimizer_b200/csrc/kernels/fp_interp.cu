// Generic fingerprint interpreter: evaluates any threadblock program in the finite ring Z_PQ on
// uint16 fingerprints.  One CUDA block per (grid block, tensor set); for every for-loop iteration
// all operators are executed in order on shared-memory tiles, output operators accumulate across
// iterations and store after the last one.
//
// Results are bit-identical to the reference interpreter compute_customizedop_fingerprint
// (src/kernel/cuda/customized_kernel.cu:307-603) and its fingerprinter classes
// (include/mirage/threadblock/cuda/*.h); the arithmetic is organised differently:
//   * matmul runs on the integer tensor cores where the shape allows (matmul_fp_tensor), else keeps an exact
//     64-bit sum of products; either way one reduction modulo PQ per output instead of one after every
//     multiply-add (same residue, valid for any uint16 operands);
//   * input tiles are fetched by the TMA engine into a multi-stage ring along the for-loop (interp_common.cuh);
//     tiles whose rows are not 16-byte aligned fall back to plain (128-bit where possible) loads;
//   * a matmul by a loop-invariant tile whose result is only summed over the for-loop is taken once, after the loop,
//     on the sum of its left operands (interp_common.cuh: same residues);
//   * lookup tables live in constant memory;
//   * shared-memory tiles keep the planned offsets, so the aliasing of the in-place exp is the same.
#include "common.cuh"
#include <cstdio>
#include "interp_common.cuh"
#include <cstdlib>
#include <cstring>

namespace mgk {

// `pitch` = elements between tile rows in shared memory (cols, or cols + 8 for a padded matmul operand)
__device__ __forceinline__ void load_tile_u16(uint16_t *dst, uint16_t const *src, int rows, int cols, int pitch, int ld,
                                              int row0, int col0, int tid, int nthreads) {
  bool vec = (cols % 8 == 0) && (ld % 8 == 0) && (col0 % 8 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
             ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
  if (vec) {
    int cv = cols / 8, n = rows * cv;
    for (int i = tid; i < n; i += nthreads) {
      int r = i / cv, c = (i % cv) * 8;
      uint4 v = __ldg(reinterpret_cast<uint4 const *>(src + (size_t)(row0 + r) * ld + col0 + c));
      *reinterpret_cast<uint4 *>(dst + r * pitch + c) = v;
    }
  } else {
    int n = rows * cols;
    for (int i = tid; i < n; i += nthreads) {
      int r = i / cols, c = i % cols;
      dst[r * pitch + c] = __ldg(src + (size_t)(row0 + r) * ld + col0 + c);
    }
  }
}

// C = A B mod PQ on the integer tensor cores, exact.  A uint16 is lo + 256 hi, so a row-major uint16 tile already is
// a byte matrix with the two planes interleaved along k.  One m16n8k32 u8 MMA covers 16 uint16 k-steps; its 16 rows
// carry three byte-masked copies of 4 rows of A - [lo,0], [0,hi] and [hi,lo] - which give, against B's interleaved
// bytes, the plane products LL, HH and LH+HL in int32 (no overflow while 2 * 255^2 * k < 2^31), and
//     A B = LL + 256 (LH + HL) + 65536 HH        reduced modulo PQ once per output.
// Same residue as the reference's multiply-add loop (TBMatmulFingerprinter, threadblock/cuda/matmul.h:773-804).
// Needs k % 16 == 0 and n % 16 == 0 (ldmatrix rows of 16 bytes); a warp owns 4 rows x 16 columns of C at a time.
// `b_swizzled`: B sits as 64-column boxes of k rows x 128 bytes with the 128-byte swizzle, as the TMA engine wrote it.
// CP = column pairs (16 columns each) a warp works on side by side: the A fragments of a k-step are loaded once for all
// of them.  KC = accumulate chains along k (k-step i goes to chain i % KC; the chains are added at the end - int32
// sums, the same total as one chain).  CP * KC * 2 MMAs are independent of each other, which is what hides the
// latency of the integer MMA (a dependent chain ran at about 300 cycles per k-step).
template <int CP, int KC>
__device__ __forceinline__ void matmul_fp_tensor_cp(uint16_t const *A, uint16_t const *B, uint16_t *C, int m, int n, int k,
                                                    int b_pitch, bool b_swizzled, int tid, int nthreads) {
  int const lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
  int const g = lane >> 2, t = lane & 3, mi = lane >> 3, rr = lane & 7;
  int const row_groups = (m + 3) >> 2, col_blocks = (n >> 4) / CP;
  uint32_t const b_base = (uint32_t)__cvta_generic_to_shared(B);
  for (int w = warp; w < row_groups * col_blocks; w += nwarps) {
    int const rg = w / col_blocks, cb = w % col_blocks;
    int const row = rg * 4 + (g & 3);
    bool const valid = row < m;
    int32_t acc[KC][CP][2][4];
#pragma unroll
    for (int kc = 0; kc < KC; kc++)
#pragma unroll
      for (int c = 0; c < CP; c++)
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc[kc][c][h][j] = 0;
    uint16_t const *arow = A + (size_t)row * k + 2 * t;
    // ldmatrix (transposed): this lane addresses k-row (mi % 2) * 8 + rr of the 8 columns starting at (mi / 2) * 8
    uint32_t baddr[CP], bstep = (uint32_t)(16 * b_pitch * 2);
#pragma unroll
    for (int c = 0; c < CP; c++) {
      int const cp = cb * CP + c;
      baddr[c] = b_base + (uint32_t)((((mi & 1) * 8 + rr) * b_pitch + cp * 16 + (mi >> 1) * 8) * 2);
      if (b_swizzled) {
        int const unit = cp * 2 + (mi >> 1); // 16-byte unit of the row: 8 per box
        baddr[c] = b_base + (uint32_t)((unit >> 3) * k * 128 + ((mi & 1) * 8 + rr) * 128 + (((unit & 7) ^ rr) << 4));
      }
    }
    if (b_swizzled) bstep = 16u * 128u;
    // one k-step (16 uint16 of A's rows against 16 rows of B) into chain `kc`
    auto step = [&](int k0, int32_t (&into)[CP][2][4]) {
      uint32_t const w0 = valid ? *reinterpret_cast<uint32_t const *>(arow + k0) : 0u;
      uint32_t const w1 = valid ? *reinterpret_cast<uint32_t const *>(arow + k0 + 8) : 0u;
      uint32_t a[4];
      if (g < 4) { // MMA rows 0-3: [lo,0] bytes; MMA rows 8-11: [hi,lo] bytes
        a[0] = w0 & 0x00FF00FFu; a[2] = w1 & 0x00FF00FFu;
        a[1] = __byte_perm(w0, 0, 0x2301); a[3] = __byte_perm(w1, 0, 0x2301);
      } else {     // MMA rows 4-7: [0,hi] bytes; MMA rows 12-15 unused
        a[0] = w0 & 0xFF00FF00u; a[2] = w1 & 0xFF00FF00u;
        a[1] = 0u; a[3] = 0u;
      }
      uint32_t bf[CP][4];
#pragma unroll
      for (int c = 0; c < CP; c++) {
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(bf[c][0]), "=r"(bf[c][1]), "=r"(bf[c][2]), "=r"(bf[c][3]) : "r"(baddr[c]));
        baddr[c] += bstep;
      }
#pragma unroll
      for (int c = 0; c < CP; c++)
#pragma unroll
        for (int h = 0; h < 2; h++)
          asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                       : "+r"(into[c][h][0]), "+r"(into[c][h][1]), "+r"(into[c][h][2]), "+r"(into[c][h][3])
                       : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(bf[c][2 * h]), "r"(bf[c][2 * h + 1]));
    };
    int k0 = 0;
    for (; k0 + 16 * KC <= k; k0 += 16 * KC) {
#pragma unroll
      for (int kc = 0; kc < KC; kc++) step(k0 + 16 * kc, acc[kc]);
    }
    for (; k0 < k; k0 += 16) step(k0, acc[0]);
#pragma unroll
    for (int kc = 1; kc < KC; kc++)
#pragma unroll
      for (int c = 0; c < CP; c++)
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc[0][c][h][j] += acc[kc][c][h][j];
#pragma unroll
    for (int c = 0; c < CP; c++)
#pragma unroll
      for (int h = 0; h < 2; h++) {
        // lanes 16-31 hold the HH sums of the rows lanes 0-15 work on
        int32_t const hh0 = __shfl_down_sync(0xffffffffu, acc[0][c][h][0], 16), hh1 = __shfl_down_sync(0xffffffffu, acc[0][c][h][1], 16);
        if (g < 4 && valid) {
          uint32_t v0 = ((uint32_t)acc[0][c][h][0] % PQ + 256u * ((uint32_t)acc[0][c][h][2] % PQ) + (65536u % PQ) * ((uint32_t)hh0 % PQ)) % PQ;
          uint32_t v1 = ((uint32_t)acc[0][c][h][1] % PQ + 256u * ((uint32_t)acc[0][c][h][3] % PQ) + (65536u % PQ) * ((uint32_t)hh1 % PQ)) % PQ;
          *reinterpret_cast<uint32_t *>(C + (size_t)row * n + (cb * CP + c) * 16 + h * 8 + 2 * t) = v0 | (v1 << 16);
        }
      }
  }
}

// WIDE: the kernel instance has registers for eight independent MMA pairs (blocks of up to 512 threads), else four
template <bool WIDE>
__device__ __forceinline__ void matmul_fp_tensor(uint16_t const *A, uint16_t const *B, uint16_t *C, int m, int n, int k,
                                                 int b_pitch, bool b_swizzled, int tid, int nthreads) {
  // as many column pairs side by side as still leave every warp a piece of the tile; the rest as chains along k
  int const row_groups = (m + 3) >> 2, col_pairs = n >> 4, nwarps = nthreads >> 5;
  if (WIDE) {
    if ((col_pairs & 3) == 0 && row_groups * (col_pairs >> 2) >= nwarps) matmul_fp_tensor_cp<4, 1>(A, B, C, m, n, k, b_pitch, b_swizzled, tid, nthreads);
    else if ((col_pairs & 1) == 0 && row_groups * (col_pairs >> 1) >= nwarps) matmul_fp_tensor_cp<2, 2>(A, B, C, m, n, k, b_pitch, b_swizzled, tid, nthreads);
    else matmul_fp_tensor_cp<1, 4>(A, B, C, m, n, k, b_pitch, b_swizzled, tid, nthreads);
  } else {
    if ((col_pairs & 1) == 0 && row_groups * (col_pairs >> 1) >= nwarps) matmul_fp_tensor_cp<2, 1>(A, B, C, m, n, k, b_pitch, b_swizzled, tid, nthreads);
    else matmul_fp_tensor_cp<1, 2>(A, B, C, m, n, k, b_pitch, b_swizzled, tid, nthreads);
  }
}

// MAXT: the largest block this instance is launched with (1024: 64 registers a thread; 512: 128)
template <int MAXT>
__global__ void __launch_bounds__(MAXT) fp_interp_kernel(const __grid_constant__ mgd_program prog,
                                                        const __grid_constant__ mgd_bindings bind,
                                                        const __grid_constant__ interp::TmaPlan tma,
                                                        const __grid_constant__ interp::TmaMaps maps, int32_t *status) {
  extern __shared__ __align__(16) unsigned char smem_dyn[];
  // swizzled boxes want their 1024-byte pattern aligned: the plan's offsets are relative to an aligned base
  // (the host leaves room for that only when a tensor-map form is in use)
  unsigned char *smem_raw = (tma.tiled_mask | tma.swizzled_mask)
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
    return reinterpret_cast<uint16_t *>(smem_raw + byte_offset + extra);
  };
  uint32_t const tma_mask = tma.moving_mask | tma.once_mask;

  if (tid == 0) {
    for (int s = 0; s <= interp::kMaxStages; s++) ptx::mbar_init(ptx::smem_u32(&bars[s]), 1);
    ptx::mbar_init_fence();
  }
  // The finite-field tables in shared memory: threads of a warp look up different entries, which the constant cache
  // serves one address at a time (an exp over a 4096-element tile took 8 k cycles that way, 0.3 k from here).
  uint16_t *const tab_exp = tma.field_tables ? reinterpret_cast<uint16_t *>(smem_dyn + tma.field_tables - 1) : nullptr;
  uint16_t *const tab_p = tab_exp + Q, *const tab_q = tab_exp + Q + P;
  if (tab_exp != nullptr) {
    for (int i = tid; i < (int)Q; i += nt) {
      tab_exp[i] = (uint16_t)((c_tables.e[i] * Q_MUL_P_MOD_1) % PQ); // the lift to Z_PQ folded in
      tab_q[i] = c_tables.q[i];
    }
    for (int i = tid; i < (int)P; i += nt) tab_p[i] = c_tables.p[i];
  }
  __syncthreads();
  // the inputs the TMA engine fetches, resolved once for this block
  __shared__ interp::TileFetch fetch[MGD_MAX_IO];
  int const n_fetch = __popc(tma_mask);
  if (tid < prog.num_ops && ((tma_mask >> tid) & 1u)) {
    int32_t const *a = prog.ops[tid].a;
    interp::resolve_fetch(fetch[__popc(tma_mask & ((1u << tid) - 1u))], a, tma, maps, tid, bind.in[a[18]],
                          set * bind.in_set_stride[a[18]], bx, by, bz, a[15] + ((a[16] >> 8) & 0xff), smem_raw);
  }
  __syncthreads();
  auto issue = [&](uint32_t mask, int it, int stage, uint32_t bar, int tx) {
    interp::issue_fetches(fetch, n_fetch, mask == tma.moving_mask ? 1 : 0, it, stage, bar, tx, lane);
  };
  int issued = 0; // iterations whose ring tiles have been requested
  if (warp == 0) {
    if (tma.once_mask) issue(tma.once_mask, 0, 0, ptx::smem_u32(&bars[interp::kMaxStages]), tma.once_tx);
    if (tma.stages > 0)
      for (; issued < tma.stages && issued <= last; issued++)
        issue(tma.moving_mask, issued, issued, ptx::smem_u32(&bars[issued]), tma.moving_tx);
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

#ifdef MG_FP_TIMING // cycles of thread 0 per operator, summed over the for-loop; block 0 prints them
  long long t_op[MGD_MAX_OPS] = {}, t_wait = 0, t_issue = 0, t_begin = clock64();
#endif
  for (int it = 0; it <= last; it++) {
#ifdef MG_FP_TIMING
    long long t_w0 = clock64();
#endif
    if (tma.stages > 0) {
      int const s = it % tma.stages;
      stage_offset = s * tma.ring_bytes;
      bool ok = ptx::mbar_wait(ptx::smem_u32(&bars[s]), (uint32_t)((it / tma.stages) & 1));
      if (!__syncthreads_and(ok)) { give_up(); return; }
    }
#ifdef MG_FP_TIMING
    t_wait += clock64() - t_w0;
#endif
    for (int oi = 0; oi < prog.num_ops; oi++) {
#ifdef MG_FP_TIMING
      long long const t_o0 = clock64();
      struct Tock { long long &acc; long long t0; __device__ ~Tock() { acc += clock64() - t0; } } tock{t_op[oi], t_o0};
#endif
      mgd_op const &op = prog.ops[oi];
      int32_t const *a = op.a;
      if (op.type == interp::kOpInput) {
        if ((tma_mask >> oi) & 1u) continue;                              // fetched by the TMA engine
        if (it > 0 && ((tma.plain_once_mask >> oi) & 1u)) continue;       // same tile as in the first iteration
      } else if (a[interp::kPhaseSlot] != 0 && it != last) {
        continue;                                                         // runs once, after the loop
      }
      bool const first = it == 0 || (op.type != interp::kOpInput && a[interp::kPhaseSlot] != 0);
      switch (op.type) {
        case interp::kOpInput: { // input tile on plain loads
          int row = bx * a[0] + by * a[1] + bz * a[2] + it * a[6];
          int col = bx * a[3] + by * a[4] + bz * a[5] + it * a[7];
          int64_t lead = (int64_t)bx * a[8] + (int64_t)by * a[9] + (int64_t)bz * a[10] + (int64_t)it * a[11];
          uint16_t const *src =
              static_cast<uint16_t const *>(bind.in[a[18]]) + set * bind.in_set_stride[a[18]] + lead;
          // layout tag a[16] is deliberately ignored: fingerprints are indexed row-major
          load_tile_u16(tile(a[17]), src, a[14], a[15], a[15] + ((a[16] >> 8) & 0xff), a[13], row, col, tid, nt);
          break;
        }
        case MG_TB_MATMUL_OP: {
          int m = a[0], n = a[1], k = a[2];
          uint16_t const *A = tile(a[3]), *B = tile(a[4]);
          uint16_t *C = tile(a[5]);
          int const bp = a[6] > 0 ? a[6] : n; // row pitch of B: padded by the host when the dense pitch conflicts
          if ((k & 15) == 0 && (n & 15) == 0 && k <= 16384 && (nt & 31) == 0) {
            matmul_fp_tensor<(MAXT <= 512)>(A, B, C, m, n, k, bp, a[7] != 0, tid, nt);
            break;
          }
          for (int i = tid; i < m * n; i += nt) {
            int r = i / n, c = i % n;
            uint16_t const *ar = A + r * k, *bc = B + c;
            unsigned long long acc = 0;
            int kk = 0;
            for (; kk + 4 <= k; kk += 4) {
              acc += (unsigned long long)((uint32_t)ar[kk] * (uint32_t)bc[(kk)*bp]);
              acc += (unsigned long long)((uint32_t)ar[kk + 1] * (uint32_t)bc[(kk + 1) * bp]);
              acc += (unsigned long long)((uint32_t)ar[kk + 2] * (uint32_t)bc[(kk + 2) * bp]);
              acc += (unsigned long long)((uint32_t)ar[kk + 3] * (uint32_t)bc[(kk + 3) * bp]);
            }
            for (; kk < k; kk++) acc += (unsigned long long)((uint32_t)ar[kk] * (uint32_t)bc[kk * bp]);
            C[i] = (uint16_t)(acc % PQ);
          }
          break;
        }
        case MG_TB_EXP_OP: {
          uint16_t *x = tile(a[0]);
          if (tab_exp != nullptr) {
            for (int i = tid; i < a[1]; i += nt) x[i] = tab_exp[x[i] % Q];
          } else {
            for (int i = tid; i < a[1]; i += nt) x[i] = (uint16_t)field_exp(x[i]);
          }
          break;
        }
        case MG_TB_DIV_OP:
        case MG_TB_ADD_OP:
        case MG_TB_MUL_OP: {
          int const xd[3] = {a[0], a[1], a[2]}, yd[3] = {a[3], a[4], a[5]};
          int const zd[3] = {max(xd[0], yd[0]), max(xd[1], yd[1]), max(xd[2], yd[2])};
          uint16_t const *x = tile(a[6]), *y = tile(a[7]);
          uint16_t *z = tile(a[8]);
          int n = zd[0] * zd[1] * zd[2];
          for (int i = tid; i < n; i += nt) {
            int rest = i, xs = 1, ys = 1, xi = 0, yi = 0;
            for (int d = 2; d >= 0; d--) { // broadcast: an extent-1 dim always maps to index 0
              xi += (rest % xd[d]) * xs;
              yi += (rest % yd[d]) * ys;
              xs *= xd[d];
              ys *= yd[d];
              rest /= zd[d];
            }
            uint32_t xv = x[xi], yv = y[yi], r;
            if (op.type == MG_TB_DIV_OP)
              r = tab_exp != nullptr ? ((xv % P) * tab_p[yv % P] * Q_MUL_P_MOD_1 + (xv % Q) * tab_q[yv % Q] * P_MUL_Q_MOD_1) % PQ
                                     : field_div(xv, yv);
            else if (op.type == MG_TB_ADD_OP) r = (xv + yv) % PQ;
            else r = (uint32_t)(((unsigned long long)xv * yv) % PQ);
            z[i] = (uint16_t)r;
          }
          break;
        }
        case MG_TB_REDUCTION_0_OP: case MG_TB_REDUCTION_1_OP: case MG_TB_REDUCTION_2_OP:
        case MG_TB_REDUCTION_0_TO_DIMX_OP: case MG_TB_REDUCTION_1_TO_DIMX_OP: case MG_TB_REDUCTION_2_TO_DIMX_OP: {
          int n_out = a[0], degree = a[1], inner = a[2];
          uint16_t const *x = tile(a[3]);
          uint16_t *y = tile(a[4]);
          if (n_out < nt && degree >= 8 && degree < 65536) {
            // fewer sums than threads: a warp per sum, lanes stride over the terms (a sum of 65535 terms fits 32 bits)
            for (int i = warp; i < n_out; i += nt >> 5) {
              int const base = (i / inner) * (inner * degree) + i % inner;
              uint32_t acc = 0;
              for (int k = lane; k < degree; k += 32) acc += x[base + k * inner];
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
              if (lane == 0) y[i] = (uint16_t)(acc % PQ);
            }
            break;
          }
          for (int i = tid; i < n_out; i += nt) {
            int pos = (i / inner) * (inner * degree) + i % inner;
            unsigned long long acc = 0;
            for (int k = 0; k < degree; k++, pos += inner) acc += x[pos];
            y[i] = (uint16_t)(acc % PQ);
          }
          break;
        }
        case MG_TB_CONCAT_0_OP: case MG_TB_CONCAT_1_OP: case MG_TB_CONCAT_2_OP: {
          int n_out = a[0], ad = a[1], bd = a[2], inner = a[3];
          uint16_t const *A = tile(a[4]), *B = tile(a[5]);
          uint16_t *y = tile(a[6]);
          for (int i = tid; i < n_out; i += nt) {
            int in_idx = i % inner, along = (i / inner) % (ad + bd), outer = (i / inner) / (ad + bd);
            y[i] = along < ad ? A[in_idx + along * inner + outer * inner * ad]
                              : B[in_idx + (along - ad) * inner + outer * inner * bd];
          }
          break;
        }
        case interp::kOpAccumulate: { // running sum of a tile over the for-loop (the hoisted matmul's left operand)
          uint16_t const *x = tile(a[1]);
          uint16_t *acc = tile(a[2]);
          if (first) {
            for (int i = tid; i < a[0]; i += nt) acc[i] = (uint16_t)((uint32_t)x[i] % PQ);
          } else {
            for (int i = tid; i < a[0]; i += nt) acc[i] = (uint16_t)(((uint32_t)x[i] + (uint32_t)acc[i]) % PQ);
          }
          break;
        }
        case interp::kOpOutput: { // output: accumulate over the for-loop, store after the last iteration
          int n = a[11] * a[12];
          uint16_t const *x = tile(a[13]);
          uint16_t *acc = tile(a[14]);
          if (first) {
            for (int i = tid; i < n; i += nt) acc[i] = x[i];
          } else {
            for (int i = tid; i < n; i += nt) acc[i] = (uint16_t)(((uint32_t)x[i] + (uint32_t)acc[i]) % PQ);
          }
          if (it == last) {
            __syncthreads();
            int row = bx * a[0] + by * a[1] + bz * a[2];
            int col = bx * a[3] + by * a[4] + bz * a[5];
            int64_t lead = (int64_t)bx * a[6] + (int64_t)by * a[7] + (int64_t)bz * a[8];
            uint16_t *dst = static_cast<uint16_t *>(bind.out[a[15]]) + set * bind.out_set_stride[a[15]] + lead;
            int cols = a[12], ld = a[10];
            if ((cols & 1) == 0 && (ld & 1) == 0 && (col & 1) == 0 && (reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
              for (int i = tid; i < n / 2; i += nt) { // two columns per store
                int const e = 2 * i;
                *reinterpret_cast<uint32_t *>(dst + (size_t)(row + e / cols) * ld + col + e % cols) =
                    *reinterpret_cast<uint32_t const *>(acc + e);
              }
            } else {
              for (int i = tid; i < n; i += nt) dst[(size_t)(row + i / cols) * ld + col + i % cols] = acc[i];
            }
          }
          break;
        }
        default: break; // rejected on the host before launch
      }
      __syncthreads();
    }
    // every thread is past its last read of this iteration's stage: request the tiles of iteration it + stages into it
#ifdef MG_FP_TIMING
    long long t_i0 = clock64();
#endif
    if (warp == 0 && tma.stages > 0 && issued <= last) {
      ptx::fence_proxy_async_smem();
      int const s = it % tma.stages;
      issue(tma.moving_mask, issued, s, ptx::smem_u32(&bars[s]), tma.moving_tx);
      issued++;
    }
#ifdef MG_FP_TIMING
    t_issue += clock64() - t_i0;
#endif
  }
#ifdef MG_FP_TIMING
  if (blockIdx.x == 0 && tid == 0) {
    printf("fp_interp: %d threads, %d iterations, ring stages %d, total %lld cycles, tile waits %lld, issue %lld\n", nt, last + 1,
           tma.stages, clock64() - t_begin, t_wait, t_issue);
    for (int oi = 0; oi < prog.num_ops; oi++)
      printf("  op %d type %d: %lld cycles  (a0..a2 %d %d %d, a6 %d, a7 %d)\n", oi, prog.ops[oi].type, t_op[oi], prog.ops[oi].a[0],
             prog.ops[oi].a[1], prog.ops[oi].a[2], prog.ops[oi].a[6], prog.ops[oi].a[7]);
  }
#endif
}

static bool op_type_known(int t) {
  return t == 2001 || t == 2002 || t == MG_TB_MATMUL_OP || t == MG_TB_EXP_OP || t == MG_TB_DIV_OP ||
         t == MG_TB_ADD_OP || t == MG_TB_MUL_OP || (t >= MG_TB_REDUCTION_0_OP && t <= MG_TB_REDUCTION_2_TO_DIMX_OP) ||
         (t >= MG_TB_CONCAT_0_OP && t <= MG_TB_CONCAT_2_OP);
}

int validate_program(mgd_program const *p, mgd_bindings const *b) {
  if (!p || !b) return set_error(MG_ERR_INVALID_ARGUMENT, "null program");
  if (p->num_ops <= 0 || p->num_ops > MGD_MAX_OPS) return set_error(MG_ERR_INVALID_ARGUMENT, "operator count out of range");
  if (p->grid[0] <= 0 || p->grid[1] <= 0 || p->grid[2] <= 0 || p->forloop_range <= 0 || b->num_sets <= 0)
    return set_error(MG_ERR_INVALID_ARGUMENT, "grid, for-loop range and set count must be positive");
  for (int i = 0; i < p->num_ops; i++)
    if (!op_type_known(p->ops[i].type)) return set_error(MG_ERR_UNSUPPORTED, "operator type without a kernel");
  for (int i = 0; i < p->num_inputs; i++)
    if (!b->in[i]) return set_error(MG_ERR_INVALID_ARGUMENT, "unbound input");
  for (int i = 0; i < p->num_outputs; i++)
    if (!b->out[i]) return set_error(MG_ERR_INVALID_ARGUMENT, "unbound output");
  return MG_OK;
}

// ---- host: shared-memory plan of this kernel ----------------------------------------------------------------------
// The reference's dense plan with three changes.  (1) ldmatrix reads 8 rows of 16 bytes of a matmul's B operand at a
// time; a row pitch that is a multiple of 128 bytes puts all 8 on the same banks, so a tile that only input loaders
// write and only matmuls read as their B operand is stored with 16 bytes of padding per row.  (2) The tiles the TMA
// engine refills every iteration come first, back to back, and that region exists `stages` times (the ring).
// (3) Every other tile follows in planned order.  Tiles keep their identity (planned offset), so the aliasing of the
// in-place exp is unchanged.
namespace {
struct FpTile {
  int planned, elems, rows, cols;
  bool only_loaded, only_b_operand;
  int offset, pad;
  bool ring;
  bool swizzled; // stored as 64-column boxes with the 128-byte swizzle (instead of padded rows)
  bool boxed;    // fetched as one dense tensor-map box
  // a tensor-map box must land on a 128-byte boundary; the swizzle pattern repeats every 1024 bytes
  size_t alignment() const { return swizzled ? 1024 : (boxed ? 128 : 16); }
};

struct FpPlan {
  mgd_program prog;
  interp::TmaPlan tma;
  interp::TmaMaps maps;
  size_t smem_bytes;
  bool ok;
};

void plan_fingerprint_program(mgd_program const &in, mgd_bindings const &bind, bool pad, bool use_tma, FpPlan *out) {
  FpTile tiles[3 * MGD_MAX_OPS + 4];
  int n = 0;
  auto touch = [&](int planned, int elems) -> FpTile & {
    for (int i = 0; i < n; i++)
      if (tiles[i].planned == planned) {
        if (elems > tiles[i].elems) tiles[i].elems = elems;
        return tiles[i];
      }
    tiles[n] = FpTile{planned, elems, 0, 0, true, true, 0, 0, false, false, false};
    return tiles[n++];
  };
  for (int i = 0; i < in.num_ops; i++) {
    int32_t const *a = in.ops[i].a;
    int const type = in.ops[i].type;
    if (type == interp::kOpInput) {
      FpTile &t = touch(a[17], a[14] * a[15]);
      t.rows = a[14]; t.cols = a[15];
    } else if (type == MG_TB_MATMUL_OP) {
      touch(a[3], a[0] * a[2]).only_b_operand = false;
      touch(a[4], a[2] * a[1]);
      FpTile &c = touch(a[5], a[0] * a[1]);
      c.only_loaded = false;
    } else if (type == MG_TB_EXP_OP) {
      FpTile &t = touch(a[0], a[1]);
      t.only_loaded = false; t.only_b_operand = false;
    } else if (interp::is_binary(type)) {
      int zx = a[0] > a[3] ? a[0] : a[3], zy = a[1] > a[4] ? a[1] : a[4], zz = a[2] > a[5] ? a[2] : a[5];
      touch(a[6], a[0] * a[1] * a[2]).only_b_operand = false;
      touch(a[7], a[3] * a[4] * a[5]).only_b_operand = false;
      touch(a[8], zx * zy * zz).only_loaded = false;
    } else if (interp::is_reduction(type)) {
      touch(a[3], a[0] * a[1]).only_b_operand = false;
      touch(a[4], a[0]).only_loaded = false;
    } else if (interp::is_concat(type)) {
      int along = a[1] + a[2];
      touch(a[4], along > 0 ? a[0] / along * a[1] : 0).only_b_operand = false;
      touch(a[5], along > 0 ? a[0] / along * a[2] : 0).only_b_operand = false;
      touch(a[6], a[0]).only_loaded = false;
    } else if (type == interp::kOpAccumulate) {
      touch(a[1], a[0]).only_b_operand = false;
      FpTile &acc = touch(a[2], a[0]);
      acc.only_loaded = false; acc.only_b_operand = false;
    } else if (type == interp::kOpOutput) {
      touch(a[13], a[11] * a[12]).only_b_operand = false;
      FpTile &acc = touch(a[14], a[11] * a[12]);
      acc.only_loaded = false; acc.only_b_operand = false;
    }
  }
  auto find = [&](int planned) -> FpTile & {
    for (int i = 0; i < n; i++)
      if (tiles[i].planned == planned) return tiles[i];
    return tiles[0];
  };
  // a padded tile must really be a B operand of matching shape somewhere
  for (int i = 0; i < n; i++) {
    FpTile &t = tiles[i];
    bool used_as_b = false;
    for (int j = 0; j < in.num_ops; j++)
      if (in.ops[j].type == MG_TB_MATMUL_OP && in.ops[j].a[4] == t.planned) {
        used_as_b = true;
        if (in.ops[j].a[2] != t.rows || in.ops[j].a[1] != t.cols) t.only_b_operand = false;
      }
    t.pad = (pad && used_as_b && t.only_loaded && t.only_b_operand && t.rows > 0 && (t.cols * 2) % 128 == 0) ? 8 : 0;
  }
  // which inputs the TMA engine fetches, and how: an input whose tile is the same in every iteration and that no
  // in-place operator overwrites is fetched once; every other eligible input goes through the ring
  interp::TmaPlan &tma = out->tma;
  std::memset(&tma, 0, sizeof(tma));
  std::memset(&out->maps, 0, sizeof(out->maps));
  for (int i = 0; i < in.num_ops; i++) {
    mgd_op const &op = in.ops[i];
    if (op.type != interp::kOpInput) continue;
    FpTile &t = find(op.a[17]);
    int writers = 0;
    bool overwritten = false;
    for (int j = 0; j < in.num_ops; j++) {
      if (interp::written_by(in.ops[j]) == t.planned) writers++;
      if (in.ops[j].type == MG_TB_EXP_OP && in.ops[j].a[0] == t.planned) overwritten = true;
    }
    bool const invariant = !interp::input_moves(op) && !overwritten && writers == 1;
    int const slot = op.a[18];
    bool const eligible = use_tma && writers <= 2 && t.elems == t.rows * t.cols &&
                          interp::tma_eligible(op, bind.in[slot], bind.in_set_stride[slot], bind.num_sets, t.cols + t.pad, false);
    if (eligible) {
      // the tiled forms need a tensor map; one input per tile only (a tile has one layout)
      int inputs_of_tile = 0;
      for (int j = 0; j < in.num_ops; j++) inputs_of_tile += in.ops[j].type == interp::kOpInput && in.ops[j].a[17] == t.planned;
      int form = inputs_of_tile == 1 ? interp::tiled_form(op, bind.in_set_stride[slot], bind.num_sets, t.pad > 0) : 0;
      if (form && !interp::make_tile_map(&out->maps.m[slot], bind.in[slot], (uint64_t)op.a[13], (uint64_t)op.a[12],
                                         interp::matrices_addressed(in, op, bind.in_set_stride[slot], bind.num_sets),
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
    if (eligible && invariant) {
      tma.once_mask |= 1u << i;
      tma.once_tx += t.rows * t.cols * 2;
    } else if (eligible && in.forloop_range > 1 && !t.ring) {
      // (a tile two inputs write cannot be in the ring twice: the second one stays on plain loads)
      bool shared_tile = false;
      for (int j = 0; j < i; j++)
        if (in.ops[j].type == interp::kOpInput && in.ops[j].a[17] == t.planned) shared_tile = true;
      if (!shared_tile) {
        tma.moving_mask |= 1u << i;
        tma.moving_tx += t.rows * t.cols * 2;
        t.ring = true;
      }
    } else if (eligible && in.forloop_range == 1 && writers == 1) {
      tma.once_mask |= 1u << i; // a single iteration: everything is fetched once
      tma.once_tx += t.rows * t.cols * 2;
    } else if (invariant) {
      tma.plain_once_mask |= 1u << i;
    }
  }
  // offsets: ring tiles first (planned order), then the rest (planned order); insertion sort, at most 76 tiles
  int order[3 * MGD_MAX_OPS + 4];
  for (int i = 0; i < n; i++) order[i] = i;
  auto before = [&](FpTile const &x, FpTile const &y) { return x.ring != y.ring ? x.ring : x.planned < y.planned; };
  for (int i = 1; i < n; i++)
    for (int j = i; j > 0 && before(tiles[order[j]], tiles[order[j - 1]]); j--) {
      int tmp = order[j]; order[j] = order[j - 1]; order[j - 1] = tmp;
    }
  auto bytes_of = [](FpTile const &t) {
    size_t b = t.pad ? (size_t)t.rows * (t.cols + t.pad) * 2 : (size_t)t.elems * 2;
    return (b + t.alignment() - 1) & ~(t.alignment() - 1);
  };
  // tiles start on their alignment; the ring then repeats at a multiple of 1024 bytes
  auto place = [](size_t at, FpTile const &t) { return (at + t.alignment() - 1) & ~(t.alignment() - 1); };
  size_t ring_bytes = 0, rest_bytes = 0;
  for (int i = 0; i < n; i++) {
    FpTile const &t = tiles[order[i]];
    if (t.ring) ring_bytes = place(ring_bytes, t) + bytes_of(t);
    else rest_bytes += bytes_of(t) + (t.alignment() > 16 ? t.alignment() : 0);
  }
  ring_bytes = (ring_bytes + 1023) & ~(size_t)1023;
  int stages = 0;
  if (ring_bytes > 0) {
    stages = in.forloop_range < 3 ? in.forloop_range : 3;
    while (stages > 1 && ring_bytes * stages + rest_bytes + 16 + 1024 > (size_t)interp::kDynSmemLimit) stages--;
  }
  tma.stages = stages;
  tma.ring_lo = 0;
  tma.ring_bytes = (int32_t)ring_bytes;
  size_t at = 0;
  for (int i = 0; i < n; i++) {
    FpTile &t = tiles[order[i]];
    if (!t.ring && at < ring_bytes * (size_t)(stages > 0 ? stages : 0)) at = ring_bytes * (size_t)stages;
    at = place(at, t);
    t.offset = (int)at;
    at += bytes_of(t);
  }
  if (at < ring_bytes * (size_t)stages) at = ring_bytes * (size_t)stages;
  out->smem_bytes = at + 16 + ((tma.tiled_mask | tma.swizzled_mask) ? 1024 : 0); // + room to align the base to 1024 bytes
  out->prog = in;
  for (int i = 0; i < in.num_ops; i++) {
    int32_t const *a = in.ops[i].a;
    int32_t *w = out->prog.ops[i].a;
    int const type = in.ops[i].type;
    if (type == interp::kOpInput) {
      w[17] = find(a[17]).offset;
      w[16] = (a[16] & 0xff) | (find(a[17]).pad << 8);
    } else if (type == MG_TB_MATMUL_OP) {
      w[3] = find(a[3]).offset; w[4] = find(a[4]).offset; w[5] = find(a[5]).offset;
      w[6] = find(a[4]).pad ? a[1] + find(a[4]).pad : 0;
      w[7] = find(a[4]).swizzled ? 1 : 0;
    } else if (type == MG_TB_EXP_OP) {
      w[0] = find(a[0]).offset;
    } else if (interp::is_binary(type)) {
      w[6] = find(a[6]).offset; w[7] = find(a[7]).offset; w[8] = find(a[8]).offset;
    } else if (interp::is_reduction(type)) {
      w[3] = find(a[3]).offset; w[4] = find(a[4]).offset;
    } else if (interp::is_concat(type)) {
      w[4] = find(a[4]).offset; w[5] = find(a[5]).offset; w[6] = find(a[6]).offset;
    } else if (type == interp::kOpAccumulate) {
      w[1] = find(a[1]).offset; w[2] = find(a[2]).offset;
    } else if (type == interp::kOpOutput) {
      w[13] = find(a[13]).offset; w[14] = find(a[14]).offset;
    }
  }
}
} // namespace
} // namespace mgk

using namespace mgk;

extern "C" int mgd_launch_fingerprint_interp(const mgd_program *prog, const mgd_bindings *bind, void *stream) {
  int st = validate_program(prog, bind);
  if (st != MG_OK) return st;
  // Rewrite (hoisted products), then plan: padded operands and the TMA ring when they fit, else step back towards
  // the reference's dense plan with plain loads.
  mgd_program rewritten = *prog;
  interp::hoist_invariant_products(rewritten);
  FpPlan plan;
  plan_fingerprint_program(rewritten, *bind, true, true, &plan);
  if (plan.smem_bytes > (size_t)interp::kDynSmemLimit) plan_fingerprint_program(rewritten, *bind, false, true, &plan);
  if (plan.smem_bytes > (size_t)interp::kDynSmemLimit) plan_fingerprint_program(*prog, *bind, false, false, &plan);
  size_t smem = plan.smem_bytes;
  if (smem > (size_t)interp::kDynSmemLimit) return set_error(MG_ERR_UNSUPPORTED, "threadblock graph needs more shared memory than an SM has");
  // room for the finite-field tables behind the plan, when the program looks anything up and an SM has the room
  plan.tma.field_tables = 0;
  for (int i = 0; i < plan.prog.num_ops; i++) {
    int const t = plan.prog.ops[i].type;
    if ((t == MG_TB_EXP_OP || t == MG_TB_DIV_OP) && ((smem + 15) & ~(size_t)15) + interp::kFieldTableBytes <= (size_t)interp::kDynSmemLimit) {
      plan.tma.field_tables = (int32_t)((smem + 15) & ~(size_t)15) + 1;
      smem = ((smem + 15) & ~(size_t)15) + interp::kFieldTableBytes;
      break;
    }
  }
  int32_t *status = device_error_word();
  if (!status) return set_error(MG_ERR_CUDA, "cannot allocate the device status word");
  prog = &plan.prog;
  static bool configured[64] = {}; // per device: both instances
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (smem > 48 * 1024 && !configured[dev]) {
    if (cudaFuncSetAttribute(fp_interp_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, interp::kDynSmemLimit) != cudaSuccess ||
        cudaFuncSetAttribute(fp_interp_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, interp::kDynSmemLimit) != cudaSuccess)
      return check_launch("cudaFuncSetAttribute(fp_interp_kernel)");
    configured[dev] = true;
  }
  int64_t blocks = (int64_t)prog->grid[0] * prog->grid[1] * prog->grid[2] * bind->num_sets;
  if (blocks > 0x7fffffffLL) return set_error(MG_ERR_UNSUPPORTED, "too many blocks for one launch");
  // Blocks run one operator at a time with a barrier after each: big tiles get more warps to hide the latency of
  // the dependent instruction chains (the largest operator decides).
  int64_t largest = 0;
  for (int i = 0; i < prog->num_ops; i++) {
    int32_t const *a = prog->ops[i].a;
    // what runs once after the loop does not size the block when the loop is long
    if (prog->ops[i].type != interp::kOpInput && a[interp::kPhaseSlot] != 0 && prog->forloop_range >= 4) continue;
    int64_t work = 0;
    switch (prog->ops[i].type) {
      case interp::kOpInput: // 16-byte plain loads; nothing for the threads to do when the TMA engine fetches it
        work = ((plan.tma.moving_mask | plan.tma.once_mask) >> i) & 1u ? 0 : (int64_t)a[14] * a[15] / 8;
        break;
      case interp::kOpOutput: work = (int64_t)a[11] * a[12] / (a[interp::kPhaseSlot] ? 4 : 1); break;
      case interp::kOpAccumulate: work = a[0]; break;
      case MG_TB_MATMUL_OP: work = (int64_t)a[0] * a[1]; break;
      case MG_TB_EXP_OP: work = a[1]; break;
      default: work = a[0]; break;
    }
    if (work > largest) largest = work;
  }
  unsigned threads = largest >= 8192 ? 1024u : (largest >= 2048 ? 512u : (largest >= 512 ? 256u : 128u));
  if (int const v = option(MGD_OPT_INTERP_THREADS)) // 128 ... 1024: for measurements
    if (v == 128 || v == 256 || v == 512 || v == 1024) threads = (unsigned)v;
  if (threads > 512) fp_interp_kernel<1024><<<(unsigned)blocks, threads, smem, (cudaStream_t)stream>>>(*prog, *bind, plan.tma, plan.maps, status);
  else fp_interp_kernel<512><<<(unsigned)blocks, threads, smem, (cudaStream_t)stream>>>(*prog, *bind, plan.tma, plan.maps, status);
  return check_launch("fp_interp_kernel");
}
