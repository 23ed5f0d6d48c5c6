// Dense attention operator on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// The operator is the first customized op of the prefill muGraph (pattern of the reference's
// cpp_examples/multi_head_attn_prefill.cc:43-98): a block owns 128 query rows of one head and walks the
// whole KV axis in for-loop tiles of 128:   S = Q K,  E = exp(S),  O' += E V,  R' += rowsum(E).
// Both contractions are 128x128x128 and run as tcgen05.mma (cta_group::1, kind::f16, M = N = 128, K = 16
// per instruction).  The A operand of both comes from tensor memory - Q is parked there once, E is handed
// over by the exp warps in place of the S values they consumed - so each MMA reads only its 4 KB B slice (a K
// or V tile in 128-byte-swizzled shared memory): with A in shared memory too, a 128 x 128 x 16 MMA needs
// 128 B/clk of shared-memory bandwidth, all an SM has, and the tensor pipe starves.  Accumulators are fp32:
//
//   TMEM columns [0,64): Q as packed 16-bit pairs      [64,192), [192,320): S, double buffered
//                [320,448): O', accumulated over all KV tiles
//   E of a tile overwrites its own S buffer: the thread that read S columns [64h, 64h+64) of a row writes the
//   32 packed columns of E to [64h, 64h+32).  MMAs issued by one thread execute in order, so the S of tile j+2
//   cannot overwrite the buffer before the second MMA of tile j has read E from it; no extra barrier is needed.
//
// Warp roles (320 threads):
//   warp 0, one lane   TMA producer: K and V tiles into a three-stage ring.
//   warp 1             allocates / frees tensor memory; one lane issues every MMA and commits to mbarriers.
//                      Issue order  S(0), S(1), O(0), S(2), O(1), ...  so the tensor pipe computes S of the
//                      next tile while the exp of the current one runs.
//   warps 2-9          two warpgroups, each thread owns one query row and one 64-column half of the tile; first
//                      it copies its half of the Q row from global memory into tensor memory, then per tile:
//                      tcgen05.ld its S half-row (32 columns at a time), exp, row sum, bf16/fp16 pack, tcgen05.st
//                      the packed E half-row back to tensor memory; at the end read O' and R' and store them
//                      (and, when the division operator is fused in, O = O' / R').  Two warps per scheduler
//                      hide each other's MUFU and tensor-memory latency.
// The reference executes this graph on its mma.sync interpreter (src/kernel/cuda/customized_kernel.cu:39-305).
//
// Every wait on an mbarrier is bounded.  A role that gives up raises a block-wide flag, the other roles stop
// at their next wait, the block frees its tensor memory, records the failure in the device status word and
// returns.
#include "common.cuh"
#include "tcgen05.cuh"
#include <cstdio>
#include <cstdlib>
#include <cuda.h>
#include <mutex>

namespace mgk {
namespace tc {

// Optional phase timing of block 0 (compile with -DMG_ROWS_TIMING; prints cycle totals from the device).
#ifdef MG_ROWS_TIMING
#define TICK(var) long long var = clock64()
#define TOCK(acc, var) acc += clock64() - var
#else
#define TICK(var)
#define TOCK(acc, var)
#endif

constexpr int kM = 128, kN = 128, kD = 128;         // query rows per block, KV positions per tile, head dim
constexpr int kSubTile = 128 * 64 * 2;                // one [128 rows][64 cols] 16-bit box: 16 KB
constexpr int kOperand = 2 * kSubTile;                // a 128 x 128 operand: two boxes
constexpr int kStages = 3;
constexpr uint32_t kTmemCols = 512;

using ptx::smem_u32;
using ptx::mbar_init;
using ptx::mbar_expect_tx;
using ptx::mbar_arrive;
using ptx::mbar_try_wait;
using ptx::tma_load_3d;
// Bounded wait that also gives up as soon as another role has raised the abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  return ptx::mbar_wait_or_abort(bar, parity, abort_flag);
}

// Shared-memory matrix descriptor of a K-major operand tile staged as [rows][64] boxes with the 128-byte
// swizzle: 8-row groups are 1024 bytes apart (stride byte offset), version 1, layout type 2 (SWIZZLE_128B).
// `byte_offset` selects the 16-element K step inside the 64-element swizzle span (32 bytes per step).
__device__ __forceinline__ uint64_t smem_desc(uint32_t tile_addr, uint32_t byte_offset) {
  uint64_t d = 0;
  d |= (uint64_t)(((tile_addr + byte_offset) & 0x3FFFF) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                                         // leading byte offset (unused for K-major SW128)
  d |= (uint64_t)(1024 >> 4) << 32;                               // stride byte offset
  d |= (uint64_t)1 << 46;                                         // descriptor version
  d |= (uint64_t)2 << 61;                                         // SWIZZLE_128B
  return d;
}
// D[tmem] (+)= A[smem] * B[smem]^T, kind::f16, issued by one thread
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// same with the A operand read from tensor memory (16-bit values packed two per column)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, uint32_t const (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                 "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
                 "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
                 "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
               : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                 "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                 "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
               : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

struct RowsParams {
  void const *q;    // [heads][seq_q][128]
  void *o_acc;      // [heads][seq_q][128]
  void *r_acc;      // [heads][seq_q][1]
  void *o_div;      // optional [heads][seq_q][128]: O' / R' (the division operator that follows, fused)
  int32_t *status;
  int heads, seq_q, kv_len, forloop;
};

struct Barriers {
  uint64_t q_ready, kv_full[kStages], kv_empty[kStages], s_full[2], e_full[2], o_full, dbg;
  uint32_t tmem_base;
  int abort_flag;
  float row_sums[2][kM]; // per column half
};

template <bool BF16>
__global__ void __launch_bounds__(320)
attn_rows_tc_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                    const __grid_constant__ CUtensorMap o_map, const __grid_constant__ CUtensorMap d_map,
                    const __grid_constant__ RowsParams p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  // [stage0: K 32 KB, V 32 KB][stage1][stage2][barriers]
  uint32_t const ring = smem_u32(smem);
  Barriers *bar = reinterpret_cast<Barriers *>(smem + kStages * 2 * kOperand);
  volatile int *abort_flag = &bar->abort_flag;

  int const tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int const qtiles = p.seq_q / kM;
  int const head = blockIdx.x / qtiles, q0 = (blockIdx.x % qtiles) * kM;

  if (tid == 0) {
    bar->abort_flag = 0;
    asm volatile("prefetch.tensormap [%0];" ::"l"(&k_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&v_map) : "memory");
    mbar_init(smem_u32(&bar->q_ready), 256);
    for (int s = 0; s < kStages; s++) {
      mbar_init(smem_u32(&bar->kv_full[s]), 1);
      mbar_init(smem_u32(&bar->kv_empty[s]), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(smem_u32(&bar->s_full[b]), 1);
      mbar_init(smem_u32(&bar->e_full[b]), 256);
    }
    mbar_init(smem_u32(&bar->o_full), 1);
    mbar_init(smem_u32(&bar->dbg), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) { // tensor memory: 512 columns (S x2, O'), allocated and later freed by this warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_base)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t const tmem = bar->tmem_base;
  uint32_t const tmem_q = tmem, tmem_s[2] = {tmem + 64, tmem + 192}, tmem_o = tmem + 320;
  int const F = p.forloop;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // (the whole warp walks the loop and waits together; one lane issues the copies)
    for (int j = 0; j < F; j++) {
      int s = j % kStages;
      if (j >= kStages && !mbar_wait(smem_u32(&bar->kv_empty[s]), (uint32_t)(((j / kStages) - 1) & 1), abort_flag)) break;
      if (lane == 0) {
        uint32_t full = smem_u32(&bar->kv_full[s]);
        uint32_t kdst = ring + (uint32_t)(s * 2 * kOperand), vdst = kdst + kOperand;
        int kv0 = j * kN;
        mbar_expect_tx(full, 2 * kOperand);
        // K memory [heads][kv][d]: rows = KV positions, two boxes over d
        tma_load_3d(kdst, &k_map, full, 0, kv0, head);
        tma_load_3d(kdst + kSubTile, &k_map, full, 64, kv0, head);
        // V memory [heads][d][kv]: rows = d, two boxes over this tile's KV positions
        tma_load_3d(vdst, &v_map, full, kv0, 0, head);
        tma_load_3d(vdst + kSubTile, &v_map, full, kv0 + 64, 0, head);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop and waits together (it stays converged); one lane issues.  Descriptors of a
    // stage differ from those of stage 0 only in the start-address field, and K steps inside a tile only by a
    // constant, so an MMA costs the issuing lane one 64-bit add.
    // instruction descriptor: fp32 accumulate, A/B format (0 = fp16, 1 = bf16), both K-major, N = 128, M = 128
    uint32_t const fmt = BF16 ? 1u : 0u;
    uint32_t const idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(kN >> 3) << 17) | ((uint32_t)(kM >> 4) << 24);
    uint64_t const desc0 = smem_desc(ring, 0);
    bool ok = mbar_wait(smem_u32(&bar->q_ready), 0, abort_flag);
#ifdef MG_ROWS_TIMING
    long long w_kv = 0, w_ef = 0, t_all = clock64();
    long long ev1s[16], ev1e[16], ev2s[16], ev2e[16];
    int dbg_n = 0; (void)dbg_n;
#endif
    for (int j = 0; j <= F && ok; j++) {
      if (j < F) { // S(j) = Q K_j^T into S buffer j % 2
        int s = j % kStages, b = j & 1;
        TICK(a0);
        ok = mbar_wait(smem_u32(&bar->kv_full[s]), (uint32_t)((j / kStages) & 1), abort_flag);
        TOCK(w_kv, a0);
        if (!ok) break;
        tc_fence_after();
#ifdef MG_ROWS_TIMING
        if (j < 16) ev1s[j] = clock64() - t_all;
#endif
        if (lane == 0) {
          uint64_t kdesc = desc0 + (uint64_t)((s * 2 * kOperand) >> 4);
#pragma unroll
          for (int ks = 0; ks < kD / 16; ks++) { // A = Q from tensor memory: 16 values = 8 packed columns per step
            uint64_t off = (uint64_t)(((ks >> 2) * kSubTile + (ks & 3) * 32) >> 4);
            umma_f16_ts(tmem_s[b], tmem_q + (uint32_t)(ks * 8), kdesc + off, idesc, ks > 0);
          }
          umma_commit(smem_u32(&bar->s_full[b]));
#ifdef MG_ROWS_TIMING2
          umma_commit(smem_u32(&bar->dbg));
#endif
        }
        __syncwarp();
#ifdef MG_ROWS_TIMING2
        mbar_wait(smem_u32(&bar->dbg), (uint32_t)(dbg_n++ & 1), abort_flag);
#endif
#ifdef MG_ROWS_TIMING
        if (j < 16) ev1e[j] = clock64() - t_all;
#endif
      }
      if (j >= 1) { // O' += E_{j-1} V_{j-1}
        int t = j - 1, s = t % kStages, eb = t & 1;
        TICK(a2);
        ok = mbar_wait(smem_u32(&bar->e_full[eb]), (uint32_t)((t >> 1) & 1), abort_flag);
        TOCK(w_ef, a2);
        if (!ok) break;
        tc_fence_after();
#ifdef MG_ROWS_TIMING
        if (t < 16) ev2s[t] = clock64() - t_all;
#endif
        if (lane == 0) {
          uint64_t vdesc = desc0 + (uint64_t)((s * 2 * kOperand + kOperand) >> 4);
#pragma unroll
          for (int ks = 0; ks < kN / 16; ks++) { // A = E in the S buffer: half h at columns [64h, 64h+32), 8 per step
            uint64_t off = (uint64_t)(((ks >> 2) * kSubTile + (ks & 3) * 32) >> 4);
            uint32_t ecol = (uint32_t)((ks >> 2) * 64 + (ks & 3) * 8);
            umma_f16_ts(tmem_o, tmem_s[eb] + ecol, vdesc + off, idesc, (t > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&bar->kv_empty[s]));  // K_t and V_t have been consumed
          if (t == F - 1) umma_commit(smem_u32(&bar->o_full));
#ifdef MG_ROWS_TIMING2
          umma_commit(smem_u32(&bar->dbg));
#endif
        }
        __syncwarp();
#ifdef MG_ROWS_TIMING2
        mbar_wait(smem_u32(&bar->dbg), (uint32_t)(dbg_n++ & 1), abort_flag);
#endif
#ifdef MG_ROWS_TIMING
        if (t < 16) ev2e[t] = clock64() - t_all;
#endif
      }
    }
#ifdef MG_ROWS_TIMING
    if (blockIdx.x == 0 && lane == 0) {
      printf("mma issuer: total %lld wait_kv %lld wait_e_full %lld (cycles, %d tiles) t0 %lld\n", clock64() - t_all, w_kv, w_ef, F, t_all);
      for (int j = 0; j < 16 && j < F; j++) printf("  tile %2d: mma1 issue %6lld..%6lld   mma2 issue %6lld..%6lld\n", j, ev1s[j], ev1e[j], ev2s[j], ev2e[j]);
    }
#endif
  } else {
    // ------------------------------------------------------------------ exp / row sums / epilogue
    // thread = (query row, 64-column half)
    int const quarter = warp & 3;                 // tensor-memory lanes this warp may touch: 32 * (warp % 4)
    int const half = (warp - 2) >> 2;             // which 64 columns of a tile
    int const row = quarter * 32 + lane;
    uint32_t const lane_base = (uint32_t)(quarter * 32) << 16;
    uint32_t const col_base = (uint32_t)(half * 64);
    float rsum = 0.f;
    bool ok = true;
    { // park this thread's half of its Q row in tensor memory: 64 values = 32 packed columns
      uint4 const *src = reinterpret_cast<uint4 const *>(static_cast<uint16_t const *>(p.q) +
                                                         ((size_t)head * p.seq_q + q0 + row) * kD + col_base);
      uint32_t qv[32];
#pragma unroll
      for (int i = 0; i < 8; i++) {
        uint4 w = __ldg(src + i);
        qv[4 * i] = w.x; qv[4 * i + 1] = w.y; qv[4 * i + 2] = w.z; qv[4 * i + 3] = w.w;
      }
      tmem_st32(tmem_q + lane_base + (uint32_t)(half * 32), qv);
      tc_fence_before();
      mbar_arrive(smem_u32(&bar->q_ready));
    }
#ifdef MG_ROWS_TIMING
    long long w_sf = 0, c_exp = 0, c_st = 0, t_all = clock64();
    long long es[16], ee[16], et[16];
#endif
    for (int j = 0; j < F && ok; j++) {
      int b = j & 1;
      TICK(b0);
      ok = mbar_wait(smem_u32(&bar->s_full[b]), (uint32_t)((j >> 1) & 1), abort_flag);
      TOCK(w_sf, b0);
      if (!ok) break;
      tc_fence_after();
      TICK(b1);
#ifdef MG_ROWS_TIMING
      if (j < 16) es[j] = clock64() - t_all;
#endif
      uint32_t packed[2][16]; // this thread's 64 values as 16-bit pairs
      {
        uint32_t v[64];
        t5::tmem_ld64(tmem_s[b] + lane_base + col_base, v); // one load, one wait per tile
        uint64_t sum2 = 0; // packed arithmetic: fewer issue slots taken from the MMA-issuing lane
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          float e0, e1;
          t5::exp_ftz2(t5::pair(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), e0, e1);
          sum2 = t5::add2(sum2, t5::pair(e0, e1));
          packed[i >> 5][(i & 31) >> 1] = pack2<BF16>(e0, e1);
        }
        float s0, s1;
        t5::unpair(sum2, s0, s1);
        rsum += s0 + s1;
      }
      TOCK(c_exp, b1);
      TICK(b3);
#ifdef MG_ROWS_TIMING
      if (j < 16) ee[j] = clock64() - t_all;
#endif
      // E replaces the S values this thread has just consumed: 32 packed columns at the start of its own half
      uint32_t flat[32];
#pragma unroll
      for (int i = 0; i < 32; i++) flat[i] = packed[i >> 4][i & 15];
      tmem_st32(tmem_s[b] + lane_base + col_base, flat);
      tc_fence_before();
      mbar_arrive(smem_u32(&bar->e_full[b]));
      TOCK(c_st, b3);
#ifdef MG_ROWS_TIMING
      if (j < 16) et[j] = clock64() - t_all;
#endif
    }
#ifdef MG_ROWS_TIMING
    if (blockIdx.x == 0 && lane == 0 && (warp == 2 || warp == 6))
    {
      printf("exp warp %d: total %lld wait_s_full %lld ld+exp %lld st %lld t0 %lld\n", warp, clock64() - t_all, w_sf, c_exp, c_st, t_all);
      if (warp == 2) for (int j = 0; j < 16 && j < F; j++) printf("  tile %2d: s_full seen %6lld  exp done %6lld  E stored %6lld\n", j, es[j], ee[j], et[j]);
    }
#endif
    // the two halves of a row add up their sums (named barrier over the 256 threads of these warps; reached
    // by all of them whether or not a wait gave up)
    bar->row_sums[half][row] = rsum;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    float const total = bar->row_sums[0][row] + bar->row_sums[1][row];
    if (ok) ok = mbar_wait(smem_u32(&bar->o_full), 0, abort_flag);
    // O' (and O'/R') leave through shared memory: a thread owns half a row, so direct stores would put 16 bytes into
    // each of 32 rows per instruction; staged in ring stage 0 (free once every MMA is done) as [128 rows][64 columns]
    // boxes with the 128-byte swizzle - one 128-byte row of a box per thread - they go out as TMA stores.
    unsigned char *const stage = smem; // [O' | O'/R'] x [column half] boxes of 16 KB
    if (ok) {
      tc_fence_after();
      float const inv = 1.0f / total;
      uint32_t const row_at = (uint32_t)(half * kSubTile + row * 128);
#pragma unroll
      for (int c = 0; c < 2; c++) {
        uint32_t v[32];
        tmem_ld32(tmem_o + lane_base + col_base + (uint32_t)(c * 32), v);
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint32_t const at = row_at + (uint32_t)((((c * 4 + q) ^ (row & 7)) << 4));
          uint4 out;
          out.x = pack2<BF16>(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1]));
          out.y = pack2<BF16>(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
          out.z = pack2<BF16>(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
          out.w = pack2<BF16>(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
          *reinterpret_cast<uint4 *>(stage + at) = out;
          if (p.o_div) {
            out.x = pack2<BF16>(__uint_as_float(v[8 * q]) * inv, __uint_as_float(v[8 * q + 1]) * inv);
            out.y = pack2<BF16>(__uint_as_float(v[8 * q + 2]) * inv, __uint_as_float(v[8 * q + 3]) * inv);
            out.z = pack2<BF16>(__uint_as_float(v[8 * q + 4]) * inv, __uint_as_float(v[8 * q + 5]) * inv);
            out.w = pack2<BF16>(__uint_as_float(v[8 * q + 6]) * inv, __uint_as_float(v[8 * q + 7]) * inv);
            *reinterpret_cast<uint4 *>(stage + kOperand + at) = out;
          }
        }
      }
      ptx::fence_proxy_async_smem(); // the staged boxes are read by the TMA engine
      if (half == 0) {
        uint32_t r2 = pack2<BF16>(total, 0.f);
        static_cast<uint16_t *>(p.r_acc)[(size_t)head * p.seq_q + q0 + row] = (uint16_t)(r2 & 0xFFFF);
      }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (warp == 2 && lane == 0 && ok && !*abort_flag) {
      uint32_t const src = smem_u32(stage);
      ptx::tma_store_3d(&o_map, src, 0, q0, head);
      ptx::tma_store_3d(&o_map, src + kSubTile, 64, q0, head);
      if (p.o_div) {
        ptx::tma_store_3d(&d_map, src + kOperand, 0, q0, head);
        ptx::tma_store_3d(&d_map, src + kOperand + kSubTile, 64, q0, head);
      }
      ptx::tma_store_commit_and_wait_read(); // the boxes must stay until the engine has read them
    }
  }

  // ---- teardown: every role arrives here, failed or not --------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && warp == 0 && lane == 0) {
    // copies this block issued may still be in flight: give them a bounded time to land before the block exits
    for (int s = 0; s < kStages; s++)
      for (int i = 0; i < 20000 && !mbar_try_wait(smem_u32(&bar->kv_full[s]), 0) && !mbar_try_wait(smem_u32(&bar->kv_full[s]), 1); i++) {
      }
    atomicExch(p.status, 2);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

using EncodeFn = TensorMapEncodeFn; // cuTensorMapEncodeTiled through the shared lookup (ptx.cuh)
static EncodeFn encode_fn() { return tensor_map_encoder(); }
// [batch][rows][cols] 16-bit array, box [1][128][64], 128-byte swizzle
static bool make_map(CUtensorMap *map, void const *base, uint64_t batch, uint64_t rows, uint64_t cols) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {cols * 2, rows * cols * 2};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool rows_supported(mgd_attn_rows const *p) {
  if (!p || p->heads <= 0 || p->forloop_range <= 0) return false;
  if (p->d != kD || p->tile_m != kM || p->tile_kv != kN) return false;
  if (p->seq_q % kM != 0 || p->kv_len != p->forloop_range * kN) return false;
  if (p->data_type != MG_DT_FLOAT16 && p->data_type != MG_DT_BFLOAT16) return false;
  // both B operands must have the contraction index contiguous: K as [kv][d], V as [d][kv]
  return p->k_layout == MG_DMEM_COLUMN_MAJOR && p->v_layout == MG_DMEM_COLUMN_MAJOR;
}
} // namespace tc
} // namespace mgk

namespace mgk {
namespace pp { // attn_rows_pp.cu: two query tiles per block, all K / V layouts
bool supported(mgd_attn_rows const *p);
int launch(mgd_attn_rows const *p, void const *q, void const *k, void const *v, void *o_acc, void *r_acc, void *o_div,
           int overlap, void *stream);
} // namespace pp
} // namespace mgk

using namespace mgk;

// MGD_OPT_ROWS_ENGINE = 1 keeps the one-tile-per-block kernel where it supports the shape (tuning, tests)
static bool use_two_tile_kernel(mgd_attn_rows const *p) {
  if (!pp::supported(p)) return false;
  if (option(MGD_OPT_ROWS_ENGINE) == 1) return !tc::rows_supported(p);
  return true;
}

extern "C" {

int mgd_attn_rows_supported(const mgd_attn_rows *p) {
  return ((tc::rows_supported(p) && tc::encode_fn() != nullptr) || pp::supported(p)) ? 1 : 0;
}

int mgd_launch_attn_rows_float(const mgd_attn_rows *p, const void *q, const void *k, const void *v, void *o_acc,
                               void *r_acc, void *stream) {
  return mgd_launch_attn_rows_float_ex(p, q, k, v, o_acc, r_acc, nullptr, stream);
}

int mgd_launch_attn_rows_float_ex(const mgd_attn_rows *p, const void *q, const void *k, const void *v, void *o_acc,
                                  void *r_acc, void *o_div, void *stream) {
  return mgd_launch_attn_rows_float_overlapped(p, q, k, v, o_acc, r_acc, o_div, 0, stream);
}

int mgd_launch_attn_rows_float_overlapped(const mgd_attn_rows *p, const void *q, const void *k, const void *v, void *o_acc,
                                          void *r_acc, void *o_div, int32_t overlap, void *stream) {
  if (!q || !k || !v || !o_acc || !r_acc) return set_error(MG_ERR_INVALID_ARGUMENT, "dense attention: null tensor");
  if (use_two_tile_kernel(p)) return pp::launch(p, q, k, v, o_acc, r_acc, o_div, overlap, stream);
  if (!tc::rows_supported(p)) return set_error(MG_ERR_UNSUPPORTED, "dense attention: shape or layout not supported");
  CUtensorMap km, vm;
  CUtensorMap om, dm; // outputs: [heads][seq_q][d], the same box geometry
  bool ok = tc::make_map(&km, k, p->heads, p->kv_len, tc::kD) && tc::make_map(&vm, v, p->heads, tc::kD, p->kv_len) &&
            tc::make_map(&om, o_acc, p->heads, p->seq_q, tc::kD) && tc::make_map(&dm, o_div ? o_div : o_acc, p->heads, p->seq_q, tc::kD);
  if (!ok) return set_error(MG_ERR_CUDA, "dense attention: cuTensorMapEncodeTiled failed");
  tc::RowsParams a;
  a.q = q; a.o_acc = o_acc; a.r_acc = r_acc; a.o_div = o_div;
  a.status = device_error_word();
  if (!a.status) return set_error(MG_ERR_CUDA, "cannot allocate the device status word");
  a.heads = p->heads; a.seq_q = p->seq_q; a.kv_len = p->kv_len; a.forloop = p->forloop_range;
  size_t smem = 1024 + tc::kOperand * (2 * tc::kStages) + sizeof(tc::Barriers) + 64;
  unsigned blocks = (unsigned)(p->heads * (p->seq_q / tc::kM));
  static bool configured[2] = {false, false};
  bool bf16 = p->data_type == MG_DT_BFLOAT16;
  if (!configured[bf16]) {
    cudaError_t e = bf16 ? cudaFuncSetAttribute(tc::attn_rows_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                         : cudaFuncSetAttribute(tc::attn_rows_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return check_launch("cudaFuncSetAttribute(attn_rows_tc_kernel)");
    configured[bf16] = true;
  }
  if (bf16) tc::attn_rows_tc_kernel<true><<<blocks, 320, smem, (cudaStream_t)stream>>>(km, vm, om, dm, a);
  else tc::attn_rows_tc_kernel<false><<<blocks, 320, smem, (cudaStream_t)stream>>>(km, vm, om, dm, a);
  return check_launch("attn_rows_tc_kernel");
}
}
