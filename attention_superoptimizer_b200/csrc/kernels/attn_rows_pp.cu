// Dense attention operator on tcgen05, two query tiles per block ("ping-pong").
//
// Same operator as attn_rows_tc.cu (first customized op of the prefill muGraph, pattern of the reference's
// cpp_examples/multi_head_attn_prefill.cc:43-98; the division that follows it can be fused in): per 128 query rows
//     S = Q K,  E = exp(S),  O' += E V,  R' += rowsum(E)        over KV tiles of 128
// One query tile alone leaves the tensor pipe idle while its exp runs and the MUFU pipe idle while its MMAs run: per
// KV tile both need about 1100 cycles (16 MMAs of 68 cycles; 16384 exps at 16 per cycle) and they depend on each
// other.  Here a block owns TWO query tiles of a head, each with its own exp warps, and one lane issues the MMAs of
// both in the order
//     S0(0) S1(0) | O0(0) S0(1) | O1(0) S1(1) | O0(1) S0(2) | ...
// so the tensor pipe works on one tile while the other tile's exp runs, and each K / V tile is fetched once for 256
// query rows.
//
// Tensor memory (all 512 columns): tile i has S_i at [128 i, 128 i + 128) and O'_i at [256 + 128 i, ...).  E of a KV
// tile overwrites its own S values (packed 16-bit pairs: the thread that read S columns [64h, 64h+64) writes E to
// [64h, 64h+32)) and is the A operand of the O' MMAs; S of the next KV tile is issued after them by the same lane, and
// MMAs of one lane execute in order.  Q stays in shared memory (A operand of the S MMAs).
// Shared memory: Q0, Q1 (32 KB each), two-slot rings of K tiles and of V tiles (32 KB per slot, a barrier pair per
// slot: a K slot is free after S1 of its tile, a V slot after O'1, each a whole round of MMAs before its next use),
// barriers.  At the end the outputs are staged in the Q buffers (tile 0) and in ring stage 0 (tile 1) as swizzled
// boxes and leave by TMA stores.
// Operand layouts: all four combinations of K and V memory order; an operand whose N index is contiguous in memory is
// described as MN-major.
//
// Warp roles (576 threads):
//   warp 0, one lane   TMA producer: Q0, K_0, Q1, V_0, K_1, then V_t and K_{t+1} as their slots come free.
//   warp 1             allocates / frees tensor memory; one lane runs the whole MMA loop and commits to mbarriers (its
//                      instruction stream sets the pace of the tensor pipe: see the comments at the loop).
//   warps 2-9          exp warps of tile 0: thread = (query row, 64-column half); tcgen05.ld its S half-row, exp, row
//   warps 10-17        sum, pack, tcgen05.st E.  Same for tile 1.  At the end: O' (and O'/R' when the division is
//                      fused) from tensor memory into the staging boxes, one thread per tile issues the TMA stores;
//                      R' by plain stores.
// Launch: with programmatic stream serialisation when the host asks for it (see the top of the kernel).
// Every wait on an mbarrier is bounded; a role that gives up raises a block-wide flag, the others stop at their next
// wait, the block frees its tensor memory, records the failure in the device status word and returns.
#include "common.cuh"
#include "tcgen05.cuh"
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <type_traits>

namespace mgk {
namespace pp {
using namespace t5;

// Optional timeline of block 0 (compile with -DMG_PP_TIMING): the MMA lane and one exp lane per query tile stamp the
// cycle counter into shared memory for a few KV tiles, thread 0 prints the stamps when the block winds down.
#ifdef MG_PP_TIMING
#define STAMP(slot) (slot) = clock64()
#else
#define STAMP(slot)
#endif

constexpr int kD = 128, kTile = 128;
constexpr int kBox = 128 * 64 * 2;   // one TMA box: 128 rows x 64 16-bit elements = 16 KB
constexpr int kOperand = 2 * kBox;   // a 128 x 128 tile
constexpr int kStages = 2;
constexpr uint32_t kTmemCols = 512;
constexpr int kThreads = 576;

struct Params {
  void *o_acc, *r_acc, *o_div;
  int32_t *status;
  int heads, seq_q, forloop;
  int overlap; // bit 0: launched with programmatic stream serialisation; bit 1: Q, K, V were not written by the kernel before
};

struct Shared {
  uint64_t q_full[2], k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages], s_full[2], e_full[2], o_full[2];
  uint32_t tmem_base;
  int abort_flag;
  float row_sums[2][2][kTile]; // [query tile][column half][row]
#ifdef MG_PP_TIMING
  long long t_block[10], t_lane[16][8], t_exp[2][16][4];
#endif
};

__device__ __forceinline__ uint32_t k_major_step(int ks) { return (uint32_t)(((ks >> 2) * kBox + (ks & 3) * 32) >> 4); }
__device__ __forceinline__ uint32_t mn_major_step(int ks) { return (uint32_t)((ks * 16 * 128) >> 4); }

// K_KV: K memory is [kv][d] (K-major B of S) else [d][kv] (MN-major); V_KV: V memory is [kv][d] (MN-major B of O')
// else [d][kv] (K-major).
template <bool BF16, bool K_KV, bool V_KV>
__global__ void __launch_bounds__(kThreads)
attn_rows_pp_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap o_map,
                    const __grid_constant__ CUtensorMap d_map, const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  // [Q0 32 KB][Q1 32 KB][stage 0: K 32 KB, V 32 KB][stage 1][barriers]
  uint32_t const q_smem = smem_u32(smem);
  uint32_t const ring = q_smem + 2 * kOperand;
  Shared *sh = reinterpret_cast<Shared *>(smem + 2 * kOperand + kStages * 2 * kOperand);
  volatile int *abort_flag = &sh->abort_flag;

  int const tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int const pairs = p.seq_q / (2 * kTile);
  int const head = blockIdx.x / pairs, q0 = (blockIdx.x % pairs) * 2 * kTile;
  int const F = p.forloop;

  // Programmatic dependent launch (both are no-ops in a plain launch).  The kernel that follows may be scheduled as
  // soon as every block of this one has released it - with 1.73 blocks per SM in the prefill configuration at once,
  // and its first blocks fill the SMs this kernel's second round leaves idle.  This kernel in turn reads Q, K and V before the
  // kernel in front of it has finished only when that kernel did not write them, and writes nothing to global
  // memory before it has finished (the exp warps wait in front of their stores).
  // The early release is only given by a grid with more blocks than SMs.  Then a kernel two launches on cannot start
  // before this one has completed: it needs every block of the kernel in between to have started, more than an SM
  // each, so some of those have exited, and a block only exits after its wait on this kernel.  The host's check of
  // the inputs (bit 1) looks at the launch directly in front and no further, which is all that can still be running.
  uint32_t sm_total;
  asm volatile("mov.u32 %0, %%nsmid;" : "=r"(sm_total));
  bool const early_release = gridDim.x > sm_total;
  if (!(p.overlap & 2)) ptx::grid_dependency_wait();
  if (early_release) ptx::grid_launch_dependents();

  if (tid == 0) {
    STAMP(sh->t_block[0]);
    sh->abort_flag = 0;
    asm volatile("prefetch.tensormap [%0];" ::"l"(&q_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&k_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&v_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&o_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&d_map) : "memory");
    mbar_init(smem_u32(&sh->q_full[0]), 1);
    mbar_init(smem_u32(&sh->q_full[1]), 1);
    for (int s = 0; s < kStages; s++) {
      mbar_init(smem_u32(&sh->k_full[s]), 1);
      mbar_init(smem_u32(&sh->k_empty[s]), 1);
      mbar_init(smem_u32(&sh->v_full[s]), 1);
      mbar_init(smem_u32(&sh->v_empty[s]), 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(smem_u32(&sh->s_full[i]), 1);
      mbar_init(smem_u32(&sh->e_full[i]), 256);
      mbar_init(smem_u32(&sh->o_full[i]), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) tmem_alloc(smem_u32(&sh->tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t const tmem = sh->tmem_base;
  if (tid == 0) STAMP(sh->t_block[1]);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // K and V tiles have rings of their own: the slot of K_j is free once S1(j) has run, the slot of V_j once O'1(j)
    // has, and both are next needed a whole round of MMAs later (K_{j+2} by S0(j+2), V_{j+2} by O'0(j+2)).
    if (lane == 0) {
      // Q memory [heads][seq_q][d]: rows = query rows, two boxes over d.  The first S needs Q0 and K_0 only, so these
      // two are asked for first: a round of blocks starts with 148 blocks fetching at once
      auto load_q = [&](int i) {
        uint32_t const full = smem_u32(&sh->q_full[i]);
        mbar_expect_tx(full, kOperand);
        tma_load_3d(q_smem + (uint32_t)(i * kOperand), &q_map, full, 0, q0 + i * kTile, head);
        tma_load_3d(q_smem + (uint32_t)(i * kOperand + kBox), &q_map, full, 64, q0 + i * kTile, head);
      };
      auto load_k = [&](int j) {
        uint32_t const bar = smem_u32(&sh->k_full[j % kStages]), dst = ring + (uint32_t)((j % kStages) * 2 * kOperand);
        int const kv0 = j * kTile;
        mbar_expect_tx(bar, kOperand);
        if (K_KV) { // rows = KV positions, boxes over d
          tma_load_3d(dst, &k_map, bar, 0, kv0, head);
          tma_load_3d(dst + kBox, &k_map, bar, 64, kv0, head);
        } else {    // rows = d, boxes over this tile's KV positions
          tma_load_3d(dst, &k_map, bar, kv0, 0, head);
          tma_load_3d(dst + kBox, &k_map, bar, kv0 + 64, 0, head);
        }
      };
      auto load_v = [&](int j) {
        uint32_t const bar = smem_u32(&sh->v_full[j % kStages]), dst = ring + (uint32_t)((j % kStages) * 2 * kOperand + kOperand);
        int const kv0 = j * kTile;
        mbar_expect_tx(bar, kOperand);
        if (V_KV) {
          tma_load_3d(dst, &v_map, bar, 0, kv0, head);
          tma_load_3d(dst + kBox, &v_map, bar, 64, kv0, head);
        } else {
          tma_load_3d(dst, &v_map, bar, kv0, 0, head);
          tma_load_3d(dst + kBox, &v_map, bar, kv0 + 64, 0, head);
        }
      };
      load_q(0);
      load_k(0);
      load_q(1);
      load_v(0);
      if (F > 1) load_k(1);
      for (int t = 1; t < F; t++) { // V_t, then K_{t+1}: the order in which their slots come free
        if (t >= kStages && !mbar_wait(smem_u32(&sh->v_empty[t % kStages]), (uint32_t)(((t / kStages) - 1) & 1), abort_flag)) break;
        load_v(t);
        if (t + 1 < F) {
          if (t + 1 >= kStages && !mbar_wait(smem_u32(&sh->k_empty[(t + 1) % kStages]), (uint32_t)((((t + 1) / kStages) - 1) & 1), abort_flag)) break;
          load_k(t + 1);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The issuing lane's instruction stream is what feeds the tensor pipe (an MMA of 128 x 128 x 16 takes the pipe
    // about 68 cycles, and the lane shares its scheduler with four exp warps), so everything an MMA needs is laid
    // out before the loop: the low descriptor words of every (tile, contraction step) of Q, of every (stage, step) of
    // K and V - a stage, a tile or a step only moves the start-address field of the low word - and the tensor-memory
    // addresses of E.  The loop body is unrolled over query tiles and ring stages, so these are plain registers.
    uint32_t const fmt = BF16 ? 1u : 0u;
    uint32_t const idesc_s = instr_desc_f16(fmt, false, !K_KV, kTile, kTile);
    uint32_t const idesc_o = instr_desc_f16(fmt, false, V_KV, kTile, kD);
    uint64_t const q_desc0 = smem_desc(q_smem, 16, 1024, 2);
    uint64_t const k_desc0 = K_KV ? smem_desc(ring, 16, 1024, 2) : smem_desc(ring, kBox, 1024, 2);
    uint64_t const v_desc0 = V_KV ? smem_desc(ring + kOperand, kBox, 1024, 2) : smem_desc(ring + kOperand, 16, 1024, 2);
    uint32_t const q_hi = (uint32_t)(q_desc0 >> 32), k_hi = (uint32_t)(k_desc0 >> 32), v_hi = (uint32_t)(v_desc0 >> 32);
    constexpr int kSteps = kD / 16; // contraction steps of either product (kD = kTile)
    uint32_t q_lo[2][kSteps], k_lo[kStages][kSteps], v_lo[kStages][kSteps], e_at[2][kSteps];
#pragma unroll
    for (int x = 0; x < 2; x++)
#pragma unroll
      for (int ks = 0; ks < kSteps; ks++) {
        q_lo[x][ks] = (uint32_t)q_desc0 + (uint32_t)((x * kOperand) >> 4) + k_major_step(ks);
        k_lo[x][ks] = (uint32_t)k_desc0 + (uint32_t)((x * 2 * kOperand) >> 4) + (K_KV ? k_major_step(ks) : mn_major_step(ks));
        v_lo[x][ks] = (uint32_t)v_desc0 + (uint32_t)((x * 2 * kOperand) >> 4) + (V_KV ? mn_major_step(ks) : k_major_step(ks));
        e_at[x][ks] = tmem + (uint32_t)(x * kTile) + (uint32_t)((ks >> 2) * 64 + (ks & 3) * 8); // half h at [64h, 64h+32), 8 per step
      }
    // One lane runs the whole loop.  An instruction of that lane that needs an answer from shared memory (a barrier
    // test) gets it only after the MMAs issued before it have been handed to the tensor pipe, and the pipe queues
    // little by itself: a test between two batches of MMAs leaves the pipe idle.  So what the next batch will wait
    // for is tested `kProbeAt` MMAs into the S batch before it, and the wait in front of a batch is only taken when
    // that test failed.  Tests and waits are `mbarrier.test_wait` polls: `try_wait` parks a thread whose phase is not
    // complete, and a parked lane came back about 500 cycles after the phase had completed.
    constexpr int kProbeAt = 5;
    if (lane == 0) {
      bool e_known = false, v_known = false, k_known = false; // barriers of the coming batches already seen complete
      // S_I(j) = Q_I K_j with K_j in stage ST, contraction steps [ks0, ks1); the last part commits to s_full
      auto issue_s = [&](auto I, auto ST, int ks0, int ks1) {
        constexpr int i = decltype(I)::value, st = decltype(ST)::value;
#pragma unroll
        for (int ks = ks0; ks < ks1; ks++)
          umma_f16_halves(tmem + (uint32_t)(i * kTile), q_lo[i][ks], q_hi, k_lo[st][ks], k_hi, idesc_s, ks > 0);
        if (ks1 == kSteps) umma_commit(smem_u32(&sh->s_full[i]));
      };
      // One batch: O'_I += E_I(j) V_j (V_j in stage ST), then S_I(j+1) (K_{j+1} in the other stage)
      auto batch = [&](auto I, auto ST, int j) -> bool {
        constexpr int i = decltype(I)::value, st = decltype(ST)::value;
        if (!e_known && !mbar_spin_or_abort(smem_u32(&sh->e_full[i]), (uint32_t)(j & 1), abort_flag)) return false;
        if (i == 0 && !v_known && !mbar_spin_or_abort(smem_u32(&sh->v_full[st]), (uint32_t)((j / kStages) & 1), abort_flag)) return false;
#ifdef MG_PP_TIMING
        if (j < 16) STAMP(sh->t_lane[j][i * 4 + 0]);
#endif
        tc_fence_after();
        uint32_t const first = j > 0 ? 1u : 0u;
#pragma unroll
        for (int ks = 0; ks < kSteps; ks++)
          umma_f16_ts_halves(tmem + 256 + (uint32_t)(i * kTile), e_at[i][ks], v_lo[st][ks], v_hi, idesc_o, ks > 0 ? 1u : first);
        if (i == 1) umma_commit(smem_u32(&sh->v_empty[st])); // V_j consumed by both query tiles
        if (j == F - 1) umma_commit(smem_u32(&sh->o_full[i]));
#ifdef MG_PP_TIMING
        if (j < 16) STAMP(sh->t_lane[j][i * 4 + 1]);
#endif
        e_known = false;
        if (j + 1 < F) {
          if (i == 0 && !k_known && !mbar_spin_or_abort(smem_u32(&sh->k_full[st ^ 1]), (uint32_t)(((j + 1) / kStages) & 1), abort_flag)) return false;
#ifdef MG_PP_TIMING
          if (j < 16) STAMP(sh->t_lane[j][i * 4 + 2]);
#endif
          issue_s(I, std::integral_constant<int, (st ^ 1)>{}, 0, kProbeAt);
          if (i == 0) { // next batch: O'1(j), S1(j+1)
            e_known = mbar_test_wait(smem_u32(&sh->e_full[1]), (uint32_t)(j & 1));
          } else {      // next batch: O'0(j+1), S0(j+2); K_{j+2} comes into stage ST (K_{j+1} stands in when there is none)
            bool const more = j + 2 < F;
            uint32_t const seen = mbar_test_wait3(smem_u32(&sh->e_full[0]), (uint32_t)((j + 1) & 1),
                                                  smem_u32(&sh->v_full[st ^ 1]), (uint32_t)(((j + 1) / kStages) & 1),
                                                  smem_u32(&sh->k_full[more ? st : (st ^ 1)]), (uint32_t)((((more ? j + 2 : j + 1)) / kStages) & 1));
            e_known = seen & 1; v_known = seen & 2; k_known = seen & 4;
          }
          issue_s(I, std::integral_constant<int, (st ^ 1)>{}, kProbeAt, kSteps);
          if (i == 1) umma_commit(smem_u32(&sh->k_empty[st ^ 1])); // K_{j+1} consumed by both query tiles
        }
#ifdef MG_PP_TIMING
        if (j < 16) STAMP(sh->t_lane[j][i * 4 + 3]);
#endif
        return true;
      };
      std::integral_constant<int, 0> const c0{};
      std::integral_constant<int, 1> const c1{};
      bool ok = mbar_spin_or_abort(smem_u32(&sh->q_full[0]), 0, abort_flag);
      STAMP(sh->t_block[2]);
      if (ok) ok = mbar_spin_or_abort(smem_u32(&sh->k_full[0]), 0, abort_flag);
      STAMP(sh->t_block[3]);
      if (ok) {
        tc_fence_after();
        issue_s(c0, c0, 0, kSteps);
        ok = mbar_spin_or_abort(smem_u32(&sh->q_full[1]), 0, abort_flag);
      }
      if (ok) {
        tc_fence_after();
        issue_s(c1, c0, 0, kSteps);
        umma_commit(smem_u32(&sh->k_empty[0]));
      }
      STAMP(sh->t_block[4]);
      for (int j = 0; j < F && ok; j += 2) {
        ok = batch(c0, c0, j) && batch(c1, c0, j);
        if (ok && j + 1 < F) ok = batch(c0, c1, j + 1) && batch(c1, c1, j + 1);
      }
      STAMP(sh->t_block[5]);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ exp / row sums / epilogue of one query tile
    int const i = (warp - 2) >> 3;                // query tile of this warp
    int const wi = (warp - 2) & 7;                // warp inside the tile's group
    int const quarter = warp & 3;                 // tensor-memory lanes this warp may touch: 32 * (warp % 4)
    int const half = wi >> 2;                     // which 64 columns of a KV tile
    int const row = quarter * 32 + lane;
    uint32_t const lane_base = (uint32_t)(quarter * 32) << 16;
    uint32_t const s_tmem = tmem + (uint32_t)(i * kTile) + lane_base + (uint32_t)(half * 64);
    float rsum = 0.f;
    bool ok = true;
    for (int j = 0; j < F && ok; j++) {
      ok = mbar_wait(smem_u32(&sh->s_full[i]), (uint32_t)(j & 1), abort_flag);
      if (!ok) break;
#ifdef MG_PP_TIMING
      bool const stamps = lane == 0 && wi == 0 && j < 16;
      if (stamps) STAMP(sh->t_exp[i][j][0]);
#endif
      tc_fence_after();
      uint32_t flat[32]; // this thread's 64 values as 16-bit pairs
      {
        uint32_t v[64];
        tmem_ld64(s_tmem, v); // one load, one wait: the tensor-memory latency is paid once per tile
#ifdef MG_PP_TIMING
        if (stamps) STAMP(sh->t_exp[i][j][1]);
#endif
        uint64_t sum2 = 0; // packed arithmetic: the exp warps share their schedulers with the MMA-issuing lane
#pragma unroll
        for (int x = 0; x < 64; x += 2) {
          float e0, e1;
          exp_ftz2(pair(__uint_as_float(v[x]), __uint_as_float(v[x + 1])), e0, e1);
          sum2 = add2(sum2, pair(e0, e1));
          flat[x >> 1] = pack2<BF16>(e0, e1);
        }
        float s0, s1;
        unpair(sum2, s0, s1);
        rsum += s0 + s1;
#ifdef MG_PP_TIMING
        if (stamps) STAMP(sh->t_exp[i][j][2]);
#endif
      }
      // E replaces the S values this thread has just consumed: 32 packed columns at the start of its own half
      tmem_st32(s_tmem, flat);
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->e_full[i]));
#ifdef MG_PP_TIMING
      if (stamps) STAMP(sh->t_exp[i][j][3]);
#endif
    }
    // the two halves of a row add up their sums (named barrier per query tile, reached whether or not a wait gave up)
    sh->row_sums[i][half][row] = rsum;
    if (i == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
    else asm volatile("bar.sync 2, 256;" ::: "memory");
    float const total = sh->row_sums[i][0][row] + sh->row_sums[i][1][row];
    if (tid == 64) STAMP(sh->t_block[6]);
    if (ok) ok = mbar_wait(smem_u32(&sh->o_full[i]), 0, abort_flag);
    if (tid == 64) STAMP(sh->t_block[7]);
    ptx::grid_dependency_wait(); // the kernel in front may still be writing these outputs (a replay of the same graph)
    if (!early_release) ptx::grid_launch_dependents();
    // O' (and O'/R') leave through shared memory: a thread owns half a row, so direct stores would put 16 bytes into
    // each of 32 rows per instruction; staged as [128 rows][64 columns] boxes (128-byte swizzle, one 128-byte row of a
    // box per thread) they go out as four TMA stores per tile.  Tile 0 stages into the Q buffers - both last read by
    // S1(F-1), which the pipe finished before O'0(F-1) - and tile 1 into ring stage 0, free once every MMA is done.
    unsigned char *const stage = smem + (i == 0 ? 0 : 2 * kOperand); // [O' | O'/R'] x [column half] boxes of 16 KB
    if (ok) {
      tc_fence_after();
      float const inv = 1.0f / total;
      uint32_t const row_at = (uint32_t)(half * kBox + row * 128);
#pragma unroll
      for (int c = 0; c < 2; c++) {
        uint32_t v[32];
        tmem_ld32(tmem + 256 + (uint32_t)(i * kTile) + lane_base + (uint32_t)(half * 64 + c * 32), v);
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
      fence_proxy_async_smem(); // the staged boxes are read by the TMA engine
      if (half == 0)
        static_cast<uint16_t *>(p.r_acc)[(size_t)head * p.seq_q + q0 + i * kTile + row] = (uint16_t)(pack2<BF16>(total, 0.f) & 0xFFFFu);
    }
    if (i == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
    else asm volatile("bar.sync 2, 256;" ::: "memory");
    if (wi == 0 && lane == 0 && ok && !*abort_flag) {
      uint32_t const src = smem_u32(stage);
      int const r0 = q0 + i * kTile;
      ptx::tma_store_3d(&o_map, src, 0, r0, head);
      ptx::tma_store_3d(&o_map, src + kBox, 64, r0, head);
      if (p.o_div) {
        ptx::tma_store_3d(&d_map, src + kOperand, 0, r0, head);
        ptx::tma_store_3d(&d_map, src + kOperand + kBox, 64, r0, head);
      }
      ptx::tma_store_commit_and_wait_read(); // the boxes must stay until the engine has read them
    }
  }

  // ---- teardown: every role arrives here, failed or not --------------------------------------------------
  if (tid == 64) STAMP(sh->t_block[8]);
  tc_fence_before();
  __syncthreads();
#ifdef MG_PP_TIMING
  if (blockIdx.x == 0 && tid == 0) {
    long long const tb = sh->t_block[0];
    printf("block 0: tensor memory %lld q_full %lld k_full0 %lld S(0) issued %lld lane loop end %lld | exp: loop end %lld o_full %lld stores done %lld\n",
           sh->t_block[1] - tb, sh->t_block[2] - tb, sh->t_block[3] - tb, sh->t_block[4] - tb, sh->t_block[5] - tb,
           sh->t_block[6] - tb, sh->t_block[7] - tb, sh->t_block[8] - tb);
    for (int j = 4; j < 8 && j < F - 1; j++) {
      long long const *l = sh->t_lane[j];
      printf("  j=%d lane: waits0 %lld O0 %lld k %lld S0 %lld | waits1 %lld O1 %lld - %lld S1 %lld\n", j, l[0] - tb, l[1] - tb, l[2] - tb,
             l[3] - tb, l[4] - tb, l[5] - tb, l[6] - tb, l[7] - tb);
      for (int i = 0; i < 2; i++)
        printf("      exp%d: s_full %lld ld %lld exp %lld arrive %lld\n", i, sh->t_exp[i][j][0] - tb, sh->t_exp[i][j][1] - tb,
               sh->t_exp[i][j][2] - tb, sh->t_exp[i][j][3] - tb);
    }
  }
#endif
  if (*abort_flag && tid == 0) {
    // copies this block issued may still be in flight: give them a bounded time to land before the block exits
    for (int s = 0; s < kStages; s++) {
      for (int n = 0; n < 20000 && !mbar_try_wait(smem_u32(&sh->k_full[s]), 0) && !mbar_try_wait(smem_u32(&sh->k_full[s]), 1); n++) {
      }
      for (int n = 0; n < 20000 && !mbar_try_wait(smem_u32(&sh->v_full[s]), 0) && !mbar_try_wait(smem_u32(&sh->v_full[s]), 1); n++) {
      }
    }
    ptx::grid_dependency_wait();
    atomicExch(p.status, 4);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ---- host side ------------------------------------------------------------------------------------------------
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

bool supported(mgd_attn_rows const *p) {
  if (!p || p->heads <= 0 || p->forloop_range <= 0) return false;
  if (p->d != kD || p->tile_m != kTile || p->tile_kv != kTile) return false;
  if (p->seq_q % (2 * kTile) != 0 || p->kv_len != p->forloop_range * kTile) return false;
  if (p->data_type != MG_DT_FLOAT16 && p->data_type != MG_DT_BFLOAT16) return false;
  if ((int64_t)p->heads * (p->seq_q / (2 * kTile)) > 0x7fffffffLL) return false;
  return encode_fn() != nullptr;
}

int launch(mgd_attn_rows const *p, void const *q, void const *k, void const *v, void *o_acc, void *r_acc, void *o_div,
           int overlap, void *stream) {
  if (!supported(p)) return set_error(MG_ERR_UNSUPPORTED, "dense attention (two query tiles per block): shape not supported");
  bool const k_kv = p->k_layout == MG_DMEM_COLUMN_MAJOR, v_kv = p->v_layout == MG_DMEM_ROW_MAJOR;
  CUtensorMap qm, km, vm, om, dm;
  bool ok = make_map(&qm, q, p->heads, p->seq_q, kD) && make_map(&om, o_acc, p->heads, p->seq_q, kD) &&
            make_map(&dm, o_div ? o_div : o_acc, p->heads, p->seq_q, kD);
  ok = ok && (k_kv ? make_map(&km, k, p->heads, p->kv_len, kD) : make_map(&km, k, p->heads, kD, p->kv_len));
  ok = ok && (v_kv ? make_map(&vm, v, p->heads, p->kv_len, kD) : make_map(&vm, v, p->heads, kD, p->kv_len));
  if (!ok) return set_error(MG_ERR_CUDA, "dense attention: cuTensorMapEncodeTiled failed");
  Params a;
  a.o_acc = o_acc; a.r_acc = r_acc; a.o_div = o_div;
  a.status = device_error_word();
  if (!a.status) return set_error(MG_ERR_CUDA, "cannot allocate the device status word");
  a.heads = p->heads; a.seq_q = p->seq_q; a.forloop = p->forloop_range;
  a.overlap = (overlap & 1) ? (overlap & 3) : 0;
  size_t const smem = 1024 + (size_t)(2 + 2 * kStages) * kOperand + sizeof(Shared) + 64;
  unsigned const blocks = (unsigned)(p->heads * (p->seq_q / (2 * kTile)));
  bool const bf16 = p->data_type == MG_DT_BFLOAT16;
  using Kernel = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, Params);
  static Kernel const kernels[8] = {
      attn_rows_pp_kernel<false, false, false>, attn_rows_pp_kernel<false, false, true>,
      attn_rows_pp_kernel<false, true, false>,  attn_rows_pp_kernel<false, true, true>,
      attn_rows_pp_kernel<true, false, false>,  attn_rows_pp_kernel<true, false, true>,
      attn_rows_pp_kernel<true, true, false>,   attn_rows_pp_kernel<true, true, true>};
  static bool configured[8] = {false, false, false, false, false, false, false, false};
  int const which = (bf16 ? 4 : 0) | (k_kv ? 2 : 0) | (v_kv ? 1 : 0);
  if (!configured[which]) {
    if (cudaFuncSetAttribute(kernels[which], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return check_launch("cudaFuncSetAttribute(attn_rows_pp_kernel)");
    configured[which] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (a.overlap & 1) {
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaLaunchKernelEx(&cfg, kernels[which], qm, km, vm, om, dm, a);
  return check_launch("attn_rows_pp_kernel");
}

} // namespace pp
} // namespace mgk
