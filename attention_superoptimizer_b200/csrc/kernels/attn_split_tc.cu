// Split-KV attention operator on the 5th-generation tensor cores, for more query rows than a decode step has:
// speculative decode and grouped-query attention with wide groups (8 < rows <= 32 per KV head).
//
// Same operator as attn_split.cu (first customized op of the grouped-query decode muGraph, pattern of the
// reference's cpp_examples/group_query_attn_inc_decode.cc:43-98): per (head, KV split)
//     S = Q K,  E = exp(S),  O' = sum over tiles E V,  R' = sum over tiles rowsum(E)
// With few query rows the natural M = rows form would leave the 128-row MMA almost empty (and the mma.sync form is
// bound by the legacy tensor pipe), so both products are computed transposed and the KV axis (or the head
// dimension) takes the 128 MMA rows:
//     S^T [128 kv x 32 q] = K_tile [128 kv x 128 d] * Q^T            tcgen05.mma M=128 N=32 K=16, 8 per tile
//     O^T [128 d  x 32 q] += V_tile^T [128 d x 128 kv] * E^T         tcgen05.mma M=128 N=32 K=16, 8 per tile
// Query rows are padded to 32 with zero rows (TMA fills rows past the tensor's extent with zeros); the padded
// columns are computed and never stored.  A and B come from shared memory: K and V tiles as TMA wrote them
// (128-byte swizzle; an operand whose MMA row index is contiguous in memory is described as MN-major instead of
// being transposed), Q as a K-major B operand, E^T as an MN-major B operand the exp warps write themselves
// (64-byte swizzle).  Accumulators live in tensor memory: S^T double buffered, O^T double buffered so that the
// epilogue of one work item overlaps the next item's tiles.
//
// The kernel is persistent: one block per SM walks the work items (input set, head, split) round robin.  Every
// role walks the block's tiles as one flat sequence, so nothing drains at an item boundary: the TMA producer runs
// ahead into the next item's tiles, S^T of an item's first tile is issued before O^T of the previous item's last.
//
// Warp roles (352 threads):
//   warp 0, one lane   TMA producer: Q of each item, K and V tiles into a ring of three 64 KB stages (K 32 KB and
//                      V 32 KB, each on its own barrier).
//   warp 1             allocates / frees tensor memory; one lane issues the S^T MMAs.
//   warp 10            one lane issues the O^T MMAs.  An MMA occupies its issuing lane for about as long as the
//                      tensor pipe works on it, so the two products have a lane each: S^T of the next tile is
//                      issued while O^T of the previous one is still being issued.
//   warps 2-5          one thread per KV position of a tile: tcgen05.ld its S^T row (32 query columns), exp, causal
//                      mask, per-thread row sums, pack to 16 bits, store its E^T row into the swizzled operand
//                      buffer.  After an item's last tile the row sums are reduced over each warp's 32 lanes and
//                      handed over in shared memory.
//   warps 6-9          epilogue, off the tile pipeline: add the four warps' row sums, read O^T (one thread per
//                      head-dim index), store the split's partial output.  (The cross-split merge is a second,
//                      small kernel launched right behind this one.)
// Every wait on an mbarrier is bounded; a role that gives up raises a block-wide flag, the others stop at their
// next wait, the block frees its tensor memory, records the failure in the device status word and returns.
#include "common.cuh"
#include "tcgen05.cuh"
#include "attn_merge.cuh"
#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace mgk {
namespace stc {
using namespace t5;

// Optional role timing (compile with -DMG_STC_TIMING; a few blocks print cycle totals from the device).
#ifdef MG_STC_TIMING
#define TICK(var) long long var = clock64()
#define TOCK(acc, var) acc += clock64() - var
#define TDECL(...) long long __VA_ARGS__
#define TPRINT(...) if (blockIdx.x == 0 || blockIdx.x == 100) printf(__VA_ARGS__)
#else
#define TICK(var)
#define TOCK(acc, var)
#define TDECL(...)
#define TPRINT(...)
#endif

constexpr int kD = 128;            // head dimension
constexpr int kTileKv = 128;       // KV positions per MMA tile (two for-loop tiles of the plan)
constexpr int kNQ = 32;            // query columns of the MMAs (rows of the operator, padded)
constexpr int kBox = 128 * 64 * 2; // one TMA box: 128 rows x 64 16-bit elements = 16 KB
constexpr int kOperand = 2 * kBox; // a 128 x 128 tile
constexpr int kStages = 3;
constexpr int kQBytes = 2 * kNQ * 128;     // Q: two boxes [32 rows][64 d]
constexpr int kEBytes = kTileKv * kNQ * 2; // E^T: [128 kv][32 q]
constexpr uint32_t kTmemCols = 128;        // S^T x2, O^T x2, 32 columns each
constexpr int kThreads = 352;

// Position in a block's flat tile sequence, advanced without divisions.  The block's tiles are consecutive tiles of
// the launch (item-major, so consecutive tiles of a head are consecutive KV positions).  A *run* is a stretch of
// them that is summed into one accumulator: one item, or - when the partials are scratch - every tile of a head that
// the block holds.  `period` = tiles per item, or per head in the second case; `pos` / `unit` = the tile's index in
// its period and the period's number (item, or (set, head)).  n = tile number in the block, ri = run number in the
// block, s / wraps = ring stage and how often the ring has wrapped (its low bit is the stage barriers' phase).
struct TileCursor {
  int n = 0, pos = 0, unit = 0, ri = 0, s = 0, wraps = 0;
  __device__ __forceinline__ void start(uint32_t first_tile, int period) {
    unit = (int)(first_tile / (uint32_t)period);
    pos = (int)(first_tile - (uint32_t)unit * (uint32_t)period);
  }
  __device__ __forceinline__ bool first() const { return n == 0 || pos == 0; }
  __device__ __forceinline__ bool last(int total, int period) const { return n == total - 1 || pos == period - 1; }
  __device__ __forceinline__ void advance(int total, int period) {
    if (last(total, period)) ri++;
    n++;
    if (++pos == period) { pos = 0; unit++; }
    if (++s == kStages) { s = 0; wraps++; }
  }
};

// start-address steps (16-byte units) of one K step of an MMA: 16 elements along a 128-byte swizzled row for a
// K-major operand, 16 rows of 128 bytes for an MN-major one
__device__ __forceinline__ uint64_t k_major_step(int ks) { return (uint64_t)(((ks >> 2) * kBox + (ks & 3) * 32) >> 4); }
__device__ __forceinline__ uint64_t mn_major_step(int ks) { return (uint64_t)((ks * 16 * 128) >> 4); }

struct Params {
  void *o_part, *r_part;
  int32_t *status;
  long long o_set_stride, r_set_stride;
  int heads, m, splits, tiles, kv_len, causal_window, num_items;
  int early_loads; // the inputs were not written by the previous kernel of the stream: load before waiting for it
  // Work split: the launch's tiles are dealt in granules (an item's tiles, or single tiles when runs are summed) -
  // block b takes `per` granules, the first `extra` blocks one more.
  int sum_runs;    // the partials are scratch: a block sums every tile of a head it holds and writes one partial per run,
                   // into slot (block - block that holds the head's first tile)
  uint32_t per, extra;
};

// the block that holds tile g of the launch (granule = tiles per granule)
__device__ __forceinline__ uint32_t block_of_tile(uint32_t g, uint32_t granule, uint32_t per, uint32_t extra) {
  uint32_t const q = g / granule, wide = extra * (per + 1);
  return q < wide ? q / (per + 1) : extra + (q - wide) / per;
}

struct Shared {
  uint64_t k_full[kStages], v_full[kStages], kv_empty[kStages];
  uint64_t q_full[2], q_empty[2], s_full[2], e_full[2], e_free[2], o_full[2], o_free[2], r_full[2], r_free[2];
  uint32_t tmem_base;
  int abort_flag;

  float rsum[2][4][kNQ]; // [item parity][exp warp][query column]
};

// K_KV: K memory is [kv][d] (K-major A of S^T) else [d][kv] (MN-major); V_KV: V memory is [kv][d] (MN-major A of
// O^T) else [d][kv] (K-major).  Compile-time so that the issuing lane's descriptors are constants plus one add.
template <bool BF16, bool K_KV, bool V_KV>
__global__ void __launch_bounds__(kThreads)
attn_split_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                     const __grid_constant__ CUtensorMap v_map, const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  // [ring: kStages x (K 32 KB, V 32 KB)][Q x2][E^T x2][barriers]
  uint32_t const ring = smem_u32(smem);
  uint32_t const q_smem = ring + kStages * 2 * kOperand;
  uint32_t const e_smem = q_smem + 2 * kQBytes;
  unsigned char *e_ptr = smem + kStages * 2 * kOperand + 2 * kQBytes;
  Shared *sh = reinterpret_cast<Shared *>(e_ptr + 2 * kEBytes);
  volatile int *abort_flag = &sh->abort_flag;

  int const tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef MG_STC_TIMING
  unsigned long long gt_entry;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt_entry));
#endif

  if (tid == 0) {
    sh->abort_flag = 0;
    asm volatile("prefetch.tensormap [%0];" ::"l"(&q_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&k_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&v_map) : "memory");
    for (int s = 0; s < kStages; s++) {
      mbar_init(smem_u32(&sh->k_full[s]), 1);
      mbar_init(smem_u32(&sh->v_full[s]), 1);
      mbar_init(smem_u32(&sh->kv_empty[s]), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(smem_u32(&sh->q_full[b]), 1);
      mbar_init(smem_u32(&sh->q_empty[b]), 1);
      mbar_init(smem_u32(&sh->s_full[b]), 1);
      mbar_init(smem_u32(&sh->e_full[b]), 128);
      mbar_init(smem_u32(&sh->e_free[b]), 1);
      mbar_init(smem_u32(&sh->o_full[b]), 1);
      mbar_init(smem_u32(&sh->o_free[b]), 128);
      mbar_init(smem_u32(&sh->r_full[b]), 128);
      mbar_init(smem_u32(&sh->r_free[b]), 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) tmem_alloc(smem_u32(&sh->tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t const tmem = sh->tmem_base;
  int const T = p.tiles;
  // a kernel launched behind this one with programmatic serialisation (the merge) may be scheduled from now on;
  // it still waits for this grid to complete before it reads anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // this block's tiles: granules [b * per + min(b, extra), + per (+ 1)) of the launch
  uint32_t const granule = p.sum_runs ? 1u : (uint32_t)T;
  uint32_t const first_tile = (blockIdx.x * p.per + (blockIdx.x < p.extra ? blockIdx.x : p.extra)) * granule;
  int const total = (int)((p.per + (blockIdx.x < p.extra ? 1u : 0u)) * granule);
  int const period = p.sum_runs ? p.splits * T : T;  // tiles of a run's period: a head, or an item
  int const parts = p.sum_runs ? 1 : p.splits;       // periods per (set, head)
  // period number -> (set, head), one coordinate of the tensor maps; tile -> first KV position
  auto batch_of = [&](int unit) { return unit / parts; };
  auto kv_of = [&](int unit, int pos) { return ((unit % parts) * period + pos) * kTileKv; };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    bool ok = true;
    TDECL(w_e = 0, t0 = clock64());
    TileCursor c;
    c.start(first_tile, period);
    if (!p.early_loads) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int n = 0; n < total && ok; n++, c.advance(total, period)) {
      int const batch = batch_of(c.unit);
      if (c.first()) { // a new run: its Q
        int const ri = c.ri, qb = ri & 1;
        if (ri >= 2) ok = mbar_wait(smem_u32(&sh->q_empty[qb]), (uint32_t)(((ri >> 1) - 1) & 1), abort_flag);
        if (!ok) break;
        if (lane == 0) {
          uint32_t full = smem_u32(&sh->q_full[qb]), dst = q_smem + (uint32_t)(qb * kQBytes);
          mbar_expect_tx(full, kQBytes);
          tma_load_3d(dst, &q_map, full, 0, 0, batch);
          tma_load_3d(dst + kQBytes / 2, &q_map, full, 64, 0, batch);
        }
      }
      int const s = c.s, kv0 = kv_of(c.unit, c.pos);
      TICK(a0);
      if (n >= kStages) ok = mbar_wait(smem_u32(&sh->kv_empty[s]), (uint32_t)((c.wraps - 1) & 1), abort_flag);
      TOCK(w_e, a0);
      if (!ok) break;
      if (lane == 0) {
        uint32_t kdst = ring + (uint32_t)(s * 2 * kOperand), vdst = kdst + kOperand;
        uint32_t kf = smem_u32(&sh->k_full[s]), vf = smem_u32(&sh->v_full[s]);
        mbar_expect_tx(kf, kOperand);
        if (K_KV) { // rows = KV positions, boxes over d
          tma_load_3d(kdst, &k_map, kf, 0, kv0, batch);
          tma_load_3d(kdst + kBox, &k_map, kf, 64, kv0, batch);
        } else {               // rows = d, boxes over this tile's KV positions
          tma_load_3d(kdst, &k_map, kf, kv0, 0, batch);
          tma_load_3d(kdst + kBox, &k_map, kf, kv0 + 64, 0, batch);
        }
        mbar_expect_tx(vf, kOperand);
        if (V_KV) {
          tma_load_3d(vdst, &v_map, vf, 0, kv0, batch);
          tma_load_3d(vdst + kBox, &v_map, vf, 64, kv0, batch);
        } else {
          tma_load_3d(vdst, &v_map, vf, kv0, 0, batch);
          tma_load_3d(vdst + kBox, &v_map, vf, kv0 + 64, 0, batch);
        }
      }
      __syncwarp();
    }
    if (lane == 0) TPRINT("[%d] producer: total %lld wait kv_empty %lld tiles %d\n", (int)blockIdx.x, clock64() - t0, w_e, total);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer, S^T(n) = K_n Q^T
    // Descriptors of stage 0 / buffer 0; a stage, a buffer or a K step only moves the start-address field, so the
    // issuing lane pays one 64-bit add per operand and MMA (a lone lane runs its instructions back to back).
    uint32_t const idesc_s = instr_desc_f16(BF16 ? 1u : 0u, !K_KV, false, 128, kNQ);
    uint64_t const k_desc0 = K_KV ? smem_desc(ring, 16, 1024, 2) : smem_desc(ring, kBox, 1024, 2);
    uint64_t const q_desc0 = smem_desc(q_smem, 16, 1024, 2);
    bool ok = true;
    TDECL(w_q = 0, w_k = 0, w_ef = 0, c_s = 0, c_lat = 0, t0 = clock64());
    TileCursor c;
    c.start(first_tile, period);
    for (int n = 0; n < total && ok; n++, c.advance(total, period)) {
      int const ri = c.ri, qb = ri & 1, s = c.s, b = n & 1;
      TICK(a0);
      if (c.first()) ok = mbar_wait(smem_u32(&sh->q_full[qb]), (uint32_t)((ri >> 1) & 1), abort_flag);
      TOCK(w_q, a0);
      TICK(a1);
      if (ok) ok = mbar_wait(smem_u32(&sh->k_full[s]), (uint32_t)(c.wraps & 1), abort_flag);
      TOCK(w_k, a1);
      TICK(a2);
      // S buffer b still holds tile n - 2 until the exp warps have read it
      if (ok && n >= 2) ok = mbar_wait(smem_u32(&sh->e_full[b]), (uint32_t)(((n >> 1) - 1) & 1), abort_flag);
      TOCK(w_ef, a2);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        uint64_t const kd = k_desc0 + (uint64_t)((s * 2 * kOperand) >> 4), qd = q_desc0 + (uint64_t)((qb * kQBytes) >> 4);
        uint32_t const tmem_s = tmem + (uint32_t)(b * kNQ);
        TICK(i0);
#pragma unroll
        for (int ks = 0; ks < kD / 16; ks++) {
          uint64_t const a = kd + (K_KV ? k_major_step(ks) : mn_major_step(ks));
          uint64_t const bq = qd + (uint64_t)(((ks >> 2) * (kQBytes / 2) + (ks & 3) * 32) >> 4);
          umma_f16(tmem_s, a, bq, idesc_s, ks > 0);
        }
        umma_commit(smem_u32(&sh->s_full[b]));
        if (c.last(total, period)) umma_commit(smem_u32(&sh->q_empty[qb])); // the run's last use of its Q
        TOCK(c_s, i0);
#ifdef MG_STC_TIMING
        for (int i = 0; i < 100000 && !mbar_try_wait(smem_u32(&sh->s_full[b]), (uint32_t)((n >> 1) & 1)); i++) {
        }
        TOCK(c_lat, i0);
#endif
      }
      __syncwarp();
    }
    if (lane == 0) TPRINT("[%d] mma S: total %lld wait q_full %lld k_full %lld e_full %lld | issue+commit %lld issue->s_full seen %lld\n", (int)blockIdx.x, clock64() - t0, w_q, w_k, w_ef, c_s, c_lat);
  } else if (warp == 10) {
    // ------------------------------------------------------------------ MMA issuer, O^T += V_t^T E_t^T
    uint32_t const idesc_o = instr_desc_f16(BF16 ? 1u : 0u, V_KV, true, 128, kNQ);
    uint64_t const v_desc0 = V_KV ? smem_desc(ring + kOperand, kBox, 1024, 2) : smem_desc(ring + kOperand, 16, 1024, 2);
    uint64_t const e_desc0 = smem_desc(e_smem, 512, 512, 4);
    bool ok = true;
    TDECL(w_of = 0, w_ef = 0, w_v = 0, c_o = 0, t0 = clock64());
    TileCursor c;
    c.start(first_tile, period);
    for (int t = 0; t < total && ok; t++, c.advance(total, period)) {
      int const ri = c.ri, ob = ri & 1, s = c.s, eb = t & 1;
      bool const run_begins = c.first();
      TICK(a2);
      if (run_begins && ri >= 2) ok = mbar_wait(smem_u32(&sh->o_free[ob]), (uint32_t)(((ri >> 1) - 1) & 1), abort_flag);
      TOCK(w_of, a2);
      TICK(a3);
      if (ok) ok = mbar_wait(smem_u32(&sh->e_full[eb]), (uint32_t)((t >> 1) & 1), abort_flag);
      TOCK(w_ef, a3);
      TICK(a4);
      if (ok) ok = mbar_wait(smem_u32(&sh->v_full[s]), (uint32_t)(c.wraps & 1), abort_flag);
      TOCK(w_v, a4);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        uint64_t const vd = v_desc0 + (uint64_t)((s * 2 * kOperand) >> 4), ed = e_desc0 + (uint64_t)((eb * kEBytes) >> 4);
        uint32_t const tmem_o = tmem + 64 + (uint32_t)(ob * kNQ);
        TICK(i2);
#pragma unroll
        for (int ks = 0; ks < kTileKv / 16; ks++) {
          uint64_t const a = vd + (V_KV ? mn_major_step(ks) : k_major_step(ks));
          uint64_t const be = ed + (uint64_t)((ks * 16 * 64) >> 4);
          umma_f16(tmem_o, a, be, idesc_o, (!run_begins || ks > 0) ? 1u : 0u);
        }
        // S^T of this tile completed before its E^T existed, so K_t and V_t are both consumed now
        umma_commit(smem_u32(&sh->kv_empty[s]));
        umma_commit(smem_u32(&sh->e_free[eb]));
        if (c.last(total, period)) umma_commit(smem_u32(&sh->o_full[ob]));
        TOCK(c_o, i2);
      }
      __syncwarp();
    }
    if (lane == 0) TPRINT("[%d] mma O: total %lld wait o_free %lld e_full %lld v_full %lld | issue+commit %lld\n", (int)blockIdx.x, clock64() - t0, w_of, w_ef, w_v, c_o);
  } else if (warp < 6) {
    // ------------------------------------------------------------------ exp and row sums
    int const quarter = warp & 3;               // tensor-memory lanes this warp may touch: 32 * (warp % 4)
    int const row = quarter * 32 + lane;        // KV position inside a tile
    uint32_t const lane_base = (uint32_t)(quarter * 32) << 16;
    int const rows_per_token = p.causal_window > 0 ? p.m / p.causal_window : 1;
    float rs[kNQ];
#pragma unroll
    for (int q = 0; q < kNQ; q++) rs[q] = 0.f;
    bool ok = true;
    TDECL(w_s = 0, w_rf = 0, c_exp = 0, t0 = clock64());
    TileCursor c;
    c.start(first_tile, period);
    for (int n = 0; n < total && ok; n++, c.advance(total, period)) {
      int const ri = c.ri, b = n & 1;
      int const kv_tile = kv_of(c.unit, c.pos); // first KV position of this tile
      TICK(a0);
      ok = mbar_wait(smem_u32(&sh->s_full[b]), (uint32_t)((n >> 1) & 1), abort_flag);
      TOCK(w_s, a0);
      if (!ok) break;
      tc_fence_after();
      TICK(a1);
      uint32_t v[32];
      tmem_ld32(tmem + lane_base + (uint32_t)(b * kNQ), v);
      float e[kNQ];
#pragma unroll
      for (int q = 0; q < kNQ; q++) e[q] = exp_ftz(__uint_as_float(v[q]));
      if (p.causal_window > 0 && kv_tile + kTileKv > p.kv_len - p.causal_window) {
        // only the last tile of the sequence reaches into the draft window
        int const pos = kv_tile + row;
#pragma unroll
        for (int q = 0; q < kNQ; q++)
          if (pos > p.kv_len - p.causal_window + q / rows_per_token) e[q] = 0.f;
      }
      uint32_t packed[kNQ / 2];
#pragma unroll
      for (int q = 0; q < kNQ; q += 2) {
        rs[q] += e[q];
        rs[q + 1] += e[q + 1];
        packed[q >> 1] = pack2<BF16>(e[q], e[q + 1]);
      }
      // the O^T MMAs of tile n - 2 must have read E^T buffer b before it is overwritten
      if (n >= 2) ok = mbar_wait(smem_u32(&sh->e_free[b]), (uint32_t)(((n >> 1) - 1) & 1), abort_flag);
      if (!ok) break;
      // E^T row of this KV position: 64 bytes = four 16-byte chunks, 64-byte swizzle (chunk ^= (row / 2) % 4)
      unsigned char *erow = e_ptr + b * kEBytes + row * 64;
#pragma unroll
      for (int c = 0; c < 4; c++)
        *reinterpret_cast<uint4 *>(erow + ((c ^ ((row >> 1) & 3)) << 4)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->e_full[b]));
      TOCK(c_exp, a1);
      if (c.last(total, period)) {
        // row sums over this warp's 32 KV lanes: transpose-reduce, lane q ends with column q
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
          bool const upper = (lane & s) != 0;
#pragma unroll
          for (int i = 0; i < s; i++) {
            float send = upper ? rs[i] : rs[i + s];
            float keep = upper ? rs[i + s] : rs[i];
            rs[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
          }
        }
        int const ob = ri & 1;
        TICK(a2);
        if (ri >= 2) ok = mbar_wait(smem_u32(&sh->r_free[ob]), (uint32_t)(((ri >> 1) - 1) & 1), abort_flag);
        TOCK(w_rf, a2);
        if (!ok) break;
        sh->rsum[ob][warp - 2][lane] = rs[0];
        mbar_arrive(smem_u32(&sh->r_full[ob]));
#pragma unroll
        for (int q = 0; q < kNQ; q++) rs[q] = 0.f;
      }
    }
    if (tid == 64) TPRINT("[%d] exp: total %lld wait s_full %lld r_free %lld exp+store %lld\n", (int)blockIdx.x, clock64() - t0, w_s, w_rf, c_exp);
  } else if (warp < 10) {
    // ------------------------------------------------------------------ epilogue and merge
    int const quarter = warp & 3;               // tensor-memory lanes this warp may touch
    int const row = quarter * 32 + lane;        // head-dim index of this thread's O^T row
    uint32_t const lane_base = (uint32_t)(quarter * 32) << 16;
    int const et = tid - 192;                   // 0..127 among the epilogue threads
    bool ok = true;
    // Launched with programmatic serialisation this grid may run while the previous kernel of the stream (the
    // merge of the call before, which reads the partials written below) is still going: no global store before it
    // has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    TDECL(w_r = 0, w_o = 0, c_out = 0, t0 = clock64());
    // one pass per run: [g, run_end) of the launch's tiles
    uint32_t const end_tile = first_tile + (uint32_t)total;
    int ri = 0;
    for (uint32_t g = first_tile; g < end_tile; ri++) {
      int const ob = ri & 1, unit = (int)(g / (uint32_t)period), batch = batch_of(unit);
      uint32_t const period_end = (uint32_t)(unit + 1) * (uint32_t)period;
      // where the run's sums go: the item's split, or the number of this block among the blocks that hold the head
      int const split = p.sum_runs ? (int)(blockIdx.x - block_of_tile((uint32_t)unit * (uint32_t)period, granule, p.per, p.extra))
                                   : unit % p.splits;
      g = period_end < end_tile ? period_end : end_tile;
      int const set = batch / p.heads, head = batch % p.heads;
      float r = 0.f;
      TICK(a0);
      if (ok) ok = mbar_wait(smem_u32(&sh->r_full[ob]), (uint32_t)((ri >> 1) & 1), abort_flag);
      TOCK(w_r, a0);
      TICK(a1);
      if (ok) {
        if (et < kNQ) r = sh->rsum[ob][0][et] + sh->rsum[ob][1][et] + sh->rsum[ob][2][et] + sh->rsum[ob][3][et];
        mbar_arrive(smem_u32(&sh->r_free[ob]));
        ok = mbar_wait(smem_u32(&sh->o_full[ob]), (uint32_t)((ri >> 1) & 1), abort_flag);
      }
      TOCK(w_o, a1);
      TICK(a2);
      if (ok) {
        uint32_t o[32];
        tc_fence_after();
        tmem_ld32(tmem + lane_base + 64 + (uint32_t)(ob * kNQ), o);
        tc_fence_before();
        mbar_arrive(smem_u32(&sh->o_free[ob]));
        // O^T: this thread holds head-dim index `row` of every query row
        int const out_ld = p.splits * kD;
        uint16_t *o_out = static_cast<uint16_t *>(p.o_part) + set * p.o_set_stride + (long long)head * p.m * out_ld + split * kD + row;
#pragma unroll
        for (int q = 0; q < kNQ; q++)
          if (q < p.m) o_out[(size_t)q * out_ld] = (uint16_t)(pack2<BF16>(__uint_as_float(o[q]), 0.f) & 0xFFFFu);
        if (et < p.m) {
          uint16_t *r_out = static_cast<uint16_t *>(p.r_part) + set * p.r_set_stride + (long long)head * p.m * p.splits + split;
          r_out[(size_t)et * p.splits] = (uint16_t)(pack2<BF16>(r, 0.f) & 0xFFFFu);
        }
      }
      TOCK(c_out, a2);
    }
#ifdef MG_STC_TIMING
    if (et == 0) {
      unsigned long long gt_now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt_now));
      if (gt_now - gt_entry > 36000)
        printf("slow [%d] epilogue done +%llu ns: wait r_full %lld o_full %lld out %lld items %d\n", (int)blockIdx.x,
               gt_now - gt_entry, w_r, w_o, c_out, ri);
    }
#endif
    if (et == 0) TPRINT("[%d] epilogue: total %lld wait r_full %lld o_full %lld out %lld tiles %d\n", (int)blockIdx.x, clock64() - t0, w_r, w_o, c_out, total);
  }

  // ---- teardown: every role arrives here, failed or not --------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && tid == 0) {
    // copies this block issued may still be in flight: give them a bounded time to land before the block exits
    for (int s = 0; s < kStages; s++)
      for (int i = 0; i < 20000 && !mbar_try_wait(smem_u32(&sh->k_full[s]), 0) && !mbar_try_wait(smem_u32(&sh->k_full[s]), 1) &&
                      !mbar_try_wait(smem_u32(&sh->v_full[s]), 0) && !mbar_try_wait(smem_u32(&sh->v_full[s]), 1); i++) {
      }
    atomicExch(p.status, 3);
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
// [batch][rows][cols] 16-bit array, box [1][box_rows][64], 128-byte swizzle, zero fill outside the array
static bool make_map(CUtensorMap *map, void const *base, uint64_t batch, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {cols * 2, rows * cols * 2};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

bool supported(mgd_attn_split const *p) {
  if (!p || p->heads <= 0 || p->splits <= 0 || p->forloop_range <= 0 || p->num_sets <= 0) return false;
  if (p->d != kD || p->m <= 0 || p->m > kNQ) return false;
  if (p->data_type != MG_DT_FLOAT16 && p->data_type != MG_DT_BFLOAT16) return false;
  int64_t per_block = (int64_t)p->forloop_range * 64; // the plan's for-loop walks tiles of 64 KV positions
  if (per_block % kTileKv != 0 || per_block * p->splits != p->kv_len) return false;
  if (p->causal_window < 0 || (p->causal_window > 0 && p->m % p->causal_window != 0)) return false;
  if (p->num_sets > 1) { // sets must be dense so that (set, head) folds into one TMA coordinate
    int64_t kv = (int64_t)p->heads * p->d * p->kv_len;
    if (p->k_set_stride != kv || p->v_set_stride != kv || p->q_set_stride != (int64_t)p->heads * p->m * p->d) return false;
  }
  if ((int64_t)p->heads * p->splits * p->num_sets > 0x7fffffffLL) return false;
  return encode_fn() != nullptr;
}

int launch(mgd_attn_split const *p, void const *q, void const *k, void const *v, void *o, void *r,
           mgd_attn_launch_opts const *opts, void *stream) {
  if (!supported(p)) return set_error(MG_ERR_UNSUPPORTED, "tensor-core split-KV attention: shape not supported");
  bool const k_kv = p->k_layout == MG_DMEM_COLUMN_MAJOR, v_kv = p->v_layout == MG_DMEM_ROW_MAJOR;
  uint64_t const batch = (uint64_t)p->heads * p->num_sets;
  CUtensorMap qm, km, vm;
  bool ok = make_map(&qm, q, batch, p->m, kD, kNQ);
  ok = ok && (k_kv ? make_map(&km, k, batch, p->kv_len, kD, 128) : make_map(&km, k, batch, kD, p->kv_len, 128));
  ok = ok && (v_kv ? make_map(&vm, v, batch, p->kv_len, kD, 128) : make_map(&vm, v, batch, kD, p->kv_len, 128));
  if (!ok) return set_error(MG_ERR_CUDA, "tensor-core split-KV attention: cuTensorMapEncodeTiled failed");
  Params a;
  a.o_part = o; a.r_part = r;
  // The merge runs as a second, small kernel right behind this one (programmatic serialisation hides its launch):
  // inside the persistent kernel the block that finishes a head last would merge serially, and a block that is
  // last once tends to be last again.
  a.status = device_error_word();
  if (!a.status) return set_error(MG_ERR_CUDA, "cannot allocate the device status word");
  a.o_set_stride = p->o_set_stride; a.r_set_stride = p->r_set_stride;
  a.heads = p->heads; a.m = p->m; a.splits = p->splits; a.tiles = p->forloop_range * 64 / kTileKv;
  a.kv_len = p->kv_len; a.causal_window = p->causal_window;
  a.num_items = (int)((int64_t)p->heads * p->splits * p->num_sets);
  // Work split.  When the merge rides along and the partials are scratch (overlap bit 3), the tiles are dealt singly
  // - every block within one tile of the average - and a block sums what it holds of a head; a head then has one
  // partial per block that touched it, which must fit the slots there are.
  int64_t const total_tiles = (int64_t)a.num_items * a.tiles, tiles_per_head = (int64_t)p->splits * a.tiles;
  if (total_tiles > 0x7fffffffLL) return set_error(MG_ERR_UNSUPPORTED, "tensor-core split-KV attention: too many tiles for one launch");
  bool sum_runs = opts && opts->merged_out && (opts->overlap & 8);
  unsigned blocks = 0;
  for (;;) {
    int64_t const granules = sum_runs ? total_tiles : (int64_t)a.num_items;
    blocks = (unsigned)(granules < sm_count() ? granules : sm_count());
    a.per = (uint32_t)(granules / blocks);
    a.extra = (uint32_t)(granules % blocks);
    if (!sum_runs) break;
    int64_t const runs_per_head = (tiles_per_head + a.per - 1) / a.per + 1;
    if (runs_per_head <= p->splits && runs_per_head <= 63) break;
    sum_runs = false;
  }
  a.sum_runs = sum_runs ? 1 : 0;
  size_t const smem = 1024 + (size_t)kStages * 2 * kOperand + 2 * kQBytes + 2 * kEBytes + sizeof(Shared) + 64;
  if (smem > (size_t)kSmemLimit) return set_error(MG_ERR_UNSUPPORTED, "tensor-core split-KV attention: shared memory plan too large");
  bool const bf16 = p->data_type == MG_DT_BFLOAT16;
  using Kernel = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, Params);
  static Kernel const kernels[8] = {
      attn_split_tc_kernel<false, false, false>, attn_split_tc_kernel<false, false, true>,
      attn_split_tc_kernel<false, true, false>,  attn_split_tc_kernel<false, true, true>,
      attn_split_tc_kernel<true, false, false>,  attn_split_tc_kernel<true, false, true>,
      attn_split_tc_kernel<true, true, false>,   attn_split_tc_kernel<true, true, true>};
  static bool configured[8] = {false, false, false, false, false, false, false, false};
  int const which = (bf16 ? 4 : 0) | (k_kv ? 2 : 0) | (v_kv ? 1 : 0);
  if (!configured[which]) {
    if (cudaFuncSetAttribute(kernels[which], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return check_launch("cudaFuncSetAttribute(attn_split_tc_kernel)");
    configured[which] = true;
  }
  a.early_loads = opts && (opts->overlap & 2) ? 1 : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (opts && (opts->overlap & 1)) {
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaLaunchKernelEx(&cfg, kernels[which], qm, km, vm, a);
  if (opts && opts->merged_out) {
    int st = check_launch("attn_split_tc_kernel");
    if (st != MG_OK) return st;
    launch_merge_rows(bf16 ? kMergeBF16 : kMergeF16, kD, static_cast<uint16_t const *>(o), static_cast<uint16_t const *>(r),
                      static_cast<uint16_t *>(opts->merged_out), p->heads, p->m, p->splits, p->num_sets, p->o_set_stride,
                      p->r_set_stride, opts->merged_set_stride, true, stream,
                      sum_runs ? MergeRuns{a.per, a.extra, (uint32_t)tiles_per_head} : MergeRuns{0, 0, 0});
    return check_launch("attn_merge_rows_kernel");
  }
  return check_launch("attn_split_tc_kernel");
}

} // namespace stc
} // namespace mgk
