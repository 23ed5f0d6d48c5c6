// Split-KV attention operator and its cross-split merge, float and fingerprint mode.
//
// The operator is the first customized op of the grouped-query decode muGraph (the pattern of the
// reference's cpp_examples/group_query_attn_inc_decode.cc:46-79): per (head, KV split) block and per
// for-loop iteration   S = Q K,  E = exp(S),  O' = E V,  R' = rowsum(E),   O' and R' summed over the
// iterations and stored as one partial per split.  The reference runs it through its interpreters
// (src/kernel/cuda/customized_kernel.cu:39-603); here it is one kernel:
//
//   * K and V tiles of 64 KV positions stream through a ring of shared-memory stages filled by TMA
//     (cp.async.bulk.tensor, 128-byte swizzle) and tracked by one mbarrier per stage; all stages are
//     requested before the first wait, so a block keeps up to `stages` x 32 KB in flight.
//   * Each warp owns 16 KV positions of a tile.  It computes its S slice with mma.sync (Q fragments stay
//     in registers for the whole kernel), exponentiates in registers, reuses the accumulator fragments
//     as the A operand of E V, and keeps its partial O' and R' in registers across all iterations; the
//     four KV slices are summed once, through shared memory, after the loop.  S, E and the partial O'
//     never touch shared memory.
//   * Float mode: fp16 / bf16 operands, fp32 accumulation (m16n8k16).  The optional causal window of
//     the speculative-decode graph is a predicate on E.
//   * Fingerprint mode: exact arithmetic modulo PQ = 227 * 113 on the integer tensor cores.  A uint16
//     fingerprint is two bytes x = lo + 256 hi, and a tile of uint16 in shared memory IS an interleaved
//     u8 matrix, so ldmatrix delivers u8 fragments of m16n8k32 without any unpacking.  The 16 rows of
//     the A operand carry three byte-masked copies of 4 query rows - [lo,0], [0,hi] and [hi,lo] - whose
//     products with the [lo,hi] bytes of the other operand are the sums LL, HH and LH+HL; then
//     sum x*y = LL + 256 (LH+HL) + 65536 HH exactly in int32, reduced modulo PQ once per element.
//     The result equals the reference's per-MAC reduction (include/mirage/threadblock/cuda/matmul.h:773-804)
//     bit for bit, for any uint16 operands.  exp is the table lookup of element_unary.h:60-66.
//
// Every mbarrier wait is bounded: a block that gives up records a code in the device status word and
// returns without touching its outputs further.
#include "common.cuh"
#include "ptx.cuh"
#include "attn_merge.cuh"
#include <atomic>
#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace mgk {
namespace stc { // attn_split_tc.cu
bool supported(mgd_attn_split const *p);
int launch(mgd_attn_split const *p, void const *q, void const *k, void const *v, void *o, void *r,
           mgd_attn_launch_opts const *opts, void *stream);
} // namespace stc
} // namespace mgk

namespace mgk {

constexpr int kTile = 64;        // KV positions per for-loop tile
constexpr int kMaxStages = 6;
constexpr int kDynSmemLimit = kSmemLimit - 1024; // the kernel also has a few bytes of static shared memory

enum AttnMode { kF16 = 0, kBF16 = 1, kFingerprint = 2 };

// ---- PTX wrappers (mbarrier, TMA: ptx.cuh) -----------------------------------------------------------------
using ptx::smem_u32;
using ptx::mbar_init;
using ptx::mbar_expect_tx;
using ptx::mbar_wait;
using ptx::tma_load_3d;
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <int MODE> struct Acc { using type = float; };
template <> struct Acc<kFingerprint> { using type = int32_t; };

template <int MODE>
__device__ __forceinline__ void mma_tile(typename Acc<MODE>::type (&c)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma_tile<kF16>(float (&c)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma_tile<kBF16>(float (&c)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma_tile<kFingerprint>(int32_t (&c)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A staged tile holds `rows` x `cols` 16-bit elements as cols/64 TMA boxes of [rows][64], each with the
// 128-byte swizzle (16-byte chunk c of row r sits at chunk c ^ (r % 8)).  `chunk` counts 8-element units.
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int rows, int row, int chunk) {
  return base + (uint32_t)((chunk >> 3) * rows * 128 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

struct AttnSplitParams {
  void const *q;   // [sets][heads][m][d]
  void *o_part;    // [sets][heads][m][splits*d]
  void *r_part;    // [sets][heads][m][splits]
  int32_t *status; // device status word
  long long q_set_stride, o_set_stride, r_set_stride;
  int heads, m, splits, forloop, stages, kv_len;
  int tile_groups;   // warp groups that work on different KV tiles of the ring at the same time
  int k_rows_are_kv; // K staged as [kv][d] (memory of a column-major K) else [d][kv]
  int v_rows_are_kv; // V staged as [kv][d] (memory of a row-major V) else [d][kv]
  int causal_window;
  void *merged_out;     // non-null: the last block of a head also merges the head's partials
  int32_t *tickets;     // one counter per (set, head)
  long long merged_set_stride;
  int early_loads;      // tile loads may be issued before the wait on the previous kernel of the stream
  int early_release;    // the next kernel of the stream is released when this one starts, not after its wait
  int wait_limit;       // polls before a tile wait gives up
  int num_sets;
  int sum_runs;         // persistent with a fused merge whose partials are scratch: consecutive splits of a head
                        // are summed in the accumulators, only sums that straddle blocks go through memory
  int persistent;       // fewer blocks than work items: a block walks items blockIdx.x, + gridDim.x, ... and the tile
                        // ring runs on across item boundaries (the reduction scratch then has room of its own)
};

// Shared-memory plan: [stages x (K tile, V tile)] (1024-byte aligned) | reduction scratch | barriers | exp table
// FORM: bit 0 = K staged as [kv][d] (else [d][kv]); bit 1 = V staged as [kv][d] (else [d][kv]).  A compile-time
// property so that every ldmatrix address is one XOR and one ADD away from a per-lane constant.
// PERSIST: the block walks several work items (a compile-time property: the one-item kernel keeps no item state in
// registers across its loop; the walking one is launched with 128 threads, three blocks to an SM).
template <int MODE, int DH, int FORM, bool PERSIST>
__global__ void __launch_bounds__(PERSIST ? 128 : 512, PERSIST ? 3 : 1)
attn_split_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                  const __grid_constant__ AttnSplitParams p) {
  using acc_t = typename Acc<MODE>::type;
  constexpr int kRowsPerGroup = MODE == kFingerprint ? 4 : 16; // query rows one warp's MMA rows carry
  constexpr int kTileBytes = kTile * DH * 2;
  constexpr int kKSteps = DH / 16;     // k-steps of Q K (contraction over head_dim)
  constexpr int kNPairs = DH / 16;     // pairs of 8-wide output tiles of E V (output over head_dim)
  constexpr bool kKRowsKv = (FORM & 1) != 0, kVRowsKv = (FORM & 2) != 0;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);

  int const tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int const slice = warp & 3;          // which 16 KV positions of a tile
  int const groups = (blockDim.x >> 7) / p.tile_groups;
  int const group = (warp >> 2) % groups;   // which group of query rows
  int const tgroup = (warp >> 2) / groups;  // which of the tiles processed concurrently
  int const g = lane >> 2, t = lane & 3;

  // Work items: one (set, head, split) each, split fastest.  A plain launch has one block per item.  A persistent
  // launch has fewer blocks than items and block b takes a contiguous run of them, [lo, lo + n_local): its tile ring
  // keeps running across item boundaries, and when the merge is fused, consecutive splits of one head simply keep
  // accumulating in registers - partials go to memory only where a head's splits straddle two blocks.
  // (item numbers fit 31 bits: the launch refuses more)
  uint32_t const n_items = (uint32_t)p.splits * (uint32_t)p.heads * (uint32_t)p.num_sets;
  uint32_t const per_block = PERSIST ? n_items / gridDim.x : 1u, extra = PERSIST ? n_items % gridDim.x : 0u; // the first `extra` blocks take one more
  uint32_t const lo = PERSIST ? blockIdx.x * per_block + (blockIdx.x < extra ? blockIdx.x : extra) : blockIdx.x;
  int const n_local = PERSIST ? (int)per_block + (blockIdx.x < extra ? 1 : 0) : 1;
  int const total_tiles = n_local * p.forloop;
  bool const fused_runs = PERSIST && p.sum_runs;
  int split = 0, head = 0, kv_base = 0; // of the item being computed
  int set = 0;
  auto select_item = [&](int li) {
    uint32_t const x = lo + (uint32_t)li, unit = x / (uint32_t)p.splits; // unit = set * heads + head
    split = (int)(x - unit * (uint32_t)p.splits);
    set = (int)(unit / (uint32_t)p.heads);
    head = (int)(unit - (uint32_t)set * (uint32_t)p.heads);
    kv_base = split * p.forloop * kTile; // first KV position of the item
  };

  uint32_t const stage_base = smem_u32(smem);
  int const rows_scratch = MODE == kFingerprint ? 4 : (p.m < 16 ? p.m : 16);
  // the reduction scratch reuses the stage memory once every tile has been consumed; a persistent block has tiles of
  // its next item arriving by then, so its scratch sits behind the stages
  size_t const scratch_bytes = (size_t)(blockDim.x >> 5) * rows_scratch * (DH + 4) * sizeof(acc_t);
  size_t const stage_bytes = (size_t)p.stages * 2 * kTileBytes;
  acc_t *scratch = reinterpret_cast<acc_t *>(smem + (PERSIST ? stage_bytes : 0));
  size_t const data_bytes = ((PERSIST ? stage_bytes + scratch_bytes : (scratch_bytes > stage_bytes ? scratch_bytes : stage_bytes)) + 15) & ~(size_t)15;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + data_bytes);
  uint16_t *exp_tab = reinterpret_cast<uint16_t *>(bars + kMaxStages);
  __shared__ int s_failed;

  if (tid == 0) {
    s_failed = 0;
    ptx::prefetch_tensormap(&k_map);
    ptx::prefetch_tensormap(&v_map);
    for (int s = 0; s < p.stages; s++) mbar_init(smem_u32(&bars[s]), 1);
    ptx::mbar_init_fence();
  }
  if (MODE == kFingerprint) // exp table with the CRT lift folded in: E = table[S mod Q]
    for (int i = tid; i < (int)Q; i += blockDim.x) exp_tab[i] = (uint16_t)((c_tables.e[i] * Q_MUL_P_MOD_1) % PQ);
  __syncthreads();

  // Requests the next tile of this block's tile sequence (items in order, `forloop` tiles each) into stage s.
  // Thread 0 keeps the coordinates of that tile: KV position and (set, head), which the tensor maps fold into one
  // coordinate.
  // (kept in shared memory: registers of every thread are scarcer than one thread's few shared-memory accesses)
  __shared__ int s_next_kv, s_next_batch, s_issued; // s_issued: tiles requested so far; tile i lands in stage i % stages
  auto issue = [&](int s) {
    uint32_t bar = smem_u32(&bars[s]);
    uint32_t kdst = stage_base + (uint32_t)(s * 2 * kTileBytes), vdst = kdst + kTileBytes;
    int const kv0 = s_next_kv, batch = s_next_batch;
    if (PERSIST && kv0 + kTile == p.kv_len) { // the head's last tile: on to the next head
      s_next_kv = 0;
      s_next_batch = batch + 1;
    } else {
      s_next_kv = kv0 + kTile;
    }
    s_issued++;
    mbar_expect_tx(bar, 2 * kTileBytes);
    if (kKRowsKv) {
      for (int c = 0; c < DH / 64; c++) tma_load_3d(kdst + c * (kTile * 128), &k_map, bar, c * 64, kv0, batch);
    } else {
      tma_load_3d(kdst, &k_map, bar, kv0, 0, batch);
    }
    if (kVRowsKv) {
      for (int c = 0; c < DH / 64; c++) tma_load_3d(vdst + c * (kTile * 128), &v_map, bar, c * 64, kv0, batch);
    } else {
      tma_load_3d(vdst, &v_map, bar, kv0, 0, batch);
    }
  };
  // ---- Q fragments, resident in registers -----------------------------------------------------------
  uint32_t qa[kKSteps][4];
  auto load_q = [&]() {
    uint16_t const *q = static_cast<uint16_t const *>(p.q) + (int64_t)set * p.q_set_stride + (int64_t)head * p.m * DH;
    if (MODE == kFingerprint) {
      int row = group * 4 + (g & 3);
      bool valid = row < p.m;
#pragma unroll
      for (int ks = 0; ks < kKSteps; ks++) {
        uint32_t w0 = valid ? __ldg(reinterpret_cast<uint32_t const *>(q + (size_t)row * DH + ks * 16 + 2 * t)) : 0u;
        uint32_t w1 = valid ? __ldg(reinterpret_cast<uint32_t const *>(q + (size_t)row * DH + ks * 16 + 8 + 2 * t)) : 0u;
        if (g < 4) { // MMA rows 0-3: [lo,0] bytes; MMA rows 8-11: [hi,lo] bytes
          qa[ks][0] = w0 & 0x00FF00FFu; qa[ks][2] = w1 & 0x00FF00FFu;
          qa[ks][1] = __byte_perm(w0, 0, 0x2301); qa[ks][3] = __byte_perm(w1, 0, 0x2301);
        } else {     // MMA rows 4-7: [0,hi] bytes; MMA rows 12-15 unused
          qa[ks][0] = w0 & 0xFF00FF00u; qa[ks][2] = w1 & 0xFF00FF00u;
          qa[ks][1] = 0u; qa[ks][3] = 0u;
        }
      }
    } else {
      int r0 = group * 16 + g, r1 = r0 + 8;
#pragma unroll
      for (int ks = 0; ks < kKSteps; ks++) {
        qa[ks][0] = r0 < p.m ? __ldg(reinterpret_cast<uint32_t const *>(q + (size_t)r0 * DH + ks * 16 + 2 * t)) : 0u;
        qa[ks][1] = r1 < p.m ? __ldg(reinterpret_cast<uint32_t const *>(q + (size_t)r1 * DH + ks * 16 + 2 * t)) : 0u;
        qa[ks][2] = r0 < p.m ? __ldg(reinterpret_cast<uint32_t const *>(q + (size_t)r0 * DH + ks * 16 + 8 + 2 * t)) : 0u;
        qa[ks][3] = r1 < p.m ? __ldg(reinterpret_cast<uint32_t const *>(q + (size_t)r1 * DH + ks * 16 + 8 + 2 * t)) : 0u;
      }
    }
  };
  auto issue_first = [&]() {
    if (tid == 0) {
      int first = total_tiles < p.stages ? total_tiles : p.stages;
      s_next_kv = kv_base, s_next_batch = set * p.heads + head, s_issued = 0; // select_item(0) came first
      for (int gt = 0; gt < first; gt++) issue(gt);
    }
  };
  // Ordering against the previous kernel of the stream (programmatic dependent launch): nothing is written
  // to global memory, and no input that kernel may have produced is read, before griddepcontrol.wait; the next
  // kernel is released right after, so at most two kernels of a stream are ever in flight.
  // With inputs that the previous kernel did not write, a block goes further: it also does its arithmetic before the
  // wait and only holds back its stores, so the previous kernel's write-out, tickets and merges run under it.
  // A walking block does the same up to the end of its first run.
  // A launch that covers more than half of the GPU's block slots may release its successor at once: the kernel after
  // that one cannot start before a block of the successor has exited, which happens after the successor's wait on
  // this kernel - three launches are never in flight, and the host's check of the inputs looks two launches back.
  bool late_wait = p.early_loads != 0;
  if (p.early_release) ptx::grid_launch_dependents();
  select_item(0);
  if (p.early_loads) {
    issue_first();
    load_q();
  }
  if (!late_wait) {
    ptx::grid_dependency_wait();
    if (!p.early_loads) {
      issue_first();
      load_q();
    }
    ptx::grid_launch_dependents();
  }

  // stage and barrier phase of this warp's tile, and stage of the round's first tile, kept without divisions
  // (tile_groups <= stages, so one conditional subtraction per round is enough); they run on across items
  int s = tgroup, round_s = 0;
  uint32_t phase = 0;
  bool failed = false;
  // Accumulators of the run of splits being summed: one item, or with a fused merge every split of the head that this
  // block holds.  run_first = the split the run began with (the slot its partial goes to).
  acc_t oacc[2 * kNPairs][4];
#pragma unroll
  for (int i = 0; i < 2 * kNPairs; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) oacc[i][j] = 0;
  acc_t racc0 = 0, racc1 = 0; // row sums of E: float: rows g and g+8; fingerprint: row g (lanes 0-15)
  int run_first = split;

  int const mi = lane >> 3, rr = lane & 7; // ldmatrix: this lane addresses row rr of matrix mi
  int const kv0 = slice * 16;               // this warp's KV positions inside a tile

  // Per-lane pieces of the ldmatrix addresses (see tile_addr): what is left per step is a compile-time offset
  // and, where the step moves along a swizzled row, one XOR.
  uint32_t k_lane, k_x, v_lane, v_x;
  if (kKRowsKv) {
    int row = kv0 + (mi >> 1) * 8 + rr;
    k_lane = (uint32_t)(row * 128);
    k_x = (uint32_t)(((row & 7) ^ (mi & 1)) << 4);
  } else {
    k_lane = (uint32_t)(((mi & 1) * 8 + rr) * 128 + ((((kv0 >> 3) + (mi >> 1)) ^ rr) << 4));
    k_x = 0;
  }
  if (kVRowsKv) {
    int row = kv0 + (mi & 1) * 8 + rr;
    v_lane = (uint32_t)(row * 128);
    v_x = (uint32_t)(((row & 7) ^ (mi >> 1)) << 4);
  } else {
    v_lane = (uint32_t)(((mi >> 1) * 8 + rr) * 128 + ((((kv0 >> 3) + (mi & 1)) ^ rr) << 4));
    v_x = 0;
  }
  // causal window (float mode): last KV position each of this thread's two rows may see
  int lim0 = 0x7fffffff, lim1 = 0x7fffffff, lim_min = 0x7fffffff;
  if (MODE != kFingerprint && p.causal_window > 0) {
    int rows_per_token = p.m / p.causal_window;
    int r0 = group * 16 + g, r1 = r0 + 8;
    lim0 = p.kv_len - p.causal_window + r0 / rows_per_token;
    lim1 = p.kv_len - p.causal_window + r1 / rows_per_token;
    lim_min = p.kv_len - p.causal_window; // positions up to here are visible to every row
  }

  // Tiles are consumed in rounds of `tile_groups`: warp group tgroup takes tile round*tile_groups + tgroup.
  int const rounds = (p.forloop + p.tile_groups - 1) / p.tile_groups;
  for (int li = 0; li < n_local; li++) {
  for (int round = 0; round < rounds; round++) {
    int const it = round * p.tile_groups + tgroup;
    bool const active = it < p.forloop;
    // After a wait has given up the block keeps walking the loop (so that every thread still meets the
    // block-wide barriers below) but stops waiting; its results are discarded at the end.
    if (active && !failed && !mbar_wait(smem_u32(&bars[s]), phase, p.wait_limit)) failed = true;
    if (active) {
    uint32_t ktile = stage_base + (uint32_t)(s * 2 * kTileBytes), vtile = ktile + kTileBytes;

    // ---- S slice = Q K over this warp's 16 KV positions: two 8-wide tiles ---------------------------
    acc_t sacc[2][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) sacc[i][j] = 0;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ks++) {
      uint32_t bfrag[4];
      if (kKRowsKv) ldsm_x4(ktile + k_lane + (uint32_t)((ks >> 2) * (kTile * 128)) + (k_x ^ (uint32_t)(((2 * ks) & 7) << 4)), bfrag);
      else ldsm_x4_trans(ktile + k_lane + (uint32_t)(ks * 16 * 128), bfrag);
      mma_tile<MODE>(sacc[0], qa[ks], bfrag[0], bfrag[1]);
      mma_tile<MODE>(sacc[1], qa[ks], bfrag[2], bfrag[3]);
    }

    // ---- E = exp(S) in registers, repacked as the A operand of E V ---------------------------------
    uint32_t ea[4];
    if (MODE == kFingerprint) {
      uint32_t e[2][2];
#pragma unroll
      for (int nt = 0; nt < 2; nt++) {
        // lanes 16-31 hold the HH sums of the query row lanes 0-15 work on
        int32_t hh0 = __shfl_down_sync(0xffffffffu, sacc[nt][0], 16), hh1 = __shfl_down_sync(0xffffffffu, sacc[nt][1], 16);
        uint32_t s0 = ((uint32_t)sacc[nt][0] % PQ + 256u * ((uint32_t)sacc[nt][2] % PQ) + (65536u % PQ) * ((uint32_t)hh0 % PQ)) % PQ;
        uint32_t s1 = ((uint32_t)sacc[nt][1] % PQ + 256u * ((uint32_t)sacc[nt][3] % PQ) + (65536u % PQ) * ((uint32_t)hh1 % PQ)) % PQ;
        e[nt][0] = exp_tab[s0 % Q];
        e[nt][1] = exp_tab[s1 % Q];
      }
      uint32_t x0 = e[0][0] | (e[0][1] << 16), x1 = e[1][0] | (e[1][1] << 16);
      uint32_t y0 = __shfl_up_sync(0xffffffffu, x0, 16), y1 = __shfl_up_sync(0xffffffffu, x1, 16);
      if (g < 4) {
        racc0 += (int32_t)(e[0][0] + e[0][1] + e[1][0] + e[1][1]);
        ea[0] = x0 & 0x00FF00FFu; ea[2] = x1 & 0x00FF00FFu;
        ea[1] = __byte_perm(x0, 0, 0x2301); ea[3] = __byte_perm(x1, 0, 0x2301);
      } else {
        ea[0] = y0 & 0xFF00FF00u; ea[2] = y1 & 0xFF00FF00u;
        ea[1] = 0u; ea[3] = 0u;
      }
    } else {
      float ev[2][4];
      int pos = kv_base + it * kTile + kv0 + 2 * t; // KV position of sacc[0][0]
      bool const in_window = pos + 9 > lim_min;      // some position of this thread's eight may be masked
#pragma unroll
      for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float v = __expf(sacc[nt][j]);
          if (in_window && pos + nt * 8 + (j & 1) > ((j >> 1) ? lim1 : lim0)) v = 0.f;
          ev[nt][j] = v;
        }
      racc0 += ev[0][0] + ev[0][1] + ev[1][0] + ev[1][1];
      racc1 += ev[0][2] + ev[0][3] + ev[1][2] + ev[1][3];
      if (MODE == kF16) {
        ea[0] = pack_f16(ev[0][0], ev[0][1]); ea[1] = pack_f16(ev[0][2], ev[0][3]);
        ea[2] = pack_f16(ev[1][0], ev[1][1]); ea[3] = pack_f16(ev[1][2], ev[1][3]);
      } else {
        ea[0] = pack_bf16(ev[0][0], ev[0][1]); ea[1] = pack_bf16(ev[0][2], ev[0][3]);
        ea[2] = pack_bf16(ev[1][0], ev[1][1]); ea[3] = pack_bf16(ev[1][2], ev[1][3]);
      }
    }

    // ---- O' += E V over this warp's 16 KV positions -------------------------------------------------
#pragma unroll
    for (int jp = 0; jp < kNPairs; jp++) {
      uint32_t bfrag[4];
      if (kVRowsKv) ldsm_x4_trans(vtile + v_lane + (uint32_t)((jp >> 2) * (kTile * 128)) + (v_x ^ (uint32_t)(((2 * jp) & 7) << 4)), bfrag);
      else ldsm_x4(vtile + v_lane + (uint32_t)(jp * 16 * 128), bfrag);
      mma_tile<MODE>(oacc[2 * jp], ea, bfrag[0], bfrag[1]);
      mma_tile<MODE>(oacc[2 * jp + 1], ea, bfrag[2], bfrag[3]);
    }

    } // active
    // ---- refill the stages of this round once every warp has read them -----------------------------------
    if (total_tiles > p.stages) {
      __syncthreads();
      if (tid == 0 && !failed) // a block that has given up requests nothing more
        for (int j = 0; j < p.tile_groups; j++) {
          int nxt = li * p.forloop + round * p.tile_groups + j + p.stages; // (a persistent block has tile_groups = 1)
          int ns = round_s + j >= p.stages ? round_s + j - p.stages : round_s + j; // the stage tile nxt - stages used
          if (nxt < total_tiles) {
            issue(ns);
          }
        }
    }
    s += p.tile_groups;
    if (s >= p.stages) { s -= p.stages; phase ^= 1u; }
    round_s += p.tile_groups;
    if (round_s >= p.stages) round_s -= p.stages;
  }

  // A run ends with the head's last split or the block's last item; without a fused merge every item is a run.
  int const covered = split - run_first + 1; // splits summed in the accumulators
  bool const run_ends = !fused_runs || split == p.splits - 1 || li == n_local - 1;
  bool const whole_head = fused_runs && covered == p.splits; // nothing of this head is anywhere else: finish it here
  int const run_head = head, run_set = set, run_slot = run_first; // where the run's sums go
  bool new_rows = false; // the next item has other query rows
  if (PERSIST && li + 1 < n_local) {
    select_item(li + 1);
    new_rows = head != run_head || set != run_set;
    if (run_ends) run_first = split;
    if (new_rows) { // on their way into L2 while this run is written out (m * DH 16-bit values, 128-byte lines)
      char const *rows = static_cast<char const *>(p.q) + ((int64_t)set * p.q_set_stride + (int64_t)head * p.m * DH) * 2;
      if (tid * 128 < p.m * DH * 2) asm volatile("prefetch.global.L2 [%0];" ::"l"(rows + tid * 128));
    }
  }
  if (!run_ends) continue; // (a run that goes on stays with its head: no new rows)

  // A block that still owes the wait on the previous kernel of the stream takes it as late as it can: the sums over
  // slices and tile groups below only touch shared memory, so each thread waits right in front of its first store
  // to global memory, and the whole block once more behind the stores, where it also releases the next kernel
  // unless it did so at its start.
  bool const release_here = late_wait && !p.early_release;
  auto wait_before_store = [&]() {
    if (late_wait) {
      ptx::grid_dependency_wait();
      late_wait = false;
    }
  };
  if (failed) s_failed = 1;
  __syncthreads(); // also: every tile has been read, the stage memory may be reused as scratch
  if (s_failed) { // a bounded wait gave up: flag it and leave the outputs alone
    wait_before_store();
    if (release_here) ptx::grid_launch_dependents();
    if (tid == 0) {
      atomicExch(p.status, 1);
      // Tile loads still in flight must land before this block's shared memory is handed to another block:
      // stage s received tiles s, s + stages, ...; wait (bounded again) for the last of them.
      int const issued = s_issued;
      for (int st = 0; st < p.stages && st < issued; st++) {
        int loads = (issued - st + p.stages - 1) / p.stages;
        mbar_wait(smem_u32(&bars[st]), (uint32_t)((loads - 1) & 1));
      }
      // The head's ticket counter must still come back to zero for the next launch: take the ticket, and reset
      // the counter if this block is the last of its head.  (A healthy last block merges whatever partials there
      // are; the status word tells the host that the outputs of this launch are incomplete.)
      if (p.merged_out != nullptr)
        for (int rest = li - (covered - 1); rest < n_local; rest++) { // the open run and the items not reached
          int const unit = (int)((lo + (uint32_t)rest) / (uint32_t)p.splits);
          int ticket = atomicAdd(&p.tickets[unit], 1);
          if (ticket == p.splits - 1) p.tickets[unit] = 0;
        }
    }
    return;
  }

  // ---- sum the four KV slices (and nothing else: rows of different groups are distinct query rows) ----
  int const ld = DH + 4; // padded row pitch of the scratch (keeps the column walk off a single bank)
  acc_t *mine = scratch + (size_t)warp * rows_scratch * ld;
  acc_t *rsum = mine + DH; // the pad holds this warp's row sums: rsum[row * ld]
  if (MODE == kFingerprint) {
#pragma unroll
    for (int nt = 0; nt < 2 * kNPairs; nt++) {
      int32_t hh0 = __shfl_down_sync(0xffffffffu, oacc[nt][0], 16), hh1 = __shfl_down_sync(0xffffffffu, oacc[nt][1], 16);
      if (g < 4) {
        uint32_t v0 = ((uint32_t)oacc[nt][0] % PQ + 256u * ((uint32_t)oacc[nt][2] % PQ) + (65536u % PQ) * ((uint32_t)hh0 % PQ)) % PQ;
        uint32_t v1 = ((uint32_t)oacc[nt][1] % PQ + 256u * ((uint32_t)oacc[nt][3] % PQ) + (65536u % PQ) * ((uint32_t)hh1 % PQ)) % PQ;
        mine[g * ld + nt * 8 + 2 * t] = (int32_t)v0;
        mine[g * ld + nt * 8 + 2 * t + 1] = (int32_t)v1;
      }
    }
    int32_t r = racc0;
    r += __shfl_xor_sync(0xffffffffu, r, 1);
    r += __shfl_xor_sync(0xffffffffu, r, 2);
    if (g < 4 && t == 0) rsum[g * ld] = (int32_t)((uint32_t)r % PQ);
  } else {
#pragma unroll
    for (int nt = 0; nt < 2 * kNPairs; nt++) {
      if (g < rows_scratch) {
        mine[g * ld + nt * 8 + 2 * t] = oacc[nt][0];
        mine[g * ld + nt * 8 + 2 * t + 1] = oacc[nt][1];
      }
      if (g + 8 < rows_scratch) {
        mine[(g + 8) * ld + nt * 8 + 2 * t] = oacc[nt][2];
        mine[(g + 8) * ld + nt * 8 + 2 * t + 1] = oacc[nt][3];
      }
    }
    float r0 = racc0, r1 = racc1;
    r0 += __shfl_xor_sync(0xffffffffu, r0, 1); r0 += __shfl_xor_sync(0xffffffffu, r0, 2);
    r1 += __shfl_xor_sync(0xffffffffu, r1, 1); r1 += __shfl_xor_sync(0xffffffffu, r1, 2);
    if (t == 0) {
      if (g < rows_scratch) rsum[g * ld] = r0;
      if (g + 8 < rows_scratch) rsum[(g + 8) * ld] = r1;
    }
  }
  __syncthreads();

  int const rows_per_group = kRowsPerGroup;
  int const out_ld = p.splits * DH;
  // a run's sums go to the slot of its first split
  uint16_t *o_out = static_cast<uint16_t *>(p.o_part) + (int64_t)run_set * p.o_set_stride + (int64_t)run_head * p.m * out_ld + run_slot * DH;
  uint16_t *r_out = static_cast<uint16_t *>(p.r_part) + (int64_t)run_set * p.r_set_stride + (int64_t)run_head * p.m * p.splits + run_slot;
  uint16_t *final_out = p.merged_out == nullptr ? nullptr : static_cast<uint16_t *>(p.merged_out) + (int64_t)run_set * p.merged_set_stride + (int64_t)run_head * p.m * DH;
  __shared__ acc_t s_den[32]; // row sums of a head that is finished in place
  // warp index = (tile group * groups + row group) * 4 + slice: sum over tile groups and slices.
  for (int i = tid; i < groups * rows_scratch; i += blockDim.x) {
    int lr = i % rows_scratch, gr = i / rows_scratch, row = gr * rows_per_group + lr;
    if (row >= p.m) continue;
    acc_t a = 0;
    for (int tg = 0; tg < p.tile_groups; tg++)
#pragma unroll
      for (int sl = 0; sl < 4; sl++) {
        acc_t v = scratch[(size_t)((tg * groups + gr) * 4 + sl) * rows_scratch * ld + lr * ld + DH];
        if (MODE == kFingerprint) a = (acc_t)(((uint32_t)a + (uint32_t)v) % PQ);
        else a += v;
      }
    if (whole_head) {
      s_den[i] = a;
      continue;
    }
    uint16_t v;
    if (MODE == kFingerprint) v = (uint16_t)((uint32_t)a % PQ);
    else if (MODE == kF16) { __half h = __float2half_rn((float)a); v = *reinterpret_cast<uint16_t *>(&h); }
    else { __nv_bfloat16 h = __float2bfloat16_rn((float)a); v = *reinterpret_cast<uint16_t *>(&h); }
    wait_before_store();
    r_out[(size_t)row * p.splits] = v;
  }
  if (whole_head) __syncthreads();
  // A thread keeps one pair of adjacent columns (one 32-bit store) and walks down the rows.
  {
    int const c = (tid % (DH / 2)) * 2, row_step = blockDim.x / (DH / 2);
    size_t const warp_pitch = (size_t)rows_scratch * ld;
    for (int gr = 0; gr < groups; gr++)
      for (int lr = tid / (DH / 2); lr < rows_scratch; lr += row_step) {
        int row = gr * rows_per_group + lr;
        if (row >= p.m) break;
        acc_t a0 = 0, a1 = 0;
        for (int tg = 0; tg < p.tile_groups; tg++) {
          acc_t const *src = scratch + (size_t)((tg * groups + gr) * 4) * warp_pitch + lr * ld + c;
#pragma unroll
          for (int sl = 0; sl < 4; sl++) {
            if (MODE == kFingerprint) { // partials are already reduced modulo PQ: no overflow for any count
              a0 = (acc_t)((uint32_t)a0 + (uint32_t)src[sl * warp_pitch]);
              a1 = (acc_t)((uint32_t)a1 + (uint32_t)src[sl * warp_pitch + 1]);
            } else {
              a0 += src[sl * warp_pitch];
              a1 += src[sl * warp_pitch + 1];
            }
          }
          if (MODE == kFingerprint) { a0 = (acc_t)((uint32_t)a0 % PQ); a1 = (acc_t)((uint32_t)a1 % PQ); }
        }
        uint32_t packed;
        if (whole_head) { // the division of the merge, on sums that never left the chip
          acc_t const den = s_den[gr * rows_scratch + lr];
          if (MODE == kFingerprint) packed = field_div((uint32_t)a0, (uint32_t)den % PQ) | (field_div((uint32_t)a1, (uint32_t)den % PQ) << 16);
          else if (MODE == kF16) packed = pack_f16((float)a0 / (float)den, (float)a1 / (float)den);
          else packed = pack_bf16((float)a0 / (float)den, (float)a1 / (float)den);
          wait_before_store();
          *reinterpret_cast<uint32_t *>(final_out + (size_t)row * DH + c) = packed;
          continue;
        }
        if (MODE == kFingerprint) packed = (uint32_t)a0 | ((uint32_t)a1 << 16);
        else if (MODE == kF16) packed = pack_f16((float)a0, (float)a1);
        else packed = pack_bf16((float)a0, (float)a1);
        wait_before_store();
        *reinterpret_cast<uint32_t *>(o_out + (size_t)row * out_ld + c) = packed;
      }
  }
  wait_before_store(); // threads without a store; the tickets and the merge below are global memory traffic too
  if (release_here) ptx::grid_launch_dependents();

  // ---- optional: the block that completes a head's splits merges the head's partials -----------------------
  if (p.merged_out != nullptr && !whole_head) {
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    int const unit = run_set * p.heads + run_head;
    if (tid == 0) {
      int ticket = atomicAdd(&p.tickets[unit], covered);
      s_last = ticket + covered == p.splits;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      uint16_t const *op = static_cast<uint16_t const *>(p.o_part) + (int64_t)run_set * p.o_set_stride + (int64_t)run_head * p.m * out_ld;
      uint16_t const *rp = static_cast<uint16_t const *>(p.r_part) + (int64_t)run_set * p.r_set_stride + (int64_t)run_head * p.m * p.splits;
      constexpr int kKind = MODE == kFingerprint ? kMergeFingerprint : (MODE == kBF16 ? kMergeBF16 : kMergeF16);
      uint64_t held = ~0ull;
      if (fused_runs) {
        // Only the slots that begin a run hold sums: split 0, and every split that is the first item of a block.
        // Thread s looks at slot s (at most 64 splits here); the votes of the first two warps make the mask.
        __shared__ uint32_t s_held[2];
        if (tid < 64) {
          uint32_t const x = (uint32_t)unit * (uint32_t)p.splits + (uint32_t)tid, wide = extra * (per_block + 1);
          bool const starts_block = x < wide ? x % (per_block + 1) == 0 : (x - wide) % per_block == 0;
          uint32_t const votes = __ballot_sync(0xffffffffu, tid < p.splits && (tid == 0 || starts_block));
          if (lane == 0) s_held[warp] = votes;
        }
        __syncthreads();
        held = (uint64_t)s_held[0] | ((uint64_t)s_held[1] << 32);
      }
      merge_head<kKind, DH>(op, rp, final_out, p.m, p.splits, tid, (int)blockDim.x, held);
      if (tid == 0) p.tickets[unit] = 0; // ready for the next launch
    }
  }
  if (PERSIST) { // the next run starts from nothing
#pragma unroll
    for (int i = 0; i < 2 * kNPairs; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) oacc[i][j] = 0;
    racc0 = 0, racc1 = 0;
    if (new_rows) load_q();
  }
  } // work items of this block
}

// ---- merge: O = sum_s O_part[.., s*d + c] / sum_s R_part[.., s] ---------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(256) attn_merge_kernel(uint16_t const *o_part, uint16_t const *r_part, uint16_t *out,
                                                         int heads, int m, int d, int splits, long long o_stride,
                                                         long long r_stride, long long out_stride) {
  int const head = blockIdx.x % heads;
  int64_t const set = blockIdx.x / heads;
  uint16_t const *op = o_part + set * o_stride + (int64_t)head * m * splits * d;
  uint16_t const *rp = r_part + set * r_stride + (int64_t)head * m * splits;
  uint16_t *dst = out + set * out_stride + (int64_t)head * m * d;
  for (int i = threadIdx.x; i < m * d; i += blockDim.x) {
    int r = i / d, c = i % d;
    if (MODE == kFingerprint) {
      uint32_t num = 0, den = 0;
#pragma unroll 8
      for (int s = 0; s < splits; s++) {
        num += op[(size_t)r * splits * d + s * d + c];
        den += rp[r * splits + s];
      }
      dst[i] = (uint16_t)field_div(num % PQ, den % PQ);
    } else {
      float num = 0.f, den = 0.f;
#pragma unroll 8
      for (int s = 0; s < splits; s++) {
        uint16_t a = op[(size_t)r * splits * d + s * d + c], bb = rp[r * splits + s];
        if (MODE == kF16) {
          num += __half2float(*reinterpret_cast<__half const *>(&a));
          den += __half2float(*reinterpret_cast<__half const *>(&bb));
        } else {
          num += __bfloat162float(*reinterpret_cast<__nv_bfloat16 const *>(&a));
          den += __bfloat162float(*reinterpret_cast<__nv_bfloat16 const *>(&bb));
        }
      }
      float v = num / den;
      if (MODE == kF16) { __half h = __float2half_rn(v); dst[i] = *reinterpret_cast<uint16_t *>(&h); }
      else { __nv_bfloat16 h = __float2bfloat16_rn(v); dst[i] = *reinterpret_cast<uint16_t *>(&h); }
    }
  }
}

// ---- merge, 8 query rows of one head per block --------------------------------------------------------------------
constexpr int kMergeRowsPerBlock = 8;
template <int KIND, int D>
__global__ void __launch_bounds__(128) attn_merge_rows_kernel(uint16_t const *o_part, uint16_t const *r_part, uint16_t *out,
                                                              int heads, int m, int splits, long long o_stride,
                                                              long long r_stride, long long out_stride, MergeRuns runs) {
  asm volatile("griddepcontrol.wait;" ::: "memory"); // no-op unless launched with programmatic serialisation
  // The kernel before this one is complete now; the one behind it may be scheduled while this small grid runs (it
  // holds back its own stores until this grid has completed).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  int const chunks = (m + kMergeRowsPerBlock - 1) / kMergeRowsPerBlock;
  int const chunk = blockIdx.x % chunks, bh = blockIdx.x / chunks, head = bh % heads;
  long long const set = bh / heads;
  int const r0 = chunk * kMergeRowsPerBlock, rows = m - r0 < kMergeRowsPerBlock ? m - r0 : kMergeRowsPerBlock;
  uint16_t const *op = o_part + set * o_stride + ((long long)head * m + r0) * splits * D;
  uint16_t const *rp = r_part + set * r_stride + ((long long)head * m + r0) * splits;
  uint16_t *dst = out + set * out_stride + ((long long)head * m + r0) * D;
  merge_head<KIND, D>(op, rp, dst, rows, splits, (int)threadIdx.x, 128, held_slots(runs, (uint32_t)bh));
}

template <int KIND, int D>
static void launch_merge_rows_t(uint16_t const *o_part, uint16_t const *r_part, uint16_t *out, int heads, int m, int splits,
                                int num_sets, long long os, long long rs, long long outs, bool pdl, void *stream, MergeRuns runs) {
  cudaLaunchConfig_t cfg = {};
  int const chunks = (m + kMergeRowsPerBlock - 1) / kMergeRowsPerBlock;
  cfg.gridDim = dim3((unsigned)(heads * num_sets * chunks), 1, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (pdl) {
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaLaunchKernelEx(&cfg, attn_merge_rows_kernel<KIND, D>, o_part, r_part, out, heads, m, splits, os, rs, outs, runs);
}

bool launch_merge_rows(int kind, int d, uint16_t const *o_part, uint16_t const *r_part, uint16_t *out, int heads, int m,
                       int splits, int num_sets, long long os, long long rs, long long outs, bool pdl, void *stream, MergeRuns runs) {
  if (d != 64 && d != 128) return false;
#define MG_MERGE_CASE(K)                                                                                           \
  if (kind == K) {                                                                                                   \
    if (d == 128) launch_merge_rows_t<K, 128>(o_part, r_part, out, heads, m, splits, num_sets, os, rs, outs, pdl, stream, runs); \
    else launch_merge_rows_t<K, 64>(o_part, r_part, out, heads, m, splits, num_sets, os, rs, outs, pdl, stream, runs);       \
    return true;                                                                                                     \
  }
  MG_MERGE_CASE(kMergeF16)
  MG_MERGE_CASE(kMergeBF16)
  MG_MERGE_CASE(kMergeFingerprint)
#undef MG_MERGE_CASE
  return false;
}

// ---- host side ------------------------------------------------------------------------------------------------
using EncodeFn = TensorMapEncodeFn; // cuTensorMapEncodeTiled through the shared lookup (ptx.cuh)
static EncodeFn encode_fn() { return tensor_map_encoder(); }

// 3-D map over a [batch][rows][cols] array of 16-bit elements, box [1][box_rows][64], 128-byte swizzle
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

constexpr int kMaxDevices = 64;
static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  return dev;
}

static int sm_count() {
  static std::atomic<int> per_device[kMaxDevices];
  int dev = current_device();
  int n = per_device[dev].load(std::memory_order_relaxed);
  if (!n) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    per_device[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

static int groups_for(mgd_attn_split const *p, bool fp) { return fp ? (p->m + 3) / 4 : (p->m + 15) / 16; }

static bool shape_supported(mgd_attn_split const *p, bool fp) {
  if (!p || p->heads <= 0 || p->m <= 0 || p->splits <= 0 || p->forloop_range <= 0 || p->num_sets <= 0) return false;
  if (p->d != 64 && p->d != 128) return false;
  if ((int64_t)p->splits * p->forloop_range * kTile != p->kv_len) return false; // tiles of 64 KV positions
  if (groups_for(p, fp) > 2) return false;                                       // at most 8 warps per block
  if (fp && p->forloop_range > 256) return false;                                // int32 accumulators stay exact
  if (!fp && p->data_type != MG_DT_FLOAT16 && p->data_type != MG_DT_BFLOAT16) return false;
  if (p->causal_window < 0 || (p->causal_window > 0 && (fp || p->m % p->causal_window != 0))) return false;
  if (p->num_sets > 1) { // sets must be dense so that (set, head) folds into one TMA coordinate
    int64_t kv = (int64_t)p->heads * p->d * p->kv_len;
    if (p->k_set_stride != kv || p->v_set_stride != kv) return false;
  }
  return true;
}

// One instantiation per (mode, head_dim, operand forms); the shared-memory opt-in is set once for each.
template <int MODE, int DH, int FORM, bool PERSIST>
static int launch_form_as(cudaLaunchConfig_t cfg, CUtensorMap const &kmap, CUtensorMap const &vmap, AttnSplitParams const &a) {
  static std::atomic<bool> configured[kMaxDevices]; // the attribute is a property of the function on one device
  int const dev = current_device();
  if (!configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(attn_split_kernel<MODE, DH, FORM, PERSIST>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynSmemLimit) != cudaSuccess)
      return check_launch("cudaFuncSetAttribute(attn_split_kernel)");
    configured[dev].store(true, std::memory_order_release);
  }
  if (PERSIST) { // as many blocks as are resident at once; each walks its share of the work items
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_split_kernel<MODE, DH, FORM, PERSIST>, (int)cfg.blockDim.x,
                                                      cfg.dynamicSmemBytes) != cudaSuccess || per_sm <= 0)
      return check_launch("cudaOccupancyMaxActiveBlocksPerMultiprocessor(attn_split_kernel)");
    // A launch whose successor may start while it drains (programmatic stream serialisation) and whose blocks would
    // walk fewer than 48 KV tiles each leaves one block slot per SM to that successor: its first tiles then arrive
    // while this launch's last ones are worked on (launches of 4 to 32 decode calls: 4-14% faster; from about 48
    // tiles per block on, the third block's loads in flight are worth more than the overlap).
    if (per_sm >= 3 && cfg.numAttrs > 0 && (uint64_t)cfg.gridDim.x * (uint64_t)a.forloop < 48ull * (uint64_t)per_sm * (uint64_t)sm_count())
      per_sm = 2;
    unsigned resident = (unsigned)per_sm * (unsigned)sm_count();
    if (resident < cfg.gridDim.x) cfg.gridDim.x = resident;
  }
  AttnSplitParams launch = a;
  if (!PERSIST && a.early_loads && cfg.numAttrs > 0) {
    // the successor is released at once when this launch holds more than half of the block slots (see the kernel)
    static std::atomic<int> slots_per_sm[kMaxDevices]; // occupancy of this instantiation at the last (threads, smem) seen
    static std::atomic<uint64_t> slots_key[kMaxDevices];
    uint64_t const key = ((uint64_t)cfg.blockDim.x << 32) | (uint64_t)cfg.dynamicSmemBytes;
    int per_sm = slots_key[dev].load(std::memory_order_acquire) == key ? slots_per_sm[dev].load(std::memory_order_relaxed) : 0;
    if (per_sm <= 0) {
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_split_kernel<MODE, DH, FORM, PERSIST>, (int)cfg.blockDim.x,
                                                        cfg.dynamicSmemBytes) != cudaSuccess || per_sm <= 0)
        return check_launch("cudaOccupancyMaxActiveBlocksPerMultiprocessor(attn_split_kernel)");
      slots_per_sm[dev].store(per_sm, std::memory_order_relaxed);
      slots_key[dev].store(key, std::memory_order_release);
    }
    launch.early_release = 2ull * cfg.gridDim.x > (uint64_t)per_sm * (uint64_t)sm_count() ? 1 : 0;
  }
  cudaLaunchKernelEx(&cfg, attn_split_kernel<MODE, DH, FORM, PERSIST>, kmap, vmap, launch);
  return check_launch("attn_split_kernel");
}

template <int MODE, int DH, int FORM>
static int launch_form(cudaLaunchConfig_t const &cfg, CUtensorMap const &kmap, CUtensorMap const &vmap, AttnSplitParams const &a) {
  return a.persistent ? launch_form_as<MODE, DH, FORM, true>(cfg, kmap, vmap, a) : launch_form_as<MODE, DH, FORM, false>(cfg, kmap, vmap, a);
}

template <int MODE, int DH>
static int launch_split(mgd_attn_split const *p, void const *q, void const *k, void const *v, void *o, void *r,
                        mgd_attn_launch_opts const *opts, void *stream, int32_t *status_word = nullptr) {
  bool const fp = MODE == kFingerprint;
  int groups = groups_for(p, fp);
  int rows_scratch = fp ? 4 : (p->m < 16 ? p->m : 16);
  size_t acc = 4, tile = (size_t)kTile * DH * 2;
  size_t fixed = 1024 + kMaxStages * 8 + 256 + 16;
  int64_t blocks = (int64_t)p->heads * p->splits * p->num_sets;
  // One wave: request the whole split up front.  Many waves: shallow rings so that several blocks share an SM
  // and one block's loads overlap another's arithmetic.
  int stages = p->forloop_range < kMaxStages ? p->forloop_range : kMaxStages;
  if (blocks > sm_count() && stages > 2) stages = 2;
  while (stages > 1 && fixed + stages * 2 * tile > (size_t)kDynSmemLimit) stages--;
  // Warp groups that each take a different resident tile: the per-tile chain S -> exp -> E V is latency
  // bound, so tiles already in shared memory are worked on side by side (at most 16 warps per block).
  // With many waves the parallelism comes from several blocks per SM instead.
  int tile_groups = blocks > sm_count() ? 1 : (stages < 4 ? stages : 4);
  // Throughput sizing asked for by the caller (several launches in flight at once): the same small blocks, so that
  // blocks of different launches share an SM and one launch's loads run under another's arithmetic and tail.
  if (opts && (opts->overlap & 4)) {
    if (stages > 2) stages = 2;
    tile_groups = 1;
  }
  // tuning overrides (MGD_OPT_ATTN_STAGES, MGD_OPT_ATTN_TILE_GROUPS; 0 = the sizing above)
  if (int forced = option(MGD_OPT_ATTN_STAGES)) stages = forced > kMaxStages ? kMaxStages : forced;
  if (int forced = option(MGD_OPT_ATTN_TILE_GROUPS)) tile_groups = forced;
  if (stages > p->forloop_range) stages = p->forloop_range;
  if (tile_groups > stages) tile_groups = stages;
  while (tile_groups > 1 && groups * tile_groups * 128 > 512) tile_groups--;
  int threads = groups * tile_groups * 128;
  size_t scratch = (size_t)(threads / 32) * rows_scratch * (DH + 4) * acc;
  // More blocks than fit at once: resident blocks that walk the work items, their tile rings running on from one
  // item to the next (MGD_OPT_ATTN_PERSISTENT: 0 = this policy, 1 = never, 2 = whenever the shape allows it).
  int const persist_opt = option(MGD_OPT_ATTN_PERSISTENT);
  bool persistent = threads == 128 && persist_opt != 1 && blocks > sm_count() &&
                    fixed + stages * 2 * tile + scratch + 16 <= (size_t)kDynSmemLimit;
  // with a fused merge over scratch partials a persistent block sums up to a whole head in its accumulators: the
  // 32-bit integer ones of fingerprint mode are exact for 256 tiles
  bool sum_runs = persistent && opts && opts->merged_out && (opts->overlap & 8);
  if (fp && (int64_t)p->splits * p->forloop_range > 256) sum_runs = false;
  if (p->splits > 64) sum_runs = false; // the merge keeps one bit per split slot
  // A fused merge that must leave every partial in memory takes a ticket per item; a walking block would stall its
  // tile ring on each of them (measured: a third slower than one block per item), so it is not used there.
  if (opts && opts->merged_out && !sum_runs && persist_opt != 2) persistent = false;
  size_t data = persistent ? stages * 2 * tile + scratch : (scratch > stages * 2 * tile ? scratch : stages * 2 * tile);
  size_t smem = fixed + ((data + 15) & ~(size_t)15);

  if (smem > (size_t)kDynSmemLimit) return set_error(MG_ERR_UNSUPPORTED, "split-KV attention: tile does not fit shared memory");

  CUtensorMap kmap, vmap;
  uint64_t batch = (uint64_t)p->heads * p->num_sets;
  // Float tensors sit in memory as their layout tag says; fingerprint buffers are always logical row-major
  // (the reference indexes them so whatever the tag): K as [d][kv], V as [kv][d].
  bool k_kv = !fp && p->k_layout == MG_DMEM_COLUMN_MAJOR, v_kv = fp || p->v_layout == MG_DMEM_ROW_MAJOR;
  bool ok = k_kv ? make_map(&kmap, k, batch, p->kv_len, DH, kTile) : make_map(&kmap, k, batch, DH, p->kv_len, DH);
  ok = ok && (v_kv ? make_map(&vmap, v, batch, p->kv_len, DH, kTile) : make_map(&vmap, v, batch, DH, p->kv_len, DH));
  if (!ok) return set_error(MG_ERR_CUDA, "split-KV attention: cuTensorMapEncodeTiled failed");

  AttnSplitParams a;
  a.q = q; a.o_part = o; a.r_part = r;
  a.status = status_word ? status_word : device_error_word();
  if (!a.status) return set_error(MG_ERR_CUDA, "cannot allocate the device status word");
  a.q_set_stride = p->q_set_stride; a.o_set_stride = p->o_set_stride; a.r_set_stride = p->r_set_stride;
  a.heads = p->heads; a.m = p->m; a.splits = p->splits; a.forloop = p->forloop_range; a.stages = stages;
  a.tile_groups = tile_groups;
  a.num_sets = p->num_sets;
  a.persistent = persistent ? 1 : 0;
  a.sum_runs = sum_runs ? 1 : 0;
  a.merged_out = opts ? opts->merged_out : nullptr;
  a.tickets = opts ? opts->tickets : nullptr;
  a.merged_set_stride = opts ? opts->merged_set_stride : 0;
  a.early_loads = opts && (opts->overlap & 2) ? 1 : 0;
  a.early_release = 0; // decided per launch form, where the block slots are known
  // MGD_OPT_WAIT_LIMIT: 0 = default, 1 = give up without polling, n = n polls
  int const forced_limit = option(MGD_OPT_WAIT_LIMIT);
  a.wait_limit = forced_limit == 0 ? ptx::kWaitLimit : (forced_limit == 1 ? 0 : forced_limit);
  if (a.merged_out && !a.tickets) return set_error(MG_ERR_INVALID_ARGUMENT, "split-KV attention: merging needs ticket counters");
  a.kv_len = p->kv_len; a.k_rows_are_kv = k_kv; a.v_rows_are_kv = v_kv; a.causal_window = p->causal_window;

  if (blocks > 0x7fffffffLL) return set_error(MG_ERR_UNSUPPORTED, "too many blocks for one launch");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks, 1, 1);
  cfg.blockDim = dim3((unsigned)threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (opts && (opts->overlap & 1)) {
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  if constexpr (MODE == kFingerprint) return launch_form<MODE, DH, 2>(cfg, kmap, vmap, a);
  else switch ((k_kv ? 1 : 0) | (v_kv ? 2 : 0)) {
    case 0: return launch_form<MODE, DH, 0>(cfg, kmap, vmap, a);
    case 1: return launch_form<MODE, DH, 1>(cfg, kmap, vmap, a);
    case 2: return launch_form<MODE, DH, 2>(cfg, kmap, vmap, a);
    default: return launch_form<MODE, DH, 3>(cfg, kmap, vmap, a);
  }
}
// ---- scratch of the allocation-free entry point ---------------------------------------------------------------
// One ticket counter per (input set, head) followed by one status word.  The array lives in the library image:
// every GPU that loads the library holds these 16.6 KB until the process exits.  On the host the name below is
// only a handle for cudaGetSymbolAddress - it is NOT a device address and must never be handed to a kernel.
constexpr int kNoAllocMaxHeads = 4096;
static __device__ __align__(256) int32_t g_noalloc_scratch[kNoAllocMaxHeads + 64];

// Device address of g_noalloc_scratch on the current device; looked up once per device.
static int noalloc_scratch(int32_t **ptr) {
  static int32_t *per_device[64] = {nullptr};
  static std::mutex mutex;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return set_error(MG_ERR_CUDA, "no current CUDA device");
  std::lock_guard<std::mutex> lock(mutex);
  if (!per_device[dev]) {
    void *addr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&addr, g_noalloc_scratch);
    if (e != cudaSuccess || !addr) {
      cudaGetLastError();
      return set_error(MG_ERR_CUDA, "cudaGetSymbolAddress(g_noalloc_scratch) failed");
    }
    per_device[dev] = static_cast<int32_t *>(addr);
  }
  *ptr = per_device[dev];
  return MG_OK;
}
} // namespace mgk

using namespace mgk;

extern "C" {

int mgd_attn_decode_fused_noalloc(const mgd_attn_split *p, const void *q, const void *k, const void *v, void *o_part,
                                  void *r_part, void *out, int32_t fingerprint_mode, int32_t check_status,
                                  void *stream) {
  if (!p || !q || !k || !v || !o_part || !r_part || !out)
    return set_error(MG_ERR_INVALID_ARGUMENT, "allocation-free decode: null argument");
  bool const fp = fingerprint_mode != 0;
  if (!shape_supported(p, fp)) return set_error(MG_ERR_UNSUPPORTED, "allocation-free decode: shape not supported");
  int64_t counters = (int64_t)p->heads * p->num_sets;
  if (counters > kNoAllocMaxHeads)
    return set_error(MG_ERR_INVALID_ARGUMENT,
                     "allocation-free decode: heads * num_sets exceeds the 4096 ticket counters of the built-in scratch");
  int32_t *scratch = nullptr;
  int st = noalloc_scratch(&scratch);
  if (st != MG_OK) return st;
  // the counters must start at zero; an earlier call that was cut short may have left some behind.  The status
  // word is cleared as well, so that what a call reports is its own: a timeout of an earlier call that nobody
  // checked (check_status = 0) is forgotten here.
  int32_t *status = scratch + kNoAllocMaxHeads;
  if (cudaMemsetAsync(scratch, 0, (size_t)counters * sizeof(int32_t), (cudaStream_t)stream) != cudaSuccess ||
      cudaMemsetAsync(status, 0, sizeof(int32_t), (cudaStream_t)stream) != cudaSuccess)
    return check_launch("cudaMemsetAsync(ticket counters)");
  mgd_attn_launch_opts opts;
  opts.merged_out = out;
  opts.tickets = scratch;
  opts.merged_set_stride = (int64_t)p->heads * p->m * p->d;
  opts.overlap = 0;
  opts.reserved = 0;
  if (fp)
    st = p->d == 128 ? launch_split<kFingerprint, 128>(p, q, k, v, o_part, r_part, &opts, stream, status)
                     : launch_split<kFingerprint, 64>(p, q, k, v, o_part, r_part, &opts, stream, status);
  else if (p->data_type == MG_DT_FLOAT16)
    st = p->d == 128 ? launch_split<kF16, 128>(p, q, k, v, o_part, r_part, &opts, stream, status)
                     : launch_split<kF16, 64>(p, q, k, v, o_part, r_part, &opts, stream, status);
  else
    st = p->d == 128 ? launch_split<kBF16, 128>(p, q, k, v, o_part, r_part, &opts, stream, status)
                     : launch_split<kBF16, 64>(p, q, k, v, o_part, r_part, &opts, stream, status);
  if (st != MG_OK || !check_status) return st;
  if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) return check_launch("cudaStreamSynchronize");
  int32_t code = 0;
  if (cudaMemcpy(&code, status, sizeof(code), cudaMemcpyDeviceToHost) != cudaSuccess) return check_launch("status read");
  if (code != 0) {
    cudaMemset(status, 0, sizeof(code));
    return set_error(MG_ERR_DEVICE_TIMEOUT, "allocation-free decode: a bounded device wait gave up; outputs are incomplete");
  }
  return MG_OK;
}

int mgd_attn_split_supported(const mgd_attn_split *p, int32_t fingerprint_mode) {
  return shape_supported(p, fingerprint_mode != 0) && encode_fn() != nullptr ? 1 : 0;
}

// Which engine runs a float launch: with more than 8 query rows the mma.sync path is bound by the legacy tensor
// pipe and the tcgen05 kernel (attn_split_tc.cu) takes over where it supports the shape.
// MGD_OPT_ATTN_ENGINE forces the choice (tuning, tests).
static bool use_tensor_memory_kernel(mgd_attn_split const *p) {
  if (!stc::supported(p)) return false;
  if (int forced = option(MGD_OPT_ATTN_ENGINE)) return forced == 2;
  return p->m > 8;
}

int mgd_launch_attn_split_float_ex(const mgd_attn_split *p, const void *q, const void *k, const void *v, void *o,
                                   void *r, const mgd_attn_launch_opts *opts, void *stream) {
  if (!q || !k || !v || !o || !r) return set_error(MG_ERR_INVALID_ARGUMENT, "split-KV attention: null tensor");
  if (!shape_supported(p, false)) return set_error(MG_ERR_UNSUPPORTED, "split-KV attention: shape not supported");
  if (use_tensor_memory_kernel(p)) return stc::launch(p, q, k, v, o, r, opts, stream);
  if (p->data_type == MG_DT_FLOAT16)
    return p->d == 128 ? launch_split<kF16, 128>(p, q, k, v, o, r, opts, stream) : launch_split<kF16, 64>(p, q, k, v, o, r, opts, stream);
  return p->d == 128 ? launch_split<kBF16, 128>(p, q, k, v, o, r, opts, stream) : launch_split<kBF16, 64>(p, q, k, v, o, r, opts, stream);
}

int mgd_launch_attn_split_fingerprint_ex(const mgd_attn_split *p, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                         uint16_t *o, uint16_t *r, const mgd_attn_launch_opts *opts, void *stream) {
  if (!q || !k || !v || !o || !r) return set_error(MG_ERR_INVALID_ARGUMENT, "split-KV attention: null tensor");
  if (!shape_supported(p, true)) return set_error(MG_ERR_UNSUPPORTED, "split-KV attention: shape not supported");
  return p->d == 128 ? launch_split<kFingerprint, 128>(p, q, k, v, o, r, opts, stream)
                     : launch_split<kFingerprint, 64>(p, q, k, v, o, r, opts, stream);
}

int mgd_launch_attn_split_float(const mgd_attn_split *p, const void *q, const void *k, const void *v, void *o,
                                void *r, void *stream) {
  return mgd_launch_attn_split_float_ex(p, q, k, v, o, r, nullptr, stream);
}

int mgd_launch_attn_split_fingerprint(const mgd_attn_split *p, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                      uint16_t *o, uint16_t *r, void *stream) {
  return mgd_launch_attn_split_fingerprint_ex(p, q, k, v, o, r, nullptr, stream);
}

int mgd_attn_merge_supported(const mgd_attn_merge *p, int32_t) {
  return p && p->heads > 0 && p->m > 0 && p->d > 0 && p->splits > 0 && p->splits <= 65536 ? 1 : 0;
}

int mgd_launch_attn_merge_float(const mgd_attn_merge *p, const void *o_part, const void *r_part, void *out, void *stream) {
  if (!p || !o_part || !r_part || !out || p->num_sets <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "attention merge: bad argument");
  if (p->data_type == MG_DT_FLOAT16 || p->data_type == MG_DT_BFLOAT16)
    if (launch_merge_rows(p->data_type == MG_DT_BFLOAT16 ? kMergeBF16 : kMergeF16, p->d, (uint16_t const *)o_part,
                          (uint16_t const *)r_part, (uint16_t *)out, p->heads, p->m, p->splits, p->num_sets,
                          p->o_part_set_stride, p->r_part_set_stride, p->out_set_stride, false, stream))
      return check_launch("attn_merge_rows_kernel");
  unsigned blocks = (unsigned)(p->heads * p->num_sets);
  if (p->data_type == MG_DT_FLOAT16)
    attn_merge_kernel<kF16><<<blocks, 256, 0, (cudaStream_t)stream>>>((uint16_t const *)o_part, (uint16_t const *)r_part, (uint16_t *)out,
        p->heads, p->m, p->d, p->splits, p->o_part_set_stride, p->r_part_set_stride, p->out_set_stride);
  else if (p->data_type == MG_DT_BFLOAT16)
    attn_merge_kernel<kBF16><<<blocks, 256, 0, (cudaStream_t)stream>>>((uint16_t const *)o_part, (uint16_t const *)r_part, (uint16_t *)out,
        p->heads, p->m, p->d, p->splits, p->o_part_set_stride, p->r_part_set_stride, p->out_set_stride);
  else
    return set_error(MG_ERR_UNSUPPORTED, "attention merge: fp16 or bf16 only");
  return check_launch("attn_merge_kernel");
}

int mgd_launch_attn_merge_fingerprint(const mgd_attn_merge *p, const uint16_t *o_part, const uint16_t *r_part, uint16_t *out, void *stream) {
  if (!p || !o_part || !r_part || !out || p->num_sets <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "attention merge: bad argument");
  if (launch_merge_rows(kMergeFingerprint, p->d, o_part, r_part, out, p->heads, p->m, p->splits, p->num_sets,
                        p->o_part_set_stride, p->r_part_set_stride, p->out_set_stride, false, stream))
    return check_launch("attn_merge_rows_kernel");
  unsigned blocks = (unsigned)(p->heads * p->num_sets);
  attn_merge_kernel<kFingerprint><<<blocks, 256, 0, (cudaStream_t)stream>>>(o_part, r_part, out, p->heads, p->m, p->d, p->splits,
                                                                            p->o_part_set_stride, p->r_part_set_stride, p->out_set_stride);
  return check_launch("attn_merge_kernel");
}
}
