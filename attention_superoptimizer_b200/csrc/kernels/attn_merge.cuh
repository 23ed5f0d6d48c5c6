// Cross-split merge of one head, shared by the split-KV kernels: O = (sum over splits of O_part) / (sum over splits
// of R_part)  - the second customized op of the reference's cpp_examples/group_query_attn_inc_decode.cc:80-103 -
// done by the block that finished the head's last split.
//
// The partials were written by other SMs a moment ago, so every load is an L2 round trip: the work is arranged
// for memory-level parallelism.  A thread owns 8 adjacent output columns of one row and issues the 16-byte loads
// of up to 16 splits - and of its row's denominators - before it uses any of them.
#pragma once
#include "common.cuh"

namespace mgk {

enum { kMergeF16 = 0, kMergeBF16 = 1, kMergeFingerprint = 2 };

template <int KIND> __device__ __forceinline__ float merge_to_float(uint16_t v) {
  if (KIND == kMergeBF16) return __bfloat162float(*reinterpret_cast<__nv_bfloat16 const *>(&v));
  return __half2float(*reinterpret_cast<__half const *>(&v));
}
template <int KIND> __device__ __forceinline__ uint32_t merge_pack(float a, float b) {
  if (KIND == kMergeBF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

// op: [m][splits * D], rp: [m][splits], dst: [m][D] of one head; t / nt: index and count of the participating
// threads.  Every thread also sums its row's denominators itself (a few 16-byte loads that travel with the others):
// one L2 round trip per 16 splits, no barrier.
// held: bit s set = slot s holds a sum (bits beyond 63 count as set).  The split-KV kernel clears bits when it has
// summed several consecutive splits on the chip and written only the first slot of the run; the other slots were
// never written: they are loaded with the others (the memory is there) and left out of the sums.
template <int KIND, int D>
__device__ __forceinline__ void merge_head(uint16_t const *op, uint16_t const *rp, uint16_t *dst, int m, int splits,
                                           int t, int nt, uint64_t held = ~0ull) {
  auto holds = [&](int sp) { return sp >= 64 || ((held >> sp) & 1ull) != 0; };
  constexpr int kGroups = D / 8;
  size_t const out_ld = (size_t)splits * D;
  bool const r_vec = (splits & 7) == 0 && (reinterpret_cast<uintptr_t>(rp) & 15) == 0; // rows of R are 16-byte pieces
  for (int u = t; u < m * kGroups; u += nt) {
    int const r = u / kGroups, c = (u % kGroups) * 8;
    uint16_t const *src = op + (size_t)r * out_ld + c;
    uint16_t const *rrow = rp + (size_t)r * splits;
    float facc[8], fden = 0.f;
    uint32_t iacc[8], iden = 0u;
#pragma unroll
    for (int i = 0; i < 8; i++) facc[i] = 0.f, iacc[i] = 0u;
    auto add = [&](uint4 w) {
      uint32_t const words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; i++) {
        if (KIND == kMergeFingerprint) {
          iacc[2 * i] += words[i] & 0xFFFFu;
          iacc[2 * i + 1] += words[i] >> 16;
        } else {
          facc[2 * i] += merge_to_float<KIND>((uint16_t)(words[i] & 0xFFFFu));
          facc[2 * i + 1] += merge_to_float<KIND>((uint16_t)(words[i] >> 16));
        }
      }
    };
    auto add_den = [&](uint16_t v) {
      if (KIND == kMergeFingerprint) iden += v;
      else fden += merge_to_float<KIND>(v);
    };
    auto add_den8 = [&](uint4 w, int first) { // denominators of slots first .. first + 7
      uint32_t const words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; i++) {
        if (holds(first + 2 * i)) add_den((uint16_t)(words[i] & 0xFFFFu));
        if (holds(first + 2 * i + 1)) add_den((uint16_t)(words[i] >> 16));
      }
    };
    int sp = 0;
    for (; sp + 16 <= splits; sp += 16) { // sums of 65536 values < 25651 still fit 32 bits
      uint4 w[16], rv[2];
      uint16_t rs[16];
#pragma unroll
      for (int i = 0; i < 16; i++) w[i] = __ldcg(reinterpret_cast<uint4 const *>(src + (size_t)(sp + i) * D));
      if (r_vec) {
        rv[0] = __ldcg(reinterpret_cast<uint4 const *>(rrow + sp));
        rv[1] = __ldcg(reinterpret_cast<uint4 const *>(rrow + sp + 8));
      } else {
#pragma unroll
        for (int i = 0; i < 16; i++) rs[i] = __ldcg(rrow + sp + i);
      }
#pragma unroll
      for (int i = 0; i < 16; i++)
        if (holds(sp + i)) add(w[i]);
      if (r_vec) {
        add_den8(rv[0], sp);
        add_den8(rv[1], sp + 8);
      } else {
#pragma unroll
        for (int i = 0; i < 16; i++)
          if (holds(sp + i)) add_den(rs[i]);
      }
    }
    for (; sp + 4 <= splits; sp += 4) {
      uint4 w[4];
      uint16_t rs[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        w[i] = __ldcg(reinterpret_cast<uint4 const *>(src + (size_t)(sp + i) * D));
        rs[i] = __ldcg(rrow + sp + i);
      }
#pragma unroll
      for (int i = 0; i < 4; i++)
        if (holds(sp + i)) {
          add(w[i]);
          add_den(rs[i]);
        }
    }
    for (; sp < splits; sp++)
      if (holds(sp)) {
        add(__ldcg(reinterpret_cast<uint4 const *>(src + (size_t)sp * D)));
        add_den(__ldcg(rrow + sp));
      }
    uint32_t o[4];
    if (KIND == kMergeFingerprint) {
      uint32_t const den = iden % PQ;
#pragma unroll
      for (int i = 0; i < 4; i++) o[i] = field_div(iacc[2 * i] % PQ, den) | (field_div(iacc[2 * i + 1] % PQ, den) << 16);
    } else {
#pragma unroll
      for (int i = 0; i < 4; i++) o[i] = merge_pack<KIND>(facc[2 * i] / fden, facc[2 * i + 1] / fden);
    }
    *reinterpret_cast<uint4 *>(dst + (size_t)r * D + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Which slots hold sums when the split-KV kernel summed runs of tiles: the launch's tiles were dealt to blocks in
// order, `per` tiles each and the first `extra` blocks one more; a head's tiles [unit * tiles_per_head, + tiles_per_head)
// then lie in consecutive blocks, and block i of them wrote slot i.  per = 0: every slot holds a sum.
struct MergeRuns {
  uint32_t per, extra, tiles_per_head;
};
__device__ __forceinline__ uint64_t held_slots(MergeRuns const &runs, uint32_t unit) {
  if (runs.per == 0) return ~0ull;
  uint32_t const wide = runs.extra * (runs.per + 1);
  auto block_of = [&](uint32_t g) { return g < wide ? g / (runs.per + 1) : runs.extra + (g - wide) / runs.per; };
  uint32_t const count = block_of((unit + 1) * runs.tiles_per_head - 1) - block_of(unit * runs.tiles_per_head) + 1;
  return count >= 64 ? ~0ull : ((1ull << count) - 1ull);
}

// Stand-alone merge launch (attn_split.cu): blocks of 128 threads take 8 query rows of one head each.  With
// `after_previous_kernel` the launch uses programmatic stream serialisation: its blocks are scheduled while the
// previous kernel of the stream drains and wait (griddepcontrol.wait) until that kernel's memory is visible.
// kind: kMergeF16 / kMergeBF16 / kMergeFingerprint; d must be 64 or 128 (returns false otherwise, nothing launched).
bool launch_merge_rows(int kind, int d, uint16_t const *o_part, uint16_t const *r_part, uint16_t *out, int heads, int m,
                       int splits, int num_sets, long long o_set_stride, long long r_set_stride, long long out_set_stride,
                       bool after_previous_kernel, void *stream, MergeRuns runs = MergeRuns{0, 0, 0});

} // namespace mgk
