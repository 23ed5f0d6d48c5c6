// Two chained threadblock matmuls with for-loop accumulation as one kernel:
//     out[block] = sum over the for-loop of (X_i W1_i) W2  =  (sum_i X_i W1_i) W2      (W2 the same in every iteration)
// - the fused "matmul chain" customized operator (two tb_matmul_op feeding a tb_output_op that accumulates over the
// for-loop, as in the reference's cpp_examples/mlp.cc and its lora.cc building blocks).  The generic interpreters run
// this plan one operator and one barrier at a time, which costs more than the arithmetic; here the whole block is two
// tensor-core loops around a cp.async pipeline:
//   phase 1  the X_i and W1_i tiles stream through a ring of stages (16-byte cp.async, all stages requested up front,
//            one refill per iteration); every warp owns 8-column slices of the [m x n1] running sum, which stays in
//            registers over the whole for-loop (fp32; int32 byte-plane sums in fingerprint mode);
//   phase 2  the running sum becomes the A operand of the second product: in float mode as a 16-bit value (bf16: plus
//            the 16-bit rounding residual, two MMAs per step), in fingerprint mode reduced modulo PQ; W2's tile [n1 x n2] was requested behind the first stages and is read in place.
// Float mode: mma.sync m16n8k16 fp16 / bf16 with fp32 accumulation.  Fingerprint mode: the exact byte-plane scheme
// of fp_interp.cu on mma.sync m16n8k32 u8.  m <= 16 rows (an MMA's height); rows beyond m are zero and never stored.
#include "common.cuh"
#include <cstring>

namespace mgk {
namespace chain {

constexpr int kThreads = 256, kWarps = 8;
constexpr int kPad = 8; // elements added to every shared-memory row: ldmatrix rows land in different banks

struct Params {
  mgd_matmul_chain c;
  void const *x, *w1, *w2;
  void *out;
  long long x_set, w1_set, w2_set, out_set;
  int stages;
};

__device__ __forceinline__ void cp_async16(void *dst, void const *src) {
  uint32_t const d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// wait until at most `pending` (0..6) of the most recent groups are still in flight
__device__ __forceinline__ void cp_wait_pending(int pending) {
  switch (pending) {
    case 0: cp_wait<0>(); break;
    case 1: cp_wait<1>(); break;
    case 2: cp_wait<2>(); break;
    case 3: cp_wait<3>(); break;
    case 4: cp_wait<4>(); break;
    case 5: cp_wait<5>(); break;
    default: cp_wait<6>(); break;
  }
}

// first element of an input tile of this block in iteration `it` (row-major tensor, `ld` = tensor columns)
__device__ __forceinline__ long long tile_origin(mgd_op const &op, int bx, int by, int bz, int it) {
  int32_t const *a = op.a;
  long long const row = (long long)bx * a[0] + (long long)by * a[1] + (long long)bz * a[2] + (long long)it * a[6];
  long long const col = (long long)bx * a[3] + (long long)by * a[4] + (long long)bz * a[5] + (long long)it * a[7];
  long long const lead = (long long)bx * a[8] + (long long)by * a[9] + (long long)bz * a[10] + (long long)it * a[11];
  return lead + row * a[MGD_IN_COLS] + col;
}

// rows x cols 16-bit elements (cols a multiple of 8) from global memory into padded shared-memory rows
__device__ __forceinline__ void request_tile(uint16_t *dst, int pitch, uint16_t const *src, int ld, int rows, int cols, int tid) {
  int const per_row = cols >> 3;
  for (int i = tid; i < rows * per_row; i += kThreads) {
    int const r = i / per_row, c = (i - r * per_row) << 3;
    cp_async16(dst + r * pitch + c, src + (long long)r * ld + c);
  }
}

template <int MODE> struct Mma; // 0 fp16, 1 bf16
template <> struct Mma<0> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t v) { return __half22float2(*reinterpret_cast<__half2 *>(&v)); }
};
template <> struct Mma<1> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t v) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&v)); }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], void const *p) {
  uint32_t const a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], void const *p) {
  uint32_t const a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// Shared-memory plan (16-bit elements): [stages x (X tile 16 x (kt + pad) | W1 tile kt x (n1 + pad))] [W2 n1 x (n2 + pad)]
// [running sum as A operand: hi 16 x (n1 + pad), lo 16 x (n1 + pad)]
struct Plan {
  int x_pitch, w1_pitch, w2_pitch, a2_pitch;
  size_t stage_elems, w2_at, a2_at, total_bytes;
};
__host__ __device__ inline Plan make_plan(int kt, int n1, int n2, int stages) {
  Plan q;
  q.x_pitch = kt + kPad; q.w1_pitch = n1 + kPad; q.w2_pitch = n2 + kPad; q.a2_pitch = n1 + kPad;
  q.stage_elems = (size_t)16 * q.x_pitch + (size_t)kt * q.w1_pitch;
  q.w2_at = (size_t)stages * q.stage_elems;
  q.a2_at = q.w2_at + (size_t)n1 * q.w2_pitch;
  q.total_bytes = (q.a2_at + (size_t)2 * 16 * q.a2_pitch) * 2;
  return q;
}

// MODE: 0 fp16, 1 bf16, 2 fingerprints
template <int MODE>
__global__ void __launch_bounds__(kThreads) chain_kernel(const __grid_constant__ Params p) {
  extern __shared__ __align__(16) uint16_t smem[];
  mgd_matmul_chain const &c = p.c;
  int const tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  int const gx = c.grid[0], gy = c.grid[1], gz = c.grid[2];
  long long const b = blockIdx.x;
  int const bx = (int)(b % gx), by = (int)((b / gx) % gy), bz = (int)((b / ((long long)gx * gy)) % gz);
  long long const set = b / ((long long)gx * gy * gz);
  int const m = c.m, kt = c.kt, n1 = c.n1, n2 = c.n2, loop = c.forloop_range, S = p.stages;
  Plan const q = make_plan(kt, n1, n2, S);
  uint16_t const *X = static_cast<uint16_t const *>(p.x) + set * p.x_set;
  uint16_t const *W1 = static_cast<uint16_t const *>(p.w1) + set * p.w1_set;
  uint16_t const *W2 = static_cast<uint16_t const *>(p.w2) + set * p.w2_set;
  // What a thread copies per stage is the same in every iteration but for the tile's position, which moves by a
  // constant: the 16-byte pieces of this thread (one of X's, up to 8 of W1's) are worked out once, so that a stage
  // request is a handful of additions (with 8 warps on the SM, address arithmetic per iteration is what the loop cost).
  constexpr int kMaxW1Pieces = 8; // kt, n1 <= 128: 128 * 128 / 8 pieces over 256 threads
  long long const x_step = (long long)c.x.a[6] * c.x.a[MGD_IN_COLS] + c.x.a[7] + c.x.a[11];
  long long const w1_step = (long long)c.w1.a[6] * c.w1.a[MGD_IN_COLS] + c.w1.a[7] + c.w1.a[11];
  uint16_t const *x_src = nullptr;
  int x_dst = 0;
  {
    int const per_row = kt >> 3;
    if (tid < m * per_row) {
      int const r = tid / per_row, cc = (tid - r * per_row) << 3;
      x_src = X + tile_origin(c.x, bx, by, bz, 0) + (long long)r * c.x.a[MGD_IN_COLS] + cc;
      x_dst = r * q.x_pitch + cc;
    }
  }
  uint16_t const *w1_src[kMaxW1Pieces];
  int w1_dst[kMaxW1Pieces];
  {
    int const per_row = n1 >> 3;
    uint16_t const *origin = W1 + tile_origin(c.w1, bx, by, bz, 0);
#pragma unroll
    for (int j = 0; j < kMaxW1Pieces; j++) {
      int const i = tid + j * kThreads;
      w1_src[j] = nullptr;
      w1_dst[j] = 0;
      if (i < kt * per_row) {
        int const r = i / per_row, cc = (i - r * per_row) << 3;
        w1_src[j] = origin + (long long)r * c.w1.a[MGD_IN_COLS] + cc;
        w1_dst[j] = 16 * q.x_pitch + r * q.w1_pitch + cc;
      }
    }
  }
  auto request_stage = [&](int it) {
    uint16_t *stage = smem + (size_t)(it % S) * q.stage_elems;
    if (x_src != nullptr) cp_async16(stage + x_dst, x_src + it * x_step);
#pragma unroll
    for (int j = 0; j < kMaxW1Pieces; j++)
      if (w1_src[j] != nullptr) cp_async16(stage + w1_dst[j], w1_src[j] + it * w1_step);
  };
  // rows of the X tiles beyond m stay zero
  if (m < 16)
    for (int s = 0; s < S; s++)
      for (int i = tid; i < (16 - m) * q.x_pitch; i += kThreads) smem[(size_t)s * q.stage_elems + m * q.x_pitch + i] = 0;
  // One group per stage: stages 0 .. S - 2 now (W2, needed last, rides in the last of them), then one per iteration.
  // Stage `it` is group number `it`, and S - 1 + it groups exist when iteration `it` waits: at most S - 2 of the
  // most recent ones may still be in flight.
  for (int s = 0; s < S - 1; s++) {
    if (s < loop) request_stage(s);
    if (s == S - 2) request_tile(smem + q.w2_at, q.w2_pitch, W2 + tile_origin(c.w2, bx, by, bz, 0), c.w2.a[MGD_IN_COLS], n1, n2, tid);
    cp_commit();
  }

  uint16_t const *w2s = smem + q.w2_at;
  int32_t const *oa = c.out.a;
  long long const orow = (long long)bx * oa[0] + (long long)by * oa[1] + (long long)bz * oa[2];
  long long const ocol = (long long)bx * oa[3] + (long long)by * oa[4] + (long long)bz * oa[5];
  long long const olead = (long long)bx * oa[6] + (long long)by * oa[7] + (long long)bz * oa[8];
  int const old = oa[MGD_OUT_COLS];
  uint16_t *O = static_cast<uint16_t *>(p.out) + set * p.out_set + olead + orow * old + ocol;
  if constexpr (MODE != 2) {
  // ---- phase 1: running sum of X_i W1_i.  The contraction is split over the warps: warp w takes the k-steps
  // w % 4, w % 4 + 4, ... of every tile and the 8-column slices w / 4, w / 4 + 2, ...: the MMAs of an iteration go
  // to different accumulators (a dependent MMA chain runs at about 100 cycles per step, the pipe takes one every 8),
  // and the four partial sums of a slice are added in shared memory afterwards.
  constexpr int kMaxSlices = 8; // n1 <= 128: 16 slices, two interleaved halves
  float acc[kMaxSlices][4];
#pragma unroll
  for (int i = 0; i < kMaxSlices; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  int const slices = n1 >> 3, kq = warp & 3, sh = warp >> 2;
  for (int it = 0; it < loop; it++) {
    cp_wait_pending(S - 2); // stage `it` has landed (for this thread's copies; the barrier makes it everybody's)
    __syncthreads();        // also: every warp is done with stage it - 1, which the refill below overwrites
    if (it + S - 1 < loop) request_stage(it + S - 1);
    cp_commit();
    uint16_t const *xs = smem + (size_t)(it % S) * q.stage_elems, *ws = xs + 16 * q.x_pitch;
    for (int ks = kq * 16; ks < kt; ks += 64) {
      uint32_t a[4];
      ldmatrix_x4(a, xs + (lane & 15) * q.x_pitch + ks + ((lane >> 4) << 3));
#pragma unroll
      for (int i = 0; i < kMaxSlices; i += 2) { // two slices per ldmatrix: columns sl*8 .. +7 and (sl + 2)*8 .. +7
        int const sl = sh + 2 * i;
        if (sl < slices) {
          uint32_t bfr[4];
          ldmatrix_x4_trans(bfr, ws + (ks + (lane & 15)) * q.w1_pitch + (sl + ((lane >> 4) << 1)) * 8);
          Mma<MODE>::run(acc[i], a, bfr[0], bfr[1]);
          if (sl + 2 < slices) Mma<MODE>::run(acc[i + 1], a, bfr[2], bfr[3]);
        }
      }
    }
  }
  // ---- the four partial sums of every slice are added, and the running sum becomes an A operand: the value
  // rounded to 16 bits, and the rounding residual -------------------------------------------------------------------
  __syncthreads(); // every stage has been read: the ring's memory is free for the partial sums [4][16][n1] (fp32)
  float *partial = reinterpret_cast<float *>(smem);
#pragma unroll
  for (int i = 0; i < kMaxSlices; i++) {
    int const sl = sh + 2 * i;
    if (sl < slices) {
      float *dst = partial + ((size_t)kq * 16) * n1 + sl * 8 + 2 * t;
      *reinterpret_cast<float2 *>(dst + (size_t)g * n1) = make_float2(acc[i][0], acc[i][1]);
      *reinterpret_cast<float2 *>(dst + (size_t)(g + 8) * n1) = make_float2(acc[i][2], acc[i][3]);
    }
  }
  __syncthreads();
  uint16_t *a2_hi = smem + q.a2_at, *a2_lo = a2_hi + 16 * q.a2_pitch;
  for (int i = tid; i < 16 * (n1 >> 1); i += kThreads) {
    int const r = i / (n1 >> 1), cc = (i - r * (n1 >> 1)) << 1;
    float2 v = make_float2(0.f, 0.f);
#pragma unroll
    for (int k4 = 0; k4 < 4; k4++) {
      float2 const u = *reinterpret_cast<float2 const *>(partial + ((size_t)k4 * 16 + r) * n1 + cc);
      v.x += u.x; v.y += u.y;
    }
    uint32_t const h = Mma<MODE>::pack(v.x, v.y);
    float2 const f = Mma<MODE>::unpack(h);
    *reinterpret_cast<uint32_t *>(a2_hi + r * q.a2_pitch + cc) = h;
    *reinterpret_cast<uint32_t *>(a2_lo + r * q.a2_pitch + cc) = Mma<MODE>::pack(v.x - f.x, v.y - f.y);
  }
  cp_wait<0>();
  __syncthreads();

  // ---- phase 2: out = running sum x W2; a warp takes 16 columns at a time --------------------------------------
  constexpr int kMaxK2 = 8; // n1 <= 128
  uint32_t ah[kMaxK2][4], al[kMaxK2][4];
  int const k2 = n1 >> 4;
#pragma unroll
  for (int ks = 0; ks < kMaxK2; ks++)
    if (ks < k2) {
      ldmatrix_x4(ah[ks], a2_hi + (lane & 15) * q.a2_pitch + ks * 16 + ((lane >> 4) << 3));
      if (MODE == 1) ldmatrix_x4(al[ks], a2_lo + (lane & 15) * q.a2_pitch + ks * 16 + ((lane >> 4) << 3));
    }
  // four 16-column blocks at a time: eight independent accumulate chains per warp
  constexpr int kCB = 4;
  for (int cb0 = warp * kCB; cb0 < (n2 >> 4); cb0 += kWarps * kCB) {
    float d[kCB][2][4];
#pragma unroll
    for (int u = 0; u < kCB; u++)
#pragma unroll
      for (int h = 0; h < 2; h++)
#pragma unroll
        for (int j = 0; j < 4; j++) d[u][h][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < kMaxK2; ks++)
      if (ks < k2) {
#pragma unroll
        for (int u = 0; u < kCB; u++)
          if (cb0 + u < (n2 >> 4)) {
            uint32_t bfr[4]; // columns (cb0+u)*16 .. +7 (registers 0, 1) and +8 .. +15 (registers 2, 3), rows ks*16 .. +15
            ldmatrix_x4_trans(bfr, w2s + (ks * 16 + (lane & 15)) * q.w2_pitch + (cb0 + u) * 16 + ((lane >> 4) << 3));
            Mma<MODE>::run(d[u][0], ah[ks], bfr[0], bfr[1]);
            Mma<MODE>::run(d[u][1], ah[ks], bfr[2], bfr[3]);
            if (MODE == 1) { // bf16: the rounding residual of the running sum (8 bits of mantissa are too few without)
              Mma<MODE>::run(d[u][0], al[ks], bfr[0], bfr[1]);
              Mma<MODE>::run(d[u][1], al[ks], bfr[2], bfr[3]);
            }
          }
      }
#pragma unroll
    for (int u = 0; u < kCB; u++)
      if (cb0 + u < (n2 >> 4)) {
        int const col = (cb0 + u) * 16 + 2 * t;
        if (g < m) {
          *reinterpret_cast<uint32_t *>(O + (long long)g * old + col) = Mma<MODE>::pack(d[u][0][0], d[u][0][1]);
          *reinterpret_cast<uint32_t *>(O + (long long)g * old + col + 8) = Mma<MODE>::pack(d[u][1][0], d[u][1][1]);
        }
        if (g + 8 < m) {
          *reinterpret_cast<uint32_t *>(O + (long long)(g + 8) * old + col) = Mma<MODE>::pack(d[u][0][2], d[u][0][3]);
          *reinterpret_cast<uint32_t *>(O + (long long)(g + 8) * old + col + 8) = Mma<MODE>::pack(d[u][1][2], d[u][1][3]);
        }
      }
  }
  } else {

  // ---- fingerprint mode: the byte-plane scheme of fp_interp.cu.  A uint16 is lo + 256 hi; the 16 rows of an
  // m16n8k32 u8 MMA carry three byte-masked copies of 4 rows of A - [lo,0], [0,hi], [hi,lo] - which give LL, HH and
  // LH+HL in int32, and A B = LL + 256 (LH+HL) + 65536 HH modulo PQ.  Warp w takes row group w % 4 (4 rows) and the
  // 16-column pairs w / 4, w / 4 + 2, ...; the plane sums stay in registers over the whole for-loop (exact while the
  // contraction has at most 16384 terms) and are reduced once.
  int const mi = lane >> 3, rr = lane & 7, rg = warp & 3, ch = warp >> 2;
  int const row = rg * 4 + (g & 3);
  auto planes = [&](uint32_t w0, uint32_t w1, uint32_t (&a)[4]) {
    if (g < 4) { // MMA rows 0-3: [lo,0] bytes; MMA rows 8-11: [hi,lo] bytes
      a[0] = w0 & 0x00FF00FFu; a[2] = w1 & 0x00FF00FFu;
      a[1] = __byte_perm(w0, 0, 0x2301); a[3] = __byte_perm(w1, 0, 0x2301);
    } else {     // MMA rows 4-7: [0,hi] bytes; MMA rows 12-15 unused
      a[0] = w0 & 0xFF00FF00u; a[2] = w1 & 0xFF00FF00u;
      a[1] = 0u; a[3] = 0u;
    }
  };
  auto imma = [&](int32_t (&d)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  };
  // the two values this lane owns of a 4 x 8 result (rows g % 4, columns 2t, 2t + 1), reduced modulo PQ
  auto reduce_planes = [&](int32_t const (&d)[4]) {
    int32_t const hh0 = __shfl_down_sync(0xffffffffu, d[0], 16), hh1 = __shfl_down_sync(0xffffffffu, d[1], 16);
    uint32_t const v0 = ((uint32_t)d[0] % PQ + 256u * ((uint32_t)d[2] % PQ) + (65536u % PQ) * ((uint32_t)hh0 % PQ)) % PQ;
    uint32_t const v1 = ((uint32_t)d[1] % PQ + 256u * ((uint32_t)d[3] % PQ) + (65536u % PQ) * ((uint32_t)hh1 % PQ)) % PQ;
    return v0 | (v1 << 16);
  };
  constexpr int kMaxUnits = 4; // n1 <= 128: 8 column pairs, two interleaved halves
  int32_t acc[kMaxUnits][2][4];
#pragma unroll
  for (int u = 0; u < kMaxUnits; u++)
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
      for (int j = 0; j < 4; j++) acc[u][h][j] = 0;
  int const cpairs = n1 >> 4;
  for (int it = 0; it < loop; it++) {
    cp_wait_pending(S - 2);
    __syncthreads();
    if (it + S - 1 < loop) request_stage(it + S - 1);
    cp_commit();
    uint16_t const *xs = smem + (size_t)(it % S) * q.stage_elems, *ws = xs + 16 * q.x_pitch;
    uint16_t const *arow = xs + row * q.x_pitch + 2 * t;
    for (int ks = 0; ks < kt; ks += 16) {
      uint32_t a[4];
      planes(*reinterpret_cast<uint32_t const *>(arow + ks), *reinterpret_cast<uint32_t const *>(arow + ks + 8), a);
#pragma unroll
      for (int u = 0; u < kMaxUnits; u++) {
        int const cp = ch + 2 * u;
        if (cp < cpairs) {
          uint32_t bf[4]; // ldmatrix (transposed): this lane addresses k-row (mi % 2) * 8 + rr of the columns (mi / 2) * 8 ..
          ldmatrix_x4_trans(bf, ws + (ks + (mi & 1) * 8 + rr) * q.w1_pitch + cp * 16 + (mi >> 1) * 8);
          imma(acc[u][0], a, bf[0], bf[1]);
          imma(acc[u][1], a, bf[2], bf[3]);
        }
      }
    }
  }
  uint16_t *a2 = smem + q.a2_at;
#pragma unroll
  for (int u = 0; u < kMaxUnits; u++) {
    int const cp = ch + 2 * u;
    if (cp < cpairs) {
#pragma unroll
      for (int h = 0; h < 2; h++) {
        uint32_t const v = reduce_planes(acc[u][h]); // (every lane takes part in the shuffles)
        if (g < 4) *reinterpret_cast<uint32_t *>(a2 + row * q.a2_pitch + cp * 16 + h * 8 + 2 * t) = v;
      }
    }
  }
  cp_wait<0>();
  __syncthreads();
  // second product: the A fragments of every k-step once, then four column pairs at a time
  constexpr int kMaxK2 = 8;
  uint32_t a2f[kMaxK2][4];
  int const k2 = n1 >> 4, cpairs2 = n2 >> 4;
  {
    uint16_t const *arow2 = a2 + row * q.a2_pitch + 2 * t;
#pragma unroll
    for (int ks = 0; ks < kMaxK2; ks++)
      if (ks < k2) planes(*reinterpret_cast<uint32_t const *>(arow2 + ks * 16), *reinterpret_cast<uint32_t const *>(arow2 + ks * 16 + 8), a2f[ks]);
  }
  for (int cb0 = ch * kMaxUnits; cb0 < cpairs2; cb0 += 2 * kMaxUnits) {
    int32_t d[kMaxUnits][2][4];
#pragma unroll
    for (int u = 0; u < kMaxUnits; u++)
#pragma unroll
      for (int h = 0; h < 2; h++)
#pragma unroll
        for (int j = 0; j < 4; j++) d[u][h][j] = 0;
#pragma unroll
    for (int ks = 0; ks < kMaxK2; ks++)
      if (ks < k2) {
#pragma unroll
        for (int u = 0; u < kMaxUnits; u++)
          if (cb0 + u < cpairs2) {
            uint32_t bf[4];
            ldmatrix_x4_trans(bf, w2s + (ks * 16 + (mi & 1) * 8 + rr) * q.w2_pitch + (cb0 + u) * 16 + (mi >> 1) * 8);
            imma(d[u][0], a2f[ks], bf[0], bf[1]);
            imma(d[u][1], a2f[ks], bf[2], bf[3]);
          }
      }
#pragma unroll
    for (int u = 0; u < kMaxUnits; u++)
      if (cb0 + u < cpairs2) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
          uint32_t const v = reduce_planes(d[u][h]);
          if (g < 4 && row < m) *reinterpret_cast<uint32_t *>(O + (long long)row * old + (cb0 + u) * 16 + h * 8 + 2 * t) = v;
        }
      }
  }
  }
}

} // namespace chain
} // namespace mgk

using namespace mgk;

namespace {
bool aligned16(void const *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
// every 16-byte piece the loader copies must be 16-byte aligned in global memory: tensor columns, tile columns and
// every stride that moves a tile along a row are multiples of 8 elements
bool input_ok(mgd_op const &op) {
  int32_t const *a = op.a;
  for (int i : {3, 4, 5, 7, 8, 9, 10, 11})
    if (a[i] & 7) return false;
  return (a[MGD_IN_COLS] & 7) == 0 && (a[MGD_IN_TILE_COLS] & 7) == 0;
}
// Ring depth: as deep as the for-loop (at most 8) and as fits; the ring's memory also has to hold the four partial
// sums [4][16][n1] in fp32 / int32 once the loop is over.
int pick_stages(mgd_matmul_chain const *c) {
  for (int s = 8; s >= 2; s--) {
    chain::Plan const q = chain::make_plan(c->kt, c->n1, c->n2, s);
    if (q.total_bytes > (size_t)kSmemLimit - 1024) continue;
    if ((size_t)s * q.stage_elems * 2 < (size_t)4 * 16 * c->n1 * 4) return 0; // deeper rings were too large already
    return s;
  }
  return 0;
}
} // namespace

extern "C" {

int mgd_matmul_chain_supported(const mgd_matmul_chain *c, int32_t fingerprint_mode) {
  if (!c) return 0;
  if (c->m <= 0 || c->m > 16 || c->kt <= 0 || (c->kt & 15) || c->kt > 128 || c->n1 <= 0 || (c->n1 & 15) || c->n1 > 128 || c->n2 <= 0 || (c->n2 & 15)) return 0;
  if (c->forloop_range <= 0 || c->grid[0] <= 0 || c->grid[1] <= 0 || c->grid[2] <= 0) return 0;
  if (!input_ok(c->x) || !input_ok(c->w1) || !input_ok(c->w2)) return 0;
  if (fingerprint_mode) {
    // fingerprint buffers are row-major whatever the layout tag says; the int32 plane sums of the first product run
    // over the whole contraction
    if ((long long)c->forloop_range * c->kt > 16384) return 0;
  } else {
    if (c->data_type != MG_DT_FLOAT16 && c->data_type != MG_DT_BFLOAT16) return 0;
    for (mgd_op const *op : {&c->x, &c->w1, &c->w2})
      if ((op->a[MGD_IN_LAYOUT] & 0xff) != MG_DMEM_ROW_MAJOR) return 0;
  }
  int32_t const *o = c->out.a;
  for (int i : {3, 4, 5, 6, 7, 8})
    if (o[i] & 1) return 0; // 32-bit stores of column pairs
  if (o[MGD_OUT_COLS] & 1) return 0;
  return pick_stages(c) >= 2;
}

static int launch_chain(const mgd_matmul_chain *c, const mgd_bindings *bind, int mode, void *stream) {
  if (!c || !bind || !mgd_matmul_chain_supported(c, mode == 2)) return set_error(MG_ERR_UNSUPPORTED, "matmul chain: shape not supported");
  chain::Params p;
  std::memset(&p, 0, sizeof(p));
  p.c = *c;
  p.x = bind->in[c->x.a[MGD_IN_SLOT]]; p.w1 = bind->in[c->w1.a[MGD_IN_SLOT]]; p.w2 = bind->in[c->w2.a[MGD_IN_SLOT]];
  p.out = bind->out[c->out.a[MGD_OUT_SLOT]];
  p.x_set = bind->in_set_stride[c->x.a[MGD_IN_SLOT]]; p.w1_set = bind->in_set_stride[c->w1.a[MGD_IN_SLOT]];
  p.w2_set = bind->in_set_stride[c->w2.a[MGD_IN_SLOT]]; p.out_set = bind->out_set_stride[c->out.a[MGD_OUT_SLOT]];
  if (!p.x || !p.w1 || !p.w2 || !p.out || bind->num_sets <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "matmul chain: unbound tensor");
  if (!aligned16(p.x) || !aligned16(p.w1) || !aligned16(p.w2) || (reinterpret_cast<uintptr_t>(p.out) & 3) ||
      (bind->num_sets > 1 && ((p.x_set | p.w1_set | p.w2_set) & 7 || (p.out_set & 1))))
    return set_error(MG_ERR_UNSUPPORTED, "matmul chain: operands must be 16-byte aligned");
  p.stages = pick_stages(c);
  size_t const smem = chain::make_plan(c->kt, c->n1, c->n2, p.stages).total_bytes;
  long long const blocks = (long long)c->grid[0] * c->grid[1] * c->grid[2] * bind->num_sets;
  if (blocks > 0x7fffffffLL) return set_error(MG_ERR_UNSUPPORTED, "too many blocks for one launch");
  using Kernel = void (*)(chain::Params);
  static Kernel const kernels[3] = {chain::chain_kernel<0>, chain::chain_kernel<1>, chain::chain_kernel<2>};
  static bool configured[64][3] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev][mode]) {
    if (cudaFuncSetAttribute(kernels[mode], cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit - 1024) != cudaSuccess)
      return check_launch("cudaFuncSetAttribute(chain_kernel)");
    configured[dev][mode] = true;
  }
  kernels[mode]<<<(unsigned)blocks, chain::kThreads, smem, (cudaStream_t)stream>>>(p);
  return check_launch("chain_kernel");
}

int mgd_launch_matmul_chain_float(const mgd_matmul_chain *c, const mgd_bindings *bind, void *stream) {
  if (!c || (c->data_type != MG_DT_FLOAT16 && c->data_type != MG_DT_BFLOAT16)) return set_error(MG_ERR_UNSUPPORTED, "matmul chain: fp16 or bf16");
  return launch_chain(c, bind, c->data_type == MG_DT_BFLOAT16 ? 1 : 0, stream);
}
int mgd_launch_matmul_chain_fingerprint(const mgd_matmul_chain *c, const mgd_bindings *bind, void *stream) {
  return launch_chain(c, bind, 2, stream);
}
}
