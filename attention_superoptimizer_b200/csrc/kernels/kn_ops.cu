// Kernel-level (un-fused) operators in both modes.  They produce the fingerprints a fused
// candidate is compared against (the reference's compute_*_fingerprint kernels under
// src/kernel/cuda/) and their float counterparts.  Memory-bound element-wise code: grid-stride
// loops sized to the SM count, one exact 64-bit sum per matmul output.  The float matmul runs on the tensor cores
// (kn_matmul_tc.cu) where its operands can be described to the TMA unit; the loop here takes the rest.
#include "common.cuh"

namespace mgk {
namespace kmm { // kn_matmul_tc.cu: the float matmul on tcgen05
bool supported(void const *a, void const *b, int batches, int m, int n, int k, int a_col_major, int b_col_major);
int launch(void const *a, void const *b, void *c, int batches, int m, int n, int k, int dtype, int a_col_major, int b_col_major,
           void *stream);
} // namespace kmm

static int blocks_for(int64_t n, int threads = 256) {
  int64_t blocks = (n + threads - 1) / threads, cap = 148 * 8;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// C[b] = A[b] x B[b] modulo PQ; dense row-major operands (matmul_kernel.cu:145-173)
__global__ void kn_matmul_fp_kernel(uint16_t const *A, uint16_t const *B, uint16_t *C, int batches, int m, int n, int k) {
  int64_t total = (int64_t)batches * m * n, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t b = i / ((int64_t)m * n);
    int r = (int)((i / n) % m), c = (int)(i % n);
    uint16_t const *a = A + b * m * k + (int64_t)r * k, *bb = B + b * k * n + c;
    unsigned long long acc = 0;
    for (int kk = 0; kk < k; kk++) acc += (unsigned long long)((uint32_t)a[kk] * (uint32_t)bb[(int64_t)kk * n]);
    C[i] = (uint16_t)(acc % PQ);
  }
}

// The same product on the integer tensor cores, exact (the byte-plane scheme of the threadblock-level matmul,
// fp_interp.cu): a uint16 is lo + 256 hi, a row-major uint16 tile is a byte matrix with the planes interleaved along
// k, and the 16 rows of an m16n8k32 u8 MMA carry three byte-masked copies of 4 rows of A - [lo,0], [0,hi], [hi,lo] -
// which give LL, HH and LH+HL in int32;  A B = LL + 256 (LH+HL) + 65536 HH, reduced modulo PQ once per output.
// A block of 4 warps owns a 16 x 64 tile of C (a warp: 4 rows x 64 columns, eight independent MMAs per k-step) and
// walks k in chunks of 64 staged in shared memory with 16-byte loads (rows padded by 16 bytes: conflict-free
// ldmatrix).  Needs k and n multiples of 8, 16-byte aligned operands and k <= 16384 (int32 sums); rows, columns and
// k-steps past the extents are zeros.
constexpr int kFpTM = 16, kFpTN = 64, kFpTK = 64, kFpPitch = 72;
__global__ void __launch_bounds__(128) kn_matmul_fp_tc_kernel(uint16_t const *A, uint16_t const *B, uint16_t *C, int batches, int m,
                                                              int n, int k) {
  __shared__ __align__(16) uint16_t As[kFpTM * kFpPitch];
  __shared__ __align__(16) uint16_t Bs[kFpTK * kFpPitch];
  int const tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int const g = lane >> 2, t = lane & 3, mi = lane >> 3, rr = lane & 7;
  int const tiles_m = (m + kFpTM - 1) / kFpTM, tiles_n = (n + kFpTN - 1) / kFpTN;
  int64_t const tiles = (int64_t)batches * tiles_m * tiles_n;
  uint32_t const bs_base = (uint32_t)__cvta_generic_to_shared(Bs);
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    int const nt_ = (int)(tile % tiles_n), mt = (int)((tile / tiles_n) % tiles_m);
    int64_t const b = tile / ((int64_t)tiles_n * tiles_m);
    int const m0 = mt * kFpTM, n0 = nt_ * kFpTN;
    uint16_t const *Ab = A + b * m * k, *Bb = B + b * k * n;
    int const row = warp * 4 + (g & 3); // row of the tile this lane's A fragments come from
    int32_t acc[4][2][4];
#pragma unroll
    for (int c = 0; c < 4; c++)
#pragma unroll
      for (int h = 0; h < 2; h++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[c][h][j] = 0;
    for (int k0 = 0; k0 < k; k0 += kFpTK) {
      __syncthreads(); // the previous chunk (or tile) has been read
      {
        int const r = tid >> 3, c8 = (tid & 7) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m0 + r < m && k0 + c8 < k) v = __ldg(reinterpret_cast<uint4 const *>(Ab + (int64_t)(m0 + r) * k + k0 + c8));
        *reinterpret_cast<uint4 *>(As + r * kFpPitch + c8) = v;
      }
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int const idx = tid + i * 128, r = idx >> 3, c8 = (idx & 7) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (k0 + r < k && n0 + c8 < n) v = __ldg(reinterpret_cast<uint4 const *>(Bb + (int64_t)(k0 + r) * n + n0 + c8));
        *reinterpret_cast<uint4 *>(Bs + r * kFpPitch + c8) = v;
      }
      __syncthreads();
      uint16_t const *arow = As + row * kFpPitch + 2 * t;
#pragma unroll
      for (int ks = 0; ks < kFpTK / 16; ks++) {
        uint32_t const w0 = *reinterpret_cast<uint32_t const *>(arow + ks * 16);
        uint32_t const w1 = *reinterpret_cast<uint32_t const *>(arow + ks * 16 + 8);
        uint32_t a[4];
        if (g < 4) { // MMA rows 0-3: [lo,0] bytes; MMA rows 8-11: [hi,lo] bytes
          a[0] = w0 & 0x00FF00FFu; a[2] = w1 & 0x00FF00FFu;
          a[1] = __byte_perm(w0, 0, 0x2301); a[3] = __byte_perm(w1, 0, 0x2301);
        } else {     // MMA rows 4-7: [0,hi] bytes; MMA rows 12-15 unused
          a[0] = w0 & 0xFF00FF00u; a[2] = w1 & 0xFF00FF00u;
          a[1] = 0u; a[3] = 0u;
        }
        uint32_t bf[4][4];
#pragma unroll
        for (int c = 0; c < 4; c++) {
          // ldmatrix (transposed): this lane addresses k-row (mi % 2) * 8 + rr of the 8 columns starting at (mi / 2) * 8
          uint32_t const addr = bs_base + (uint32_t)(((ks * 16 + (mi & 1) * 8 + rr) * kFpPitch + c * 16 + (mi >> 1) * 8) * 2);
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(bf[c][0]), "=r"(bf[c][1]), "=r"(bf[c][2]), "=r"(bf[c][3]) : "r"(addr));
        }
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
          for (int h = 0; h < 2; h++)
            asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+r"(acc[c][h][0]), "+r"(acc[c][h][1]), "+r"(acc[c][h][2]), "+r"(acc[c][h][3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(bf[c][2 * h]), "r"(bf[c][2 * h + 1]));
      }
    }
#pragma unroll
    for (int c = 0; c < 4; c++)
#pragma unroll
      for (int h = 0; h < 2; h++) {
        // lanes 16-31 hold the HH sums of the rows lanes 0-15 work on
        int32_t const hh0 = __shfl_down_sync(0xffffffffu, acc[c][h][0], 16), hh1 = __shfl_down_sync(0xffffffffu, acc[c][h][1], 16);
        int const col = n0 + c * 16 + h * 8 + 2 * t;
        if (g < 4 && m0 + row < m && col < n) {
          uint32_t v0 = ((uint32_t)acc[c][h][0] % PQ + 256u * ((uint32_t)acc[c][h][2] % PQ) + (65536u % PQ) * ((uint32_t)hh0 % PQ)) % PQ;
          uint32_t v1 = ((uint32_t)acc[c][h][1] % PQ + 256u * ((uint32_t)acc[c][h][3] % PQ) + (65536u % PQ) * ((uint32_t)hh1 % PQ)) % PQ;
          *reinterpret_cast<uint32_t *>(C + (b * m + m0 + row) * (int64_t)n + col) = v0 | (v1 << 16);
        }
      }
  }
}

__global__ void kn_exp_fp_kernel(uint16_t const *x, uint16_t *y, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = (uint16_t)field_exp(x[i]);
}

struct Dims4 { int d[4]; };

__device__ __forceinline__ void broadcast_index(int64_t i, Dims4 const &xd, Dims4 const &yd, Dims4 const &zd,
                                                int64_t &xi, int64_t &yi) {
  int64_t xs = 1, ys = 1;
  xi = yi = 0;
  for (int d = 3; d >= 0; d--) {
    xi += (i % xd.d[d]) * xs;
    yi += (i % yd.d[d]) * ys;
    xs *= xd.d[d];
    ys *= yd.d[d];
    i /= zd.d[d];
  }
}

__global__ void kn_binary_fp_kernel(int op, uint16_t const *x, Dims4 xd, uint16_t const *y, Dims4 yd, uint16_t *z, Dims4 zd) {
  int64_t n = (int64_t)zd.d[0] * zd.d[1] * zd.d[2] * zd.d[3], stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t xi, yi;
    broadcast_index(i, xd, yd, zd, xi, yi);
    uint32_t xv = x[xi], yv = y[yi], r;
    if (op == MG_KN_DIV_OP) r = field_div(xv, yv);
    else if (op == MG_KN_ADD_OP) r = (xv + yv) % PQ;
    else r = (uint32_t)(((unsigned long long)xv * yv) % PQ);
    z[i] = (uint16_t)r;
  }
}

// out[i] = sum_k in[(i / os) * is + i % os + k * os]  (reduction_kernel.cu:80-108)
__global__ void kn_reduction_fp_kernel(uint16_t const *x, uint16_t *y, int64_t n_out, int factor, int64_t is, int64_t os) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_out; i += stride) {
    int64_t base = (i / os) * is + i % os;
    unsigned long long acc = 0;
    for (int k = 0; k < factor; k++) acc += x[base + (int64_t)k * os];
    y[i] = (uint16_t)(acc % PQ);
  }
}

// The same with a warp per output (lanes stride over the terms): for few outputs of many terms each, e.g. row sums
// of a wide matrix, where a thread per output leaves most of the GPU idle.  A sum of 65535 terms fits 32 bits.
__global__ void kn_reduction_fp_warp_kernel(uint16_t const *x, uint16_t *y, int64_t n_out, int factor, int64_t is, int64_t os) {
  int const lane = threadIdx.x & 31;
  int64_t const warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n_out; i += warps) {
    int64_t const base = (i / os) * is + i % os;
    uint32_t acc = 0;
    for (int k = lane; k < factor; k += 32) acc += x[base + (int64_t)k * os];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[i] = (uint16_t)(acc % PQ);
  }
}

// ---- float mode ------------------------------------------------------------------------------------------
template <typename T>
__global__ void kn_matmul_float_kernel(T const *A, T const *B, T *C, int batches, int m, int n, int k, int a_col_major,
                                       int b_col_major) {
  int64_t total = (int64_t)batches * m * n, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t b = i / ((int64_t)m * n);
    int r = (int)((i / n) % m), c = (int)(i % n);
    T const *a = A + b * m * k, *bb = B + b * k * n;
    float acc = 0.f;
    for (int kk = 0; kk < k; kk++) {
      float av = to_float<T>(a_col_major ? a[(int64_t)kk * m + r] : a[(int64_t)r * k + kk]);
      float bv = to_float<T>(b_col_major ? bb[(int64_t)c * k + kk] : bb[(int64_t)kk * n + c]);
      acc = fmaf(av, bv, acc);
    }
    C[i] = from_float<T>(acc);
  }
}
template <typename T> __global__ void kn_exp_float_kernel(T const *x, T *y, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = from_float<T>(expf(to_float<T>(x[i])));
}
template <typename T>
__global__ void kn_binary_float_kernel(int op, T const *x, Dims4 xd, T const *y, Dims4 yd, T *z, Dims4 zd) {
  int64_t n = (int64_t)zd.d[0] * zd.d[1] * zd.d[2] * zd.d[3], stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t xi, yi;
    broadcast_index(i, xd, yd, zd, xi, yi);
    float xv = to_float<T>(x[xi]), yv = to_float<T>(y[yi]);
    z[i] = from_float<T>(op == MG_KN_DIV_OP ? xv / yv : (op == MG_KN_ADD_OP ? xv + yv : xv * yv));
  }
}
template <typename T>
__global__ void kn_reduction_float_kernel(T const *x, T *y, int64_t n_out, int factor, int64_t is, int64_t os) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_out; i += stride) {
    int64_t base = (i / os) * is + i % os;
    float acc = 0.f;
    for (int k = 0; k < factor; k++) acc += to_float<T>(x[base + (int64_t)k * os]);
    y[i] = from_float<T>(acc);
  }
}

template <typename T>
__global__ void kn_reduction_float_warp_kernel(T const *x, T *y, int64_t n_out, int factor, int64_t is, int64_t os) {
  int const lane = threadIdx.x & 31;
  int64_t const warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n_out; i += warps) {
    int64_t const base = (i / os) * is + i % os;
    float acc = 0.f;
    for (int k = lane; k < factor; k += 32) acc += to_float<T>(x[base + (int64_t)k * os]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[i] = from_float<T>(acc);
  }
}

// a warp per output pays when there are too few outputs to fill the GPU with a thread each
static bool reduce_by_warps(int64_t n_out, int factor) { return factor >= 32 && factor < 65536 && n_out < 148 * 256; }

static bool dims_ok(int32_t const *d) { return d && d[0] > 0 && d[1] > 0 && d[2] > 0 && d[3] > 0; }
static Dims4 pack(int32_t const *d) { return Dims4{{d[0], d[1], d[2], d[3]}}; }
} // namespace mgk

using namespace mgk;
#define ST(s) ((cudaStream_t)(s))

extern "C" {

int mgd_kn_matmul_fingerprint(const uint16_t *a, const uint16_t *b, uint16_t *c, int32_t batches, int32_t m, int32_t n,
                              int32_t k, void *stream) {
  if (!a || !b || !c || batches <= 0 || m <= 0 || n <= 0 || k <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "kn matmul: bad argument");
  // integer tensor cores where the operands allow 16-byte loads and the int32 plane sums cannot overflow
  // (MGD_OPT_KN_MATMUL_ENGINE: 1 = CUDA cores)
  if (option(MGD_OPT_KN_MATMUL_ENGINE) != 1 && (k & 7) == 0 && (n & 7) == 0 && k <= 16384 &&
      ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0) {
    int64_t const tiles = (int64_t)batches * ((m + kFpTM - 1) / kFpTM) * ((n + kFpTN - 1) / kFpTN);
    int64_t const cap = 148 * 16;
    kn_matmul_fp_tc_kernel<<<(unsigned)(tiles < cap ? tiles : cap), 128, 0, ST(stream)>>>(a, b, c, batches, m, n, k);
    return check_launch("kn_matmul_fp_tc_kernel");
  }
  kn_matmul_fp_kernel<<<blocks_for((int64_t)batches * m * n), 256, 0, ST(stream)>>>(a, b, c, batches, m, n, k);
  return check_launch("kn_matmul_fp_kernel");
}
int mgd_kn_exp_fingerprint(const uint16_t *x, uint16_t *y, int64_t n, void *stream) {
  if (!x || !y || n <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "kn exp: bad argument");
  kn_exp_fp_kernel<<<blocks_for(n), 256, 0, ST(stream)>>>(x, y, n);
  return check_launch("kn_exp_fp_kernel");
}
int mgd_kn_binary_fingerprint(int32_t op, const uint16_t *x, const int32_t *xd, const uint16_t *y, const int32_t *yd,
                              uint16_t *z, const int32_t *zd, void *stream) {
  if (!x || !y || !z || !dims_ok(xd) || !dims_ok(yd) || !dims_ok(zd)) return set_error(MG_ERR_INVALID_ARGUMENT, "kn binary: bad argument");
  if (op != MG_KN_ADD_OP && op != MG_KN_MUL_OP && op != MG_KN_DIV_OP) return set_error(MG_ERR_UNSUPPORTED, "kn binary: unknown operator");
  int64_t n = (int64_t)zd[0] * zd[1] * zd[2] * zd[3];
  kn_binary_fp_kernel<<<blocks_for(n), 256, 0, ST(stream)>>>(op, x, pack(xd), y, pack(yd), z, pack(zd));
  return check_launch("kn_binary_fp_kernel");
}
int mgd_kn_reduction_fingerprint(const uint16_t *x, uint16_t *y, int64_t n_out, int32_t factor, int64_t is, int64_t os,
                                 void *stream) {
  if (!x || !y || n_out <= 0 || factor <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "kn reduction: bad argument");
  if (reduce_by_warps(n_out, factor)) {
    kn_reduction_fp_warp_kernel<<<blocks_for(n_out * 32), 256, 0, ST(stream)>>>(x, y, n_out, factor, is, os);
    return check_launch("kn_reduction_fp_warp_kernel");
  }
  kn_reduction_fp_kernel<<<blocks_for(n_out), 256, 0, ST(stream)>>>(x, y, n_out, factor, is, os);
  return check_launch("kn_reduction_fp_kernel");
}

#define DISPATCH_16(dt, CALL_H, CALL_B)                                              \
  if ((dt) == MG_DT_FLOAT16) { CALL_H; }                                              \
  else if ((dt) == MG_DT_BFLOAT16) { CALL_B; }                                        \
  else return set_error(MG_ERR_UNSUPPORTED, "float mode runs on fp16 or bf16 tensors");

int mgd_kn_matmul_float(const void *a, const void *b, void *c, int32_t batches, int32_t m, int32_t n, int32_t k,
                        int32_t al, int32_t bl, int32_t dt, void *stream) {
  if (!a || !b || !c || batches <= 0 || m <= 0 || n <= 0 || k <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "kn matmul: bad argument");
  int g = blocks_for((int64_t)batches * m * n), ac = al == MG_DMEM_COLUMN_MAJOR, bc = bl == MG_DMEM_COLUMN_MAJOR;
  // tensor cores (tcgen05) wherever a tensor map can describe the operands; MGD_OPT_KN_MATMUL_ENGINE: 1 = CUDA cores
  if ((dt == MG_DT_FLOAT16 || dt == MG_DT_BFLOAT16) && option(MGD_OPT_KN_MATMUL_ENGINE) != 1 &&
      kmm::supported(a, b, batches, m, n, k, ac, bc))
    return kmm::launch(a, b, c, batches, m, n, k, dt, ac, bc, stream);
  DISPATCH_16(dt, (kn_matmul_float_kernel<__half><<<g, 256, 0, ST(stream)>>>((__half const *)a, (__half const *)b, (__half *)c, batches, m, n, k, ac, bc)),
              (kn_matmul_float_kernel<__nv_bfloat16><<<g, 256, 0, ST(stream)>>>((__nv_bfloat16 const *)a, (__nv_bfloat16 const *)b, (__nv_bfloat16 *)c, batches, m, n, k, ac, bc)))
  return check_launch("kn_matmul_float_kernel");
}
int mgd_kn_exp_float(const void *x, void *y, int64_t n, int32_t dt, void *stream) {
  if (!x || !y || n <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "kn exp: bad argument");
  int g = blocks_for(n);
  DISPATCH_16(dt, (kn_exp_float_kernel<__half><<<g, 256, 0, ST(stream)>>>((__half const *)x, (__half *)y, n)),
              (kn_exp_float_kernel<__nv_bfloat16><<<g, 256, 0, ST(stream)>>>((__nv_bfloat16 const *)x, (__nv_bfloat16 *)y, n)))
  return check_launch("kn_exp_float_kernel");
}
int mgd_kn_binary_float(int32_t op, const void *x, const int32_t *xd, const void *y, const int32_t *yd, void *z,
                        const int32_t *zd, int32_t dt, void *stream) {
  if (!x || !y || !z || !dims_ok(xd) || !dims_ok(yd) || !dims_ok(zd)) return set_error(MG_ERR_INVALID_ARGUMENT, "kn binary: bad argument");
  if (op != MG_KN_ADD_OP && op != MG_KN_MUL_OP && op != MG_KN_DIV_OP) return set_error(MG_ERR_UNSUPPORTED, "kn binary: unknown operator");
  int g = blocks_for((int64_t)zd[0] * zd[1] * zd[2] * zd[3]);
  DISPATCH_16(dt, (kn_binary_float_kernel<__half><<<g, 256, 0, ST(stream)>>>(op, (__half const *)x, pack(xd), (__half const *)y, pack(yd), (__half *)z, pack(zd))),
              (kn_binary_float_kernel<__nv_bfloat16><<<g, 256, 0, ST(stream)>>>(op, (__nv_bfloat16 const *)x, pack(xd), (__nv_bfloat16 const *)y, pack(yd), (__nv_bfloat16 *)z, pack(zd))))
  return check_launch("kn_binary_float_kernel");
}
int mgd_kn_reduction_float(const void *x, void *y, int64_t n_out, int32_t factor, int64_t is, int64_t os, int32_t dt,
                           void *stream) {
  if (!x || !y || n_out <= 0 || factor <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "kn reduction: bad argument");
  if (reduce_by_warps(n_out, factor)) {
    int const gw = blocks_for(n_out * 32);
    DISPATCH_16(dt, (kn_reduction_float_warp_kernel<__half><<<gw, 256, 0, ST(stream)>>>((__half const *)x, (__half *)y, n_out, factor, is, os)),
                (kn_reduction_float_warp_kernel<__nv_bfloat16><<<gw, 256, 0, ST(stream)>>>((__nv_bfloat16 const *)x, (__nv_bfloat16 *)y, n_out, factor, is, os)))
    return check_launch("kn_reduction_float_warp_kernel");
  }
  int g = blocks_for(n_out);
  DISPATCH_16(dt, (kn_reduction_float_kernel<__half><<<g, 256, 0, ST(stream)>>>((__half const *)x, (__half *)y, n_out, factor, is, os)),
              (kn_reduction_float_kernel<__nv_bfloat16><<<g, 256, 0, ST(stream)>>>((__nv_bfloat16 const *)x, (__nv_bfloat16 *)y, n_out, factor, is, os)))
  return check_launch("kn_reduction_float_kernel");
}
}
