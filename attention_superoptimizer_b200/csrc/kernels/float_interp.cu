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
//   * an input tile that does not move with the for-loop is loaded in the first iteration only.
// Loads honour the tensor's DmemLayout: a column-major tensor keeps each [rows, cols] matrix with the
// row index contiguous.  Outputs are rounded to nearest on store.
#include "common.cuh"

namespace mgk {
int validate_program(mgd_program const *p, mgd_bindings const *b);

// flag bits the host packs into operator arguments after replanning
constexpr int kIn16 = 1 << 8;         // input a[16]: the tile keeps 16-bit elements
constexpr int kInInvariant = 1 << 9;  // input a[16]: same tile every iteration, load once

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

// C (fp32, m x n) = or += A (m x k) B (k x n), all row-major in shared memory.  Threads own 4x4 or 1x4
// patches of C (registers) when n is a multiple of four, so a B row segment is one vector load.
template <typename T, bool A16, bool B16>
__device__ void matmul_tiles(unsigned char const *Ap, unsigned char const *Bp, float *C, int m, int n, int k, bool add,
                             int tid, int nt) {
  auto a_at = [&](int idx) -> float {
    return A16 ? to_float<T>(reinterpret_cast<T const *>(Ap)[idx]) : reinterpret_cast<float const *>(Ap)[idx];
  };
  auto b4_at = [&](int idx, float *f) {
    if (B16) cvt4<T>(*reinterpret_cast<uint2 const *>(Bp + (size_t)idx * 2), f);
    else {
      float4 v = *reinterpret_cast<float4 const *>(Bp + (size_t)idx * 4);
      f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
  };
  if ((n & 3) == 0) {
    int const nq = n >> 2;
    if ((m & 3) == 0 && (m >> 2) * nq >= nt) {
      for (int i = tid; i < (m >> 2) * nq; i += nt) {
        int const r = (i / nq) * 4, c = (i % nq) * 4;
        float acc[4][4];
#pragma unroll
        for (int x = 0; x < 4; x++)
#pragma unroll
          for (int y = 0; y < 4; y++) acc[x][y] = 0.f;
        for (int kk = 0; kk < k; kk++) {
          float b[4];
          b4_at(kk * n + c, b);
#pragma unroll
          for (int x = 0; x < 4; x++) {
            float av = a_at((r + x) * k + kk);
#pragma unroll
            for (int y = 0; y < 4; y++) acc[x][y] = fmaf(av, b[y], acc[x][y]);
          }
        }
#pragma unroll
        for (int x = 0; x < 4; x++) {
          float4 *dst = reinterpret_cast<float4 *>(C + (r + x) * n + c);
          float4 v = make_float4(acc[x][0], acc[x][1], acc[x][2], acc[x][3]);
          if (add) { float4 o = *dst; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
          *dst = v;
        }
      }
    } else {
      for (int i = tid; i < m * nq; i += nt) {
        int const r = i / nq, c = (i % nq) * 4;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int kk = 0; kk < k; kk++) {
          float b[4];
          b4_at(kk * n + c, b);
          float av = a_at(r * k + kk);
#pragma unroll
          for (int y = 0; y < 4; y++) acc[y] = fmaf(av, b[y], acc[y]);
        }
        float4 *dst = reinterpret_cast<float4 *>(C + r * n + c);
        float4 v = make_float4(acc[0], acc[1], acc[2], acc[3]);
        if (add) { float4 o = *dst; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
        *dst = v;
      }
    }
  } else {
    for (int i = tid; i < m * n; i += nt) {
      int const r = i / n, c = i % n;
      float acc = 0.f;
      for (int kk = 0; kk < k; kk++) {
        float bv = B16 ? to_float<T>(reinterpret_cast<T const *>(Bp)[kk * n + c]) : reinterpret_cast<float const *>(Bp)[kk * n + c];
        acc = fmaf(a_at(r * k + kk), bv, acc);
      }
      C[i] = add ? C[i] + acc : acc;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(1024) float_interp_kernel(const __grid_constant__ mgd_program prog,
                                                           const __grid_constant__ mgd_bindings bind) {
  extern __shared__ __align__(16) unsigned char smem_b[];
  int const tid = threadIdx.x, nt = blockDim.x;
  int const gx = prog.grid[0], gy = prog.grid[1], gz = prog.grid[2];
  int64_t b = blockIdx.x;
  int const bx = (int)(b % gx), by = (int)((b / gx) % gy), bz = (int)((b / ((int64_t)gx * gy)) % gz);
  int64_t const set = b / ((int64_t)gx * gy * gz);
  auto tile = [&](int byte_offset) { return smem_b + byte_offset; };
  auto ftile = [&](int byte_offset) { return reinterpret_cast<float *>(smem_b + byte_offset); };

  for (int it = 0; it < prog.forloop_range; it++) {
    for (int oi = 0; oi < prog.num_ops; oi++) {
      mgd_op const &op = prog.ops[oi];
      int32_t const *a = op.a;
      switch (op.type) {
        case 2001: {
          if ((a[16] & kInInvariant) && it > 0) break; // uniform over the block
          int row = bx * a[0] + by * a[1] + bz * a[2] + it * a[6];
          int col = bx * a[3] + by * a[4] + bz * a[5] + it * a[7];
          int64_t lead = (int64_t)bx * a[8] + (int64_t)by * a[9] + (int64_t)bz * a[10] + (int64_t)it * a[11];
          T const *src = static_cast<T const *>(bind.in[a[18]]) + set * bind.in_set_stride[a[18]] + lead;
          bool const keep16 = (a[16] & kIn16) != 0;
          T *dst16 = reinterpret_cast<T *>(tile(a[17]));
          float *dst32 = ftile(a[17]);
          int rows = a[14], cols = a[15], n = rows * cols;
          if ((a[16] & 0xff) == MG_DMEM_COLUMN_MAJOR) {
            int ld = a[12]; // rows of the whole matrix: consecutive rows are adjacent in memory
            for (int i = tid; i < n; i += nt) {
              int c = i / rows, r = i % rows;
              T v = src[(size_t)(col + c) * ld + row + r];
              if (keep16) dst16[r * cols + c] = v;
              else dst32[r * cols + c] = to_float<T>(v);
            }
          } else {
            int ld = a[13];
            T const *first = src + (size_t)row * ld + col;
            if (keep16 && (cols & 7) == 0 && (ld & 7) == 0 && (reinterpret_cast<uintptr_t>(first) & 15) == 0) {
              int const cv = cols >> 3; // 16-byte pieces per tile row
              for (int i = tid; i < rows * cv; i += nt) {
                int r = i / cv, c = i % cv;
                reinterpret_cast<uint4 *>(dst16)[i] = __ldg(reinterpret_cast<uint4 const *>(first + (size_t)r * ld) + c);
              }
            } else {
              for (int i = tid; i < n; i += nt) {
                int r = i / cols, c = i % cols;
                T v = first[(size_t)r * ld + c];
                if (keep16) dst16[i] = v;
                else dst32[i] = to_float<T>(v);
              }
            }
          }
          break;
        }
        case MG_TB_MATMUL_OP: {
          int m = a[0], n = a[1], k = a[2];
          unsigned char const *A = tile(a[3]), *B = tile(a[4]);
          float *C = ftile(a[5]);
          bool const add = a[8] != 0 && it > 0;
          if (a[6] && a[7]) matmul_tiles<T, true, true>(A, B, C, m, n, k, add, tid, nt);
          else if (a[6]) matmul_tiles<T, true, false>(A, B, C, m, n, k, add, tid, nt);
          else if (a[7]) matmul_tiles<T, false, true>(A, B, C, m, n, k, add, tid, nt);
          else matmul_tiles<T, false, false>(A, B, C, m, n, k, add, tid, nt);
          break;
        }
        case MG_TB_EXP_OP: {
          float *x = ftile(a[0]);
          for (int i = tid; i < a[1]; i += nt) x[i] = expf(x[i]);
          break;
        }
        case MG_TB_DIV_OP:
        case MG_TB_ADD_OP:
        case MG_TB_MUL_OP: {
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
        }
        case MG_TB_REDUCTION_0_OP: case MG_TB_REDUCTION_1_OP: case MG_TB_REDUCTION_2_OP:
        case MG_TB_REDUCTION_0_TO_DIMX_OP: case MG_TB_REDUCTION_1_TO_DIMX_OP: case MG_TB_REDUCTION_2_TO_DIMX_OP: {
          int n_out = a[0], degree = a[1], inner = a[2];
          unsigned char const *x = tile(a[3]);
          bool const x16 = a[5] != 0;
          float *y = ftile(a[4]);
          for (int i = tid; i < n_out; i += nt) {
            int pos = (i / inner) * (inner * degree) + i % inner;
            float acc = 0.f;
            for (int k = 0; k < degree; k++, pos += inner) acc += rd<T>(x, x16, pos);
            y[i] = acc;
          }
          break;
        }
        case MG_TB_CONCAT_0_OP: case MG_TB_CONCAT_1_OP: case MG_TB_CONCAT_2_OP: {
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
        }
        case 2002: {
          int n = a[11] * a[12];
          float *acc = ftile(a[14]);
          if (!a[17]) { // a[17]: the producing matmul already added into the accumulator
            unsigned char const *x = tile(a[13]);
            bool const x16 = a[16] != 0;
            if (it == 0) {
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
            T *dst = static_cast<T *>(bind.out[a[15]]) + set * bind.out_set_stride[a[15]] + lead;
            int cols = a[12], ld = a[10];
            for (int i = tid; i < n; i += nt) dst[(size_t)(row + i / cols) * ld + col + i % cols] = from_float<T>(acc[i]);
          }
          break;
        }
        default: break;
      }
      __syncthreads();
    }
  }
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
  bool is16() const { return loaded && !computed; }
};

struct Replanned {
  mgd_program prog;
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
      t[i] = TileUse{planned, elems, false, false, false, 0};
    } else if (elems > t[i].elems) {
      t[i].elems = elems;
    }
    return i;
  }
};

bool is_reduction(int type) { return type >= MG_TB_REDUCTION_0_OP && type <= MG_TB_REDUCTION_2_TO_DIMX_OP; }
bool is_concat(int type) { return type == MG_TB_CONCAT_0_OP || type == MG_TB_CONCAT_1_OP || type == MG_TB_CONCAT_2_OP; }
bool is_binary(int type) { return type == MG_TB_DIV_OP || type == MG_TB_ADD_OP || type == MG_TB_MUL_OP; }

// number of operand reads of tile `planned` by operator `op` (an in-place exp counts as a read)
int reads_of(mgd_op const &op, int planned) {
  int32_t const *a = op.a;
  int n = 0;
  if (op.type == MG_TB_MATMUL_OP) n = (a[3] == planned) + (a[4] == planned);
  else if (op.type == MG_TB_EXP_OP) n = a[0] == planned;
  else if (is_binary(op.type)) n = (a[6] == planned) + (a[7] == planned);
  else if (is_reduction(op.type)) n = a[3] == planned;
  else if (is_concat(op.type)) n = (a[4] == planned) + (a[5] == planned);
  else if (op.type == 2002) n = a[13] == planned;
  return n;
}

// tile written by `op`, or -1
int written_by(mgd_op const &op) {
  int32_t const *a = op.a;
  if (op.type == 2001) return a[17];
  if (op.type == MG_TB_MATMUL_OP) return a[5];
  if (op.type == MG_TB_EXP_OP) return a[0];
  if (is_binary(op.type)) return a[8];
  if (is_reduction(op.type)) return a[4];
  if (is_concat(op.type)) return a[6];
  if (op.type == 2002) return a[14];
  return -1;
}

void replan(mgd_program const &in, Replanned *out) {
  TileTable tt;
  out->prog = in;
  mgd_program &p = out->prog;
  // pass 1: every tile with its size and who writes it
  for (int i = 0; i < in.num_ops; i++) {
    mgd_op const &op = in.ops[i];
    int32_t const *a = op.a;
    if (op.type == 2001) {
      tt.t[tt.touch(a[17], a[14] * a[15])].loaded = true;
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
    } else if (op.type == 2002) {
      tt.touch(a[13], a[11] * a[12]);
      tt.t[tt.touch(a[14], a[11] * a[12])].computed = true;
    }
  }
  // pass 2: a matmul whose result only an output operator reads accumulates in place of that operator
  int fused_matmul[MGD_MAX_OPS];
  for (int i = 0; i < in.num_ops; i++) fused_matmul[i] = -1;
  for (int o = 0; o < in.num_ops; o++) {
    if (in.ops[o].type != 2002) continue;
    int src = in.ops[o].a[13], writer = -1, writers = 0, reads = 0;
    for (int i = 0; i < in.num_ops; i++) {
      if (written_by(in.ops[i]) == src) { writers++; writer = i; }
      reads += reads_of(in.ops[i], src);
    }
    if (writers == 1 && reads == 1 && writer < o && in.ops[writer].type == MG_TB_MATMUL_OP) {
      fused_matmul[o] = writer;
      tt.t[tt.find(src)].dropped = true;
    }
  }
  // pass 3: offsets, 16-byte aligned
  size_t at = 0;
  for (int i = 0; i < tt.n; i++) {
    if (tt.t[i].dropped) continue;
    tt.t[i].offset = (int)at;
    at += ((size_t)tt.t[i].elems * (tt.t[i].is16() ? 2 : 4) + 15) & ~(size_t)15;
  }
  out->smem_bytes = at + 16;
  // pass 4: rewrite operands
  auto off = [&](int planned) { return tt.t[tt.find(planned)].offset; };
  auto is16 = [&](int planned) { return tt.t[tt.find(planned)].is16() ? 1 : 0; };
  for (int i = 0; i < in.num_ops; i++) {
    int32_t const *a = in.ops[i].a;
    int32_t *w = p.ops[i].a;
    int type = in.ops[i].type;
    if (type == 2001) {
      w[17] = off(a[17]);
      w[16] = (a[16] & 0xff) | (is16(a[17]) ? kIn16 : 0);
      // no for-loop stride and nothing overwrites the tile: the first iteration's copy stays valid
      if (is16(a[17]) && a[6] == 0 && a[7] == 0 && a[11] == 0) w[16] |= kInInvariant;
    } else if (type == MG_TB_MATMUL_OP) {
      w[3] = off(a[3]); w[4] = off(a[4]);
      w[6] = is16(a[3]); w[7] = is16(a[4]);
      w[8] = 0;
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
  replan(*prog, &r);
  *bytes = r.smem_bytes;
  *fits = *bytes <= (size_t)kSmemLimit;
  return MG_OK;
}

extern "C" int mgd_launch_float_interp(const mgd_program *prog, const mgd_bindings *bind, int32_t dt, void *stream) {
  int st = validate_program(prog, bind);
  if (st != MG_OK) return st;
  Replanned r;
  replan(*prog, &r);
  size_t smem = r.smem_bytes;
  if (smem > (size_t)kSmemLimit)
    return set_error(MG_ERR_UNSUPPORTED,
                     "the generic float interpreter keeps computed tiles in fp32 and this graph needs more than 227 KB "
                     "that way; only graphs matched by a specialised kernel can run at this size");
  int64_t blocks = (int64_t)prog->grid[0] * prog->grid[1] * prog->grid[2] * bind->num_sets;
  if (blocks > 0x7fffffffLL) return set_error(MG_ERR_UNSUPPORTED, "too many blocks for one launch");
  // Blocks run one operator at a time with a barrier after each: big tiles get more warps to hide the latency of
  // the dependent instruction chains (the largest operator decides; a matmul thread owns up to 16 outputs).
  int64_t largest = 0;
  for (int i = 0; i < prog->num_ops; i++) {
    int32_t const *a = prog->ops[i].a;
    int64_t work = 0;
    switch (prog->ops[i].type) {
      case 2001: work = (int64_t)a[14] * a[15] / 8; break;
      case 2002: work = (int64_t)a[11] * a[12]; break;
      case MG_TB_MATMUL_OP: work = (int64_t)a[0] * a[1] / 4; break;
      case MG_TB_EXP_OP: work = a[1]; break;
      default: work = a[0]; break;
    }
    if (work > largest) largest = work;
  }
  unsigned const threads = largest >= 8192 ? 1024u : (largest >= 2048 ? 512u : 256u);
  static bool configured_h = false, configured_b = false;
  if (dt == MG_DT_FLOAT16) {
    if (smem > 48 * 1024 && !configured_h) {
      if (cudaFuncSetAttribute(float_interp_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(float_interp_kernel)");
      configured_h = true;
    }
    float_interp_kernel<__half><<<(unsigned)blocks, threads, smem, (cudaStream_t)stream>>>(r.prog, *bind);
  } else if (dt == MG_DT_BFLOAT16) {
    if (smem > 48 * 1024 && !configured_b) {
      if (cudaFuncSetAttribute(float_interp_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(float_interp_kernel)");
      configured_b = true;
    }
    float_interp_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, smem, (cudaStream_t)stream>>>(r.prog, *bind);
  } else {
    return set_error(MG_ERR_UNSUPPORTED, "float mode runs on fp16 or bf16 tensors");
  }
  return check_launch("float_interp_kernel");
}
