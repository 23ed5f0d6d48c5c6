// Generic float interpreter: evaluates any threadblock program on fp16 / bf16 tensors.
//
// Semantics (the ones the reference's fingerprint interpreter and its Triton generator define,
// src/kernel/cuda/customized_kernel.cu:307-603 and src/kernel/triton_code_gen.cc:222-268): per
// for-loop iteration every operator is recomputed from freshly loaded tiles; output operators add
// their operand into an accumulator across iterations and store it, row-major, after the last one.
// The reference's own float kernel (customized_kernel.cu:39-305) is a timing stand-in that never
// writes its accumulators; this kernel computes the values.
//
// Tiles are held in shared memory as fp32 (twice the planned bytes) so that chained operators do
// not round to 16 bits between steps; inputs are widened on load and outputs rounded to nearest on
// store.  Loads honour the tensor's DmemLayout: a column-major tensor keeps each [rows, cols]
// matrix with the row index contiguous.
#include "common.cuh"

namespace mgk {
int validate_program(mgd_program const *p, mgd_bindings const *b);

template <typename T>
__global__ void __launch_bounds__(256) float_interp_kernel(const __grid_constant__ mgd_program prog,
                                                           const __grid_constant__ mgd_bindings bind) {
  extern __shared__ __align__(16) float smem_f[];
  int const tid = threadIdx.x, nt = blockDim.x;
  int const gx = prog.grid[0], gy = prog.grid[1], gz = prog.grid[2];
  int64_t b = blockIdx.x;
  int const bx = (int)(b % gx), by = (int)((b / gx) % gy), bz = (int)((b / ((int64_t)gx * gy)) % gz);
  int64_t const set = b / ((int64_t)gx * gy * gz);
  // planned offsets count 2 bytes per element: element index = offset / 2
  auto tile = [&](int byte_offset) { return smem_f + (byte_offset >> 1); };

  for (int it = 0; it < prog.forloop_range; it++) {
    for (int oi = 0; oi < prog.num_ops; oi++) {
      mgd_op const &op = prog.ops[oi];
      int32_t const *a = op.a;
      switch (op.type) {
        case 2001: {
          int row = bx * a[0] + by * a[1] + bz * a[2] + it * a[6];
          int col = bx * a[3] + by * a[4] + bz * a[5] + it * a[7];
          int64_t lead = (int64_t)bx * a[8] + (int64_t)by * a[9] + (int64_t)bz * a[10] + (int64_t)it * a[11];
          T const *src = static_cast<T const *>(bind.in[a[18]]) + set * bind.in_set_stride[a[18]] + lead;
          float *dst = tile(a[17]);
          int rows = a[14], cols = a[15], n = rows * cols;
          if (a[16] == MG_DMEM_COLUMN_MAJOR) {
            int ld = a[12]; // rows of the whole matrix: consecutive rows are adjacent in memory
            for (int i = tid; i < n; i += nt) {
              int c = i / rows, r = i % rows;
              dst[r * cols + c] = to_float<T>(src[(size_t)(col + c) * ld + row + r]);
            }
          } else {
            int ld = a[13];
            for (int i = tid; i < n; i += nt) {
              int r = i / cols, c = i % cols;
              dst[i] = to_float<T>(src[(size_t)(row + r) * ld + col + c]);
            }
          }
          break;
        }
        case MG_TB_MATMUL_OP: {
          int m = a[0], n = a[1], k = a[2];
          float const *A = tile(a[3]), *B = tile(a[4]);
          float *C = tile(a[5]);
          for (int i = tid; i < m * n; i += nt) {
            int r = i / n, c = i % n;
            float acc = 0.f;
            for (int kk = 0; kk < k; kk++) acc = fmaf(A[r * k + kk], B[kk * n + c], acc);
            C[i] = acc;
          }
          break;
        }
        case MG_TB_EXP_OP: {
          float *x = tile(a[0]);
          for (int i = tid; i < a[1]; i += nt) x[i] = expf(x[i]);
          break;
        }
        case MG_TB_DIV_OP:
        case MG_TB_ADD_OP:
        case MG_TB_MUL_OP: {
          int const xd[3] = {a[0], a[1], a[2]}, yd[3] = {a[3], a[4], a[5]};
          int const zd[3] = {max(xd[0], yd[0]), max(xd[1], yd[1]), max(xd[2], yd[2])};
          float const *x = tile(a[6]), *y = tile(a[7]);
          float *z = tile(a[8]);
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
            float xv = x[xi], yv = y[yi];
            z[i] = op.type == MG_TB_DIV_OP ? xv / yv : (op.type == MG_TB_ADD_OP ? xv + yv : xv * yv);
          }
          break;
        }
        case MG_TB_REDUCTION_0_OP: case MG_TB_REDUCTION_1_OP: case MG_TB_REDUCTION_2_OP:
        case MG_TB_REDUCTION_0_TO_DIMX_OP: case MG_TB_REDUCTION_1_TO_DIMX_OP: case MG_TB_REDUCTION_2_TO_DIMX_OP: {
          int n_out = a[0], degree = a[1], inner = a[2];
          float const *x = tile(a[3]);
          float *y = tile(a[4]);
          for (int i = tid; i < n_out; i += nt) {
            int pos = (i / inner) * (inner * degree) + i % inner;
            float acc = 0.f;
            for (int k = 0; k < degree; k++, pos += inner) acc += x[pos];
            y[i] = acc;
          }
          break;
        }
        case MG_TB_CONCAT_0_OP: case MG_TB_CONCAT_1_OP: case MG_TB_CONCAT_2_OP: {
          int n_out = a[0], ad = a[1], bd = a[2], inner = a[3];
          float const *A = tile(a[4]), *B = tile(a[5]);
          float *y = tile(a[6]);
          for (int i = tid; i < n_out; i += nt) {
            int in_idx = i % inner, along = (i / inner) % (ad + bd), outer = (i / inner) / (ad + bd);
            y[i] = along < ad ? A[in_idx + along * inner + outer * inner * ad]
                              : B[in_idx + (along - ad) * inner + outer * inner * bd];
          }
          break;
        }
        case 2002: {
          int n = a[11] * a[12];
          float const *x = tile(a[13]);
          float *acc = tile(a[14]);
          if (it == 0) {
            for (int i = tid; i < n; i += nt) acc[i] = x[i];
          } else {
            for (int i = tid; i < n; i += nt) acc[i] += x[i];
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
} // namespace mgk

using namespace mgk;

extern "C" int mgd_float_interp_smem(const mgd_program *prog, size_t *bytes, int32_t *fits) {
  if (!prog || !bytes || !fits) return set_error(MG_ERR_INVALID_ARGUMENT, "null pointer");
  *bytes = (size_t)prog->smem_bytes * 2 + 16;
  *fits = *bytes <= (size_t)kSmemLimit;
  return MG_OK;
}

extern "C" int mgd_launch_float_interp(const mgd_program *prog, const mgd_bindings *bind, int32_t dt, void *stream) {
  int st = validate_program(prog, bind);
  if (st != MG_OK) return st;
  size_t smem = (size_t)prog->smem_bytes * 2 + 16;
  if (smem > (size_t)kSmemLimit)
    return set_error(MG_ERR_UNSUPPORTED,
                     "the generic float interpreter keeps fp32 tiles and this graph needs more than 227 KB that way; "
                     "only graphs matched by a specialised kernel can run at this size");
  int64_t blocks = (int64_t)prog->grid[0] * prog->grid[1] * prog->grid[2] * bind->num_sets;
  if (blocks > 0x7fffffffLL) return set_error(MG_ERR_UNSUPPORTED, "too many blocks for one launch");
  static bool configured_h = false, configured_b = false;
  if (dt == MG_DT_FLOAT16) {
    if (smem > 48 * 1024 && !configured_h) {
      if (cudaFuncSetAttribute(float_interp_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(float_interp_kernel)");
      configured_h = true;
    }
    float_interp_kernel<__half><<<(unsigned)blocks, 256, smem, (cudaStream_t)stream>>>(*prog, *bind);
  } else if (dt == MG_DT_BFLOAT16) {
    if (smem > 48 * 1024 && !configured_b) {
      if (cudaFuncSetAttribute(float_interp_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(float_interp_kernel)");
      configured_b = true;
    }
    float_interp_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, smem, (cudaStream_t)stream>>>(*prog, *bind);
  } else {
    return set_error(MG_ERR_UNSUPPORTED, "float mode runs on fp16 or bf16 tensors");
  }
  return check_launch("float_interp_kernel");
}
