/* f32_oracle.c - fp32 host evaluation of a threadblock program.  TEST INFRASTRUCTURE ONLY.
 *
 * Float mode has no usable reference implementation (the reference's fp16 interpreter,
 * src/kernel/cuda/customized_kernel.cu:39-305, never writes its accumulators), so the parity target
 * is an fp32 evaluation of the graph semantics the fingerprint interpreter (:307-603) and the Triton
 * generator (src/kernel/triton_code_gen.cc:222-268) define: per for-loop iteration every operator is
 * recomputed from freshly loaded tiles, output operators add across iterations and store row-major.
 * This file is the compiled, multi-threaded form of mugraph_oracle.run_float and is what the
 * benchmark times as the CPU baseline of the float path; tests check it against the numpy version.
 *
 * Inputs arrive as fp32 values already rounded to the 16-bit storage type, in memory order (a
 * column-major tensor keeps each [rows, cols] matrix with the row index contiguous).  Operator
 * records are the 20-int records documented in oracle/fp_oracle.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#define REC 20

static void run_block_f32(const int32_t *ops, int num_ops, int forloop_range, int bx, int by, int bz,
                          const float *const *in, float *const *out, float *smem) {
  for (int it = 0; it < forloop_range; it++) {
    for (int o = 0; o < num_ops; o++) {
      const int32_t *r = ops + o * REC, *a = r + 1;
      int type = r[0];
      if (type == 2001) {
        int row = bx * a[0] + by * a[1] + bz * a[2] + it * a[6];
        int col = bx * a[3] + by * a[4] + bz * a[5] + it * a[7];
        long glob = (long)bx * a[8] + (long)by * a[9] + (long)bz * a[10] + (long)it * a[11];
        const float *src = in[a[18]] + glob;
        float *dst = smem + a[17] / 2;
        int rows = a[14], cols = a[15];
        if (a[16] == 101) { /* column-major: leading dimension = rows of the whole matrix */
          int ld = a[12];
          for (int c = 0; c < cols; c++)
            for (int rr = 0; rr < rows; rr++) dst[rr * cols + c] = src[(long)(col + c) * ld + row + rr];
        } else {
          int ld = a[13];
          for (int i = 0; i < rows * cols; i++) dst[i] = src[(long)(row + i / cols) * ld + col + i % cols];
        }
      } else if (type == 2003) {
        int m = a[0], n = a[1], k = a[2];
        const float *A = smem + a[3] / 2, *B = smem + a[4] / 2;
        float *C = smem + a[5] / 2;
        for (int i = 0; i < m * n; i++) C[i] = 0.f;
        for (int mm = 0; mm < m; mm++)
          for (int x = 0; x < k; x++) {
            float av = A[mm * k + x];
            const float *brow = B + x * n;
            float *crow = C + mm * n;
            for (int nn = 0; nn < n; nn++) crow[nn] += av * brow[nn];
          }
      } else if (type == 2007) {
        float *p = smem + a[0] / 2;
        for (int i = 0; i < a[1]; i++) p[i] = expf(p[i]);
      } else if (type == 2010 || type == 2008 || type == 2009) {
        const int xd[3] = {a[0], a[1], a[2]}, yd[3] = {a[3], a[4], a[5]};
        int zd[3];
        for (int d = 0; d < 3; d++) zd[d] = xd[d] > yd[d] ? xd[d] : yd[d];
        const float *X = smem + a[6] / 2, *Y = smem + a[7] / 2;
        float *Z = smem + a[8] / 2;
        int n = zd[0] * zd[1] * zd[2];
        for (int i = 0; i < n; i++) {
          int idx = i, xs = 1, ys = 1, xi = 0, yi = 0;
          for (int d = 2; d >= 0; d--) {
            xi += (idx % xd[d]) * xs;
            yi += (idx % yd[d]) * ys;
            xs *= xd[d];
            ys *= yd[d];
            idx /= zd[d];
          }
          Z[i] = type == 2010 ? X[xi] / Y[yi] : (type == 2008 ? X[xi] + Y[yi] : X[xi] * Y[yi]);
        }
      } else if (type >= 2101 && type <= 2106) {
        int n_out = a[0], deg = a[1], inner = a[2];
        const float *X = smem + a[3] / 2;
        float *Y = smem + a[4] / 2;
        for (int i = 0; i < n_out; i++) {
          int pos = (i / inner) * (inner * deg) + i % inner;
          float acc = 0.f;
          for (int k = 0; k < deg; k++, pos += inner) acc += X[pos];
          Y[i] = acc;
        }
      } else if (type >= 2200 && type <= 2202) {
        int n_out = a[0], ad = a[1], bd = a[2], inner = a[3];
        const float *A = smem + a[4] / 2, *B = smem + a[5] / 2;
        float *Y = smem + a[6] / 2;
        for (int i = 0; i < n_out; i++) {
          int ii = i % inner, along = (i / inner) % (ad + bd), outer = (i / inner) / (ad + bd);
          Y[i] = along < ad ? A[ii + along * inner + outer * inner * ad] : B[ii + (along - ad) * inner + outer * inner * bd];
        }
      } else if (type == 2002) {
        int n = a[11] * a[12];
        const float *X = smem + a[13] / 2;
        float *acc = smem + a[14] / 2;
        if (it == 0) {
          for (int i = 0; i < n; i++) acc[i] = X[i];
        } else {
          for (int i = 0; i < n; i++) acc[i] += X[i];
        }
        if (it == forloop_range - 1) {
          int row = bx * a[0] + by * a[1] + bz * a[2], col = bx * a[3] + by * a[4] + bz * a[5];
          long glob = (long)bx * a[6] + (long)by * a[7] + (long)bz * a[8];
          float *dst = out[a[15]] + glob;
          int cols = a[12], ld = a[10];
          for (int i = 0; i < n; i++) dst[(long)(row + i / cols) * ld + col + i % cols] = acc[i];
        }
      }
    }
  }
}

int f32_oracle_run(const int32_t *ops, int num_ops, const int32_t *grid, int forloop_range, int smem_bytes,
                   int num_in, const float *const *in, int num_out, float *const *out, int threads) {
  int gx = grid[0], gy = grid[1], gz = grid[2];
  long blocks = (long)gx * gy * gz;
  int used = 1;
  (void)num_in;
  (void)num_out;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
  used = threads > 0 ? threads : omp_get_max_threads();
#endif
#pragma omp parallel
  {
    float *smem = (float *)malloc(((size_t)smem_bytes / 2 + 16) * sizeof(float));
#pragma omp for schedule(dynamic, 1)
    for (long b = 0; b < blocks; b++) {
      int bx = (int)(b % gx), by = (int)((b / gx) % gy), bz = (int)(b / ((long)gx * gy));
      run_block_f32(ops, num_ops, forloop_range, bx, by, bz, in, out, smem);
    }
    free(smem);
  }
  return used;
}
