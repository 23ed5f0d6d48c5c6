/* fp_oracle.c - plain-C restatement of the fingerprint interpreter.  TEST INFRASTRUCTURE ONLY.
 *
 * Used as the timed CPU baseline ("port") and as a second checker at sizes where the numpy oracle is
 * slow.  It walks blocks x for-loop iterations x operators like the reference kernel
 * compute_customizedop_fingerprint (src/kernel/cuda/customized_kernel.cu:307-603) and performs each
 * operator with the reference's arithmetic, including the modulo after every multiply-add of
 * TBMatmulFingerprinter (include/mirage/threadblock/cuda/matmul.h:773-804), the table exp of
 * element_unary.h:60-66, the CRT division of element_binary.h:89-106, the strided reduction of
 * reduction.h:147-156, the concat of concat.h:90-101 and the accumulate / save pair of
 * output_saver.h:374-447.  Loader indexing is row-major whatever the layout (input_loader.h:457-467).
 *
 * The program arrives as flat int records produced by oracle/fp_oracle.py from the numpy oracle's
 * graph builder: per operator 20 ints {type, a[0..18]} with the meaning documented there.
 * Parity status: pinned through tests/test_oracle_c.py (equal to the numpy oracle, which is pinned
 * against the reference-host golden vectors).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define FP_P 227u
#define FP_Q 113u
#define FP_PQ 25651u
#define Q_MUL_P_MOD_1 25425u
#define P_MUL_Q_MOD_1 227u
#define REC 20

static uint16_t exp_tbl[FP_Q], divp_tbl[FP_P], divq_tbl[FP_Q];
static int tables_ready = 0;

/* src/kernel/device_memory_manager.cu:41-90 */
static void build_tables(void) {
  exp_tbl[0] = 1;
  for (unsigned i = 1; i < FP_Q; i++) exp_tbl[i] = (uint16_t)((exp_tbl[i - 1] * 3u) % FP_P);
  for (unsigned i = 0; i < FP_P; i++) {
    divp_tbl[i] = 1;
    for (unsigned j = 1; j < FP_P; j++)
      if ((i * j) % FP_P == 1) divp_tbl[i] = (uint16_t)j;
  }
  for (unsigned i = 0; i < FP_Q; i++) {
    divq_tbl[i] = 1;
    for (unsigned j = 1; j < FP_Q; j++)
      if ((i * j) % FP_Q == 1) divq_tbl[i] = (uint16_t)j;
  }
  tables_ready = 1;
}

static void run_block(const int32_t *ops, int num_ops, int forloop_range, int bx, int by, int bz,
                      const uint16_t *const *in, uint16_t *const *out, unsigned char *smem) {
  for (int it = 0; it < forloop_range; it++) {
    for (int o = 0; o < num_ops; o++) {
      const int32_t *r = ops + o * REC;
      const int32_t *a = r + 1;
      int type = r[0];
      if (type == 2001) { /* input loader */
        int row = bx * a[0] + by * a[1] + bz * a[2] + it * a[6];
        int col = bx * a[3] + by * a[4] + bz * a[5] + it * a[7];
        long glob = (long)bx * a[8] + (long)by * a[9] + (long)bz * a[10] + (long)it * a[11];
        const uint16_t *src = in[a[18]] + glob;
        uint16_t *dst = (uint16_t *)(smem + a[17]);
        int rows = a[14], cols = a[15], ld = a[13];
        for (int i = 0; i < rows * cols; i++) dst[i] = src[(long)(row + i / cols) * ld + col + i % cols];
      } else if (type == 2003) { /* matmul, reduce after every multiply-add */
        int m = a[0], n = a[1], k = a[2];
        const uint16_t *A = (const uint16_t *)(smem + a[3]), *B = (const uint16_t *)(smem + a[4]);
        uint16_t *C = (uint16_t *)(smem + a[5]);
        for (int i = 0; i < m * n; i++) {
          uint32_t res = 0;
          int mm = i / n, nn = i % n;
          for (int x = 0; x < k; x++) res = (res + (uint32_t)A[mm * k + x] * (uint32_t)B[x * n + nn]) % FP_PQ;
          C[i] = (uint16_t)res;
        }
      } else if (type == 2007) { /* exp */
        uint16_t *p = (uint16_t *)(smem + a[0]);
        for (int i = 0; i < a[1]; i++) p[i] = (uint16_t)(((uint32_t)exp_tbl[p[i] % FP_Q] * Q_MUL_P_MOD_1) % FP_PQ);
      } else if (type == 2010) { /* div with broadcast over the last three dims */
        const int xd[3] = {a[0], a[1], a[2]}, yd[3] = {a[3], a[4], a[5]};
        int zd[3];
        for (int d = 0; d < 3; d++) zd[d] = xd[d] > yd[d] ? xd[d] : yd[d];
        const uint16_t *X = (const uint16_t *)(smem + a[6]), *Y = (const uint16_t *)(smem + a[7]);
        uint16_t *Z = (uint16_t *)(smem + a[8]);
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
          uint32_t x = X[xi], y = Y[yi];
          uint32_t z = (x % FP_P) * divp_tbl[y % FP_P] * Q_MUL_P_MOD_1 + (x % FP_Q) * divq_tbl[y % FP_Q] * P_MUL_Q_MOD_1;
          Z[i] = (uint16_t)(z % FP_PQ);
        }
      } else if (type >= 2101 && type <= 2106) { /* reduction / reduction to dimx */
        int n_out = a[0], deg = a[1], inner = a[2];
        const uint16_t *X = (const uint16_t *)(smem + a[3]);
        uint16_t *Y = (uint16_t *)(smem + a[4]);
        for (int i = 0; i < n_out; i++) {
          int pos = (i / inner) * (inner * deg) + i % inner;
          uint32_t res = 0;
          for (int k = 0; k < deg; k++, pos += inner) res = (res + X[pos]) % FP_PQ;
          Y[i] = (uint16_t)res;
        }
      } else if (type >= 2200 && type <= 2202) { /* concat */
        int n_out = a[0], ad = a[1], bd = a[2], inner = a[3];
        const uint16_t *A = (const uint16_t *)(smem + a[4]), *B = (const uint16_t *)(smem + a[5]);
        uint16_t *Y = (uint16_t *)(smem + a[6]);
        for (int i = 0; i < n_out; i++) {
          int ii = i % inner, along = (i / inner) % (ad + bd), outer = (i / inner) / (ad + bd);
          Y[i] = along < ad ? A[ii + along * inner + outer * inner * ad] : B[ii + (along - ad) * inner + outer * inner * bd];
        }
      } else if (type == 2002) { /* output: accumulate, save on the last iteration */
        int n = a[11] * a[12];
        const uint16_t *X = (const uint16_t *)(smem + a[13]);
        uint16_t *acc = (uint16_t *)(smem + a[14]);
        if (it == 0) {
          for (int i = 0; i < n; i++) acc[i] = X[i];
        } else {
          for (int i = 0; i < n; i++) acc[i] = (uint16_t)(((uint32_t)X[i] + acc[i]) % FP_PQ);
        }
        if (it == forloop_range - 1) {
          int row = bx * a[0] + by * a[1] + bz * a[2], col = bx * a[3] + by * a[4] + bz * a[5];
          long glob = (long)bx * a[6] + (long)by * a[7] + (long)bz * a[8];
          uint16_t *dst = out[a[15]] + glob;
          int cols = a[12], ld = a[10];
          for (int i = 0; i < n; i++) dst[(long)(row + i / cols) * ld + col + i % cols] = acc[i];
        }
      }
    }
  }
}

/* Evaluates one customized operator on `num_sets` tensor sets (set s at in[i] + s*in_stride[i]).
 * threads <= 0 uses every core OpenMP sees.  Returns the number of threads used. */
int fp_oracle_run(const int32_t *ops, int num_ops, const int32_t *grid, int forloop_range, int smem_bytes,
                  int num_in, const uint16_t *const *in, const int64_t *in_stride, int num_out, uint16_t *const *out,
                  const int64_t *out_stride, int num_sets, int threads) {
  if (!tables_ready) build_tables();
  int gx = grid[0], gy = grid[1], gz = grid[2];
  long blocks = (long)gx * gy * gz * num_sets;
  int used = 1;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
  used = threads > 0 ? threads : omp_get_max_threads();
#endif
#pragma omp parallel
  {
    unsigned char *smem = (unsigned char *)malloc((size_t)smem_bytes + 64);
    const uint16_t *ins[8];
    uint16_t *outs[8];
#pragma omp for schedule(dynamic, 4)
    for (long b = 0; b < blocks; b++) {
      int bx = (int)(b % gx), by = (int)((b / gx) % gy), bz = (int)((b / ((long)gx * gy)) % gz);
      long set = b / ((long)gx * gy * gz);
      for (int i = 0; i < num_in; i++) ins[i] = in[i] + set * in_stride[i];
      for (int i = 0; i < num_out; i++) outs[i] = out[i] + set * out_stride[i];
      run_block(ops, num_ops, forloop_range, bx, by, bz, ins, outs, smem);
    }
    free(smem);
  }
  return used;
}
