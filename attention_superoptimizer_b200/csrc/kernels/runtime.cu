// Launch bookkeeping, fills, comparison and the device status word.
#include "common.cuh"
#include "ptx.cuh"
#include "mugraph_rng.h"
#include <atomic>
#include <cstring>
#include <mutex>
#include <string>

namespace mgk {
static std::atomic<uint64_t> g_launches{0};
static thread_local std::string g_err;
static int32_t *g_error_word = nullptr;

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
int set_error(int code, char const *msg) {
  g_err = msg;
  return code;
}
int check_launch(char const *name) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) {
    count_launch();
    return MG_OK;
  }
  g_err = std::string(name) + ": " + cudaGetErrorString(e);
  return MG_ERR_CUDA;
}
static std::atomic<int32_t> g_options[MGD_OPT_COUNT];
int option(int key) { return key >= 0 && key < MGD_OPT_COUNT ? g_options[key].load(std::memory_order_relaxed) : 0; }

// cuTensorMapEncodeTiled is a pure function of its arguments and costs about a microsecond of host time; a launch
// encodes two to five maps.  Callers get a wrapper that remembers the last few results per thread, so that a host
// which calls again and again on the same buffers (a serving loop on a resident KV cache) pays for the encoding once.
namespace {
TensorMapEncodeFn g_driver_encode = nullptr;
struct MapKey {
  int32_t data_type, interleave, swizzle, l2_promotion, oob_fill;
  uint32_t rank;
  void *base;
  uint64_t dims[5], strides[4];
  uint32_t box[5], element_strides[5];
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kCachedMaps = 16;

CUresult encode_tiled_remembered(CUtensorMap *map, CUtensorMapDataType data_type, cuuint32_t rank, void *base,
                                 cuuint64_t const *dims, cuuint64_t const *strides, cuuint32_t const *box,
                                 cuuint32_t const *element_strides, CUtensorMapInterleave interleave,
                                 CUtensorMapSwizzle swizzle, CUtensorMapL2promotion l2_promotion,
                                 CUtensorMapFloatOOBfill oob_fill) {
  if (rank < 1 || rank > 5)
    return g_driver_encode(map, data_type, rank, base, dims, strides, box, element_strides, interleave, swizzle, l2_promotion, oob_fill);
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.data_type = (int32_t)data_type; key.interleave = (int32_t)interleave; key.swizzle = (int32_t)swizzle;
  key.l2_promotion = (int32_t)l2_promotion; key.oob_fill = (int32_t)oob_fill;
  key.rank = rank;
  key.base = base;
  for (uint32_t i = 0; i < rank; i++) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
    key.element_strides[i] = element_strides[i];
    if (i + 1 < rank) key.strides[i] = strides[i];
  }
  thread_local MapEntry table[kCachedMaps];
  thread_local unsigned next = 0;
  for (MapEntry const &e : table)
    if (e.used && std::memcmp(&e.key, &key, sizeof(key)) == 0) {
      *map = e.map;
      return CUDA_SUCCESS;
    }
  CUresult const r = g_driver_encode(map, data_type, rank, base, dims, strides, box, element_strides, interleave, swizzle, l2_promotion, oob_fill);
  if (r == CUDA_SUCCESS) {
    MapEntry &e = table[next++ % kCachedMaps];
    e.key = key;
    e.map = *map;
    e.used = true;
  }
  return r;
}
} // namespace

TensorMapEncodeFn tensor_map_encoder() {
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_driver_encode = reinterpret_cast<TensorMapEncodeFn>(sym);
  });
  return g_driver_encode ? &encode_tiled_remembered : nullptr;
}

int32_t *device_error_word() {
  if (!g_error_word) {
    if (cudaMalloc((void **)&g_error_word, 256) != cudaSuccess) return nullptr;
    cudaMemset(g_error_word, 0, 256);
  }
  return g_error_word;
}

// ---- kernels ------------------------------------------------------------------------------------------
__global__ void fill_fp_reference_kernel(uint16_t *p, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = (uint16_t)(i % PQ);
}

__global__ void fill_fp_seeded_kernel(uint16_t *p, int64_t n, uint64_t seed, uint32_t modulus) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    p[i] = (uint16_t)mg_rng_uniform(seed, (uint64_t)i, modulus);
}

template <typename T> __global__ void fill_data_seeded_kernel(T *p, int64_t n, uint64_t seed, float sigma) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    p[i] = from_float<T>(mg_rng_normal(seed, (uint64_t)i) * sigma);
}

// flag starts at 1; any block that sees a difference clears it
__global__ void compare_init_kernel(int32_t *flag) { *flag = 1; }
__global__ void compare_u16_kernel(uint16_t const *a, uint16_t const *b, int64_t n, int32_t *flag) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  bool diff = false;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) diff |= a[i] != b[i];
  if (__syncthreads_or(diff) && threadIdx.x == 0) *flag = 0;
}

// One block, one barrier with a single expected arrival that never comes: exercises the bounded wait and the
// status word without any other work.
__global__ void bounded_wait_selftest_kernel(int limit, int32_t *status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::mbar_init_fence();
    if (!ptx::mbar_wait(ptx::smem_u32(&bar), 0, limit)) atomicExch(status, 2);
  }
}

// One block per row (grid-stride over rows): 128-bit loads when the rows allow it, one flag per row.
__global__ void compare_rows_u16_kernel(uint16_t const *a, uint16_t const *b, int64_t rows, int64_t row_elems, int vec_ok,
                                        int32_t *flags, int32_t *mismatches) {
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    uint16_t const *pa = a + r * row_elems, *pb = b + r * row_elems;
    bool diff = false;
    if (vec_ok) {
      uint4 const *va = reinterpret_cast<uint4 const *>(pa), *vb = reinterpret_cast<uint4 const *>(pb);
      for (int64_t i = threadIdx.x; i < row_elems / 8; i += blockDim.x) {
        uint4 x = __ldg(va + i), y = __ldg(vb + i);
        diff |= (x.x != y.x) | (x.y != y.y) | (x.z != y.z) | (x.w != y.w);
      }
    } else {
      for (int64_t i = threadIdx.x; i < row_elems; i += blockDim.x) diff |= pa[i] != pb[i];
    }
    int any = __syncthreads_or(diff);
    if (threadIdx.x == 0) {
      flags[r] = any ? 0 : 1;
      if (any && mismatches) atomicAdd(mismatches, 1);
    }
  }
}

static int grid_for(int64_t n, int threads) {
  int64_t blocks = (n + threads - 1) / threads;
  int64_t cap = 148 * 16;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}
} // namespace mgk

using namespace mgk;

extern "C" {

int mgd_fill_fingerprint_reference(uint16_t *p, int64_t n, void *stream) {
  if (!p || n < 0) return set_error(MG_ERR_INVALID_ARGUMENT, "fill: null pointer");
  if (n == 0) return MG_OK;
  fill_fp_reference_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(p, n);
  return check_launch("fill_fp_reference_kernel");
}

int mgd_fill_fingerprint_seeded(uint16_t *p, int64_t n, uint64_t seed, uint32_t modulus, void *stream) {
  if (!p || n < 0 || modulus == 0) return set_error(MG_ERR_INVALID_ARGUMENT, "fill: bad argument");
  if (n == 0) return MG_OK;
  fill_fp_seeded_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(p, n, seed, modulus);
  return check_launch("fill_fp_seeded_kernel");
}

int mgd_fill_data_seeded(void *p, int64_t n, uint64_t seed, float sigma, int32_t dt, void *stream) {
  if (!p || n < 0) return set_error(MG_ERR_INVALID_ARGUMENT, "fill: bad argument");
  if (n == 0) return MG_OK;
  if (dt == MG_DT_FLOAT16)
    fill_data_seeded_kernel<__half><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((__half *)p, n, seed, sigma);
  else if (dt == MG_DT_BFLOAT16)
    fill_data_seeded_kernel<__nv_bfloat16>
        <<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16 *)p, n, seed, sigma);
  else
    return set_error(MG_ERR_UNSUPPORTED, "fill: 16-bit float types only");
  return check_launch("fill_data_seeded_kernel");
}

int mgd_compare_u16(const uint16_t *a, const uint16_t *b, int64_t n, int32_t *flag, void *stream) {
  if (!a || !b || !flag || n < 0) return set_error(MG_ERR_INVALID_ARGUMENT, "compare: null pointer");
  compare_init_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(flag);
  if (n > 0) compare_u16_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(a, b, n, flag);
  return check_launch("compare_u16_kernel");
}

int mgd_compare_rows_u16(const uint16_t *a, const uint16_t *b, int64_t rows, int64_t row_elems, int32_t *flags,
                         int32_t *mismatches, void *stream) {
  if (!a || !b || !flags || rows < 0 || row_elems <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "compare rows: bad argument");
  if (mismatches && cudaMemsetAsync(mismatches, 0, sizeof(int32_t), (cudaStream_t)stream) != cudaSuccess)
    return check_launch("cudaMemsetAsync(mismatch count)");
  if (rows == 0) return MG_OK;
  int const vec_ok = row_elems % 8 == 0 && (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) % 16 == 0;
  int64_t const blocks = rows < 148 * 16 ? rows : 148 * 16;
  compare_rows_u16_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(a, b, rows, row_elems, vec_ok, flags, mismatches);
  return check_launch("compare_rows_u16_kernel");
}

int mgd_tables_init(const uint16_t *e, const uint16_t *p, const uint16_t *q) {
  // The kernels carry compile-time tables; this verifies that the caller's tables agree with them.
  FieldTables t;
  if (!e || !p || !q) return set_error(MG_ERR_INVALID_ARGUMENT, "tables: null pointer");
  if (std::memcmp(e, t.e, sizeof(t.e)) || std::memcmp(p, t.p, sizeof(t.p)) || std::memcmp(q, t.q, sizeof(t.q)))
    return set_error(MG_ERR_INVALID_ARGUMENT, "tables: lookup tables differ from the built-in ones");
  return MG_OK;
}

int mgd_read_and_clear_device_error(int32_t *code) {
  if (!code) return set_error(MG_ERR_INVALID_ARGUMENT, "null pointer");
  *code = 0;
  int32_t *w = device_error_word();
  if (!w) return set_error(MG_ERR_CUDA, "cannot allocate the device status word");
  if (cudaMemcpy(code, w, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return set_error(MG_ERR_CUDA, "status word read failed");
  if (*code != 0) cudaMemset(w, 0, 4);
  return MG_OK;
}

int mgd_set_option(int32_t key, int32_t value) {
  if (key < 0 || key >= MGD_OPT_COUNT || value < 0) return set_error(MG_ERR_INVALID_ARGUMENT, "unknown option or negative value");
  g_options[key].store(value, std::memory_order_relaxed);
  return MG_OK;
}
int mgd_get_option(int32_t key, int32_t *value) {
  if (key < 0 || key >= MGD_OPT_COUNT || !value) return set_error(MG_ERR_INVALID_ARGUMENT, "unknown option");
  *value = option(key);
  return MG_OK;
}

int mgd_selftest_bounded_wait(int32_t poll_limit, void *stream) {
  if (poll_limit < 1 || poll_limit > ptx::kWaitLimit) return set_error(MG_ERR_INVALID_ARGUMENT, "poll limit out of range");
  int32_t *w = device_error_word();
  if (!w) return set_error(MG_ERR_CUDA, "cannot allocate the device status word");
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(poll_limit, w);
  return check_launch("bounded_wait_selftest_kernel");
}

uint64_t mgd_launch_count(void) { return g_launches.load(); }
const char *mgd_last_error(void) { return g_err.c_str(); }
}
