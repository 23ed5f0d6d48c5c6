// A customized operator that is one threadblock reduction - input tile, tb_reduction_*_op (plain or "to dimx"),
// output tile, for-loop of one - as a kernel of its own: the kernel-level cross-block reduction behind a split
// operator (the second customized op of the reference's matmul-chain and attention examples sums the partial results
// of the first one's blocks).  Nothing is staged in shared memory: output element i of a block's tile is
//     sum over k < degree of  in_tile[(i / inner) * inner * degree + i % inner + k * inner]
// in the tile's dense row-major numbering (what the threadblock operator computes on its shared-memory copy); thread
// i reads its `degree` terms straight from global memory, neighbouring threads neighbouring addresses.  Float mode sums
// in fp32 and rounds once; fingerprint mode sums exactly and reduces modulo PQ.
#include "common.cuh"
#include <cstring>

namespace mgk {
namespace tred {

struct Params {
  mgd_tile_reduce c;
  void const *in;
  void *out;
  long long in_set, out_set;
};

template <int MODE> // 0 fp16, 1 bf16, 2 fingerprint
__global__ void __launch_bounds__(256) tile_reduce_kernel(const __grid_constant__ Params p) {
  mgd_tile_reduce const &c = p.c;
  int const gx = c.grid[0], gy = c.grid[1], gz = c.grid[2];
  long long const blocks_per_set = (long long)gx * gy * gz;
  long long const b = blockIdx.x / c.chunks;
  int const chunk = (int)(blockIdx.x % c.chunks);
  int const bx = (int)(b % gx), by = (int)((b / gx) % gy), bz = (int)((b / ((long long)gx * gy)) % gz);
  long long const set = b / blocks_per_set;
  int32_t const *ia = c.in.a, *oa = c.out.a;
  long long const irow = (long long)bx * ia[0] + (long long)by * ia[1] + (long long)bz * ia[2];
  long long const icol = (long long)bx * ia[3] + (long long)by * ia[4] + (long long)bz * ia[5];
  long long const ilead = (long long)bx * ia[8] + (long long)by * ia[9] + (long long)bz * ia[10];
  int const ild = ia[MGD_IN_COLS], itc = ia[MGD_IN_TILE_COLS];
  uint16_t const *src = static_cast<uint16_t const *>(p.in) + set * p.in_set + ilead + irow * ild + icol;
  long long const orow = (long long)bx * oa[0] + (long long)by * oa[1] + (long long)bz * oa[2];
  long long const ocol = (long long)bx * oa[3] + (long long)by * oa[4] + (long long)bz * oa[5];
  long long const olead = (long long)bx * oa[6] + (long long)by * oa[7] + (long long)bz * oa[8];
  int const old = oa[MGD_OUT_COLS], otc = oa[MGD_OUT_TILE_COLS];
  uint16_t *dst = static_cast<uint16_t *>(p.out) + set * p.out_set + olead + orow * old + ocol;
  int const inner = c.inner, degree = c.degree;
  for (int i = chunk * 256 + threadIdx.x; i < c.out_elements; i += c.chunks * 256) {
    int pos = (i / inner) * (inner * degree) + i % inner;
    float facc = 0.f;
    unsigned long long iacc = 0;
#pragma unroll 4
    for (int k = 0; k < degree; k++, pos += inner) {
      int const r = pos / itc, cc = pos - r * itc;
      uint16_t const v = __ldg(src + (long long)r * ild + cc);
      if (MODE == 2) iacc += v;
      else if (MODE == 1) facc += __bfloat162float(*reinterpret_cast<__nv_bfloat16 const *>(&v));
      else facc += __half2float(*reinterpret_cast<__half const *>(&v));
    }
    uint16_t res;
    if (MODE == 2) res = (uint16_t)(iacc % PQ);
    else if (MODE == 1) { __nv_bfloat16 h = __float2bfloat16_rn(facc); res = *reinterpret_cast<uint16_t *>(&h); }
    else { __half h = __float2half_rn(facc); res = *reinterpret_cast<uint16_t *>(&h); }
    int const r = i / otc, cc = i - r * otc;
    dst[(long long)r * old + cc] = res;
  }
}

} // namespace tred
} // namespace mgk

using namespace mgk;

extern "C" {

int mgd_tile_reduce_supported(const mgd_tile_reduce *c, int32_t fingerprint_mode) {
  if (!c || c->out_elements <= 0 || c->degree <= 0 || c->inner <= 0) return 0;
  if (c->grid[0] <= 0 || c->grid[1] <= 0 || c->grid[2] <= 0) return 0;
  if (!fingerprint_mode) {
    if (c->data_type != MG_DT_FLOAT16 && c->data_type != MG_DT_BFLOAT16) return 0;
    if ((c->in.a[MGD_IN_LAYOUT] & 0xff) != MG_DMEM_ROW_MAJOR) return 0; // float tensors sit as their layout tag says
  }
  return 1;
}

int mgd_launch_tile_reduce(const mgd_tile_reduce *c, const mgd_bindings *bind, int32_t fingerprint_mode, void *stream) {
  if (!c || !bind || !mgd_tile_reduce_supported(c, fingerprint_mode)) return set_error(MG_ERR_UNSUPPORTED, "tile reduction: not supported");
  tred::Params p;
  std::memset(&p, 0, sizeof(p));
  p.c = *c;
  p.in = bind->in[c->in.a[MGD_IN_SLOT]];
  p.out = bind->out[c->out.a[MGD_OUT_SLOT]];
  p.in_set = bind->in_set_stride[c->in.a[MGD_IN_SLOT]];
  p.out_set = bind->out_set_stride[c->out.a[MGD_OUT_SLOT]];
  if (!p.in || !p.out || bind->num_sets <= 0) return set_error(MG_ERR_INVALID_ARGUMENT, "tile reduction: unbound tensor");
  // a tile's outputs go over `chunks` blocks of 256 threads, as many as keep the launch at a few waves
  long long const tiles = (long long)c->grid[0] * c->grid[1] * c->grid[2] * bind->num_sets;
  int chunks = (c->out_elements + 255) / 256;
  while (chunks > 1 && tiles * chunks > 148 * 8) chunks = (chunks + 1) / 2;
  p.c.chunks = chunks;
  if (tiles * chunks > 0x7fffffffLL) return set_error(MG_ERR_UNSUPPORTED, "too many blocks for one launch");
  unsigned const grid = (unsigned)(tiles * chunks);
  if (fingerprint_mode) tred::tile_reduce_kernel<2><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  else if (c->data_type == MG_DT_BFLOAT16) tred::tile_reduce_kernel<1><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  else tred::tile_reduce_kernel<0><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  return check_launch("tile_reduce_kernel");
}
}
