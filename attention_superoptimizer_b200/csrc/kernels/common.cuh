// Shared device/host helpers of the sm_100a kernels: finite-field constants and lookup tables,
// modular arithmetic, 16-bit float conversion, launch bookkeeping.
#pragma once
#include "mugraph.h"
#include "mugraph_device.h"
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace mgk {

constexpr uint32_t P = MG_FP_P, Q = MG_FP_Q, PQ = MG_FP_PQ;
constexpr uint32_t Q_MUL_P_MOD_1 = MG_FP_Q_MUL_P_MOD_1; // multiple of Q that is 1 mod P
constexpr uint32_t P_MUL_Q_MOD_1 = MG_FP_P_MUL_Q_MOD_1; // multiple of P that is 1 mod Q

// Lookup tables of the finite-field exp and div, evaluated at compile time:
//   e[i] = 3^i mod P for i < Q (3 has multiplicative order Q modulo P),
//   p[i] = inverse of i modulo P, q[i] = inverse of i modulo Q, with 0 (and 1) mapped to 1.
// The arena copies built by the device memory manager hold the same values.
struct FieldTables {
  uint16_t e[MG_FP_Q];
  uint16_t p[MG_FP_P];
  uint16_t q[MG_FP_Q];
  constexpr FieldTables() : e{}, p{}, q{} {
    e[0] = 1;
    for (int i = 1; i < MG_FP_Q; i++) e[i] = (uint16_t)((e[i - 1] * MG_FP_EXP_BASE) % MG_FP_P);
    for (int i = 0; i < MG_FP_P; i++) {
      p[i] = 1;
      for (int j = 1; j < MG_FP_P; j++)
        if ((i * j) % MG_FP_P == 1) p[i] = (uint16_t)j;
    }
    for (int i = 0; i < MG_FP_Q; i++) {
      q[i] = 1;
      for (int j = 1; j < MG_FP_Q; j++)
        if ((i * j) % MG_FP_Q == 1) q[i] = (uint16_t)j;
    }
  }
};
static __constant__ FieldTables c_tables = FieldTables();

// y = 3^(x mod Q) lifted to the ring Z_PQ with a zero mod-Q component
__device__ __forceinline__ uint32_t field_exp(uint32_t x) {
  return (c_tables.e[x % Q] * Q_MUL_P_MOD_1) % PQ;
}
// x / y through the two residue fields, recombined by the Chinese remainder theorem
__device__ __forceinline__ uint32_t field_div(uint32_t x, uint32_t y) {
  uint32_t z = (x % P) * c_tables.p[y % P] * Q_MUL_P_MOD_1 + (x % Q) * c_tables.q[y % Q] * P_MUL_Q_MOD_1;
  return z % PQ;
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- host-side bookkeeping (defined in runtime.cu) ------------------------------------------------
void count_launch();
int set_error(int code, char const *msg);
int check_launch(char const *kernel_name); // cudaGetLastError -> MG_* status
int32_t *device_error_word();              // 4-byte device status word, lazily allocated
int option(int key);                       // current value of a MGD_OPT_* switch (0 = automatic)

constexpr int kSmemLimit = 227 * 1024;

} // namespace mgk
