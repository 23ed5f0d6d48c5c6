// threadblock::STensor - a tile in the shared-memory plan of a threadblock graph
// (reference: include/mirage/threadblock/smem_tensor.h:32-167).  `smem_offset`
// is a byte offset in a plan that counts 2 bytes per 16-bit element; the
// kernels map it onto their own staging (fp32 tiles, TMA-swizzled stages, TMEM).
#pragma once
#include "mirage/layout.h"
#include "mirage/type.h"
#include <cstddef>
#include <functional>

#ifndef MAX_TENSOR_DIMS
#define MAX_TENSOR_DIMS 4
#endif

namespace mirage {
namespace threadblock {

class TBOperator;

struct alignas(16) STensor {
  STensor();
  bool operator==(STensor const &b) const;
  bool operator!=(STensor const &b) const { return !(*this == b); }
  size_t num_elements() const {
    size_t n = 1;
    for (int i = 0; i < num_dims; i++) n *= (size_t)dim[i];
    return n;
  }
  size_t size() const; // bytes in the plan

  mirage::type::DataType data_type;
  mirage::layout::SmemLayout layout;
  int num_dims;
  int dim[MAX_TENSOR_DIMS];
  int guid;
  TBOperator *owner_op;
  int owner_ts_idx;
  int smem_offset;
  static int next_guid;
};

} // namespace threadblock
} // namespace mirage

namespace std {
template <> struct hash<mirage::threadblock::STensor> {
  size_t operator()(mirage::threadblock::STensor const &t) const;
};
} // namespace std
