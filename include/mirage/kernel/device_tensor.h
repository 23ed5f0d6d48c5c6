// kernel::DTensor - descriptor of a tensor in the device arena
// (reference: include/mirage/kernel/device_tensor.h:31-124).  A POD copied by
// value; `data_ptr` holds the 16-bit float image, `fp_ptr` the uint16 fingerprints.
#pragma once
#include "mirage/layout.h"
#include "mirage/type.h"
#include <cstddef>
#include <functional>

#ifndef MAX_TENSOR_DIMS
#define MAX_TENSOR_DIMS 4
#endif

namespace mirage {
namespace kernel {

class KNOperator;

struct alignas(16) DTensor {
  DTensor();
  bool operator==(DTensor const &b) const;
  bool operator!=(DTensor const &b) const { return !(*this == b); }
  size_t num_elements() const {
    size_t n = 1;
    for (int i = 0; i < num_dims; i++) n *= (size_t)dim[i];
    return n;
  }
  size_t data_size() const { return num_elements() * mirage::type::get_datatype_size(data_type); }
  size_t fingerprint_size() const { return num_elements() * sizeof(mirage::type::FPType); }
  // device-side comparison of the two fingerprint buffers; one 4-byte flag comes back
  bool has_same_fingerprint(DTensor const &ref) const;

  mirage::type::DataType data_type;
  mirage::layout::DmemLayout layout;
  int num_dims;
  int dim[MAX_TENSOR_DIMS];
  size_t guid;
  KNOperator *owner_op;
  int owner_ts_idx;
  void *data_ptr;
  mirage::type::FPType *fp_ptr;
  static int next_guid;
};

} // namespace kernel
} // namespace mirage

namespace std {
template <> struct hash<mirage::kernel::DTensor> {
  size_t operator()(mirage::kernel::DTensor const &t) const;
};
} // namespace std
