// kernel::KNOperator - a node of the kernel graph (reference: include/mirage/kernel/operator.h:26-57).
// `fingerprint()` evaluates the operator in the finite field on its tensors' fp_ptr buffers,
// `profile()` times the float kernel; both keep the reference's bool convention.
#pragma once
#include "mirage/kernel/device_tensor.h"
#include "mirage/profile_result.h"
#include <vector>

namespace mirage {
namespace kernel {

class KNOperator {
public:
  explicit KNOperator(mirage::type::KNOperatorType type);
  KNOperator(mirage::type::KNOperatorType type, DTensor const &in1);
  KNOperator(mirage::type::KNOperatorType type, DTensor const &in1, DTensor const &in2);
  KNOperator(mirage::type::KNOperatorType type, std::vector<DTensor> const &inputs);
  virtual ~KNOperator();
  virtual bool profile(ProfileResult &result) = 0;
  virtual bool fingerprint(void) = 0;
  // asynchronous launches on a stream (status code from mugraph.h); the bool API above wraps these
  virtual int launch_fingerprint(void *stream) = 0;
  virtual int launch_float(void *stream) = 0;
  mirage::type::KNOperatorType op_type;
  std::vector<DTensor> input_tensors;
  std::vector<DTensor> output_tensors;

protected:
  bool profile_with_events(ProfileResult &result, int warmup, int iters);
};

class KNInputOp : public KNOperator {
public:
  KNInputOp(std::vector<int> const &dims, mirage::type::DataType data_type, mirage::layout::DmemLayout layout);
  ~KNInputOp() override;
  bool profile(ProfileResult &result) override;
  bool fingerprint(void) override; // fills fp[i] = i % FP_PQ like the reference
  int launch_fingerprint(void *stream) override;
  int launch_float(void *stream) override;
  bool skip_fill = false; // set once the caller uploaded its own contents
};

class KNMatmulOp : public KNOperator {
public:
  KNMatmulOp(DTensor const &A, DTensor const &B);
  ~KNMatmulOp() override;
  bool profile(ProfileResult &result) override;
  bool fingerprint(void) override;
  int launch_fingerprint(void *stream) override;
  int launch_float(void *stream) override;
};

class KNElementUnaryOp : public KNOperator {
public:
  KNElementUnaryOp(DTensor const &A, mirage::type::KNOperatorType type);
  ~KNElementUnaryOp() override;
  bool profile(ProfileResult &result) override;
  bool fingerprint(void) override;
  int launch_fingerprint(void *stream) override;
  int launch_float(void *stream) override;
};

class KNElementBinaryOp : public KNOperator {
public:
  KNElementBinaryOp(DTensor const &A, DTensor const &B, mirage::type::KNOperatorType type);
  ~KNElementBinaryOp() override;
  bool profile(ProfileResult &result) override;
  bool fingerprint(void) override;
  int launch_fingerprint(void *stream) override;
  int launch_float(void *stream) override;
};

class KNReductionOp : public KNOperator {
public:
  KNReductionOp(DTensor const &A, int dim, int size);
  ~KNReductionOp() override;
  bool profile(ProfileResult &result) override;
  bool fingerprint(void) override;
  int launch_fingerprint(void *stream) override;
  int launch_float(void *stream) override;
  int reduction_dim_idx, reduction_dim_size;
};

} // namespace kernel
} // namespace mirage
