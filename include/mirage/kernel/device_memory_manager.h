// kernel::DeviceMemoryManager - the device arena and the finite-field lookup tables
// (reference: include/mirage/kernel/device_memory_manager.h:28-53,
// src/kernel/device_memory_manager.cu:26-145).  One cudaMalloc, bump allocation with LIFO
// release (frees must mirror allocations), tables at the arena base.  Differences from the
// reference: allocations are 256-byte aligned (TMA descriptors and 128-bit accesses), the
// arena size and device are configurable before first use, no cuBLAS handle, and exhaustion
// is reported instead of asserted.  A negative device number creates a planning-only manager
// (addresses but no memory) so that host logic can run where there is no GPU.
#pragma once
#include "mirage/kernel/device_tensor.h"
#include <cstddef>
#include <sys/types.h>
#include <utility>
#include <vector>

namespace mirage {
namespace kernel {

class DeviceMemoryManager {
public:
  static DeviceMemoryManager *singleton;
  static DeviceMemoryManager *get_instance();
  // configure the singleton before its first use; returns an MG_* status
  static int create(int device, size_t arena_bytes, char const **error);
  static void destroy();

  bool allocate(DTensor &tensor, bool allocate_fingerprint = true);
  bool free(DTensor &tensor);
  bool can_allocate(size_t data_bytes, size_t fp_bytes) const;
  // raw LIFO scratch for launch workspaces
  void *allocate_raw(size_t bytes);
  bool free_raw(void *ptr);

  char *base_ptr;
  off_t offset;
  size_t total_size;
  std::vector<std::pair<void *, size_t>> allocated_tensors;
  mirage::type::FPType *exp_lookup_table;
  mirage::type::FPType *div_p_lookup_table;
  mirage::type::FPType *div_q_lookup_table;
  int device;
  size_t max_smem;     // budget handed to new threadblock graphs
  int specialise;      // 0 = generic interpreters only, 1 = pattern-specialised kernels, 2 = also fuse a
                       // split-KV attention operator with the merge operator that consumes it (default)
  int launch_policy;   // 0 = size launches for the latency of one call, 1 = for the throughput of many calls in flight
  int *flag_word;      // 4-byte device scratch for comparisons
  bool dry;            // planning-only: no device memory behind the arena, launches refused

private:
  DeviceMemoryManager(int device, size_t arena_bytes);
  ~DeviceMemoryManager();
  bool ok_;
};

} // namespace kernel
} // namespace mirage
