// Split-KV attention kernels (placeholder translation unit while the kernels are brought up):
// every query reports "not supported", which makes the host keep such graphs on the interpreters.
#include "common.cuh"
using namespace mgk;
extern "C" {
int mgd_attn_split_supported(const mgd_attn_split *, int32_t) { return 0; }
int mgd_attn_merge_supported(const mgd_attn_merge *, int32_t) { return 0; }
int mgd_launch_attn_split_float(const mgd_attn_split *, const void *, const void *, const void *, void *, void *, void *) {
  return set_error(MG_ERR_UNSUPPORTED, "split-KV attention kernel not available");
}
int mgd_launch_attn_split_fingerprint(const mgd_attn_split *, const uint16_t *, const uint16_t *, const uint16_t *,
                                      uint16_t *, uint16_t *, void *) {
  return set_error(MG_ERR_UNSUPPORTED, "split-KV attention kernel not available");
}
int mgd_launch_attn_merge_float(const mgd_attn_merge *, const void *, const void *, void *, void *) {
  return set_error(MG_ERR_UNSUPPORTED, "attention merge kernel not available");
}
int mgd_launch_attn_merge_fingerprint(const mgd_attn_merge *, const uint16_t *, const uint16_t *, uint16_t *, void *) {
  return set_error(MG_ERR_UNSUPPORTED, "attention merge kernel not available");
}
}
