// Thread-local error message shared by the host library and the C ABI.
#pragma once
#include <string>
namespace mg {
void set_error(std::string const &msg);
char const *last_error();
// wraps a cudaError_t-returning call: on failure records the message and returns MG_ERR_CUDA
int cuda_status(int cuda_error, char const *what);
// Stream bookkeeping of the early input loads (kn_graph.cc): work the library cannot see into was enqueued on
// `stream`, so the next split-KV launch there must not read its inputs before the stream's previous kernel is done.
void stream_wrote_anything(void *stream);
void forget_streams();
} // namespace mg
#define MG_CUDA_TRY(expr)                                  \
  do {                                                     \
    int mg_st_ = mg::cuda_status((int)(expr), #expr);      \
    if (mg_st_ != 0) return mg_st_;                        \
  } while (0)
