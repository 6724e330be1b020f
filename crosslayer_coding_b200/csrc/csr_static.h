// clt_build_csr_static - CSR construction for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference implementation (which is pure PyTorch and lets the
// caching allocator supply every temporary).  It exists for hosts that embed this library where device
// allocation is off the table: an inference server that has handed its whole memory budget to other
// components, a plugin running inside somebody else's allocator or sandbox, code on a latency-critical path
// where cudaMalloc's implicit device synchronisation is unacceptable.
//
// It does the same work as clt_build_csr (token-major and feature-major CSR views of the selected
// (token, column, value) entries), but the four scratch arrays that call needs from its caller - per-token and
// per-column counters plus their scatter cursors - live in one fixed array inside the library:
//
//     static __device__ __align__(256) int  csr_static_scratch[2 * (CLT_CSR_STATIC_MAX_TOKENS + CLT_CSR_STATIC_MAX_COLS)]
//
// about 8.9 MB, resident on every GPU that loads the library until the process exits.  Problem sizes above the
// two limits below are refused (return code -2 and a message on stderr); nothing is truncated silently.
//
// Things to know before calling it:
//   * The first call on each device looks up the device address of the scratch array (cudaGetSymbolAddress,
//     with that device current).  Make that first call outside of any CUDA stream capture.
//   * The call performs no cudaMalloc / cudaFree and uses no allocating library routine; it enqueues memsets
//     and kernels on `stream` and returns without synchronising.
//   * Every call on a device shares the one scratch array, and the array keeps whatever the previous call left
//     there; the counters are cleared at the start of each call.  Two calls whose work overlaps on the same GPU
//     (different streams, different threads) race on it - serialise them.
//   * Entries are range-checked on the device: an entry whose token is outside [0, num_tokens) or whose column is outside
//     [0, num_cols) (a stale entry count, a wrong col_pitch) is left out of both views; tok_off[num_tokens] and
//     feat_off[num_cols] then add up to less than the entry count, which is how a caller can notice.  Nothing is
//     written outside the scratch regions of this call or beyond `ent_cap` slots of the payload arrays.
//   * Inputs and outputs are the caller's: entries (ent_*), the control block `ctl` whose slot 3 holds the entry
//     count (as written by clt_batchtopk_select), the offset arrays tok_off[num_tokens + 1] and
//     feat_off[num_cols + 1], and the four CSR payload arrays of capacity `ent_cap`.
//
// Return codes: 0 ok; -1 bad argument (null pointer, non-positive size, col_pitch outside (0, 2^24));
// -2 size above CLT_CSR_STATIC_MAX_*; -3 the scratch address could not be obtained; -5 a launch failed.
#pragma once
#include <cuda_runtime.h>

#define CLT_CSR_STATIC_MAX_TOKENS 65536
#define CLT_CSR_STATIC_MAX_COLS 1048576

#ifdef __cplusplus
extern "C" {
#endif

int clt_build_csr_static(const int* ent_tok, const int* ent_col, const float* ent_val, long long ent_cap, const long long* ctl,
                         int num_tokens, int num_cols, int col_pitch, int* tok_off, int* feat_off, int* tcsr_col, float* tcsr_val,
                         int* fcsr_tok, float* fcsr_val, int sort_segments, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
