// Column sums without any allocation by the caller or by this library.
//
// This entry point has no counterpart in the reference; it exists for callers of
// libtb200_cuda.so that are not in a position to allocate device memory when they need
// a bias gradient: a plugin that runs inside someone else's memory budget and was handed
// exactly its inputs and outputs, a host thread that must not trigger the implicit
// device-wide synchronisation cudaMalloc / cudaFree can cause while other streams are
// busy, or code that runs after the framework's allocator has been torn down.
// tb_col_sum (layers.cu) needs a caller-provided fp32 scratch of 32 * N floats; this
// variant keeps that scratch in a fixed array inside the library instead.
//
//   out[c] = sum over r < M of x[r * ld + c]      x: bf16 [M, ld], out: bf16 [N]
//
// Limits and rules:
//   * N <= TB_COLSUM_NOALLOC_MAX_N.  Larger N is refused with TB_NOALLOC_TOO_WIDE and
//     nothing is launched; tb_noalloc_last_error() then says why.
//   * M <= 0 (no rows) is the empty sum: out[0 .. N) is set to zero (a cudaMemsetAsync on `stream`,
//     which allocates nothing), as tb_col_sum does.
//   * The scratch is a file-scope __device__ array of 32 * TB_COLSUM_NOALLOC_MAX_N floats
//     (1 MiB).  Every GPU on which this library is loaded holds it until the process exits.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress) with that device current.  Make that first call outside any
//     stream capture.  Later calls on the same device only launch kernels.
//   * The call allocates and frees nothing: no cudaMalloc, no cudaFree, no library routine
//     that allocates.
//   * All calls on a device share the one array, and it keeps whatever the previous call
//     left there.  The kernels write every partial sum before they read it, so nothing has
//     to be cleared between calls; but two calls that overlap on the GPU (different streams,
//     no ordering between them) race on the array and produce garbage.  Order them.
//   * tb_noalloc_last_error() returns the text of the most recent refusal in this process.  There is one
//     buffer per process and it is not synchronised: do not rely on it when several host threads call in
//     at once (the return codes are always reliable).  The per-device address cache is filled the same way;
//     two threads racing on a device's first call both look the address up and store the same value.
#pragma once
#include <cuda_runtime.h>

#define TB_COLSUM_NOALLOC_MAX_N 8192
#define TB_NOALLOC_TOO_WIDE (-30)
#define TB_NOALLOC_SETUP_FAILED (-31)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, a negative TB_NOALLOC_* code, or a positive cudaError_t from the launch.
int tb_col_sum_noalloc(const void* x_bf16, int M, int N, int ld, void* out_bf16, cudaStream_t stream);

// Why the last call that returned a TB_NOALLOC_* code was refused ("" if none was).
const char* tb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
