// Symmetric-memory plumbing: device allocations that other processes map
// through CUDA IPC, a host-mapped status block, and last-error text.
// The reference shares per-peer slot arrays the same way
// (tandem/csrc/cuda_links.cpp:43-118); here whole heaps are shared once and
// kernels address peers' copies directly.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

static thread_local char g_last_error[256] = "";

static int fail(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
  return (int)e;
}

static long long g_launches = 0;

extern "C" {

// Every kernel launcher in this library reports its launches here, so a caller
// can count how many of these kernels ran in a region of its program.
void tb_note_launch(int n) { g_launches += n; }

long long tb_launch_count(int reset) {
  long long v = g_launches;
  if (reset) g_launches = 0;
  return v;
}

const char* tb_last_error() { return g_last_error; }

const char* tb_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

int tb_malloc(void** out, size_t bytes) {
  int rc = fail(cudaMalloc(out, bytes), "cudaMalloc");
  if (rc == 0) rc = fail(cudaMemset(*out, 0, bytes), "cudaMemset");
  return rc;
}

int tb_free(void* p) { return fail(cudaFree(p), "cudaFree"); }

// 64-byte handle that another process on this machine can open.
int tb_ipc_export(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  int rc = fail(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
  if (rc == 0) memcpy(handle64, &h, sizeof(h));
  return rc;
}

int tb_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return fail(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

int tb_ipc_close(void* p) { return fail(cudaIpcCloseMemHandle(p), "cudaIpcCloseMemHandle"); }

// Peer access for ranks that live in ONE process (single-process tests on several GPUs).
int tb_enable_peer(int peer_device) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return fail(e, "cudaDeviceEnablePeerAccess");
}

int tb_can_access_peer(int device, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, device, peer) != cudaSuccess) return 0;
  return ok;
}

// Pinned host words the GPU can write (the kernels' error report).
int tb_status_alloc(void** host, void** dev, size_t bytes) {
  int rc = fail(cudaHostAlloc(host, bytes, cudaHostAllocMapped), "cudaHostAlloc");
  if (rc) return rc;
  memset(*host, 0, bytes);
  return fail(cudaHostGetDevicePointer(dev, *host, 0), "cudaHostGetDevicePointer");
}

int tb_status_free(void* host) { return fail(cudaFreeHost(host), "cudaFreeHost"); }

int tb_memset_async(void* p, int value, size_t bytes, cudaStream_t stream) {
  return fail(cudaMemsetAsync(p, value, bytes, stream), "cudaMemsetAsync");
}

int tb_memcpy_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  return fail(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, stream), "cudaMemcpyAsync");
}

int tb_device_sync() { return fail(cudaDeviceSynchronize(), "cudaDeviceSynchronize"); }

}  // extern "C"
