// Shared device helpers for the communication kernels: system-scope flag
// signalling between GPUs, bounded waits, 16-byte vector arithmetic.
//
// Every wait in this library is bounded: a block that does not see its peers'
// flag within `timeout_ns` writes {code, rank, peer, epoch, block} to a
// host-mapped status block, marks itself failed, skips the rest of its work and
// returns normally.  Nothing traps, asserts or spins without a limit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TB_MAX_RANKS 8
#define TB_MAX_BLOCKS 128
#define TB_COMM_THREADS 128

// Launch shape of the communication kernels: many small blocks.  128 threads at no more than 85 registers
// each (launch bounds of 6 blocks per SM) let a block share an SM with a resident GEMM CTA (320 threads x
// 168 registers, ~225 KB of shared memory), so a collective overlaps backward without waiting for whole
// SMs to drain; latency over NVLink is covered by each thread keeping eight independent 16-byte loads in
// flight.
//
// Everything a communication kernel needs to know about the group.  In a real
// multi-GPU run gridDim.y == 1 and this GPU is `rank0`.  For single-GPU tests of
// the multi-rank logic all ranks' buffers live on one device and ONE cooperative
// launch covers them: blockIdx.y is the rank, so blocks that wait on one another
// are co-resident by construction.
struct CommCtx {
  int n;
  int rank0;
  uint32_t* flags[TB_MAX_RANKS];  // rank p's signal pad as mapped on this GPU: [TB_MAX_BLOCKS][TB_MAX_RANKS]
  uint32_t* epoch[TB_MAX_RANKS];  // rank p's private barrier counters: [TB_MAX_BLOCKS]
  uint32_t* status;               // host-mapped: code, rank, peer, epoch, block
  unsigned long long timeout_ns;
};

struct PeerPtrs {
  char* p[TB_MAX_RANKS];
};

enum { TB_OK = 0, TB_TIMEOUT = 1 };

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ int comm_rank(const CommCtx& c) { return c.rank0 + blockIdx.y; }

// Spins until *flag has reached `want` (wrap-safe), at most timeout_ns.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, unsigned long long timeout_ns) {
  unsigned long long start = 0;
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_sys(flag) - want) < 0) {
    if ((++spins & 0xff) == 0) {
      unsigned long long now = global_ns();
      if (start == 0) start = now;
      else if (now - start > timeout_ns) return false;
    }
  }
  return true;
}

// Block-level barrier across ranks: block b of every rank meets block b of
// every other rank.  Writes made by this block before the call are visible to
// the peers' block b after it returns there (release / acquire at system
// scope, made cumulative over the block by the bar.sync before the store).
// sh[0]: scratch for the epoch, sh[1]: sticky failure flag (must start at 0).
__device__ __forceinline__ void comm_barrier(const CommCtx& c, int* sh) {
  const int rank = comm_rank(c);
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t e = c.epoch[rank][blockIdx.x] + 1;
    c.epoch[rank][blockIdx.x] = e;
    sh[0] = (int)e;
  }
  __syncthreads();
  const uint32_t e = (uint32_t)sh[0];
  if (threadIdx.x < c.n && !sh[1]) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(c.flags[p] + blockIdx.x * TB_MAX_RANKS + rank, e);
    if (!wait_flag(c.flags[rank] + blockIdx.x * TB_MAX_RANKS + p, e, c.timeout_ns)) {
      if (atomicCAS(c.status, TB_OK, TB_TIMEOUT) == TB_OK) {
        c.status[1] = rank;
        c.status[2] = p;
        c.status[3] = e;
        c.status[4] = blockIdx.x;
        __threadfence_system();
      }
      sh[1] = 1;
    }
  }
  __syncthreads();
}

// ---------------------------------------------------------------- 16-byte vectors
template <typename T>
struct VecOf {
  static constexpr int N = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__device__ __forceinline__ void unpack(const uint4& v, float* f) {
  const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < VecOf<T>::N; ++i) f[i] = to_f<T>(e[i]);
}

template <typename T>
__device__ __forceinline__ uint4 pack(const float* f) {
  uint4 v;
  T* e = reinterpret_cast<T*>(&v);
#pragma unroll
  for (int i = 0; i < VecOf<T>::N; ++i) e[i] = from_f<T>(f[i]);
  return v;
}

// Rounds through T (a no-op for float): the "every partial sum is rounded to
// the tensor's dtype" behaviour of an element-wise add on 16-bit tensors.
template <typename T>
__device__ __forceinline__ float round_via(float v) { return to_f<T>(from_f<T>(v)); }

// Gradient averaging divides each operand before the sum.  For a power-of-two
// group the reciprocal multiply is exact; otherwise divide (round to nearest).
enum { SCALE_NONE = 0, SCALE_MUL = 1, SCALE_DIV = 2 };
__device__ __forceinline__ float scaled(float x, int mode, float s) {
  return mode == SCALE_NONE ? x : (mode == SCALE_MUL ? __fmul_rn(x, s) : __fdiv_rn(x, s));
}

__device__ __forceinline__ uint4 ld_vec(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st_vec(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

// Peer data changes between kernels without this SM's L1 knowing: read it
// with a volatile (L1-bypassing) load.
__device__ __forceinline__ uint4 ld_vec_peer(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
