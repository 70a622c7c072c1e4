// Collectives as single kernels over symmetric (peer-mapped) buffers.
//
// Every rank launches the same kernel with the same grid.  Block b of a rank
// only ever synchronises with block b of the other ranks (comm_barrier), and
// data moves by plain 16-byte loads from / stores to the peers' mapped memory
// over NVLink.  There is no ring, no staging slot and no per-piece handshake
// (compare the reference's host-driven loop of D2D copies, events and
// `dst += src` launches: tandem/csrc/collectives.cpp:231-311, reduce.cu:23-102).
//
// Reduction order.  The element at flat index i belongs to chunk c of
// torch.tensor_split(numel, n) (or of the explicit sizes); its operands are
// folded in the order of ranks c+1, c+2, ..., c.  That is the association a
// ring reduce-scatter produces, so fp32 results are bit-identical to the CPU
// engine and to the reference on any group size, and identical on every rank.
// 16-bit types accumulate in fp32 and round once; EXACT=true instead rounds
// every partial sum to the dtype, as an element-wise add chain does.
//
// The gradient-averaging divide is applied to each operand as it is loaded.
#include "adam.cuh"
#include "common.cuh"

namespace {

// Per-rank pointers that are NOT symmetric (a rank's private input, output,
// gradient shard ...), indexed by blockIdx.y: entry 0 in a real run, one entry per
// rank when a single launch emulates all ranks.
struct Locals {
  char* p[TB_MAX_RANKS];
};

struct Bounds {
  long long off[TB_MAX_RANKS + 1];  // chunk c of the flat tensor is [off[c], off[c+1])
};

struct Chunking {
  long long base;  // numel / n
  long long rem;   // numel % n  (the first `rem` chunks are one longer)
};

__device__ __forceinline__ void chunk_range(const Chunking& k, int c, long long* lo, long long* hi) {
  long long extra = c < k.rem ? c : k.rem;
  *lo = c * k.base + extra;
  *hi = *lo + k.base + (c < k.rem ? 1 : 0);
}

__device__ __forceinline__ int chunk_of(const Chunking& k, long long i) {
  long long wide = k.rem * (k.base + 1);
  if (i < wide) return (int)(i / (k.base + 1));
  return (int)(k.rem + (i - wide) / (k.base > 0 ? k.base : 1));
}

// Element load that bypasses L1 (the data was written by another GPU).
template <typename T>
__device__ __forceinline__ float ld_elem_peer(const char* base, long long i);
template <>
__device__ __forceinline__ float ld_elem_peer<float>(const char* base, long long i) {
  return *reinterpret_cast<volatile const float*>(base + i * 4);
}
template <>
__device__ __forceinline__ float ld_elem_peer<__nv_bfloat16>(const char* base, long long i) {
  unsigned short b = *reinterpret_cast<volatile const unsigned short*>(base + i * 2);
  return __uint_as_float((unsigned)b << 16);
}
template <>
__device__ __forceinline__ float ld_elem_peer<__half>(const char* base, long long i) {
  unsigned short b = *reinterpret_cast<volatile const unsigned short*>(base + i * 2);
  return __half2float(__ushort_as_half(b));
}

// Folds the vectors x[0..n) IN THE ORDER GIVEN (x[0] first).
template <typename T, bool EXACT>
__device__ __forceinline__ uint4 fold_vec(const uint4 (&x)[TB_MAX_RANKS], int n, int smode, float sval) {
  constexpr int N = VecOf<T>::N;
  float acc[N], t[N];
  unpack<T>(x[0], acc);
#pragma unroll
  for (int e = 0; e < N; ++e) {
    acc[e] = scaled(acc[e], smode, sval);
    if (EXACT) acc[e] = round_via<T>(acc[e]);
  }
#pragma unroll
  for (int j = 1; j < TB_MAX_RANKS; ++j) {
    if (j < n) {
      unpack<T>(x[j], t);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        float u = scaled(t[e], smode, sval);
        if (EXACT) u = round_via<T>(u);
        acc[e] = __fadd_rn(acc[e], u);
        if (EXACT) acc[e] = round_via<T>(acc[e]);
      }
    }
  }
  return pack<T>(acc);
}

// Loads the operand vectors of chunk c at byte offset `off`, in fold order (ranks c+1, ..., c).
__device__ __forceinline__ void load_ordered(const PeerPtrs& buf, int n, int c, long long off, uint4 (&x)[TB_MAX_RANKS]) {
  int q = c;
#pragma unroll
  for (int j = 0; j < TB_MAX_RANKS; ++j) {
    if (j < n) {
      q = q + 1 == n ? 0 : q + 1;
      x[j] = ld_vec_peer(buf.p[q] + off);
    }
  }
}

template <typename T, bool EXACT>
__device__ __forceinline__ T fold_one(const PeerPtrs& buf, int n, int c, long long i, int smode, float sval) {
  int q = c + 1 == n ? 0 : c + 1;
  float acc = scaled(ld_elem_peer<T>(buf.p[q], i), smode, sval);
  if (EXACT) acc = round_via<T>(acc);
  for (int j = 2; j <= n; ++j) {
    q = q + 1 == n ? 0 : q + 1;
    float t = scaled(ld_elem_peer<T>(buf.p[q], i), smode, sval);
    if (EXACT) t = round_via<T>(t);
    acc = __fadd_rn(acc, t);
    if (EXACT) acc = round_via<T>(acc);
  }
  return from_f<T>(acc);
}

// Vector body shared by the two-shot all-reduce and reduce-scatter: folds `nvec` 16-byte vectors of chunk
// `rank` starting at byte offset `off0`.  NR is the group size when it is 2, 4 or 8 (loops unroll exactly and
// eight operand vectors are in flight per thread), 0 otherwise (predicated over TB_MAX_RANKS).
template <typename T, bool EXACT, int NR, typename Sink>
__device__ __forceinline__ void fold_vectors(const PeerPtrs& buf, int n_runtime, int rank, long long off0, long long nvec, int smode,
                                             float sval, long long tid, long long nth, Sink&& sink) {
  constexpr int U = NR ? 8 / NR : 1;
  const int n = NR ? NR : n_runtime;
  const char* ord[TB_MAX_RANKS];  // operands in fold order: ranks rank+1, ..., rank
  {
    int q = rank;
#pragma unroll
    for (int j = 0; j < TB_MAX_RANKS; ++j) {
      q = q + 1 >= n ? 0 : q + 1;
      ord[j] = j < n ? buf.p[q] : nullptr;
    }
  }
  for (long long v = tid; v < nvec; v += nth * U) {
    uint4 x[U][TB_MAX_RANKS];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long vv = v + u * nth;
      if (vv < nvec) {
#pragma unroll
        for (int j = 0; j < TB_MAX_RANKS; ++j)
          if (j < n) x[u][j] = ld_vec_peer(ord[j] + off0 + vv * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long vv = v + u * nth;
      if (vv < nvec) sink(off0 + vv * 16, fold_vec<T, EXACT>(x[u], n, smode, sval));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Local copy helper: dst[i] = scale(src[i]) for i in [0, numel), all blocks of this rank.
template <typename T>
__device__ __forceinline__ void local_copy(char* dst, const char* src, long long numel, int smode, float sval) {
  constexpr int N = VecOf<T>::N;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  const bool aligned = (((uintptr_t)dst | (uintptr_t)src) & 15) == 0;
  long long nvec = aligned ? numel / N : 0;
  for (long long v = tid; v < nvec; v += nth) {
    uint4 x = ld_vec_peer(src + v * 16);
    if (smode != SCALE_NONE) {
      float f[N];
      unpack<T>(x, f);
#pragma unroll
      for (int e = 0; e < N; ++e) f[e] = scaled(f[e], smode, sval);
      x = pack<T>(f);
    }
    st_vec(dst + v * 16, x);
  }
  for (long long i = nvec * N + tid; i < numel; i += nth) {
    float f = to_f<T>(reinterpret_cast<const T*>(src)[i]);
    reinterpret_cast<T*>(dst)[i] = from_f<T>(scaled(f, smode, sval));
  }
}

// ---------------------------------------------------------------------------------------------
// Two-shot all-reduce, in place on buf[rank] (and therefore on every rank's buf).
//   [copy local_in -> buf]  barrier  reduce own chunk from all peers, store it to all peers
//   barrier  [copy buf -> local_out]
template <typename T, bool EXACT, int NR>
__global__ void __launch_bounds__(TB_COMM_THREADS, 6)
k_allreduce_twoshot(CommCtx c, PeerPtrs buf, Locals lin, Locals lout, long long numel, int smode, float sval) {
  __shared__ int sh[2];
  if (threadIdx.x == 0) sh[1] = 0;
  const int n = c.n, rank = comm_rank(c);
  constexpr int N = VecOf<T>::N;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  const char* local_in = lin.p[blockIdx.y];
  char* local_out = lout.p[blockIdx.y];
  if (local_in != nullptr) {
    local_copy<T>(buf.p[rank], local_in, numel, smode, sval);
    smode = SCALE_NONE;  // operands are already divided
  }
  comm_barrier(c, sh);
  if (!sh[1]) {
    Chunking k{numel / n, numel % n};
    long long lo, hi;
    chunk_range(k, rank, &lo, &hi);
    // scalar head up to the first 16-byte boundary, vector body, scalar tail
    long long head = (long long)((16 - (((uintptr_t)buf.p[rank] + lo * sizeof(T)) & 15)) & 15) / (long long)sizeof(T);
    if (head > hi - lo) head = hi - lo;
    long long nvec = (hi - lo - head) / N;
    long long body = lo + head;
    fold_vectors<T, EXACT, NR>(buf, n, rank, body * (long long)sizeof(T), nvec, smode, sval, tid, nth, [&](long long off, const uint4& r) {
#pragma unroll
      for (int q = 0; q < TB_MAX_RANKS; ++q)
        if (q < (NR ? NR : n)) st_vec(buf.p[q] + off, r);
    });
    const long long ntail = (hi - lo) - nvec * N;  // head + tail elements
    for (long long t = tid; t < ntail; t += nth) {
      long long i = t < head ? lo + t : body + nvec * N + (t - head);
      T r = fold_one<T, EXACT>(buf, n, rank, i, smode, sval);
      for (int q = 0; q < n; ++q) reinterpret_cast<T*>(buf.p[q])[i] = r;
    }
  }
  comm_barrier(c, sh);
  if (local_out != nullptr && !sh[1]) local_copy<T>(local_out, buf.p[rank], numel, SCALE_NONE, 1.f);
}

// ---------------------------------------------------------------------------------------------
// One-shot all-reduce for small messages: every rank reads all n buffers.
//   in place:            barrier  load+fold (registers)  barrier  store to buf[rank]
//   through a scratch:   copy local_in -> buf  barrier  load+fold  store to local_out
// The second form needs no trailing barrier because the caller alternates between
// two scratch halves: a rank can only be one collective behind its peers.
#define TB_ONESHOT_UNROLL 4
template <typename T, bool EXACT>
__global__ void __launch_bounds__(TB_COMM_THREADS, 6)
k_allreduce_oneshot(CommCtx c, PeerPtrs buf, Locals lin, Locals lout, long long numel, int smode, float sval) {
  __shared__ int sh[2];
  if (threadIdx.x == 0) sh[1] = 0;
  const int n = c.n, rank = comm_rank(c);
  constexpr int N = VecOf<T>::N;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  const char* local_in = lin.p[blockIdx.y];
  char* local_out = lout.p[blockIdx.y];
  if (local_in != nullptr) {
    local_copy<T>(buf.p[rank], local_in, numel, smode, sval);
    smode = SCALE_NONE;
  }
  comm_barrier(c, sh);
  Chunking k{numel / n, numel % n};
  const long long nvec = numel / N;
  uint4 out[TB_ONESHOT_UNROLL];
  T tail_val = from_f<T>(0.f);
  const long long tail_i = nvec * N + tid;  // at most N-1 tail elements, one per thread
  if (!sh[1]) {
#pragma unroll
    for (int u = 0; u < TB_ONESHOT_UNROLL; ++u) {
      const long long v = tid + u * nth;
      if (v < nvec) {
        const int c0 = chunk_of(k, v * N), c1 = chunk_of(k, v * N + N - 1);
        if (c0 == c1) {
          uint4 x[TB_MAX_RANKS];
          load_ordered(buf, n, c0, v * 16, x);
          out[u] = fold_vec<T, EXACT>(x, n, smode, sval);
        } else {  // the vector straddles a chunk boundary: fold element by element
          T* o = reinterpret_cast<T*>(&out[u]);
          for (int e = 0; e < N; ++e) o[e] = fold_one<T, EXACT>(buf, n, chunk_of(k, v * N + e), v * N + e, smode, sval);
        }
      }
    }
    if (tail_i < numel) tail_val = fold_one<T, EXACT>(buf, n, chunk_of(k, tail_i), tail_i, smode, sval);
  }
  char* dst = local_out != nullptr ? local_out : buf.p[rank];
  if (local_out == nullptr) comm_barrier(c, sh);  // everyone has read this rank's operands
  if (!sh[1]) {
    const bool aligned = ((uintptr_t)dst & 15) == 0;
#pragma unroll
    for (int u = 0; u < TB_ONESHOT_UNROLL; ++u) {
      const long long v = tid + u * nth;
      if (v < nvec) {
        if (aligned) {
          st_vec(dst + v * 16, out[u]);
        } else {
          const T* o = reinterpret_cast<const T*>(&out[u]);
          for (int e = 0; e < N; ++e) reinterpret_cast<T*>(dst)[v * N + e] = o[e];
        }
      }
    }
    if (tail_i < numel) reinterpret_cast<T*>(dst)[tail_i] = tail_val;
  }
}

// ---------------------------------------------------------------------------------------------
// Reduce-scatter: this rank's chunk [lo, hi) of every peer's buffer is folded and
//   (a) stored to buf[rank][lo:hi) (the returned view), and optionally
//   (b) accumulated into acc_out[i - lo] (a gradient shard), or
//   (c) consumed by a fused AdamW update of param/exp_avg/exp_avg_sq (+ bf16 shadow).
// A trailing barrier lets the caller reuse the staging buffer as soon as the
// kernel has finished on its own rank.
struct AdamSet {
  AdamArgs a[TB_MAX_RANKS];
};

__device__ __forceinline__ void adam_elem(const AdamArgs& a, long long j, float g) {
  float p = a.param[j], m = a.exp_avg[j], v = a.exp_avg_sq[j];
  adam_update(p, m, v, g, a.s);
  a.param[j] = p;
  a.exp_avg[j] = m;
  a.exp_avg_sq[j] = v;
  if (a.shadow != nullptr) a.shadow[j] = __float2bfloat16_rn(p);
}

// The same for N consecutive elements (N = 4 or 8: one 16-byte gradient vector).  Where the optimizer state is 16-byte
// aligned at j0 it moves as float4 vectors (and the shadow as one 8- or 16-byte store) instead of 4-byte accesses that
// use an eighth of every sector they touch; same arithmetic, same results.
template <int N>
__device__ __forceinline__ void adam_vec(const AdamArgs& a, long long j0, const float* g) {
  const uintptr_t state = (uintptr_t)(a.param + j0) | (uintptr_t)(a.exp_avg + j0) | (uintptr_t)(a.exp_avg_sq + j0);
  const bool aligned = (state & 15) == 0 && (a.shadow == nullptr || ((uintptr_t)(a.shadow + j0) & (N * 2 - 1)) == 0);
  if (!aligned) {
#pragma unroll
    for (int e = 0; e < N; ++e) adam_elem(a, j0 + e, g[e]);
    return;
  }
  float p[N], m[N], v[N];
#pragma unroll
  for (int q = 0; q < N / 4; ++q) {
    *reinterpret_cast<float4*>(p + 4 * q) = *reinterpret_cast<const float4*>(a.param + j0 + 4 * q);
    *reinterpret_cast<float4*>(m + 4 * q) = *reinterpret_cast<const float4*>(a.exp_avg + j0 + 4 * q);
    *reinterpret_cast<float4*>(v + 4 * q) = *reinterpret_cast<const float4*>(a.exp_avg_sq + j0 + 4 * q);
  }
#pragma unroll
  for (int e = 0; e < N; ++e) adam_update(p[e], m[e], v[e], g[e], a.s);
#pragma unroll
  for (int q = 0; q < N / 4; ++q) {
    *reinterpret_cast<float4*>(a.param + j0 + 4 * q) = *reinterpret_cast<const float4*>(p + 4 * q);
    *reinterpret_cast<float4*>(a.exp_avg + j0 + 4 * q) = *reinterpret_cast<const float4*>(m + 4 * q);
    *reinterpret_cast<float4*>(a.exp_avg_sq + j0 + 4 * q) = *reinterpret_cast<const float4*>(v + 4 * q);
  }
  if (a.shadow != nullptr) {
    __nv_bfloat162 h[N / 2];
#pragma unroll
    for (int e = 0; e < N / 2; ++e) h[e] = __floats2bfloat162_rn(p[2 * e], p[2 * e + 1]);
    if (N == 8) *reinterpret_cast<uint4*>(a.shadow + j0) = *reinterpret_cast<const uint4*>(h);
    else *reinterpret_cast<uint2*>(a.shadow + j0) = *reinterpret_cast<const uint2*>(h);
  }
}

template <typename T, bool EXACT, int EPI, int NR>  // EPI 0: store only, 1: += into acc_out, 2: fused AdamW (T must be float)
__global__ void __launch_bounds__(TB_COMM_THREADS, 6)
k_reduce_scatter(CommCtx c, PeerPtrs buf, Locals lin, long long numel, Bounds bounds, int smode, float sval, Locals acc,
                 AdamSet adams) {
  __shared__ int sh[2];
  if (threadIdx.x == 0) sh[1] = 0;
  const int n = c.n, rank = comm_rank(c);
  constexpr int N = VecOf<T>::N;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  const char* local_in = lin.p[blockIdx.y];
  T* acc_out = reinterpret_cast<T*>(acc.p[blockIdx.y]);
  AdamArgs adam = adams.a[blockIdx.y];
  if (EPI == 2 && adam.s_dev != nullptr) adam.s = *adam.s_dev;
  const long long lo = bounds.off[rank], hi = bounds.off[rank + 1];
  if (local_in != nullptr) {
    local_copy<T>(buf.p[rank], local_in, numel, smode, sval);
    smode = SCALE_NONE;
  }
  comm_barrier(c, sh);
  if (!sh[1]) {
    long long head = (long long)((16 - (((uintptr_t)buf.p[rank] + lo * sizeof(T)) & 15)) & 15) / (long long)sizeof(T);
    if (head > hi - lo) head = hi - lo;
    const long long nvec = (hi - lo - head) / N;
    const long long body = lo + head;
    fold_vectors<T, EXACT, NR>(buf, n, rank, body * (long long)sizeof(T), nvec, smode, sval, tid, nth, [&](long long off, const uint4& r) {
      st_vec(buf.p[rank] + off, r);
      if (EPI != 0) {
        const long long i0 = off / (long long)sizeof(T);
        const T* e = reinterpret_cast<const T*>(&r);
        if (EPI == 1) {
#pragma unroll
          for (int j = 0; j < N; ++j) acc_out[i0 - lo + j] = from_f<T>(__fadd_rn(to_f<T>(acc_out[i0 - lo + j]), to_f<T>(e[j])));
        }
        if (EPI == 2) {
          float gv[N];
#pragma unroll
          for (int j = 0; j < N; ++j) gv[j] = to_f<T>(e[j]);
          adam_vec<N>(adam, i0 - lo, gv);
        }
      }
    });
    const long long ntail = (hi - lo) - nvec * N;
    for (long long t = tid; t < ntail; t += nth) {
      long long i = t < head ? lo + t : body + nvec * N + (t - head);
      T r = fold_one<T, EXACT>(buf, n, rank, i, smode, sval);
      reinterpret_cast<T*>(buf.p[rank])[i] = r;
      if (EPI == 1) acc_out[i - lo] = from_f<T>(__fadd_rn(to_f<T>(acc_out[i - lo]), to_f<T>(r)));
      if (EPI == 2) adam_elem(adam, i - lo, to_f<T>(r));
    }
  }
  comm_barrier(c, sh);
}

// ---------------------------------------------------------------------------------------------
// Gather by pulling: dst (local) receives src.p[q][src_off[q] : +len[q]) at dst_off[q] for
// every q.  sync == 1: a barrier precedes the reads (the sources were written
// by this step's kernels) and one follows them (the sources may be overwritten next).
// sync == 2: no handshake, only a system-scope fence before the reads -- for sources that change only
// between barriers issued elsewhere (parameter shards between optimizer steps); the fence is what makes
// the loads observe the peers' latest stores.  sync == 0: neither.
struct GatherPlan {
  long long src_off[TB_MAX_RANKS];  // bytes
  long long dst_off[TB_MAX_RANKS];  // bytes
  long long len[TB_MAX_RANKS];      // bytes
};

__global__ void __launch_bounds__(TB_COMM_THREADS, 6)
k_gather_pull(CommCtx c, PeerPtrs src, Locals dsts, GatherPlan plan, Locals stage, int sync) {
  __shared__ int sh[2];
  if (threadIdx.x == 0) sh[1] = 0;
  const int n = c.n, rank = comm_rank(c);
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  char* dst = dsts.p[blockIdx.y];
  const char* stage_in = stage.p[blockIdx.y];
  if (stage_in != nullptr) {  // publish this rank's piece through its symmetric staging area
    const long long stage_bytes = plan.len[rank];
    char* s = src.p[rank] + plan.src_off[rank];
    const bool al = (((uintptr_t)s | (uintptr_t)stage_in) & 15) == 0;
    long long nv = al ? stage_bytes / 16 : 0;
    for (long long v = tid; v < nv; v += nth) st_vec(s + v * 16, ld_vec(stage_in + v * 16));
    for (long long i = nv * 16 + tid; i < stage_bytes; i += nth) s[i] = stage_in[i];
  }
  if (sync == 1) comm_barrier(c, sh);
  if (sync == 2) __threadfence_system();
  if (!sh[1]) {
    for (int j = 0; j < n; ++j) {
      const int q = (rank + j) % n;  // start at home, then walk the peers: spreads load over the switch
      const char* s = src.p[q] + plan.src_off[q];
      char* d = dst + plan.dst_off[q];
      const long long len = plan.len[q];
      if (len <= 0 || s == d) continue;
      const bool al = (((uintptr_t)s | (uintptr_t)d) & 15) == 0;
      const long long nv = al ? len / 16 : 0;
      for (long long v = tid; v < nv; v += nth * 8) {  // eight independent 16-byte loads in flight per thread
        uint4 x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v + u * nth < nv) x[u] = ld_vec_peer(s + (v + u * nth) * 16);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v + u * nth < nv) st_vec(d + (v + u * nth) * 16, x[u]);
      }
      for (long long i = nv * 16 + tid; i < len; i += nth) d[i] = *reinterpret_cast<volatile const char*>(s + i);
    }
  }
  if (sync == 1) comm_barrier(c, sh);
}

// ---------------------------------------------------------------------------------------------
// NVLS all-reduce: the buffer is also mapped through an NVSwitch multicast address.  Each rank owns a
// 16-byte-aligned slice; multimem.ld_reduce returns the SUM OVER ALL RANKS of a 16-byte vector (the
// switch adds the ranks' copies), the mean's factor is applied, and multimem.st writes the result into
// every rank's copy at once.  Half the NVLink bytes of the two-shot kernel and no per-peer loads; the
// switch's order of additions is not specified, so results are not tied to the ring order.
template <typename T>
__device__ __forceinline__ uint4 multimem_ld_reduce(const char* mc);
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce<float>(const char* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce<__nv_bfloat16>(const char* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}

__device__ __forceinline__ void multimem_st(char* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(TB_COMM_THREADS, 6)
k_allreduce_nvls(CommCtx c, char* mc, long long nvec, int smode, float sval) {
  __shared__ int sh[2];
  if (threadIdx.x == 0) sh[1] = 0;
  const int n = c.n, rank = comm_rank(c);
  constexpr int N = VecOf<T>::N;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  comm_barrier(c, sh);
  if (!sh[1]) {
    const long long lo = nvec * rank / n, hi = nvec * (rank + 1) / n;  // this rank's slice, in vectors
    for (long long v = lo + tid; v < hi; v += nth * 4) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * nth < hi) x[u] = multimem_ld_reduce<T>(mc + (v + u * nth) * 16);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (v + u * nth < hi) {
          if (smode != SCALE_NONE) {
            float f[N];
            unpack<T>(x[u], f);
#pragma unroll
            for (int e = 0; e < N; ++e) f[e] = scaled(f[e], smode, sval);
            x[u] = pack<T>(f);
          }
          multimem_st(mc + (v + u * nth) * 16, x[u]);
        }
      }
    }
  }
  comm_barrier(c, sh);
}

// NVLS all-gather: each rank streams ITS chunk of the buffer to the multicast address, and the switch
// writes it into every rank's copy (its own included).  A rank sends len bytes once instead of
// serving n - 1 peers' loads.  off and len are multiples of 16.
__global__ void __launch_bounds__(TB_COMM_THREADS, 6)
k_allgather_nvls(CommCtx c, const char* local, char* mc, long long off, long long len) {
  __shared__ int sh[2];
  if (threadIdx.x == 0) sh[1] = 0;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  comm_barrier(c, sh);  // every rank's buffer may be written from here on
  if (!sh[1]) {
    const long long nvec = len / 16;
    for (long long v = tid; v < nvec; v += nth * 4) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * nth < nvec) x[u] = ld_vec(local + off + (v + u * nth) * 16);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * nth < nvec) multimem_st(mc + off + (v + u * nth) * 16, x[u]);
    }
  }
  comm_barrier(c, sh);
}

// NVLS reduce-scatter: this rank's chunk [lo, hi) (bytes, multiples of 16) of the buffer is read through the multicast
// address with multimem.ld_reduce -- the switch returns the sum over all ranks' copies -- scaled, stored into this
// rank's own copy and handed to the same epilogues as k_reduce_scatter (accumulate into a gradient shard, or the fused
// AdamW update).  Each rank pulls bytes/n through the switch instead of (n-1)/n * bytes/n from every peer separately.
template <typename T, int EPI>
__global__ void __launch_bounds__(TB_COMM_THREADS, 6)
k_reduce_scatter_nvls(CommCtx c, const char* mc, char* local, long long lo, long long hi, int smode, float sval, char* acc, AdamSet adams) {
  __shared__ int sh[2];
  if (threadIdx.x == 0) sh[1] = 0;
  constexpr int N = VecOf<T>::N;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  T* acc_out = reinterpret_cast<T*>(acc);
  AdamArgs adam = adams.a[0];
  if (EPI == 2 && adam.s_dev != nullptr) adam.s = *adam.s_dev;
  comm_barrier(c, sh);
  if (!sh[1]) {
    const long long nvec = (hi - lo) / 16;
    for (long long v = tid; v < nvec; v += nth * 4) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * nth < nvec) x[u] = multimem_ld_reduce<T>(mc + lo + (v + u * nth) * 16);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long vv = v + u * nth;
        if (vv < nvec) {
          float f[N];
          unpack<T>(x[u], f);
          if (smode != SCALE_NONE) {
#pragma unroll
            for (int e = 0; e < N; ++e) f[e] = scaled(f[e], smode, sval);
            x[u] = pack<T>(f);
          }
          st_vec(local + lo + vv * 16, x[u]);
          if (EPI != 0) {
            const T* r = reinterpret_cast<const T*>(&x[u]);  // the value as stored (rounded to T), like the peer-to-peer kernel
            if (EPI == 1) {
#pragma unroll
              for (int e = 0; e < N; ++e) acc_out[vv * N + e] = from_f<T>(__fadd_rn(to_f<T>(acc_out[vv * N + e]), to_f<T>(r[e])));
            }
            if (EPI == 2) {
              float gv[N];
#pragma unroll
              for (int e = 0; e < N; ++e) gv[e] = to_f<T>(r[e]);
              adam_vec<N>(adam, vv * N, gv);
            }
          }
        }
      }
    }
  }
  comm_barrier(c, sh);  // every rank has read every copy: the buffers may be refilled
}

// NVLS broadcast: the root streams its buffer to the multicast address and the switch writes every rank's copy.
__global__ void __launch_bounds__(TB_COMM_THREADS, 6)
k_broadcast_nvls(CommCtx c, const char* local, char* mc, long long bytes, int root) {
  __shared__ int sh[2];
  if (threadIdx.x == 0) sh[1] = 0;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  comm_barrier(c, sh);  // every rank's buffer may be written from here on
  if (!sh[1] && comm_rank(c) == root) {
    const long long nvec = bytes / 16;
    for (long long v = tid; v < nvec; v += nth * 4) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * nth < nvec) x[u] = ld_vec(local + (v + u * nth) * 16);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * nth < nvec) multimem_st(mc + (v + u * nth) * 16, x[u]);
    }
  }
  comm_barrier(c, sh);
}

// A barrier and nothing else (one block per rank).
__global__ void k_barrier(CommCtx c) {
  __shared__ int sh[2];
  if (threadIdx.x == 0) sh[1] = 0;
  comm_barrier(c, sh);
}

// Generic element types (double, integers): one-shot over scalars, sum only.
template <typename T>
__global__ void __launch_bounds__(TB_COMM_THREADS, 6)
k_allreduce_generic(CommCtx c, PeerPtrs buf, Locals lin, Locals lout, long long numel, int divide, Bounds bounds,
                    int scatter_only) {
  __shared__ int sh[2];
  if (threadIdx.x == 0) sh[1] = 0;
  const int n = c.n, rank = comm_rank(c);
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  const char* local_in = lin.p[blockIdx.y];
  char* local_out = lout.p[blockIdx.y];
  if (local_in != nullptr)
    for (long long i = tid; i < numel; i += nth) reinterpret_cast<T*>(buf.p[rank])[i] = reinterpret_cast<const T*>(local_in)[i];
  comm_barrier(c, sh);
  Chunking k{numel / n, numel % n};
  if (!sh[1]) {
    long long lo = bounds.off[rank], hi = bounds.off[rank + 1];
    if (!scatter_only) chunk_range(k, rank, &lo, &hi);
    for (long long i = lo + tid; i < hi; i += nth) {
      int q = rank + 1 == n ? 0 : rank + 1;
      T acc = *reinterpret_cast<volatile const T*>(buf.p[q] + i * sizeof(T));
      if (divide) acc = acc / (T)n;
      for (int j = 2; j <= n; ++j) {
        q = q + 1 == n ? 0 : q + 1;
        T t = *reinterpret_cast<volatile const T*>(buf.p[q] + i * sizeof(T));
        if (divide) t = t / (T)n;
        acc = acc + t;
      }
      if (scatter_only) {
        reinterpret_cast<T*>(buf.p[rank])[i] = acc;
      } else {
        for (int p = 0; p < n; ++p) reinterpret_cast<T*>(buf.p[p])[i] = acc;
      }
    }
  }
  comm_barrier(c, sh);
  if (local_out != nullptr && !sh[1])
    for (long long i = tid; i < numel; i += nth) reinterpret_cast<T*>(local_out)[i] = reinterpret_cast<volatile const T*>(buf.p[rank])[i];
}

}  // namespace

// ================================================================================================
// Host API (C symbols; called through ctypes).  A Comm describes the group as seen
// from this process.  emulated != 0: all `n` ranks are local allocations on one
// GPU and each call is one cooperative launch with gridDim.y == n (tests only).
struct TbComm {
  CommCtx ctx;
  int emulated;
  int rank;
  int max_blocks;
};

enum { TB_F32 = 0, TB_F64 = 1, TB_BF16 = 2, TB_F16 = 3, TB_I64 = 4, TB_I32 = 5, TB_I16 = 6, TB_I8 = 7, TB_U8 = 8 };
enum { TB_ALGO_AUTO = 0, TB_ALGO_ONESHOT = 1, TB_ALGO_TWOSHOT = 2 };

static int elem_size(int dtype) {
  switch (dtype) {
    case TB_F32: case TB_I32: return 4;
    case TB_F64: case TB_I64: return 8;
    case TB_BF16: case TB_F16: case TB_I16: return 2;
    default: return 1;
  }
}

// Averaging multiplies each operand by float(1/n) before the sum.  That is what
// ATen's CUDA `div_(n)` does (a host scalar divisor becomes a reciprocal multiply),
// so results equal a `flat.div_(n)` followed by ordered adds on the GPU; for a
// power-of-two group it also equals true division.
static void scale_mode(int n, int average, int* smode, float* sval) {
  if (!average || n == 1) {
    *smode = SCALE_NONE;
    *sval = 1.f;
  } else {
    *smode = SCALE_MUL;
    *sval = 1.f / (float)n;
  }
}

extern "C" void tb_note_launch(int n);

template <typename T>
struct Same {
  using type = T;
};

template <typename... Args>
static cudaError_t launch(const TbComm* comm, void (*kernel)(Args...), int blocks, cudaStream_t stream,
                          typename Same<Args>::type... args) {
  dim3 grid(blocks, comm->emulated ? comm->ctx.n : 1);
  void* params[] = {(void*)&args...};
  tb_note_launch(1);
  if (comm->emulated) return cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3(TB_COMM_THREADS), params, 0, stream);
  return cudaLaunchKernel((const void*)kernel, grid, dim3(TB_COMM_THREADS), params, 0, stream);
}

static int blocks_for(const TbComm* comm, long long bytes, long long per_block) {
  long long b = (bytes + per_block - 1) / per_block;
  if (b < 1) b = 1;
  int cap = comm->max_blocks;
  if (comm->emulated) {
    int fit = 128 / comm->ctx.n;  // one cooperative launch must be fully resident
    if (cap > fit) cap = fit;
  }
  return (int)(b > cap ? cap : b);
}

static int locals_of(const TbComm* c) { return c->emulated ? c->ctx.n : 1; }

static Locals locals(const TbComm* c, void* const* ptrs) {
  Locals l{};
  if (ptrs != nullptr)
    for (int i = 0; i < locals_of(c); ++i) l.p[i] = (char*)ptrs[i];
  return l;
}

static PeerPtrs peers(const TbComm* c, void* const* ptrs) {
  PeerPtrs b{};
  for (int q = 0; q < c->ctx.n; ++q) b.p[q] = (char*)ptrs[q];
  return b;
}

extern "C" {

// flags[q] / epochs[q]: rank q's signal pad (TB_MAX_BLOCKS * TB_MAX_RANKS words, zeroed) as mapped
// in this process, and barrier counters (TB_MAX_BLOCKS words, zeroed; only this rank's are touched
// unless emulated).  status: five host-mapped words, zeroed.
TbComm* tb_comm_create(int n, int rank, int emulated, void* const* flags, void* const* epochs, void* status, double timeout_s,
                       int max_blocks) {
  if (n < 1 || n > TB_MAX_RANKS) return nullptr;
  TbComm* c = new TbComm();
  c->ctx.n = n;
  c->ctx.rank0 = emulated ? 0 : rank;
  for (int i = 0; i < TB_MAX_RANKS; ++i) {
    c->ctx.flags[i] = i < n ? (uint32_t*)flags[i] : nullptr;
    c->ctx.epoch[i] = i < n ? (uint32_t*)epochs[i] : nullptr;
  }
  c->ctx.status = (uint32_t*)status;
  c->ctx.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  c->emulated = emulated;
  c->rank = rank;
  c->max_blocks = max_blocks < 1 ? 1 : (max_blocks > TB_MAX_BLOCKS ? TB_MAX_BLOCKS : max_blocks);
  return c;
}

void tb_comm_destroy(TbComm* c) { delete c; }

void tb_comm_set_timeout(TbComm* c, double timeout_s) { c->ctx.timeout_ns = (unsigned long long)(timeout_s * 1e9); }

void tb_comm_set_max_blocks(TbComm* c, int max_blocks) {
  c->max_blocks = max_blocks < 1 ? 1 : (max_blocks > TB_MAX_BLOCKS ? TB_MAX_BLOCKS : max_blocks);
}

int tb_barrier(TbComm* c, cudaStream_t stream) {
  dim3 grid(1, c->emulated ? c->ctx.n : 1);
  void* params[] = {(void*)&c->ctx};
  tb_note_launch(1);
  if (c->emulated) return (int)cudaLaunchCooperativeKernel((const void*)k_barrier, grid, dim3(32), params, 0, stream);
  return (int)cudaLaunchKernel((const void*)k_barrier, grid, dim3(32), params, 0, stream);
}

// bufs[q]: rank q's copy of the symmetric buffer (same offset in every rank's heap).
// local_in / local_out: optional arrays (one entry; n entries when emulated) of private tensors
// to stage through the buffer: in -> buf before the reduction, buf -> out after it.  Only valid
// for single-block launches: a block synchronises with the peers' block of the same index, not with
// their whole grid, so with several blocks a peer could read a part of the buffer that another block
// has not copied in yet.  Multi-block callers stage with separate copies before and after the call.
int tb_all_reduce(TbComm* c, void* const* bufs, void* const* local_in, void* const* local_out, long long numel, int dtype,
                  int average, int exact, int algo, cudaStream_t stream) {
  if (numel <= 0) return 0;
  PeerPtrs buf = peers(c, bufs);
  Locals in = locals(c, local_in), out = locals(c, local_out);
  int smode;
  float sval;
  scale_mode(c->ctx.n, average, &smode, &sval);
  const long long bytes = numel * elem_size(dtype);
  if (dtype != TB_F32 && dtype != TB_BF16 && dtype != TB_F16) {
    int blocks = blocks_for(c, bytes, 64 << 10);
    Bounds none{};
#define GEN(T) return (int)launch(c, k_allreduce_generic<T>, blocks, stream, c->ctx, buf, in, out, numel, average, none, 0)
    switch (dtype) {
      case TB_F64: GEN(double);
      case TB_I64: GEN(long long);
      case TB_I32: GEN(int);
      case TB_I16: GEN(short);
      case TB_I8: GEN(signed char);
      default: GEN(unsigned char);
    }
#undef GEN
  }
  const long long per_pass = (long long)TB_COMM_THREADS * 16 * TB_ONESHOT_UNROLL;
  int cap = c->max_blocks;
  if (c->emulated && cap > 128 / c->ctx.n) cap = 128 / c->ctx.n;
  const bool base_aligned = (((uintptr_t)bufs[c->emulated ? 0 : c->rank]) & 15) == 0;
  const bool oneshot_ok = bytes <= cap * per_pass && base_aligned;
  if (algo == TB_ALGO_AUTO) algo = (bytes <= (256 << 10) && oneshot_ok) ? TB_ALGO_ONESHOT : TB_ALGO_TWOSHOT;
  if (algo == TB_ALGO_ONESHOT) {
    if (!oneshot_ok) return -2;  // too large for one pass, or the buffer is not 16-byte aligned
    int blocks = blocks_for(c, bytes, per_pass);
#define ONE(T, E) return (int)launch(c, k_allreduce_oneshot<T, E>, blocks, stream, c->ctx, buf, in, out, numel, smode, sval)
    if (dtype == TB_F32) ONE(float, false);
    if (dtype == TB_BF16) {
      if (exact) ONE(__nv_bfloat16, true);
      ONE(__nv_bfloat16, false);
    }
    if (exact) ONE(__half, true);
    ONE(__half, false);
#undef ONE
  }
  int blocks = blocks_for(c, bytes / c->ctx.n, (long long)TB_COMM_THREADS * 16 * 8);
  const int nr = c->ctx.n;
#define TWO(T, E)                                                                                                                    \
  do {                                                                                                                               \
    if (nr == 2) return (int)launch(c, k_allreduce_twoshot<T, E, 2>, blocks, stream, c->ctx, buf, in, out, numel, smode, sval);      \
    if (nr == 4) return (int)launch(c, k_allreduce_twoshot<T, E, 4>, blocks, stream, c->ctx, buf, in, out, numel, smode, sval);      \
    if (nr == 8) return (int)launch(c, k_allreduce_twoshot<T, E, 8>, blocks, stream, c->ctx, buf, in, out, numel, smode, sval);      \
    return (int)launch(c, k_allreduce_twoshot<T, E, 0>, blocks, stream, c->ctx, buf, in, out, numel, smode, sval);                   \
  } while (0)
  if (dtype == TB_F32) TWO(float, false);
  if (dtype == TB_BF16) {
    if (exact) TWO(__nv_bfloat16, true);
    TWO(__nv_bfloat16, false);
  }
  if (exact) TWO(__half, true);
  TWO(__half, false);
#undef TWO
}

// In-switch all-reduce of a buffer that every rank has bound to one multicast object: mc is the multicast
// address of the buffer (the same offset in every rank's copy).  numel * element size must be a multiple of
// 16 and mc 16-byte aligned; dtype fp32 or bf16.  Not available when emulating ranks on one GPU.
int tb_all_reduce_nvls(TbComm* c, void* mc, long long numel, int dtype, int average, cudaStream_t stream) {
  if (numel <= 0) return 0;
  if (c->emulated || (dtype != TB_F32 && dtype != TB_BF16)) return -4;
  const long long bytes = numel * elem_size(dtype);
  if ((bytes & 15) || ((uintptr_t)mc & 15)) return -4;
  int smode;
  float sval;
  scale_mode(c->ctx.n, average, &smode, &sval);
  int blocks = blocks_for(c, bytes / c->ctx.n, (long long)TB_COMM_THREADS * 16 * 4);
  if (dtype == TB_F32) return (int)launch(c, k_allreduce_nvls<float>, blocks, stream, c->ctx, (char*)mc, bytes / 16, smode, sval);
  return (int)launch(c, k_allreduce_nvls<__nv_bfloat16>, blocks, stream, c->ctx, (char*)mc, bytes / 16, smode, sval);
}

// In-switch all-gather, in place: rank r's chunk is bytes [off, off + len) of the buffer whose local address is
// `local` and whose multicast address is `mc`; grid_bytes (the largest chunk) fixes the grid on every rank.
int tb_all_gather_nvls(TbComm* c, const void* local, void* mc, long long off, long long len, long long grid_bytes, cudaStream_t stream) {
  if (c->emulated || (off & 15) || (len & 15) || (((uintptr_t)mc | (uintptr_t)local) & 15)) return -4;
  int blocks = blocks_for(c, grid_bytes, (long long)TB_COMM_THREADS * 16 * 4);
  return (int)launch(c, k_allgather_nvls, blocks, stream, c->ctx, (const char*)local, (char*)mc, off, len);
}

// Folds chunk r = [offs[r], offs[r+1]) of every rank's buffer into rank r's buffer.
// acc_out (array like local_in; entries may be null): also acc_out[i - lo] += result.
// adam (array of AdamArgs like local_in, fp32 only): fused AdamW on {param, exp_avg, exp_avg_sq}[i - lo]
// with the result as the gradient.
int tb_reduce_scatter(TbComm* c, void* const* bufs, void* const* local_in, long long numel, const long long* offs, int dtype,
                      int average, int exact, void* const* acc_out, const AdamArgs* adam, cudaStream_t stream) {
  if (numel <= 0) return 0;
  PeerPtrs buf = peers(c, bufs);
  Locals in = locals(c, local_in), acc = locals(c, acc_out);
  Bounds bounds{};
  long long most = 0;
  for (int q = 0; q <= c->ctx.n; ++q) bounds.off[q] = offs[q];
  for (int q = 0; q < c->ctx.n; ++q) most = offs[q + 1] - offs[q] > most ? offs[q + 1] - offs[q] : most;
  AdamSet adams{};
  if (adam != nullptr)
    for (int i = 0; i < locals_of(c); ++i) adams.a[i] = adam[i];
  int smode;
  float sval;
  scale_mode(c->ctx.n, average, &smode, &sval);
  int blocks = blocks_for(c, most * elem_size(dtype), (long long)TB_COMM_THREADS * 16 * 8);
  const int nr = c->ctx.n;
  if (dtype != TB_F32 && dtype != TB_BF16 && dtype != TB_F16) {
    if (acc_out != nullptr || adam != nullptr) return -3;
    Locals none{};
#define GEN(T) return (int)launch(c, k_allreduce_generic<T>, blocks, stream, c->ctx, buf, in, none, numel, average, bounds, 1)
    switch (dtype) {
      case TB_F64: GEN(double);
      case TB_I64: GEN(long long);
      case TB_I32: GEN(int);
      case TB_I16: GEN(short);
      case TB_I8: GEN(signed char);
      default: GEN(unsigned char);
    }
#undef GEN
  }
#define RS(T, E, EPI)                                                                                                                      \
  do {                                                                                                                                 \
    if (nr == 2) return (int)launch(c, k_reduce_scatter<T, E, EPI, 2>, blocks, stream, c->ctx, buf, in, numel, bounds, smode, sval, acc, adams); \
    if (nr == 4) return (int)launch(c, k_reduce_scatter<T, E, EPI, 4>, blocks, stream, c->ctx, buf, in, numel, bounds, smode, sval, acc, adams); \
    if (nr == 8) return (int)launch(c, k_reduce_scatter<T, E, EPI, 8>, blocks, stream, c->ctx, buf, in, numel, bounds, smode, sval, acc, adams); \
    return (int)launch(c, k_reduce_scatter<T, E, EPI, 0>, blocks, stream, c->ctx, buf, in, numel, bounds, smode, sval, acc, adams);    \
  } while (0)
  if (dtype == TB_F32) {
    if (adam != nullptr) RS(float, false, 2);
    if (acc_out != nullptr) RS(float, false, 1);
    RS(float, false, 0);
  }
  if (dtype == TB_BF16 && adam != nullptr) RS(__nv_bfloat16, false, 2);  // bf16 gradients into fp32 master weights
  if (adam != nullptr) return -3;
  if (dtype == TB_BF16) {
    if (acc_out != nullptr) {
      if (exact) RS(__nv_bfloat16, true, 1);
      RS(__nv_bfloat16, false, 1);
    }
    if (exact) RS(__nv_bfloat16, true, 0);
    RS(__nv_bfloat16, false, 0);
  }
  if (acc_out != nullptr) {
    if (exact) RS(__half, true, 1);
    RS(__half, false, 1);
  }
  if (exact) RS(__half, true, 0);
  RS(__half, false, 0);
#undef RS
}

// In-switch reduce-scatter: mc / local are the multicast and local addresses of the symmetric buffer; chunk r is
// elements [offs[r], offs[r+1]).  Every chunk boundary must fall on a 16-byte boundary (the caller checks and otherwise
// uses tb_reduce_scatter); dtype fp32 or bf16.  acc_out / adam as in tb_reduce_scatter (single entries).
int tb_reduce_scatter_nvls(TbComm* c, const void* mc, void* local, long long numel, const long long* offs, int dtype, int average,
                           void* acc_out, const AdamArgs* adam, cudaStream_t stream) {
  if (numel <= 0) return 0;
  if (c->emulated || (dtype != TB_F32 && dtype != TB_BF16)) return -4;
  const int esz = elem_size(dtype);
  long long most = 0;
  for (int q = 0; q <= c->ctx.n; ++q)
    if ((offs[q] * esz) & 15) return -4;
  for (int q = 0; q < c->ctx.n; ++q) most = offs[q + 1] - offs[q] > most ? offs[q + 1] - offs[q] : most;
  if (((uintptr_t)mc | (uintptr_t)local) & 15) return -4;
  int smode;
  float sval;
  scale_mode(c->ctx.n, average, &smode, &sval);
  AdamSet adams{};
  if (adam != nullptr) adams.a[0] = *adam;
  const long long lo = offs[c->rank] * esz, hi = offs[c->rank + 1] * esz;
  const int blocks = blocks_for(c, most * esz, (long long)TB_COMM_THREADS * 16 * 4);
#define RSN(T, EPI) return (int)launch(c, k_reduce_scatter_nvls<T, EPI>, blocks, stream, c->ctx, (const char*)mc, (char*)local, lo, hi, smode, sval, (char*)acc_out, adams)
  if (dtype == TB_F32) {
    if (adam != nullptr) RSN(float, 2);
    if (acc_out != nullptr) RSN(float, 1);
    RSN(float, 0);
  }
  if (adam != nullptr) RSN(__nv_bfloat16, 2);
  if (acc_out != nullptr) RSN(__nv_bfloat16, 1);
  RSN(__nv_bfloat16, 0);
#undef RSN
}

// In-switch broadcast of `bytes` (a multiple of 16) from rank `root`.
int tb_broadcast_nvls(TbComm* c, const void* local, void* mc, long long bytes, int root, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  if (c->emulated || (bytes & 15) || (((uintptr_t)mc | (uintptr_t)local) & 15)) return -4;
  const int blocks = blocks_for(c, bytes, (long long)TB_COMM_THREADS * 16 * 4);
  return (int)launch(c, k_broadcast_nvls, blocks, stream, c->ctx, (const char*)local, (char*)mc, bytes, root);
}

// Every rank's dst receives, for every rank q, len[q] bytes from srcs[q] + src_off[q] at dst + dst_off[q].
// stage_in (array like dsts, entries may be null): first copy len[rank] bytes from it to srcs[rank] + src_off[rank].
// grid_bytes: what the grid is sized for.  Every rank must pass the same value (ranks synchronise block by
// block, so their grids must match even when their plans differ); 0 means "the largest len[q]".
int tb_gather_pull(TbComm* c, void* const* srcs, void* const* dsts, const long long* src_off, const long long* dst_off,
                   const long long* len, void* const* stage_in, int sync, long long grid_bytes, cudaStream_t stream) {
  PeerPtrs src = peers(c, srcs);
  GatherPlan plan{};
  long long most = 0;
  for (int q = 0; q < c->ctx.n; ++q) {
    plan.src_off[q] = src_off[q];
    plan.dst_off[q] = dst_off[q];
    plan.len[q] = len[q];
    if (len[q] > most) most = len[q];
  }
  int blocks = blocks_for(c, grid_bytes > 0 ? grid_bytes : most, (long long)TB_COMM_THREADS * 16 * 8);
  return (int)launch(c, k_gather_pull, blocks, stream, c->ctx, src, locals(c, dsts), plan, locals(c, stage_in), sync);
}

}  // extern "C"
