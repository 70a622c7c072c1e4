// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = A . B (+ epilogue), fp32 accumulation in TMEM.
//
// Structure (one persistent CTA per SM, 320 threads, no cluster, no TMA multicast):
//   warp 0      TMA producer: cp.async.bulk.tensor.2d loads A and B tiles (128B swizzle) into a
//               3- to 6-stage shared-memory ring, signalling `full[s]` by transaction bytes.
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma.cta_group::1.kind::f16
//               (128 x BN x 16 per instruction, 4 per stage), releases stages with
//               tcgen05.commit -> `empty[s]`, and hands a finished accumulator to the epilogue
//               with tcgen05.commit -> `acc_full[b]`.  TMEM holds two accumulators (2 x BN
//               columns), so the next tile's MMAs overlap this tile's epilogue.
//   warps 2-9   epilogue: tcgen05.ld 32 lanes x 32 columns at a time (the next load in flight while
//               one chunk is processed), then bias / GELU / residual / dGELU / accumulate in
//               registers and 16-byte stores.
//
// Operand layouts.  Each operand is either K-major (the reduction dimension is contiguous in
// global memory) or MN-major (the other dimension is).  That covers all three GEMMs of a linear
// layer without transposing anything in memory:
//   forward   Y[M,N]  = X[M,K] . W[N,K]^T          A K-major,  B K-major
//   dX        dX[M,K] = dY[M,N] . W[N,K]            A K-major,  B MN-major   (reduction over N)
//   dW        dW[N,K] = dY[M,N]^T . X[M,K]          A MN-major, B MN-major   (reduction over M)
// MN-major tiles are loaded as 64-element-wide (128-byte) column strips so the same 128B
// swizzle applies; the shared-memory descriptors carry the strip stride (LBO) and the 8-row
// group stride (SBO).
//
// Every mbarrier wait is bounded; a wait that runs out sets a host-visible error word and the CTA
// winds down (frees its TMEM, returns).  The reference has no GEMM of its own: its Linear layers
// call cuBLAS through torch (tandem/model.py:36-37,53-54,75).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "tcgen05.cuh"

namespace {

constexpr int BK = 64;
constexpr int SMEM_BUDGET = 192 * 1024;   // operand ring
constexpr int EPI_STAGING = 8 * 4096;     // per epilogue warp: a 32-row x 128-byte block for coalescing its stores

enum EpilogueFlags {
  EPI_BIAS = 1,        // + bias[col]
  EPI_GELU = 2,        // out = gelu(v); with aux_out: also write v (pre-activation) there
  EPI_RESIDUAL = 4,    // + aux_in[row, col]
  EPI_DGELU = 8,       // out = v * gelu'(aux_in[row, col])
  EPI_ACCUMULATE = 16, // out += v  (gradient accumulation)
  EPI_OUT_F32 = 32,    // out is fp32 (else bf16)
  EPI_DISCARD = 64,    // measurement aid: drain the accumulator but compute and store nothing
  EPI_NO_STORE = 128,  // measurement aid: everything except the final global stores
  EPI_LOAD_ONLY = 256, // measurement aid: read the accumulator from TMEM and do nothing with it
};

struct GemmArgs {
  int M, N, K;
  int ldc;            // leading dimension of out / aux (elements)
  int flags;
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux_in;   // residual or pre-activation, [M, ldc]
  __nv_bfloat16* aux_out;        // pre-activation out for EPI_GELU, [M, ldc]
  int* error;                    // host-mapped; set to 1 when a wait runs out
};

// All-gather fused into the GEMM (B operand = a weight whose flat bytes are sharded over the ranks).
// Two extra warps per CTA pull the weight, chunk by chunk, from the owners' shard memory (plain 16-byte
// loads over NVLink from peer pointers) into this GPU's buffer and publish one flag per chunk; the TMA
// producer waits for the flags that cover a tile's weight panel before it loads it -- from local memory,
// never from the peer, and without multicast.  Transfer and math overlap panel by panel inside ONE
// kernel, launched cooperatively so that every CTA (hence every chunk's fetcher) is resident.
struct GatherArgs {
  const char* shard[8];   // shard[q]: rank q's shard as mapped here; its byte 0 is byte shard_lo[q] of the unit's flat buffer
  long long shard_lo[8];  // byte ranges of the shards within the unit's flat buffer
  long long shard_hi[8];
  char* full;             // this GPU's copy of the unit's flat buffer; the weight occupies [w_off, w_off + N*K*2)
  long long w_off, w_bytes;  // w_bytes: everything fetched = the weight plus tail_bytes
  long long tail_bytes;   // bytes right behind the weight that are fetched with it (the layer's bias)
  uint32_t* ready;        // one word per chunk of the weight; chunk c is complete once ready[c] == epoch
  uint32_t epoch;
  int n;                  // ranks
  int chunk_bytes;
  int n_start;            // the n-panel this rank visits first (the one its own shard feeds)
};

using namespace tc;

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait for chunk flags [c_lo, c_hi] to reach `epoch`.
__device__ __forceinline__ bool wait_chunks(const uint32_t* ready, int c_lo, int c_hi, uint32_t epoch, int* error) {
  const long long start = clock64();
  for (int c = c_lo; c <= c_hi; ++c) {
    while (ld_acquire_gpu(ready + c) != epoch) {
      if (clock64() - start > (1ll << WAIT_LIMIT_CYCLES_SHIFT)) {
        *error = 1;
        __threadfence_system();
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ float gelu_exact(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752440f)); }

__device__ __forceinline__ float gelu_grad(float x) {
  const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752440f));
  const float pdf = 0.39894228040143267794f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}

// ------------------------------------------------------------------------------------------ kernel
// One 32-column chunk of one accumulator row: the general path (tile edges, padded rows, any flags).
__device__ __forceinline__ void epilogue_chunk_generic(const uint32_t (&raw)[32], int row, int col0, const GemmArgs& g, bool out_f32) {
  if (row < g.M && col0 < g.N) {
    const size_t base = (size_t)row * g.ldc + col0;
#pragma unroll
    for (int v8 = 0; v8 < 4; ++v8) {  // 8 columns at a time
      const int col = col0 + v8 * 8;
      if (col >= g.N) break;
      float x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(raw[v8 * 8 + j]);
      if (g.flags & EPI_BIAS) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (col + j < g.N) x[j] += __bfloat162float(g.bias[col + j]);
      }
      const bool full8 = col + 8 <= g.ldc;  // the padded row has room for a whole vector
      if (g.flags & (EPI_RESIDUAL | EPI_DGELU)) {
        __nv_bfloat16 aux[8];
        if (full8) {
          *reinterpret_cast<uint4*>(aux) = *reinterpret_cast<const uint4*>(g.aux_in + base + v8 * 8);
        } else {
          for (int j = 0; j < 8; ++j) aux[j] = col + j < g.N ? g.aux_in[base + v8 * 8 + j] : __float2bfloat16(0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float a = __bfloat162float(aux[j]);
          x[j] = (g.flags & EPI_RESIDUAL) ? x[j] + a : x[j] * gelu_grad(a);
        }
      }
      if (g.flags & EPI_GELU) {
        if (g.aux_out != nullptr) {
          __nv_bfloat16 pre[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) pre[j] = __float2bfloat16_rn(x[j]);
          if (full8) {
            *reinterpret_cast<uint4*>(g.aux_out + base + v8 * 8) = *reinterpret_cast<const uint4*>(pre);
          } else {
            for (int j = 0; j < 8; ++j)
              if (col + j < g.N) g.aux_out[base + v8 * 8 + j] = pre[j];
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = gelu_exact(x[j]);
      }
      if (out_f32) {
        float* o = reinterpret_cast<float*>(g.out) + base + v8 * 8;
        if (full8) {
          float4 lo = make_float4(x[0], x[1], x[2], x[3]), hi = make_float4(x[4], x[5], x[6], x[7]);
          if (g.flags & EPI_ACCUMULATE) {
            const float4 a = *reinterpret_cast<const float4*>(o), b = *reinterpret_cast<const float4*>(o + 4);
            lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
            hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
          }
          *reinterpret_cast<float4*>(o) = lo;
          *reinterpret_cast<float4*>(o + 4) = hi;
        } else {
          for (int j = 0; j < 8; ++j)
            if (col + j < g.N) o[j] = (g.flags & EPI_ACCUMULATE) ? o[j] + x[j] : x[j];
        }
      } else {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(g.out) + base + v8 * 8;
        __nv_bfloat16 y[8];
        if (g.flags & EPI_ACCUMULATE) {
          if (full8) {
            *reinterpret_cast<uint4*>(y) = *reinterpret_cast<const uint4*>(o);
          } else {
            for (int j = 0; j < 8; ++j) y[j] = col + j < g.N ? o[j] : __float2bfloat16(0.f);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] += __bfloat162float(y[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = __float2bfloat16_rn(x[j]);
        if (full8) {
          *reinterpret_cast<uint4*>(o) = *reinterpret_cast<const uint4*>(y);
        } else {
          for (int j = 0; j < 8; ++j)
            if (col + j < g.N) o[j] = y[j];
        }
      }
    }
  }
}

// The same for a chunk that lies wholly inside the matrix with 16-byte-aligned rows: no per-element
// bounds checks, bias fetched as four 16-byte vectors.
__device__ __forceinline__ void epilogue_chunk_interior(const uint32_t (&raw)[32], int row, int col0, const GemmArgs& g, bool out_f32,
                                                        bool bias_vec) {
  const size_t base = (size_t)row * g.ldc + col0;
#pragma unroll
  for (int v8 = 0; v8 < 4; ++v8) {
    float x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(raw[v8 * 8 + j]);
    if (g.flags & EPI_BIAS) {
      __nv_bfloat16 bv[8];
      if (bias_vec) {
        *reinterpret_cast<uint4*>(bv) = __ldg(reinterpret_cast<const uint4*>(g.bias + col0 + v8 * 8));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) bv[j] = g.bias[col0 + v8 * 8 + j];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] += __bfloat162float(bv[j]);
    }
    if (g.flags & (EPI_RESIDUAL | EPI_DGELU)) {
      __nv_bfloat16 aux[8];
      *reinterpret_cast<uint4*>(aux) = *reinterpret_cast<const uint4*>(g.aux_in + base + v8 * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = __bfloat162float(aux[j]);
        x[j] = (g.flags & EPI_RESIDUAL) ? x[j] + a : x[j] * gelu_grad(a);
      }
    }
    if (g.flags & EPI_GELU) {
      if (g.aux_out != nullptr) {
        __nv_bfloat162 pre[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) pre[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
        *reinterpret_cast<uint4*>(g.aux_out + base + v8 * 8) = *reinterpret_cast<const uint4*>(pre);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = gelu_exact(x[j]);
    }
    if (out_f32) {
      float* o = reinterpret_cast<float*>(g.out) + base + v8 * 8;
      float4 lo = make_float4(x[0], x[1], x[2], x[3]), hi = make_float4(x[4], x[5], x[6], x[7]);
      if (g.flags & EPI_ACCUMULATE) {
        const float4 a = *reinterpret_cast<const float4*>(o), b = *reinterpret_cast<const float4*>(o + 4);
        lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
        hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
      }
      *reinterpret_cast<float4*>(o) = lo;
      *reinterpret_cast<float4*>(o + 4) = hi;
    } else {
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(g.out) + base + v8 * 8;
      if (g.flags & EPI_ACCUMULATE) {
        __nv_bfloat16 y[8];
        *reinterpret_cast<uint4*>(y) = *reinterpret_cast<const uint4*>(o);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] += __bfloat162float(y[j]);
      }
      __nv_bfloat162 y2[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) y2[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
      *reinterpret_cast<uint4*>(o) = *reinterpret_cast<const uint4*>(y2);
    }
  }
}

// Writes a warp's 32-row x 64-column bf16 block (lane = row, `v` = that row's 128 bytes as eight
// 16-byte vectors) to row-major global memory through shared memory, so that each store instruction
// covers four complete 128-byte lines instead of 32 scattered 16-byte pieces.  The 16-byte slots are
// XOR-swizzled by row so neither the writes (lane = row) nor the reads (8 lanes per row) conflict.
__device__ __forceinline__ void store_block_coalesced(uint8_t* stage, const uint4 (&v)[8], __nv_bfloat16* out, size_t ldc,
                                                      int row0, int rows_valid, int col0, int lane, bool skip) {
  __syncwarp();
#pragma unroll
  for (int sgm = 0; sgm < 8; ++sgm) *reinterpret_cast<uint4*>(stage + lane * 128 + ((sgm ^ (lane & 7)) << 4)) = v[sgm];
  __syncwarp();
  const int sgm = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = (lane >> 3) + 4 * i;
    const uint4 x = *reinterpret_cast<const uint4*>(stage + r * 128 + ((sgm ^ (r & 7)) << 4));
    if (r < rows_valid && !skip) *reinterpret_cast<uint4*>(out + (size_t)(row0 + r) * ldc + col0 + sgm * 8) = x;
    if (skip && x.x == 0x7fc0dead) stage[0] = 1;  // keeps the loads alive when stores are skipped
  }
}

// Two adjacent 32-column chunks (64 columns) of an interior tile with a bf16 output: element-wise
// work in registers, then coalesced stores of the result (and of the pre-activation, if kept).
__device__ __forceinline__ void epilogue_pair_interior(const uint32_t (&ra)[32], const uint32_t (&rb)[32], uint8_t* stage, int row,
                                                       int row0, int rows_valid, int col0, const GemmArgs& g, bool bias_vec, int lane) {
  uint4 outv[8], prev[8];
  const bool keep_pre = (g.flags & EPI_GELU) && g.aux_out != nullptr;
  const bool row_ok = row < g.M;
  const size_t base = (size_t)(row_ok ? row : row0) * g.ldc + col0;  // rows past M only feed the staging shuffle
#pragma unroll
  for (int v8 = 0; v8 < 8; ++v8) {
    float x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(v8 < 4 ? ra[v8 * 8 + j] : rb[(v8 - 4) * 8 + j]);
    if (g.flags & EPI_BIAS) {
      __nv_bfloat16 bv[8];
      if (bias_vec) {
        *reinterpret_cast<uint4*>(bv) = __ldg(reinterpret_cast<const uint4*>(g.bias + col0 + v8 * 8));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) bv[j] = g.bias[col0 + v8 * 8 + j];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] += __bfloat162float(bv[j]);
    }
    if (g.flags & (EPI_RESIDUAL | EPI_DGELU | EPI_ACCUMULATE)) {
      __nv_bfloat16 aux[8];
      const __nv_bfloat16* src = (g.flags & EPI_ACCUMULATE) && !(g.flags & (EPI_RESIDUAL | EPI_DGELU))
                                     ? reinterpret_cast<const __nv_bfloat16*>(g.out) : g.aux_in;
      *reinterpret_cast<uint4*>(aux) = *reinterpret_cast<const uint4*>(src + base + v8 * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = __bfloat162float(aux[j]);
        x[j] = (g.flags & EPI_DGELU) ? x[j] * gelu_grad(a) : x[j] + a;
      }
    }
    if (g.flags & EPI_GELU) {
      __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&prev[v8]);
#pragma unroll
      for (int j = 0; j < 4; ++j) pp[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = gelu_exact(x[j]);
    }
    __nv_bfloat162* oo = reinterpret_cast<__nv_bfloat162*>(&outv[v8]);
#pragma unroll
    for (int j = 0; j < 4; ++j) oo[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
  }
  const bool skip = g.flags & EPI_NO_STORE;
  store_block_coalesced(stage, outv, reinterpret_cast<__nv_bfloat16*>(g.out), g.ldc, row0, rows_valid, col0, lane, skip);
  if (keep_pre) store_block_coalesced(stage, prev, g.aux_out, g.ldc, row0, rows_valid, col0, lane, skip);
}

// Tile shapes.  BM = 128: one 128-row accumulator per tile, two of them in TMEM so the next tile's
// MMAs overlap this tile's epilogue.  BM = 256: two 128-row MMAs per k-step share one B tile (a
// third less operand traffic per flop and twice the work per pipeline stage, which is what hides
// the load latency); its two accumulators fill TMEM, so only the halves overlap.
template <int BM, int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES > 8 ? 8 : SMEM_BUDGET / STAGE_BYTES;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_STAGING + 1024 /* alignment slack */ + 256 /* barriers */;
  static constexpr int THREADS = 64 + 256;  // producer warp, MMA warp, eight epilogue warps
};

template <int BM, int BN, bool A_MN, bool B_MN, bool GATHER = false>
__global__ void __launch_bounds__(GATHER ? 384 : 320, 1)
k_gemm(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs g, const GatherArgs ga) {
  extern __shared__ uint8_t smem_raw[];
  using L = SmemLayout<BM, BN>;
  constexpr int STAGES = L::STAGES;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * L::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + EPI_STAGING);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (g.M + BM - 1) / BM, tiles_n = (g.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (g.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: a power of two
  // Tile t -> (m0, n0).  m runs fastest, so the CTAs sweep one weight panel at a time; with GATHER the panels
  // are visited starting from the one this rank's own shard feeds, the order in which the chunks arrive.
  auto tile_origin = [&](int tile, int* m0, int* n0) {
    int n_idx = tile / tiles_m;
    if (GATHER) n_idx = (n_idx + ga.n_start) % tiles_n;
    *m0 = (tile % tiles_m) * BM;
    *n0 = n_idx * BN;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], BM == 128 ? 8 : 4);  // one arrival per epilogue warp that drains it
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m0, n0;
        tile_origin(tile, &m0, &n0);
        if (GATHER) {  // the panel's bytes must have arrived (they are row-contiguous: rows n0 .. n0+BN of [N, K])
          const long long lo = (long long)n0 * g.K * 2;
          long long hi = (long long)(n0 + BN < g.N ? n0 + BN : g.N) * g.K * 2;
          if (!(ok = wait_chunks(ga.ready, (int)(lo / ga.chunk_bytes), (int)((hi - 1) / ga.chunk_bytes), ga.epoch, g.error))) break;
          asm volatile("fence.proxy.async;" ::: "memory");  // the fetchers' generic-proxy stores, then TMA's async-proxy loads
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&empty[s], phase ^ 1, g.error))) break;
          uint8_t* a_dst = smem + s * L::STAGE_BYTES;
          uint8_t* b_dst = a_dst + L::A_BYTES;
          mbar_expect_tx(&full[s], L::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(a_dst, &map_a, &full[s], k0, m0);  // box {64 k, BM rows}
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &map_a, &full[s], m0 + j * 64, k0);  // box {64 mn, 64 k}
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &map_b, &full[s], k0, n0);  // box {64 k, BN rows}
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &map_b, &full[s], n0 + j * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(128, BN, A_MN, B_MN);
      constexpr int HALVES = BM / 128;
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        // BM = 128: accumulators alternate between the two TMEM regions.  BM = 256: region h holds rows [128h, 128h+128).
        const uint32_t first_buf = HALVES == 1 ? (local_tile & 1) : 0;
        const uint32_t acc_phase = HALVES == 1 ? ((local_tile >> 1) & 1) : (local_tile & 1);
        for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&full[s], phase, g.error))) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t b_addr = a_addr + L::A_BYTES;
          // K-major: rows of 128 B, 8-row groups 1024 B apart; one K=16 step is 32 B along the row.
          // MN-major: 64-wide strips 8192 B apart (LBO), 8 k-rows 1024 B apart (SBO); one K=16 step is 16 rows = 2048 B.
          const uint64_t b_desc = B_MN ? smem_desc(b_addr, 8192, 1024) : smem_desc(b_addr, 16, 1024);
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            const uint32_t buf = first_buf + h;
            if (kb == 0) {  // the epilogue has drained this accumulator
              if (!(ok = mbar_wait(&acc_empty[buf], acc_phase ^ 1, g.error))) break;
              tc_fence_after();
            }
            const uint32_t d_tmem = tmem_base + buf * BN;
            const uint32_t a_half = a_addr + h * 16384;  // 128 rows x 128 B, or two 64-wide strips
            const uint64_t a_desc = A_MN ? smem_desc(a_half, 8192, 1024) : smem_desc(a_half, 16, 1024);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint64_t a_k = a_desc + (uint64_t)((A_MN ? 2048 : 32) * k >> 4);
              const uint64_t b_k = b_desc + (uint64_t)((B_MN ? 2048 : 32) * k >> 4);
              mma_bf16(d_tmem, a_k, b_k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          if (ok) mma_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
        }
        if (ok) {
#pragma unroll
          for (int h = 0; h < HALVES; ++h) mma_commit(&acc_full[first_buf + h]);
        }
      }
    }
  } else if (GATHER && warp >= 10) {
    // ------------------------------------------------------------------ weight fetchers (warps 10, 11)
    const int ft = threadIdx.x - 320;  // 0..63
    const int nchunks = (int)((ga.w_bytes + ga.chunk_bytes - 1) / ga.chunk_bytes);
    const int first = (int)(((long long)ga.n_start * BN * g.K * 2) / ga.chunk_bytes);
    __threadfence_system();  // observe the owners' latest stores to their shards
    for (int ci = blockIdx.x; ci < nchunks; ci += gridDim.x) {
      const int c = (first + ci) % nchunks;
      const long long c0 = ga.w_off + (long long)c * ga.chunk_bytes;
      const long long c1 = ga.w_off + ((long long)(c + 1) * ga.chunk_bytes < ga.w_bytes ? (long long)(c + 1) * ga.chunk_bytes : ga.w_bytes);
      for (int q = 0; q < ga.n; ++q) {
        const long long lo = c0 > ga.shard_lo[q] ? c0 : ga.shard_lo[q];
        const long long hi = c1 < ga.shard_hi[q] ? c1 : ga.shard_hi[q];
        if (lo >= hi) continue;
        const char* src = ga.shard[q] + (lo - ga.shard_lo[q]);
        char* dst = ga.full + lo;
        const long long len = hi - lo;
        const bool al = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
        const long long nv = al ? len / 16 : 0;
        for (long long v = ft; v < nv; v += 64 * 4) {  // four independent 16-byte loads in flight per thread
          uint4 x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (v + u * 64 < nv)
              asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(x[u].x), "=r"(x[u].y), "=r"(x[u].z), "=r"(x[u].w) : "l"(src + (v + u * 64) * 16));
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (v + u * 64 < nv) *reinterpret_cast<uint4*>(dst + (v + u * 64) * 16) = x[u];
        }
        for (long long i = nv * 16 + ft; i < len; i += 64) dst[i] = *reinterpret_cast<volatile const char*>(src + i);
      }
      __threadfence();
      asm volatile("bar.sync 1, 64;" ::: "memory");  // the two fetch warps only
      if (ft == 0) st_release_gpu(ga.ready + c, ga.epoch);
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ epilogue (warps 2 .. 9)
    // Eight epilogue warps in two groups of four (one warp per TMEM lane quarter in each group).
    // BM = 128: both groups drain the same accumulator, each taking half of its columns.
    // BM = 256: group h drains the accumulator of rows [128h, 128h + 128).
    const int quarter = warp & 3;        // TMEM lanes [32*quarter, 32*quarter + 32) belong to this warp
    const int group = (warp - 2) >> 2;
    const int half = BM == 128 ? 0 : group;
    uint32_t local_tile = 0;
    bool ok = true;
    const bool out_f32 = g.flags & EPI_OUT_F32;
    if (GATHER && (g.flags & EPI_BIAS) && ga.tail_bytes > 0) {
      // the bias sits right behind the weight in the flat buffer and is fetched with it: wait for its chunks
      const long long lo = (long long)g.N * g.K * 2, hi = lo + ga.tail_bytes;
      ok = wait_chunks(ga.ready, (int)(lo / ga.chunk_bytes), (int)((hi - 1) / ga.chunk_bytes), ga.epoch, g.error);
      ok = __all_sync(0xffffffffu, ok);
    }
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      int m0, n0;
      tile_origin(tile, &m0, &n0);
      const uint32_t buf = BM == 128 ? (local_tile & 1) : half;
      const uint32_t acc_phase = BM == 128 ? ((local_tile >> 1) & 1) : (local_tile & 1);
      ok = mbar_wait(&acc_full[buf], acc_phase, g.error);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + half * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      // Chunks of 32 columns, the TMEM load of the next one in flight while this one is processed.
      const bool interior_rows = row < g.M && (g.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(g.out) & 15) == 0;
      const bool bias_vec = (g.flags & EPI_BIAS) && (reinterpret_cast<uintptr_t>(g.bias) & 15) == 0;
      constexpr int CHUNKS = BN / 32;
      const int c_begin = BM == 128 ? group * (CHUNKS / 2) : 0;
      const int c_end = BM == 128 ? c_begin + CHUNKS / 2 : CHUNKS;
      if (!(g.flags & EPI_DISCARD)) {
        uint32_t ra[32], rb[32];
        uint8_t* stage = staging + (warp - 2) * 4096;
        const int row0 = m0 + half * 128 + quarter * 32;           // first row of this warp's block
        const int rows_valid = g.M - row0 < 32 ? g.M - row0 : 32;   // may be <= 0 on the last tile row
        // bf16 outputs whose rows are 16-byte aligned go through the coalescing path; accumulate-with-aux combinations
        // and fp32 outputs take the direct path.
        const bool pair_ok = !out_f32 && (g.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(g.out) & 15) == 0 && rows_valid > 0 &&
                             !((g.flags & EPI_ACCUMULATE) && (g.flags & (EPI_RESIDUAL | EPI_DGELU)));
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 2) {  // c_end - c_begin is even: 2 or 4 or 8 chunks
          tmem_ld32(taddr + c * 32, ra);
          tmem_ld32(taddr + (c + 1) * 32, rb);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (g.flags & EPI_LOAD_ONLY) {
            if (ra[0] == 0x7fc0dead && rb[31] == 0x7fc0dead) stage[0] = 1;  // keeps the loads alive
            continue;
          }
          if (pair_ok && col0 + 64 <= g.N) {
            epilogue_pair_interior(ra, rb, stage, row, row0, rows_valid, col0, g, bias_vec, lane);
          } else {
            if (interior_rows && col0 + 32 <= g.N) epilogue_chunk_interior(ra, row, col0, g, out_f32, bias_vec);
            else epilogue_chunk_generic(ra, row, col0, g, out_f32);
            if (interior_rows && col0 + 64 <= g.N) epilogue_chunk_interior(rb, row, col0 + 32, g, out_f32, bias_vec);
            else epilogue_chunk_generic(rb, row, col0 + 32, g, out_f32);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
  static EncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)p;
  }
  return fn;
}

char g_map_error[256] = "";

// A 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows of `row_stride` elements.
int make_map(CUtensorMap* map, const void* ptr, long long inner, long long outer, long long row_stride, int box_inner, int box_outer) {
  // cuTensorMapEncodeTiled is a driver entry point: it needs this thread to have a current context, which a
  // thread that has so far only been handed cached allocations (an autograd worker) may not have yet.
  static thread_local bool context_ready = false;
  if (!context_ready) {
    cudaFree(nullptr);
    context_ready = true;
  }
  EncodeTiled enc = encoder();
  if (enc == nullptr) return -10;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    snprintf(g_map_error, sizeof(g_map_error), "cuTensorMapEncodeTiled -> %d (ptr %p, dims %lld x %lld, row stride %lld el, box %d x %d)",
             (int)r, ptr, inner, outer, row_stride, box_inner, box_outer);
  return r == CUDA_SUCCESS ? 0 : -11;
}

int* g_error_host = nullptr;
int* g_error_dev = nullptr;
int g_sm_count = 0;

template <int BM, int BN, bool A_MN, bool B_MN>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& g, int max_ctas, cudaStream_t stream) {
  auto kernel = k_gemm<BM, BN, A_MN, B_MN>;
  using L = SmemLayout<BM, BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN);
  int ctas = tiles < g_sm_count ? tiles : g_sm_count;
  if (max_ctas > 0 && ctas > max_ctas) ctas = max_ctas;
  kernel<<<ctas, L::THREADS, L::TOTAL, stream>>>(ma, mb, g, GatherArgs{});
  return (int)cudaGetLastError();
}

// Picks the tile shape with the least estimated time: rounds of tiles over the SMs times the relative
// cost of one tile.  Measured on B200 (tandem_b200/ops/bench_gemm.py --tile): with a short reduction
// (K <= 1024) the epilogue sets the pace and the double-buffered 128x256 tile wins; with a long one the
// 256x256 tile wins (a third less operand traffic per flop) unless it leaves most SMs idle, and the
// weight-gradient shapes (few output tiles, K = tokens) want 128x128 tiles to fill the machine.
void choose_tile(int M, int N, int K, int sms, int forced, int* bm, int* bn) {
  struct Shape { int bm, bn; double cost; };  // cost: relative time of one tile at equal K
  const Shape shapes[3] = {{256, 256, K <= 1024 ? 5.0 : 4.0}, {128, 256, 2.3}, {128, 128, 1.5}};
  if (forced >= 0 && forced < 3) {
    *bm = shapes[forced].bm;
    *bn = shapes[forced].bn;
    return;
  }
  double best = 1e30;
  for (const Shape& s : shapes) {
    if (s.bn > 128 && N <= 128) continue;
    const long long tiles = (long long)((M + s.bm - 1) / s.bm) * ((N + s.bn - 1) / s.bn);
    const long long rounds = (tiles + sms - 1) / sms;
    const double t = rounds * s.cost;
    if (t < best - 1e-9) {
      best = t;
      *bm = s.bm;
      *bn = s.bn;
    }
  }
}

int g_forced_tile = -1;

}  // namespace

extern "C" void tb_note_launch(int n);

extern "C" {

// 0 while every GEMM wait so far has completed; 1 after one ran out.
int tb_gemm_error() { return g_error_host != nullptr ? *g_error_host : 0; }

// D[M,N] = op(A) . op(B) with bf16 operands, then the epilogue selected by `flags` (EpilogueFlags).
//   a_mn == 0: A is [M, K] with leading dimension lda (K contiguous); a_mn == 1: A is [K, M], lda (M contiguous).
//   b_mn == 0: B is [N, K] with leading dimension ldb (K contiguous); b_mn == 1: B is [K, N], ldb (N contiguous).
// Leading dimensions must be multiples of 8 elements and base pointers 16-byte aligned (TMA).
int tb_gemm_bf16(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn,
                 int flags, const void* bias, const void* aux_in, void* aux_out, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (((uintptr_t)A | (uintptr_t)B) & 15)) return -12;
  if (g_error_host == nullptr) {
    if (cudaHostAlloc((void**)&g_error_host, 64, cudaHostAllocMapped) != cudaSuccess) return -13;
    *g_error_host = 0;
    if (cudaHostGetDevicePointer((void**)&g_error_dev, g_error_host, 0) != cudaSuccess) return -13;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  int BM = 128, BN = 128;
  choose_tile(M, N, K, g_sm_count, g_forced_tile, &BM, &BN);
  CUtensorMap ma, mb;
  int rc;
  if (!a_mn) rc = make_map(&ma, A, K, M, lda, 64, BM);
  else rc = make_map(&ma, A, M, K, lda, 64, 64);
  if (rc) return rc;
  if (!b_mn) rc = make_map(&mb, B, K, N, ldb, 64, BN);
  else rc = make_map(&mb, B, N, K, ldb, 64, 64);
  if (rc) return rc;
  GemmArgs g{M, N, K, ldc, flags, out, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)aux_in, (__nv_bfloat16*)aux_out, g_error_dev};
  tb_note_launch(1);
#define GO(BM_, BN_) \
  do { \
    if (!a_mn && !b_mn) return launch_gemm<BM_, BN_, false, false>(ma, mb, g, max_ctas, stream); \
    if (!a_mn && b_mn) return launch_gemm<BM_, BN_, false, true>(ma, mb, g, max_ctas, stream); \
    if (a_mn && b_mn) return launch_gemm<BM_, BN_, true, true>(ma, mb, g, max_ctas, stream); \
    return launch_gemm<BM_, BN_, true, false>(ma, mb, g, max_ctas, stream); \
  } while (0)
  if (BM == 256) GO(256, 256);
  if (BN == 256) GO(128, 256);
  GO(128, 128);
#undef GO
}

// out[M, N] = A[M, K] . W[N, K]^T (+ epilogue) where W is gathered by the kernel itself: rank q's shard (peer
// address shards[q]) holds bytes [shard_lo[q], shard_hi[q]) of the unit's flat buffer; W is the byte range
// [w_off, w_off + N*K*2) of it and is assembled in `full` (this GPU's copy) while the GEMM runs.
// tail_bytes: bytes right behind W in the flat buffer to fetch as well (the layer's bias; pass bias = full + w_off +
// N*K*2 then).  ready: one zero-initialised word per chunk (ceil((N*K*2 + tail_bytes) / chunk_bytes)); epoch: a value not used by an earlier
// call on the same words.  One cooperative launch; returns a CUDA error if the grid cannot be co-resident.
int tb_gemm_gathered(const void* A, void* out, int M, int N, int K, int lda, int ldc, int flags, const void* bias, const void* aux_in,
                     void* aux_out, void* const* shards, const long long* shard_lo, const long long* shard_hi, int n_ranks, void* full,
                     long long w_off, long long tail_bytes, void* ready, unsigned epoch, int chunk_bytes, int n_start,
                     cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (K & 7) || (w_off & 15) || (((uintptr_t)A | (uintptr_t)full) & 15) || n_ranks < 1 || n_ranks > 8) return -12;
  if (g_error_host == nullptr) {
    if (cudaHostAlloc((void**)&g_error_host, 64, cudaHostAllocMapped) != cudaSuccess) return -13;
    *g_error_host = 0;
    if (cudaHostGetDevicePointer((void**)&g_error_dev, g_error_host, 0) != cudaSuccess) return -13;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  constexpr int BM = 128, BN = 256;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, A, K, M, lda, 64, BM);
  if (rc) return rc;
  rc = make_map(&mb, (const char*)full + w_off, K, N, K, 64, BN);
  if (rc) return rc;
  GemmArgs g{M, N, K, ldc, flags, out, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)aux_in, (__nv_bfloat16*)aux_out, g_error_dev};
  GatherArgs ga{};
  for (int q = 0; q < n_ranks; ++q) {
    ga.shard[q] = (const char*)shards[q];
    ga.shard_lo[q] = shard_lo[q];
    ga.shard_hi[q] = shard_hi[q];
  }
  ga.full = (char*)full;
  ga.w_off = w_off;
  ga.w_bytes = (long long)N * K * 2 + tail_bytes;
  ga.tail_bytes = tail_bytes;
  ga.ready = (uint32_t*)ready;
  ga.epoch = epoch;
  ga.n = n_ranks;
  ga.chunk_bytes = chunk_bytes;
  const int tiles_n = (N + BN - 1) / BN;
  ga.n_start = ((n_start % tiles_n) + tiles_n) % tiles_n;
  auto kernel = k_gemm<BM, BN, false, false, true>;
  using L = SmemLayout<BM, BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * tiles_n;
  int ctas = tiles < g_sm_count ? tiles : g_sm_count;
  void* params[] = {(void*)&ma, (void*)&mb, (void*)&g, (void*)&ga};
  tb_note_launch(1);
  return (int)cudaLaunchCooperativeKernel((const void*)kernel, dim3(ctas), dim3(384), params, L::TOTAL, stream);
}

// Forces a tile shape for every later call (0: 256x256, 1: 128x256, 2: 128x128; -1: automatic).  For tuning.
void tb_gemm_force_tile(int which) { g_forced_tile = which; }

const char* tb_gemm_last_error() { return g_map_error; }

}  // extern "C"
