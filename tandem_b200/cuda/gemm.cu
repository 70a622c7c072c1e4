// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = A . B (+ epilogue), fp32 accumulation in TMEM.
//
// Two kernels share the epilogue code: k_gemm (below: one persistent CTA per SM) and k_gemm_pair (further down: CTA
// pairs driving tcgen05.mma.cta_group::2).  Neither uses TMA multicast.  Outputs in bf16 leave through TMA stores.
//
// Structure of k_gemm (one persistent CTA per SM, 320 threads, no cluster):
//   warp 0      TMA producer: cp.async.bulk.tensor.2d loads A and B tiles (128B swizzle) into a
//               3- to 6-stage shared-memory ring, signalling `full[s]` by transaction bytes.
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma.cta_group::1.kind::f16
//               (128 x BN x 16 per instruction, 4 per stage), releases stages with
//               tcgen05.commit -> `empty[s]`, and hands a finished accumulator to the epilogue
//               with tcgen05.commit -> `acc_full[b]`.  TMEM holds two accumulators (2 x BN
//               columns), so the next tile's MMAs overlap this tile's epilogue.
//   warps 2-9   epilogue: tcgen05.ld 32 lanes x 64 columns at a time, then bias / GELU / residual /
//               dGELU / accumulate in registers; a bf16 block is staged in shared memory (128-byte
//               swizzle) and written by one cp.async.bulk.tensor store, fp32 outputs by 16-byte stores.
// Tile shapes: 256x256, 128x256, 128x192, 128x128 (choose_tile); split-K for outputs with very few tiles.
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
#include <atomic>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "launch.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BK = 64;
constexpr int SMEM_BUDGET = 192 * 1024;   // operand ring
constexpr int EPI_STAGING = 8 * 4096;     // per epilogue warp: a 32-row x 128-byte block for coalescing its stores

enum EpilogueFlags {
  EPI_BIAS = 1,        // + bias[col]
  EPI_GELU = 2,        // out = gelu(v); with aux_out: also write gelu'(v) there (what backward multiplies by)
  EPI_RESIDUAL = 4,    // + aux_in[row, col]
  EPI_DGELU = 8,       // out = v * aux_in[row, col]  (aux_in = the gelu'(.) that the forward GEMM saved)
  EPI_ACCUMULATE = 16, // out += v  (gradient accumulation)
  EPI_OUT_F32 = 32,    // out is fp32 (else bf16)
};

struct GemmArgs {
  int M, N, K;
  int ldc;            // leading dimension of out / aux (elements)
  int flags;
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux_in;   // residual, or the saved gelu' factors, [M, ldc]
  __nv_bfloat16* aux_out;        // gelu'(pre-activation) out for EPI_GELU, [M, ldc]
  int* error;                    // host-mapped; set to 1 when a wait runs out
  int tma_store;                 // map_out (and map_pre) are valid: bf16 output blocks leave through TMA stores
  // Split-K of the last wave.  Output tiles [0, whole_tiles) -- as many full rounds of one tile per CTA as there are --
  // are computed whole.  The remaining tiles, too few to occupy the SMs, have their reduction cut into `splits`
  // parts and each (tile, part) is a work item: parts 1 .. splits-1 ("producers") park their raw fp32 accumulator
  // tile in `partials` and raise one flag per epilogue warp; part 0 ("consumer") adds the parked tiles to its own
  // accumulator, in part order, and runs the ordinary epilogue (bias, GELU, residual, TMA store ...).  Items are
  // ordered whole tiles, producers, consumers; every CTA works through its items in that order and a producer
  // never waits, so the scheme cannot deadlock whatever the grid.  One kernel, no reduction pass, and the result
  // does not depend on scheduling.
  int splits;             // 1: nothing is split
  int whole_tiles;        // tiles computed by one item each (0 when every tile is split)
  float* partials;        // [split tile][splits - 1][column quad][row][4] floats
  unsigned* split_flags;  // [split tile][splits - 1][8 epilogue warps], zero between launches (the consumer resets them)
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

// Exact (erf) GELU and its derivative from one evaluation:  erf through Abramowitz & Stegun 7.1.26 (absolute error
// below 1.5e-7, far inside a bf16 rounding), whose exp(-z^2) with z = |x| / sqrt(2) is the very exp(-x^2 / 2) that the
// density needs.  One ex2 and one reciprocal on the special-function unit plus a dozen FMAs, against erff + expf before;
// the element-wise epilogue is what bounds the K = 768 GEMMs.
//   gelu(x)  = x * Phi(x)          Phi(x) = (1 + erf(x / sqrt 2)) / 2
//   gelu'(x) = Phi(x) + x * phi(x)  phi(x) = exp(-x^2 / 2) / sqrt(2 pi)
__device__ __forceinline__ void gelu_and_grad(float x, float* g, float* dg) {
  const float z = fabsf(x) * 0.70710678118654752440f;
  const float t = __frcp_rn(fmaf(0.3275911f, z, 1.f));
  const float e = ex2_approx(-0.72134752044448170368f * x * x);  // exp(-x^2 / 2)
  const float poly = t * fmaf(t, fmaf(t, fmaf(t, fmaf(t, 1.061405429f, -1.453152027f), 1.421413741f), -0.284496736f), 0.254829592f);
  const float erf_abs = fmaf(-poly, e, 1.f);
  const float cdf = 0.5f * (1.f + copysignf(erf_abs, x));
  *g = x * cdf;
  *dg = fmaf(x * 0.39894228040143267794f, e, cdf);
}

// ------------------------------------------------------------------------------------------ kernel
// One 32-column chunk of one accumulator row: the general path (tile edges, padded rows, any flags).
__device__ __forceinline__ void epilogue_chunk_generic(const uint32_t (&raw)[32], int row, int col0, const GemmArgs& g, void* out,
                                                       bool out_f32) {
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
          x[j] = (g.flags & EPI_RESIDUAL) ? x[j] + a : x[j] * a;
        }
      }
      if (g.flags & EPI_GELU) {
        float dg[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) gelu_and_grad(x[j], &x[j], &dg[j]);
        if (g.aux_out != nullptr) {
          __nv_bfloat16 pre[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) pre[j] = __float2bfloat16_rn(dg[j]);
          if (full8) {
            *reinterpret_cast<uint4*>(g.aux_out + base + v8 * 8) = *reinterpret_cast<const uint4*>(pre);
          } else {
            for (int j = 0; j < 8; ++j)
              if (col + j < g.N) g.aux_out[base + v8 * 8 + j] = pre[j];
          }
        }
      }
      if (out_f32) {
        float* o = reinterpret_cast<float*>(out) + base + v8 * 8;
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
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + base + v8 * 8;
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
__device__ __forceinline__ void epilogue_chunk_interior(const uint32_t (&raw)[32], int row, int col0, const GemmArgs& g, void* out,
                                                        bool out_f32, bool bias_vec) {
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
        x[j] = (g.flags & EPI_RESIDUAL) ? x[j] + a : x[j] * a;
      }
    }
    if (g.flags & EPI_GELU) {
      float dg[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) gelu_and_grad(x[j], &x[j], &dg[j]);
      if (g.aux_out != nullptr) {
        __nv_bfloat162 pre[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) pre[j] = __floats2bfloat162_rn(dg[2 * j], dg[2 * j + 1]);
        *reinterpret_cast<uint4*>(g.aux_out + base + v8 * 8) = *reinterpret_cast<const uint4*>(pre);
      }
    }
    if (out_f32) {
      float* o = reinterpret_cast<float*>(out) + base + v8 * 8;
      float4 lo = make_float4(x[0], x[1], x[2], x[3]), hi = make_float4(x[4], x[5], x[6], x[7]);
      if (g.flags & EPI_ACCUMULATE) {
        const float4 a = *reinterpret_cast<const float4*>(o), b = *reinterpret_cast<const float4*>(o + 4);
        lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
        hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
      }
      *reinterpret_cast<float4*>(o) = lo;
      *reinterpret_cast<float4*>(o + 4) = hi;
    } else {
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + base + v8 * 8;
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

// Writes a warp's 32-row x 64-column bf16 block (lane = row, `v` = that row's 128 bytes as eight 16-byte
// vectors) to row-major global memory through a 4 KB shared-memory block.  The 16-byte slots are
// XOR-swizzled by row, which is both conflict-free for the writes (lane = row) and the 128-byte swizzle
// of a TMA tile.
//   map != nullptr: one cp.async.bulk.tensor store of the block {64 columns, 32 rows} at (col0, row0); the
//     tensor map clips rows >= M and columns >= N.  Shared memory carries the bytes once in and once out, and
//     the stores never pass through the load/store unit, whose global stores (measured on B200) slow the
//     MMA/TMA traffic of the main loop several times more than their size would suggest.
//   map == nullptr: the warp reads the block back and stores complete 128-byte lines itself.
__device__ __forceinline__ void store_block(uint8_t* stage, const uint4 (&v)[8], const CUtensorMap* map, __nv_bfloat16* out, size_t ldc,
                                            int row0, int rows_valid, int col0, int lane) {
  if (map != nullptr) {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the previous store has read the block
    __syncwarp();
#pragma unroll
    for (int sgm = 0; sgm < 8; ++sgm) *reinterpret_cast<uint4*>(stage + lane * 128 + ((sgm ^ (lane & 7)) << 4)) = v[sgm];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes, then the async proxy's read
    __syncwarp();
    if (lane == 0) {
      asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_u32(stage)),
                   "r"(col0), "r"(row0)
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    return;
  }
  __syncwarp();
#pragma unroll
  for (int sgm = 0; sgm < 8; ++sgm) *reinterpret_cast<uint4*>(stage + lane * 128 + ((sgm ^ (lane & 7)) << 4)) = v[sgm];
  __syncwarp();
  const int sgm = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = (lane >> 3) + 4 * i;
    const uint4 x = *reinterpret_cast<const uint4*>(stage + r * 128 + ((sgm ^ (r & 7)) << 4));
    if (r < rows_valid) *reinterpret_cast<uint4*>(out + (size_t)(row0 + r) * ldc + col0 + sgm * 8) = x;
  }
}

// Before an epilogue warp leaves: its bulk stores have read their shared-memory blocks (the writes themselves
// complete with the grid).
__device__ __forceinline__ void drain_stores(int lane) {
  if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  __syncwarp();
}

// Two adjacent 32-column chunks (64 columns) of an interior tile with a bf16 output: element-wise
// work in registers, then coalesced stores of the result (and of the pre-activation, if kept).
__device__ __forceinline__ void epilogue_pair_interior(const uint32_t (&ra)[32], const uint32_t (&rb)[32], uint8_t* stage, int row,
                                                       int row0, int rows_valid, int col0, const GemmArgs& g, void* out, bool bias_vec,
                                                       int lane, const CUtensorMap* map_out, const CUtensorMap* map_pre) {
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
                                     ? reinterpret_cast<const __nv_bfloat16*>(out) : g.aux_in;
      *reinterpret_cast<uint4*>(aux) = *reinterpret_cast<const uint4*>(src + base + v8 * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = __bfloat162float(aux[j]);
        x[j] = (g.flags & EPI_DGELU) ? x[j] * a : x[j] + a;
      }
    }
    if (g.flags & EPI_GELU) {
      float dg[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) gelu_and_grad(x[j], &x[j], &dg[j]);
      __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&prev[v8]);
#pragma unroll
      for (int j = 0; j < 4; ++j) pp[j] = __floats2bfloat162_rn(dg[2 * j], dg[2 * j + 1]);
    }
    __nv_bfloat162* oo = reinterpret_cast<__nv_bfloat162*>(&outv[v8]);
#pragma unroll
    for (int j = 0; j < 4; ++j) oo[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
  }
  store_block(stage, outv, map_out, reinterpret_cast<__nv_bfloat16*>(out), g.ldc, row0, rows_valid, col0, lane);
  if (keep_pre) store_block(stage, prev, map_pre, g.aux_out, g.ldc, row0, rows_valid, col0, lane);
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
__global__ void __launch_bounds__(GATHER ? 448 : 320, 1)
k_gemm(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_out,
       const __grid_constant__ CUtensorMap map_pre, const GemmArgs g, const GatherArgs ga) {
  const CUtensorMap* out_map = g.tma_store ? &map_out : nullptr;
  const CUtensorMap* pre_map = g.tma_store ? &map_pre : nullptr;
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
  const int splits = g.splits > 1 ? g.splits : 1;
  const int out_tiles = tiles_m * tiles_n;
  const int whole = splits > 1 ? g.whole_tiles : out_tiles, tail = out_tiles - whole;
  const int num_tiles = whole + tail * splits;  // work items: whole tiles, then the tail's producers, then its consumers
  const int k_blocks_all = (g.K + BK - 1) / BK;
  const int k_per = (k_blocks_all + splits - 1) / splits;
  // item -> output tile and k-part (-1: the whole reduction)
  auto tile_of = [&](int item) { return item < whole ? item : whole + (item - whole) % tail; };
  auto part_of = [&](int item) { return item < whole ? -1 : (item - whole < tail * (splits - 1) ? 1 + (item - whole) / tail : 0); };
  auto k_range = [&](int item, int* kb0, int* kb1) {
    const int part = part_of(item);
    *kb0 = part < 0 ? 0 : part * k_per;
    *kb1 = part < 0 || (part + 1) * k_per > k_blocks_all ? k_blocks_all : (part + 1) * k_per;
  };
  constexpr uint32_t ACC_COLS = BN == 192 ? 256 : BN;  // column stride between the two accumulators
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;         // 256 or 512: a power of two
  // Tile t -> (m0, n0).  m runs fastest, so the CTAs sweep one weight panel at a time; with GATHER the panels
  // are visited starting from the one this rank's own shard feeds, the order in which the chunks arrive.
  auto tile_origin = [&](int item, int* m0, int* n0) {
    const int tile = tile_of(item);
    int n_idx = tile / tiles_m;
    if (GATHER) n_idx = (n_idx + ga.n_start) % tiles_n;
    *m0 = (tile % tiles_m) * BM;
    *n0 = n_idx * BN;
  };

  if (warp == 0) {  // one lane per barrier; warp 1 allocates TMEM meanwhile
    if (lane < STAGES) {
      mbar_init(&full[lane], 1);
      mbar_init(&empty[lane], 1);
    } else if (lane < STAGES + 2) {
      mbar_init(&acc_full[lane - STAGES], 1);
      mbar_init(&acc_empty[lane - STAGES], BM == 128 ? 8 : 4);  // one arrival per epilogue warp that drains it
    } else if (lane == STAGES + 2) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      if (g.tma_store) prefetch_tensormap(&map_out);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tb::pdl_launch_dependents();  // the next kernel may set itself up while this one computes
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  tb::pdl_wait();  // barriers and TMEM are ready; from here on global memory written by earlier kernels is read

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
        int kb0, kb1;
        k_range(tile, &kb0, &kb1);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
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
        int kb0, kb1;
        k_range(tile, &kb0, &kb1);
        for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
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
            if (kb == kb0) {  // the epilogue has drained this accumulator
              if (!(ok = mbar_wait(&acc_empty[buf], acc_phase ^ 1, g.error))) break;
              tc_fence_after();
            }
            const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
            const uint32_t a_half = a_addr + h * 16384;  // 128 rows x 128 B, or two 64-wide strips
            const uint64_t a_desc = A_MN ? smem_desc(a_half, 8192, 1024) : smem_desc(a_half, 16, 1024);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint64_t a_k = a_desc + (uint64_t)((A_MN ? 2048 : 32) * k >> 4);
              const uint64_t b_k = b_desc + (uint64_t)((B_MN ? 2048 : 32) * k >> 4);
              mma_bf16(d_tmem, a_k, b_k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
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
    // ------------------------------------------------------------------ weight fetchers (warps 10 - 13)
    const int ft = threadIdx.x - 320;  // 0..127: four fetch warps
    constexpr int FT = 128, DEPTH = 8;  // eight independent 16-byte loads in flight per thread: 16 KB per CTA, ~2.4 MB per GPU
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
        for (long long v = ft; v < nv; v += FT * DEPTH) {
          uint4 x[DEPTH];
#pragma unroll
          for (int u = 0; u < DEPTH; ++u)
            if (v + u * FT < nv)
              asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(x[u].x), "=r"(x[u].y), "=r"(x[u].z), "=r"(x[u].w) : "l"(src + (v + u * FT) * 16));
#pragma unroll
          for (int u = 0; u < DEPTH; ++u)
            if (v + u * FT < nv) *reinterpret_cast<uint4*>(dst + (v + u * FT) * 16) = x[u];
        }
        for (long long i = nv * 16 + ft; i < len; i += FT) dst[i] = *reinterpret_cast<volatile const char*>(src + i);
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the fetch warps only
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
    const bool out_f32 = g.flags & EPI_OUT_F32;  // split-K: the host passes "store the fp32 partial tile" as the flags
    if (GATHER && (g.flags & EPI_BIAS) && ga.tail_bytes > 0) {
      // the bias sits right behind the weight in the flat buffer and is fetched with it: wait for its chunks
      const long long lo = (long long)g.N * g.K * 2, hi = lo + ga.tail_bytes;
      ok = wait_chunks(ga.ready, (int)(lo / ga.chunk_bytes), (int)((hi - 1) / ga.chunk_bytes), ga.epoch, g.error);
      ok = __all_sync(0xffffffffu, ok);
    }
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      int m0, n0;
      tile_origin(tile, &m0, &n0);
      void* out = g.out;
      const int part = part_of(tile), split_tile = tile_of(tile) - whole;
      // this warp's share of the parked partial tiles of its output tile: [part - 1][column quad][row][4]
      float* parked = part >= 0 ? g.partials + (size_t)split_tile * (splits - 1) * (BM * BN) : nullptr;
      unsigned* my_flags = part >= 0 ? g.split_flags + ((size_t)split_tile * (splits - 1)) * 8 + (warp - 2) : nullptr;
      const int tile_row = half * 128 + quarter * 32 + lane;
      if (part == 0) {  // consumer: every producer's matching warp must have parked its share
        for (int p = 0; p < splits - 1 && ok; ++p) {
          bool seen = true;
          if (lane == 0) {
            const long long start = clock64();
            while (ld_acquire_gpu(my_flags + p * 8) == 0u) {
              if (clock64() - start > (1ll << WAIT_LIMIT_CYCLES_SHIFT)) {
                *g.error = 1;
                __threadfence_system();
                seen = false;
                break;
              }
            }
          }
          ok = __shfl_sync(0xffffffffu, seen ? 1 : 0, 0) != 0;
        }
      }
      const uint32_t buf = BM == 128 ? (local_tile & 1) : half;
      const uint32_t acc_phase = BM == 128 ? ((local_tile >> 1) & 1) : (local_tile & 1);
      ok = mbar_wait_warp(&acc_full[buf], acc_phase, g.error);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + half * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS;
      // Chunks of 32 columns, the TMEM load of the next one in flight while this one is processed.
      const bool interior_rows = row < g.M && (g.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
      const bool bias_vec = (g.flags & EPI_BIAS) && (reinterpret_cast<uintptr_t>(g.bias) & 15) == 0;
      constexpr int CHUNKS = BN / 32;
      // BM = 128: the two warp groups split the columns (BN = 192: four chunks and two, so each takes whole pairs)
      const int c_split = BN == 192 ? 4 : CHUNKS / 2;
      const int c_begin = BM == 128 ? group * c_split : 0;
      const int c_end = BM == 128 ? (group == 0 ? c_split : CHUNKS) : CHUNKS;
      {
        uint32_t ra[32], rb[32];
        uint8_t* stage = staging + (warp - 2) * 4096;
        const int row0 = m0 + half * 128 + quarter * 32;           // first row of this warp's block
        const int rows_valid = g.M - row0 < 32 ? g.M - row0 : 32;   // may be <= 0 on the last tile row
        // bf16 outputs whose rows are 16-byte aligned go through the coalescing path; accumulate-with-aux combinations
        // and fp32 outputs take the direct path.
        const bool pair_ok = !out_f32 && (g.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && rows_valid > 0 &&
                             !((g.flags & EPI_ACCUMULATE) && (g.flags & (EPI_RESIDUAL | EPI_DGELU)));
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 2) {  // c_end - c_begin is even: 2 or 4 or 8 chunks
          tmem_ld32(taddr + c * 32, ra);
          tmem_ld32(taddr + (c + 1) * 32, rb);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          // Parked layout: [part - 1][column quad][row][4 floats].  A lane's four consecutive columns are one 16-byte
          // vector and consecutive lanes (rows) are consecutive vectors, so a warp moves 512 contiguous bytes per
          // instruction, 16 instructions per 64 columns.
          if (part > 0) {  // producer: park the raw accumulator
            float4* dst = reinterpret_cast<float4*>(parked + (size_t)(part - 1) * (BM * BN)) + (size_t)c * 8 * BM + tile_row;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              __stcg(dst + (size_t)q * BM, make_float4(__uint_as_float(ra[4 * q]), __uint_as_float(ra[4 * q + 1]),
                                                       __uint_as_float(ra[4 * q + 2]), __uint_as_float(ra[4 * q + 3])));
              __stcg(dst + (size_t)(8 + q) * BM, make_float4(__uint_as_float(rb[4 * q]), __uint_as_float(rb[4 * q + 1]),
                                                             __uint_as_float(rb[4 * q + 2]), __uint_as_float(rb[4 * q + 3])));
            }
            continue;
          }
          if (part == 0) {  // consumer: fold the parked tiles in, in part order
            if (!ok) continue;
            for (int p = 0; p < splits - 1; ++p) {
              const float4* src = reinterpret_cast<const float4*>(parked + (size_t)p * (BM * BN)) + (size_t)c * 8 * BM + tile_row;
              // all sixteen loads of a part are issued before the first add: one trip to L2 per part, not one per batch
              // the compiler happens to pick (volatile asm statements keep their order)
              float4 v[16];
#pragma unroll
              for (int q = 0; q < 16; ++q)
                asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(v[q].x), "=f"(v[q].y), "=f"(v[q].z), "=f"(v[q].w)
                             : "l"(src + (size_t)q * BM)
                             : "memory");
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                ra[4 * q] = __float_as_uint(__uint_as_float(ra[4 * q]) + v[q].x);
                ra[4 * q + 1] = __float_as_uint(__uint_as_float(ra[4 * q + 1]) + v[q].y);
                ra[4 * q + 2] = __float_as_uint(__uint_as_float(ra[4 * q + 2]) + v[q].z);
                ra[4 * q + 3] = __float_as_uint(__uint_as_float(ra[4 * q + 3]) + v[q].w);
                rb[4 * q] = __float_as_uint(__uint_as_float(rb[4 * q]) + v[8 + q].x);
                rb[4 * q + 1] = __float_as_uint(__uint_as_float(rb[4 * q + 1]) + v[8 + q].y);
                rb[4 * q + 2] = __float_as_uint(__uint_as_float(rb[4 * q + 2]) + v[8 + q].z);
                rb[4 * q + 3] = __float_as_uint(__uint_as_float(rb[4 * q + 3]) + v[8 + q].w);
              }
            }
          }
          if (pair_ok && col0 + 64 <= g.N) {
            epilogue_pair_interior(ra, rb, stage, row, row0, rows_valid, col0, g, out, bias_vec, lane, out_map, pre_map);
          } else {
            if (interior_rows && col0 + 32 <= g.N) epilogue_chunk_interior(ra, row, col0, g, out, out_f32, bias_vec);
            else epilogue_chunk_generic(ra, row, col0, g, out, out_f32);
            if (interior_rows && col0 + 64 <= g.N) epilogue_chunk_interior(rb, row, col0 + 32, g, out, out_f32, bias_vec);
            else epilogue_chunk_generic(rb, row, col0 + 32, g, out, out_f32);
          }
        }
      }
      if (part > 0) {  // the parked share is complete: publish it
        __threadfence();
        __syncwarp();
        if (lane == 0) st_release_gpu(my_flags + (part - 1) * 8, 1u);
      } else if (part == 0) {  // leave the flags at zero for the next launch that is handed these words
        __syncwarp();
        if (lane < splits - 1) my_flags[lane * 8] = 0u;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    drain_stores(lane);
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------------ CTA-pair kernel
// The same GEMM with tcgen05.mma.cta_group::2: two CTAs of a cluster, on neighbouring SMs, compute one
// 256 x BN tile together.  Each CTA loads its own 128 rows of A and HALF of the B tile (BN/2 rows), and the
// leader's MMA instructions read B from both CTAs' shared memory, so per flop each SM moves a third less
// operand data through TMA and reads a third less of it from shared memory than the 128 x 256 single-CTA
// tile -- the resource that bounds the single-CTA kernel.  Roles per CTA are the same as above (warp 0 TMA
// producer, warp 1 MMA issuer in the leader only, warps 2-9 epilogue of this CTA's 128 accumulator rows).
//   full[s]       leader's barrier: one arrive.expect_tx by the leader's producer + the bytes of BOTH CTAs' loads
//   empty[s]      each CTA's own barrier, signalled in both by one multicast tcgen05.commit
//   acc_full[b]   each CTA's own barrier, signalled in both by one multicast tcgen05.commit
//   acc_empty[b]  leader's barrier: 16 arrivals, one per epilogue warp of either CTA
// No TMA load uses multicast: each CTA reads its own tiles from global memory.
template <int BN>
struct PairLayout {
  static constexpr int A_BYTES = 128 * BK * 2;       // this CTA's 128 rows of the 256-row A tile
  static constexpr int B_BYTES = (BN / 2) * BK * 2;  // this CTA's half of the B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES > 8 ? 8 : SMEM_BUDGET / STAGE_BYTES;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_STAGING + 1024 /* alignment slack */ + 256 /* barriers */;
  static constexpr int THREADS = 64 + 256;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1)
k_gemm_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_out,
            const __grid_constant__ CUtensorMap map_pre, const GemmArgs g) {
  const CUtensorMap* out_map = g.tma_store ? &map_out : nullptr;
  const CUtensorMap* pre_map = g.tma_store ? &map_pre : nullptr;
  extern __shared__ uint8_t smem_raw[];
  using L = PairLayout<BN>;
  constexpr int STAGES = L::STAGES;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * L::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + EPI_STAGING);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: the leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (g.M + 255) / 256, tiles_n = (g.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (g.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators of BN fp32 columns

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 16);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tb::pdl_launch_dependents();
  tc_fence_before();
  cluster_sync_all();  // both CTAs' barriers are initialised before either one signals the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  tb::pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile % tiles_m) * 256 + (int)rank * 128;
        const int n0 = (tile / tiles_m) * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&empty[s], phase ^ 1, g.error))) break;
          uint8_t* a_dst = smem + s * L::STAGE_BYTES;
          uint8_t* b_dst = a_dst + L::A_BYTES;
          if (rank == 0) mbar_expect_tx(&full[s], 2 * L::STAGE_BYTES);
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d_pair(a_dst, &map_a, bar, k0, m0);  // box {64 k, 128 rows}
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(a_dst + j * 8192, &map_a, bar, m0 + j * 64, k0);  // box {64 m, 64 k}
          }
          if (!B_MN) {
            tma_load_2d_pair(b_dst, &map_b, bar, k0, n0);  // box {64 k, BN/2 rows}
          } else {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) tma_load_2d_pair(b_dst + j * 8192, &map_b, bar, n0 + j * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = instr_desc(256, BN, A_MN, B_MN);
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
        const uint32_t buf = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&full[s], phase, g.error))) break;
          tc_fence_after();
          if (kb == 0) {  // both CTAs' epilogues have drained this accumulator
            if (!(ok = mbar_wait(&acc_empty[buf], acc_phase ^ 1, g.error))) break;
            tc_fence_after();
          }
          const uint32_t a_addr = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t b_addr = a_addr + L::A_BYTES;
          const uint64_t a_desc = A_MN ? smem_desc(a_addr, 8192, 1024) : smem_desc(a_addr, 16, 1024);
          const uint64_t b_desc = B_MN ? smem_desc(b_addr, 8192, 1024) : smem_desc(b_addr, 16, 1024);
          const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t a_k = a_desc + (uint64_t)((A_MN ? 2048 : 32) * k >> 4);
            const uint64_t b_k = b_desc + (uint64_t)((B_MN ? 2048 : 32) * k >> 4);
            mma_bf16_pair(d_tmem, a_k, b_k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit_pair(&empty[s], 3);  // both CTAs may refill the stage once these MMAs have read it
        }
        if (ok) mma_commit_pair(&acc_full[buf], 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2 .. 9, both CTAs)
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    uint32_t local_tile = 0;
    bool ok = true;
    const bool out_f32 = g.flags & EPI_OUT_F32;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
      const int m0 = (tile % tiles_m) * 256 + (int)rank * 128;
      const int n0 = (tile / tiles_m) * BN;
      const uint32_t buf = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      ok = mbar_wait_warp(&acc_full[buf], acc_phase, g.error);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      const bool interior_rows = row < g.M && (g.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(g.out) & 15) == 0;
      const bool bias_vec = (g.flags & EPI_BIAS) && (reinterpret_cast<uintptr_t>(g.bias) & 15) == 0;
      constexpr int CHUNKS = BN / 32;
      const int c_begin = group * (CHUNKS / 2), c_end = c_begin + CHUNKS / 2;
      {
        uint32_t ra[32], rb[32];
        uint8_t* stage = staging + (warp - 2) * 4096;
        const int row0 = m0 + quarter * 32;
        const int rows_valid = g.M - row0 < 32 ? g.M - row0 : 32;
        const bool pair_ok = !out_f32 && (g.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(g.out) & 15) == 0 && rows_valid > 0 &&
                             !((g.flags & EPI_ACCUMULATE) && (g.flags & (EPI_RESIDUAL | EPI_DGELU)));
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 2) {
          tmem_ld32(taddr + c * 32, ra);
          tmem_ld32(taddr + (c + 1) * 32, rb);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (pair_ok && col0 + 64 <= g.N) {
            epilogue_pair_interior(ra, rb, stage, row, row0, rows_valid, col0, g, g.out, bias_vec, lane, out_map, pre_map);
          } else {
            if (interior_rows && col0 + 32 <= g.N) epilogue_chunk_interior(ra, row, col0, g, g.out, out_f32, bias_vec);
            else epilogue_chunk_generic(ra, row, col0, g, g.out, out_f32);
            if (interior_rows && col0 + 64 <= g.N) epilogue_chunk_interior(rb, row, col0 + 32, g, g.out, out_f32, bias_vec);
            else epilogue_chunk_generic(rb, row, col0 + 32, g, g.out, out_f32);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
    }
    drain_stores(lane);
  }

  // ------------------------------------------------------------------ teardown
  // Neither CTA may leave (or free TMEM) while its partner can still signal its barriers or read its tiles.
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
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

// Tensor maps for the epilogue's TMA stores: 32-row x 64-column bf16 blocks of out (and of the kept pre-activation).
// Returns 1 if the output qualifies (bf16, 16-byte aligned rows), 0 if the epilogue must store by itself.
int g_tma_store_enabled = 1;
int make_store_maps(CUtensorMap* mo, CUtensorMap* mp, void* out, void* aux_out, int M, int N, int ldc, int flags) {
  memset(mo, 0, sizeof(*mo));
  memset(mp, 0, sizeof(*mp));
  if (!g_tma_store_enabled || (flags & EPI_OUT_F32) || (ldc & 7) || ((uintptr_t)out & 15) || N < 64 || M < 32) return 0;
  const bool keep_pre = (flags & EPI_GELU) && aux_out != nullptr;
  if (keep_pre && ((uintptr_t)aux_out & 15)) return 0;
  if (make_map(mo, out, N, M, ldc, 64, 32)) return 0;
  if (keep_pre && make_map(mp, aux_out, N, M, ldc, 64, 32)) return 0;
  return 1;
}

int* g_error_host = nullptr;
int* g_error_dev = nullptr;
int g_sm_count = 0;

template <int BM, int BN, bool A_MN, bool B_MN>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mp, const GemmArgs& g, int max_ctas,
                cudaStream_t stream) {
  auto kernel = k_gemm<BM, BN, A_MN, B_MN>;
  using L = SmemLayout<BM, BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int out_tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN);
  const int tiles = g.splits > 1 ? g.whole_tiles + (out_tiles - g.whole_tiles) * g.splits : out_tiles;
  int ctas = tiles < g_sm_count ? tiles : g_sm_count;
  if (max_ctas > 0 && ctas > max_ctas) ctas = max_ctas;
  return (int)tb::launch(kernel, dim3(ctas), dim3(L::THREADS), L::TOTAL, stream, ma, mb, mo, mp, g, GatherArgs{});
}


template <int BN, bool A_MN, bool B_MN>
int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mp, const GemmArgs& g,
                     int max_ctas, cudaStream_t stream) {
  auto kernel = k_gemm_pair<BN, A_MN, B_MN>;
  using L = PairLayout<BN>;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(g_sm_count & ~1);
    cfg.blockDim = dim3(L::THREADS);
    cfg.dynamicSmemBytes = L::TOTAL;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = g_sm_count / 2;
    }
    max_pairs = n < g_sm_count / 2 ? n : g_sm_count / 2;
  }
  const int tiles = ((g.M + 255) / 256) * ((g.N + BN - 1) / BN);
  int pairs = tiles < max_pairs ? tiles : max_pairs;
  if (max_ctas > 1 && pairs > max_ctas / 2) pairs = max_ctas / 2;
  kernel<<<2 * pairs, L::THREADS, L::TOTAL, stream>>>(ma, mb, mo, mp, g);
  return (int)cudaGetLastError();
}

// Tile shape and tail split with the least estimated time.  One CTA per SM takes output tiles round-robin; the last,
// partial round leaves SMs idle, so the tiles of that round ("tail") may have their reduction cut into parts that are
// spread over the idle SMs (GemmArgs).  The estimate, in microseconds, is
//     start-up + full rounds x (k-blocks x per-k-block + per-tile) + [tail: k-blocks per part x per-k-block + per-tile + fold]
// with constants fitted to sweeps on B200 (bench/bench_gemm.py --sweep, CUDA-graph timing, cold L2): a k-block costs
// 0.34 - 0.43 us on the 128-row tiles whatever their width (the main loop is bound by bytes in flight / load latency,
// not by the tensor pipe) and 0.77 us on the 256 x 256 tile, whose two accumulators fill TMEM so that its epilogue
// (about 5 us) cannot overlap the next tile; a kernel's start-up and drain cost about 5 us; folding parked partial
// tiles costs about 2.5 us plus 1.7 us per extra part (producer drain, flag, one trip to L2 per part) plus 0.3 us per
// parked megabyte.  With those prices the split pays where a round of tiles is less than about half full and the
// reduction is long: the weight gradients (K = tokens) and, at 1024 - 2048 tokens, the K = 3072 products.
struct TileShape { int id, bm, bn; double per_kblock, per_tile; };
constexpr TileShape SHAPES[4] = {{0, 256, 256, 0.77, 5.3}, {1, 128, 256, 0.43, 0.5}, {2, 128, 128, 0.34, 0.6}, {5, 128, 192, 0.41, 0.6}};
constexpr int MAX_SPLITS = 8;
constexpr double START_US = 5.0, FOLD_US = 2.5, FOLD_PART_US = 1.7, FOLD_US_PER_MB = 0.3;

// Tuning and test hooks (tb_gemm_force_tile / tb_gemm_force_splits): process-wide, read once per call into locals.
// Atomic so that a setter racing with a launch on another thread (an autograd worker) yields one value or the other.
std::atomic<int> g_forced_tile{-1};   // 0: 256x256, 1: 128x256, 2: 128x128, 3 / 4: CTA pair 256x256 / 256x128, 5: 128x192; -1: planned
std::atomic<int> g_forced_splits{0};  // > 0: that many k-parts for the tail (where the reduction is long enough); 0: planned

struct GemmPlan { int bm, bn, splits, whole_tiles; };

GemmPlan plan_gemm(int M, int N, int K, int ctas) {
  const int k_blocks = (K + BK - 1) / BK;
  const int forced_tile = g_forced_tile.load(std::memory_order_relaxed), forced_splits = g_forced_splits.load(std::memory_order_relaxed);
  if (forced_tile == 3 || forced_tile == 4) return {512, forced_tile == 3 ? 256 : 128, 1, 0};  // CTA-pair kernel (bm = 512 marks it)
  auto valid_splits = [&](int s) {  // every part gets at least two k-blocks and none is empty
    const int per = (k_blocks + s - 1) / s;
    return s == 1 || (per >= 2 && (s - 1) * per < k_blocks);
  };
  GemmPlan best{128, 128, 1, 0};
  double best_us = 1e300;
  for (const TileShape& t : SHAPES) {
    if (forced_tile >= 0 && forced_tile != t.id) continue;
    if (forced_tile < 0 && t.bn > 128 && N <= 128) continue;
    const long long tiles = (long long)((M + t.bm - 1) / t.bm) * ((N + t.bn - 1) / t.bn);
    const long long rounds = tiles / ctas, tail = tiles % ctas;
    const double whole_us = rounds * (k_blocks * t.per_kblock + t.per_tile);
    for (int sp = 1; sp <= MAX_SPLITS; ++sp) {
      if (!valid_splits(sp) || (sp > 1 && (tail == 0 || tail * sp > ctas))) continue;
      if (forced_splits > 0 && sp != forced_splits && tail > 0 && valid_splits(forced_splits) && tail * forced_splits <= ctas) continue;
      double us = START_US + whole_us;
      if (tail > 0) {
        const int per = (k_blocks + sp - 1) / sp;
        us += per * t.per_kblock + t.per_tile;
        if (sp > 1) us += FOLD_US + FOLD_PART_US * (sp - 1) + FOLD_US_PER_MB * (double)tail * (sp - 1) * t.bm * t.bn * 4 / 1e6;
      }
      if (us < best_us - 1e-9) {
        best_us = us;
        best = {t.bm, t.bn, sp, (int)(rounds * ctas)};
      }
    }
  }
  if (best.splits == 1) best.whole_tiles = 0;
  return best;
}

// Flag words for split-K, handed out round-robin to launches (a launch that is handed words still in use by an earlier
// one would need a pool's worth of launches in flight at once); all zero between launches.
constexpr int SPLIT_FLAG_POOL = 1 << 16;
__device__ unsigned g_split_flags[SPLIT_FLAG_POOL];

}  // namespace

extern "C" void tb_note_launch(int n);

extern "C" {

// 0 while every GEMM wait so far has completed; 1 after one ran out.
int tb_gemm_error() { return g_error_host != nullptr ? *g_error_host : 0; }

// D[M,N] = op(A) . op(B) with bf16 operands, then the epilogue selected by `flags` (EpilogueFlags).
//   a_mn == 0: A is [M, K] with leading dimension lda (K contiguous); a_mn == 1: A is [K, M], lda (M contiguous).
//   b_mn == 0: B is [N, K] with leading dimension ldb (K contiguous); b_mn == 1: B is [K, N], ldb (N contiguous).
// Leading dimensions must be multiples of 8 elements and base pointers 16-byte aligned (TMA).
int tb_gemm_bf16(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int flags,
                 const void* bias, const void* aux_in, void* aux_out, int max_ctas, void* workspace, long long workspace_bytes,
                 cudaStream_t stream) {
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
  const int ctas = max_ctas > 0 && max_ctas < g_sm_count ? max_ctas : g_sm_count;
  const GemmPlan plan = plan_gemm(M, N, K, ctas);
  const int BM = plan.bm, BN = plan.bn;
  int splits = plan.splits;
  const bool paired = BM == 512;  // a 256 x BN tile shared by a CTA pair: per CTA 128 rows of A, BN/2 rows of B
  unsigned* split_flags = nullptr;
  if (splits > 1) {
    const long long tiles = (long long)((M + BM - 1) / BM) * ((N + BN - 1) / BN), tail = tiles - plan.whole_tiles;
    const long long need = tail * (splits - 1) * BM * BN * 4, words = tail * (splits - 1) * 8;
    if (workspace == nullptr || workspace_bytes < need || ((uintptr_t)workspace & 15) || words > SPLIT_FLAG_POOL) {
      splits = 1;  // no room to park partial tiles: compute unsplit (same result up to summation order)
    } else {
      static unsigned* pool = nullptr;
      static int pool_device = -1;
      static long long next = 0;
      int dev = 0;
      cudaGetDevice(&dev);
      if (pool == nullptr || pool_device != dev) {
        if (cudaGetSymbolAddress((void**)&pool, g_split_flags) != cudaSuccess) return (int)cudaGetLastError();
        pool_device = dev;
      }
      if (next + words > SPLIT_FLAG_POOL) next = 0;
      split_flags = pool + next;
      next += words;
    }
  }
  CUtensorMap ma, mb;
  int rc;
  if (!a_mn) rc = make_map(&ma, A, K, M, lda, 64, paired ? 128 : BM);
  else rc = make_map(&ma, A, M, K, lda, 64, 64);
  if (rc) return rc;
  if (!b_mn) rc = make_map(&mb, B, K, N, ldb, 64, paired ? BN / 2 : BN);
  else rc = make_map(&mb, B, N, K, ldb, 64, 64);
  if (rc) return rc;
  CUtensorMap mo, mp;
  const int tma_store = make_store_maps(&mo, &mp, out, aux_out, M, N, ldc, flags);
  GemmArgs g{M, N, K, ldc, flags, out, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)aux_in, (__nv_bfloat16*)aux_out, g_error_dev, tma_store,
             splits, splits > 1 ? plan.whole_tiles : 0, (float*)workspace, split_flags};
  tb_note_launch(1);
#define GO2(BN_) \
  do { \
    if (!a_mn && !b_mn) return launch_gemm_pair<BN_, false, false>(ma, mb, mo, mp, g, max_ctas, stream); \
    if (!a_mn && b_mn) return launch_gemm_pair<BN_, false, true>(ma, mb, mo, mp, g, max_ctas, stream); \
    if (a_mn && b_mn) return launch_gemm_pair<BN_, true, true>(ma, mb, mo, mp, g, max_ctas, stream); \
    return launch_gemm_pair<BN_, true, false>(ma, mb, mo, mp, g, max_ctas, stream); \
  } while (0)
  if (paired && BN == 256) GO2(256);
  if (paired) GO2(128);
#undef GO2
#define GO(BM_, BN_) \
  do { \
    if (!a_mn && !b_mn) return launch_gemm<BM_, BN_, false, false>(ma, mb, mo, mp, g, max_ctas, stream); \
    if (!a_mn && b_mn) return launch_gemm<BM_, BN_, false, true>(ma, mb, mo, mp, g, max_ctas, stream); \
    if (a_mn && b_mn) return launch_gemm<BM_, BN_, true, true>(ma, mb, mo, mp, g, max_ctas, stream); \
    return launch_gemm<BM_, BN_, true, false>(ma, mb, mo, mp, g, max_ctas, stream); \
  } while (0)
  if (BM == 256) GO(256, 256);
  if (BN == 256) GO(128, 256);
  if (BN == 192) GO(128, 192);
  GO(128, 128);
#undef GO
}

// Bytes of workspace tb_gemm_bf16 wants for this problem (0: it will not split the reduction).  The caller allocates
// at least that much (any stream-ordered allocator will do: the kernel is done with it when it completes) and passes it.
long long tb_gemm_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (g_sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      g_sm_count = 0;
    cudaGetLastError();
  }
  const GemmPlan plan = plan_gemm(M, N, K, g_sm_count > 0 ? g_sm_count : 148);
  if (plan.splits <= 1) return 0;
  const long long tiles = (long long)((M + plan.bm - 1) / plan.bm) * ((N + plan.bn - 1) / plan.bn);
  return (tiles - plan.whole_tiles) * (plan.splits - 1) * plan.bm * plan.bn * 4;
}

// What the planner picks: writes {BM (512: CTA pair), BN, parts the tail tiles are cut into, tiles computed whole}.
void tb_gemm_plan(int M, int N, int K, int* out4) {
  if (g_sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      g_sm_count = 0;
    cudaGetLastError();
  }
  // without a device (a build machine) the plan is the one a B200's 148 SMs would get
  const GemmPlan plan = plan_gemm(M, N, K, g_sm_count > 0 ? g_sm_count : 148);
  out4[0] = plan.bm;
  out4[1] = plan.bn;
  out4[2] = plan.splits;
  out4[3] = plan.whole_tiles;
}

// Pins the number of k-parts (0: planned) / the tile shape (-1: planned) for every later call.  For tuning and tests.
void tb_gemm_force_splits(int n) { g_forced_splits.store(n, std::memory_order_relaxed); }

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
  // 256-row tiles (two MMAs per weight panel in shared memory: a third less operand traffic per flop) once the problem
  // has enough of them for every SM; 128-row tiles otherwise.  The weight panel is 256 columns wide in both.
  constexpr int BN = 256;
  const int tiles_n = (N + BN - 1) / BN;
  const bool tall = (long long)((M + 255) / 256) * tiles_n >= g_sm_count;
  const int BM = tall ? 256 : 128;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, A, K, M, lda, 64, BM);
  if (rc) return rc;
  rc = make_map(&mb, (const char*)full + w_off, K, N, K, 64, BN);
  if (rc) return rc;
  CUtensorMap mo, mp;
  const int tma_store = make_store_maps(&mo, &mp, out, aux_out, M, N, ldc, flags);
  GemmArgs g{M, N, K, ldc, flags, out, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)aux_in, (__nv_bfloat16*)aux_out, g_error_dev, tma_store,
             1, 0, nullptr, nullptr};
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
  ga.n_start = ((n_start % tiles_n) + tiles_n) % tiles_n;
  const void* kernel = tall ? (const void*)k_gemm<256, BN, false, false, true> : (const void*)k_gemm<128, BN, false, false, true>;
  const int smem = tall ? SmemLayout<256, BN>::TOTAL : SmemLayout<128, BN>::TOTAL;
  static bool configured[2] = {false, false};
  if (!configured[tall]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured[tall] = true;
  }
  const int tiles = ((M + BM - 1) / BM) * tiles_n;
  int ctas = tiles < g_sm_count ? tiles : g_sm_count;
  void* params[] = {(void*)&ma, (void*)&mb, (void*)&mo, (void*)&mp, (void*)&g, (void*)&ga};
  tb_note_launch(1);
  return (int)cudaLaunchCooperativeKernel(kernel, dim3(ctas), dim3(448), params, smem, stream);
}

void tb_gemm_force_tile(int which) { g_forced_tile.store(which, std::memory_order_relaxed); }

// 1 (default): bf16 outputs leave through TMA stores; 0: the epilogue warps store them.  For measurements.
void tb_gemm_tma_store(int on) { g_tma_store_enabled = on; }

const char* tb_gemm_last_error() { return g_map_error; }

}  // extern "C"
