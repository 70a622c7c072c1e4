// Causal self-attention on tcgen05 / TMEM, forward and backward, over a packed qkv tensor.
//
// qkv is [B*T, 3*d] bf16 (q | k | v along the row, head h at columns h*HD .. h*HD+HD of each part), T a
// multiple of 128, HD 64 or 128.  One TMA tensor map over that matrix serves every tile load
// (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast): a 128-row x 64-column box is a K-major
// operand when the reduction runs over the head dimension (Q.K^T, dO.V^T) and, with the same bytes,
// an MN-major operand when it runs over the rows (P.V, P^T.dO, dS^T.Q, dS.K).
//
// Three warp-specialised kernels (one TMA producer warp, one MMA-issuing thread, eight element-wise warps):
//   k_attn_fwd_ws    two 128-query tiles per CTA alternate on the tensor pipe; single pass, online softmax with a lazy
//                    rescale of the accumulator in TMEM; P stays in TMEM as the A operand of P.V
//   k_attn_bwd_dq    per query tile: S, dP -> dS (TMEM) -> dQ += dS.K; also produces delta = rowsum(dO * O)
//   k_attn_bwd_dkv   per key tile, transposed scores: P^T, dS^T (TMEM) -> dV += P^T.dO, dK += dS^T.Q
// Probabilities and score gradients never pass through shared memory, nothing is accumulated with atomics, and
// the results do not depend on scheduling.  Consecutive CTAs work on the same head so its K and V stay in L2.
//
// Every wait is bounded (tcgen05.cuh); on expiry the CTA raises the host-visible error word, frees its
// TMEM and returns.  The reference calls torch's scaled_dot_product_attention (tandem/model.py:43).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "launch.cuh"
#include "tcgen05.cuh"

extern "C" void tb_note_launch(int n);

namespace {

using namespace tc;

constexpr int TILE = 128;           // queries per CTA, keys per step
constexpr int STRIP = TILE * 128;   // bytes of one 128-row x 64-column bf16 strip (128-byte rows)

// Loads one [128 rows x HD cols] operand tile (HD/64 strips) whose first element is (row, col) of qkv.
template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int col, int row) {
#pragma unroll
  for (int s = 0; s < HD / 64; ++s) tma_load_2d(dst + s * STRIP, map, bar, col + s * 64, row);
}

// D[128, N] (+)= A[128, K=HD] . B[N=128, K=HD]^T with both operands K-major strips.
template <int HD>
__device__ __forceinline__ void mma_kmajor(uint32_t d_tmem, const uint8_t* a, const uint8_t* b, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int s = 0; s < HD / 64; ++s)
#pragma unroll
    for (int k = 0; k < 4; ++k)
      mma_bf16(d_tmem, smem_desc(smem_u32(a + s * STRIP) + k * 32, 16, 1024), smem_desc(smem_u32(b + s * STRIP) + k * 32, 16, 1024),
               idesc, (accumulate || s > 0 || k > 0) ? 1u : 0u);
}

// ------------------------------------------------------------------------------------------ forward, warp-specialised
// One CTA per PAIR of 128-query tiles of one head, 320 threads in four roles:
//   warp 0       TMA producer: both Q tiles once, then K_0, V_0, K_1, V_1, ... through a ring of tile slots
//   warp 1       MMA issuer (one thread): S_i = Q_i.K_j^T and O_i += P_i.V_j for the two query tiles i in turn
//   warps 2-5    softmax of query tile 0: one thread per query row (= TMEM lane)
//   warps 6-9    softmax of query tile 1
// Single pass with an online softmax: a row keeps the maximum it is currently scaled by (m_used) and only rescales its
// accumulator row in TMEM (tcgen05.ld, multiply, tcgen05.st) when a new maximum exceeds it by more than 2^8; otherwise
// the probabilities simply run up to 256, which fp32 accumulation and bf16 probabilities absorb.  The rescale needs no
// barrier of its own: S_i(j) is committed after O_i += P.V of step j-1 on the in-order tensor pipe, and the next one is
// only issued after this row's thread has arrived on p_full.
// The two tiles alternate on the tensor pipe: while the softmax threads of one tile work on S_i(j) (exponentials), the
// MMAs of the other tile run.  P stays in TMEM: it is written as bf16 pairs over the first 64 columns of S and is the
// A operand of a TMEM-sourced MMA (measured against staging P in shared memory: 198 vs 223 us at T = 2048, head dim 128).
// TMEM: S_0 [0,128)  S_1 [128,256)  O_0 [256,256+HD)  O_1 [256+HD, 256+2HD).
template <int HD>
struct Fwd2Smem {
  static constexpr int TILE_BYTES = (HD / 64) * STRIP;
  static constexpr int Q = 0;                                       // two query tiles
  static constexpr int RING = Q + 2 * TILE_BYTES;
  static constexpr int BUDGET = 224 * 1024;
  static constexpr int SLOTS_FIT = (BUDGET - RING) / TILE_BYTES;
  static constexpr int SLOTS = SLOTS_FIT > 6 ? 6 : SLOTS_FIT;       // K and V tiles in flight
  static constexpr int BARS = RING + SLOTS * TILE_BYTES;
  static constexpr int TOTAL = BARS + 256;
  static_assert(SLOTS >= 3, "the K/V ring needs at least three slots");
};

template <int HD>
__global__ void __launch_bounds__(320, 1)
k_attn_fwd_ws(const __grid_constant__ CUtensorMap map, __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int B, int T, int H,
              int d, float scale_log2e, int* error) {
  extern __shared__ __align__(1024) uint8_t fwd2_smem[];
  uint8_t* smem = fwd2_smem;
  if (smem_u32(smem) & 1023) {  // the swizzled tiles need 1024-byte alignment; nothing is allocated yet
    if (threadIdx.x == 0) {
      *error = 1;
      __threadfence_system();
    }
    return;
  }
  using L = Fwd2Smem<HD>;
  constexpr int TILE_BYTES = L::TILE_BYTES, SLOTS = L::SLOTS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
  uint64_t *q_full = bars, *s_full = bars + 2, *p_full = bars + 4, *o_full = bars + 6, *kv_full = bars + 8, *kv_empty = bars + 8 + SLOTS;
  uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 8 + 2 * SLOTS);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_qt = T / TILE, n_pairs = (n_qt + 1) / 2;
  // consecutive CTAs share one head's K and V (they stay in L2), longest pair first within the head
  const int pair = n_pairs - 1 - (int)blockIdx.x % n_pairs;
  const int rest = (int)blockIdx.x / n_pairs;
  const int h = rest % H, b = rest / H;
  const int qt0 = 2 * pair, qt1 = 2 * pair + 1;
  const int n0 = qt0 + 1, n1 = qt1 < n_qt ? qt1 + 1 : 0;  // key tiles each query tile visits
  const int n_steps = n1 > n0 ? n1 : n0;
  constexpr uint32_t TMEM_COLS = 512;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);  // one arrival per softmax warp of the tile
      mbar_init(&o_full[i], 1);
    }
    for (int s = 0; s < SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tensormap(&map);
  }
  if (warp == 1) {
    tmem_alloc(holder, TMEM_COLS);
    tmem_relinquish();
  }
  tb::pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *holder;
  tb::pdl_wait();  // set-up is done; everything below reads what earlier kernels wrote

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&q_full[0], TILE_BYTES);
      load_tile<HD>(smem + L::Q, &map, &q_full[0], h * HD, b * T + qt0 * TILE);
      if (n1) {
        mbar_expect_tx(&q_full[1], TILE_BYTES);
        load_tile<HD>(smem + L::Q + TILE_BYTES, &map, &q_full[1], h * HD, b * T + qt1 * TILE);
      }
      bool ok = true;
      for (int ld = 0; ld < 2 * n_steps && ok; ++ld) {  // load 2j: K_j, load 2j+1: V_j
        const int s = ld % SLOTS, j = ld >> 1, part = ld & 1;
        if (!(ok = mbar_wait(&kv_empty[s], ((ld / SLOTS) & 1) ^ 1, error))) break;
        mbar_expect_tx(&kv_full[s], TILE_BYTES);
        load_tile<HD>(smem + L::RING + s * TILE_BYTES, &map, &kv_full[s], (1 + part) * d + h * HD, b * T + j * TILE);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc(128, 128, false, false);
      constexpr uint32_t idesc_o = instr_desc(128, HD, false, true);
      auto slot_of = [&](int ld) { return smem + L::RING + (ld % SLOTS) * TILE_BYTES; };
      auto wait_slot = [&](int ld) { return mbar_wait(&kv_full[ld % SLOTS], (ld / SLOTS) & 1, error); };
      auto issue_s = [&](int i, int j) {  // S_i = Q_i . K_j^T
        mma_kmajor<HD>(tmem + i * 128, smem + L::Q + i * TILE_BYTES, slot_of(2 * j), idesc_s, false);
        mma_commit(&s_full[i]);
      };
      auto issue_pv = [&](int i, int j) {  // O_i (+)= P_i . V_j: eight steps of 16 keys; V is MN-major (head dim contiguous)
        const uint32_t tO = tmem + 256 + i * HD;
        const uint32_t v_addr = smem_u32(slot_of(2 * j + 1));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t v_desc = smem_desc(v_addr + kk * 2048, STRIP, 1024);
          mma_bf16_ts(tO, tmem + i * 128 + kk * 8, v_desc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);  // 16 keys = 8 TMEM columns of P
        }
      };
      bool ok = mbar_wait(&q_full[0], 0, error) && (!n1 || mbar_wait(&q_full[1], 0, error)) && wait_slot(0);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        if (n1) issue_s(1, 0);
        mma_commit(&kv_empty[0]);  // K_0 is free once these have read it
      }
      for (int j = 0; j < n_steps && ok; ++j) {
        if (!(ok = wait_slot(2 * j + 1))) break;                       // V_j
        if (j + 1 < n_steps && !(ok = wait_slot(2 * j + 2))) break;    // K_{j+1}
        tc_fence_after();
        for (int i = 0; i < 2 && ok; ++i) {
          const int n_i = i == 0 ? n0 : n1;
          if (j >= n_i) continue;
          if (!(ok = mbar_wait(&p_full[i], j & 1, error))) break;      // P_i(j) is in place, O_i rescaled if it had to be
          tc_fence_after();
          issue_pv(i, j);
          if (j == n_i - 1) mma_commit(&o_full[i]);
          else issue_s(i, j + 1);
        }
        if (!ok) break;
        mma_commit(&kv_empty[(2 * j + 1) % SLOTS]);                    // V_j
        if (j + 1 < n_steps) mma_commit(&kv_empty[(2 * j + 2) % SLOTS]);  // K_{j+1}
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax (warps 2-5: tile 0, warps 6-9: tile 1)
    const int i = (warp - 2) >> 2;
    const int n_i = i == 0 ? n0 : n1;
    const int qt = i == 0 ? qt0 : qt1;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                      // query row within the tile = TMEM lane
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + i * 128 + lane_base;
    const uint32_t tO = tmem + 256 + i * HD + lane_base;
    float m_used = -INFINITY, l = 0.f;  // m_used in raw score units
    bool ok = true;
    for (int j = 0; j < n_i && ok; ++j) {
      if (!(ok = mbar_wait_warp_spin(&s_full[i], j & 1, error))) break;
      tc_fence_after();
      uint32_t raw[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, raw[c]);
      tmem_ld_wait();
      float mx = -INFINITY;
      if (j == qt) {  // the diagonal tile: keys beyond the query are masked
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (c * 32 + e > r) raw[c][e] = 0xff800000u;  // -inf
      }
      {
        // eight independent running maxima: a single chain of 128 dependent FMNMX would cost ~5 cycles each
        float part[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) part[e] = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) part[e & 7] = fmaxf(part[e & 7], __uint_as_float(raw[c][e]));
        mx = fmaxf(fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])), fmaxf(fmaxf(part[4], part[5]), fmaxf(part[6], part[7])));
      }
      if (j == 0) {
        m_used = mx;
      } else {
        const bool need = (mx - m_used) * scale_log2e > 8.f;
        if (__any_sync(0xffffffffu, need)) {  // rare after the first tiles: rescale this warp's accumulator rows
          const float f = need ? ex2_approx((m_used - mx) * scale_log2e) : 1.f;
          if (need) m_used = mx;
          l *= f;
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tO + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
            tmem_st32(tO + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      const float mc = m_used * scale_log2e;
      float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {  // 64 keys at a time: 32 registers of bf16 pairs
        uint32_t pk[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int col = hh * 64 + 2 * e;
          const float p0 = ex2_approx(fmaf(__uint_as_float(raw[col >> 5][col & 31]), scale_log2e, -mc));
          const float p1 = ex2_approx(fmaf(__uint_as_float(raw[(col + 1) >> 5][(col + 1) & 31]), scale_log2e, -mc));
          sums[(2 * e) & 3] += p0;
          sums[(2 * e + 1) & 3] += p1;
          const __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
          pk[e] = *reinterpret_cast<const uint32_t*>(&pp);
        }
        tmem_st32(tS + hh * 32, pk);  // P over the first 64 columns of S: keys 2c, 2c+1 in column c
      }
      l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[i]);
    }
    if (ok && n_i > 0) ok = mbar_wait_warp_spin(&o_full[i], 0, error);
    if (ok && n_i > 0) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      const int q_idx = qt * TILE + r;
      __nv_bfloat16* o_row = out + (size_t)(b * T + q_idx) * d + h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          __nv_bfloat162 y[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            y[e] = __floats2bfloat162_rn(__uint_as_float(o[v * 8 + 2 * e]) * inv_l, __uint_as_float(o[v * 8 + 2 * e + 1]) * inv_l);
          *reinterpret_cast<uint4*>(o_row + c * 32 + v * 8) = *reinterpret_cast<const uint4*>(y);
        }
      }
      lse[((size_t)b * H + h) * T + q_idx] = (m_used * scale_log2e + log2f(l)) * 0.69314718055994530942f;  // natural log
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------ backward, warp-specialised
// Two kernels, no atomics: k_attn_bwd_dq owns a tile of 128 queries and walks the key tiles at or below the
// diagonal (dQ accumulates in TMEM); k_attn_bwd_dkv owns a tile of 128 keys and walks the query tiles at or above it
// (dK and dV accumulate in TMEM).  Both recompute S and dP; results are deterministic.  Roles per CTA (320 threads):
// warp 0 TMA producer, warp 1 MMA issuer (one thread), warps 2-9 element-wise work, two threads per TMEM lane (warps
// w and w + 4 share a lane quarter and split the 128 columns).  Probabilities and dS never touch shared memory: they
// are written back to TMEM as bf16 pairs and feed the next MMA as its A operand.

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void named_barrier(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// ---- dQ.  Per key tile j <= qt:  S = Q.K_j^T, dP = dO.V_j^T (TMEM) -> dS = P * (dP - delta) * scale as bf16 in TMEM
// (two buffers) -> dQ += dS.K_j.  The S / dP MMAs of tile j+1 are issued as soon as the element-wise warps have pulled
// tile j into registers, so the tensor pipe works on j+1 while they compute dS(j).  The kernel also produces
// delta[row] = sum_c dO[row, c] * O[row, c] for its queries (needed here and by the dK/dV kernel, which runs after it).
// TMEM: S [0,128)  dP [128,256)  dQ [256,256+HD)  dS buffers [256+HD, +64) and [320+HD, +64).
template <int HD>
struct BwdDqSmem {
  static constexpr int TILE_BYTES = (HD / 64) * STRIP;
  static constexpr int Q = 0, DO = TILE_BYTES, RING = 2 * TILE_BYTES;
  static constexpr int SLOTS_FIT = (225 * 1024 - RING) / TILE_BYTES;
  static constexpr int SLOTS = SLOTS_FIT > 6 ? 6 : SLOTS_FIT;
  static constexpr int DELTA = RING + SLOTS * TILE_BYTES;  // [2 halves][128 rows] floats
  static constexpr int BARS = DELTA + 1024;
  static constexpr int TOTAL = BARS + 256;
  static_assert(SLOTS >= 4, "K_j, V_j, K_j+1 and V_j+1 are in flight together");
};

template <int HD>
__global__ void __launch_bounds__(320, 1)
k_attn_bwd_dq(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do, const __nv_bfloat16* __restrict__ o,
              const __nv_bfloat16* __restrict__ d_o, const float* __restrict__ lse, float* __restrict__ delta_out,
              __nv_bfloat16* __restrict__ dqkv, int B, int T, int H, int d, float scale, int* error) {
  extern __shared__ __align__(1024) uint8_t dq_smem[];
  uint8_t* smem = dq_smem;
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) {
      *error = 1;
      __threadfence_system();
    }
    return;
  }
  using L = BwdDqSmem<HD>;
  constexpr int TILE_BYTES = L::TILE_BYTES, SLOTS = L::SLOTS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
  uint64_t *qdo_full = bars, *sdp_full = bars + 1, *sdp_read = bars + 2, *ds_full = bars + 3 /* [2] */, *dq_full = bars + 5,
           *kv_full = bars + 6, *kv_empty = bars + 6 + SLOTS;
  uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 6 + 2 * SLOTS);
  float* delta_sm = reinterpret_cast<float*>(smem + L::DELTA);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_qt = T / TILE;
  const int qt = n_qt - 1 - (int)blockIdx.x % n_qt;  // consecutive CTAs share a head (its K, V stay in L2); longest first
  const int rest = (int)blockIdx.x / n_qt;
  const int h = rest % H, b = rest / H;
  const int n = qt + 1;  // key tiles
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t C_S = 0, C_DP = 128, C_DQ = 256, C_DS = 256 + HD;

  if (tid == 0) {
    mbar_init(qdo_full, 1);
    mbar_init(sdp_full, 1);
    mbar_init(sdp_read, 8);
    mbar_init(&ds_full[0], 8);
    mbar_init(&ds_full[1], 8);
    mbar_init(dq_full, 1);
    for (int s = 0; s < SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tensormap(&map_qkv);
    prefetch_tensormap(&map_do);
  }
  if (warp == 1) {
    tmem_alloc(holder, TMEM_COLS);
    tmem_relinquish();
  }
  tb::pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *holder;
  tb::pdl_wait();  // set-up is done; everything below reads what earlier kernels wrote

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(qdo_full, 2 * TILE_BYTES);
      load_tile<HD>(smem + L::Q, &map_qkv, qdo_full, h * HD, b * T + qt * TILE);
      load_tile<HD>(smem + L::DO, &map_do, qdo_full, h * HD, b * T + qt * TILE);
      bool ok = true;
      for (int ld = 0; ld < 2 * n && ok; ++ld) {  // load 2j: K_j, load 2j+1: V_j
        const int s = ld % SLOTS, j = ld >> 1, part = ld & 1;
        if (!(ok = mbar_wait(&kv_empty[s], ((ld / SLOTS) & 1) ^ 1, error))) break;
        mbar_expect_tx(&kv_full[s], TILE_BYTES);
        load_tile<HD>(smem + L::RING + s * TILE_BYTES, &map_qkv, &kv_full[s], (1 + part) * d + h * HD, b * T + j * TILE);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc(128, 128, false, false);
      constexpr uint32_t idesc_dq = instr_desc(128, HD, false, true);
      auto slot_of = [&](int ld) { return smem + L::RING + (ld % SLOTS) * TILE_BYTES; };
      auto wait_slot = [&](int ld) { return mbar_wait(&kv_full[ld % SLOTS], (ld / SLOTS) & 1, error); };
      auto issue_scores = [&](int j) {
        mma_kmajor<HD>(tmem + C_S, smem + L::Q, slot_of(2 * j), idesc_s, false);        // S  = Q . K_j^T
        mma_kmajor<HD>(tmem + C_DP, smem + L::DO, slot_of(2 * j + 1), idesc_s, false);  // dP = dO . V_j^T
        mma_commit(sdp_full);
        mma_commit(&kv_empty[(2 * j + 1) % SLOTS]);  // V_j has no other reader
      };
      bool ok = mbar_wait(qdo_full, 0, error) && wait_slot(0) && wait_slot(1);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      for (int j = 0; j < n && ok; ++j) {
        if (j + 1 < n) {
          if (!(ok = mbar_wait(sdp_read, j & 1, error))) break;  // tile j's S and dP are in registers
          if (!(ok = wait_slot(2 * j + 2) && wait_slot(2 * j + 3))) break;
          tc_fence_after();
          issue_scores(j + 1);
        }
        if (!(ok = mbar_wait(&ds_full[j & 1], (j >> 1) & 1, error))) break;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(slot_of(2 * j));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // dQ += dS . K_j: dS from TMEM (16 keys = 8 columns per step), K_j MN-major over the keys
          mma_bf16_ts(tmem + C_DQ, tmem + C_DS + (j & 1) * 64 + kk * 8, smem_desc(k_addr + kk * 2048, STRIP, 1024), idesc_dq,
                      (j > 0 || kk > 0) ? 1u : 0u);
        mma_commit(&kv_empty[(2 * j) % SLOTS]);
      }
      if (ok) mma_commit(dq_full);
    }
  } else {
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int q_idx = qt * TILE + r;
    const size_t row = (size_t)b * T + q_idx;
    // delta for this row: each of the row's two threads sums half of the head dimension
    {
      constexpr int COLS = HD / 2;
      const __nv_bfloat16* a = o + row * d + h * HD + half * COLS;
      const __nv_bfloat16* g = d_o + row * d + h * HD + half * COLS;
      float acc = 0.f;
#pragma unroll
      for (int c = 0; c < COLS; c += 8) {
        const uint4 av = *reinterpret_cast<const uint4*>(a + c), gv = *reinterpret_cast<const uint4*>(g + c);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = __bfloat1622float2(a2[e]), y = __bfloat1622float2(g2[e]);
          acc = fmaf(x.x, y.x, acc);
          acc = fmaf(x.y, y.y, acc);
        }
      }
      delta_sm[half * TILE + r] = acc;
    }
    named_barrier(1, 256);
    const float delta = delta_sm[r] + delta_sm[TILE + r];
    if (half == 0) delta_out[((size_t)b * H + h) * T + q_idx] = delta;
    const float c2 = scale * 1.4426950408889634f;
    const float neg_lse2 = -lse[((size_t)b * H + h) * T + q_idx] * 1.4426950408889634f;
    bool ok = true;
    for (int j = 0; j < n && ok; ++j) {
      if (!(ok = mbar_wait_warp_spin(sdp_full, j & 1, error))) break;
      tc_fence_after();
      uint32_t s[2][32], dp[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tmem_ld32(tmem + C_S + lane_base + half * 64 + c * 32, s[c]);
        tmem_ld32(tmem + C_DP + lane_base + half * 64 + c * 32, dp[c]);
      }
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sdp_read);
      uint32_t pk[32];
      const bool diagonal = j == qt;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        float ds2[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int col = 2 * e + u;  // within this thread's 64 columns
          float p = ex2_approx(fmaf(__uint_as_float(s[col >> 5][col & 31]), c2, neg_lse2));
          if (diagonal && half * 64 + col > r) p = 0.f;
          ds2[u] = p * (__uint_as_float(dp[col >> 5][col & 31]) - delta) * scale;
        }
        pk[e] = pack_bf16(ds2[0], ds2[1]);
      }
      tmem_st32(tmem + C_DS + (j & 1) * 64 + lane_base + half * 32, pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[j & 1]);
    }
    if (ok) ok = mbar_wait_warp_spin(dq_full, 0, error);
    if (ok) {
      tc_fence_after();
      constexpr int COLS = HD / 2;
      __nv_bfloat16* dq_row = dqkv + row * 3 * d + h * HD + half * COLS;
#pragma unroll 1
      for (int c = 0; c < COLS / 32; ++c) {
        uint32_t raw[32];
        tmem_ld32(tmem + C_DQ + lane_base + half * COLS + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t y[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) y[e] = pack_bf16(__uint_as_float(raw[v * 8 + 2 * e]), __uint_as_float(raw[v * 8 + 2 * e + 1]));
          *reinterpret_cast<uint4*>(dq_row + c * 32 + v * 8) = *reinterpret_cast<const uint4*>(y);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---- dK, dV.  Transposed scores, so that the thread that owns a KEY row produces P^T and dS^T rows, which are the A
// operands (M = keys) of the accumulating MMAs:  S^T = K.Q_i^T, dP^T = V.dO_i^T  ->  P^T = exp(S^T*scale - lse[q]) to
// TMEM (bf16)  ->  dV += P^T.dO_i;  dS^T = P^T * (dP^T - delta[q]) * scale to TMEM  ->  dK += dS^T.Q_i.
// lse and delta of the query tile travel with Q_i and dO_i in a stage (plain bulk copies onto the same barrier).
// Each half-warp pair of a lane writes its bf16 result over the first 32 columns of ITS OWN half of the fp32 tile it
// has just consumed (columns [0,32) and [64,96)), so no thread overwrites columns the other has yet to read.
// TMEM: S^T [0,128)  dP^T [128,256)  dV [256,256+HD)  dK [256+HD, 256+2HD).
template <int HD>
struct BwdDkvSmem {
  static constexpr int TILE_BYTES = (HD / 64) * STRIP;
  static constexpr int K = 0, V = TILE_BYTES, STAGES_AT = 2 * TILE_BYTES;
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES + 1024;  // Q_i, dO_i, lse[128], delta[128]
  static constexpr int STAGES_FIT = (223 * 1024 - STAGES_AT) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 4 ? 4 : STAGES_FIT;
  static constexpr int BARS = STAGES_AT + STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BARS + 256;
  static_assert(STAGES >= 2, "two query tiles must be in flight");
};

template <int HD>
__global__ void __launch_bounds__(320, 1)
k_attn_bwd_dkv(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do, const float* __restrict__ lse,
               const float* __restrict__ delta, __nv_bfloat16* __restrict__ dqkv, int B, int T, int H, int d, float scale, int* error) {
  extern __shared__ __align__(1024) uint8_t dkv_smem[];
  uint8_t* smem = dkv_smem;
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) {
      *error = 1;
      __threadfence_system();
    }
    return;
  }
  using L = BwdDkvSmem<HD>;
  constexpr int TILE_BYTES = L::TILE_BYTES, STAGES = L::STAGES, STAGE_BYTES = L::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
  uint64_t *kv_full = bars, *s_full = bars + 1, *dp_full = bars + 2, *p_full = bars + 3, *ds_full = bars + 4, *acc_full = bars + 5,
           *st_full = bars + 6, *st_empty = bars + 6 + STAGES;
  uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 6 + 2 * STAGES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = T / TILE;
  const int kt = (int)blockIdx.x % n_tiles;  // consecutive CTAs share a head; key tile 0 visits every query tile: longest first
  const int rest = (int)blockIdx.x / n_tiles;
  const int h = rest % H, b = rest / H;
  const int nt = n_tiles - kt;  // query tiles kt .. n_tiles-1
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t C_S = 0, C_DP = 128, C_DV = 256, C_DK = 256 + HD;

  if (tid == 0) {
    mbar_init(kv_full, 1);
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_full, 8);
    mbar_init(ds_full, 8);
    mbar_init(acc_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&st_full[s], 1);
      mbar_init(&st_empty[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tensormap(&map_qkv);
    prefetch_tensormap(&map_do);
  }
  if (warp == 1) {
    tmem_alloc(holder, TMEM_COLS);
    tmem_relinquish();
  }
  tb::pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *holder;
  tb::pdl_wait();  // set-up is done; everything below reads what earlier kernels wrote
  auto stage_at = [&](int t) { return smem + L::STAGES_AT + (t % STAGES) * STAGE_BYTES; };

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      load_tile<HD>(smem + L::K, &map_qkv, kv_full, d + h * HD, b * T + kt * TILE);
      load_tile<HD>(smem + L::V, &map_qkv, kv_full, 2 * d + h * HD, b * T + kt * TILE);
      bool ok = true;
      for (int t = 0; t < nt && ok; ++t) {
        const int s = t % STAGES, i = kt + t;
        if (!(ok = mbar_wait(&st_empty[s], ((t / STAGES) & 1) ^ 1, error))) break;
        uint8_t* st = stage_at(t);
        mbar_expect_tx(&st_full[s], STAGE_BYTES);
        load_tile<HD>(st, &map_qkv, &st_full[s], h * HD, b * T + i * TILE);
        load_tile<HD>(st + TILE_BYTES, &map_do, &st_full[s], h * HD, b * T + i * TILE);
        const size_t stat0 = ((size_t)b * H + h) * T + (size_t)i * TILE;
        bulk_load_1d(st + 2 * TILE_BYTES, lse + stat0, 512, &st_full[s]);
        bulk_load_1d(st + 2 * TILE_BYTES + 512, delta + stat0, 512, &st_full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc(128, 128, false, false);
      constexpr uint32_t idesc_acc = instr_desc(128, HD, false, true);
      auto wait_stage = [&](int t) { return mbar_wait(&st_full[t % STAGES], (t / STAGES) & 1, error); };
      // bf16 A operand written over an fp32 tile: keys k-step kk sits at columns (kk / 4) * 64 + (kk % 4) * 8
      auto a_cols = [](int kk) { return (uint32_t)((kk >> 2) * 64 + (kk & 3) * 8); };
      bool ok = mbar_wait(kv_full, 0, error) && wait_stage(0);
      if (ok) {
        tc_fence_after();
        mma_kmajor<HD>(tmem + C_S, smem + L::K, stage_at(0), idesc_s, false);  // S^T = K . Q_i^T
        mma_commit(s_full);
        mma_kmajor<HD>(tmem + C_DP, smem + L::V, stage_at(0) + TILE_BYTES, idesc_s, false);  // dP^T = V . dO_i^T
        mma_commit(dp_full);
      }
      for (int t = 0; t < nt && ok; ++t) {
        const uint32_t q_addr = smem_u32(stage_at(t)), do_addr = q_addr + TILE_BYTES;
        if (!(ok = mbar_wait(p_full, t & 1, error))) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // dV += P^T . dO_i (16 queries per step; dO_i MN-major over the queries)
          mma_bf16_ts(tmem + C_DV, tmem + C_S + a_cols(kk), smem_desc(do_addr + kk * 2048, STRIP, 1024), idesc_acc, (t > 0 || kk > 0) ? 1u : 0u);
        if (t + 1 < nt) {
          if (!(ok = wait_stage(t + 1))) break;
          tc_fence_after();
          mma_kmajor<HD>(tmem + C_S, smem + L::K, stage_at(t + 1), idesc_s, false);
          mma_commit(s_full);
        }
        if (!(ok = mbar_wait(ds_full, t & 1, error))) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // dK += dS^T . Q_i
          mma_bf16_ts(tmem + C_DK, tmem + C_DP + a_cols(kk), smem_desc(q_addr + kk * 2048, STRIP, 1024), idesc_acc, (t > 0 || kk > 0) ? 1u : 0u);
        mma_commit(&st_empty[t % STAGES]);  // Q_i, dO_i (and its lse / delta, read before ds_full) are done with
        if (t + 1 < nt) {
          mma_kmajor<HD>(tmem + C_DP, smem + L::V, stage_at(t + 1) + TILE_BYTES, idesc_s, false);
          mma_commit(dp_full);
        }
      }
      if (ok) mma_commit(acc_full);
    }
  } else {
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;  // key row within the tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float c2 = scale * 1.4426950408889634f;
    bool ok = true;
    for (int t = 0; t < nt && ok; ++t) {
      const int i = kt + t;
      const float* stat = reinterpret_cast<const float*>(stage_at(t) + 2 * TILE_BYTES) + half * 64;  // lse, then (+128) delta
      if (!(ok = mbar_wait_warp_spin(&st_full[t % STAGES], (t / STAGES) & 1, error))) break;  // lse / delta have landed
      if (!(ok = mbar_wait_warp_spin(s_full, t & 1, error))) break;
      tc_fence_after();
      float p[64];
      {
        uint32_t s[2][32];
        tmem_ld32(tmem + C_S + lane_base + half * 64, s[0]);
        tmem_ld32(tmem + C_S + lane_base + half * 64 + 32, s[1]);
        tmem_ld_wait();
        const bool diagonal = i == kt;
#pragma unroll
        for (int col = 0; col < 64; ++col) {
          const float x = ex2_approx(fmaf(__uint_as_float(s[col >> 5][col & 31]), c2, -1.4426950408889634f * stat[col]));
          p[col] = (diagonal && r > half * 64 + col) ? 0.f : x;  // key after the query
        }
      }
      {
        uint32_t pk[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) pk[e] = pack_bf16(p[2 * e], p[2 * e + 1]);
        tmem_st32(tmem + C_S + lane_base + half * 64, pk);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      if (!(ok = mbar_wait_warp_spin(dp_full, t & 1, error))) break;
      tc_fence_after();
      {
        uint32_t dp[2][32], pk[32];
        tmem_ld32(tmem + C_DP + lane_base + half * 64, dp[0]);
        tmem_ld32(tmem + C_DP + lane_base + half * 64 + 32, dp[1]);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float a = p[2 * e] * (__uint_as_float(dp[(2 * e) >> 5][(2 * e) & 31]) - stat[128 + 2 * e]) * scale;
          const float c = p[2 * e + 1] * (__uint_as_float(dp[(2 * e + 1) >> 5][(2 * e + 1) & 31]) - stat[128 + 2 * e + 1]) * scale;
          pk[e] = pack_bf16(a, c);
        }
        tmem_st32(tmem + C_DP + lane_base + half * 64, pk);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok) ok = mbar_wait_warp_spin(acc_full, 0, error);
    if (ok) {
      tc_fence_after();
      constexpr int COLS = HD / 2;
      __nv_bfloat16* dk = dqkv + ((size_t)b * T + kt * TILE + r) * 3 * d + d + h * HD + half * COLS;
      __nv_bfloat16* dv = dk + d;
#pragma unroll 1
      for (int part = 0; part < 2; ++part) {
        __nv_bfloat16* dst = part == 0 ? dv : dk;
        const uint32_t src = tmem + (part == 0 ? C_DV : C_DK) + lane_base + half * COLS;
#pragma unroll 1
        for (int c = 0; c < COLS / 32; ++c) {
          uint32_t raw[32];
          tmem_ld32(src + c * 32, raw);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t y[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] = pack_bf16(__uint_as_float(raw[v * 8 + 2 * e]), __uint_as_float(raw[v * 8 + 2 * e + 1]));
            *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = *reinterpret_cast<const uint4*>(y);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_map(CUtensorMap* map, const void* ptr, long long cols, long long rows, long long row_stride) {
  static thread_local bool context_ready = false;  // the driver entry point below needs a current context in this thread
  if (!context_ready) {
    cudaFree(nullptr);
    context_ready = true;
  }
  static EncodeTiled enc = nullptr;
  if (enc == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return -10;
    enc = (EncodeTiled)p;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t elem[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? 0 : -11;
}

int* g_err_host = nullptr;
int* g_err_dev = nullptr;

int ensure_error_word() {
  if (g_err_host != nullptr) return 0;
  if (cudaHostAlloc((void**)&g_err_host, 64, cudaHostAllocMapped) != cudaSuccess) return -13;
  *g_err_host = 0;
  return cudaHostGetDevicePointer((void**)&g_err_dev, g_err_host, 0) == cudaSuccess ? 0 : -13;
}

}  // namespace

extern "C" {

int tb_attn_error() { return g_err_host != nullptr ? *g_err_host : 0; }

// out[B*T, d] = causal softmax(q k^T / sqrt(HD)) v per head; lse[B, H, T] (fp32) kept for backward.
int tb_attn_fwd(const void* qkv, void* out, float* lse, int B, int T, int H, int HD, cudaStream_t stream) {
  if (T % TILE || (HD != 64 && HD != 128)) return -21;
  if (ensure_error_word()) return -13;
  const int d = H * HD;
  CUtensorMap map;
  int rc = make_map(&map, qkv, 3LL * d, (long long)B * T, 3LL * d);
  if (rc) return rc;
  const float scale_log2e = 1.4426950408889634f / sqrtf((float)HD);
  const int n_pairs = (T / TILE + 1) / 2;
  const unsigned ctas = (unsigned)(n_pairs * H * B);
  tb_note_launch(1);
#define LAUNCH_FWD(HD_) \
  do { \
    static bool once = false; \
    if (!once) { \
      cudaError_t e = cudaFuncSetAttribute(k_attn_fwd_ws<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd2Smem<HD_>::TOTAL); \
      if (e != cudaSuccess) return (int)e; \
      once = true; \
    } \
    return (int)tb::launch(k_attn_fwd_ws<HD_>, dim3(ctas), dim3(320), Fwd2Smem<HD_>::TOTAL, stream, map, (__nv_bfloat16*)out, lse, B, T, H, d, \
                           scale_log2e, g_err_dev); \
  } while (0)
  if (HD == 64) LAUNCH_FWD(64);
  LAUNCH_FWD(128);
#undef LAUNCH_FWD
}

// dqkv[B*T, 3d] from qkv, out, d_out, lse.  delta: fp32 [B*H*T], written by the dQ kernel and read by the dK/dV kernel.
int tb_attn_bwd(const void* qkv, const void* out, const void* d_out, const float* lse, void* dqkv, float* delta, int B, int T, int H, int HD,
                cudaStream_t stream) {
  if (T % TILE || (HD != 64 && HD != 128)) return -21;
  if (ensure_error_word()) return -13;
  const int d = H * HD;
  const long long rows = (long long)B * T;
  CUtensorMap map_qkv, map_do;
  int rc = make_map(&map_qkv, qkv, 3LL * d, rows, 3LL * d);
  if (rc) return rc;
  rc = make_map(&map_do, d_out, d, rows, d);
  if (rc) return rc;
  const float scale = 1.f / sqrtf((float)HD);
  const unsigned ctas = (unsigned)((T / TILE) * H * B);
  tb_note_launch(2);
#define LAUNCH_BWD(HD_) \
  do { \
    static bool once = false; \
    if (!once) { \
      cudaError_t e = cudaFuncSetAttribute(k_attn_bwd_dq<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdDqSmem<HD_>::TOTAL); \
      if (e == cudaSuccess) e = cudaFuncSetAttribute(k_attn_bwd_dkv<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdDkvSmem<HD_>::TOTAL); \
      if (e != cudaSuccess) return (int)e; \
      once = true; \
    } \
    cudaError_t e = tb::launch(k_attn_bwd_dq<HD_>, dim3(ctas), dim3(320), BwdDqSmem<HD_>::TOTAL, stream, map_qkv, map_do, (const __nv_bfloat16*)out, \
                               (const __nv_bfloat16*)d_out, lse, delta, (__nv_bfloat16*)dqkv, B, T, H, d, scale, g_err_dev); \
    if (e != cudaSuccess) return (int)e; \
    return (int)tb::launch(k_attn_bwd_dkv<HD_>, dim3(ctas), dim3(320), BwdDkvSmem<HD_>::TOTAL, stream, map_qkv, map_do, lse, (const float*)delta, \
                           (__nv_bfloat16*)dqkv, B, T, H, d, scale, g_err_dev); \
  } while (0)
  if (HD == 64) LAUNCH_BWD(64);
  LAUNCH_BWD(128);
#undef LAUNCH_BWD
}

}  // extern "C"
