// Causal self-attention on tcgen05 / TMEM, forward and backward, over a packed qkv tensor.
//
// qkv is [B*T, 3*d] bf16 (q | k | v along the row, head h at columns h*HD .. h*HD+HD of each part), T a
// multiple of 128, HD 64 or 128.  One TMA tensor map over that matrix serves every tile load
// (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast): a 128-row x 64-column box is a K-major
// operand when the reduction runs over the head dimension (Q.K^T, dO.V^T) and, with the same bytes,
// an MN-major operand when it runs over the rows (P.V, P^T.dO, dS^T.Q, dS.K).
//
// Forward (one CTA per 128 queries of one head; 256 threads, two per query row = TMEM lane):
//   pass 1  for every key tile:  S = Q.K^T (tcgen05.mma into TMEM) -> running row max
//   pass 2  for every key tile:  S again -> P = exp2(S*c - max) written to shared memory as bf16
//           in the swizzled K-major layout (summed on the way) -> O += P.V (accumulator stays in TMEM)
//   end     O / sum -> bf16, and the row's log-sum-exp for backward
// Two passes trade one extra Q.K^T (attention is ~5 % of this model's flops) for never having to
// rescale an accumulator that lives in TMEM.
//
// Backward (one CTA per 128 keys of one head; loops over the query tiles at or below the diagonal):
//   S = Q.K^T,  dP = dO.V^T   (TMEM)      P = exp(S*scale - lse),  dS = P * (dP - D) * scale
//   dV += P^T.dO,  dK += dS^T.Q            (accumulated in TMEM across query tiles)
//   dQ_tile = dS.K                          (TMEM) -> fp32 atomic adds into a dQ scratch
// D = rowsum(dO * O) comes from a small pre-kernel; a post-kernel converts dQ to bf16.
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

int g_bwd_two_per_sm = 0;
int g_bwd_variant = 1;  // 0: one kernel with fp32 atomics for dQ; 1: the two warp-specialised kernels
int g_fwd_variant = 2;  // 0: two-pass kernel; 1: warp-specialised, P through shared memory; 2: warp-specialised, P in TMEM

using namespace tc;

constexpr int TILE = 128;           // queries per CTA, keys per step
constexpr int STRIP = TILE * 128;   // bytes of one 128-row x 64-column bf16 strip (128-byte rows)

// Byte offset of the 16-byte slot holding elements [8*slot, 8*slot+8) of row r in a swizzled strip.
__device__ __forceinline__ int swz(int r, int slot) { return r * 128 + ((slot ^ (r & 7)) << 4); }

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

struct Waiter {
  uint64_t* bar;
  uint32_t phase;
  int* error;
  // Called by every thread of the CTA.  The verdict is made uniform, so that after a wait that ran out all
  // threads leave the loops together and meet at the same __syncthreads on the way out.
  __device__ __forceinline__ bool wait() {
    bool ok = mbar_wait(bar, phase, error);
    phase ^= 1;
    return __syncthreads_and(ok);
  }
};

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

// ------------------------------------------------------------------------------------------ forward
// 256 threads: thread t owns query row t % 128 and the key columns [64*(t/128), 64*(t/128)+64) of every key
// tile (warps w and w+4 share TMEM lanes 32*(w%4)..).  K (and V) tiles are double-buffered: thread 0 issues
// the loads of the next step before it issues this step's MMAs.
template <int HD>
struct FwdSmem {
  static constexpr int TILE_BYTES = (HD / 64) * STRIP;
  // STATS (the two column halves' row maxima / sums, 1 KB) shares P's bytes: it is written at the end of pass 0 and
  // after the last step, read at the start of pass 1 and at the very end, never while P is live.  With HD = 64 the
  // total stays under 113 KB, so that two CTAs fit one SM (each also holds 256 TMEM columns): one computes its
  // softmax while the other's MMAs run.  The buffer is declared 1024-byte aligned instead of being rounded up.
  static constexpr int Q = 0, KV = Q + TILE_BYTES /* [2 buffers][K, V] */, P = KV + 4 * TILE_BYTES, STATS = P,
                       BARS = P + 2 * STRIP;
  static constexpr int TOTAL = BARS + 64;
};

template <int HD>
__global__ void __launch_bounds__(256, HD == 64 ? 2 : 1)
k_attn_fwd(const __grid_constant__ CUtensorMap map, __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int T, int H, int d,
           float scale_log2e, int* error) {
  extern __shared__ __align__(1024) uint8_t fwd_smem[];
  uint8_t* smem = fwd_smem;
  if (smem_u32(smem) & 1023) {  // the swizzled tiles need 1024-byte alignment; nothing is allocated yet
    if (threadIdx.x == 0) {
      *error = 1;
      __threadfence_system();
    }
    return;
  }
  using L = FwdSmem<HD>;
  constexpr int TILE_BYTES = L::TILE_BYTES;
  uint8_t *sQ = smem + L::Q, *sKV = smem + L::KV, *sP = smem + L::P;
  float* stats = reinterpret_cast<float*>(smem + L::STATS);  // [2 halves][128 rows]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);  // 0: Q, 1-2: K/V buffers, 3: MMA
  uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 4);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid & 127, half = tid >> 7;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int row0 = b * T + qt * TILE;
  constexpr uint32_t TMEM_COLS = 256;  // S: [0,128), O: [128, 128+HD)

  if (tid == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(&bars[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *holder;
  const uint32_t tS = tmem, tO = tmem + 128;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  Waiter wq{&bars[0], 0, error}, wkv[2] = {{&bars[1], 0, error}, {&bars[2], 0, error}}, mm{&bars[3], 0, error};
  constexpr uint32_t idesc_s = instr_desc(128, 128, false, false);
  constexpr uint32_t idesc_o = instr_desc(128, HD, false, true);
  const int steps = 2 * (qt + 1);  // pass 0 over key tiles 0..qt (row maxima), then pass 1 (P and O)

  auto issue_loads = [&](int it) {  // thread 0 only
    const int pass = it > qt, j = pass ? it - (qt + 1) : it, buf = it & 1;
    uint8_t* k_dst = sKV + buf * 2 * TILE_BYTES;
    mbar_expect_tx(&bars[1 + buf], TILE_BYTES * (pass ? 2 : 1));
    load_tile<HD>(k_dst, &map, &bars[1 + buf], d + h * HD, b * T + j * TILE);
    if (pass) load_tile<HD>(k_dst + TILE_BYTES, &map, &bars[1 + buf], 2 * d + h * HD, b * T + j * TILE);
  };

  if (tid == 0) {
    mbar_expect_tx(&bars[0], TILE_BYTES);
    load_tile<HD>(sQ, &map, &bars[0], h * HD, row0);
    issue_loads(0);
  }
  bool ok = wq.wait();

  float m2 = -INFINITY, l = 0.f;
  const int q_idx = qt * TILE + r;
  for (int it = 0; it < steps && ok; ++it) {
    const int pass = it > qt, j = pass ? it - (qt + 1) : it, buf = it & 1;
    const uint8_t* sK = sKV + buf * 2 * TILE_BYTES;
    const uint8_t* sV = sK + TILE_BYTES;
    if (tid == 0 && it + 1 < steps) issue_loads(it + 1);  // the other buffer was released by the previous step's last wait
    if (!(ok = wkv[buf].wait())) break;
    tc_fence_after();
    if (tid == 0) {
      mma_kmajor<HD>(tS, sQ, sK, idesc_s, false);
      mma_commit(&bars[3]);
    }
    if (!(ok = mm.wait())) break;
    tc_fence_after();
    if (it == qt + 1) {  // first step of pass 1: combine the two halves' row maxima
      m2 = fmaxf(stats[r], stats[TILE + r]);
      __syncthreads();  // everyone has read the maxima before P (the same bytes) is written
    }
    const bool diagonal = j == qt;
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      const int col0 = half * 64 + c * 32;
      uint32_t raw[32];
      tmem_ld32(tS + lane_base + col0, raw);
      tmem_ld_wait();
      float x[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        x[i] = __uint_as_float(raw[i]) * scale_log2e;
        if (diagonal && (j * TILE + col0 + i) > q_idx) x[i] = -INFINITY;
      }
      if (!pass) {
#pragma unroll
        for (int i = 0; i < 32; ++i) m2 = fmaxf(m2, x[i]);
      } else {
        uint8_t* strip = sP + half * STRIP;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          __nv_bfloat162 p2[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float p0 = exp2f(x[v * 8 + 2 * i] - m2), p1 = exp2f(x[v * 8 + 2 * i + 1] - m2);
            l += p0 + p1;
            p2[i] = __floats2bfloat162_rn(p0, p1);
          }
          *reinterpret_cast<uint4*>(strip + swz(r, c * 4 + v)) = *reinterpret_cast<const uint4*>(p2);
        }
      }
    }
    if (it == qt) stats[half * TILE + r] = m2;  // end of pass 0
    tc_fence_before();
    if (pass) fence_async_smem();
    __syncthreads();  // every row of S has been read (and P written) before the next MMA touches them
    if (pass) {
      if (tid == 0) {
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // 8 steps of 16 keys: P strip kk/4 (K-major), V rows 16*kk.. (MN-major, strips 16 KB apart)
          mma_bf16(tO, smem_desc(smem_u32(sP + (kk >> 2) * STRIP) + (kk & 3) * 32, 16, 1024),
                   smem_desc(smem_u32(sV) + kk * 2048, STRIP, 1024), idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        mma_commit(&bars[3]);
      }
      if (!(ok = mm.wait())) break;  // P, this K/V buffer and S may be reused
      tc_fence_after();
    }
  }
  if (ok) {
    stats[half * TILE + r] = l;
    __syncthreads();
    l = stats[r] + stats[TILE + r];
    const float inv_l = 1.f / l;
    constexpr int COLS = HD / 2;  // this thread's share of the row
    __nv_bfloat16* o = out + (size_t)(row0 + r) * d + h * HD + half * COLS;
#pragma unroll 1
    for (int c = 0; c < COLS / 32; ++c) {
      uint32_t raw[32];
      tmem_ld32(tO + lane_base + half * COLS + c * 32, raw);
      tmem_ld_wait();
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        __nv_bfloat162 y[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          y[i] = __floats2bfloat162_rn(__uint_as_float(raw[v * 8 + 2 * i]) * inv_l, __uint_as_float(raw[v * 8 + 2 * i + 1]) * inv_l);
        *reinterpret_cast<uint4*>(o + c * 32 + v * 8) = *reinterpret_cast<const uint4*>(y);
      }
    }
    if (half == 0) lse[((size_t)b * H + h) * T + q_idx] = (m2 + log2f(l)) * 0.69314718055994530942f;  // natural log
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
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
// MMAs of the other tile run.  P goes to the MMA either through shared memory (bf16, swizzled K-major strips) or, with
// P_TMEM, stays in TMEM over the first 64 columns of S (bf16 pairs) and is the A operand of a TMEM-sourced MMA.
// TMEM: S_0 [0,128)  S_1 [128,256)  O_0 [256,256+HD)  O_1 [256+HD, 256+2HD).
template <int HD, bool P_TMEM>
struct Fwd2Smem {
  static constexpr int TILE_BYTES = (HD / 64) * STRIP;
  static constexpr int Q = 0;                                       // two query tiles
  static constexpr int P = Q + 2 * TILE_BYTES;                      // two P tiles of 2 strips (absent with P_TMEM)
  static constexpr int RING = P + (P_TMEM ? 0 : 4 * STRIP);
  static constexpr int BUDGET = 224 * 1024;
  static constexpr int SLOTS_FIT = (BUDGET - RING) / TILE_BYTES;
  static constexpr int SLOTS = SLOTS_FIT > 6 ? 6 : SLOTS_FIT;       // K and V tiles in flight
  static constexpr int BARS = RING + SLOTS * TILE_BYTES;
  static constexpr int TOTAL = BARS + 256;
  static_assert(SLOTS >= 3, "the K/V ring needs at least three slots");
};

template <int HD, bool P_TMEM>
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
  using L = Fwd2Smem<HD, P_TMEM>;
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
          if (P_TMEM) {
            mma_bf16_ts(tO, tmem + i * 128 + kk * 8, v_desc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
          } else {
            const uint8_t* sP = smem + L::P + i * 2 * STRIP;
            mma_bf16(tO, smem_desc(smem_u32(sP + (kk >> 2) * STRIP) + (kk & 3) * 32, 16, 1024), v_desc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
          }
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
    uint8_t* sP = smem + L::P + i * 2 * STRIP;
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
        if (P_TMEM) {
          tmem_st32(tS + hh * 32, pk);  // P over the first 64 columns of S: keys 2c, 2c+1 in column c
        } else {
          uint8_t* strip = sP + hh * STRIP;
#pragma unroll
          for (int v = 0; v < 8; ++v) *reinterpret_cast<uint4*>(strip + swz(r, v)) = *reinterpret_cast<const uint4*>(&pk[4 * v]);
        }
      }
      l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
      if (P_TMEM) tmem_st_wait();
      else fence_async_smem();
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

// ------------------------------------------------------------------------------------------ backward
// delta[b, h, t] = sum_c dO[b, t, h*HD + c] * O[b, t, h*HD + c]
__global__ void __launch_bounds__(256)
k_attn_delta(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta, int T, int H, int HD,
             long long rows) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (row, head)
  if (idx >= rows * H) return;
  const long long row = idx / H;
  const int h = (int)(idx % H);
  const __nv_bfloat16* a = o + row * (long long)H * HD + h * HD;
  const __nv_bfloat16* g = d_o + row * (long long)H * HD + h * HD;
  float acc = 0.f;
  for (int c = 0; c < HD; c += 8) {
    uint4 av = *reinterpret_cast<const uint4*>(a + c), gv = *reinterpret_cast<const uint4*>(g + c);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(g2[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  delta[((row / T) * H + h) * T + row % T] = acc;
}

// 256 threads, same row / column-half split as the forward.  Q and dO tiles are double-buffered when they fit
// (HD = 64).  TMEM: [0,128) S, then dQ;  [128,256) dP;  [256, 256+HD) dV;  [256+HD, 256+2HD) dK.
template <int HD>
struct BwdSmem {
  static constexpr int TILE_BYTES = (HD / 64) * STRIP;
  static constexpr int NBUF = HD == 64 ? 2 : 1;
  static constexpr int K = 0, V = K + TILE_BYTES, QDO = V + TILE_BYTES /* [NBUF][Q, dO] */, P = QDO + NBUF * 2 * TILE_BYTES,
                       DS = P + 2 * STRIP, BARS = DS + 2 * STRIP;
  static constexpr int TOTAL = BARS + 64 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(256)
k_attn_bwd(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do, const float* __restrict__ lse,
           const float* __restrict__ delta, float* __restrict__ dq32, __nv_bfloat16* __restrict__ dqkv, int T, int H, int d,
           float scale, int* error) {
  extern __shared__ uint8_t raw_smem[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  using L = BwdSmem<HD>;
  constexpr int TILE_BYTES = L::TILE_BYTES, NBUF = L::NBUF;
  uint8_t *sK = smem + L::K, *sV = smem + L::V, *sQDO = smem + L::QDO, *sP = smem + L::P, *sDS = smem + L::DS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);  // 0: K/V, 1-2: Q/dO buffers, 3: MMA
  uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 4);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid & 127, half = tid >> 7;
  const int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_tiles = T / TILE;
  constexpr uint32_t TMEM_COLS = 512;

  if (tid == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(&bars[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *holder;
  const uint32_t tS = tmem, tDP = tmem + 128, tDV = tmem + 256, tDK = tmem + 256 + HD, tDQ = tmem;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  Waiter wkv{&bars[0], 0, error}, wq[2] = {{&bars[1], 0, error}, {&bars[2], 0, error}}, mm{&bars[3], 0, error};
  constexpr uint32_t idesc_s = instr_desc(128, 128, false, false);   // S, dP: K-major x K-major over HD
  constexpr uint32_t idesc_kv = instr_desc(128, HD, true, true);     // dV = P^T.dO, dK = dS^T.Q: both MN-major over queries
  constexpr uint32_t idesc_dq = instr_desc(128, HD, false, true);    // dQ = dS.K: A K-major over keys, B MN-major

  auto issue_q = [&](int i) {  // thread 0 only
    const int buf = NBUF == 2 ? (i - kt) & 1 : 0;
    uint8_t* q_dst = sQDO + buf * 2 * TILE_BYTES;
    mbar_expect_tx(&bars[1 + buf], 2 * TILE_BYTES);
    load_tile<HD>(q_dst, &map_qkv, &bars[1 + buf], h * HD, b * T + i * TILE);
    load_tile<HD>(q_dst + TILE_BYTES, &map_do, &bars[1 + buf], h * HD, b * T + i * TILE);
  };

  if (tid == 0) {
    mbar_expect_tx(&bars[0], 2 * TILE_BYTES);
    load_tile<HD>(sK, &map_qkv, &bars[0], d + h * HD, b * T + kt * TILE);
    load_tile<HD>(sV, &map_qkv, &bars[0], 2 * d + h * HD, b * T + kt * TILE);
    issue_q(kt);
  }
  bool ok = wkv.wait();

  for (int i = kt; i < n_tiles && ok; ++i) {
    const int buf = NBUF == 2 ? (i - kt) & 1 : 0;
    const uint8_t* sQ = sQDO + buf * 2 * TILE_BYTES;
    const uint8_t* sDO = sQ + TILE_BYTES;
    const int qrow0 = b * T + i * TILE;
    if (NBUF == 2 && tid == 0 && i + 1 < n_tiles) issue_q(i + 1);
    if (!(ok = wq[buf].wait())) break;
    tc_fence_after();
    if (tid == 0) {
      mma_kmajor<HD>(tS, sQ, sK, idesc_s, false);     // S[q, k]
      mma_kmajor<HD>(tDP, sDO, sV, idesc_s, false);   // dP[q, k]
      mma_commit(&bars[3]);
    }
    if (!(ok = mm.wait())) break;
    tc_fence_after();
    const int q_idx = i * TILE + r;
    const float row_lse = lse[((size_t)b * H + h) * T + q_idx];
    const float row_delta = delta[((size_t)b * H + h) * T + q_idx];
    const bool diagonal = i == kt;
    uint8_t* p_strip = sP + half * STRIP;
    uint8_t* ds_strip = sDS + half * STRIP;
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      const int col0 = half * 64 + c * 32;
      uint32_t rs[32], rp[32];
      tmem_ld32(tS + lane_base + col0, rs);
      tmem_ld32(tDP + lane_base + col0, rp);
      tmem_ld_wait();
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        __nv_bfloat162 p2[4], s2[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float pv[2], dv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int col = col0 + v * 8 + 2 * e + u;
            float p = __expf(__uint_as_float(rs[v * 8 + 2 * e + u]) * scale - row_lse);
            if (diagonal && kt * TILE + col > q_idx) p = 0.f;
            pv[u] = p;
            dv[u] = p * (__uint_as_float(rp[v * 8 + 2 * e + u]) - row_delta) * scale;
          }
          p2[e] = __floats2bfloat162_rn(pv[0], pv[1]);
          s2[e] = __floats2bfloat162_rn(dv[0], dv[1]);
        }
        *reinterpret_cast<uint4*>(p_strip + swz(r, c * 4 + v)) = *reinterpret_cast<const uint4*>(p2);
        *reinterpret_cast<uint4*>(ds_strip + swz(r, c * 4 + v)) = *reinterpret_cast<const uint4*>(s2);
      }
    }
    tc_fence_before();
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      // P and dS are stored [query row][key]: as A operands over the queries they are MN-major (M = keys):
      // key strips 16 KB apart (LBO), 8-query groups 1024 B apart (SBO), 16 queries per step = 2048 B.
      // dO and Q are [query row][head dim]: MN-major B operands (N = head dim) with the same geometry.
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        mma_bf16(tDV, smem_desc(smem_u32(sP) + kk * 2048, STRIP, 1024), smem_desc(smem_u32(sDO) + kk * 2048, STRIP, 1024), idesc_kv,
                 (i > kt || kk > 0) ? 1u : 0u);
        mma_bf16(tDK, smem_desc(smem_u32(sDS) + kk * 2048, STRIP, 1024), smem_desc(smem_u32(sQ) + kk * 2048, STRIP, 1024), idesc_kv,
                 (i > kt || kk > 0) ? 1u : 0u);
      }
      // dQ[q, hd] = dS[q, keys] . K[keys, hd]: dS K-major over keys (strip kk/4, 32 B per step), K MN-major over keys.
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        mma_bf16(tDQ, smem_desc(smem_u32(sDS + (kk >> 2) * STRIP) + (kk & 3) * 32, 16, 1024), smem_desc(smem_u32(sK) + kk * 2048, STRIP, 1024),
                 idesc_dq, kk > 0 ? 1u : 0u);
      mma_commit(&bars[3]);
    }
    if (!(ok = mm.wait())) break;
    tc_fence_after();
    if (NBUF == 1 && tid == 0 && i + 1 < n_tiles) issue_q(i + 1);  // single buffer: Q and dO are free only now
    constexpr int COLS = HD / 2;
    float* dq_row = dq32 + (size_t)(qrow0 + r) * d + h * HD + half * COLS;
#pragma unroll 1
    for (int c = 0; c < COLS / 32; ++c) {
      uint32_t raw[32];
      tmem_ld32(tDQ + lane_base + half * COLS + c * 32, raw);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 8; ++e)
        atomicAdd(reinterpret_cast<float4*>(dq_row + c * 32 + e * 4),
                  make_float4(__uint_as_float(raw[4 * e]), __uint_as_float(raw[4 * e + 1]), __uint_as_float(raw[4 * e + 2]),
                              __uint_as_float(raw[4 * e + 3])));
    }
    tc_fence_before();
    __syncthreads();  // dQ has left TMEM, and P / dS may be overwritten
  }
  if (ok) {
    // dK and dV rows (this CTA's keys) into the k and v parts of dqkv; each thread writes half of its row
    constexpr int COLS = HD / 2;
    __nv_bfloat16* dk = dqkv + (size_t)(b * T + kt * TILE + r) * 3 * d + d + h * HD + half * COLS;
    __nv_bfloat16* dv = dk + d;
#pragma unroll 1
    for (int part = 0; part < 2; ++part) {
      __nv_bfloat16* dst = part == 0 ? dv : dk;
      const uint32_t src = (part == 0 ? tDV : tDK) + half * COLS;
#pragma unroll 1
      for (int c = 0; c < COLS / 32; ++c) {
        uint32_t raw[32];
        tmem_ld32(src + lane_base + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          __nv_bfloat162 y[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) y[e] = __floats2bfloat162_rn(__uint_as_float(raw[v * 8 + 2 * e]), __uint_as_float(raw[v * 8 + 2 * e + 1]));
          *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = *reinterpret_cast<const uint4*>(y);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}


// Backward for HD = 64 shaped so that TWO CTAs share an SM (256 TMEM columns and under 113 KB of shared memory
// each): while one CTA computes its exponentials the other's MMAs run.  S and dP take turns in the same 128 TMEM
// columns (P stays packed in registers between them), dQ follows in the first 64 of those; P and dS take turns in
// one shared-memory buffer; Q and dO are single-buffered.  Per query tile:
//   S = Q.K^T                     -> P = exp(S*scale - lse) to registers (bf16 pairs) and shared memory
//   dV += P^T.dO ;  dP = dO.V^T   -> dS = P * (dP - D) * scale over P's bytes in shared memory
//   dK += dS^T.Q ;  dQ = dS.K     -> fp32 atomic adds into the dQ scratch
// TMEM: [0,128) S / dP / dQ;  [128,192) dV;  [192,256) dK.
struct Bwd64Smem {
  static constexpr int K = 0, V = K + STRIP, Q = V + STRIP, DO = Q + STRIP, PS = DO + STRIP, BARS = PS + 2 * STRIP;
  static constexpr int TOTAL = BARS + 64;
};

__global__ void __launch_bounds__(256, 2)
k_attn_bwd64(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do, const float* __restrict__ lse,
             const float* __restrict__ delta, float* __restrict__ dq32, __nv_bfloat16* __restrict__ dqkv, int T, int H, int d, float scale,
             int* error) {
  constexpr int HD = 64;
  extern __shared__ __align__(1024) uint8_t bwd_smem[];
  uint8_t* smem = bwd_smem;
  if (smem_u32(smem) & 1023) {  // the swizzled tiles need 1024-byte alignment; nothing is allocated yet
    if (threadIdx.x == 0) {
      *error = 1;
      __threadfence_system();
    }
    return;
  }
  using L = Bwd64Smem;
  uint8_t *sK = smem + L::K, *sV = smem + L::V, *sQ = smem + L::Q, *sDO = smem + L::DO, *sPS = smem + L::PS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);  // 0: K/V, 1: Q/dO, 2: MMA
  uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 4);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid & 127, half = tid >> 7;
  const int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_tiles = T / TILE;
  constexpr uint32_t TMEM_COLS = 256;

  if (tid == 0) {
    for (int i = 0; i < 3; ++i) mbar_init(&bars[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *holder;
  const uint32_t tSP = tmem, tDQ = tmem, tDV = tmem + 128, tDK = tmem + 192;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  Waiter wkv{&bars[0], 0, error}, wq{&bars[1], 0, error}, mm{&bars[2], 0, error};
  constexpr uint32_t idesc_s = instr_desc(128, 128, false, false);
  constexpr uint32_t idesc_kv = instr_desc(128, HD, true, true);
  constexpr uint32_t idesc_dq = instr_desc(128, HD, false, true);

  auto issue_q = [&](int i) {  // thread 0 only
    mbar_expect_tx(&bars[1], 2 * STRIP);
    load_tile<HD>(sQ, &map_qkv, &bars[1], h * HD, b * T + i * TILE);
    load_tile<HD>(sDO, &map_do, &bars[1], h * HD, b * T + i * TILE);
  };

  if (tid == 0) {
    mbar_expect_tx(&bars[0], 2 * STRIP);
    load_tile<HD>(sK, &map_qkv, &bars[0], d + h * HD, b * T + kt * TILE);
    load_tile<HD>(sV, &map_qkv, &bars[0], 2 * d + h * HD, b * T + kt * TILE);
    issue_q(kt);
  }
  bool ok = wkv.wait();
  uint8_t* my_strip = sPS + half * STRIP;

  for (int i = kt; i < n_tiles && ok; ++i) {
    const int qrow0 = b * T + i * TILE;
    if (!(ok = wq.wait())) break;
    tc_fence_after();
    if (tid == 0) {
      mma_kmajor<HD>(tSP, sQ, sK, idesc_s, false);  // S[q, k]
      mma_commit(&bars[2]);
    }
    if (!(ok = mm.wait())) break;
    tc_fence_after();
    const int q_idx = i * TILE + r;
    const float row_lse = lse[((size_t)b * H + h) * T + q_idx];
    const float row_delta = delta[((size_t)b * H + h) * T + q_idx];
    const bool diagonal = i == kt;
    uint4 packed[8];  // this thread's 64 probabilities as bf16 pairs
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int col0 = half * 64 + c * 32;
      uint32_t rs[32];
      tmem_ld32(tSP + lane_base + col0, rs);
      tmem_ld_wait();
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&packed[c * 4 + v]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float pv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int col = col0 + v * 8 + 2 * e + u;
            float p = __expf(__uint_as_float(rs[v * 8 + 2 * e + u]) * scale - row_lse);
            if (diagonal && kt * TILE + col > q_idx) p = 0.f;
            pv[u] = p;
          }
          p2[e] = __floats2bfloat162_rn(pv[0], pv[1]);
        }
        *reinterpret_cast<uint4*>(my_strip + swz(r, c * 4 + v)) = packed[c * 4 + v];
      }
    }
    tc_fence_before();
    fence_async_smem();
    __syncthreads();  // S has been read everywhere (dP may overwrite it) and P is complete
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)  // dV += P^T.dO: P and dO MN-major over the queries
        mma_bf16(tDV, smem_desc(smem_u32(sPS) + kk * 2048, STRIP, 1024), smem_desc(smem_u32(sDO) + kk * 2048, STRIP, 1024), idesc_kv,
                 (i > kt || kk > 0) ? 1u : 0u);
      mma_kmajor<HD>(tSP, sDO, sV, idesc_s, false);  // dP[q, k]
      mma_commit(&bars[2]);
    }
    if (!(ok = mm.wait())) break;  // P's bytes may be overwritten: the dV MMAs have read them
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int col0 = half * 64 + c * 32;
      uint32_t rp[32];
      tmem_ld32(tSP + lane_base + col0, rp);
      tmem_ld_wait();
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&packed[c * 4 + v]);
        __nv_bfloat162 s2[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 p = __bfloat1622float2(p2[e]);
          s2[e] = __floats2bfloat162_rn(p.x * (__uint_as_float(rp[v * 8 + 2 * e]) - row_delta) * scale,
                                        p.y * (__uint_as_float(rp[v * 8 + 2 * e + 1]) - row_delta) * scale);
        }
        *reinterpret_cast<uint4*>(my_strip + swz(r, c * 4 + v)) = *reinterpret_cast<const uint4*>(s2);
      }
    }
    tc_fence_before();
    fence_async_smem();
    __syncthreads();  // dP has been read everywhere (dQ may overwrite it) and dS is complete
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)  // dK += dS^T.Q
        mma_bf16(tDK, smem_desc(smem_u32(sPS) + kk * 2048, STRIP, 1024), smem_desc(smem_u32(sQ) + kk * 2048, STRIP, 1024), idesc_kv,
                 (i > kt || kk > 0) ? 1u : 0u);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)  // dQ = dS.K: dS K-major over the keys, K MN-major over the keys
        mma_bf16(tDQ, smem_desc(smem_u32(sPS + (kk >> 2) * STRIP) + (kk & 3) * 32, 16, 1024), smem_desc(smem_u32(sK) + kk * 2048, STRIP, 1024),
                 idesc_dq, kk > 0 ? 1u : 0u);
      mma_commit(&bars[2]);
    }
    if (!(ok = mm.wait())) break;
    tc_fence_after();
    if (tid == 0 && i + 1 < n_tiles) issue_q(i + 1);  // Q and dO are free only now
    constexpr int COLS = HD / 2;
    float* dq_row = dq32 + (size_t)(qrow0 + r) * d + h * HD + half * COLS;
    {
      uint32_t raw[32];
      tmem_ld32(tDQ + lane_base + half * COLS, raw);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 8; ++e)
        atomicAdd(reinterpret_cast<float4*>(dq_row + e * 4),
                  make_float4(__uint_as_float(raw[4 * e]), __uint_as_float(raw[4 * e + 1]), __uint_as_float(raw[4 * e + 2]),
                              __uint_as_float(raw[4 * e + 3])));
    }
    tc_fence_before();
    __syncthreads();  // dQ has left TMEM before the next tile's S lands there
  }
  if (ok) {
    constexpr int COLS = HD / 2;
    __nv_bfloat16* dk = dqkv + (size_t)(b * T + kt * TILE + r) * 3 * d + d + h * HD + half * COLS;
    __nv_bfloat16* dv = dk + d;
#pragma unroll 1
    for (int part = 0; part < 2; ++part) {
      __nv_bfloat16* dst = part == 0 ? dv : dk;
      uint32_t raw[32];
      tmem_ld32((part == 0 ? tDV : tDK) + half * COLS + lane_base, raw);
      tmem_ld_wait();
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        __nv_bfloat162 y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = __floats2bfloat162_rn(__uint_as_float(raw[v * 8 + 2 * e]), __uint_as_float(raw[v * 8 + 2 * e + 1]));
        *reinterpret_cast<uint4*>(dst + v * 8) = *reinterpret_cast<const uint4*>(y);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
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

// dqkv[row, 0:d] = bf16(dq32[row, :])
__global__ void __launch_bounds__(256) k_attn_dq_out(const float* __restrict__ dq32, __nv_bfloat16* __restrict__ dqkv, long long rows, int d) {
  const long long n8 = rows * (d / 8);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / (d / 8);
    const int c = (int)(i % (d / 8)) * 8;
    const float4 a = *reinterpret_cast<const float4*>(dq32 + row * d + c), bq = *reinterpret_cast<const float4*>(dq32 + row * d + c + 4);
    __nv_bfloat162 y[4] = {__floats2bfloat162_rn(a.x, a.y), __floats2bfloat162_rn(a.z, a.w), __floats2bfloat162_rn(bq.x, bq.y),
                           __floats2bfloat162_rn(bq.z, bq.w)};
    *reinterpret_cast<uint4*>(dqkv + row * 3 * d + c) = *reinterpret_cast<const uint4*>(y);
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
  dim3 grid(T / TILE, H, B);
  tb_note_launch(1);
  if (g_fwd_variant > 0) {
    const int n_pairs = (T / TILE + 1) / 2;
    const unsigned ctas = (unsigned)(n_pairs * H * B);
#define LAUNCH_WS(HD_, PT_) \
  do { \
    static bool once = false; \
    if (!once) { \
      cudaError_t e = cudaFuncSetAttribute(k_attn_fwd_ws<HD_, PT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd2Smem<HD_, PT_>::TOTAL); \
      if (e != cudaSuccess) return (int)e; \
      once = true; \
    } \
    tb::launch(k_attn_fwd_ws<HD_, PT_>, dim3(ctas), dim3(320), Fwd2Smem<HD_, PT_>::TOTAL, stream, map, (__nv_bfloat16*)out, lse, B, T, H, d, scale_log2e, g_err_dev); \
  } while (0)
    if (HD == 64 && g_fwd_variant == 1) LAUNCH_WS(64, false);
    else if (HD == 64) LAUNCH_WS(64, true);
    else if (g_fwd_variant == 1) LAUNCH_WS(128, false);
    else LAUNCH_WS(128, true);
#undef LAUNCH_WS
    return (int)cudaGetLastError();
  }
  if (HD == 64) {
    static bool once = false;
    if (!once) {
      cudaFuncSetAttribute(k_attn_fwd<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<64>::TOTAL);
      cudaFuncSetAttribute(k_attn_fwd<64>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);  // two CTAs per SM
      once = true;
    }
    k_attn_fwd<64><<<grid, 256, FwdSmem<64>::TOTAL, stream>>>(map, (__nv_bfloat16*)out, lse, T, H, d, scale_log2e, g_err_dev);
  } else {
    static bool once = false;
    if (!once) { cudaFuncSetAttribute(k_attn_fwd<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<128>::TOTAL); once = true; }
    k_attn_fwd<128><<<grid, 256, FwdSmem<128>::TOTAL, stream>>>(map, (__nv_bfloat16*)out, lse, T, H, d, scale_log2e, g_err_dev);
  }
  return (int)cudaGetLastError();
}

void tb_attn_fwd_variant(int v) { g_fwd_variant = v; }

void tb_attn_bwd_kernels(int v) { g_bwd_variant = v; }

// 1: the HD = 64 backward runs as k_attn_bwd64 (two CTAs per SM); 0: as k_attn_bwd<64>.  For measurements.
void tb_attn_bwd_variant(int two_per_sm) { g_bwd_two_per_sm = two_per_sm; }

// dqkv[B*T, 3d] from qkv, out, d_out, lse.  delta: fp32 [B*H*T] scratch; dq32: fp32 [B*T*d] scratch (zeroed here).
int tb_attn_bwd(const void* qkv, const void* out, const void* d_out, const float* lse, void* dqkv, float* delta, float* dq32, int B, int T,
                int H, int HD, cudaStream_t stream) {
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
  if (g_bwd_variant > 0) {
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
    tb::launch(k_attn_bwd_dq<HD_>, dim3(ctas), dim3(320), BwdDqSmem<HD_>::TOTAL, stream, map_qkv, map_do, (const __nv_bfloat16*)out, \
               (const __nv_bfloat16*)d_out, lse, delta, (__nv_bfloat16*)dqkv, B, T, H, d, scale, g_err_dev); \
    tb::launch(k_attn_bwd_dkv<HD_>, dim3(ctas), dim3(320), BwdDkvSmem<HD_>::TOTAL, stream, map_qkv, map_do, lse, (const float*)delta, \
               (__nv_bfloat16*)dqkv, B, T, H, d, scale, g_err_dev); \
  } while (0)
    if (HD == 64) LAUNCH_BWD(64);
    else LAUNCH_BWD(128);
#undef LAUNCH_BWD
    return (int)cudaGetLastError();
  }
  tb_note_launch(4);
  cudaMemsetAsync(dq32, 0, sizeof(float) * rows * d, stream);
  k_attn_delta<<<(unsigned)((rows * H + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out, delta, T, H, HD, rows);
  dim3 grid(T / TILE, H, B);
  if (HD == 64 && g_bwd_two_per_sm) {
    static bool once = false;
    if (!once) {
      cudaFuncSetAttribute(k_attn_bwd64, cudaFuncAttributeMaxDynamicSharedMemorySize, Bwd64Smem::TOTAL);
      cudaFuncSetAttribute(k_attn_bwd64, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      once = true;
    }
    k_attn_bwd64<<<grid, 256, Bwd64Smem::TOTAL, stream>>>(map_qkv, map_do, lse, delta, dq32, (__nv_bfloat16*)dqkv, T, H, d, scale, g_err_dev);
  } else if (HD == 64) {
    static bool once = false;
    if (!once) { cudaFuncSetAttribute(k_attn_bwd<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<64>::TOTAL); once = true; }
    k_attn_bwd<64><<<grid, 256, BwdSmem<64>::TOTAL, stream>>>(map_qkv, map_do, lse, delta, dq32, (__nv_bfloat16*)dqkv, T, H, d, scale, g_err_dev);
  } else {
    static bool once = false;
    if (!once) { cudaFuncSetAttribute(k_attn_bwd<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<128>::TOTAL); once = true; }
    k_attn_bwd<128><<<grid, 256, BwdSmem<128>::TOTAL, stream>>>(map_qkv, map_do, lse, delta, dq32, (__nv_bfloat16*)dqkv, T, H, d, scale, g_err_dev);
  }
  k_attn_dq_out<<<592, 256, 0, stream>>>(dq32, (__nv_bfloat16*)dqkv, rows, d);
  return (int)cudaGetLastError();
}

}  // extern "C"
