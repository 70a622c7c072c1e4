// Memory-bound layer kernels around the GEMMs, bf16 in / bf16 out with fp32 math:
// LayerNorm forward/backward, fused softmax-cross-entropy forward/backward, token+position
// embedding forward/backward and column sums (bias gradients).  Each reads its input once and
// writes its output once.  The reference runs these as separate ATen calls
// (nn.LayerNorm, F.cross_entropy, nn.Embedding, autograd's bias reductions: tandem/model.py:50-116).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "launch.cuh"
#include "noalloc.h"

extern "C" void tb_note_launch(int n);

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = v;
}

// ------------------------------------------------------------------------------------ LayerNorm
// One warp per row; D is a multiple of 8.  MAXV 16-byte vectors per lane cover D <= 32*8*MAXV.
template <int MAXV>
__global__ void __launch_bounds__(256)
k_ln_fwd(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
         __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int M, int D, float eps) {
  tb::pdl_enter();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= M) return;
  const int nvec = D >> 3;
  float v[MAXV][8];
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int vi = lane + 32 * j;
    if (vi < nvec) {
      load8(x + (size_t)row * D + vi * 8, v[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += v[j][e];
    }
  }
  const float mean = warp_sum(sum) / D;
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    if (lane + 32 * j < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float d = v[j][e] - mean;
        sq += d * d;
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / D + eps);
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int vi = lane + 32 * j;
    if (vi < nvec) {
      float wv[8], bv[8], o[8];
      load8(w + vi * 8, wv);
      load8(b + vi * 8, bv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[j][e] - mean) * rstd * wv[e] + bv[e];
      store8(y + (size_t)row * D + vi * 8, o);
    }
  }
}

// dx for each row, and per-block partial sums of dw = sum dy*xhat and db = sum dy into
// part[blockIdx.x][2][D] (fp32).  A second kernel adds the partials in a fixed order.
// add (optional): a second gradient of the same input, summed into dx in fp32 before the one rounding
// -- the residual branch's gradient in a pre-LayerNorm block, which autograd would otherwise add with a
// separate pass over the activations.
// Rows are software-pipelined: while a warp works on one row, the 16-byte loads of its next row (dy and x, kept
// packed as bf16 so that they cost half the registers) are already in flight, and the residual gradient of the
// current row is requested before the row's reductions start.  With one row per warp in flight the kernel ran at
// the pace of one memory round trip per row (0.42 of the copy bandwidth); two rows per warp and two blocks per SM
// keep about 100 KB per SM on the way.
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

template <int MAXV>
__global__ void __launch_bounds__(256, MAXV <= 4 ? 2 : 1)
k_ln_bwd(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
         const float* __restrict__ mean_in, const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ add,
         __nv_bfloat16* __restrict__ dx, float* __restrict__ part, int M, int D) {
  tb::pdl_enter();
  extern __shared__ float sh[];  // [warps][2][D]
  const int warps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = D >> 3;
  float dw[MAXV][8], db[MAXV][8];
#pragma unroll
  for (int j = 0; j < MAXV; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) dw[j][e] = db[j][e] = 0.f;
  const int stride = gridDim.x * warps;
  int row = blockIdx.x * warps + warp;
  constexpr bool AHEAD = MAXV <= 4;  // wider rows have no registers left for a second row
  uint4 ndy[MAXV], nx[MAXV];  // the next row, packed
  float nmean = 0.f, nrstd = 0.f;
  auto fetch = [&](int r) {
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int vi = lane + 32 * j;
      if (vi < nvec) {
        ndy[j] = __ldg(reinterpret_cast<const uint4*>(dy + (size_t)r * D + vi * 8));
        nx[j] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * D + vi * 8));
      }
    }
    nmean = mean_in[r];
    nrstd = rstd_in[r];
  };
  if (AHEAD && row < M) fetch(row);
  for (; row < M; row += stride) {
    if (!AHEAD) fetch(row);
    uint4 cdy[MAXV], cx[MAXV], cadd[MAXV];
    const float mean = nmean, rstd = nrstd;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      cdy[j] = ndy[j];
      cx[j] = nx[j];
    }
    if (AHEAD && row + stride < M) fetch(row + stride);
    if (add != nullptr) {  // may alias dx: this row's dx is written only after these loads have been consumed
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        const int vi = lane + 32 * j;
        if (vi < nvec) cadd[j] = *reinterpret_cast<const uint4*>(add + (size_t)row * D + vi * 8);
      }
    }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int vi = lane + 32 * j;
      if (vi < nvec) {
        float dyv[8], xv[8], wv[8];
        unpack8(cdy[j], dyv);
        unpack8(cx[j], xv);
        load8(w + vi * 8, wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = (xv[e] - mean) * rstd;
          const float gv = dyv[e] * wv[e];
          s1 += gv;
          s2 += gv * xh;
          dw[j][e] += dyv[e] * xh;
          db[j][e] += dyv[e];
        }
      }
    }
    s1 = warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int vi = lane + 32 * j;
      if (vi < nvec) {
        float dyv[8], xv[8], wv[8], o[8];
        unpack8(cdy[j], dyv);
        unpack8(cx[j], xv);
        load8(w + vi * 8, wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = (xv[e] - mean) * rstd;  // the same operations as above: the same values
          o[e] = rstd * (dyv[e] * wv[e] - s1 - xh * s2);
        }
        if (add != nullptr) {
          float a[8];
          unpack8(cadd[j], a);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += a[e];
        }
        store8(dx + (size_t)row * D + vi * 8, o);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int vi = lane + 32 * j;
    if (vi < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sh[(warp * 2 + 0) * D + vi * 8 + e] = dw[j][e];
        sh[(warp * 2 + 1) * D + vi * 8 + e] = db[j][e];
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
    float acc = 0.f;
    for (int wv = 0; wv < warps; ++wv) acc += sh[wv * 2 * D + i];
    part[(size_t)blockIdx.x * 2 * D + i] = acc;
  }
}

// out[c] = sum over p of part[p][c], written as bf16.  32 columns x 8 row lanes per block: each lane adds
// every 8th partial, then the 8 lanes are combined in a fixed order (deterministic).
__global__ void __launch_bounds__(256)
k_reduce_partials(const float* __restrict__ part, int parts, int width, __nv_bfloat16* __restrict__ out0,
                  __nv_bfloat16* __restrict__ out1, int split) {
  tb::pdl_enter();
  __shared__ float sh[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float acc = 0.f;
  if (c < width)
    for (int p = ry; p < parts; p += 8) acc += part[(size_t)p * width + c];
  sh[ry][cx] = acc;
  __syncthreads();
  if (ry == 0 && c < width) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sh[k][cx];
    if (c < split) out0[c] = __float2bfloat16_rn(t);
    else out1[c - split] = __float2bfloat16_rn(t);
  }
}

// ------------------------------------------------------------------------------------ column sums
// Ticket words for k_col_sum's single-launch mode: all zero between launches.
__device__ unsigned g_col_sum_tickets[8192];

// part[blockIdx.y][c] = sum of x[r, c] over the block's row slice; 32 columns x 32 row lanes.
// With `tickets` (one zero word per column group) the kernel also finishes the job: the last row slice of a
// column group to arrive adds the group's partials -- in slice order, with the same grouping as
// k_reduce_partials, so the result does not depend on which block came last -- writes out[c] and leaves the
// ticket at zero for the next launch.
__global__ void __launch_bounds__(1024)
k_col_sum(const __nv_bfloat16* __restrict__ x, int M, int N, int ld, float* __restrict__ part, unsigned* tickets,
          __nv_bfloat16* __restrict__ out) {
  tb::pdl_enter();
  __shared__ float sh[32][33];
  __shared__ int is_last;
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;
  const int rows_per = (M + gridDim.y - 1) / gridDim.y;
  const int r0 = blockIdx.y * rows_per, r1 = min(M, r0 + rows_per);
  float acc = 0.f;
  if (col < N)
    for (int r = r0 + ry; r < r1; r += 32) acc += __bfloat162float(x[(size_t)r * ld + col]);
  sh[ry][cx] = acc;
  __syncthreads();
  if (ry == 0 && col < N) {
    float t = 0.f;
    for (int k = 0; k < 32; ++k) t += sh[k][cx];
    part[(size_t)blockIdx.y * N + col] = t;
  }
  if (tickets == nullptr) return;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&tickets[blockIdx.x], 1u) == gridDim.y - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float lane_sum = 0.f;
  if (ry < 8 && col < N)
    for (int p = ry; p < (int)gridDim.y; p += 8) lane_sum += __ldcg(part + (size_t)p * N + col);
  if (ry < 8) sh[ry][cx] = lane_sum;
  __syncthreads();
  if (ry == 0 && col < N) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sh[k][cx];
    out[col] = __float2bfloat16_rn(t);
  }
  if (threadIdx.x == 0) tickets[blockIdx.x] = 0;
}

// The same job for matrices whose rows are 16-byte aligned (N, ld multiples of 8): every thread reads 16-byte vectors
// (8 columns) and keeps four row-strided loads in flight, so the kernel runs at memory speed instead of at the pace of
// 2-byte loads.  256 threads = 32 column vectors (256 columns) x 8 row lanes; grid.x = column groups of 256, grid.y = row
// slices.  Same partials, tickets and summation order per column as k_col_sum, hence the same result.
__global__ void __launch_bounds__(256)
k_col_sum_vec(const __nv_bfloat16* __restrict__ x, int M, int N, int ld, float* __restrict__ part, unsigned* tickets,
              __nv_bfloat16* __restrict__ out) {
  tb::pdl_enter();
  __shared__ float sh[8][256 + 8];
  __shared__ int is_last;
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + cx * 8;
  const int rows_per = (M + gridDim.y - 1) / gridDim.y;
  const int r0 = blockIdx.y * rows_per, r1 = min(M, r0 + rows_per);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < N) {
    int r = r0 + ry;
    for (; r + 24 < r1; r += 32) {
      float v[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) load8(x + (size_t)(r + 8 * u) * ld + col, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += v[u][e];
    }
    for (; r < r1; r += 8) {
      float v[8];
      load8(x + (size_t)r * ld + col, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) sh[ry][cx * 8 + e] = acc[e];
  __syncthreads();
  {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < N) {
      float t = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) t += sh[k][threadIdx.x];
      part[(size_t)blockIdx.y * N + c] = t;
    }
  }
  if (tickets == nullptr) return;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&tickets[blockIdx.x], 1u) == gridDim.y - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < N) {
      // eight lanes of every-eighth slice, combined in lane order: the grouping of k_reduce_partials
      float lanes[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int p = 0; p < (int)gridDim.y; ++p) lanes[p & 7] += __ldcg(part + (size_t)p * N + c);
      float t = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) t += lanes[k];
      out[c] = __float2bfloat16_rn(t);
    }
  }
  if (threadIdx.x == 0) tickets[blockIdx.x] = 0;
}

// ------------------------------------------------------------------------------------ cross-entropy
// One block per row.  Forward: lse[row] and loss[row] = lse - logit[target].
__global__ void __launch_bounds__(256)
k_xent_fwd(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ lse_out,
           float* __restrict__ loss_out, int V, int ld) {
  tb::pdl_enter();
  __shared__ float red[8];
  const int row = blockIdx.x;
  const __nv_bfloat16* z = logits + (size_t)row * ld;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, __bfloat162float(z[i]));
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = red[0];
  for (int k = 1; k < warps; ++k) m = fmaxf(m, red[k]);
  __syncthreads();
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(__bfloat162float(z[i]) - m);
  s = warp_sum(s);
  if (lane == 0) red[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int k = 0; k < warps; ++k) t += red[k];
    const float lse = m + logf(t);
    lse_out[row] = lse;
    loss_out[row] = lse - __bfloat162float(z[targets[row]]);
  }
}

// Backward, in place: logits[row, i] <- (softmax_i - [i == target]) * scale.  Columns [V, width) <- 0
// (row padding, when the caller owns it).
__global__ void __launch_bounds__(256)
k_xent_bwd(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets, const float* __restrict__ lse,
           const float* __restrict__ grad_scale, float inv_rows, int V, int ld, int width) {
  tb::pdl_enter();
  const int row = blockIdx.x;
  __nv_bfloat16* z = logits + (size_t)row * ld;
  const float l = lse[row];
  const float scale = grad_scale[0] * inv_rows;
  const int t = (int)targets[row];
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float g = 0.f;
    if (i < V) g = (__expf(__bfloat162float(z[i]) - l) - (i == t ? 1.f : 0.f)) * scale;
    z[i] = __float2bfloat16_rn(g);
  }
}

// loss = mean(per_row) in a fixed order (one block).
__global__ void __launch_bounds__(1024) k_mean(const float* __restrict__ v, int n, float* __restrict__ out) {
  tb::pdl_enter();
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += v[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) out[0] = t / n;
  }
}

// ------------------------------------------------------------------------------------ embedding
__global__ void __launch_bounds__(256)
k_embed_fwd(const long long* __restrict__ idx, const __nv_bfloat16* __restrict__ tok, const __nv_bfloat16* __restrict__ pos,
            __nv_bfloat16* __restrict__ out, int rows, int T, int D) {
  tb::pdl_enter();
  const int nvec = D >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)rows * nvec; i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / nvec), v = (int)(i % nvec);
    float a[8], b[8];
    load8(tok + (size_t)idx[row] * D + v * 8, a);
    load8(pos + (size_t)(row % T) * D + v * 8, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] += b[e];
    store8(out + (size_t)row * D + v * 8, a);
  }
}

// dtok32[idx[row]] += dy[row] (fp32 atomics); dpos[t] = sum over batch of dy[b, t] (fixed order).
__global__ void __launch_bounds__(256)
k_embed_bwd_tok(const long long* __restrict__ idx, const __nv_bfloat16* __restrict__ dy, float* __restrict__ dtok32, int rows, int D) {
  tb::pdl_enter();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)rows * D; i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / D), c = (int)(i % D);
    atomicAdd(dtok32 + (size_t)idx[row] * D + c, __bfloat162float(dy[i]));
  }
}

__global__ void __launch_bounds__(256)
k_embed_bwd_pos(const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dpos, int B, int T, int D) {
  tb::pdl_enter();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)T * D; i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int b = 0; b < B; ++b) acc += __bfloat162float(dy[(size_t)b * T * D + i]);
    dpos[i] = __float2bfloat16_rn(acc);
  }
}

__global__ void __launch_bounds__(256) k_f32_to_bf16(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  tb::pdl_enter();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(in[i]);
}

int grid_for(long long work, int per_block, int cap) {
  long long b = (work + per_block - 1) / per_block;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

extern "C" {

int tb_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int M, int D, float eps,
                     cudaStream_t s) {
  if (D % 8 || D > 32 * 8 * 8) return -20;
  const int blocks = (M + 7) / 8;
  tb_note_launch(1);
#define LN(V) tb::launch(k_ln_fwd<V>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, mean, rstd, M, D, eps)
  if (D <= 256 * 1) LN(1);
  else if (D <= 256 * 2) LN(2);
  else if (D <= 256 * 4) LN(4);
  else LN(8);
#undef LN
  return (int)cudaGetLastError();
}

// scratch: fp32 [blocks * 2 * D] with blocks = tb_layernorm_bwd_blocks(M).
// Few rows: one row per warp on as many SMs as it takes (at 1024 rows four rows per warp would leave 116 SMs idle);
// many rows: several rows per warp, so that the row look-ahead has something to fetch.
int tb_layernorm_bwd_blocks(int M) { return M < 8192 ? grid_for(M, 8, 296) : grid_for(M, 8 * 4, 592); }

int tb_layernorm_bwd_add(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, const void* add, void* dx,
                         void* dw, void* db, float* scratch, int M, int D, cudaStream_t s);

int tb_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx, void* dw,
                     void* db, float* scratch, int M, int D, cudaStream_t s) {
  return tb_layernorm_bwd_add(dy, x, w, mean, rstd, nullptr, dx, dw, db, scratch, M, D, s);
}

// The same with `add` ([M, D] bf16, may be null; may alias dx) summed into dx.
int tb_layernorm_bwd_add(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, const void* add, void* dx,
                         void* dw, void* db, float* scratch, int M, int D, cudaStream_t s) {
  if (D % 8 || D > 32 * 8 * 8) return -20;
  const int blocks = tb_layernorm_bwd_blocks(M);
  const size_t smem = (size_t)8 * 2 * D * sizeof(float);
  tb_note_launch(2);
#define LN(V)                                                                                                          \
  do {                                                                                                                 \
    if (smem > 48 * 1024) cudaFuncSetAttribute(k_ln_bwd<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    tb::launch(k_ln_bwd<V>, dim3(blocks), dim3(256), smem, s, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,          \
               (const __nv_bfloat16*)w, mean, rstd, (const __nv_bfloat16*)add, (__nv_bfloat16*)dx, scratch, M, D);          \
  } while (0)
  if (D <= 256 * 1) LN(1);
  else if (D <= 256 * 2) LN(2);
  else if (D <= 256 * 3) LN(3);
  else if (D <= 256 * 4) LN(4);
  else LN(8);
#undef LN
  tb::launch(k_reduce_partials, dim3((2 * D + 31) / 32), dim3(256), 0, s, (const float*)scratch, blocks, 2 * D, (__nv_bfloat16*)dw, (__nv_bfloat16*)db, D);
  return (int)cudaGetLastError();
}

// out[c] = sum_r x[r, c]; scratch: fp32 [32 * N].
int tb_col_sum(const void* x, int M, int N, int ld, void* out_bf16, float* scratch, cudaStream_t s) {
  const int slices = M >= 2048 ? 32 : (M >= 256 ? 8 : 1);
  const bool vectors = (N & 7) == 0 && (ld & 7) == 0 && ((uintptr_t)x & 15) == 0;
  dim3 grid(vectors ? (N + 255) / 256 : (N + 31) / 32, slices);
  // One launch: each column group's last block finishes the sum.  The ticket words come from a fixed pool handed
  // out round-robin, so launches in flight at the same time never share one (a pool's worth of launches would
  // have to overlap); matrices wider than the pool take the two-kernel path.
  constexpr int POOL = 8192;
  static unsigned* pool = nullptr;
  static int pool_device = -1, next = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (pool == nullptr || pool_device != dev) {
    if (cudaGetSymbolAddress((void**)&pool, g_col_sum_tickets) != cudaSuccess) return (int)cudaGetLastError();
    pool_device = dev;
  }
  if ((int)grid.x <= POOL) {
    if (next + (int)grid.x > POOL) next = 0;
    unsigned* tickets = pool + next;
    next += grid.x;
    tb_note_launch(1);
    if (vectors)
      tb::launch(k_col_sum_vec, grid, dim3(256), 0, s, (const __nv_bfloat16*)x, M, N, ld, scratch, tickets, (__nv_bfloat16*)out_bf16);
    else
      tb::launch(k_col_sum, grid, dim3(1024), 0, s, (const __nv_bfloat16*)x, M, N, ld, scratch, tickets, (__nv_bfloat16*)out_bf16);
    return (int)cudaGetLastError();
  }
  grid = dim3((N + 31) / 32, slices);
  tb_note_launch(2);
  tb::launch(k_col_sum, grid, dim3(1024), 0, s, (const __nv_bfloat16*)x, M, N, ld, scratch, (unsigned*)nullptr, (__nv_bfloat16*)nullptr);
  tb::launch(k_reduce_partials, dim3((N + 31) / 32), dim3(256), 0, s, (const float*)scratch, slices, N, (__nv_bfloat16*)out_bf16,
             (__nv_bfloat16*)nullptr, N);
  return (int)cudaGetLastError();
}

int tb_xent_fwd(const void* logits, const long long* targets, float* lse, float* row_loss, float* loss, int rows, int V, int ld,
                cudaStream_t s) {
  const int threads = V <= 128 ? 32 : (V <= 2048 ? 128 : 256);
  tb_note_launch(2);
  tb::launch(k_xent_fwd, dim3(rows), dim3(threads), 0, s, (const __nv_bfloat16*)logits, targets, lse, row_loss, V, ld);
  tb::launch(k_mean, dim3(1), dim3(1024), 0, s, (const float*)row_loss, rows, loss);
  return (int)cudaGetLastError();
}

int tb_xent_bwd(void* logits, const long long* targets, const float* lse, const float* grad_scale, int rows, int V, int ld,
                int width, cudaStream_t s) {
  const int threads = ld <= 128 ? 32 : (ld <= 2048 ? 128 : 256);
  tb_note_launch(1);
  tb::launch(k_xent_bwd, dim3(rows), dim3(threads), 0, s, (__nv_bfloat16*)logits, targets, lse, grad_scale, 1.f / rows, V, ld, width);
  return (int)cudaGetLastError();
}

int tb_embed_fwd(const long long* idx, const void* tok, const void* pos, void* out, int rows, int T, int D, cudaStream_t s) {
  if (D % 8) return -20;
  tb_note_launch(1);
  tb::launch(k_embed_fwd, dim3(grid_for((long long)rows * (D / 8), 256, 148 * 8)), dim3(256), 0, s, idx, (const __nv_bfloat16*)tok,
             (const __nv_bfloat16*)pos, (__nv_bfloat16*)out, rows, T, D);
  return (int)cudaGetLastError();
}

// dtok32: zeroed fp32 [V, D] scratch; dtok / dpos: bf16 outputs.
int tb_embed_bwd(const long long* idx, const void* dy, float* dtok32, void* dtok, void* dpos, int B, int T, int D, int V,
                 cudaStream_t s) {
  tb_note_launch(3);
  tb::launch(k_embed_bwd_tok, dim3(grid_for((long long)B * T * D, 256, 148 * 8)), dim3(256), 0, s, idx, (const __nv_bfloat16*)dy, dtok32, B * T, D);
  tb::launch(k_f32_to_bf16, dim3(grid_for((long long)V * D, 256, 148 * 8)), dim3(256), 0, s, (const float*)dtok32, (__nv_bfloat16*)dtok, (long long)V * D);
  tb::launch(k_embed_bwd_pos, dim3(grid_for((long long)T * D, 256, 148 * 8)), dim3(256), 0, s, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dpos, B, T, D);
  return (int)cudaGetLastError();
}

}  // extern "C"

// ------------------------------------------------------------------------------------ no-allocation variant
// See noalloc.h.  The scratch lives in this file so that both host and device code here can
// name it; host code must not pass the name itself to a kernel (on the host it is only a
// stand-in for the symbol), so the device address is looked up once per device.
static __device__ __align__(256) float g_colsum_scratch[32 * TB_COLSUM_NOALLOC_MAX_N];
static float* g_colsum_scratch_addr[64] = {nullptr};
static char g_noalloc_error[160] = "";

extern "C" const char* tb_noalloc_last_error() { return g_noalloc_error; }

extern "C" int tb_col_sum_noalloc(const void* x_bf16, int M, int N, int ld, void* out_bf16, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (M <= 0) return (int)cudaMemsetAsync(out_bf16, 0, (size_t)N * sizeof(__nv_bfloat16), stream);  // the sum over no rows
  if (N > TB_COLSUM_NOALLOC_MAX_N) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "tb_col_sum_noalloc: N = %d exceeds the built-in scratch (max %d columns)",
             N, TB_COLSUM_NOALLOC_MAX_N);
    return TB_NOALLOC_TOO_WIDE;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "tb_col_sum_noalloc: no usable current device");
    return TB_NOALLOC_SETUP_FAILED;
  }
  if (g_colsum_scratch_addr[dev] == nullptr) {  // first call on this device: resolve the symbol here, with it current
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_colsum_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_noalloc_error, sizeof(g_noalloc_error), "tb_col_sum_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return TB_NOALLOC_SETUP_FAILED;
    }
    g_colsum_scratch_addr[dev] = p;
  }
  float* scratch = g_colsum_scratch_addr[dev];
  const int slices = M >= 2048 ? 32 : (M >= 256 ? 8 : 1);
  dim3 grid((N + 31) / 32, slices);
  tb_note_launch(2);
  k_col_sum<<<grid, 1024, 0, stream>>>((const __nv_bfloat16*)x_bf16, M, N, ld, scratch, nullptr, nullptr);
  k_reduce_partials<<<(N + 31) / 32, 256, 0, stream>>>(scratch, slices, N, (__nv_bfloat16*)out_bf16, nullptr, N);
  return (int)cudaGetLastError();
}
