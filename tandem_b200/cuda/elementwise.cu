// Fused element-wise kernels: multi-tensor AdamW and bucket pack/unpack.
//
// adamw: one pass over {param, grad, exp_avg, exp_avg_sq} instead of the nine
// ATen kernels of torch's single-tensor AdamW (the reference's ShardedAdamW,
// tandem/optim.py:28-37, and torch.optim.AdamW(foreach=False) used by its DDP
// path); the arithmetic is in adam.cuh.  Optionally also writes a bf16 copy of
// the updated parameter (the compute copy under mixed precision).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "adam.cuh"
#include "launch.cuh"

namespace {

template <typename G>
__device__ __forceinline__ float grad_of(G g);
template <>
__device__ __forceinline__ float grad_of<float>(float g) { return g; }
template <>
__device__ __forceinline__ float grad_of<__nv_bfloat16>(__nv_bfloat16 g) { return __bfloat162float(g); }

template <typename G>
__global__ void __launch_bounds__(256)
k_adamw(float* __restrict__ param, const G* __restrict__ grad, float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq,
        __nv_bfloat16* __restrict__ shadow, long long n, AdamScalars s, float grad_scale) {
  tb::pdl_enter();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g = grad_of<G>(grad[i]);
    if (grad_scale != 1.f) g = __fmul_rn(g, grad_scale);
    float p = param[i], m = exp_avg[i], v = exp_avg_sq[i];
    adam_update(p, m, v, g, s);
    param[i] = p;
    exp_avg[i] = m;
    exp_avg_sq[i] = v;
    if (shadow != nullptr) shadow[i] = __float2bfloat16_rn(p);
  }
}

// Same update with the step-dependent scalars read from device memory, so the launch can sit in a
// CUDA graph and still see a new bias correction on every replay.
template <typename G>
__global__ void __launch_bounds__(256)
k_adamw_dev(float* __restrict__ param, const G* __restrict__ grad, float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq,
            __nv_bfloat16* __restrict__ shadow, long long n, const AdamScalars* __restrict__ scalars) {
  tb::pdl_enter();
  const AdamScalars s = *scalars;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g = grad_of<G>(grad[i]);
    float p = param[i], m = exp_avg[i], v = exp_avg_sq[i];
    adam_update(p, m, v, g, s);
    param[i] = p;
    exp_avg[i] = m;
    exp_avg_sq[i] = v;
    if (shadow != nullptr) shadow[i] = __float2bfloat16_rn(p);
  }
}

// One thread: step += 1, then the scalars of that step, in double precision as the host would.
__global__ void k_adam_prepare(double* step, double lr, double beta1, double beta2, double eps, double wd, AdamScalars* out) {
  tb::pdl_enter();
  const double t = *step + 1.0;
  *step = t;
  const double bc1 = 1.0 - pow(beta1, t), bc2 = 1.0 - pow(beta2, t);
  AdamScalars s;
  s.decay = (float)(1.0 - lr * wd);
  s.w1 = (float)(1.0 - beta1);
  s.b2 = (float)beta2;
  s.w2 = (float)(1.0 - beta2);
  s.inv_bias2_sqrt = 1.0f / (float)sqrt(bc2);
  s.eps = (float)eps;
  s.neg_step = (float)(-(lr / bc1));
  s.do_decay = wd != 0.0;
  *out = s;
}

// ---------------------------------------------------------------- multi-tensor copy
#define TB_COPY_MAX 48
struct CopyTable {
  const char* src[TB_COPY_MAX];
  char* dst[TB_COPY_MAX];
  long long bytes[TB_COPY_MAX];
  int count;
};

// blockIdx.y picks the tensor, blockIdx.x strides over it.
__global__ void __launch_bounds__(256) k_multi_copy(CopyTable t) {
  tb::pdl_enter();
  const int k = blockIdx.y;
  const char* s = t.src[k];
  char* d = t.dst[k];
  const long long n = t.bytes[k];
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  const bool aligned = ((((uintptr_t)s) | ((uintptr_t)d)) & 15) == 0;
  const long long nvec = aligned ? n / 16 : 0;
  for (long long v = tid; v < nvec; v += nth) reinterpret_cast<uint4*>(d)[v] = reinterpret_cast<const uint4*>(s)[v];
  for (long long i = nvec * 16 + tid; i < n; i += nth) d[i] = s[i];
}

}  // namespace

extern "C" void tb_note_launch(int n);

extern "C" {

// 1 (default): kernels are launched with programmatic dependent launch; 0: plain launches (for A/B measurements).
void tb_set_pdl(int on) { tb::pdl_enabled() = on ? 1 : 0; }

// scalars: {1-lr*wd, 1-beta1, beta2, 1-beta2, sqrt(bias_correction2), eps, -lr/bias_correction1}
int tb_adamw(void* param, const void* grad, int grad_is_bf16, void* exp_avg, void* exp_avg_sq, void* shadow_bf16, long long n,
             const float* scalars, int do_decay, float grad_scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  AdamScalars s{scalars[0], scalars[1], scalars[2], scalars[3], 1.0f / scalars[4], scalars[5], scalars[6], do_decay};
  long long want = (n + 256 * 4 - 1) / (256 * 4);
  int blocks = (int)(want > 148 * 8 ? 148 * 8 : want);
  tb_note_launch(1);
  if (grad_is_bf16)
    tb::launch(k_adamw<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (float*)param, (const __nv_bfloat16*)grad, (float*)exp_avg,
               (float*)exp_avg_sq, (__nv_bfloat16*)shadow_bf16, n, s, grad_scale);
  else
    tb::launch(k_adamw<float>, dim3(blocks), dim3(256), 0, stream, (float*)param, (const float*)grad, (float*)exp_avg, (float*)exp_avg_sq,
               (__nv_bfloat16*)shadow_bf16, n, s, grad_scale);
  return (int)cudaGetLastError();
}

// Advances the device-resident step counter (a double) and writes that step's AdamScalars (32 bytes) to `scalars`.
int tb_adam_prepare(void* step_counter, double lr, double beta1, double beta2, double eps, double wd, void* scalars,
                    cudaStream_t stream) {
  tb_note_launch(1);
  tb::launch(k_adam_prepare, dim3(1), dim3(1), 0, stream, (double*)step_counter, lr, beta1, beta2, eps, wd, (AdamScalars*)scalars);
  return (int)cudaGetLastError();
}

// tb_adamw with the scalars taken from device memory (written by tb_adam_prepare).
int tb_adamw_dev(void* param, const void* grad, int grad_is_bf16, void* exp_avg, void* exp_avg_sq, void* shadow_bf16, long long n,
                 const void* scalars, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long want = (n + 256 * 4 - 1) / (256 * 4);
  int blocks = (int)(want > 148 * 8 ? 148 * 8 : want);
  tb_note_launch(1);
  if (grad_is_bf16)
    tb::launch(k_adamw_dev<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (float*)param, (const __nv_bfloat16*)grad, (float*)exp_avg,
               (float*)exp_avg_sq, (__nv_bfloat16*)shadow_bf16, n, (const AdamScalars*)scalars);
  else
    tb::launch(k_adamw_dev<float>, dim3(blocks), dim3(256), 0, stream, (float*)param, (const float*)grad, (float*)exp_avg, (float*)exp_avg_sq,
               (__nv_bfloat16*)shadow_bf16, n, (const AdamScalars*)scalars);
  return (int)cudaGetLastError();
}

// Copies count tensors (src[k] -> dst[k], bytes[k] each) with ceil(count / 48) launches.
int tb_multi_copy(const void* const* src, void* const* dst, const long long* bytes, int count, cudaStream_t stream) {
  for (int base = 0; base < count; base += TB_COPY_MAX) {
    CopyTable t{};
    long long most = 0;
    t.count = count - base < TB_COPY_MAX ? count - base : TB_COPY_MAX;
    for (int k = 0; k < t.count; ++k) {
      t.src[k] = (const char*)src[base + k];
      t.dst[k] = (char*)dst[base + k];
      t.bytes[k] = bytes[base + k];
      if (t.bytes[k] > most) most = t.bytes[k];
    }
    long long want = (most + 256 * 16 * 4 - 1) / (256 * 16 * 4);
    dim3 grid((unsigned)(want < 1 ? 1 : (want > 64 ? 64 : want)), t.count);
    tb_note_launch(1);
    tb::launch(k_multi_copy, grid, dim3(256), 0, stream, t);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
