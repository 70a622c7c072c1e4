// One AdamW element update, shared by the stand-alone optimizer kernel and the
// reduce-scatter epilogue.
//
// It reproduces torch.optim.AdamW's single-tensor sequence as ATen's CUDA
// kernels evaluate it, including where nvcc contracts a multiply-add inside one
// ATen kernel into an FMA and where ATen divides by a host scalar by multiplying
// with its float reciprocal:
//   p  = p * (1 - lr*wd)                          mul_
//   m  = fma(1-b1, g - m, m)                      lerp_ (weight < 0.5)
//   v  = fma((1-b2) * g, g, v * b2)               mul_ then addcmul_
//   d  = sqrt(v) * (1 / sqrt(bc2)) + eps          sqrt, div by scalar, add_
//   p  = fma(-lr/bc1, m / d, p)                   addcdiv_
#pragma once
#include <cuda_bf16.h>

struct AdamScalars {
  float decay, w1, b2, w2, inv_bias2_sqrt, eps, neg_step;
  int do_decay;
};

__device__ __forceinline__ void adam_update(float& p, float& m, float& v, float g, const AdamScalars& s) {
  if (s.do_decay) p = __fmul_rn(p, s.decay);
  m = s.w1 < 0.5f ? __fmaf_rn(s.w1, __fsub_rn(g, m), m) : __fsub_rn(g, __fmul_rn(__fsub_rn(g, m), __fsub_rn(1.f, s.w1)));
  v = __fmaf_rn(__fmul_rn(s.w2, g), g, __fmul_rn(v, s.b2));
  float denom = __fadd_rn(__fmul_rn(__fsqrt_rn(v), s.inv_bias2_sqrt), s.eps);
  p = __fmaf_rn(s.neg_step, __fdiv_rn(m, denom), p);
}

// Arguments of a fused AdamW epilogue (the reduce-scatter kernel applies it to the
// freshly reduced gradient chunk): element j of the chunk updates element j of each array.
struct AdamArgs {
  float* param;
  float* exp_avg;
  float* exp_avg_sq;
  __nv_bfloat16* shadow;  // optional bf16 copy of the updated parameter
  AdamScalars s;          // s.inv_bias2_sqrt is filled in by the host wrapper
  const AdamScalars* s_dev;  // if not null: the scalars are read from device memory when the kernel starts (written by
                             // k_adam_prepare), so a launch recorded in a CUDA graph sees each replay's step
};

