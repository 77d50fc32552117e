// Mixed-precision Adam / AdamW on a flat shard: fp32 master weights and moments,
// bf16 (or fp32) gradient in, bf16 model weights out, all in one pass.
//
// One launch does what the reference spreads over three: the grad cast to fp32
// (mist/re_swap_manager/optimizer.py:514-518), apex multi_tensor_adam with
// inv_scale (mist/optimizers/fused_adam.py:583-690) and the master -> model
// cast-copy (mist/re_swap_manager/optimizer.py:571-599).
#include "common.cuh"

namespace {

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay;
  float bias_c1, bias_c2;  // 1 - beta^t
  float inv_scale;         // gradients are multiplied by this first (loss scale, 1/dp, ...)
  int adamw;               // 1: decoupled weight decay, 0: L2 added to the gradient
};

template <typename GradT>
__device__ __forceinline__ void load_grad8(const GradT* g, size_t i, float* f);
template <>
__device__ __forceinline__ void load_grad8<__nv_bfloat16>(const __nv_bfloat16* g, size_t i,
                                                          float* f) {
  mb::unpack8(reinterpret_cast<const mb::bf16x8*>(g)[i], f);
}
template <>
__device__ __forceinline__ void load_grad8<float>(const float* g, size_t i, float* f) {
  float4 a = reinterpret_cast<const float4*>(g)[2 * i];
  float4 b = reinterpret_cast<const float4*>(g)[2 * i + 1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

__device__ __forceinline__ void adam_update(float& p, float& m, float& v, float g,
                                            const AdamArgs& a) {
  g *= a.inv_scale;
  if (!a.adamw) g += a.weight_decay * p;
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  float mh = m / a.bias_c1;
  float vh = v / a.bias_c2;
  float upd = mh / (sqrtf(vh) + a.eps);
  if (a.adamw) upd += a.weight_decay * p;
  p -= a.lr * upd;
}

template <typename GradT>
__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ master, float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq,
            const GradT* __restrict__ grad, __nv_bfloat16* __restrict__ model, size_t n,
            AdamArgs a) {
  const size_t nvec = n >> 3;
  for (size_t i = blockIdx.x * static_cast<size_t>(256) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * 256) {
    float g[8], p[8], m[8], v[8];
    load_grad8<GradT>(grad, i, g);
    load_grad8<float>(master, i, p);
    load_grad8<float>(exp_avg, i, m);
    load_grad8<float>(exp_avg_sq, i, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) adam_update(p[k], m[k], v[k], g[k], a);
    reinterpret_cast<float4*>(master)[2 * i] = make_float4(p[0], p[1], p[2], p[3]);
    reinterpret_cast<float4*>(master)[2 * i + 1] = make_float4(p[4], p[5], p[6], p[7]);
    reinterpret_cast<float4*>(exp_avg)[2 * i] = make_float4(m[0], m[1], m[2], m[3]);
    reinterpret_cast<float4*>(exp_avg)[2 * i + 1] = make_float4(m[4], m[5], m[6], m[7]);
    reinterpret_cast<float4*>(exp_avg_sq)[2 * i] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(exp_avg_sq)[2 * i + 1] = make_float4(v[4], v[5], v[6], v[7]);
    if (model) reinterpret_cast<mb::bf16x8*>(model)[i] = mb::pack8(p);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    size_t j = (nvec << 3) + threadIdx.x;
    float p = master[j], m = exp_avg[j], v = exp_avg_sq[j];
    adam_update(p, m, v, static_cast<float>(grad[j]), a);
    master[j] = p;
    exp_avg[j] = m;
    exp_avg_sq[j] = v;
    if (model) model[j] = __float2bfloat16(p);
  }
}

}  // namespace

// All arrays hold `n` elements and must be 32-byte aligned.  `model` may be null.
MB_API int mb_adam_step(float* master, float* exp_avg, float* exp_avg_sq, const void* grad,
                        int grad_is_fp32, void* model, size_t n, float lr, float beta1, float beta2,
                        float eps, float weight_decay, int step, float inv_scale, int adamw,
                        cudaStream_t stream) {
  if (!n) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias_c1 = 1.f - powf(beta1, static_cast<float>(step));
  a.bias_c2 = 1.f - powf(beta2, static_cast<float>(step));
  a.inv_scale = inv_scale;
  a.adamw = adamw;
  size_t nvec = (n + 7) / 8;
  size_t g = (nvec + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  if (grad_is_fp32)
    adam_kernel<float><<<static_cast<int>(g), 256, 0, stream>>>(
        master, exp_avg, exp_avg_sq, reinterpret_cast<const float*>(grad),
        reinterpret_cast<__nv_bfloat16*>(model), n, a);
  else
    adam_kernel<__nv_bfloat16><<<static_cast<int>(g), 256, 0, stream>>>(
        master, exp_avg, exp_avg_sq, reinterpret_cast<const __nv_bfloat16*>(grad),
        reinterpret_cast<__nv_bfloat16*>(model), n, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
