// Row-wise softmax family: vocab-parallel cross entropy and the scaled causal
// softmax of the non-flash attention path.
//
// Cross entropy (reference: pure-torch _VocabParallelCrossEntropy,
// mist/modules/losses.py:48-176; unused csrc/xentropy/xentropy_kernel.cu:429-744):
//   stage 1  per row, over this rank's vocab slice [v0, v1): running max, sum of
//            exp relative to that max, and the target logit when the label falls in
//            the slice -> stats[row] = {max, sumexp, target}.  One read of the row.
//   (the tensor-parallel group combines the stats with max / sum all-reduces)
//   stage 2  loss = log(sumexp) + max - target; the backward pass rewrites the
//            logits in place as (softmax - onehot) * grad_scale.
//
// Scaled causal softmax (reference: csrc/fused_softmax/
// scaled_upper_triang_masked_softmax.h:113-367): one CTA per row of [.., sq, sk].
#include "common.cuh"

namespace {

constexpr int kThreads = 512;

__global__ void __launch_bounds__(kThreads)
xent_stats_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ labels,
                  float* __restrict__ stats, int cols, int ld, int v0) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* x = logits + row * ld;
  const int nvec = cols >> 3;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += kThreads) {
    float f[8];
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(x + 8 * i), f);
    float lm = f[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) lm = fmaxf(lm, f[k]);
    float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc += __expf(f[k] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < cols; i += kThreads) {
    float f = __bfloat162float(x[i]);
    float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  float gm = mb::block_max(m, red);
  float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  float gs = mb::block_sum(contrib, red);
  if (threadIdx.x == 0) {
    int64_t lab = labels[row] - v0;
    float t = (lab >= 0 && lab < cols) ? __bfloat162float(x[lab]) : 0.f;
    stats[3 * row + 0] = gm;
    stats[3 * row + 1] = gs;
    stats[3 * row + 2] = t;
  }
}

// loss[row] = log(sum) + max - target ; lse[row] = log(sum) + max
__global__ void xent_loss_kernel(const float* __restrict__ stats, const int64_t* __restrict__ labels,
                                 float* __restrict__ loss, float* __restrict__ lse, int rows,
                                 int ignore_index) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float l = __logf(stats[3 * r + 1]) + stats[3 * r];
  lse[r] = l;
  loss[r] = (labels[r] == ignore_index) ? 0.f : l - stats[3 * r + 2];
}

// logits <- (exp(logit - lse) - [col == label]) * gscale[row] * scale   (in place)
__global__ void __launch_bounds__(kThreads)
xent_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ labels,
                const float* __restrict__ lse, const float* __restrict__ gloss, float scale,
                int cols, int ld, int v0, int ignore_index, int gloss_is_scalar) {
  const size_t row = blockIdx.x;
  __nv_bfloat16* x = logits + row * ld;
  const int nvec = cols >> 3;
  const int64_t lab_g = labels[row];
  const int64_t lab = lab_g - v0;
  const float l = lse[row];
  const float g = (lab_g == ignore_index) ? 0.f : (gloss_is_scalar ? gloss[0] : gloss[row]) * scale;
  for (int i = threadIdx.x; i < nvec; i += kThreads) {
    float f[8];
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(x + 8 * i), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float p = __expf(f[k] - l);
      if (8 * i + k == lab) p -= 1.f;
      f[k] = p * g;
    }
    *reinterpret_cast<mb::bf16x8*>(x + 8 * i) = mb::pack8(f);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < cols; i += kThreads) {
    float p = __expf(__bfloat162float(x[i]) - l);
    if (i == lab) p -= 1.f;
    x[i] = __float2bfloat16(p * g);
  }
}

// y[r, c] = softmax_c(scale * x[r, c]) over c <= (r % sq) + (sk - sq)   (causal), else 0
__global__ void __launch_bounds__(256)
causal_softmax_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                          int sq, int sk, float scale, int causal) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const int qi = static_cast<int>(row % sq);
  const int valid = causal ? min(sk, qi + 1 + (sk - sq)) : sk;
  const __nv_bfloat16* xr = x + row * sk;
  __nv_bfloat16* yr = y + row * sk;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < valid; c += blockDim.x)
    m = fmaxf(m, __bfloat162float(xr[c]) * scale);
  m = mb::block_max(m, red);
  float s = 0.f;
  for (int c = threadIdx.x; c < valid; c += blockDim.x)
    s += __expf(__bfloat162float(xr[c]) * scale - m);
  s = mb::block_sum(s, red);
  const float inv = 1.f / s;
  for (int c = threadIdx.x; c < sk; c += blockDim.x) {
    float p = c < valid ? __expf(__bfloat162float(xr[c]) * scale - m) * inv : 0.f;
    yr[c] = __float2bfloat16(p);
  }
}
// dx = scale * y * (dy - sum_c(dy * y))
__global__ void __launch_bounds__(256)
causal_softmax_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ y,
                          __nv_bfloat16* __restrict__ dx, int sk, float scale) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* dyr = dy + row * sk;
  const __nv_bfloat16* yr = y + row * sk;
  __nv_bfloat16* dxr = dx + row * sk;
  float s = 0.f;
  for (int c = threadIdx.x; c < sk; c += blockDim.x)
    s += __bfloat162float(dyr[c]) * __bfloat162float(yr[c]);
  s = mb::block_sum(s, red);
  for (int c = threadIdx.x; c < sk; c += blockDim.x) {
    float yy = __bfloat162float(yr[c]);
    dxr[c] = __float2bfloat16(scale * yy * (__bfloat162float(dyr[c]) - s));
  }
}

}  // namespace

// stats: [rows][3] floats.  logits row stride `ld` elements (ld % 8 == 0).
MB_API int mb_xent_stats(const void* logits, const int64_t* labels, float* stats, int rows,
                         int cols, int ld, int v0, cudaStream_t s) {
  if (ld % 8) return -1;
  if (!rows) return 0;
  xent_stats_kernel<<<rows, kThreads, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(logits), labels,
                                              stats, cols, ld, v0);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
MB_API int mb_xent_loss(const float* stats, const int64_t* labels, float* loss, float* lse, int rows,
                        int ignore_index, cudaStream_t s) {
  if (!rows) return 0;
  xent_loss_kernel<<<(rows + 255) / 256, 256, 0, s>>>(stats, labels, loss, lse, rows, ignore_index);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
MB_API int mb_xent_bwd(void* logits, const int64_t* labels, const float* lse, const float* gloss,
                       float scale, int rows, int cols, int ld, int v0, int ignore_index,
                       int gloss_is_scalar, cudaStream_t s) {
  if (ld % 8) return -1;
  if (!rows) return 0;
  xent_bwd_kernel<<<rows, kThreads, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(logits), labels, lse,
                                            gloss, scale, cols, ld, v0, ignore_index,
                                            gloss_is_scalar);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
MB_API int mb_causal_softmax_fwd(const void* x, void* y, size_t rows, int sq, int sk, float scale,
                                 int causal, cudaStream_t s) {
  if (!rows) return 0;
  causal_softmax_fwd_kernel<<<static_cast<unsigned>(rows), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(y), sq, sk, scale,
      causal);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
MB_API int mb_causal_softmax_bwd(const void* dy, const void* y, void* dx, size_t rows, int sk,
                                 float scale, cudaStream_t s) {
  if (!rows) return 0;
  causal_softmax_bwd_kernel<<<static_cast<unsigned>(rows), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(y),
      reinterpret_cast<__nv_bfloat16*>(dx), sk, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
