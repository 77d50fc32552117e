// Single-query attention against a key/value cache (autoregressive decoding).
//
//   o[b, h, :] = softmax(scale * q[b, h, :] . K[b, 0:len, kv(h), :]) V[b, 0:len, kv(h), :]
//
// One CTA per (head, batch element), eight warps that take the cached positions round-robin.
// A lane owns eight consecutive head-dimension elements (one 16-byte load of K and of V per
// position), the dot product is a warp reduction, and each warp keeps a running (max, sum,
// output) triple that the CTA merges at the end.  The kernel is bound by reading the cache
// once; there is no tensor-core work in a 1 x len product.
//
// Reference counterpart: csrc/ft_attention (FasterTransformer masked_multihead_attention,
// decoder_masked_multihead_attention_template.hpp:865; binding ft_attention.cpp:226), used by
// the inference path of mist/modules/mha.py:531-575.
#include "common.cuh"

#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFM(p) reinterpret_cast<__nv_bfloat16*>(p)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -4)

namespace {

constexpr int kWarps = 8;
constexpr int kMaxD = 256;

__global__ void __launch_bounds__(kWarps * 32)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ o, int nh, int group, int d,
                   int len, long k_sb, long k_ss, long k_sh, long v_sb, long v_ss, long v_sh, float scale_log2) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e0 = lane * 8;
  const bool live = e0 < d;                 // d is a multiple of 8, so a lane is all in or all out
  const int hk = h / group;

  float qf[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live) mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(q + (static_cast<long>(b) * nh + h) * d + e0), qf);
  const __nv_bfloat16* kb = k + b * k_sb + hk * k_sh + e0;
  const __nv_bfloat16* vb = v + b * v_sb + hk * v_sh + e0;

  float m = -INFINITY, l = 0.f;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = warp; j < len; j += kWarps) {
    float kf[8], vf[8], dot = 0.f;
    if (live) {
      mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(kb + j * k_ss), kf);
      mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(vb + j * v_ss), vf);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot += qf[i] * kf[i];
    }
    dot = mb::warp_sum(dot) * scale_log2;           // every lane gets the full score (log2 domain)
    const float m_new = fmaxf(m, dot);
    const float corr = exp2f(m - m_new);             // exp2f(-inf) = 0 on the first position
    const float p = exp2f(dot - m_new);
    l = l * corr + p;
    if (live) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = acc[i] * corr + p * vf[i];
    }
    m = m_new;
  }

  __shared__ float s_m[kWarps], s_l[kWarps];
  __shared__ float s_acc[kWarps][kMaxD];
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < 8; ++i) s_acc[warp][e0 + i] = acc[i];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < d; e += kWarps * 32) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w]);
    float L = 0.f, out = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float f = (s_m[w] == -INFINITY) ? 0.f : exp2f(s_m[w] - M);   // warps that saw no position
      L += s_l[w] * f;
      out += s_acc[w][e] * f;
    }
    o[(static_cast<long>(b) * nh + h) * d + e] = __float2bfloat16(L > 0.f ? out / L : 0.f);
  }
}

}  // namespace

// q, o: [batch][nh][d] contiguous bf16.  k, v: element strides (batch, position, kv head) with unit
// stride along d; every row start must be 16-byte aligned (strides multiples of 8).  d % 8 == 0,
// d <= 256, nh % nh_kv == 0, len >= 1.
MB_API int mb_decode_attn(const void* q, const void* k, const void* v, void* o, int batch, int nh, int nh_kv, int d,
                          int len, long k_sb, long k_ss, long k_sh, long v_sb, long v_ss, long v_sh, float scale,
                          cudaStream_t stream) {
  if (batch <= 0 || nh <= 0) return 0;
  if (d % 8 || d > kMaxD || d <= 0 || nh_kv <= 0 || nh % nh_kv || len < 1) return -1;
  if ((k_sb | k_ss | k_sh | v_sb | v_ss | v_sh) & 7) return -1;
  dim3 grid(nh, batch);
  decode_attn_kernel<<<grid, kWarps * 32, 0, stream>>>(BF(q), BF(k), BF(v), BFM(o), nh, nh / nh_kv, d, len, k_sb, k_ss,
                                                     k_sh, v_sb, v_ss, v_sh, scale * 1.4426950408889634f);
  return LAUNCH_OK();
}
