// Bandwidth-bound elementwise kernels of the transformer block, all on 16-byte
// bf16 vectors: GELU(tanh) and SwiGLU forward/backward, bias-dropout-add, rotary
// embedding on packed qkv, embedding lookup / scatter, bias-gradient column sums,
// dtype casts and gradient accumulation.
//
// Reference counterparts: jiterator swiglu (mist/modules/activations.py:115-149),
// TorchScript bias_gelu / bias_dropout_add (mist/modules/activations.py:16-112,
// mist/model/transformer.py:535-546), Triton rotary kernel
// (mist/modules/triton/rotary.py:20-51), csrc/rotary/rotary_cuda.cu:9-44,
// embedding modules (mist/modules/embedding.py:207-281).
#include "common.cuh"

namespace {

constexpr int kBlock = 256;

inline int grid_for(size_t nvec, int cap = 148 * 16) {
  size_t g = (nvec + kBlock - 1) / kBlock;
  if (g > static_cast<size_t>(cap)) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

// ------------------------------------------------------------------ philox
// Philox4x32-10 counter RNG: 4 uniform 32-bit words per (seed, counter).
__device__ __forceinline__ uint4 philox(uint64_t seed, uint64_t ctr) {
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  uint32_t c0 = static_cast<uint32_t>(ctr), c1 = static_cast<uint32_t>(ctr >> 32), c2 = 0, c3 = 0;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// ------------------------------------------------------------- activations
// y = gelu_tanh(x + bias)
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ bias,
                                __nv_bfloat16* __restrict__ y, size_t nvec, int cols) {
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    float f[8];
    mb::unpack8(reinterpret_cast<const mb::bf16x8*>(x)[i], f);
    if (bias) {
      float b[8];
      mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(bias + (i * 8) % cols), b);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] += b[k];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = mb::gelu_tanh(f[k]);
    reinterpret_cast<mb::bf16x8*>(y)[i] = mb::pack8(f);
  }
}
// dx = dy * gelu'(x + bias)
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ bias,
                                __nv_bfloat16* __restrict__ dx, size_t nvec, int cols) {
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    float f[8], g[8];
    mb::unpack8(reinterpret_cast<const mb::bf16x8*>(x)[i], f);
    mb::unpack8(reinterpret_cast<const mb::bf16x8*>(dy)[i], g);
    if (bias) {
      float b[8];
      mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(bias + (i * 8) % cols), b);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] += b[k];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] *= mb::gelu_tanh_grad(f[k]);
    reinterpret_cast<mb::bf16x8*>(dx)[i] = mb::pack8(g);
  }
}

// in: [rows][2F] = [gate | up];  out[rows][F] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in,
                                  __nv_bfloat16* __restrict__ out, size_t rows, int F) {
  const int vpr = F >> 3;
  const size_t nvec = rows * vpr;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    size_t r = i / vpr;
    int c = static_cast<int>(i - r * vpr) * 8;
    float g[8], u[8];
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(in + r * 2 * F + c), g);
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(in + r * 2 * F + F + c), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = mb::silu(g[k]) * u[k];
    *reinterpret_cast<mb::bf16x8*>(out + r * F + c) = mb::pack8(g);
  }
}
// din[rows][2F] = [dgate | dup]
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                  const __nv_bfloat16* __restrict__ in,
                                  __nv_bfloat16* __restrict__ din, size_t rows, int F) {
  const int vpr = F >> 3;
  const size_t nvec = rows * vpr;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    size_t r = i / vpr;
    int c = static_cast<int>(i - r * vpr) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(in + r * 2 * F + c), g);
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(in + r * 2 * F + F + c), u);
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(dout + r * F + c), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float s = 1.f / (1.f + __expf(-g[k]));
      float sl = g[k] * s;
      dg[k] = d[k] * u[k] * (s + sl * (1.f - s));
      du[k] = d[k] * sl;
    }
    *reinterpret_cast<mb::bf16x8*>(din + r * 2 * F + c) = mb::pack8(dg);
    *reinterpret_cast<mb::bf16x8*>(din + r * 2 * F + F + c) = mb::pack8(du);
  }
}

// out = residual + dropout(x + bias, p).  The mask is not stored: the backward
// pass regenerates it from (seed, element index).
__global__ void bias_dropout_add_kernel(const __nv_bfloat16* __restrict__ x,
                                        const __nv_bfloat16* __restrict__ bias,
                                        const __nv_bfloat16* __restrict__ residual,
                                        __nv_bfloat16* __restrict__ out, size_t nvec, int cols,
                                        float p, uint64_t seed) {
  const float scale = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const uint32_t thresh = static_cast<uint32_t>(p * 4294967296.0);
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    float f[8];
    mb::unpack8(reinterpret_cast<const mb::bf16x8*>(x)[i], f);
    if (bias) {
      float b[8];
      mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(bias + (i * 8) % cols), b);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] += b[k];
    }
    if (p > 0.f) {
      uint4 r0 = philox(seed, 2 * i), r1 = philox(seed, 2 * i + 1);
      uint32_t rr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = rr[k] < thresh ? 0.f : f[k] * scale;
    }
    if (residual) {
      float r[8];
      mb::unpack8(reinterpret_cast<const mb::bf16x8*>(residual)[i], r);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] += r[k];
    }
    reinterpret_cast<mb::bf16x8*>(out)[i] = mb::pack8(f);
  }
}
// dx = dropout_mask(dout) (same seed)
__global__ void dropout_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                   __nv_bfloat16* __restrict__ dx, size_t nvec, float p,
                                   uint64_t seed) {
  const float scale = 1.f / (1.f - p);
  const uint32_t thresh = static_cast<uint32_t>(p * 4294967296.0);
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    float f[8];
    mb::unpack8(reinterpret_cast<const mb::bf16x8*>(dout)[i], f);
    uint4 r0 = philox(seed, 2 * i), r1 = philox(seed, 2 * i + 1);
    uint32_t rr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = rr[k] < thresh ? 0.f : f[k] * scale;
    reinterpret_cast<mb::bf16x8*>(dx)[i] = mb::pack8(f);
  }
}

// ------------------------------------------------------------------ rotary
// In place on packed qkv [tokens][3][heads][d]; rotates the first `rot` channels of
// q and k, non-interleaved halves (x1 = [0, rot/2), x2 = [rot/2, rot)).
// cos/sin: [seq][rot/2] fp32; token t has position t % seq.  conj negates sin.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosv,
                            const float* __restrict__ sinv, size_t tokens, int seq, int heads,
                            int d, int rot, int conj, int n_rotated /* 2 = q and k */,
                            int row_stride) {
  const int half = rot >> 1;
  const int vph = half >> 3;  // 8-wide vectors per half
  const size_t total = tokens * n_rotated * heads * vph;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    int v = static_cast<int>(i % vph);
    size_t r = i / vph;
    int hd = static_cast<int>(r % heads);
    r /= heads;
    int which = static_cast<int>(r % n_rotated);
    size_t tok = r / n_rotated;
    int pos = static_cast<int>(tok % seq);
    __nv_bfloat16* base =
        qkv + tok * row_stride + (static_cast<size_t>(which) * heads + hd) * d + 8 * v;
    float x1[8], x2[8], o1[8], o2[8];
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(base), x1);
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(base + half), x2);
    const float* c = cosv + static_cast<size_t>(pos) * half + 8 * v;
    const float* s = sinv + static_cast<size_t>(pos) * half + 8 * v;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float cs = c[k], sn = conj ? -s[k] : s[k];
      o1[k] = x1[k] * cs - x2[k] * sn;
      o2[k] = x1[k] * sn + x2[k] * cs;
    }
    *reinterpret_cast<mb::bf16x8*>(base) = mb::pack8(o1);
    *reinterpret_cast<mb::bf16x8*>(base + half) = mb::pack8(o2);
  }
}

// --------------------------------------------------------------- embedding
// out[t] = wte[ids[t] - v0] (zero when the id is outside [v0, v1)) + wpe[t % seq]
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ wte,
                                     const __nv_bfloat16* __restrict__ wpe,
                                     __nv_bfloat16* __restrict__ out, size_t tokens, int seq, int h,
                                     int v0, int v1) {
  const int vpr = h >> 3;
  const size_t nvec = tokens * vpr;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    size_t t = i / vpr;
    int c = static_cast<int>(i - t * vpr) * 8;
    int64_t id = ids[t];
    float f[8];
    if (id >= v0 && id < v1)
      mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(wte + (id - v0) * h + c), f);
    else {
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = 0.f;
    }
    if (wpe) {
      float p[8];
      mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(wpe + (t % seq) * h + c), p);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] += p[k];
    }
    *reinterpret_cast<mb::bf16x8*>(out + t * h + c) = mb::pack8(f);
  }
}
// dwte[ids[t] - v0] += dout[t]   (fp32 accumulation buffer, atomics)
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dwte, size_t tokens, int h, int v0,
                                     int v1) {
  const int vpr = h >> 3;
  const size_t nvec = tokens * vpr;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    size_t t = i / vpr;
    int c = static_cast<int>(i - t * vpr) * 8;
    int64_t id = ids[t];
    if (id < v0 || id >= v1) continue;
    float f[8];
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(dout + t * h + c), f);
    float* dst = dwte + (id - v0) * h + c;
#pragma unroll
    for (int k = 0; k < 8; ++k) atomicAdd(dst + k, f[k]);
  }
}
// dwpe[s] = sum_b dout[b*seq + s]
__global__ void pos_embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                         float* __restrict__ dwpe, int batch, int seq, int h) {
  const int vpr = h >> 3;
  const size_t nvec = static_cast<size_t>(seq) * vpr;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    size_t s = i / vpr;
    int c = static_cast<int>(i - s * vpr) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int b = 0; b < batch; ++b) {
      float f[8];
      mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(
                      dout + (static_cast<size_t>(b) * seq + s) * h + c), f);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += f[k];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) dwpe[s * h + c + k] += acc[k];
  }
}

// --------------------------------------------------------- column reduction
// out[c] (+)= sum_r x[r][c]; used for bias gradients.  Two stages through scratch:
// stage 1 writes [parts][cols] partial sums, stage 2 adds them up.
__global__ void colsum_stage1(const __nv_bfloat16* __restrict__ x, float* __restrict__ part,
                              int rows, int cols, int rows_per_part) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= cols) return;
  const int r0 = blockIdx.y * rows_per_part;
  const int r1 = min(rows, r0 + rows_per_part);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int r = r0; r < r1; ++r) {
    float f[8];
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(x + static_cast<size_t>(r) * cols + c), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += f[k];
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) part[static_cast<size_t>(blockIdx.y) * cols + c + k] = acc[k];
}
template <typename OutT>
__global__ void colsum_stage2(const float* __restrict__ part, OutT* __restrict__ out, int parts,
                              int cols, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float a = 0.f;
  for (int p = 0; p < parts; ++p) a += part[static_cast<size_t>(p) * cols + c];
  if (accumulate) a += static_cast<float>(out[c]);
  out[c] = static_cast<OutT>(a);
}

// ------------------------------------------------------------------- casts
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                        size_t n, float scale) {
  const size_t nvec = n >> 3;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    float4 a = reinterpret_cast<const float4*>(in)[2 * i];
    float4 b = reinterpret_cast<const float4*>(in)[2 * i + 1];
    float f[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale,
                  b.x * scale, b.y * scale, b.z * scale, b.w * scale};
    reinterpret_cast<mb::bf16x8*>(out)[i] = mb::pack8(f);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    size_t j = (nvec << 3) + threadIdx.x;
    out[j] = __float2bfloat16(in[j] * scale);
  }
}
// dst(fp32) = (accumulate ? dst : 0) + scale * src(bf16)
__global__ void axpy_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src,
                                        float* __restrict__ dst, size_t n, float scale,
                                        int accumulate) {
  const size_t nvec = n >> 3;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    float f[8];
    mb::unpack8(reinterpret_cast<const mb::bf16x8*>(src)[i], f);
    float4 a = make_float4(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale);
    float4 b = make_float4(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale);
    if (accumulate) {
      float4 ea = reinterpret_cast<const float4*>(dst)[2 * i];
      float4 eb = reinterpret_cast<const float4*>(dst)[2 * i + 1];
      a.x += ea.x; a.y += ea.y; a.z += ea.z; a.w += ea.w;
      b.x += eb.x; b.y += eb.y; b.z += eb.z; b.w += eb.w;
    }
    reinterpret_cast<float4*>(dst)[2 * i] = a;
    reinterpret_cast<float4*>(dst)[2 * i + 1] = b;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    size_t j = (nvec << 3) + threadIdx.x;
    float v = __bfloat162float(src[j]) * scale;
    dst[j] = accumulate ? dst[j] + v : v;
  }
}
// dst(bf16) += src(bf16)
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ src,
                                __nv_bfloat16* __restrict__ dst, size_t n) {
  const size_t nvec = n >> 3;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    float a[8], b[8];
    mb::unpack8(reinterpret_cast<const mb::bf16x8*>(src)[i], a);
    mb::unpack8(reinterpret_cast<const mb::bf16x8*>(dst)[i], b);
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] += b[k];
    reinterpret_cast<mb::bf16x8*>(dst)[i] = mb::pack8(a);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    size_t j = (nvec << 3) + threadIdx.x;
    dst[j] = __float2bfloat16(__bfloat162float(dst[j]) + __bfloat162float(src[j]));
  }
}

#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFM(p) reinterpret_cast<__nv_bfloat16*>(p)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -4)

}  // namespace

MB_API int mb_gelu_fwd(const void* x, const void* bias, void* y, size_t rows, int cols,
                       cudaStream_t s) {
  if (cols % 8) return -1;
  size_t nvec = rows * cols / 8;
  if (!nvec) return 0;
  gelu_fwd_kernel<<<grid_for(nvec), kBlock, 0, s>>>(BF(x), BF(bias), BFM(y), nvec, cols);
  return LAUNCH_OK();
}
MB_API int mb_gelu_bwd(const void* dy, const void* x, const void* bias, void* dx, size_t rows,
                       int cols, cudaStream_t s) {
  if (cols % 8) return -1;
  size_t nvec = rows * cols / 8;
  if (!nvec) return 0;
  gelu_bwd_kernel<<<grid_for(nvec), kBlock, 0, s>>>(BF(dy), BF(x), BF(bias), BFM(dx), nvec, cols);
  return LAUNCH_OK();
}
MB_API int mb_swiglu_fwd(const void* in, void* out, size_t rows, int F, cudaStream_t s) {
  if (F % 8) return -1;
  if (!rows) return 0;
  swiglu_fwd_kernel<<<grid_for(rows * F / 8), kBlock, 0, s>>>(BF(in), BFM(out), rows, F);
  return LAUNCH_OK();
}
MB_API int mb_swiglu_bwd(const void* dout, const void* in, void* din, size_t rows, int F,
                         cudaStream_t s) {
  if (F % 8) return -1;
  if (!rows) return 0;
  swiglu_bwd_kernel<<<grid_for(rows * F / 8), kBlock, 0, s>>>(BF(dout), BF(in), BFM(din), rows, F);
  return LAUNCH_OK();
}
MB_API int mb_bias_dropout_add(const void* x, const void* bias, const void* residual, void* out,
                               size_t rows, int cols, float p, uint64_t seed, cudaStream_t s) {
  if (cols % 8) return -1;
  size_t nvec = rows * cols / 8;
  if (!nvec) return 0;
  bias_dropout_add_kernel<<<grid_for(nvec), kBlock, 0, s>>>(BF(x), BF(bias), BF(residual), BFM(out),
                                                           nvec, cols, p, seed);
  return LAUNCH_OK();
}
MB_API int mb_dropout_bwd(const void* dout, void* dx, size_t n, float p, uint64_t seed,
                          cudaStream_t s) {
  if (n % 8) return -1;
  if (!n) return 0;
  dropout_bwd_kernel<<<grid_for(n / 8), kBlock, 0, s>>>(BF(dout), BFM(dx), n / 8, p, seed);
  return LAUNCH_OK();
}
// qkv: [tokens][row_stride]; q heads at offset 0, k heads at heads*d.
MB_API int mb_rope(void* qkv, const float* cosv, const float* sinv, size_t tokens, int seq,
                   int heads, int d, int rot, int conj, int n_rotated, int row_stride,
                   cudaStream_t s) {
  if (rot % 16 || d % 8 || row_stride % 8) return -1;
  size_t total = tokens * n_rotated * heads * (rot / 16);
  if (!total) return 0;
  rope_kernel<<<grid_for(total), kBlock, 0, s>>>(BFM(qkv), cosv, sinv, tokens, seq, heads, d, rot,
                                                conj, n_rotated, row_stride);
  return LAUNCH_OK();
}
MB_API int mb_embedding_fwd(const int64_t* ids, const void* wte, const void* wpe, void* out,
                            size_t tokens, int seq, int h, int v0, int v1, cudaStream_t s) {
  if (h % 8) return -1;
  if (!tokens) return 0;
  embedding_fwd_kernel<<<grid_for(tokens * h / 8), kBlock, 0, s>>>(ids, BF(wte), BF(wpe), BFM(out),
                                                                  tokens, seq, h, v0, v1);
  return LAUNCH_OK();
}
MB_API int mb_embedding_bwd(const int64_t* ids, const void* dout, float* dwte, float* dwpe,
                            int batch, int seq, int h, int v0, int v1, cudaStream_t s) {
  if (h % 8) return -1;
  size_t tokens = static_cast<size_t>(batch) * seq;
  if (!tokens) return 0;
  embedding_bwd_kernel<<<grid_for(tokens * h / 8), kBlock, 0, s>>>(ids, BF(dout), dwte, tokens, h,
                                                                  v0, v1);
  if (dwpe)
    pos_embedding_bwd_kernel<<<grid_for(static_cast<size_t>(seq) * h / 8), kBlock, 0, s>>>(
        BF(dout), dwpe, batch, seq, h);
  return LAUNCH_OK();
}
// scratch: ceil(rows / 256) * cols floats.
MB_API int mb_colsum(const void* x, void* out, float* scratch, int rows, int cols, int out_fp32,
                     int accumulate, cudaStream_t s) {
  if (cols % 8) return -1;
  if (!rows) return 0;
  const int rpp = 256;
  int parts = (rows + rpp - 1) / rpp;
  dim3 g1((cols / 8 + 127) / 128, parts);
  colsum_stage1<<<g1, 128, 0, s>>>(BF(x), scratch, rows, cols, rpp);
  if (out_fp32)
    colsum_stage2<float><<<(cols + 255) / 256, 256, 0, s>>>(scratch, reinterpret_cast<float*>(out),
                                                            parts, cols, accumulate);
  else
    colsum_stage2<__nv_bfloat16><<<(cols + 255) / 256, 256, 0, s>>>(scratch, BFM(out), parts, cols,
                                                                    accumulate);
  return LAUNCH_OK();
}
MB_API int mb_cast_f32_to_bf16(const float* in, void* out, size_t n, float scale, cudaStream_t s) {
  if (!n) return 0;
  cast_f32_to_bf16_kernel<<<grid_for((n + 7) / 8), kBlock, 0, s>>>(in, BFM(out), n, scale);
  return LAUNCH_OK();
}
MB_API int mb_axpy_bf16_to_f32(const void* src, float* dst, size_t n, float scale, int accumulate,
                               cudaStream_t s) {
  if (!n) return 0;
  axpy_bf16_to_f32_kernel<<<grid_for((n + 7) / 8), kBlock, 0, s>>>(BF(src), dst, n, scale,
                                                                  accumulate);
  return LAUNCH_OK();
}
MB_API int mb_add_bf16(const void* src, void* dst, size_t n, cudaStream_t s) {
  if (!n) return 0;
  add_bf16_kernel<<<grid_for((n + 7) / 8), kBlock, 0, s>>>(BF(src), BFM(dst), n);
  return LAUNCH_OK();
}

// ------------------------------------------------------------- allocation-free variant
// Column sums with the inter-stage partial sums in a fixed device array (see no_alloc.h).
#include "no_alloc.h"
#include <stdio.h>

namespace {
constexpr long kStaticScratchFloats = 1L << 20;   // 4 MiB per GPU
constexpr int kMaxDevices = 64;
}  // namespace

// In host code this name is only a handle for the runtime; the device address is obtained
// once per GPU with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_colsum_scratch[kStaticScratchFloats];

namespace {
float* g_colsum_scratch_addr[kMaxDevices] = {nullptr};

float* colsum_static_scratch() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (!g_colsum_scratch_addr[dev]) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_colsum_scratch) != cudaSuccess) return nullptr;
    g_colsum_scratch_addr[dev] = p;
  }
  return g_colsum_scratch_addr[dev];
}
}  // namespace

MB_API long mb_colsum_static_capacity(void) { return kStaticScratchFloats; }

MB_API int mb_colsum_static(const void* x, void* out, int rows, int cols, int out_fp32, int accumulate,
                            cudaStream_t s) {
  if (cols <= 0 || rows < 0 || cols % 8) return -1;
  if (!rows) return 0;
  const int rpp = 256;
  const int parts = (rows + rpp - 1) / rpp;
  const long need = static_cast<long>(parts) * cols;
  if (need > kStaticScratchFloats) {
    fprintf(stderr,
            "mb_colsum_static: %d x %d needs %ld scratch floats, the built-in array holds %ld; "
            "use mb_colsum with a caller-provided buffer\n",
            rows, cols, need, kStaticScratchFloats);
    return -22;
  }
  float* scratch = colsum_static_scratch();
  if (!scratch) return -3;
  dim3 g1((cols / 8 + 127) / 128, parts);
  colsum_stage1<<<g1, 128, 0, s>>>(BF(x), scratch, rows, cols, rpp);
  if (out_fp32)
    colsum_stage2<float><<<(cols + 255) / 256, 256, 0, s>>>(scratch, reinterpret_cast<float*>(out), parts, cols,
                                                            accumulate);
  else
    colsum_stage2<__nv_bfloat16><<<(cols + 255) / 256, 256, 0, s>>>(scratch, BFM(out), parts, cols, accumulate);
  return LAUNCH_OK();
}
