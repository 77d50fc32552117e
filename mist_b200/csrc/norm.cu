// LayerNorm / RMSNorm forward and backward with the residual add folded in.
//
//   forward :  x = x0 (+ residual);  z = (x - mean) * rstd * gamma (+ beta)
//              optionally writes x back as the new residual stream
//   backward:  dx = rstd * (dz*gamma - mean(dz*gamma) - xhat * mean(dz*gamma*xhat)) (+ dres_in)
//              dgamma / dbeta reduced per CTA into a scratch matrix, then summed by
//              a second kernel
//
// Same operator family as the reference's dropout_add_ln extension
// (reference: csrc/layer_norm/ln_api.cpp:832-846, ln_fwd_kernels.cuh:18-20,
// ln_bwd_kernels.cuh:10-12,301-303) but written for one shape-generic kernel:
// rows are kept in registers as 16-byte vectors, `tpr` threads cooperate on a
// row and several rows share a CTA, the grid is persistent over row groups.
// The kernels are bandwidth bound; they touch each element once per pass.
#include "common.cuh"
#include <stdlib.h>

namespace {

constexpr int kMaxVPT = 4;  // 16-byte vectors per thread (covers hidden <= 8 * VPT * tpr)

// Sum over the `tpr` threads that share a row.  `red` holds [rows_per_cta][8] floats.
template <int NVAL>
__device__ __forceinline__ void row_reduce(float (&v)[NVAL], float* red, int tpr, int rl, int tr) {
#pragma unroll
  for (int i = 0; i < NVAL; ++i) v[i] = mb::warp_sum(v[i]);
  if (tpr > 32) {
    const int wpr = tpr >> 5;  // warps per row
    const int w = tr >> 5;
    __syncthreads();
    if ((tr & 31) == 0) {
#pragma unroll
      for (int i = 0; i < NVAL; ++i) red[(rl * 8 + w) * NVAL + i] = v[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NVAL; ++i) {
      float s = 0.f;
      for (int j = 0; j < wpr; ++j) s += red[(rl * 8 + j) * NVAL + i];
      v[i] = s;
    }
  }
}

template <bool RMS, int VPT>
__global__ void __launch_bounds__(256, 4)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x0, const __nv_bfloat16* __restrict__ residual,
                const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
                __nv_bfloat16* __restrict__ z, __nv_bfloat16* __restrict__ x_out,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int h,
                float eps, int tpr, int rpc) {
  __shared__ float red[8 * 8 * 2];
  const int rl = threadIdx.x / tpr;  // row slot in this CTA
  const int tr = threadIdx.x % tpr;  // thread within the row
  const int nvec = h >> 3;
  const int groups = (rows + rpc - 1) / rpc;

  for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const int row = grp * rpc + rl;
    const bool active = row < rows;
    // The row stays in registers as packed bf16 (what later passes and the backward
    // pass see); gamma / beta are re-read per row and hit L1.
    mb::bf16x8 xp[VPT];
    float acc[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int vi = tr + i * tpr;
      if (active && vi < nvec) {
        size_t off = static_cast<size_t>(row) * h + 8 * vi;
        xp[i] = *reinterpret_cast<const mb::bf16x8*>(x0 + off);
        float x[8];
        mb::unpack8(xp[i], x);
        if (residual) {
          float r[8];
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(residual + off), r);
#pragma unroll
          for (int k = 0; k < 8; ++k) x[k] += r[k];
          xp[i] = mb::pack8(x);
          mb::unpack8(xp[i], x);
        }
        if (x_out) *reinterpret_cast<mb::bf16x8*>(x_out + off) = xp[i];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          acc[0] += x[k];
          acc[1] += x[k] * x[k];
        }
      }
    }
    row_reduce<2>(acc, red, tpr, rl, tr);
    float mean = RMS ? 0.f : acc[0] / h;
    float var = acc[1] / h - mean * mean;
    float rstd = rsqrtf(fmaxf(var, 0.f) + eps);
    if (active && tr == 0) {
      if (mean_out) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int vi = tr + i * tpr;
      if (active && vi < nvec) {
        float x[8], g[8], o[8];
        mb::unpack8(xp[i], x);
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(gamma + 8 * vi), g);
        if (!RMS && beta) {
          float b[8];
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(beta + 8 * vi), b);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] = (x[k] - mean) * rstd * g[k] + b[k];
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] = (x[k] - mean) * rstd * g[k];
        }
        *reinterpret_cast<mb::bf16x8*>(z + static_cast<size_t>(row) * h + 8 * vi) = mb::pack8(o);
      }
    }
  }
}

template <bool RMS, int VPT>
__global__ void __launch_bounds__(256, 2)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dz, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres_in,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ part_dgamma,
                float* __restrict__ part_dbeta, int rows, int h, int tpr, int rpc) {
  __shared__ float red[8 * 8 * 2];
  const int rl = threadIdx.x / tpr;
  const int tr = threadIdx.x % tpr;
  const int nvec = h >> 3;
  const int groups = (rows + rpc - 1) / rpc;

  float dg[VPT][8], db[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
#pragma unroll
    for (int k = 0; k < 8; ++k) dg[i][k] = db[i][k] = 0.f;
  }

  for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const int row = grp * rpc + rl;
    const bool active = row < rows;
    const float mean = (active && !RMS) ? mean_in[row] : 0.f;
    const float rstd = active ? rstd_in[row] : 0.f;
    mb::bf16x8 xp[VPT], dzp[VPT];  // packed: half the registers of fp32 copies
    float acc[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int vi = tr + i * tpr;
      if (active && vi < nvec) {
        size_t off = static_cast<size_t>(row) * h + 8 * vi;
        xp[i] = *reinterpret_cast<const mb::bf16x8*>(x + off);
        dzp[i] = *reinterpret_cast<const mb::bf16x8*>(dz + off);
        float xv[8], dzv[8], g[8];
        mb::unpack8(xp[i], xv);
        mb::unpack8(dzp[i], dzv);
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(gamma + 8 * vi), g);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float xh = (xv[k] - mean) * rstd;
          float dy = dzv[k] * g[k];
          dg[i][k] += dzv[k] * xh;
          db[i][k] += dzv[k];
          acc[0] += dy;
          acc[1] += dy * xh;
        }
      }
    }
    row_reduce<2>(acc, red, tpr, rl, tr);
    const float m1 = RMS ? 0.f : acc[0] / h;
    const float m2 = acc[1] / h;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int vi = tr + i * tpr;
      if (active && vi < nvec) {
        size_t off = static_cast<size_t>(row) * h + 8 * vi;
        float xv[8], dzv[8], g[8], o[8];
        mb::unpack8(xp[i], xv);
        mb::unpack8(dzp[i], dzv);
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(gamma + 8 * vi), g);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float xh = (xv[k] - mean) * rstd;
          o[k] = rstd * (dzv[k] * g[k] - m1 - xh * m2);
        }
        if (dres_in) {
          float r[8];
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(dres_in + off), r);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += r[k];
        }
        *reinterpret_cast<mb::bf16x8*>(dx + off) = mb::pack8(o);
      }
    }
  }
  // one partial row per (CTA, row slot)
  const size_t prow = static_cast<size_t>(blockIdx.x) * rpc + rl;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int vi = tr + i * tpr;
    if (vi < nvec) {
      float* pg = part_dgamma + prow * h + 8 * vi;
      *reinterpret_cast<float4*>(pg) = make_float4(dg[i][0], dg[i][1], dg[i][2], dg[i][3]);
      *reinterpret_cast<float4*>(pg + 4) = make_float4(dg[i][4], dg[i][5], dg[i][6], dg[i][7]);
      if (!RMS && part_dbeta) {
        float* pb = part_dbeta + prow * h + 8 * vi;
        *reinterpret_cast<float4*>(pb) = make_float4(db[i][0], db[i][1], db[i][2], db[i][3]);
        *reinterpret_cast<float4*>(pb + 4) = make_float4(db[i][4], db[i][5], db[i][6], db[i][7]);
      }
    }
  }
}

// norm_bwd_kernel with the next row group's loads issued before the current group's reduction: the
// CTA-wide barriers of the row sums no longer leave the memory system idle.  Same arithmetic.
template <bool RMS, int VPT>
__global__ void __launch_bounds__(256, 2)
norm_bwd_prefetch_kernel(const __nv_bfloat16* __restrict__ dz, const __nv_bfloat16* __restrict__ x,
                         const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                         const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres_in,
                         __nv_bfloat16* __restrict__ dx, float* __restrict__ part_dgamma,
                         float* __restrict__ part_dbeta, int rows, int h, int tpr, int rpc) {
  __shared__ float red[8 * 8 * 2];
  const int rl = threadIdx.x / tpr;
  const int tr = threadIdx.x % tpr;
  const int nvec = h >> 3;
  const int groups = (rows + rpc - 1) / rpc;

  float dg[VPT][8], db[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
#pragma unroll
    for (int k = 0; k < 8; ++k) dg[i][k] = db[i][k] = 0.f;
  }

  struct RowRegs {
    mb::bf16x8 xp[VPT], dzp[VPT], rp[VPT];
    float mean, rstd;
    int row;
    bool active;
  };
  auto load = [&](RowRegs& r, int grp) {
    r.row = grp * rpc + rl;
    r.active = grp < groups && r.row < rows;
    r.mean = (r.active && !RMS) ? mean_in[r.row] : 0.f;
    r.rstd = r.active ? rstd_in[r.row] : 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * tpr;
      if (r.active && vi < nvec) {
        const size_t off = static_cast<size_t>(r.row) * h + 8 * vi;
        r.xp[i] = *reinterpret_cast<const mb::bf16x8*>(x + off);
        r.dzp[i] = *reinterpret_cast<const mb::bf16x8*>(dz + off);
        if (dres_in) r.rp[i] = *reinterpret_cast<const mb::bf16x8*>(dres_in + off);
      }
    }
  };

  RowRegs cur;
  load(cur, blockIdx.x);
  for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    RowRegs nxt;
    load(nxt, grp + gridDim.x);        // in flight during the reduction below
    const float mean = cur.mean, rstd = cur.rstd;
    float acc[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * tpr;
      if (cur.active && vi < nvec) {
        float xv[8], dzv[8], g[8];
        mb::unpack8(cur.xp[i], xv);
        mb::unpack8(cur.dzp[i], dzv);
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(gamma + 8 * vi), g);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float xh = (xv[k] - mean) * rstd;
          float dy = dzv[k] * g[k];
          dg[i][k] += dzv[k] * xh;
          db[i][k] += dzv[k];
          acc[0] += dy;
          acc[1] += dy * xh;
        }
      }
    }
    row_reduce<2>(acc, red, tpr, rl, tr);
    const float m1 = RMS ? 0.f : acc[0] / h;
    const float m2 = acc[1] / h;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * tpr;
      if (cur.active && vi < nvec) {
        const size_t off = static_cast<size_t>(cur.row) * h + 8 * vi;
        float xv[8], dzv[8], g[8], o[8];
        mb::unpack8(cur.xp[i], xv);
        mb::unpack8(cur.dzp[i], dzv);
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(gamma + 8 * vi), g);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float xh = (xv[k] - mean) * rstd;
          o[k] = rstd * (dzv[k] * g[k] - m1 - xh * m2);
        }
        if (dres_in) {
          float r[8];
          mb::unpack8(cur.rp[i], r);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += r[k];
        }
        *reinterpret_cast<mb::bf16x8*>(dx + off) = mb::pack8(o);
      }
    }
    cur = nxt;
  }
  const size_t prow = static_cast<size_t>(blockIdx.x) * rpc + rl;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int vi = tr + i * tpr;
    if (vi < nvec) {
      float* pg = part_dgamma + prow * h + 8 * vi;
      *reinterpret_cast<float4*>(pg) = make_float4(dg[i][0], dg[i][1], dg[i][2], dg[i][3]);
      *reinterpret_cast<float4*>(pg + 4) = make_float4(dg[i][4], dg[i][5], dg[i][6], dg[i][7]);
      if (!RMS && part_dbeta) {
        float* pb = part_dbeta + prow * h + 8 * vi;
        *reinterpret_cast<float4*>(pb) = make_float4(db[i][0], db[i][1], db[i][2], db[i][3]);
        *reinterpret_cast<float4*>(pb + 4) = make_float4(db[i][4], db[i][5], db[i][6], db[i][7]);
      }
    }
  }
}

// Column sums of the partial matrices -> bf16 (or accumulate into fp32) gradients.
__global__ void norm_bwd_finalize_kernel(const float* __restrict__ part_dgamma,
                                         const float* __restrict__ part_dbeta,
                                         __nv_bfloat16* __restrict__ dgamma,
                                         __nv_bfloat16* __restrict__ dbeta, int nparts, int h,
                                         int accumulate) {
  // 32 x 32 threads: 32 columns per CTA, the partial rows dealt round-robin to the 32 row threads, four
  // independent running sums per thread so the loads of a column do not serialise on one add chain.
  __shared__ float sg[32][33], sb[32][33];
  const int col = blockIdx.x * 32 + threadIdx.x;
  float ag = 0.f, ab = 0.f;
  if (col < h) {
    float g0 = 0.f, g1 = 0.f, g2 = 0.f, g3 = 0.f, b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
    const int step = blockDim.y;
    int r = threadIdx.y;
    for (; r + 3 * step < nparts; r += 4 * step) {
      g0 += part_dgamma[static_cast<size_t>(r) * h + col];
      g1 += part_dgamma[static_cast<size_t>(r + step) * h + col];
      g2 += part_dgamma[static_cast<size_t>(r + 2 * step) * h + col];
      g3 += part_dgamma[static_cast<size_t>(r + 3 * step) * h + col];
      if (part_dbeta) {
        b0 += part_dbeta[static_cast<size_t>(r) * h + col];
        b1 += part_dbeta[static_cast<size_t>(r + step) * h + col];
        b2 += part_dbeta[static_cast<size_t>(r + 2 * step) * h + col];
        b3 += part_dbeta[static_cast<size_t>(r + 3 * step) * h + col];
      }
    }
    for (; r < nparts; r += step) {
      g0 += part_dgamma[static_cast<size_t>(r) * h + col];
      if (part_dbeta) b0 += part_dbeta[static_cast<size_t>(r) * h + col];
    }
    ag = (g0 + g1) + (g2 + g3);
    ab = (b0 + b1) + (b2 + b3);
  }
  sg[threadIdx.y][threadIdx.x] = ag;
  sb[threadIdx.y][threadIdx.x] = ab;
  __syncthreads();
  if (threadIdx.y == 0 && col < h) {
    for (int r = 1; r < static_cast<int>(blockDim.y); ++r) {
      ag += sg[r][threadIdx.x];
      ab += sb[r][threadIdx.x];
    }
    if (accumulate) {
      ag += __bfloat162float(dgamma[col]);
      if (dbeta) ab += __bfloat162float(dbeta[col]);
    }
    dgamma[col] = __float2bfloat16(ag);
    if (dbeta && part_dbeta) dbeta[col] = __float2bfloat16(ab);
  }
}

int g_sms = 0;
int num_sms() {
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sms;
}

// CTAs per SM of the persistent grids; MB_NORM_FWD_CTAS_PER_SM / MB_NORM_BWD_CTAS_PER_SM override the
// defaults for tuning runs (read once per process).
int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  if (!v || !*v) return dflt;
  int x = atoi(v);
  return x > 0 ? x : dflt;
}
int fwd_ctas_per_sm() {
  static int v = env_int("MB_NORM_FWD_CTAS_PER_SM", 8);
  return v;
}
int bwd_ctas_per_sm() {
  static int v = env_int("MB_NORM_BWD_CTAS_PER_SM", 4);
  return v;
}

// Two vectors per thread when a row then still fits 256 threads (more, lighter warps hide the
// memory latency better), else four.  MB_NORM_VPT forces a choice for tuning runs.
int pick_vpt(int h) {
  static int forced = env_int("MB_NORM_VPT", 0);
  int nvec = h / 8;
  if (forced == 2 && nvec <= 2 * 256) return 2;
  if (forced == 4) return 4;
  return (nvec <= 2 * 256) ? 2 : 4;
}

void pick_shape(int h, int& tpr, int& rpc) {
  const int VPT = pick_vpt(h);
  int nvec = h / 8;
  tpr = ((nvec + VPT - 1) / VPT + 31) / 32 * 32;
  if (tpr > 256) tpr = 256;
  rpc = 256 / tpr;
  if (rpc < 1) rpc = 1;
  if (rpc > 8) rpc = 8;
}

}  // namespace

// Number of scratch rows (each of `h` floats, once for dgamma and once for dbeta)
// that mb_norm_bwd needs for a given problem.
MB_API int mb_norm_bwd_scratch_rows(int rows, int h) {
  int tpr, rpc;
  pick_shape(h, tpr, rpc);
  int groups = (rows + rpc - 1) / rpc;
  int grid = num_sms() * bwd_ctas_per_sm();
  if (grid > groups) grid = groups;
  return grid * rpc;
}

// rms != 0 selects RMSNorm (no mean, no beta).  residual / x_out / beta / mean may be null.
MB_API int mb_norm_fwd(const void* x0, const void* residual, const void* gamma, const void* beta,
                       void* z, void* x_out, float* mean, float* rstd, int rows, int h, float eps,
                       int rms, cudaStream_t stream) {
  if (h % 8 != 0 || h > 8 * kMaxVPT * 256) return -1;
  if (rows == 0) return 0;
  int tpr, rpc;
  pick_shape(h, tpr, rpc);
  int groups = (rows + rpc - 1) / rpc;
  int grid = num_sms() * fwd_ctas_per_sm();
  if (grid > groups) grid = groups;
  auto a = reinterpret_cast<const __nv_bfloat16*>(x0);
  auto r = reinterpret_cast<const __nv_bfloat16*>(residual);
  auto g = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto b = reinterpret_cast<const __nv_bfloat16*>(beta);
  auto zz = reinterpret_cast<__nv_bfloat16*>(z);
  auto xo = reinterpret_cast<__nv_bfloat16*>(x_out);
  const bool v2 = pick_vpt(h) == 2;
#define MB_FWD(R_, V_) norm_fwd_kernel<R_, V_><<<grid, tpr * rpc, 0, stream>>>(a, r, g, b, zz, xo, mean, rstd, rows, h, eps, tpr, rpc)
  if (rms) { if (v2) MB_FWD(true, 2); else MB_FWD(true, 4); }
  else { if (v2) MB_FWD(false, 2); else MB_FWD(false, 4); }
#undef MB_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// scratch: 2 * mb_norm_bwd_scratch_rows(rows, h) * h floats (first half dgamma, second dbeta).
MB_API int mb_norm_bwd(const void* dz, const void* x, const void* gamma, const float* mean,
                       const float* rstd, const void* dres_in, void* dx, void* dgamma, void* dbeta,
                       float* scratch, int rows, int h, int rms, int accumulate,
                       cudaStream_t stream) {
  if (h % 8 != 0 || h > 8 * kMaxVPT * 256) return -1;
  if (rows == 0) return 0;
  int tpr, rpc;
  pick_shape(h, tpr, rpc);
  int groups = (rows + rpc - 1) / rpc;
  int grid = num_sms() * bwd_ctas_per_sm();
  if (grid > groups) grid = groups;
  int nparts = grid * rpc;
  float* pg = scratch;
  float* pb = rms ? nullptr : scratch + static_cast<size_t>(nparts) * h;
  auto dzz = reinterpret_cast<const __nv_bfloat16*>(dz);
  auto xx = reinterpret_cast<const __nv_bfloat16*>(x);
  auto g = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto dr = reinterpret_cast<const __nv_bfloat16*>(dres_in);
  auto dxx = reinterpret_cast<__nv_bfloat16*>(dx);
  const bool v2 = pick_vpt(h) == 2;
#define MB_BWD(K_, R_, V_) K_<R_, V_><<<grid, tpr * rpc, 0, stream>>>(dzz, xx, g, mean, rstd, dr, dxx, pg, pb, rows, h, tpr, rpc)
  if (v2) {
    // two vectors per thread: the kernel that loads the next row group before it reduces the current one
    // 121 registers: three CTAs of up to 256 threads stay resident per SM, so the persistent grid is
    // sized for three (the scratch matrix was sized for the larger default grid)
    const int g3 = num_sms() * 3;
    if (grid > g3) {
      grid = g3;
      nparts = grid * rpc;
      pb = rms ? nullptr : scratch + static_cast<size_t>(nparts) * h;
    }
    if (rms) MB_BWD(norm_bwd_prefetch_kernel, true, 2); else MB_BWD(norm_bwd_prefetch_kernel, false, 2);
  } else if (rms) {
    MB_BWD(norm_bwd_kernel, true, 4);
  } else {
    MB_BWD(norm_bwd_kernel, false, 4);
  }
#undef MB_BWD
  dim3 fb(32, 32);
  norm_bwd_finalize_kernel<<<(h + 31) / 32, fb, 0, stream>>>(
      pg, pb, reinterpret_cast<__nv_bfloat16*>(dgamma), reinterpret_cast<__nv_bfloat16*>(dbeta),
      nparts, h, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Column sums of partial-gradient matrices ([nparts][h] fp32 each, part_dbeta may be null) into the bf16
// gradient vectors; used after the pipelined backward kernel (norm_pipe.cu), which writes one partial row
// per CTA.
MB_API int mb_norm_bwd_finalize(const float* part_dgamma, const float* part_dbeta, void* dgamma, void* dbeta,
                                int nparts, int h, cudaStream_t stream) {
  if (nparts <= 0 || h <= 0) return -1;
  dim3 fb(32, 32);
  norm_bwd_finalize_kernel<<<(h + 31) / 32, fb, 0, stream>>>(part_dgamma, part_dbeta,
                                                             reinterpret_cast<__nv_bfloat16*>(dgamma),
                                                             reinterpret_cast<__nv_bfloat16*>(dbeta), nparts, h, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
