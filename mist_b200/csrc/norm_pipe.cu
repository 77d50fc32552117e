// LayerNorm / RMSNorm forward and backward as software pipelines over rows: a producer thread streams
// whole rows from global memory into rings of shared-memory slots with bulk async copies (cp.async.bulk,
// completion on mbarriers); teams of four consumer warps own one row each, normalise it out of shared
// memory and write the results with coalesced 16-byte stores.  The loads of the next rows are always in
// flight while a row is reduced, and no CTA-wide barrier sits in the loop (a team meets on a named barrier
// of its own for the two row sums).
//
// Folded into the same pass, as in the reference's dropout_add_ln extension
// (csrc/layer_norm/ln_api.cpp:832-846 dropout_add_ln_fwd / bwd and the parallel-residual pair,
// called from mist/modules/layer_norm.py:738, 808):
//   x  = dropout(x0) [+ dropout(x1)] [+ residual]          residual stream in bf16 or fp32
//   z  = norm(x; gamma, beta)     [z1 = norm(x; gamma1, beta1)]   (parallel blocks: two norms of one stream)
// and in the backward pass
//   dx = norm'(dz) [+ norm1'(dz1)] [+ dres_in];   dx0 = mask0 * dx / (1 - p)   [dx1 = mask1 * dx / (1 - p)]
// with the dropout masks regenerated from (seed, element index) instead of being stored.
//
// dgamma / dbeta: every team adds its rows' contributions into its own fp32 vectors in shared memory (each
// thread owns fixed columns, no atomics: a fixed summation order, the same result on every run); the CTA
// then writes one partial row, and norm_bwd_finalize (norm.cu) sums the partial rows.
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int kMaxWarps = 4;          // teams of consumer warps per CTA (one more warp produces)
constexpr int kTeamWarps = 4;         // warps per team, i.e. per row
constexpr int kTeam = kTeamWarps * 32;
constexpr int kThreadsPipe = (kMaxWarps * kTeamWarps + 1) * 32;
constexpr int kMaxSlots = 4;          // ring depth per team
constexpr int kHeaderBytes = 2 * kMaxWarps * kMaxSlots * 8 + kMaxWarps * 2 * 8 * 4;   // barriers + team sums
constexpr int kSmemBudget = 225 * 1024;      // of the 227 KB a CTA may have

__device__ __forceinline__ uint4 philox4(uint64_t seed, uint64_t ctr) {
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

// keep[k] * 1/(1-p) for the 8 elements of vector `vec` (global vector index) of the tensor tagged `seed`
__device__ __forceinline__ void dropout_scale8(uint64_t seed, uint64_t vec, float p, float inv_keep, float* s) {
  const uint4 a = philox4(seed, 2 * vec), b = philox4(seed, 2 * vec + 1);
  const uint32_t r[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  const uint32_t thr = static_cast<uint32_t>(fminf(p, 1.f) * 4294967295.f);
#pragma unroll
  for (int k = 0; k < 8; ++k) s[k] = r[k] >= thr ? inv_keep : 0.f;
}

// Sums (a, b) over the four warps of a team.  `red`: 8 floats of this team for this row parity.
__device__ __forceinline__ void team_sum2(float& a, float& b, float* red, int wit, int lane, int bar_id) {
  a = mb::warp_sum(a);
  b = mb::warp_sum(b);
  if (lane == 0) {
    red[2 * wit] = a;
    red[2 * wit + 1] = b;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(kTeam) : "memory");
  a = (red[0] + red[2]) + (red[4] + red[6]);
  b = (red[1] + red[3]) + (red[5] + red[7]);
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

struct FwdArgs {
  const __nv_bfloat16* x0;
  const __nv_bfloat16* x1;        // second branch of a parallel block, or null
  const void* residual;           // bf16 or fp32 (res_fp32), or null
  const __nv_bfloat16* gamma;
  const __nv_bfloat16* beta;      // null for RMSNorm or no bias
  const __nv_bfloat16* gamma1;    // second norm of a parallel block, or null
  const __nv_bfloat16* beta1;
  __nv_bfloat16* z;
  __nv_bfloat16* z1;
  void* x_out;                    // the new residual stream (same dtype as residual), or null
  float* mean;                    // null for RMSNorm
  float* rstd;
  int rows, h;
  float eps, drop_p;
  unsigned long long seed;
  int res_fp32;
  int nwarps, nslots;             // consumer warps, ring depth (chosen by the host from the shared-memory budget)
  int row_bytes;                  // bytes of one slot
  int* status;
};

// Slot layout: [x0 row: 2h bytes][x1 row: 2h bytes, if any][residual row: 2h or 4h bytes, if any]
template <bool RMS>
__global__ void __launch_bounds__(kThreadsPipe, 1)
norm_fwd_pipe_kernel(const FwdArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int NW = a.nwarps, NS = a.nslots;                              // NW: teams
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);                  // [NW][NS]
  uint64_t* empty = full + kMaxWarps * kMaxSlots;                      // [NW][NS]
  float* red_all = reinterpret_cast<float*>(smem + 2 * kMaxWarps * kMaxSlots * 8);   // [teams][2 parities][8]
  uint8_t* slots = smem + 2 * kMaxWarps * kMaxSlots * 8 + kMaxWarps * 2 * 8 * 4;     // header: 512 bytes
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 7;                                   // team index; kMaxWarps.. = producer warp
  const int wit = (threadIdx.x >> 5) & 3;                              // warp within the team
  const int tid = threadIdx.x & (kTeam - 1);
  const int h = a.h, nvec = h >> 3;
  const size_t x_bytes = static_cast<size_t>(h) * 2;
  const size_t res_bytes = a.residual ? static_cast<size_t>(h) * (a.res_fp32 ? 4 : 2) : 0;
  const int off_x1 = static_cast<int>(x_bytes);
  const int off_res = static_cast<int>(x_bytes * (a.x1 ? 2 : 1));

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxWarps * kMaxSlots; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kTeamWarps);
    }
    fence_barrier_init();
  }
  __syncthreads();

  // rows of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; its k-th row goes to team k % NW
  const int my_rows = (a.rows > static_cast<int>(blockIdx.x)) ? (a.rows - 1 - blockIdx.x) / gridDim.x + 1 : 0;

  if (threadIdx.x >= kMaxWarps * kTeam) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      for (int k = 0; k < my_rows; ++k) {
        const int w = k % NW, j = k / NW, s = j % NS;
        if (j >= NS && !mbar_wait(&empty[w * kMaxSlots + s], ((j / NS) - 1) & 1)) {
          if (a.status) atomicCAS(a.status, 0, MB_ERR_TIMEOUT_EMPTY);
          break;
        }
        const size_t row = static_cast<size_t>(blockIdx.x) + static_cast<size_t>(k) * gridDim.x;
        uint8_t* dst = slots + (static_cast<size_t>(w) * NS + s) * a.row_bytes;
        uint64_t* bar = &full[w * kMaxSlots + s];
        mbar_expect_tx(bar, static_cast<uint32_t>(x_bytes * (a.x1 ? 2 : 1) + res_bytes));
        bulk_g2s(dst, a.x0 + row * h, static_cast<uint32_t>(x_bytes), bar);
        if (a.x1) bulk_g2s(dst + off_x1, a.x1 + row * h, static_cast<uint32_t>(x_bytes), bar);
        if (a.residual)
          bulk_g2s(dst + off_res, reinterpret_cast<const uint8_t*>(a.residual) + row * res_bytes,
                   static_cast<uint32_t>(res_bytes), bar);
      }
    }
  } else if (warp < NW) {
    // ------------------------------------------------------------------ consumers
    const bool drop = a.drop_p > 0.f;
    const float inv_keep = drop ? 1.f / (1.f - a.drop_p) : 1.f;
    for (int k = warp, j = 0; k < my_rows; k += NW, ++j) {   // all four warps of the team walk the same rows
      const int s = j % NS;
      if (!mbar_wait(&full[warp * kMaxSlots + s], (j / NS) & 1)) {
        if (lane == 0 && a.status) atomicCAS(a.status, 0, MB_ERR_TIMEOUT_FULL);
        break;
      }
      const size_t row = static_cast<size_t>(blockIdx.x) + static_cast<size_t>(k) * gridDim.x;
      uint8_t* slot = slots + (static_cast<size_t>(warp) * NS + s) * a.row_bytes;
      // pass 1: x = dropout(x0) + dropout(x1) + residual, kept in the slot (bf16 over x0, or fp32 over the
      // fp32 residual); row sums of x and x^2 taken from the values as they are stored
      float s1 = 0.f, s2 = 0.f;
      for (int vi = tid; vi < nvec; vi += kTeam) {
        float x[8];
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(slot + 16 * vi), x);
        if (drop) {
          float m[8];
          dropout_scale8(a.seed, row * nvec + vi, a.drop_p, inv_keep, m);
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] *= m[e];
        }
        if (a.x1) {
          float y[8];
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(slot + off_x1 + 16 * vi), y);
          if (drop) {
            float m[8];
            dropout_scale8(a.seed + 0x9E3779B97F4A7C15ull, row * nvec + vi, a.drop_p, inv_keep, m);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] *= m[e];
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] += y[e];
        }
        if (a.residual) {
          if (a.res_fp32) {
            float4* rp = reinterpret_cast<float4*>(slot + off_res + 32 * vi);
            float4 r0 = rp[0], r1 = rp[1];
            x[0] += r0.x; x[1] += r0.y; x[2] += r0.z; x[3] += r0.w;
            x[4] += r1.x; x[5] += r1.y; x[6] += r1.z; x[7] += r1.w;
            rp[0] = make_float4(x[0], x[1], x[2], x[3]);
            rp[1] = make_float4(x[4], x[5], x[6], x[7]);
          } else {
            float r[8];
            mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(slot + off_res + 16 * vi), r);
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] += r[e];
          }
        }
        if (!(a.residual && a.res_fp32)) {
          const mb::bf16x8 packed = mb::pack8(x);          // what the stream stores is what gets normalised
          *reinterpret_cast<mb::bf16x8*>(slot + 16 * vi) = packed;
          mb::unpack8(packed, x);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          s1 += x[e];
          s2 += x[e] * x[e];
        }
      }
      team_sum2(s1, s2, red_all + (warp * 2 + (j & 1)) * 8, wit, lane, 1 + warp);
      const float mean = RMS ? 0.f : s1 / h;
      const float var = s2 / h - mean * mean;
      const float rstd = rsqrtf(fmaxf(var, 0.f) + a.eps);
      if (tid == 0) {
        if (a.mean) a.mean[row] = mean;
        a.rstd[row] = rstd;
      }
      // pass 2: normalise out of the slot
      const bool f32x = a.residual && a.res_fp32;
      for (int vi = tid; vi < nvec; vi += kTeam) {
        float x[8], g[8], o[8];
        if (f32x) {
          const float4* rp = reinterpret_cast<const float4*>(slot + off_res + 32 * vi);
          float4 r0 = rp[0], r1 = rp[1];
          x[0] = r0.x; x[1] = r0.y; x[2] = r0.z; x[3] = r0.w; x[4] = r1.x; x[5] = r1.y; x[6] = r1.z; x[7] = r1.w;
          if (a.x_out) {
            float4* xo = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.x_out) + row * h + 8 * vi);
            xo[0] = r0;
            xo[1] = r1;
          }
        } else {
          const mb::bf16x8 packed = *reinterpret_cast<const mb::bf16x8*>(slot + 16 * vi);
          mb::unpack8(packed, x);
          if (a.x_out) *reinterpret_cast<mb::bf16x8*>(reinterpret_cast<__nv_bfloat16*>(a.x_out) + row * h + 8 * vi) = packed;
        }
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(a.gamma + 8 * vi), g);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (x[e] - mean) * rstd * g[e];
        if (!RMS && a.beta) {
          float bb[8];
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(a.beta + 8 * vi), bb);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += bb[e];
        }
        *reinterpret_cast<mb::bf16x8*>(a.z + row * h + 8 * vi) = mb::pack8(o);
        if (a.z1) {
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(a.gamma1 + 8 * vi), g);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = (x[e] - mean) * rstd * g[e];
          if (!RMS && a.beta1) {
            float bb[8];
            mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(a.beta1 + 8 * vi), bb);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] += bb[e];
          }
          *reinterpret_cast<mb::bf16x8*>(a.z1 + row * h + 8 * vi) = mb::pack8(o);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[warp * kMaxSlots + s]);
    }
  }
}

struct BwdArgs {
  const __nv_bfloat16* dz;
  const __nv_bfloat16* dz1;       // gradient of the second norm of a parallel block, or null
  const void* x;                  // the normalised stream saved by the forward pass (bf16 or fp32)
  const void* dres_in;            // gradient arriving on the residual stream (same dtype as x), or null
  const __nv_bfloat16* gamma;
  const __nv_bfloat16* gamma1;
  const float* mean;              // null for RMSNorm
  const float* rstd;
  void* dx;                       // gradient of the stream (dtype of x): goes to the residual input
  __nv_bfloat16* dx0;             // gradient of x0 when it differs from dx (dropout, or fp32 stream), or null
  __nv_bfloat16* dx1;             // gradient of x1 likewise, or null
  float* part_dgamma;             // [gridDim.x][h] partial sums (and the three below)
  float* part_dbeta;
  float* part_dgamma1;
  float* part_dbeta1;
  int rows, h;
  float drop_p;
  unsigned long long seed;
  int x_fp32;
  int nwarps, nslots, row_bytes;
  int* status;
};

// Slot layout: [dz row: 2h][dz1 row: 2h, if any][x row: 2h or 4h][dres_in row: 2h or 4h, if any]
// After the slots: per consumer warp, fp32 vectors of h floats: dgamma, dbeta [, dgamma1, dbeta1].
template <bool RMS>
__global__ void __launch_bounds__(kThreadsPipe, 1)
norm_bwd_pipe_kernel(const BwdArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int NW = a.nwarps, NS = a.nslots;                              // NW: teams
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kMaxWarps * kMaxSlots;
  float* red_all = reinterpret_cast<float*>(smem + 2 * kMaxWarps * kMaxSlots * 8);
  uint8_t* slots = smem + 2 * kMaxWarps * kMaxSlots * 8 + kMaxWarps * 2 * 8 * 4;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 7;                                   // team index
  const int wit = (threadIdx.x >> 5) & 3;
  const int tid = threadIdx.x & (kTeam - 1);
  const int h = a.h, nvec = h >> 3;
  const size_t dz_bytes = static_cast<size_t>(h) * 2;
  const size_t x_bytes = static_cast<size_t>(h) * (a.x_fp32 ? 4 : 2);
  const int off_dz1 = static_cast<int>(dz_bytes);
  const int off_x = static_cast<int>(dz_bytes * (a.dz1 ? 2 : 1));
  const int off_dres = off_x + static_cast<int>(x_bytes);
  const int nacc = (RMS ? 1 : 2) * (a.dz1 ? 2 : 1);           // accumulator vectors per warp
  float* acc_base = reinterpret_cast<float*>(slots + static_cast<size_t>(NW) * NS * a.row_bytes);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxWarps * kMaxSlots; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kTeamWarps);
    }
    fence_barrier_init();
  }
  if (warp < NW) {
    float* acc = acc_base + static_cast<size_t>(warp) * nacc * h;
    for (int i = tid; i < nacc * h; i += kTeam) acc[i] = 0.f;
  }
  __syncthreads();

  const int my_rows = (a.rows > static_cast<int>(blockIdx.x)) ? (a.rows - 1 - blockIdx.x) / gridDim.x + 1 : 0;

  if (threadIdx.x >= kMaxWarps * kTeam) {
    if (lane == 0) {
      for (int k = 0; k < my_rows; ++k) {
        const int w = k % NW, j = k / NW, s = j % NS;
        if (j >= NS && !mbar_wait(&empty[w * kMaxSlots + s], ((j / NS) - 1) & 1)) {
          if (a.status) atomicCAS(a.status, 0, MB_ERR_TIMEOUT_EMPTY);
          break;
        }
        const size_t row = static_cast<size_t>(blockIdx.x) + static_cast<size_t>(k) * gridDim.x;
        uint8_t* dst = slots + (static_cast<size_t>(w) * NS + s) * a.row_bytes;
        uint64_t* bar = &full[w * kMaxSlots + s];
        mbar_expect_tx(bar, static_cast<uint32_t>(dz_bytes * (a.dz1 ? 2 : 1) + x_bytes * (a.dres_in ? 2 : 1)));
        bulk_g2s(dst, a.dz + row * h, static_cast<uint32_t>(dz_bytes), bar);
        if (a.dz1) bulk_g2s(dst + off_dz1, a.dz1 + row * h, static_cast<uint32_t>(dz_bytes), bar);
        bulk_g2s(dst + off_x, reinterpret_cast<const uint8_t*>(a.x) + row * x_bytes, static_cast<uint32_t>(x_bytes), bar);
        if (a.dres_in)
          bulk_g2s(dst + off_dres, reinterpret_cast<const uint8_t*>(a.dres_in) + row * x_bytes,
                   static_cast<uint32_t>(x_bytes), bar);
      }
    }
  } else if (warp < NW) {
    float* acc = acc_base + static_cast<size_t>(warp) * nacc * h;
    float* dg_s = acc;
    float* db_s = RMS ? nullptr : acc + h;
    float* dg1_s = a.dz1 ? acc + (RMS ? 1 : 2) * h : nullptr;
    float* db1_s = (a.dz1 && !RMS) ? acc + 3 * h : nullptr;
    const bool drop = a.drop_p > 0.f;
    const float inv_keep = drop ? 1.f / (1.f - a.drop_p) : 1.f;
    for (int k = warp, j = 0; k < my_rows; k += NW, ++j) {   // all four warps of the team walk the same rows
      const int s = j % NS;
      if (!mbar_wait(&full[warp * kMaxSlots + s], (j / NS) & 1)) {
        if (lane == 0 && a.status) atomicCAS(a.status, 0, MB_ERR_TIMEOUT_FULL);
        break;
      }
      const size_t row = static_cast<size_t>(blockIdx.x) + static_cast<size_t>(k) * gridDim.x;
      uint8_t* slot = slots + (static_cast<size_t>(warp) * NS + s) * a.row_bytes;
      const float mean = (RMS || !a.mean) ? 0.f : a.mean[row];
      const float rstd = a.rstd[row];
      auto load_x = [&](int vi, float* x) {
        if (a.x_fp32) {
          const float4* p = reinterpret_cast<const float4*>(slot + off_x + 32 * vi);
          float4 r0 = p[0], r1 = p[1];
          x[0] = r0.x; x[1] = r0.y; x[2] = r0.z; x[3] = r0.w; x[4] = r1.x; x[5] = r1.y; x[6] = r1.z; x[7] = r1.w;
        } else {
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(slot + off_x + 16 * vi), x);
        }
      };
      // pass 1: row sums of dy and dy * xhat; the warp's dgamma / dbeta vectors take this row's share
      float s1 = 0.f, s2 = 0.f;
      for (int vi = tid; vi < nvec; vi += kTeam) {
        float x[8], dz[8], g[8];
        load_x(vi, x);
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(slot + 16 * vi), dz);
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(a.gamma + 8 * vi), g);
        float4* dgp = reinterpret_cast<float4*>(dg_s + 8 * vi);
        float4 d0 = dgp[0], d1 = dgp[1];
        float xh[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) xh[e] = (x[e] - mean) * rstd;
        d0.x += dz[0] * xh[0]; d0.y += dz[1] * xh[1]; d0.z += dz[2] * xh[2]; d0.w += dz[3] * xh[3];
        d1.x += dz[4] * xh[4]; d1.y += dz[5] * xh[5]; d1.z += dz[6] * xh[6]; d1.w += dz[7] * xh[7];
        dgp[0] = d0;
        dgp[1] = d1;
        if (db_s) {
          float4* dbp = reinterpret_cast<float4*>(db_s + 8 * vi);
          float4 b0 = dbp[0], b1 = dbp[1];
          b0.x += dz[0]; b0.y += dz[1]; b0.z += dz[2]; b0.w += dz[3];
          b1.x += dz[4]; b1.y += dz[5]; b1.z += dz[6]; b1.w += dz[7];
          dbp[0] = b0;
          dbp[1] = b1;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float dy = dz[e] * g[e];
          s1 += dy;
          s2 += dy * xh[e];
        }
        if (a.dz1) {
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(slot + off_dz1 + 16 * vi), dz);
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(a.gamma1 + 8 * vi), g);
          float4* dg1p = reinterpret_cast<float4*>(dg1_s + 8 * vi);
          float4 e0 = dg1p[0], e1 = dg1p[1];
          e0.x += dz[0] * xh[0]; e0.y += dz[1] * xh[1]; e0.z += dz[2] * xh[2]; e0.w += dz[3] * xh[3];
          e1.x += dz[4] * xh[4]; e1.y += dz[5] * xh[5]; e1.z += dz[6] * xh[6]; e1.w += dz[7] * xh[7];
          dg1p[0] = e0;
          dg1p[1] = e1;
          if (db1_s) {
            float4* dbp = reinterpret_cast<float4*>(db1_s + 8 * vi);
            float4 b0 = dbp[0], b1 = dbp[1];
            b0.x += dz[0]; b0.y += dz[1]; b0.z += dz[2]; b0.w += dz[3];
            b1.x += dz[4]; b1.y += dz[5]; b1.z += dz[6]; b1.w += dz[7];
            dbp[0] = b0;
            dbp[1] = b1;
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float dy = dz[e] * g[e];
            s1 += dy;
            s2 += dy * xh[e];
          }
        }
      }
      team_sum2(s1, s2, red_all + (warp * 2 + (j & 1)) * 8, wit, lane, 1 + warp);
      const float m1 = RMS ? 0.f : s1 / h;
      const float m2 = s2 / h;
      // pass 2: dx
      for (int vi = tid; vi < nvec; vi += kTeam) {
        float x[8], dz[8], g[8], o[8];
        load_x(vi, x);
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(slot + 16 * vi), dz);
        mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(a.gamma + 8 * vi), g);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = dz[e] * g[e];
        if (a.dz1) {
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(slot + off_dz1 + 16 * vi), dz);
          mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(a.gamma1 + 8 * vi), g);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += dz[e] * g[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rstd * (o[e] - m1 - (x[e] - mean) * rstd * m2);
        if (a.dres_in) {
          if (a.x_fp32) {
            const float4* p = reinterpret_cast<const float4*>(slot + off_dres + 32 * vi);
            float4 r0 = p[0], r1 = p[1];
            o[0] += r0.x; o[1] += r0.y; o[2] += r0.z; o[3] += r0.w; o[4] += r1.x; o[5] += r1.y; o[6] += r1.z; o[7] += r1.w;
          } else {
            float r[8];
            mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(slot + off_dres + 16 * vi), r);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] += r[e];
          }
        }
        if (a.dx) {
          if (a.x_fp32) {
            float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.dx) + row * h + 8 * vi);
            d[0] = make_float4(o[0], o[1], o[2], o[3]);
            d[1] = make_float4(o[4], o[5], o[6], o[7]);
          } else {
            *reinterpret_cast<mb::bf16x8*>(reinterpret_cast<__nv_bfloat16*>(a.dx) + row * h + 8 * vi) = mb::pack8(o);
          }
        }
        if (a.dx0) {
          float t[8];
          if (drop) {
            float m[8];
            dropout_scale8(a.seed, row * nvec + vi, a.drop_p, inv_keep, m);
#pragma unroll
            for (int e = 0; e < 8; ++e) t[e] = o[e] * m[e];
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) t[e] = o[e];
          }
          *reinterpret_cast<mb::bf16x8*>(a.dx0 + row * h + 8 * vi) = mb::pack8(t);
        }
        if (a.dx1) {
          float t[8];
          if (drop) {
            float m[8];
            dropout_scale8(a.seed + 0x9E3779B97F4A7C15ull, row * nvec + vi, a.drop_p, inv_keep, m);
#pragma unroll
            for (int e = 0; e < 8; ++e) t[e] = o[e] * m[e];
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) t[e] = o[e];
          }
          *reinterpret_cast<mb::bf16x8*>(a.dx1 + row * h + 8 * vi) = mb::pack8(t);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[warp * kMaxSlots + s]);
    }
  }
  // one partial row per CTA: the consumer warps' vectors summed in warp order
  __syncthreads();
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    float g = 0.f, b = 0.f, g1 = 0.f, b1 = 0.f;
    for (int w = 0; w < NW; ++w) {
      const float* acc = acc_base + static_cast<size_t>(w) * nacc * h;
      g += acc[i];
      if (!RMS) b += acc[h + i];
      if (a.dz1) {
        g1 += acc[(RMS ? 1 : 2) * h + i];
        if (!RMS) b1 += acc[3 * h + i];
      }
    }
    const size_t o = static_cast<size_t>(blockIdx.x) * h + i;
    a.part_dgamma[o] = g;
    if (!RMS && a.part_dbeta) a.part_dbeta[o] = b;
    if (a.dz1) {
      a.part_dgamma1[o] = g1;
      if (!RMS && a.part_dbeta1) a.part_dbeta1[o] = b1;
    }
  }
}

int g_sms = 0;
int sms() {
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sms;
}

// Teams and ring depth for a slot of `row_bytes` plus `acc_bytes` of accumulators per team.
bool plan(int row_bytes, int acc_bytes, int& nwarps, int& nslots) {
  for (nwarps = kMaxWarps; nwarps >= 1; nwarps >>= 1) {
    for (nslots = kMaxSlots; nslots >= 2; --nslots) {
      if (kHeaderBytes + static_cast<long>(nwarps) * (static_cast<long>(nslots) * row_bytes + acc_bytes) <= kSmemBudget)
        return true;
    }
  }
  return false;
}

}  // namespace

MB_API int* mb_status_device_ptr();

// Rows of the partial-gradient matrices that mb_norm_bwd_pipe writes (one per CTA); 0 when the shape does not
// fit the pipelined kernels (callers then use mb_norm_bwd).
MB_API int mb_norm_pipe_parts(int rows, int h, int x_fp32, int parallel, int has_dres, int rms) {
  if (h % 8 || h < 8) return 0;
  const int row_bytes = h * 2 * (parallel ? 2 : 1) + h * (x_fp32 ? 4 : 2) * (has_dres ? 2 : 1);
  const int acc_bytes = h * 4 * (rms ? 1 : 2) * (parallel ? 2 : 1);
  int nw, ns;
  if (!plan(row_bytes, acc_bytes, nw, ns)) return 0;
  int grid = sms();
  if (grid > rows) grid = rows;
  return grid;
}

// z = norm(dropout(x0) [+ dropout(x1)] [+ residual]) (* gamma + beta) [, z1 with gamma1 / beta1]; x_out receives
// the sum (the new residual stream) when not null.  residual / x_out are bf16, or fp32 when res_fp32.  Returns 1
// (nothing launched) when the shape does not fit; all row pointers 16-byte aligned, h % 8 == 0.
MB_API int mb_norm_fwd_pipe(const void* x0, const void* x1, const void* residual, const void* gamma, const void* beta,
                            const void* gamma1, const void* beta1, void* z, void* z1, void* x_out, float* mean,
                            float* rstd, int rows, int h, float eps, int rms, int res_fp32, float drop_p,
                            unsigned long long seed, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (h % 8 || h < 8) return 1;
  FwdArgs a;
  a.x0 = reinterpret_cast<const __nv_bfloat16*>(x0);
  a.x1 = reinterpret_cast<const __nv_bfloat16*>(x1);
  a.residual = residual;
  a.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
  a.beta = reinterpret_cast<const __nv_bfloat16*>(beta);
  a.gamma1 = reinterpret_cast<const __nv_bfloat16*>(gamma1);
  a.beta1 = reinterpret_cast<const __nv_bfloat16*>(beta1);
  a.z = reinterpret_cast<__nv_bfloat16*>(z);
  a.z1 = reinterpret_cast<__nv_bfloat16*>(z1);
  a.x_out = x_out;
  a.mean = mean; a.rstd = rstd; a.rows = rows; a.h = h; a.eps = eps; a.drop_p = drop_p; a.seed = seed;
  a.res_fp32 = res_fp32;
  a.row_bytes = h * 2 * (x1 ? 2 : 1) + (residual ? h * (res_fp32 ? 4 : 2) : 0);
  if (!plan(a.row_bytes, 0, a.nwarps, a.nslots)) return 1;
  a.status = mb_status_device_ptr();
  const int smem = kHeaderBytes + a.nwarps * a.nslots * a.row_bytes;
  int grid = sms();
  if (grid > rows) grid = rows;
  auto kern = rms ? norm_fwd_pipe_kernel<true> : norm_fwd_pipe_kernel<false>;
  static bool cfg[2] = {false, false};
  if (!cfg[rms ? 1 : 0]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 1024) != cudaSuccess) return -3;
    cfg[rms ? 1 : 0] = true;
  }
  kern<<<grid, kThreadsPipe, smem, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Backward of mb_norm_fwd_pipe.  x: the stream the forward pass normalised (its x_out; bf16 or fp32); dres_in: the
// gradient arriving on the stream (same dtype) or null; dx: gradient of the stream (same dtype), may be null when
// only dx0 is wanted; dx0 / dx1: bf16 gradients of the branch inputs when they differ from dx (dropout or an fp32
// stream), else null.  part_*: [mb_norm_pipe_parts(...)][h] fp32, to be summed by mb_norm_bwd_finalize.
MB_API int mb_norm_bwd_pipe(const void* dz, const void* dz1, const void* x, const void* dres_in, const void* gamma,
                            const void* gamma1, const float* mean, const float* rstd, void* dx, void* dx0, void* dx1,
                            float* part_dgamma, float* part_dbeta, float* part_dgamma1, float* part_dbeta1, int rows,
                            int h, int rms, int x_fp32, float drop_p, unsigned long long seed, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (h % 8 || h < 8) return 1;
  BwdArgs a;
  a.dz = reinterpret_cast<const __nv_bfloat16*>(dz);
  a.dz1 = reinterpret_cast<const __nv_bfloat16*>(dz1);
  a.x = x; a.dres_in = dres_in;
  a.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
  a.gamma1 = reinterpret_cast<const __nv_bfloat16*>(gamma1);
  a.mean = mean; a.rstd = rstd; a.dx = dx;
  a.dx0 = reinterpret_cast<__nv_bfloat16*>(dx0);
  a.dx1 = reinterpret_cast<__nv_bfloat16*>(dx1);
  a.part_dgamma = part_dgamma; a.part_dbeta = part_dbeta; a.part_dgamma1 = part_dgamma1; a.part_dbeta1 = part_dbeta1;
  a.rows = rows; a.h = h; a.drop_p = drop_p; a.seed = seed; a.x_fp32 = x_fp32;
  a.row_bytes = h * 2 * (dz1 ? 2 : 1) + h * (x_fp32 ? 4 : 2) * (dres_in ? 2 : 1);
  const int acc_bytes = h * 4 * (rms ? 1 : 2) * (dz1 ? 2 : 1);
  if (!plan(a.row_bytes, acc_bytes, a.nwarps, a.nslots)) return 1;
  a.status = mb_status_device_ptr();
  const int smem = kHeaderBytes + a.nwarps * (a.nslots * a.row_bytes + acc_bytes);
  int grid = sms();
  if (grid > rows) grid = rows;
  auto kern = rms ? norm_bwd_pipe_kernel<true> : norm_bwd_pipe_kernel<false>;
  static bool cfg[2] = {false, false};
  if (!cfg[rms ? 1 : 0]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 1024) != cudaSuccess) return -3;
    cfg[rms ? 1 : 0] = true;
  }
  kern<<<grid, kThreadsPipe, smem, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
