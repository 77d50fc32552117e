// Attention backward on tcgen05 tensor cores.
//
// One CTA owns a 128-row key/value block of one (batch, head) and loops over the
// 64-row query blocks that can see it.  Everything is computed transposed, rows = keys,
// so that the probabilities land in shared memory directly in the layout the following
// MMAs need:
//
//   S^T  = K Q^T            [128 kv x 64 q]   A = K (K-major)        B = Q  (K-major)
//   dP^T = V dO^T           [128 kv x 64 q]   A = V (K-major)        B = dO (K-major)
//   P^T  = exp2(S^T*c - LSE[q]);  dS^T = scale * P^T o (dP^T - delta[q])   (registers -> smem)
//   dV  += P^T  dO          [128 kv x d]      A = P^T  (K-major)     B = dO (MN-major)
//   dK  += dS^T Q           [128 kv x d]      A = dS^T (K-major)     B = Q  (MN-major)
//   dQ^T = K^T dS           [d x 64 q]        A = K (MN-major)       B = dS^T (MN-major)
//
// dV and dK stay in tensor memory for the whole loop; dQ^T is read back every iteration,
// transposed through shared memory and added to an fp32 accumulator in global memory
// with a TMA reduce (several key blocks contribute to the same query rows).
// Helper kernels compute delta = rowsum(dO o O) and convert the fp32 dQ to bf16.
//
// Replaces the reference's flash-attention v2 backward (reference:
// csrc/flash_attn/src/flash_bwd_kernel.h, flash_bwd_launch_template.h:12-43; the kernel
// families dot_do_o / dq_dk_dv_loop / convert_dq map onto the three kernels here).
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BKV = 128;
constexpr int BQ = 64;
constexpr int kThreads = 320;   // 8 softmax warps + TMA warp + MMA warp
constexpr int kWG = 256;        // softmax / write-out threads

struct BwdParams {
  const float* lse;     // [b][nh][sq]
  const float* delta;   // [b][nh][sq]
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long dk_bs, dk_ts, dk_hs, dv_bs, dv_ts, dv_hs;
  int sq, sk, nh, d, nchunks;
  float scale, scale_log2;
  int causal;
  const int* seqlens_q;   // per-sample token counts of a right-padded batch, or null
  const int* seqlens_k;
  int* status;
};

struct Smem {
  static constexpr int kKV = 2 * BKV * 128;     // K or V: up to 2 chunks of [128][64 bf16]
  static constexpr int kQ = 2 * BQ * 128;       // Q or dO stage: up to 2 chunks of [64][64 bf16]
  static constexpr int kP = BKV * 128;          // P^T / dS^T: [128 kv][64 q]
  static constexpr int kDQ = 4 * BQ * 128;      // dQ staging: 4 chunks of [64 q][32 fp32]
  static constexpr int oK = 0;
  static constexpr int oV = oK + kKV;
  static constexpr int oQ = oV + kKV;           // 2 stages of (Q, dO)
  static constexpr int oP = oQ + 2 * 2 * kQ;
  static constexpr int oDS = oP + kP;
  static constexpr int oDQ = oDS + kP;
  static constexpr int oBar = oDQ + kDQ;
  // kv_full, q_full[2], q_empty[2], sdp_full, pds_full, dq_full, final_full
  static constexpr int kNumBars = 9;
  static constexpr int oVec = oBar + kNumBars * 8 + 16;   // lse / delta of the query block, 2 buffers each
  static constexpr int kTotal = oVec + 2 * 2 * BQ * 4;
};

__device__ __forceinline__ void report(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_dq, const BwdParams p) {
  using L = Smem;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::oBar);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;
  uint64_t* q_empty = bars + 3;
  uint64_t* sdp_full = bars + 5;
  uint64_t* pds_full = bars + 6;
  uint64_t* dq_full = bars + 7;
  uint64_t* final_full = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int jb = blockIdx.x;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  // real tokens of this sample (right-padded batches); the tensors keep their padded extents p.sq / p.sk
  const int sq_b = p.seqlens_q ? min(p.sq, p.seqlens_q[batch]) : p.sq;
  const int sk_b = p.seqlens_k ? min(p.sk, p.seqlens_k[batch]) : p.sk;
  const int kv0 = jb * BKV;
  const int coff = sk_b - sq_b;
  const int nq_blocks = (sq_b + BQ - 1) / BQ;
  int i_start = 0;
  if (p.causal) {
    int first_q = kv0 - coff;  // first query row that can see key kv0
    i_start = first_q <= 0 ? 0 : first_q / BQ;
  }
  const int n_iter = max(0, nq_blocks - i_start);

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report(p.status, MB_ERR_BAD_ARG);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, kWG);
    mbar_init(dq_full, 1);
    mbar_init(final_full, 1);
    fence_barrier_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
    prefetch_tmap(&tm_do);
    prefetch_tmap(&tm_dq);
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 64, t_dq = tmem_base + 128;
  const uint32_t t_dv = tmem_base + 192, t_dk = tmem_base + 320;

  const uint32_t ck = BKV * 128;  // chunk stride of K / V tiles
  const uint32_t cq = BQ * 128;   // chunk stride of Q / dO tiles

  if (warp == 8) {
    // ----------------------------------------------------------- TMA producer
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(kv_full, 2 * p.nchunks * ck);
      for (int c = 0; c < p.nchunks; ++c) {
        tma_load_4d(smem + L::oK + c * ck, &tm_k, kv_full, 64 * c, head, kv0, batch);
        tma_load_4d(smem + L::oV + c * ck, &tm_v, kv_full, 64 * c, head, kv0, batch);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        if (it >= 2 && !mbar_wait(&q_empty[st], ((it >> 1) - 1) & 1)) {
          report(p.status, MB_ERR_TIMEOUT_EMPTY);
          break;
        }
        uint8_t* sq_ = smem + L::oQ + st * 2 * L::kQ;
        uint8_t* sdo_ = sq_ + L::kQ;
        const int q0 = (i_start + it) * BQ;
        mbar_expect_tx(&q_full[st], 2 * p.nchunks * cq);
        for (int c = 0; c < p.nchunks; ++c) {
          tma_load_4d(sq_ + c * cq, &tm_q, &q_full[st], 64 * c, head, q0, batch);
          tma_load_4d(sdo_ + c * cq, &tm_do, &q_full[st], 64 * c, head, q0, batch);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------- MMA issuer
    if (n_iter > 0) {
      const uint32_t idesc_sq = make_idesc_bf16(128, BQ, 0, 0);        // S^T, dP^T
      const uint32_t idesc_dkv = make_idesc_bf16(128, p.d, 0, 1);      // dV, dK
      const uint32_t idesc_dq = make_idesc_bf16(128, BQ, 1, 1);        // dQ^T
      const uint32_t sk_ = smem_u32(smem + L::oK), sv_ = smem_u32(smem + L::oV);
      const uint32_t sp_ = smem_u32(smem + L::oP), sds_ = smem_u32(smem + L::oDS);
      const int ksteps = p.d / 16;
      bool ok = mbar_wait(kv_full, 0);
      if (!ok) report(p.status, MB_ERR_TIMEOUT_FULL);

      auto issue_sdp = [&](int it) -> bool {
        const int st = it & 1;
        if (!mbar_wait(&q_full[st], (it >> 1) & 1)) return false;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sq_ = smem_u32(smem + L::oQ + st * 2 * L::kQ), sdo_ = sq_ + L::kQ;
          for (int kk = 0; kk < ksteps; ++kk) {
            const uint32_t ch = kk >> 2, in = (kk & 3) * 32;
            mma_f16_ss(t_s, make_smem_desc_sw128(sk_ + ch * ck + in, 16, 1024),
                       make_smem_desc_sw128(sq_ + ch * cq + in, 16, 1024), idesc_sq, kk != 0);
          }
          for (int kk = 0; kk < ksteps; ++kk) {
            const uint32_t ch = kk >> 2, in = (kk & 3) * 32;
            mma_f16_ss(t_dp, make_smem_desc_sw128(sv_ + ch * ck + in, 16, 1024),
                       make_smem_desc_sw128(sdo_ + ch * cq + in, 16, 1024), idesc_sq, kk != 0);
          }
          mma_commit(sdp_full);
        }
        __syncwarp();
        return true;
      };

      if (ok && !issue_sdp(0)) { report(p.status, MB_ERR_TIMEOUT_FULL); ok = false; }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1;
        if (!mbar_wait(pds_full, it & 1)) {
          report(p.status, MB_ERR_TIMEOUT_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sq_ = smem_u32(smem + L::oQ + st * 2 * L::kQ), sdo_ = sq_ + L::kQ;
          // dV += P^T dO ; dK += dS^T Q   (K = 64 query rows -> 4 steps)
#pragma unroll
          for (int kk = 0; kk < BQ / 16; ++kk) {
            mma_f16_ss(t_dv, make_smem_desc_sw128(sp_ + kk * 32, 16, 1024),
                       make_smem_desc_sw128(sdo_ + kk * 2048, cq, 1024), idesc_dkv, (it | kk) != 0);
          }
#pragma unroll
          for (int kk = 0; kk < BQ / 16; ++kk) {
            mma_f16_ss(t_dk, make_smem_desc_sw128(sds_ + kk * 32, 16, 1024),
                       make_smem_desc_sw128(sq_ + kk * 2048, cq, 1024), idesc_dkv, (it | kk) != 0);
          }
          // dQ^T = K^T dS   (K = 128 key rows -> 8 steps); A = K as MN-major, B = dS^T as MN-major
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk) {
            mma_f16_ss(t_dq, make_smem_desc_sw128(sk_ + kk * 2048, ck, 1024),
                       make_smem_desc_sw128(sds_ + kk * 2048, ck, 1024), idesc_dq, kk != 0);
          }
          mma_commit(&q_empty[st]);
          mma_commit(dq_full);
        }
        __syncwarp();
        if (it + 1 < n_iter && !issue_sdp(it + 1)) {
          report(p.status, MB_ERR_TIMEOUT_FULL);
          ok = false;
          break;
        }
      }
      if (ok && lane == 0) mma_commit(final_full);
      __syncwarp();
    }
  } else {
    // ------------------------------------------- softmax / dS / dQ write-out / epilogue
    // Two warpgroups share the 128 TMEM lanes: warps 0-3 take query columns 0-31 of every
    // key row, warps 4-7 columns 32-63 (a warp may touch lanes 32*(warp%4) .. +31).
    const int r = threadIdx.x & 127;   // key row of the block == TMEM lane; d index for dQ^T
    const int half = threadIdx.x >> 7; // which 32 query columns
    const int c0 = half * 32;
    const int kv_idx = kv0 + r;
    const int kv_last = kv0 + BKV - 1;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const bool leader = (threadIdx.x == 0);
    uint8_t* sp_ = smem + L::oP;
    uint8_t* sds_ = smem + L::oDS;
    uint8_t* sdq_ = smem + L::oDQ;
    float* s_lse = reinterpret_cast<float*>(smem + L::oVec);        // [2][BQ], pre-multiplied by log2(e)
    float* s_delta = s_lse + 2 * BQ;                                 // [2][BQ]
    const long row_base = (static_cast<long>(batch) * p.nh + head) * p.sq;
    bool ok = true;

    // per-block vectors: thread t < 64 stages lse, 64 <= t < 128 stages delta
    auto fetch_vec = [&](int it) -> float {
      const int q = (i_start + it) * BQ + (threadIdx.x & 63);
      if (threadIdx.x >= 128 || q >= sq_b) return 0.f;
      return threadIdx.x < 64 ? p.lse[row_base + q] * 1.4426950408889634f : p.delta[row_base + q];
    };
    auto stash_vec = [&](int buf, float v) {
      if (threadIdx.x < 64) s_lse[buf * BQ + threadIdx.x] = v;
      else if (threadIdx.x < 128) s_delta[buf * BQ + threadIdx.x - 64] = v;
    };
    if (n_iter > 0) stash_vec(0, fetch_vec(0));
    asm volatile("bar.sync 1, 256;" ::: "memory");

    for (int it = 0; it < n_iter && ok; ++it) {
      const int q0 = (i_start + it) * BQ;
      const int vb = it & 1;
      const float nxt = (it + 1 < n_iter) ? fetch_vec(it + 1) : 0.f;   // in flight during this iteration
      if (!mbar_wait(sdp_full, it & 1)) {
        report(p.status, MB_ERR_TIMEOUT_TMEM);
        ok = false;
        break;
      }
      tc_fence_after();
      float pf[32];
      uint32_t pk[16];
      {
        uint32_t sr[32];
        tmem_ld32(t_s + c0 + lane_off, sr);
        tmem_ld_wait();
        // Only blocks on the diagonal or at the end of the queries / keys need the mask (the test
        // is uniform over the CTA): the others take the shorter loop.
        const bool need_mask = (q0 + BQ > sq_b) || (kv_last >= sk_b) || (p.causal && kv_last > q0 + coff);
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int qi = q0 + c0 + c;
            const bool valid = (qi < sq_b) && (kv_idx < sk_b) && (!p.causal || kv_idx <= qi + coff);
            const float e = mb::fast_exp2(fmaf(__uint_as_float(sr[c]), p.scale_log2, -s_lse[vb * BQ + c0 + c]));
            pf[c] = valid ? e : 0.f;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c)
            pf[c] = mb::fast_exp2(fmaf(__uint_as_float(sr[c]), p.scale_log2, -s_lse[vb * BQ + c0 + c]));
        }
#pragma unroll
        for (int c = 0; c < 32; c += 2) pk[c >> 1] = pack2(pf[c], pf[c + 1]);
      }
      // The previous iteration's MMAs are done with the P / dS tiles: this thread waited
      // for that iteration's dq_full before coming back here.
#pragma unroll
      for (int g = 0; g < 4; ++g)
        *reinterpret_cast<uint4*>(sp_ + r * 128 + (((half * 4 + g) ^ (r & 7)) << 4)) =
            make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
      {
        uint32_t dr[32];
        tmem_ld32(t_dp + c0 + lane_off, dr);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float a = p.scale * pf[c] * (__uint_as_float(dr[c]) - s_delta[vb * BQ + c0 + c]);
          const float b = p.scale * pf[c + 1] * (__uint_as_float(dr[c + 1]) - s_delta[vb * BQ + c0 + c + 1]);
          pk[c >> 1] = pack2(a, b);
        }
      }
#pragma unroll
      for (int g = 0; g < 4; ++g)
        *reinterpret_cast<uint4*>(sds_ + r * 128 + (((half * 4 + g) ^ (r & 7)) << 4)) =
            make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(pds_full);
      stash_vec(vb ^ 1, nxt);   // next block's vectors; made visible by the barriers below

      // ---- dQ^T of this iteration: TMEM -> transposed staging -> TMA reduce-add
      if (!mbar_wait(dq_full, it & 1)) {
        report(p.status, MB_ERR_TIMEOUT_TMEM);
        ok = false;
        break;
      }
      tc_fence_after();
      if (leader) tma_wait_read<0>();            // previous reduce has read the staging tile
      asm volatile("bar.sync 1, 256;" ::: "memory");
      {
        uint32_t qr[32];
        tmem_ld32(t_dq + c0 + lane_off, qr);
        tmem_ld_wait();
        // thread holds dQ[q0 + c0 + c][d = r]; staging chunk r / 32 is [64 q][32 d] fp32
        uint8_t* chunk = sdq_ + (r >> 5) * cq;
        const int dl = r & 31;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int qc = c0 + c;
          *reinterpret_cast<uint32_t*>(chunk + qc * 128 + ((((dl >> 2) ^ (qc & 7)) << 4) | ((dl & 3) << 2))) = qr[c];
        }
      }
      fence_async_smem();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (leader) {
        for (int w = 0; w * 32 < p.d; ++w) {
          asm volatile(
              "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group "
              "[%0, {%2, %3, %4}], [%1];\n" ::"l"(reinterpret_cast<uint64_t>(&tm_dq)),
              "r"(smem_u32(sdq_ + w * cq)), "r"(32 * w), "r"(q0), "r"(batch * p.nh + head)
              : "memory");
        }
        tma_commit();
      }
    }

    // ---- dK, dV: TMEM -> bf16 -> global (one key row per thread, column chunks split
    // between the two warpgroups)
    if (ok && n_iter > 0 && !mbar_wait(final_full, 0)) {
      report(p.status, MB_ERR_TIMEOUT_TMEM);
      ok = false;
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dkrow = p.dk + batch * p.dk_bs + static_cast<long>(kv_idx) * p.dk_ts + head * p.dk_hs;
      __nv_bfloat16* dvrow = p.dv + batch * p.dv_bs + static_cast<long>(kv_idx) * p.dv_ts + head * p.dv_hs;
      for (int c = half; c < p.d / 16; c += 2) {
        uint32_t a[16], b[16];
        if (n_iter > 0) {
          tmem_ld16(t_dv + c * 16 + lane_off, a);
          tmem_ld16(t_dk + c * 16 + lane_off, b);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) a[i] = b[i] = 0;
        }
        if (kv_idx < p.sk) {
          float fa[16], fb[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            fa[i] = __uint_as_float(a[i]);
            fb[i] = __uint_as_float(b[i]);
          }
          *reinterpret_cast<mb::bf16x8*>(dvrow + c * 16) = mb::pack8(fa);
          *reinterpret_cast<mb::bf16x8*>(dvrow + c * 16 + 8) = mb::pack8(fa + 8);
          *reinterpret_cast<mb::bf16x8*>(dkrow + c * 16) = mb::pack8(fb);
          *reinterpret_cast<mb::bf16x8*>(dkrow + c * 16 + 8) = mb::pack8(fb + 8);
        }
      }
    }
    if (leader) tma_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// Pipelined variant.  Same math, tiles and shared-memory layouts as the kernel
// above; what changes is who waits for whom:
//
//   * S^T and dP^T are double buffered in tensor memory and the MMA warp issues the two products
//     of query block it+1 before it waits for the probabilities of block it, so the tensor cores
//     work on the next block while the softmax warps are busy with the current one;
//   * Q / dO arrive through three stages, so the early S^T / dP^T issue never waits for a load
//     that was only just requested;
//   * the dQ^T read-out (tensor memory -> transposed staging -> TMA reduce-add) has its own four
//     warps, so the softmax warps go straight from one block to the next.
//
// Tensor memory (512 columns), head size <= 96: S^T[2] 0..127, dP^T[2] 128..255, dQ^T 256..319,
// dV 320..415, dK 416..511; the products of block it wait until the dQ warps have read dQ^T of block
// it-1.  Head size up to 128: dV 256..383, dK 384..511 and dQ^T of block it is written over
// S^T[it & 1] (by then that buffer is in the softmax warps' registers); the next product that writes
// the buffer, S^T of block it+2, waits until the dQ warps have read dQ^T out.
// Warps 0-7 softmax / dS (and the dK, dV epilogue), warps 8-11 dQ, 12 TMA, 13 MMA.
//
// Barriers and the iteration `it` they belong to (b = it & 1, st = it % 3):
//   q_full[st]   producer -> MMA      Q, dO of block it are in stage st
//   q_empty[st]  MMA commit -> producer  the dV / dK / dQ products of block it have read stage st
//   sdp_full[b]  MMA commit -> softmax   S^T[b], dP^T[b] of block it are complete
//   pds_full     softmax (256) -> MMA    P^T, dS^T of block it are in shared memory (and S^T[b],
//                                        dP^T[b] are in registers: dQ^T of this block may overwrite
//                                        S^T[b], block it+2 may overwrite dP^T[b])
//   pds_empty    MMA commit -> softmax   the products of block it have read P^T, dS^T
//   dq_full[b]   MMA commit -> dQ warps  dQ^T of block it is complete (one barrier per buffer: the
//                                        products of block it+1 do not wait for the dQ warps, so a
//                                        single barrier could run two phases ahead of them)
//   dq_empty     dQ warps (128) -> MMA   dQ^T of block it is in registers
// A thread can arrive on pds_full / dq_empty for block it+1 only after a wait that itself needs the
// phase of block it to have completed, so no phase is entered twice.
constexpr int kThreadsPipe = 448;
constexpr int kQStages = 3;
constexpr int kDQWarp0 = 8;       // first dQ warp; 8 % 4 == 0, so warp w owns TMEM lanes 32 * (w - 8) ...
constexpr int kTmaWarp = 12, kMmaWarp = 13;

struct SmemPipe {
  static constexpr int kKV = 2 * BKV * 128;
  static constexpr int kQ = 2 * BQ * 128;
  static constexpr int kP = BKV * 128;
  static constexpr int kDQ = 4 * BQ * 128;      // four chunks of [64 q][32 fp32]
  static constexpr int oK = 0;
  static constexpr int oV = oK + kKV;
  static constexpr int oQ = oV + kKV;           // kQStages stages of (Q, dO)
  static constexpr int oP = oQ + kQStages * 2 * kQ;
  static constexpr int oDS = oP + kP;
  static constexpr int oDQ = oDS + kP;
  static constexpr int oBar = oDQ + kDQ;
  // kv_full, q_full[3], q_empty[3], sdp_full[2], pds_full, pds_empty, dq_full[2], dq_empty, final_full
  static constexpr int kNumBars = 15;
  static constexpr int oVec = oBar + kNumBars * 8 + 16;
  static constexpr int kTotal = oVec + 2 * 2 * BQ * 4;
};
static_assert(SmemPipe::kTotal <= 232448, "pipelined attention backward: shared memory over the per-CTA limit");

__global__ void __launch_bounds__(kThreadsPipe, 1)
attn_bwd_pipe_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_dq, const BwdParams p) {
  using L = SmemPipe;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::oBar);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;
  uint64_t* q_empty = bars + 4;
  uint64_t* sdp_full = bars + 7;
  uint64_t* pds_full = bars + 9;
  uint64_t* pds_empty = bars + 10;
  uint64_t* dq_full = bars + 11;
  uint64_t* dq_empty = bars + 13;
  uint64_t* final_full = bars + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int jb = blockIdx.x;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  // real tokens of this sample (right-padded batches); the tensors keep their padded extents p.sq / p.sk
  const int sq_b = p.seqlens_q ? min(p.sq, p.seqlens_q[batch]) : p.sq;
  const int sk_b = p.seqlens_k ? min(p.sk, p.seqlens_k[batch]) : p.sk;
  const int kv0 = jb * BKV;
  const int coff = sk_b - sq_b;
  const int nq_blocks = (sq_b + BQ - 1) / BQ;
  int i_start = 0;
  if (p.causal) {
    int first_q = kv0 - coff;
    i_start = first_q <= 0 ? 0 : first_q / BQ;
  }
  const int n_iter = max(0, nq_blocks - i_start);

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report(p.status, MB_ERR_BAD_ARG);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) mbar_init(&sdp_full[s], 1);
    mbar_init(pds_full, kWG);
    mbar_init(pds_empty, 1);
    mbar_init(&dq_full[0], 1);
    mbar_init(&dq_full[1], 1);
    mbar_init(dq_empty, 128);
    mbar_init(final_full, 1);
    fence_barrier_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
    prefetch_tmap(&tm_do);
    prefetch_tmap(&tm_dq);
  }
  if (warp == kTmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool alias_dq = p.d > 96;      // no room for a dQ^T buffer of its own
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128;   // + 64 * (it & 1)
  const uint32_t t_dv = tmem_base + (alias_dq ? 256 : 320), t_dk = tmem_base + (alias_dq ? 384 : 416);
  auto t_dq = [&](int it) -> uint32_t { return alias_dq ? t_s + (it & 1) * BQ : tmem_base + 256; };

  const uint32_t ck = BKV * 128;
  const uint32_t cq = BQ * 128;

  if (warp == kTmaWarp) {
    // ----------------------------------------------------------- TMA producer
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(kv_full, 2 * p.nchunks * ck);
      for (int c = 0; c < p.nchunks; ++c) {
        tma_load_4d(smem + L::oK + c * ck, &tm_k, kv_full, 64 * c, head, kv0, batch);
        tma_load_4d(smem + L::oV + c * ck, &tm_v, kv_full, 64 * c, head, kv0, batch);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % kQStages;
        if (it >= kQStages && !mbar_wait(&q_empty[st], ((it / kQStages) - 1) & 1)) {
          report(p.status, MB_ERR_TIMEOUT_EMPTY);
          break;
        }
        uint8_t* sq_ = smem + L::oQ + st * 2 * L::kQ;
        uint8_t* sdo_ = sq_ + L::kQ;
        const int q0 = (i_start + it) * BQ;
        mbar_expect_tx(&q_full[st], 2 * p.nchunks * cq);
        for (int c = 0; c < p.nchunks; ++c) {
          tma_load_4d(sq_ + c * cq, &tm_q, &q_full[st], 64 * c, head, q0, batch);
          tma_load_4d(sdo_ + c * cq, &tm_do, &q_full[st], 64 * c, head, q0, batch);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------- MMA issuer
    if (n_iter > 0) {
      const uint32_t idesc_sq = make_idesc_bf16(128, BQ, 0, 0);        // S^T, dP^T
      const uint32_t idesc_dkv = make_idesc_bf16(128, p.d, 0, 1);      // dV, dK
      const uint32_t idesc_dq = make_idesc_bf16(128, BQ, 1, 1);        // dQ^T
      const uint32_t sk_ = smem_u32(smem + L::oK), sv_ = smem_u32(smem + L::oV);
      const uint32_t sp_ = smem_u32(smem + L::oP), sds_ = smem_u32(smem + L::oDS);
      const int ksteps = p.d / 16;
      bool ok = mbar_wait(kv_full, 0);
      if (!ok) report(p.status, MB_ERR_TIMEOUT_FULL);

      // S^T[b] = K Q^T, dP^T[b] = V dO^T of block `it`
      auto issue_sdp = [&](int it) -> bool {
        const int st = it % kQStages, b = it & 1;
        if (!mbar_wait(&q_full[st], (it / kQStages) & 1)) return false;
        // S^T[b], dP^T[b] of block it-2 are free (the caller waited for pds_full of that block); with
        // the shared buffer S^T[b] held dQ^T of block it-2 since then
        if (alias_dq && it >= 2 && !mbar_wait(dq_empty, (it - 2) & 1)) return false;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sq_ = smem_u32(smem + L::oQ + st * 2 * L::kQ), sdo_ = sq_ + L::kQ;
          for (int kk = 0; kk < ksteps; ++kk) {
            const uint32_t ch = kk >> 2, in = (kk & 3) * 32;
            mma_f16_ss(t_s + b * BQ, make_smem_desc_sw128(sk_ + ch * ck + in, 16, 1024),
                       make_smem_desc_sw128(sq_ + ch * cq + in, 16, 1024), idesc_sq, kk != 0);
          }
          for (int kk = 0; kk < ksteps; ++kk) {
            const uint32_t ch = kk >> 2, in = (kk & 3) * 32;
            mma_f16_ss(t_dp + b * BQ, make_smem_desc_sw128(sv_ + ch * ck + in, 16, 1024),
                       make_smem_desc_sw128(sdo_ + ch * cq + in, 16, 1024), idesc_sq, kk != 0);
          }
          mma_commit(&sdp_full[b]);
        }
        __syncwarp();
        return true;
      };

      if (ok && !issue_sdp(0)) { report(p.status, MB_ERR_TIMEOUT_FULL); ok = false; }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it % kQStages;
        // next block's products first: they run while the softmax warps work on this block
        if (it + 1 < n_iter && !issue_sdp(it + 1)) {
          report(p.status, MB_ERR_TIMEOUT_FULL);
          ok = false;
          break;
        }
        if (!mbar_wait(pds_full, it & 1) || (!alias_dq && it > 0 && !mbar_wait(dq_empty, (it - 1) & 1))) {
          report(p.status, MB_ERR_TIMEOUT_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sq_ = smem_u32(smem + L::oQ + st * 2 * L::kQ), sdo_ = sq_ + L::kQ;
#pragma unroll
          for (int kk = 0; kk < BQ / 16; ++kk) {
            mma_f16_ss(t_dv, make_smem_desc_sw128(sp_ + kk * 32, 16, 1024),
                       make_smem_desc_sw128(sdo_ + kk * 2048, cq, 1024), idesc_dkv, (it | kk) != 0);
          }
#pragma unroll
          for (int kk = 0; kk < BQ / 16; ++kk) {
            mma_f16_ss(t_dk, make_smem_desc_sw128(sds_ + kk * 32, 16, 1024),
                       make_smem_desc_sw128(sq_ + kk * 2048, cq, 1024), idesc_dkv, (it | kk) != 0);
          }
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk) {
            mma_f16_ss(t_dq(it), make_smem_desc_sw128(sk_ + kk * 2048, ck, 1024),
                       make_smem_desc_sw128(sds_ + kk * 2048, ck, 1024), idesc_dq, kk != 0);
          }
          mma_commit(&q_empty[st]);
          mma_commit(pds_empty);
          mma_commit(&dq_full[it & 1]);
        }
        __syncwarp();
      }
      if (ok && lane == 0) mma_commit(final_full);
      __syncwarp();
    }
  } else if (warp >= kDQWarp0) {
    // --------------------------------- dQ^T: TMEM -> transposed staging -> TMA reduce-add
    const int r = threadIdx.x - kDQWarp0 * 32;     // d index == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const bool leader = (r == 0);
    uint8_t* sdq_ = smem + L::oDQ;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int q0 = (i_start + it) * BQ;
      if (!mbar_wait(&dq_full[it & 1], (it >> 1) & 1)) {
        report(p.status, MB_ERR_TIMEOUT_TMEM);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t qr[BQ];
      tmem_ld32(t_dq(it) + lane_off, qr);
      tmem_ld32(t_dq(it) + 32 + lane_off, qr + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dq_empty);
      if (leader) tma_wait_read<0>();            // the previous reduce has read the staging tile
      asm volatile("bar.sync 2, 128;" ::: "memory");
      {
        // thread holds dQ[q0 + c][d = r]; staging chunk r / 32 is [64 q][32 d] fp32, 128-byte swizzled
        uint8_t* chunk = sdq_ + (r >> 5) * cq;
        const int dl = r & 31;
#pragma unroll
        for (int c = 0; c < BQ; ++c)
          *reinterpret_cast<uint32_t*>(chunk + c * 128 + ((((dl >> 2) ^ (c & 7)) << 4) | ((dl & 3) << 2))) = qr[c];
      }
      fence_async_smem();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (leader) {
        for (int w = 0; w * 32 < p.d; ++w) {
          asm volatile(
              "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group "
              "[%0, {%2, %3, %4}], [%1];\n" ::"l"(reinterpret_cast<uint64_t>(&tm_dq)),
              "r"(smem_u32(sdq_ + w * cq)), "r"(32 * w), "r"(q0), "r"(batch * p.nh + head)
              : "memory");
        }
        tma_commit();
      }
    }
    if (leader) tma_wait_all<0>();
  } else {
    // ------------------------------------------------------ softmax / dS / dK, dV epilogue
    const int r = threadIdx.x & 127;
    const int half = threadIdx.x >> 7;
    const int c0 = half * 32;
    const int kv_idx = kv0 + r;
    const int kv_last = kv0 + BKV - 1;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint8_t* sp_ = smem + L::oP;
    uint8_t* sds_ = smem + L::oDS;
    float* s_lse = reinterpret_cast<float*>(smem + L::oVec);
    float* s_delta = s_lse + 2 * BQ;
    const long row_base = (static_cast<long>(batch) * p.nh + head) * p.sq;
    bool ok = true;

    auto fetch_vec = [&](int it) -> float {
      const int q = (i_start + it) * BQ + (threadIdx.x & 63);
      if (threadIdx.x >= 128 || q >= sq_b) return 0.f;
      return threadIdx.x < 64 ? p.lse[row_base + q] * 1.4426950408889634f : p.delta[row_base + q];
    };
    auto stash_vec = [&](int buf, float v) {
      if (threadIdx.x < 64) s_lse[buf * BQ + threadIdx.x] = v;
      else if (threadIdx.x < 128) s_delta[buf * BQ + threadIdx.x - 64] = v;
    };
    if (n_iter > 0) stash_vec(0, fetch_vec(0));
    asm volatile("bar.sync 1, 256;" ::: "memory");

    for (int it = 0; it < n_iter && ok; ++it) {
      const int q0 = (i_start + it) * BQ;
      const int vb = it & 1;
      const float nxt = (it + 1 < n_iter) ? fetch_vec(it + 1) : 0.f;
      if (!mbar_wait(&sdp_full[vb], (it >> 1) & 1)) {
        report(p.status, MB_ERR_TIMEOUT_TMEM);
        ok = false;
        break;
      }
      tc_fence_after();
      float pf[32];
      uint32_t pk[16], dk_[16];
      {
        uint32_t sr[32];
        tmem_ld32(t_s + vb * BQ + c0 + lane_off, sr);
        tmem_ld_wait();
        const bool need_mask = (q0 + BQ > sq_b) || (kv_last >= sk_b) || (p.causal && kv_last > q0 + coff);
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int qi = q0 + c0 + c;
            const bool valid = (qi < sq_b) && (kv_idx < sk_b) && (!p.causal || kv_idx <= qi + coff);
            const float e = mb::fast_exp2(fmaf(__uint_as_float(sr[c]), p.scale_log2, -s_lse[vb * BQ + c0 + c]));
            pf[c] = valid ? e : 0.f;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c)
            pf[c] = mb::fast_exp2(fmaf(__uint_as_float(sr[c]), p.scale_log2, -s_lse[vb * BQ + c0 + c]));
        }
#pragma unroll
        for (int c = 0; c < 32; c += 2) pk[c >> 1] = pack2(pf[c], pf[c + 1]);
      }
      {
        uint32_t dr[32];
        tmem_ld32(t_dp + vb * BQ + c0 + lane_off, dr);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float a = p.scale * pf[c] * (__uint_as_float(dr[c]) - s_delta[vb * BQ + c0 + c]);
          const float b = p.scale * pf[c + 1] * (__uint_as_float(dr[c + 1]) - s_delta[vb * BQ + c0 + c + 1]);
          dk_[c >> 1] = pack2(a, b);
        }
      }
      // the previous block's products must be done with the P^T / dS^T tiles before they are rewritten
      if (it > 0) {
        if (!mbar_wait(pds_empty, (it - 1) & 1)) {
          report(p.status, MB_ERR_TIMEOUT_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint32_t off = r * 128 + (((half * 4 + g) ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(sp_ + off) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
        *reinterpret_cast<uint4*>(sds_ + off) = make_uint4(dk_[4 * g], dk_[4 * g + 1], dk_[4 * g + 2], dk_[4 * g + 3]);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(pds_full);
      stash_vec(vb ^ 1, nxt);
      asm volatile("bar.sync 1, 256;" ::: "memory");   // next block's lse / delta visible to all 256
    }

    if (ok && n_iter > 0 && !mbar_wait(final_full, 0)) {
      report(p.status, MB_ERR_TIMEOUT_TMEM);
      ok = false;
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dkrow = p.dk + batch * p.dk_bs + static_cast<long>(kv_idx) * p.dk_ts + head * p.dk_hs;
      __nv_bfloat16* dvrow = p.dv + batch * p.dv_bs + static_cast<long>(kv_idx) * p.dv_ts + head * p.dv_hs;
      for (int c = half; c < p.d / 16; c += 2) {
        uint32_t a[16], b[16];
        if (n_iter > 0) {
          tmem_ld16(t_dv + c * 16 + lane_off, a);
          tmem_ld16(t_dk + c * 16 + lane_off, b);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) a[i] = b[i] = 0;
        }
        if (kv_idx < p.sk) {
          float fa[16], fb[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            fa[i] = __uint_as_float(a[i]);
            fb[i] = __uint_as_float(b[i]);
          }
          *reinterpret_cast<mb::bf16x8*>(dvrow + c * 16) = mb::pack8(fa);
          *reinterpret_cast<mb::bf16x8*>(dvrow + c * 16 + 8) = mb::pack8(fa + 8);
          *reinterpret_cast<mb::bf16x8*>(dkrow + c * 16) = mb::pack8(fb);
          *reinterpret_cast<mb::bf16x8*>(dkrow + c * 16 + 8) = mb::pack8(fb + 8);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b][h][q] = sum_d dO[b][q][h][d] * O[b][q][h][d]; one warp per (b, q, h)
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ o,
                                  float* __restrict__ delta, int batch, int sq, int nh, int d, long do_bs,
                                  long do_ts, long do_hs, long o_bs, long o_ts, long o_hs) {
  const long w = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long total = static_cast<long>(batch) * sq * nh;
  if (w >= total) return;
  const int h = static_cast<int>(w % nh);
  const long t = w / nh;
  const int q = static_cast<int>(t % sq);
  const int b = static_cast<int>(t / sq);
  const __nv_bfloat16* a = dout + b * do_bs + q * do_ts + h * do_hs;
  const __nv_bfloat16* c = o + b * o_bs + q * o_ts + h * o_hs;
  float acc = 0.f;
  for (int i = lane * 8; i < d; i += 256) {
    float x[8], y[8];
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(a + i), x);
    mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(c + i), y);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc += x[k] * y[k];
  }
  acc = mb::warp_sum(acc);
  if (lane == 0) delta[(static_cast<long>(b) * nh + h) * sq + q] = acc;
}

// dq[b][q][h][:] = bf16(dq_acc[b][h][q][:])
__global__ void attn_convert_dq_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int batch,
                                       int sq, int nh, int d, long dq_bs, long dq_ts, long dq_hs) {
  const int vpr = d >> 3;
  const long nvec = static_cast<long>(batch) * nh * sq * vpr;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vpr);
    long t = i / vpr;
    const int q = static_cast<int>(t % sq);
    t /= sq;
    const int h = static_cast<int>(t % nh);
    const int b = static_cast<int>(t / nh);
    const float4 x = reinterpret_cast<const float4*>(acc)[2 * i];
    const float4 y = reinterpret_cast<const float4*>(acc)[2 * i + 1];
    float f[8] = {x.x, x.y, x.z, x.w, y.x, y.y, y.z, y.w};
    *reinterpret_cast<mb::bf16x8*>(dq + b * dq_bs + static_cast<long>(q) * dq_ts + h * dq_hs + 8 * v) = mb::pack8(f);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

bool make_map4(CUtensorMap* m, const void* base, int batch, int tokens, int heads, int d, long bs, long ts,
               long hs, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(hs) * 2, static_cast<cuuint64_t>(ts) * 2,
                           static_cast<cuuint64_t>(bs) * 2};
  cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_with_context([&] {
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

// dq accumulator [b*nh][sq][d] fp32, box [1][64][32]
bool make_map_dq(CUtensorMap* m, float* base, int bh, int sq, int d) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(sq), static_cast<cuuint64_t>(bh)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(d) * 4, static_cast<cuuint64_t>(sq) * d * 4};
  cuuint32_t box[3] = {32, static_cast<cuuint32_t>(BQ), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return encode_with_context([&] {
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

int g_bwd_variant = 0;        // 0: one block at a time; 1: pipelined
int g_bwd_last_variant = 0;

}  // namespace

MB_API int* mb_status_device_ptr();

// Chooses the main backward kernel for later calls: 0 = the kernel that finishes one query block
// before it starts the next (default), 1 = the pipelined kernel.
MB_API void mb_attn_bwd_set_variant(int v) { g_bwd_variant = (v == 1) ? 1 : 0; }
// Variant the last call of mb_attn_bwd launched.
MB_API int mb_attn_bwd_last_variant() { return g_bwd_last_variant; }

// dout, o: [b][sq][nh][d] with the given element strides for dout (o is contiguous);
// delta: [b][nh][sq] fp32 scratch; dq_acc: [b][nh][sq][d] fp32 scratch, zeroed by this call.
// q/k/v and dq/dk/dv may be strided views (packed qkv).  Requires nh_kv == nh.  seqlens_q / seqlens_k:
// optional device arrays of `batch` ints (real tokens per sample of a right-padded batch, as in the forward
// pass): padded queries and keys take no part, their gradient rows are zeros.
MB_API int mb_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o,
                       const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv, int batch,
                       int sq, int sk, int nh, int d, long q_bs, long q_ts, long q_hs, long k_bs, long k_ts,
                       long k_hs, long v_bs, long v_ts, long v_hs, long dq_bs, long dq_ts, long dq_hs,
                       long dk_bs, long dk_ts, long dk_hs, long dv_bs, long dv_ts, long dv_hs, float scale,
                       int causal, const int* seqlens_q, const int* seqlens_k, cudaStream_t stream) {
  if (d % 16 || d > 128 || d < 16) return -1;
  if ((q_bs | q_ts | q_hs | k_bs | k_ts | k_hs | v_bs | v_ts | v_hs | dq_bs | dq_ts | dq_hs | dk_bs | dk_ts |
       dk_hs | dv_bs | dv_ts | dv_hs) & 7)
    return -1;
  if (batch == 0 || sq == 0 || sk == 0) return 0;
  const long o_ts = static_cast<long>(nh) * d, o_bs = o_ts * sq;
  {
    long warps = static_cast<long>(batch) * sq * nh;
    long blocks = (warps * 32 + 255) / 256;
    attn_delta_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dout), reinterpret_cast<const __nv_bfloat16*>(o), delta, batch, sq,
        nh, d, o_bs, o_ts, d, o_bs, o_ts, d);
  }
  if (cudaMemsetAsync(dq_acc, 0, sizeof(float) * batch * nh * static_cast<size_t>(sq) * d, stream) != cudaSuccess)
    return -4;
  CUtensorMap tq, tk, tv, tdo, tdq;
  if (!make_map4(&tq, q, batch, sq, nh, d, q_bs, q_ts, q_hs, BQ)) return -2;
  if (!make_map4(&tk, k, batch, sk, nh, d, k_bs, k_ts, k_hs, BKV)) return -2;
  if (!make_map4(&tv, v, batch, sk, nh, d, v_bs, v_ts, v_hs, BKV)) return -2;
  if (!make_map4(&tdo, dout, batch, sq, nh, d, o_bs, o_ts, d, BQ)) return -2;
  if (!make_map_dq(&tdq, dq_acc, batch * nh, sq, d)) return -2;
  BwdParams p;
  p.lse = lse; p.delta = delta;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.dk_bs = dk_bs; p.dk_ts = dk_ts; p.dk_hs = dk_hs;
  p.dv_bs = dv_bs; p.dv_ts = dv_ts; p.dv_hs = dv_hs;
  p.sq = sq; p.sk = sk; p.nh = nh; p.d = d;
  p.nchunks = (d + 63) / 64;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.seqlens_q = seqlens_q;
  p.seqlens_k = seqlens_k;
  p.status = mb_status_device_ptr();
  dim3 grid((sk + BKV - 1) / BKV, nh, batch);
  if (g_bwd_variant == 1) {
    static bool cfg_pipe = false;
    if (!cfg_pipe) {
      if (cudaFuncSetAttribute(attn_bwd_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               SmemPipe::kTotal) != cudaSuccess)
        return -3;
      cfg_pipe = true;
    }
    attn_bwd_pipe_kernel<<<grid, kThreadsPipe, SmemPipe::kTotal, stream>>>(tq, tk, tv, tdo, tdq, p);
    g_bwd_last_variant = 1;
  } else {
    static bool cfg = false;
    if (!cfg) {
      if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal) !=
          cudaSuccess)
        return -3;
      cfg = true;
    }
    attn_bwd_kernel<<<grid, kThreads, Smem::kTotal, stream>>>(tq, tk, tv, tdo, tdq, p);
    g_bwd_last_variant = 0;
  }
  {
    long nvec = static_cast<long>(batch) * nh * sq * (d / 8);
    long blocks = (nvec + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    attn_convert_dq_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        dq_acc, reinterpret_cast<__nv_bfloat16*>(dq), batch, sq, nh, d, dq_bs, dq_ts, dq_hs);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
