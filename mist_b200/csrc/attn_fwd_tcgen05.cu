// Causal / full multi-head attention forward on tcgen05 tensor cores.
//
//   O = softmax(scale * Q K^T + causal mask) V,   LSE = logsumexp per row
//
// One CTA owns a 128-row query tile of one (batch, head) and walks the key/value
// sequence in blocks of BN rows (flash-attention recurrence).  Both GEMMs of a block
// run on tcgen05.mma with the accumulators in tensor memory:
//   S  = Q K^T   (A = Q K-major, B = K K-major)      -> TMEM, double buffered
//   O += P V     (A = P K-major from shared memory, B = V MN-major) -> TMEM
// Q, K and V tiles arrive by per-CTA TMA (4-D tensor maps over [batch][token][head][d],
// so a packed qkv projection output is consumed in place; head sizes that are not a
// multiple of 64, e.g. 80, are zero-filled by the TMA bounds check instead of being
// padded in memory).  Warps 0-3 do the softmax (one query row per thread, read with
// tcgen05.ld), warp 4 issues TMA, warp 5 issues the MMAs.  With BN = 64 two CTAs fit
// on an SM, so one CTA's exponentials overlap the other's tensor-core work.
//
// Replaces the reference's flash-attention v2 forward, an sm_80 mma.sync kernel
// (reference: csrc/flash_attn/src/flash_fwd_kernel.h, flash_fwd_launch_template.h:13-28,
// dispatch mist/modules/flash_attn.py:46-213).
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128;
constexpr int kThreads = 192;
constexpr int kStages = 2;

struct AttnParams {
  __nv_bfloat16* o;
  float* lse;
  int sq, sk, nh, nh_kv, d, d_mma, nchunks;
  long o_batch_stride, o_tok_stride, o_head_stride;
  float scale_log2;
  int causal;
  // per-sample lengths of a right-padded batch (null: every sample has sq / sk tokens): queries and keys
  // at or past a sample's length are padding -- such keys are masked, such query rows come out as zeros
  const int* seqlens_q;
  const int* seqlens_k;
  int* status;
};

template <int BN>
struct Smem {
  // every tile is a stack of [rows][64 bf16] chunks, 128-byte swizzled
  static constexpr int kQ = 2 * BM * 128;           // up to 2 chunks
  static constexpr int kKV = 2 * BN * 128;          // one stage of K or V
  static constexpr int kP = (BN / 64) * BM * 128;
  static constexpr int oQ = 0;
  static constexpr int oK = oQ + kQ;
  static constexpr int oV = oK + kStages * kKV;
  static constexpr int oP = oV + kStages * kKV;
  static constexpr int oBar = oP + kP;
  // q_full, k_full[2], v_full[2], kv_empty[2], s_full[2], s_empty[2], p_full, pv_done, k_empty[2]
  static constexpr int kNumBars = 1 + 2 + 2 + 2 + 2 + 2 + 1 + 1 + 2;
  static constexpr int kTotal = oBar + kNumBars * 8 + 16;
};

__device__ __forceinline__ void report(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

template <int BN>
__global__ void __launch_bounds__(kThreads, (BN == 64 ? 2 : 1))
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using L = Smem<BN>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::oBar);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* v_full = bars + 3;
  uint64_t* kv_empty = bars + 5;
  uint64_t* s_full = bars + 7;
  uint64_t* s_empty = bars + 9;
  uint64_t* p_full = bars + 11;
  uint64_t* pv_done = bars + 12;
  uint64_t* k_empty = bars + 13;   // K stage free as soon as its S MMA has read it (V waits for PV)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heavy (late) query tiles first: under the causal mask they have the most blocks
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int head_kv = head / (p.nh / p.nh_kv);
  const int q0 = qt * BM;
  const int sq_b = p.seqlens_q ? min(p.sq, p.seqlens_q[batch]) : p.sq;   // real tokens of this sample
  const int sk_b = p.seqlens_k ? min(p.sk, p.seqlens_k[batch]) : p.sk;
  const int coff = sk_b - sq_b;  // causal: key j visible to query i when j <= i + coff

  int nblocks = (q0 < sq_b) ? (sk_b + BN - 1) / BN : 0;   // a tile of padding rows has nothing to attend to
  if (p.causal) {
    int last = q0 + BM - 1 + coff;  // last visible key of the tile's last row
    int nb = last < 0 ? 0 : last / BN + 1;
    nblocks = min(nblocks, nb);
  }

  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte base
    if (threadIdx.x == 0) report(p.status, MB_ERR_BAD_ARG);
    return;
  }

  constexpr int kTmemCols = (BN == 64) ? 256 : 512;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    fence_barrier_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;           // S0 at +0, S1 at +BN
  const uint32_t tmem_o = tmem_base + 2 * BN;  // O accumulator

  const uint32_t chunk_q = BM * 128, chunk_kv = BN * 128;

  if (warp == 4) {
    // ----------------------------------------------------------- TMA producer
    if (lane == 0 && nblocks > 0) {
      bool ok = true;
      mbar_expect_tx(q_full, p.nchunks * chunk_q);
      for (int c = 0; c < p.nchunks; ++c)
        tma_load_4d(smem + L::oQ + c * chunk_q, &tm_q, q_full, 64 * c, head, q0, batch);
      for (int j = 0; j < nblocks && ok; ++j) {
        int st = j % kStages;
        if (j >= kStages && !mbar_wait(&k_empty[st], ((j / kStages) - 1) & 1)) {
          report(p.status, MB_ERR_TIMEOUT_EMPTY);
          ok = false;
          break;
        }
        uint8_t* sk_ = smem + L::oK + st * L::kKV;
        uint8_t* sv_ = smem + L::oV + st * L::kKV;
        mbar_expect_tx(&k_full[st], p.nchunks * chunk_kv);
        for (int c = 0; c < p.nchunks; ++c)
          tma_load_4d(sk_ + c * chunk_kv, &tm_k, &k_full[st], 64 * c, head_kv, j * BN, batch);
        if (j >= kStages && !mbar_wait(&kv_empty[st], ((j / kStages) - 1) & 1)) {
          report(p.status, MB_ERR_TIMEOUT_EMPTY);
          ok = false;
          break;
        }
        mbar_expect_tx(&v_full[st], p.nchunks * chunk_kv);
        for (int c = 0; c < p.nchunks; ++c)
          tma_load_4d(sv_ + c * chunk_kv, &tm_v, &v_full[st], 64 * c, head_kv, j * BN, batch);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------- MMA issuer
    if (nblocks > 0) {
      const uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(BM, p.d_mma, 0, 1);
      const uint32_t sq_ = smem_u32(smem + L::oQ);
      const uint32_t sp_ = smem_u32(smem + L::oP);
      const int ksteps = p.d_mma / 16;
      bool ok = true;

      auto issue_s = [&](int j) -> bool {
        int st = j % kStages, b = j & 1;
        if (!mbar_wait(&k_full[st], (j / kStages) & 1)) return false;
        if (j >= 2 && !mbar_wait(&s_empty[b], ((j >> 1) - 1) & 1)) return false;
        tc_fence_after();
        if (lane == 0) {
          uint32_t sk_ = smem_u32(smem + L::oK + st * L::kKV);
          for (int kk = 0; kk < ksteps; ++kk) {
            uint32_t ch = kk >> 2, in = (kk & 3) * 32;
            uint64_t ad = make_smem_desc_sw128(sq_ + ch * chunk_q + in, 16, 1024);
            uint64_t bd = make_smem_desc_sw128(sk_ + ch * chunk_kv + in, 16, 1024);
            mma_f16_ss(tmem_s + b * BN, ad, bd, idesc_s, kk != 0 ? 1u : 0u);
          }
          mma_commit(&k_empty[st]);
          mma_commit(&s_full[b]);
        }
        __syncwarp();
        return true;
      };

      if (!mbar_wait(q_full, 0)) { report(p.status, MB_ERR_TIMEOUT_FULL); ok = false; }
      if (ok && !issue_s(0)) { report(p.status, MB_ERR_TIMEOUT_FULL); ok = false; }
      for (int j = 0; j < nblocks && ok; ++j) {
        if (j + 1 < nblocks && !issue_s(j + 1)) {
          report(p.status, MB_ERR_TIMEOUT_FULL);
          ok = false;
          break;
        }
        int st = j % kStages;
        if (!mbar_wait(p_full, j & 1) || !mbar_wait(&v_full[st], (j / kStages) & 1)) {
          report(p.status, MB_ERR_TIMEOUT_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          uint32_t sv_ = smem_u32(smem + L::oV + st * L::kKV);
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t ch = kk >> 2, in = (kk & 3) * 32;
            uint64_t ad = make_smem_desc_sw128(sp_ + ch * chunk_q + in, 16, 1024);
            // V: [kv rows][64-wide d atoms]; 16 kv rows = 2048 B, next d atom = chunk_kv
            uint64_t bd = make_smem_desc_sw128(sv_ + kk * 2048, chunk_kv, 1024);
            mma_f16_ss(tmem_o, ad, bd, idesc_o, (j | kk) != 0 ? 1u : 0u);
          }
          mma_commit(&kv_empty[st]);
          mma_commit(pv_done);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax
    const int r = threadIdx.x;  // row of the tile == TMEM lane
    const int qi = q0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    uint8_t* sp_ = smem + L::oP;

    for (int j = 0; j < nblocks && ok; ++j) {
      const int b = j & 1;
      if (!mbar_wait(&s_full[b], (j >> 1) & 1)) {
        report(p.status, MB_ERR_TIMEOUT_TMEM);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sr[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) tmem_ld32(tmem_s + b * BN + c * 32 + lane_off, sr + 32 * c);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_empty[b]);

      const int kv0 = j * BN;
      const int vis = p.causal ? min(sk_b - 1, qi + coff) : sk_b - 1;  // last visible key
      // Only tiles that touch the diagonal or the end of the keys need the mask; the test is the
      // same for every thread of the CTA (first row of the tile has the smallest horizon).
      const int vis_tile = p.causal ? min(sk_b - 1, q0 + coff) : sk_b - 1;
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      if (kv0 + BN - 1 > vis_tile) {
#pragma unroll
        for (int i = 0; i < BN; i += 4) {
          float v0 = (kv0 + i <= vis) ? __uint_as_float(sr[i]) : -INFINITY;
          float v1 = (kv0 + i + 1 <= vis) ? __uint_as_float(sr[i + 1]) : -INFINITY;
          float v2 = (kv0 + i + 2 <= vis) ? __uint_as_float(sr[i + 2]) : -INFINITY;
          float v3 = (kv0 + i + 3 <= vis) ? __uint_as_float(sr[i + 3]) : -INFINITY;
          sr[i] = __float_as_uint(v0); sr[i + 1] = __float_as_uint(v1);
          sr[i + 2] = __float_as_uint(v2); sr[i + 3] = __float_as_uint(v3);
          mx0 = fmaxf(mx0, v0); mx1 = fmaxf(mx1, v1); mx2 = fmaxf(mx2, v2); mx3 = fmaxf(mx3, v3);
        }
      } else {
#pragma unroll
        for (int i = 0; i < BN; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(sr[i]));
          mx1 = fmaxf(mx1, __uint_as_float(sr[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(sr[i + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(sr[i + 3]));
        }
      }
      // raw scores; the softmax scale (> 0, so maxima commute with it) is folded into the FFMA below
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      // Lazy rescaling: keep the old reference maximum unless the new one is much
      // larger; probabilities then stay below 2^8, harmless in fp32 / bf16.
      const float m_new = fmaxf(m_run, mx);
      const float m_use = (m_new - m_run > 8.f || m_run == -INFINITY) ? m_new : m_run;
      const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_use);
      const float m_neg = (m_use == -INFINITY) ? 0.f : -m_use;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pk[BN / 2];
#pragma unroll
      for (int i = 0; i < BN; i += 2) {
        const float xa = fmaf(__uint_as_float(sr[i]), p.scale_log2, m_neg);
        const float xc = fmaf(__uint_as_float(sr[i + 1]), p.scale_log2, m_neg);
        const float a = mb::fast_exp2(xa);
        const float c = mb::fast_exp2(xc);
        sum0 += a;
        sum1 += c;
        pk[i >> 1] = pack_bf16x2(a, c);
      }
      const float sum = sum0 + sum1;
      l_run = l_run * alpha + sum;
      m_run = m_use;

      if (j > 0) {
        if (!mbar_wait(pv_done, (j - 1) & 1)) {
          report(p.status, MB_ERR_TIMEOUT_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
      }
      // P tile -> shared memory in the swizzled K-major layout the MMA reads
#pragma unroll
      for (int g = 0; g < BN / 8; ++g) {
        uint32_t ch = g >> 3, gg = g & 7;
        uint4 val = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
        *reinterpret_cast<uint4*>(sp_ + ch * chunk_q + r * 128 + ((gg ^ (r & 7)) << 4)) = val;
      }
      // Rescale the running output when this warp's reference maxima moved.
      const bool need = (j > 0) && (alpha != 1.f);
      if (__any_sync(0xffffffffu, need)) {
        for (int c = 0; c < p.d_mma / 16; ++c) {
          uint32_t o[16];
          tmem_ld16(tmem_o + c * 16 + lane_off, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st16(tmem_o + c * 16 + lane_off, o);
        }
        tmem_st_wait();
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }

    if (ok && nblocks > 0) {
      if (!mbar_wait(pv_done, (nblocks - 1) & 1)) {
        report(p.status, MB_ERR_TIMEOUT_TMEM);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after();
      const bool real_row = qi < sq_b;
      const float inv = (real_row && l_run > 0.f) ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.o + batch * p.o_batch_stride + static_cast<long>(qi) * p.o_tok_stride +
                            static_cast<long>(head) * p.o_head_stride;
      for (int c = 0; c < p.d_mma / 16; ++c) {
        uint32_t o[16];
        if (nblocks > 0) {
          tmem_ld16(tmem_o + c * 16 + lane_off, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = 0;
        }
        if (qi < p.sq && c * 16 < p.d) {
          float f[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(o[i]) * inv;
          *reinterpret_cast<mb::bf16x8*>(orow + c * 16) = mb::pack8(f);
          *reinterpret_cast<mb::bf16x8*>(orow + c * 16 + 8) = mb::pack8(f + 8);
        }
      }
      if (qi < p.sq)
        p.lse[(static_cast<long>(batch) * p.nh + head) * p.sq + qi] =
            (real_row && l_run > 0.f) ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
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
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) !=
            cudaSuccess || q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// [batch][tokens][heads][d] bf16 with element strides; box = [1][rows][1][64].
bool make_map(CUtensorMap* m, const void* base, int batch, int tokens, int heads, int d,
              long batch_stride, long tok_stride, long head_stride, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(head_stride) * 2,
                           static_cast<cuuint64_t>(tok_stride) * 2,
                           static_cast<cuuint64_t>(batch_stride) * 2};
  cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_with_context([&] {
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

}  // namespace

MB_API int* mb_status_device_ptr();

// q: [batch][sq][nh][d], k/v: [batch][sk][nh_kv][d], element strides given per tensor
// (so views into a packed qkv buffer work).  o: [batch][sq][nh][d] with its own strides.
// lse: [batch][nh][sq] fp32.  Head size d: multiple of 16, <= 128; all strides
// multiples of 8 elements and base pointers 16-byte aligned.  seqlens_q / seqlens_k: optional device
// arrays of `batch` ints, the number of real tokens of each sample of a right-padded batch (what the
// reference handles by removing the padding and calling its variable-length kernels,
// csrc/flash_attn/flash_api.cpp:427); padded query rows get zeros and lse = -inf.
MB_API int mb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch,
                       int sq, int sk, int nh, int nh_kv, int d, long q_bs, long q_ts, long q_hs,
                       long k_bs, long k_ts, long k_hs, long v_bs, long v_ts, long v_hs, long o_bs,
                       long o_ts, long o_hs, float scale, int causal, int block_n, const int* seqlens_q,
                       const int* seqlens_k, cudaStream_t stream) {
  if (d % 16 || d > 128 || d < 16 || nh % nh_kv) return -1;
  if ((q_ts | q_hs | q_bs | k_ts | k_hs | k_bs | v_ts | v_hs | v_bs | o_ts | o_hs | o_bs) & 7) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
       reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(o)) & 15)
    return -1;
  if (batch == 0 || sq == 0) return 0;
  const int bn = (block_n == 128) ? 128 : 64;
  CUtensorMap tq, tk, tv;
  if (!make_map(&tq, q, batch, sq, nh, d, q_bs, q_ts, q_hs, BM)) return -2;
  if (!make_map(&tk, k, batch, sk, nh_kv, d, k_bs, k_ts, k_hs, bn)) return -2;
  if (!make_map(&tv, v, batch, sk, nh_kv, d, v_bs, v_ts, v_hs, bn)) return -2;
  AttnParams p;
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.sq = sq; p.sk = sk; p.nh = nh; p.nh_kv = nh_kv; p.d = d;
  p.d_mma = d;
  p.nchunks = (d + 63) / 64;
  p.o_batch_stride = o_bs; p.o_tok_stride = o_ts; p.o_head_stride = o_hs;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.seqlens_q = seqlens_q;
  p.seqlens_k = seqlens_k;
  p.status = mb_status_device_ptr();
  dim3 grid((sq + BM - 1) / BM, nh, batch);
#define MB_ATTN_LAUNCH(BN_)                                                                        \
  do {                                                                                             \
    auto kern = attn_fwd_kernel<BN_>;                                                              \
    static bool cfg = false;                                                                       \
    if (!cfg) {                                                                                    \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                               Smem<BN_>::kTotal) != cudaSuccess) return -3;                       \
      cfg = true;                                                                                  \
    }                                                                                              \
    kern<<<grid, kThreads, Smem<BN_>::kTotal, stream>>>(tq, tk, tv, p);                            \
  } while (0)
  if (bn == 64) MB_ATTN_LAUNCH(64);
  else MB_ATTN_LAUNCH(128);
#undef MB_ATTN_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
