// bf16 GEMM on CTA pairs: two CTAs on neighbouring SMs compute one 256 x 256 output tile with
// `tcgen05.mma.cta_group::2`.  Each CTA stages 128 rows of A and 128 rows of B per k-block
// (32 KB instead of the 48 KB a lone CTA needs for a 128 x 256 tile), so the shared-memory
// read traffic per MMA drops by a third and six stages fit.  The leader CTA issues the MMAs;
// each CTA keeps its 128 x 256 half of the accumulator in its own TMEM and runs its own
// epilogue (TMEM -> registers -> swizzled staging tile -> TMA store / reduce-add).
//
//   C[M,N] (op)= A[M,K] * B[N,K]^T, operands K-major or MN-major as in the single-CTA kernel.
//
// Same role split per CTA (192 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA
// only), warps 2..5 epilogue; two accumulator stages in TMEM.  Loads are per-CTA TMA copies
// (never multicast) whose completion bytes are counted on the leader's barrier.
//
// Reference counterpart: the cuBLAS(Lt) calls of csrc/fused_dense_lib/fused_dense_cuda.cu:19-167.
#include "sm100_pair.cuh"
#include <string.h>
#include <stdio.h>

using namespace sm100;

namespace {

constexpr int BM = 128;       // rows per CTA (256 per pair)
constexpr int BN = 256;       // columns per pair; each CTA stages BN / 2 rows of B
constexpr int BNH = BN / 2;
constexpr int BK = 64;
// Six pipeline stages; the kernels whose epilogue reads a second operand (gelu' or residual) give one
// stage up for two staging tiles that TMA fills with that operand ahead of the epilogue.
constexpr int kStagesPlain = 6;
constexpr int kStagesAux = 5;
constexpr int kThreads = 192;

enum EpiFlags : int {
  EPI_BIAS = 1, EPI_GELU = 2, EPI_SAVE_PRE = 4, EPI_ACCUM = 8, EPI_DGELU = 16, EPI_OUT_FP32 = 32, EPI_RESIDUAL = 64
};

struct PairParams {
  int M, N, K;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux;   // DGELU: pre-activation, RESIDUAL: tensor to add; [M][N] bf16 with row stride ldc
  int ldc;
  int flags;
  float alpha;
  int* status;
};

template <bool AUX>
struct Layout {
  static constexpr int kStages = AUX ? kStagesAux : kStagesPlain;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BNH * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = BM * 128;
  static constexpr int kStagingOffset = kStages * kStageBytes;
  static constexpr int kAuxOffset = kStagingOffset + 2 * kStagingBytes;          // two tiles, AUX only
  static constexpr int kBarOffset = kAuxOffset + (AUX ? 2 * kStagingBytes : 0);
  // full[S], empty[S], tmem_full[2], tmem_empty[2], aux_full[2], tmem base word
  static constexpr int kTotal = kBarOffset + (2 * kStages + 6) * 8 + 16;
};

__device__ __forceinline__ void report(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

template <bool A_MN, bool B_MN, bool AUX>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_aux,
                 const PairParams p) {
  using L = Layout<AUX>;
  constexpr int STAGES = L::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // Both CTAs of the pair must use the same offsets: the dynamic segment starts at the same
  // shared-memory address in every CTA of a launch, so the same rounding applies.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* aux_full = tempty_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux_full + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader_cta = (rank == 0);
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int num_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr int GM = 4;  // 256-row tiles per raster group: neighbours share B panels in L2

  auto tile_coords = [&](int t, int& m0, int& n0) {
    int per_group = GM * num_n;
    int g = t / per_group;
    int first_m = g * GM;
    int gsz = min(num_m - first_m, GM);
    int r = t - g * per_group;
    m0 = (first_m + r % gsz) * (2 * BM) + static_cast<int>(rank) * BM;   // this CTA's rows
    n0 = (r / gsz) * BN;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);    // leader's: its own arrive.expect_tx covering both CTAs' bytes
      mbar_init(&empty_bar[s], 1);   // one MMA commit, broadcast to both CTAs
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);   // one MMA commit, broadcast to both CTAs
      mbar_init(&tempty_bar[a], 8);  // leader's: 4 epilogue warps of each CTA
      mbar_init(&aux_full[a], 1);    // second epilogue operand staged by TMA (AUX kernels)
    }
    fence_barrier_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_b);
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, 2 * BN);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t armed[STAGES];
      for (int s = 0; s < STAGES; ++s) armed[s] = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int m0, n0;
        tile_coords(t, m0, n0);
        const int nb0 = n0 + static_cast<int>(rank) * BNH;   // this CTA's rows of B
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            report(p.status, MB_ERR_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          if (leader_cta) {
            mbar_expect_tx(&full_bar[s], 2 * L::kStageBytes);
            armed[s]++;
          }
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
          if (!A_MN) {
            tma_load_2d_pair(sa, &tma_a, bar, kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tma_a, bar, m0 + 64 * j, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tma_b, bar, kb * BK, nb0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j)
              tma_load_2d_pair(sb + j * (BK * 128), &tma_b, bar, nb0 + 64 * j, kb * BK);
          }
        }
      }
      if (!ok && leader_cta) {
        for (int s = 0; s < STAGES; ++s)
          if (armed[s]) mbar_wait(&full_bar[s], (armed[s] - 1) & 1, 50);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------- MMA issuer (leader CTA only)
    if (leader_cta) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tcount) {
        int acc = tcount & 1;
        uint32_t acc_ph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1)) {
          report(p.status, MB_ERR_TIMEOUT_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph)) {
            report(p.status, MB_ERR_TIMEOUT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            uint32_t sa = smem_u32(smem + s * L::kStageBytes);
            uint32_t sb = sa + L::kABytes;
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              uint64_t ad = A_MN ? make_smem_desc_sw128(sa + k * 2048, BK * 128, 1024)
                                 : make_smem_desc_sw128(sa + k * 32, 16, 1024);
              uint64_t bd = B_MN ? make_smem_desc_sw128(sb + k * 2048, BK * 128, 1024)
                                 : make_smem_desc_sw128(sb + k * 32, 16, 1024);
              mma_f16_ss_pair(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            mma_commit_pair(&empty_bar[s]);   // frees the stage in both CTAs
          }
          __syncwarp();
        }
        if (ok && lane == 0) mma_commit_pair(&tfull_bar[acc]);
        __syncwarp();
      }
    }
  } else {
    // ----------------------------------------------------------- epilogue (both CTAs)
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const bool leader = (threadIdx.x == 64);
    const bool out_fp32 = (p.flags & EPI_OUT_FP32) != 0;
    const int cols_per_unit = out_fp32 ? 32 : 64;
    const int units = BN / cols_per_unit;
    const int npass = (p.flags & EPI_SAVE_PRE) ? 2 : 1;
    uint32_t tcount = 0, epi_units = 0, aux_units = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tcount) {
      int m0, n0;
      tile_coords(t, m0, n0);
      int acc = tcount & 1;
      uint32_t acc_ph = (tcount >> 1) & 1;
      if (AUX && leader && m0 < p.M) {
        // the first two operand tiles of this output tile travel while the main loop still runs
        const int live = min(units, (p.N - n0 + cols_per_unit - 1) / cols_per_unit);
        for (int u = 0; u < 2 && u < live; ++u) {
          const uint32_t au = aux_units + u;
          mbar_expect_tx(&aux_full[au & 1], L::kStagingBytes);
          tma_load_2d(smem + L::kAuxOffset + (au & 1) * L::kStagingBytes, &tma_aux, &aux_full[au & 1],
                      n0 + u * cols_per_unit, m0);
        }
      }
      if (!mbar_wait(&tfull_bar[acc], acc_ph)) {
        report(p.status, MB_ERR_TIMEOUT_TMEM);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const bool rows_live = m0 < p.M;   // the second CTA of a pair can hang over the bottom edge
      int units_live = 0;
      if (rows_live) units_live = min(units, (p.N - n0 + cols_per_unit - 1) / cols_per_unit);
      for (int u = 0; u < units && rows_live; ++u) {
        const int ucol0 = n0 + u * cols_per_unit;
        if (ucol0 >= p.N) break;
        if (AUX) {
          const uint32_t au = aux_units + u;
          if (!mbar_wait(&aux_full[au & 1], (au >> 1) & 1)) {
            report(p.status, MB_ERR_TIMEOUT_FULL);
            ok = false;
            break;
          }
        }
        for (int pass = 0; pass < npass; ++pass) {
          uint8_t* stg = smem + L::kStagingOffset + (epi_units & 1) * L::kStagingBytes;
          if (leader) tma_wait_read<1>();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int halves = out_fp32 ? 1 : 2;
          for (int hh = 0; hh < halves; ++hh) {
            uint32_t rr[32];
            tmem_ld32(taddr + u * cols_per_unit + hh * 32, rr);
            tmem_ld_wait();
            float v[32];
            const int col0 = ucol0 + hh * 32;
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rr[i]) * p.alpha;
            if (p.flags & EPI_BIAS) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] += __bfloat162float(p.bias[min(col0 + i, p.N - 1)]);
            }
            if (AUX) {
              // second operand from the tile TMA staged for this unit (same swizzle as the output tile)
              const uint8_t* at = smem + L::kAuxOffset + ((aux_units + u) & 1) * L::kStagingBytes;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float f[8];
                mb::unpack8(*reinterpret_cast<const mb::bf16x8*>(at + r * 128 + (((hh * 4 + j) ^ (r & 7)) << 4)), f);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  if (p.flags & EPI_DGELU) v[8 * j + i] *= mb::gelu_tanh_grad(f[i]);
                  else v[8 * j + i] += f[i];
                }
              }
            }
            if ((p.flags & EPI_GELU) && (pass == npass - 1)) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = mb::gelu_tanh(v[i]);
            }
            if (out_fp32) {
#pragma unroll
              for (int g = 0; g < 8; ++g)
                *reinterpret_cast<float4*>(stg + r * 128 + ((g ^ (r & 7)) << 4)) =
                    make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
            } else {
#pragma unroll
              for (int g = 0; g < 4; ++g)
                *reinterpret_cast<mb::bf16x8*>(stg + r * 128 + (((hh * 4 + g) ^ (r & 7)) << 4)) = mb::pack8(v + 8 * g);
            }
          }
          fence_async_smem();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (AUX && leader && u + 2 < units_live) {
            // every thread has read this unit's operand tile: refill the buffer for the unit after next
            const uint32_t au = aux_units + u + 2;
            mbar_expect_tx(&aux_full[au & 1], L::kStagingBytes);
            tma_load_2d(smem + L::kAuxOffset + (au & 1) * L::kStagingBytes, &tma_aux, &aux_full[au & 1],
                        n0 + (u + 2) * cols_per_unit, m0);
          }
          if (leader) {
            const CUtensorMap* dst = (npass == 2 && pass == 0) ? &tma_aux : &tma_c;
            if ((p.flags & EPI_ACCUM) && out_fp32) {
              asm volatile(
                  "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];\n" ::
                      "l"(reinterpret_cast<uint64_t>(dst)),
                  "r"(smem_u32(stg)), "r"(ucol0), "r"(m0)
                  : "memory");
            } else {
              tma_store_2d(dst, stg, ucol0, m0);
            }
            tma_commit();
          }
          ++epi_units;
        }
      }
      aux_units += units_live;
      // accumulator stage read: tell the leader's MMA warp (one arrival per warp)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
    }
    if (leader) tma_wait_all<0>();
  }

  // Neither CTA may leave while the other can still read its shared memory, signal its
  // barriers or use the paired TMEM allocation.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * BN);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
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
bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
              uint32_t box_rows, bool fp32, bool promote) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * (fp32 ? 4u : 2u)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return encode_with_context([&] {
    return fn(m, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
            const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, promote ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

int g_sms = 0;

template <bool A_MN, bool B_MN, bool AUX>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tx,
           const PairParams& p, int max_ctas, cudaStream_t stream) {
  constexpr int smem = Layout<AUX>::kTotal + 1024;
  static bool configured = false;
  auto kern = gemm_pair_kernel<A_MN, B_MN, AUX>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -3;
    configured = true;
  }
  int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN);
  int pairs = max_ctas / 2;
  if (pairs > tiles) pairs = tiles;
  if (pairs < 1) return -1;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, tx, p) == cudaSuccess ? 0 : -4;
}

template <bool AUX>
int dispatch(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
             const CUtensorMap& tx, const PairParams& p, int max_ctas, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch<false, false, AUX>(ta, tb, tc, tx, p, max_ctas, stream);
  if (!a_mn && b_mn) return launch<false, true, AUX>(ta, tb, tc, tx, p, max_ctas, stream);
  if (a_mn && !b_mn) return launch<true, false, AUX>(ta, tb, tc, tx, p, max_ctas, stream);
  return launch<true, true, AUX>(ta, tb, tc, tx, p, max_ctas, stream);
}

}  // namespace

MB_API int* mb_status_device_ptr();

// Same contract as mb_gemm_bf16 for the epilogues the TMA-store path covers (bias, GELU with
// optional pre-activation copy, bf16 or fp32 output, fp32 accumulation, and for bf16 output
// multiplication by gelu'(aux) or addition of aux).  Returns 1 without
// launching when the arguments need the single-CTA kernel (other epilogue flags, unaligned C,
// fewer than two 256 x 256 tiles); the caller then uses mb_gemm_bf16.
static char g_pair_err[256] = "";
// Arguments of the last mb_gemm_pair_bf16 call that got as far as building its tensor maps.
MB_API const char* mb_gemm_pair_last_error(void) { return g_pair_err; }

MB_API int mb_gemm_pair_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                             int a_mn_major, int b_mn_major, int flags, const void* bias, void* aux, float alpha,
                             int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -1;
  const bool out_fp32 = (flags & EPI_OUT_FP32) != 0;
  const int esz = out_fp32 ? 4 : 2;
  const int ok_flags = EPI_BIAS | EPI_GELU | EPI_SAVE_PRE | EPI_OUT_FP32 | (out_fp32 ? EPI_ACCUM : 0) |
                       (out_fp32 ? 0 : (EPI_DGELU | EPI_RESIDUAL));
  if ((flags & ~ok_flags) || (reinterpret_cast<uintptr_t>(C) & 15) || ((static_cast<long>(ldc) * esz) % 16) ||
      ((flags & EPI_GELU) && out_fp32))
    return 1;
  if ((flags & EPI_SAVE_PRE) && (!aux || (reinterpret_cast<uintptr_t>(aux) & 15) || !(flags & EPI_GELU))) return 1;
  if (flags & (EPI_DGELU | EPI_RESIDUAL)) {
    // one second operand only, read with 16-byte loads at row stride ldc
    if (!aux || (reinterpret_cast<uintptr_t>(aux) & 15) || (ldc & 7) || (flags & (EPI_GELU | EPI_SAVE_PRE)) ||
        ((flags & EPI_DGELU) && (flags & EPI_RESIDUAL)))
      return 1;
  }
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (max_ctas <= 0 || max_ctas > g_sms) max_ctas = g_sms;
  const long tiles = static_cast<long>((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  if (tiles < max_ctas / 2) return 1;     // cannot fill the machine with 256 x 256 tiles
  CUtensorMap ta, tb, tc, tx;
  memset(&tx, 0, sizeof(tx));
  // a tensor map that cannot be encoded: -21 (A), -22 (B), -23 (C), -24 (second epilogue operand); the arguments
  // of the refused call can be read back with mb_gemm_pair_last_error
  snprintf(g_pair_err, sizeof(g_pair_err), "A=%p B=%p C=%p aux=%p M=%d N=%d K=%d lda=%d ldb=%d ldc=%d a_mn=%d b_mn=%d flags=%d",
           A, B, C, aux, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, flags);
  if (!(a_mn_major ? make_map(&ta, A, K, M, lda, 64, BK, false, true) : make_map(&ta, A, M, K, lda, 64, BM, false, true)))
    return -21;
  if (!(b_mn_major ? make_map(&tb, B, K, N, ldb, 64, BK, false, true) : make_map(&tb, B, N, K, ldb, 64, BNH, false, true)))
    return -22;
  if (!make_map(&tc, C, M, N, ldc, out_fp32 ? 32 : 64, BM, out_fp32, false)) return -23;
  const bool has_aux = (flags & (EPI_DGELU | EPI_RESIDUAL)) != 0;
  if (((flags & EPI_SAVE_PRE) || has_aux) && !make_map(&tx, aux, M, N, ldc, 64, BM, false, false)) return -24;
  PairParams p;
  p.M = M; p.N = N; p.K = K;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.aux = reinterpret_cast<const __nv_bfloat16*>(aux);
  p.ldc = ldc;
  p.flags = flags;
  p.alpha = alpha;
  p.status = mb_status_device_ptr();
  if (has_aux) return dispatch<true>(a_mn_major != 0, b_mn_major != 0, ta, tb, tc, tx, p, max_ctas, stream);
  return dispatch<false>(a_mn_major != 0, b_mn_major != 0, ta, tb, tc, tx, p, max_ctas, stream);
}
