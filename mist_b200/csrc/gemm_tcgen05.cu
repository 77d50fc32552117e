// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM),
// operands staged by per-CTA TMA, persistent warp-specialised CTAs.
//
//   C[M,N] (op)= A[M,K] * B[N,K]^T         with either operand K-major or MN-major,
//
// which covers the three GEMMs of a linear layer without any transposed copy:
//   forward  y  = x  W^T     A = x  (K-major)          B = W  (K-major)
//   dgrad    dx = dy W       A = dy (K-major)          B = W  (MN-major, stored [red][out])
//   wgrad    dW = dy^T x     A = dy (MN-major)         B = x  (MN-major)
//
// This replaces the cuBLAS / cuBLASLt calls behind the reference's fused dense
// layer (reference: csrc/fused_dense_lib/fused_dense_cuda.cu:19-92 gemm_bias,
// :137-167 epilogue selection; mist/modules/fused_dense.py:75,122,145).
//
// CTA layout (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer,
// warps 2..5 = epilogue (TMEM -> registers -> global).  Two accumulator stages in
// TMEM let the epilogue of tile i overlap the main loop of tile i+1.
#include "sm100.cuh"
#include <string.h>

using namespace sm100;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kThreads = 192;

enum EpiFlags : int {
  EPI_BIAS = 1,         // + bias[n]
  EPI_GELU = 2,         // gelu_tanh(.)
  EPI_SAVE_PRE = 4,     // store the pre-activation to aux (bf16, same ld as C)
  EPI_ACCUM = 8,        // C += result
  EPI_DGELU = 16,       // result *= gelu'(aux[m,n])
  EPI_OUT_FP32 = 32,    // C is fp32 (else bf16)
  EPI_RESIDUAL = 64,    // + aux[m,n] (bf16 residual stream, same ld as C)
};

struct GemmParams {
  int M, N, K;
  void* C;
  int ldc;
  const __nv_bfloat16* bias;
  __nv_bfloat16* aux;
  int flags;
  float alpha;
  int* status;
  int tma_epilogue;  // 1: stage tiles in shared memory and write them with TMA stores
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = BM * 128;  // one [128 rows][128 bytes] swizzled tile
  static constexpr int kStagingOffset = STAGES * kStageBytes;
  static constexpr int kBarOffset = kStagingOffset + 2 * kStagingBytes;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem base word
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 4) * 8 + 16;
};

__device__ __forceinline__ void report(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_aux,
                 const GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // Dynamic shared memory is only guaranteed 16-byte aligned; the swizzle needs 1024.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr int GM = 8;  // m-tiles per raster group: neighbours share B panels in L2

  auto tile_coords = [&](int t, int& m0, int& n0) {
    int per_group = GM * num_n;
    int g = t / per_group;
    int first_m = g * GM;
    int gsz = min(num_m - first_m, GM);
    int r = t - g * per_group;
    m0 = (first_m + r % gsz) * BM;
    n0 = (r / gsz) * BN;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 128);
    }
    fence_barrier_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_b);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;  // global k-block counter -> stage / phase
      uint32_t armed[STAGES];
      for (int s = 0; s < STAGES; ++s) armed[s] = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m0, n0;
        tile_coords(t, m0, n0);
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
          mbar_expect_tx(&full_bar[s], L::kStageBytes);
          armed[s]++;
          if (!A_MN) {
            tma_load_2d(sa, &tma_a, &full_bar[s], kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &tma_a, &full_bar[s], m0 + 64 * j, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tma_b, &full_bar[s], kb * BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &tma_b, &full_bar[s], n0 + 64 * j, kb * BK);
          }
        }
      }
      if (!ok) {
        // Gave up: let the copies already in flight land before the CTA exits.
        for (int s = 0; s < STAGES; ++s)
          if (armed[s]) mbar_wait(&full_bar[s], (armed[s] - 1) & 1, 50);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
    uint32_t it = 0;
    uint32_t tcount = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tcount) {
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
            mma_f16_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          mma_commit(&empty_bar[s]);  // stage is free once these MMAs have read it
        }
        __syncwarp();
      }
      if (ok && lane == 0) mma_commit(&tfull_bar[acc]);
      __syncwarp();
    }
  } else {
    // --------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t tcount = 0;
    bool ok = true;
    const bool out_fp32 = (p.flags & EPI_OUT_FP32) != 0;
    uint32_t epi_units = 0;  // staging tiles handed to TMA so far (selects the buffer)
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tcount) {
      int m0, n0;
      tile_coords(t, m0, n0);
      int acc = tcount & 1;
      uint32_t acc_ph = (tcount >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_ph)) {
        report(p.status, MB_ERR_TIMEOUT_TMEM);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (p.tma_epilogue) {
        // Coalesced path: each thread writes its row's 128 bytes into a swizzled staging
        // tile, one elected thread hands the tile to TMA (store, or reduce-add for
        // accumulation into an fp32 gradient bucket).  Two staging tiles alternate.
        const int r = q * 32 + lane;
        const bool leader = (threadIdx.x == 64);
        const int cols_per_unit = out_fp32 ? 32 : 64;
        const int units = BN / cols_per_unit;
        const int npass = (p.flags & EPI_SAVE_PRE) ? 2 : 1;
        for (int u = 0; u < units; ++u) {
          const int ucol0 = n0 + u * cols_per_unit;
          if (ucol0 >= p.N) break;  // uniform over the CTA: nothing to store further right
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
                for (int i = 0; i < 32; ++i)
                  v[i] += __bfloat162float(p.bias[min(col0 + i, p.N - 1)]);
              }
              const bool act = (p.flags & EPI_GELU) && (pass == npass - 1);
              if (act) {
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
                  *reinterpret_cast<mb::bf16x8*>(stg + r * 128 + (((hh * 4 + g) ^ (r & 7)) << 4)) =
                      mb::pack8(v + 8 * g);
              }
            }
            fence_async_smem();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (leader) {
              const CUtensorMap* dst = (npass == 2 && pass == 0) ? &tma_aux : &tma_c;
              if ((p.flags & EPI_ACCUM) && out_fp32) {
                asm volatile(
                    "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group "
                    "[%0, {%2, %3}], [%1];\n" ::"l"(reinterpret_cast<uint64_t>(dst)),
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
        tc_fence_before();
        mbar_arrive(&tempty_bar[acc]);
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
          const int ncols = min(32, p.N - col0);
          const size_t off = static_cast<size_t>(row) * p.ldc + col0;
          const bool vec_ok = (ncols == 32) && ((p.ldc & 7) == 0);
          if (p.flags & EPI_BIAS) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < ncols) v[i] += __bfloat162float(p.bias[col0 + i]);
          }
          if (p.flags & EPI_RESIDUAL) {
            if (vec_ok) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                mb::bf16x8 pk = *reinterpret_cast<const mb::bf16x8*>(p.aux + off + 8 * j);
                float f[8];
                mb::unpack8(pk, f);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[8 * j + i] += f[i];
              }
            } else {
              for (int i = 0; i < ncols; ++i) v[i] += __bfloat162float(p.aux[off + i]);
            }
          }
          if (p.flags & EPI_SAVE_PRE) {
            if (vec_ok) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                *reinterpret_cast<mb::bf16x8*>(p.aux + off + 8 * j) = mb::pack8(v + 8 * j);
            } else {
              for (int i = 0; i < ncols; ++i) p.aux[off + i] = __float2bfloat16(v[i]);
            }
          }
          if (p.flags & EPI_GELU) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = mb::gelu_tanh(v[i]);
          }
          if (p.flags & EPI_DGELU) {
            if (vec_ok) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                mb::bf16x8 pk = *reinterpret_cast<const mb::bf16x8*>(p.aux + off + 8 * j);
                float f[8];
                mb::unpack8(pk, f);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[8 * j + i] *= mb::gelu_tanh_grad(f[i]);
              }
            } else {
              for (int i = 0; i < ncols; ++i)
                v[i] *= mb::gelu_tanh_grad(__bfloat162float(p.aux[off + i]));
            }
          }
          if (out_fp32) {
            float* c_out = reinterpret_cast<float*>(p.C) + off;
            if (ncols == 32 && (p.ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                if (p.flags & EPI_ACCUM) {
                  float4 e = *reinterpret_cast<const float4*>(c_out + 4 * j);
                  o.x += e.x; o.y += e.y; o.z += e.z; o.w += e.w;
                }
                *reinterpret_cast<float4*>(c_out + 4 * j) = o;
              }
            } else {
              for (int i = 0; i < ncols; ++i)
                c_out[i] = (p.flags & EPI_ACCUM) ? c_out[i] + v[i] : v[i];
            }
          } else {
            __nv_bfloat16* c_out = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
            if (vec_ok) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (p.flags & EPI_ACCUM) {
                  mb::bf16x8 pk = *reinterpret_cast<const mb::bf16x8*>(c_out + 8 * j);
                  float f[8];
                  mb::unpack8(pk, f);
#pragma unroll
                  for (int i = 0; i < 8; ++i) v[8 * j + i] += f[i];
                }
                *reinterpret_cast<mb::bf16x8*>(c_out + 8 * j) = mb::pack8(v + 8 * j);
              }
            } else {
              for (int i = 0; i < ncols; ++i) {
                float o = v[i];
                if (p.flags & EPI_ACCUM) o += __bfloat162float(c_out[i]);
                c_out[i] = __float2bfloat16(o);
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tempty_bar[acc]);
    }
    if (p.tma_epilogue && threadIdx.x == 64) tma_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) !=
            cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows][cols] matrix with row stride `ld`
// elements; box = [box_rows][64 cols], 128-byte swizzle.
bool make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                    uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return encode_with_context([&] {
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

// Output tile map: [rows][cols] of bf16 (64-column box) or fp32 (32-column box), i.e. 128-byte
// swizzled rows matching the epilogue's staging tile.
bool make_tmap_out(CUtensorMap* map, void* base, uint64_t rows, uint64_t cols, uint64_t ld, bool fp32) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * (fp32 ? 4u : 2u)};
  cuuint32_t box[2] = {fp32 ? 32u : 64u, static_cast<cuuint32_t>(BM)};
  cuuint32_t estr[2] = {1, 1};
  return encode_with_context([&] {
    return fn(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base,
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

int g_num_sms = 0;

template <int BN, int STAGES, bool A_MN, bool B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tx,
           const GemmParams& p, int max_ctas, cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  constexpr int smem = L::kTotal + 1024;
  static bool configured = false;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -3;
    configured = true;
  }
  int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  int grid = num_tiles < max_ctas ? num_tiles : max_ctas;
  kern<<<grid, kThreads, smem, stream>>>(ta, tb, tc, tx, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace

// Device word that kernels of this library set when a bounded wait gives up.
__device__ int g_mb_status = 0;

MB_API int mb_status_read_and_clear() {
  int h = 0;
  if (cudaMemcpyFromSymbol(&h, g_mb_status, sizeof(int)) != cudaSuccess) return -1;
  if (h != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_mb_status, &z, sizeof(int));
  }
  return h;
}

MB_API int* mb_status_device_ptr() {
  static int* p = nullptr;  // one process drives one device
  if (!p && cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_mb_status) != cudaSuccess)
    return nullptr;
  return p;
}

// A: K-major -> [M][K] row stride lda;  MN-major -> [K][M] row stride lda.
// B: K-major -> [N][K] row stride ldb;  MN-major -> [K][N] row stride ldb.
// Requirements: pointers 16-byte aligned, lda/ldb multiples of 8 elements.
// `max_ctas` <= 0 means one CTA per SM; a smaller value leaves SMs free for a
// concurrent communication kernel.
MB_API int mb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda,
                        int ldb, int ldc, int a_mn_major, int b_mn_major, int flags,
                        const void* bias, void* aux, float alpha, int tile_n, int max_ctas,
                        cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -1;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (max_ctas <= 0 || max_ctas > g_num_sms) max_ctas = g_num_sms;
  int bn = tile_n;
  if (bn != 128 && bn != 256) {
    // Wide tiles have the better smem-read / MMA ratio; fall back to the narrow
    // tile when the wide one cannot fill the machine.
    long tiles256 = static_cast<long>((M + BM - 1) / BM) * ((N + 255) / 256);
    bn = (tiles256 >= max_ctas) ? 256 : 128;
  }
  CUtensorMap ta, tb;
  bool ok;
  if (!a_mn_major) ok = make_tmap_bf16(&ta, A, M, K, lda, BM);
  else ok = make_tmap_bf16(&ta, A, K, M, lda, BK);
  if (!ok) return -2;
  if (!b_mn_major) ok = make_tmap_bf16(&tb, B, N, K, ldb, bn);
  else ok = make_tmap_bf16(&tb, B, K, N, ldb, BK);
  if (!ok) return -2;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.aux = reinterpret_cast<__nv_bfloat16*>(aux);
  p.flags = flags;
  p.alpha = alpha;
  p.status = mb_status_device_ptr();
  // The TMA epilogue covers the hot epilogues; anything else takes the direct-store path.
  const bool out_fp32 = (flags & EPI_OUT_FP32) != 0;
  const int esz = out_fp32 ? 4 : 2;
  const int fast_ok_flags = EPI_BIAS | EPI_GELU | EPI_SAVE_PRE | EPI_OUT_FP32 | (out_fp32 ? EPI_ACCUM : 0);
  bool fast = ((flags & ~fast_ok_flags) == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0) &&
              ((static_cast<long>(ldc) * esz) % 16 == 0) && !((flags & EPI_GELU) && out_fp32);
  if ((flags & EPI_SAVE_PRE) &&
      (!aux || (reinterpret_cast<uintptr_t>(aux) & 15) || !(flags & EPI_GELU)))
    fast = false;
  CUtensorMap tc, tx;
  memset(&tc, 0, sizeof(tc));
  memset(&tx, 0, sizeof(tx));
  if (fast) {
    if (!make_tmap_out(&tc, C, M, N, ldc, out_fp32)) fast = false;
    if (fast && (flags & EPI_SAVE_PRE) && !make_tmap_out(&tx, aux, M, N, ldc, false)) fast = false;
  }
  p.tma_epilogue = fast ? 1 : 0;

#define MB_DISPATCH(BN_, ST_)                                                                \
  do {                                                                                       \
    if (!a_mn_major && !b_mn_major) return launch<BN_, ST_, false, false>(ta, tb, tc, tx, p, max_ctas, stream); \
    if (!a_mn_major && b_mn_major) return launch<BN_, ST_, false, true>(ta, tb, tc, tx, p, max_ctas, stream);   \
    if (a_mn_major && !b_mn_major) return launch<BN_, ST_, true, false>(ta, tb, tc, tx, p, max_ctas, stream);   \
    return launch<BN_, ST_, true, true>(ta, tb, tc, tx, p, max_ctas, stream);                        \
  } while (0)

  if (bn == 256) MB_DISPATCH(256, 4);
  MB_DISPATCH(128, 6);
#undef MB_DISPATCH
}
