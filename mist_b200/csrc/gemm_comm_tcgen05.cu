// Tensor-parallel GEMMs fused with their sequence-parallel collective, one kernel each.
//
//   mode AG -> GEMM   C = allgather(A_shard) * B^T
//       A lives in a symmetric [T][K] buffer; every rank has written its own rows.  Some
//       CTAs of the persistent grid ("gather CTAs", 8 to 64, chosen per launch from the bytes
//       to fetch and the FLOPs of the GEMM) pull the peers' row chunks over NVLink with bulk
//       async copies (peer global -> shared -> local global), sharing every chunk among them
//       (gather_plan.cuh), and publish a flag per chunk; the compute CTAs' TMA warp waits for
//       the flag that covers its tile before loading it, and visits the locally owned rows
//       first.  Each remote byte crosses NVLink once; afterwards the whole gathered A sits in
//       local memory for any other consumer.
//
//   mode GEMM -> RS   C_shard = reduce_scatter(A * B^T)
//       The epilogue sends every output tile to the rank that owns those rows as soon as the tile is
//       finished, so the transfer overlaps the main loop tile by tile.  Default form ("store"): the
//       tile goes, as bf16, into the slot that the owner keeps for this source rank (a TMA store,
//       through NVLink for remote owners); after the closing flag round (all stores landed) the
//       owner sums its R slots in rank order (mb_rs_sum), so the result does not depend on arrival
//       order for any number of ranks, and nothing has to be zeroed first.  The slots alternate
//       between two sets from launch to launch, which is what lets a rank start its next launch
//       while a peer is still summing the previous one.  Older form ("add"): TMA reduce-add into
//       one zeroed accumulator per owner, bracketed by an opening flag round as well.
//
//   mode weight-AG -> GEMM   C = A * W^T + bias, W inside a flat parameter buffer sharded over ranks
//       ZeRO-3 keeps 1/R of a block's flat bf16 parameters per rank.  Every rank holds its
//       shard at its place in a symmetric full-size buffer; the gather CTAs pull all remote
//       shards in pieces ("chunks", one flag each), from all peers at once and starting with
//       the pieces that hold the weight matrix of this GEMM, and the TMA warp of a compute CTA
//       waits for the chunks under its B tile.  When the kernel ends the whole block's parameters are local for
//       the block's other operators.
//
// All share the tcgen05 main loop of the plain GEMM (TMA-fed smem stages, accumulators in
// TMEM).  No TMA load is multicast; peer memory is only read by plain bulk copies and only
// written by TMA reduce / stores.  Waits on peers are bounded.
//
// Reference equivalents: all_gather + F.linear and F.linear + reduce_scatter in
// mist/modules/fused_dense.py:54-75 and :320-327 (NCCL + cuBLAS, overlapped at best with a
// weight cast), disabled in the reference's models (mist/model/transformer.py:477-479).
#include "sm100_pair.cuh"
#include "gather_plan.cuh"
#include <string.h>
#include <algorithm>

using namespace sm100;

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr int kMaxRanks = 8;
constexpr int kCopyBufs = 11;   // ring of 11 x 16 KB buffers in the 192 KB stage area of a gather CTA
constexpr int kCopyBytes = 16384;
// At most this many peer loads are outstanding; the other buffers of the ring hold data whose store to
// local memory is still running.  A buffer is loaded into again once the store that read it is among the
// completed ones: with kCopyLoads loads ahead at most kCopyBufs - 1 - kCopyLoads younger stores may still
// be pending then, so the wait before a load never drains the whole store queue.
constexpr int kCopyLoads = 6;
constexpr int kCopyStoresPending = kCopyBufs - 1 - kCopyLoads;
constexpr int kPublishLag = 6;              // a sub-chunk is counted once this many younger stores were issued
constexpr int kAgCounterOffset = 2048;      // AG: the chunk counters follow the chunk flags at this index

static_assert(kGatherRowsPerChunk == BM, "one gather flag per row block of a tile");
static_assert(kGatherSubBytes % kCopyBytes == 0, "sub-chunks are whole ring buffers");

enum Mode : int { MODE_AG = 1, MODE_RS = 2, MODE_AGW = 3 };

struct CommParams {
  int M, N, K;
  int mode;
  int nranks, me, epoch;
  int rows_per_rank;
  int n_gather;                         // gather CTAs at the end of the grid (AG mode)
  int acc_bf16;                         // RS: accumulators are bf16 (two ranks: order-independent sum)
  int rs_store;                         // RS: store bf16 tiles into per-source slots instead of reduce-add
  // AG: every rank's gathered-A buffer (row-major [M][K] bf16); weight-AG: every rank's flat buffer
  const uint8_t* a_peer[kMaxRanks];
  uint8_t* a_local;
  int* chunk_flags;                     // local: [nranks][chunks_per_rank]
  int* chunk_cnt;                       // local, same shape, zero between launches: finished sub-chunks per chunk
  // weight-AG: layout of the flat parameter buffer (bytes)
  unsigned long long shard_bytes, chunk_bytes, b_off, bias_off;
  int chunks_per_rank;
  int n_shift;                          // first column tile whose weights are local (tile order starts there)
  // plain output (AG mode): bf16 C with bias
  void* C;
  int ldc;
  const __nv_bfloat16* bias;
  // flags: [0..R) ready, [R..2R) done, [2R] counter  (same layout as the p2p kernels)
  int* flags[kMaxRanks];
  int* status;
  unsigned long long wait_ns;
};

// PAIR: two CTAs of a cluster share each 256 x 256 tile (tcgen05 cta_group::2): a CTA stages its own
// 128 rows of A and 128 of the 256 rows of B, so a stage is 32 KB and six fit where the single-CTA
// kernel has four of 48 KB.
template <bool PAIR>
struct Smem {
  static constexpr int kStages = PAIR ? 6 : 4;
  static constexpr int kBRows = PAIR ? BN / 2 : BN;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = kBRows * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingOffset = kStages * kStageBytes;
  static constexpr int kStagingBytes = BM * 128;
  static constexpr int kBarOffset = kStagingOffset + 2 * kStagingBytes;
  static constexpr int kNumBars = 2 * kStages + 4 + kCopyBufs;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
};

__device__ __forceinline__ void report(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}
__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(int* addr, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* addr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded poll of one flag (single thread).
__device__ bool wait_flag(const int* flag, int epoch, bool sys, unsigned long long limit_ns, int* status) {
  const unsigned long long t0 = global_ns();
  while ((sys ? ld_acquire_sys(flag) : ld_acquire_gpu(flag)) < epoch) {
    if (global_ns() - t0 > limit_ns) {
      report(status, MB_ERR_TIMEOUT_PEER);
      return false;
    }
    __nanosleep(100);
  }
  return true;
}

// peer global -> shared (completion on an mbarrier) and shared -> local global (bulk group)
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(gdst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

// Weight-AG: waits (single thread) for every remote chunk that overlaps bytes [lo, hi) of the flat buffer.
__device__ bool wait_range(const CommParams& p, unsigned long long lo, unsigned long long hi) {
  unsigned long long x = lo;
  while (x < hi) {
    const int r = static_cast<int>(x / p.shard_bytes);
    const unsigned long long base = static_cast<unsigned long long>(r) * p.shard_bytes;
    const int c = static_cast<int>((x - base) / p.chunk_bytes);
    if (r != p.me &&
        !wait_flag(p.chunk_flags + r * p.chunks_per_rank + c, p.epoch, false, p.wait_ns, p.status))
      return false;
    unsigned long long next = base + static_cast<unsigned long long>(c + 1) * p.chunk_bytes;
    if (next > base + p.shard_bytes) next = base + p.shard_bytes;
    x = next;
  }
  return true;
}

template <bool B_MN, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap acc0,
                 const __grid_constant__ CUtensorMap acc1, const __grid_constant__ CUtensorMap acc2,
                 const __grid_constant__ CUtensorMap acc3, const __grid_constant__ CUtensorMap acc4,
                 const __grid_constant__ CUtensorMap acc5, const __grid_constant__ CUtensorMap acc6,
                 const __grid_constant__ CUtensorMap acc7, const CommParams p) {
  using L = Smem<PAIR>;
  constexpr int STAGES = L::kStages;
  constexpr int TM = PAIR ? 2 * BM : BM;          // rows of an output tile (per CTA always BM)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* copy_bar = tempty_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(copy_bar + kCopyBufs);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int R = p.nranks;
  int* my_flags = p.flags[p.me];
  const bool gathers = (p.mode == MODE_AG) || (p.mode == MODE_AGW);
  const int n_compute = gridDim.x - (gathers ? p.n_gather : 0);   // CTAs; even when PAIR
  const bool is_gather = gathers && (static_cast<int>(blockIdx.x) >= n_compute);
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;            // CTA of the pair; 0 leads
  const bool leader_cta = (rank == 0);
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);   // tile loop index
  const int n_workers = PAIR ? (n_compute >> 1) : n_compute;

  const int num_m = (p.M + TM - 1) / TM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int m_tiles_per_rank = p.rows_per_rank / TM;
  const int ag_chunks_per_rank = p.rows_per_rank / BM;   // all-gather flags: one per 128-row block

  // Tile order: all column tiles of one row block; AG: row blocks starting with the locally owned ones
  // (their data is there at once); RS: row blocks of the owners in turn.
  auto tile_coords = [&](int t, int& m0, int& n0) {
    if (p.mode == MODE_AGW) {
      // all row tiles of one column tile, column tiles in the order their weights arrive
      int nt = t / num_m, mt = t - nt * num_m;
      m0 = mt * TM + static_cast<int>(rank) * BM;
      n0 = ((nt + p.n_shift) % num_n) * BN;
      return;
    }
    int mt = t / num_n, nt = t - mt * num_n;
    int mt_rot;
    if (p.mode == MODE_AG) {
      mt_rot = (mt + p.me * m_tiles_per_rank) % num_m;
    } else {
      // RS: consecutive row blocks go to different owners (the next rank first, this rank every R-th
      // time), so the tiles that cross NVLink are spread over the whole kernel instead of filling its
      // first (R - 1) / R and leaving the links idle afterwards
      const int owner = (mt % R + p.me + 1) % R;
      mt_rot = owner * m_tiles_per_rank + mt / R;
    }
    m0 = mt_rot * TM + static_cast<int>(rank) * BM;      // this CTA's rows
    n0 = nt * BN;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], PAIR ? 8 : 128);   // PAIR: one arrival per epilogue warp of both CTAs
    }
    for (int b = 0; b < kCopyBufs; ++b) mbar_init(&copy_bar[b], 1);
    fence_barrier_init();
  }
  if (warp == 2 && !is_gather) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, 2 * BN);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 2 * BN);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = is_gather ? 0u : *tmem_slot;

  // ---- phase A: announce that this rank's inputs (A rows / zeroed accumulator) are ready
  if (blockIdx.x == 0 && threadIdx.x < R && static_cast<int>(threadIdx.x) != p.me) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + p.me, p.epoch);
  }

  if (is_gather) {
    // ------------------------------------------------------------------ gather CTAs
    // The remote chunks are cut into sub-chunks dealt to the gather CTAs in fetch order (gather_plan.cuh), so
    // that every gather CTA works on the chunk that the GEMM needs next (a whole chunk on one CTA would arrive
    // only after ~100 us).  A CTA streams the 16 KB pieces of all its sub-chunks through one ring without draining
    // it in between, counts a finished sub-chunk on the chunk's counter once its stores have completed, and the
    // CTA that counts the last one publishes the chunk's flag.
    if (threadIdx.x == 0) {
      const int g = blockIdx.x - n_compute;
      uint8_t* bufs = smem;                                              // reuse the stage area
      bool ok = true;
      unsigned ready_mask = 0;
      GatherPlan plan;
      if (p.mode == MODE_AG)
        plan.init_activations(R, p.me, p.K, p.rows_per_rank);
      else
        plan.init_weights(R, p.me, p.shard_bytes, p.chunk_bytes,
                          p.b_off + static_cast<unsigned long long>(p.n_shift) * BN * p.K * 2);
      const int total_subs = plan.total_subs;
      struct Cursor {
        int q;
        int piece, pieces;
        bool live;
        GatherSeg s;
      };
      auto seek = [&](Cursor& c) {           // moves to this CTA's next sub-chunk that has bytes, from c.q on
        c.live = false;
        for (; c.q < total_subs; c.q += p.n_gather) {
          if (plan.segment(c.q, c.s)) {
            c.live = true;
            c.piece = 0;
            c.pieces = static_cast<int>((c.s.bytes + kCopyBytes - 1) / kCopyBytes);
            return;
          }
        }
      };
      Cursor ld, st;
      ld.q = st.q = g;
      seek(ld);
      seek(st);
      uint32_t issued = 0, stored = 0;
      // sub-chunks whose last store has been issued but not yet counted: (flag, expected, stores issued by then)
      constexpr int kFifo = 8;
      int f_flag[kFifo], f_expected[kFifo];
      uint32_t f_mark[kFifo];
      uint32_t f_head = 0, f_tail = 0;
      auto count_done = [&](int flag, int expected) {
        fence_proxy_async_all();
        __threadfence();
        const int old = atomicAdd(p.chunk_cnt + flag, 1);
        if (old == expected - 1) {
          p.chunk_cnt[flag] = 0;                    // for the next launch
          __threadfence();
          st_release_gpu(p.chunk_flags + flag, p.epoch);
        }
      };
      while (st.live && ok) {
        while (ld.live && issued - stored < kCopyLoads) {
          if (!(ready_mask >> ld.s.r & 1u)) {
            ok = wait_flag(my_flags + ld.s.r, p.epoch, true, p.wait_ns, p.status);
            if (!ok) break;
            ready_mask |= 1u << ld.s.r;
          }
          const uint32_t b = issued % kCopyBufs;
          if (issued >= kCopyBufs) tma_wait_read<kCopyStoresPending>();   // the store that last used this buffer has read it
          const uint32_t nb = min(static_cast<uint32_t>(kCopyBytes), ld.s.bytes - static_cast<uint32_t>(ld.piece) * kCopyBytes);
          mbar_expect_tx(&copy_bar[b], nb);
          bulk_load(bufs + b * kCopyBytes, p.a_peer[ld.s.r] + ld.s.off + static_cast<size_t>(ld.piece) * kCopyBytes, nb,
                    &copy_bar[b]);
          ++issued;
          if (++ld.piece == ld.pieces) {
            ld.q += p.n_gather;
            seek(ld);
          }
        }
        if (!ok) break;
        const uint32_t b = stored % kCopyBufs;
        if (!mbar_wait(&copy_bar[b], (stored / kCopyBufs) & 1)) {
          report(p.status, MB_ERR_TIMEOUT_FULL);
          ok = false;
          break;
        }
        const uint32_t nb = min(static_cast<uint32_t>(kCopyBytes), st.s.bytes - static_cast<uint32_t>(st.piece) * kCopyBytes);
        bulk_store(p.a_local + st.s.off + static_cast<size_t>(st.piece) * kCopyBytes, bufs + b * kCopyBytes, nb);
        tma_commit();
        ++stored;
        if (++st.piece == st.pieces) {
          f_flag[f_tail % kFifo] = st.s.flag;
          f_expected[f_tail % kFifo] = st.s.expected;
          f_mark[f_tail % kFifo] = stored;
          ++f_tail;
          st.q += p.n_gather;
          seek(st);
        }
        // stores complete in order: all but the kPublishLag youngest are done after this wait
        if (f_head != f_tail && stored - f_mark[f_head % kFifo] >= kPublishLag) {
          tma_wait_all<kPublishLag>();
          while (f_head != f_tail && stored - f_mark[f_head % kFifo] >= kPublishLag) {
            count_done(f_flag[f_head % kFifo], f_expected[f_head % kFifo]);
            ++f_head;
          }
        }
      }
      tma_wait_all<0>();
      if (ok) {
        for (; f_head != f_tail; ++f_head) count_done(f_flag[f_head % kFifo], f_expected[f_head % kFifo]);
      } else {
        // loads still in flight land in this CTA's shared memory: wait for them (bounded) before leaving
        for (; stored < issued; ++stored)
          if (!mbar_wait(&copy_bar[stored % kCopyBufs], (stored / kCopyBufs) & 1)) break;
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t armed[STAGES];
      for (int s = 0; s < STAGES; ++s) armed[s] = 0;
      bool ok = true;
      for (int t = worker; t < num_tiles && ok; t += n_workers) {
        int m0, n0;
        tile_coords(t, m0, n0);
        if (p.mode == MODE_AG) {
          const int owner = m0 / p.rows_per_rank;
          if (owner != p.me) {
            const int c = (m0 - owner * p.rows_per_rank) / BM;
            ok = wait_flag(p.chunk_flags + owner * ag_chunks_per_rank + c, p.epoch, false, p.wait_ns, p.status);
            if (!ok) break;
            fence_proxy_async_all();   // the chunk was written through the async proxy of another SM
          }
        } else if (p.mode == MODE_AGW) {
          const int nlo = PAIR ? n0 + static_cast<int>(rank) * (BN / 2) : n0;       // this CTA's rows of W
          const int nhi = min(PAIR ? nlo + BN / 2 : n0 + BN, p.N);
          const unsigned long long lo = p.b_off + static_cast<unsigned long long>(min(nlo, p.N)) * p.K * 2;
          const unsigned long long hi = p.b_off + static_cast<unsigned long long>(nhi) * p.K * 2;
          ok = wait_range(p, lo, hi);
          if (!ok) break;
          fence_proxy_async_all();
        }
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
          if (PAIR) {
            // both CTAs' bytes are counted on the leader's barrier; each CTA loads its own halves
            if (leader_cta) {
              mbar_expect_tx(&full_bar[s], 2 * L::kStageBytes);
              armed[s]++;
            }
            const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
            const int nb0 = n0 + static_cast<int>(rank) * (BN / 2);
            tma_load_2d_pair(sa, &tma_a, bar, kb * BK, m0);
            if (!B_MN) {
              tma_load_2d_pair(sb, &tma_b, bar, kb * BK, nb0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j) tma_load_2d_pair(sb + j * (BK * 128), &tma_b, bar, nb0 + 64 * j, kb * BK);
            }
          } else {
            mbar_expect_tx(&full_bar[s], L::kStageBytes);
            armed[s]++;
            tma_load_2d(sa, &tma_a, &full_bar[s], kb * BK, m0);
            if (!B_MN) {
              tma_load_2d(sb, &tma_b, &full_bar[s], kb * BK, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * (BK * 128), &tma_b, &full_bar[s], n0 + 64 * j, kb * BK);
            }
          }
        }
      }
      if (!ok)
        for (int s = 0; s < STAGES; ++s)
          if (armed[s]) mbar_wait(&full_bar[s], (armed[s] - 1) & 1, 50);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc = make_idesc_bf16(TM, BN, 0, B_MN ? 1 : 0);
    uint32_t it = 0, tcount = 0;
    bool ok = leader_cta;          // PAIR: only the leader CTA issues MMAs (for both CTAs' accumulators)
    for (int t = worker; t < num_tiles && ok; t += n_workers, ++tcount) {
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
        if (!mbar_wait(&full_bar[s], ph, (p.mode != MODE_RS) ? 4000u : kSpinLimit)) {
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
            uint64_t ad = make_smem_desc_sw128(sa + k * 32, 16, 1024);
            uint64_t bd = B_MN ? make_smem_desc_sw128(sb + k * 2048, BK * 128, 1024)
                               : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            if (PAIR) mma_f16_ss_pair(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
            else mma_f16_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (PAIR) mma_commit_pair(&empty_bar[s]);   // frees the stage in both CTAs
          else mma_commit(&empty_bar[s]);
        }
        __syncwarp();
      }
      if (ok && lane == 0) {
        if (PAIR) mma_commit_pair(&tfull_bar[acc]);
        else mma_commit(&tfull_bar[acc]);
      }
      __syncwarp();
    }
  } else {
    // --------------------------------------------------------------- epilogue
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const bool leader = (threadIdx.x == 64);
    uint32_t tcount = 0, epi_units = 0;
    bool ok = true;
    const bool rs = (p.mode == MODE_RS);
    __shared__ int peers_ok_s;
    if (rs && !p.rs_store) {
      // peers' accumulators are zeroed once their ready flag shows this epoch
      if (leader) {
        int okf = 1;
        for (int rr = 0; rr < R && okf; ++rr)
          if (rr != p.me) okf = wait_flag(my_flags + rr, p.epoch, true, p.wait_ns, p.status) ? 1 : 0;
        peers_ok_s = okf;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      ok = peers_ok_s != 0;
    }
    if (p.mode == MODE_AGW && p.bias) {
      // the bias vector is part of the flat buffer and may still be on its way
      if (leader) peers_ok_s = wait_range(p, p.bias_off, p.bias_off + static_cast<unsigned long long>(p.N) * 2) ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      ok = peers_ok_s != 0;
    }
    const CUtensorMap* acc_maps[kMaxRanks] = {&acc0, &acc1, &acc2, &acc3, &acc4, &acc5, &acc6, &acc7};
    for (int t = worker; t < num_tiles && ok; t += n_workers, ++tcount) {
      int m0, n0;
      tile_coords(t, m0, n0);
      int acc = tcount & 1;
      uint32_t acc_ph = (tcount >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, (p.mode != MODE_RS) ? 4000u : kSpinLimit)) {
        report(p.status, MB_ERR_TIMEOUT_TMEM);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const int owner = rs ? (m0 / p.rows_per_rank) : 0;
      const bool f32_units = rs && !p.acc_bf16 && !p.rs_store;
      const int cols_per_unit = f32_units ? 32 : 64;     // fp32 accumulator tiles vs bf16 tiles
      const int units = BN / cols_per_unit;
      for (int u = 0; u < units; ++u) {
        const int ucol0 = n0 + u * cols_per_unit;
        if (ucol0 >= p.N) break;
        uint8_t* stg = smem + L::kStagingOffset + (epi_units & 1) * L::kStagingBytes;
        if (leader) tma_wait_read<1>();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int halves = f32_units ? 1 : 2;
        for (int hh = 0; hh < halves; ++hh) {
          uint32_t rr[32];
          tmem_ld32(taddr + u * cols_per_unit + hh * 32, rr);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rr[i]);
          if (p.bias) {     // RS: only the rank that holds the row-parallel bias passes it, so it is counted once
            const int col0 = ucol0 + hh * 32;
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] += __bfloat162float(p.bias[min(col0 + i, p.N - 1)]);
          }
          if (f32_units) {
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
        if (leader) {
          if (rs && p.rs_store) {
            tma_store_2d(acc_maps[owner], stg, ucol0, m0 - owner * p.rows_per_rank);
          } else if (rs) {
            asm volatile(
                "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];\n" ::
                    "l"(reinterpret_cast<uint64_t>(acc_maps[owner])),
                "r"(smem_u32(stg)), "r"(ucol0), "r"(m0 - owner * p.rows_per_rank)
                : "memory");
          } else {
            tma_store_2d(&tma_c, stg, ucol0, m0);
          }
          tma_commit();
        }
        ++epi_units;
      }
      tc_fence_before();
      if (PAIR) {
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
      } else {
        mbar_arrive(&tempty_bar[acc]);
      }
    }
    if (leader) tma_wait_all<0>();
  }

  // ---- phase C: whole grid done -> tell the peers; the last CTA waits for theirs
  __threadfence_system();
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // neither CTA leaves while the other may still use its memory or barriers
  if (warp == 2 && !is_gather) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN);
    else tmem_dealloc(tmem_base, 2 * BN);
  }
  __shared__ int last_s;
  if (threadIdx.x == 0) {
    int prev = atomicAdd(my_flags + 2 * R, 1);
    last_s = (prev + 1 == static_cast<int>(gridDim.x) * p.epoch);
  }
  __syncthreads();
  if (last_s) {
    if (threadIdx.x < R && static_cast<int>(threadIdx.x) != p.me) {
      __threadfence_system();
      st_release_sys(p.flags[threadIdx.x] + R + p.me, p.epoch);
    }
    __syncthreads();
    if (threadIdx.x == 0)
      for (int rr = 0; rr < R; ++rr)
        if (rr != p.me && !wait_flag(my_flags + R + rr, p.epoch, true, p.wait_ns, p.status)) break;
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
              uint32_t box_rows, bool fp32) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * (fp32 ? 4u : 2u)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return encode_with_context([&] {
    return fn(m, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
            const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

int g_sms = 0;

int g_pair = 1;   // CTA pairs (cta_group::2) when the shape allows; mb_gemm_comm_set_pair switches it
int g_last_pair = 0;   // whether the most recent launch ran on pairs (tests ask)

template <bool B_MN, bool PAIR>
int launch_t(int grid, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
             const CUtensorMap* acc, const CommParams& p) {
  constexpr int smem = Smem<PAIR>::kTotal + 1024;
  static bool configured = false;
  auto kern = gemm_comm_kernel<B_MN, PAIR>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -3;
    configured = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, acc[0], acc[1], acc[2], acc[3], acc[4], acc[5], acc[6], acc[7],
                            p) == cudaSuccess ? 0 : -4;
}

int launch(bool b_mn, bool pair, int grid, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb,
           const CUtensorMap& tc, const CUtensorMap* acc, const CommParams& p) {
  g_last_pair = pair ? 1 : 0;
  if (pair) return b_mn ? launch_t<true, true>(grid, stream, ta, tb, tc, acc, p)
                        : launch_t<false, true>(grid, stream, ta, tb, tc, acc, p);
  return b_mn ? launch_t<true, false>(grid, stream, ta, tb, tc, acc, p)
              : launch_t<false, false>(grid, stream, ta, tb, tc, acc, p);
}

// Gather CTAs for a launch that brings `inbound` bytes over NVLink beside a GEMM of `flops`.  One gather CTA keeps
// 96 KB in flight and moved 13-15 GB/s in measurements; the link stops scaling near 520 GB/s; the GEMM slows down by
// the share of SMs that it gives up.  More CTAs are taken only for a clear gain.
int pick_gather_ctas(double inbound, double flops) {
  const int cand[] = {8, 16, 24, 32, 48, 64};
  double best = 1e30;
  int arg = 8;
  for (int n : cand) {
    const double t_gather = inbound / std::min(n * 14e9, 520e9);
    const double t_gemm = flops / 1.4e15 * g_sms / (g_sms - n);
    const double t = std::max(t_gather, t_gemm);
    if (t < best * 0.97) best = t, arg = n;
  }
  return arg;
}

// Grid for one launch: `n_gather` gather CTAs after the compute CTAs; with pairs both counts are even.
int plan_grid(bool pair, long tiles, int& n_gather) {
  if (pair) {
    n_gather = (n_gather + 1) & ~1;
    int compute = (g_sms - n_gather) & ~1;
    if (compute > 2 * tiles) compute = static_cast<int>(2 * tiles);
    return compute;
  }
  int compute = g_sms - n_gather;
  if (compute > tiles) compute = static_cast<int>(tiles);
  return compute;
}

}  // namespace

MB_API int* mb_status_device_ptr();

// mode 1 (AG -> GEMM): a_ptrs[r] = rank r's symmetric [M][K] bf16 buffer (own rows valid), C [M][N] bf16.
// mode 2 (GEMM -> RS): A = local [M][K]; C unused.  acc_bf16 = 2 (store form): acc_ptrs[r] = the bf16 slot
// [M/R][N] that rank r keeps for tiles from this rank (nothing to zero; sum the slots with mb_rs_sum after the
// launch).  acc_bf16 = 0 / 1 (add form): acc_ptrs[r] = rank r's fp32 / bf16 accumulator [M/R][N], zeroed by its
// owner before the launch.  B: [N][K] (b_mn = 0) or [K][N] (b_mn = 1).  chunk_flags: local int array
// of 4096 (AG only: flags [R][M/R/128] from 0, counters of the same shape from 2048; zero before the first launch).  flag_ptrs[r]: per-rank flag block (2R + 1 ints) reserved for this call site; `epoch`
// counts launches on it from 1.  M/R must be a multiple of 128, K of 8.
MB_API int mb_gemm_comm(int mode, void* const* a_ptrs, const void* A, const void* B, void* C, void* const* acc_ptrs,
                        void* const* flag_ptrs, int* chunk_flags, int M, int N, int K, int ldb, int ldc, int b_mn,
                        const void* bias, int nranks, int me, int epoch, int n_gather, int wait_ms, int acc_bf16,
                        cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxRanks || M % nranks) return -1;
  const int rows_per_rank = M / nranks;
  if (rows_per_rank % BM || (K & 7) || (ldb & 7)) return -1;
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CommParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.mode = mode;
  p.nranks = nranks; p.me = me; p.epoch = epoch;
  p.rows_per_rank = rows_per_rank;
  if (mode == MODE_AG && M / BM > kAgCounterOffset) return -1;
  p.n_gather = 0;
  if (mode == MODE_AG)
    p.n_gather = n_gather > 0 ? n_gather
                              : pick_gather_ctas(2.0 * (M - rows_per_rank) * static_cast<double>(K),
                                                 2.0 * M * static_cast<double>(N) * K);
  p.acc_bf16 = acc_bf16 ? 1 : 0;
  p.rs_store = (acc_bf16 == 2) ? 1 : 0;
  if (nranks == 1) p.n_gather = 0, p.mode = (mode == MODE_AG) ? MODE_AG : MODE_RS;
  p.chunk_flags = chunk_flags;
  p.chunk_cnt = chunk_flags ? chunk_flags + kAgCounterOffset : nullptr;
  p.C = C; p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.status = mb_status_device_ptr();
  p.wait_ns = static_cast<unsigned long long>(wait_ms > 0 ? wait_ms : 2000) * 1000000ull;
  for (int r = 0; r < nranks; ++r) {
    p.flags[r] = reinterpret_cast<int*>(flag_ptrs[r]);
    if (mode == MODE_AG) p.a_peer[r] = reinterpret_cast<const uint8_t*>(a_ptrs[r]);
  }
  const void* a_base = A;
  if (mode == MODE_AG) {
    p.a_local = reinterpret_cast<uint8_t*>(a_ptrs[me]);
    a_base = a_ptrs[me];
  }
  CUtensorMap ta, tb, tc, acc[kMaxRanks];
  memset(&tc, 0, sizeof(tc));
  memset(acc, 0, sizeof(acc));
  // pairs need whole 256-row tiles per rank and enough of them to occupy the machine
  const bool pair = g_pair && (rows_per_rank % (2 * BM) == 0) &&
                    (static_cast<long>(M / (2 * BM)) * ((N + BN - 1) / BN) >= (g_sms - p.n_gather) / 2);
  if (!make_map(&ta, a_base, M, K, K, 64, BM, false)) return -2;
  if (!b_mn) {
    if (!make_map(&tb, B, N, K, ldb, 64, pair ? BN / 2 : BN, false)) return -2;
  } else {
    if (!make_map(&tb, B, K, N, ldb, 64, BK, false)) return -2;
  }
  if (mode == MODE_AG) {
    if (!make_map(&tc, C, M, N, ldc, 64, BM, false)) return -2;
  } else {
    for (int r = 0; r < nranks; ++r)
      if (!make_map(&acc[r], acc_ptrs[r], rows_per_rank, N, N, acc_bf16 ? 64 : 32, BM, !acc_bf16)) return -2;
  }
  const long tiles = static_cast<long>((M + (pair ? 2 : 1) * BM - 1) / ((pair ? 2 : 1) * BM)) * ((N + BN - 1) / BN);
  const int compute = plan_grid(pair, tiles, p.n_gather);
  return launch(b_mn != 0, pair, compute + p.n_gather, stream, ta, tb, tc, acc, p);
}

// 1 (default): the fused kernels run on CTA pairs when the shape allows; 0: always single CTAs.
MB_API void mb_gemm_comm_set_pair(int on) { g_pair = on ? 1 : 0; }
MB_API int mb_gemm_comm_last_pair(void) { return g_last_pair; }

// Weight all-gather fused into the GEMM that consumes the first weights of a ZeRO-3 block.
//   w_ptrs[r]: rank r's symmetric flat bf16 parameter buffer of R * shard_elems elements; rank r's own
//              shard [r * shard_elems, (r + 1) * shard_elems) must be valid there before the launch.
//   C[M][N] = A[M][K] * W^T (+ bias), W = [N][K] row-major at element b_off of the flat buffer, bias (N
//   elements) at bias_off or none when bias_off < 0.  On return of the kernel the local flat buffer holds
//   every rank's shard.  chunk_flags: local int array [2][R][ceil(shard_bytes / chunk_bytes)] (flags, then counters), zero before the
//   first launch.  shard_elems % 8 == 0, chunk_bytes % 16 == 0, b_off % 8 == 0, K % 8 == 0.
MB_API int mb_gemm_param_gather(void* const* w_ptrs, const void* A, void* C, void* const* flag_ptrs,
                                int* chunk_flags, int M, int N, int K, int ldc, long long b_off, long long bias_off,
                                long long shard_elems, long long chunk_bytes, int nranks, int me, int epoch,
                                int n_gather, int wait_ms, cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxRanks || (K & 7) || (b_off & 7) || (shard_elems & 7) || chunk_bytes <= 0 ||
      (chunk_bytes & 15) || b_off < 0 || (bias_off >= 0 && (bias_off & 7)))
    return -1;
  if (b_off + static_cast<long long>(N) * K > shard_elems * nranks) return -1;
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CommParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.mode = MODE_AGW;
  p.nranks = nranks; p.me = me; p.epoch = epoch;
  p.rows_per_rank = M;
  p.n_gather = 0;
  if (nranks > 1)
    p.n_gather = n_gather > 0 ? n_gather
                              : pick_gather_ctas(static_cast<double>(shard_elems) * 2.0 * (nranks - 1),
                                                 2.0 * M * static_cast<double>(N) * K);
  p.chunk_flags = chunk_flags;
  p.C = C; p.ldc = ldc;
  p.status = mb_status_device_ptr();
  p.wait_ns = static_cast<unsigned long long>(wait_ms > 0 ? wait_ms : 2000) * 1000000ull;
  p.shard_bytes = static_cast<unsigned long long>(shard_elems) * 2;
  p.chunk_bytes = static_cast<unsigned long long>(chunk_bytes);
  p.chunks_per_rank = static_cast<int>((p.shard_bytes + p.chunk_bytes - 1) / p.chunk_bytes);
  p.chunk_cnt = chunk_flags + static_cast<long>(nranks) * p.chunks_per_rank;
  p.b_off = static_cast<unsigned long long>(b_off) * 2;
  for (int r = 0; r < nranks; ++r) {
    p.flags[r] = reinterpret_cast<int*>(flag_ptrs[r]);
    p.a_peer[r] = reinterpret_cast<const uint8_t*>(w_ptrs[r]);
  }
  p.a_local = reinterpret_cast<uint8_t*>(w_ptrs[me]);
  if (bias_off >= 0) {
    p.bias_off = static_cast<unsigned long long>(bias_off) * 2;
    p.bias = reinterpret_cast<const __nv_bfloat16*>(p.a_local + p.bias_off);
  }
  // start with the first column tile whose weights are entirely in the local shard, if there is one
  const int num_n = (N + BN - 1) / BN;
  const unsigned long long tile_bytes = static_cast<unsigned long long>(BN) * K * 2;
  const unsigned long long my_lo = static_cast<unsigned long long>(me) * p.shard_bytes, my_hi = my_lo + p.shard_bytes;
  for (int nt = 0; nt < num_n; ++nt) {
    const unsigned long long lo = p.b_off + nt * tile_bytes;
    const unsigned long long hi = p.b_off + static_cast<unsigned long long>(min(N, (nt + 1) * BN)) * K * 2;
    if (lo >= my_lo && hi <= my_hi) {
      p.n_shift = nt;
      break;
    }
  }
  CUtensorMap ta, tb, tc, acc[kMaxRanks];
  memset(acc, 0, sizeof(acc));
  const bool pair = g_pair && (static_cast<long>((M + 2 * BM - 1) / (2 * BM)) * num_n >= (g_sms - p.n_gather) / 2);
  if (!make_map(&ta, A, M, K, K, 64, BM, false)) return -2;
  if (!make_map(&tb, p.a_local + p.b_off, N, K, K, 64, pair ? BN / 2 : BN, false)) return -2;
  if (!make_map(&tc, C, M, N, ldc, 64, BM, false)) return -2;
  const long tiles = static_cast<long>((M + (pair ? 2 : 1) * BM - 1) / ((pair ? 2 : 1) * BM)) * num_n;
  const int compute = plan_grid(pair, tiles, p.n_gather);
  return launch(false, pair, compute + p.n_gather, stream, ta, tb, tc, acc, p);
}

// The gather CTAs' fetch order computed on the host, for tests (the same GatherPlan code that the kernel runs).
// weights = 0: activation gather of AG -> GEMM (K, rows_per_rank); weights = 1: flat parameter buffer
// (shard_bytes, chunk_bytes, first_byte = offset of the first weights the GEMM reads).  q < 0: returns the length
// of the sequence.  Otherwise fills out[0..4] = byte offset, bytes, flag index, sub-chunks of that chunk, source
// rank and returns 1, or returns 0 for an empty entry (beyond the end of a short last chunk).
MB_API int mb_gather_plan_segment(int weights, int nranks, int me, int K, int rows_per_rank, long long shard_bytes,
                                  long long chunk_bytes, long long first_byte, int q, long long* out) {
  GatherPlan plan;
  if (weights)
    plan.init_weights(nranks, me, static_cast<unsigned long long>(shard_bytes),
                      static_cast<unsigned long long>(chunk_bytes), static_cast<unsigned long long>(first_byte));
  else
    plan.init_activations(nranks, me, K, rows_per_rank);
  if (q < 0) return plan.total_subs;
  GatherSeg s;
  if (!plan.segment(q, s)) return 0;
  out[0] = static_cast<long long>(s.off);
  out[1] = s.bytes;
  out[2] = s.flag;
  out[3] = s.expected;
  out[4] = s.r;
  return 1;
}
