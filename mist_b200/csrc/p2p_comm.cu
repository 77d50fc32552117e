// Collectives over NVLink peer memory, fused with the arithmetic that follows them.
//
// Every rank maps every peer's buffers (CUDA IPC) once; kernels then read and write peer
// memory directly with 16-byte loads / stores.  Cross-rank ordering uses small flag
// arrays that live in each rank's own memory and are written remotely by its peers
// (release stores at system scope) and polled locally (acquire loads), always with a
// time limit: a peer that never arrives ends the kernel with status MB_ERR_TIMEOUT_PEER
// instead of hanging the GPU.
//
//   mb_fused_grad_reduce_adam   reduce-scatter of a gradient bucket + (optional) fp32
//                               accumulation + Adam on this rank's shard + write of the
//                               new bf16 weights into every rank's weight buffer
//                               (= reduce-scatter + cast/scale + optimizer + all-gather
//                               in one launch)
//   mb_p2p_all_gather           pull-based all-gather (ZeRO-3 weights, activations)
//   mb_p2p_reduce_scatter       pull-based reduce-scatter with fp32 accumulation
//
// What this replaces in the reference: NCCL reduce_scatter_tensor on a side stream
// (mist/re_swap_manager/flat_param.py:1496-1501), grad.float() (optimizer.py:514-518),
// apex multi_tensor_adam (fused_adam.py:583-690), the master->model cast (optimizer.py:
// 571-599) and the NCCL all_gather of updated weights (optimizer.py:577-585).
#include "common.cuh"
#include <string.h>

namespace {

constexpr int kMaxRanks = 8;
// time limit of a wait on peer flags; mb_set_peer_wait_ms changes it (tests use a short one)
__device__ unsigned long long g_peer_wait_ns = 2000000000ull;

struct PeerPtrs {
  void* p[kMaxRanks];
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* addr) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer16(void* addr, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Waits until flags[r] >= epoch for every r != me.  One thread polls, the block follows.
__device__ bool wait_flags(const int* flags, int nranks, int me, int epoch, int* status) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    int ok = 1;
    const unsigned long long t0 = now_ns();
    for (int r = 0; r < nranks && ok; ++r) {
      if (r == me) continue;
      while (ld_acquire_sys(flags + r) < epoch) {
        if (now_ns() - t0 > g_peer_wait_ns) {
          ok = 0;
          if (status) atomicCAS(status, 0, MB_ERR_TIMEOUT_PEER);
          break;
        }
        __nanosleep(200);
      }
    }
    ok_s = ok;
  }
  __syncthreads();
  return ok_s != 0;
}

// Flag block of one communication slot, in every rank's memory:
//   [0 .. R)      ready[r]: rank r's input is complete for this epoch
//   [R .. 2R)     done[r] : rank r has finished reading / writing peer memory
//   [2R]          blocks_done (local counter)
struct FlagPtrs {
  int* p[kMaxRanks];
};

struct FusedArgs {
  PeerPtrs grads;        // every rank's full gradient bucket
  PeerPtrs params;       // every rank's full bf16 weight buffer (may be null -> no write-back)
  FlagPtrs flags;
  float* master;
  float* exp_avg;
  float* exp_avg_sq;
  float* grad_acc;       // optional fp32 accumulator of the reduced shard
  size_t shard_numel;    // elements per rank (multiple of 8)
  int nranks, me, epoch;
  int grad_is_fp32;
  int do_step;           // 0: only reduce into grad_acc (a micro step before the last one)
  float lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, inv_scale;
  int adamw;
  int* status;
};

__device__ __forceinline__ void add8_bf16(float* acc, uint4 raw) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

// One vector (8 elements) of the fused update: reduced gradient in g[], Adam on the fp32 state, new bf16
// weights to every rank.
__device__ __forceinline__ void fused_step8(const FusedArgs& a, size_t i, size_t base, float* g, int R) {
  if (a.grad_acc) {
    float4 x = reinterpret_cast<float4*>(a.grad_acc)[2 * i];
    float4 y = reinterpret_cast<float4*>(a.grad_acc)[2 * i + 1];
    g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w;
    g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
    if (!a.do_step) {
      reinterpret_cast<float4*>(a.grad_acc)[2 * i] = make_float4(g[0], g[1], g[2], g[3]);
      reinterpret_cast<float4*>(a.grad_acc)[2 * i + 1] = make_float4(g[4], g[5], g[6], g[7]);
    } else {
      reinterpret_cast<float4*>(a.grad_acc)[2 * i] = make_float4(0, 0, 0, 0);
      reinterpret_cast<float4*>(a.grad_acc)[2 * i + 1] = make_float4(0, 0, 0, 0);
    }
  }
  if (!a.do_step) return;
  float4 p0 = reinterpret_cast<float4*>(a.master)[2 * i], p1 = reinterpret_cast<float4*>(a.master)[2 * i + 1];
  float4 m0 = reinterpret_cast<float4*>(a.exp_avg)[2 * i], m1 = reinterpret_cast<float4*>(a.exp_avg)[2 * i + 1];
  float4 v0 = reinterpret_cast<float4*>(a.exp_avg_sq)[2 * i], v1 = reinterpret_cast<float4*>(a.exp_avg_sq)[2 * i + 1];
  float p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
  float m[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
  float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float gg = g[k] * a.inv_scale;
    if (!a.adamw) gg += a.weight_decay * p[k];
    m[k] = a.beta1 * m[k] + (1.f - a.beta1) * gg;
    v[k] = a.beta2 * v[k] + (1.f - a.beta2) * gg * gg;
    float upd = (m[k] / a.bias_c1) / (sqrtf(v[k] / a.bias_c2) + a.eps);
    if (a.adamw) upd += a.weight_decay * p[k];
    p[k] -= a.lr * upd;
  }
  reinterpret_cast<float4*>(a.master)[2 * i] = make_float4(p[0], p[1], p[2], p[3]);
  reinterpret_cast<float4*>(a.master)[2 * i + 1] = make_float4(p[4], p[5], p[6], p[7]);
  reinterpret_cast<float4*>(a.exp_avg)[2 * i] = make_float4(m[0], m[1], m[2], m[3]);
  reinterpret_cast<float4*>(a.exp_avg)[2 * i + 1] = make_float4(m[4], m[5], m[6], m[7]);
  reinterpret_cast<float4*>(a.exp_avg_sq)[2 * i] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(a.exp_avg_sq)[2 * i + 1] = make_float4(v[4], v[5], v[6], v[7]);
  mb::bf16x8 w = mb::pack8(p);
  const uint4 wr = *reinterpret_cast<uint4*>(&w);
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    if (r < R && a.params.p[r])
      st_peer16(reinterpret_cast<__nv_bfloat16*>(a.params.p[r]) + base + 8 * i, wr);
}

// RMAX: upper bound of the rank count this instantiation serves; U: vectors whose peer loads a thread
// issues before it consumes any of them.  NVLink loads take microseconds, so the bytes a thread keeps in
// flight decide the bandwidth: U * R loads of 16 bytes per thread, bounded by the registers they land in.
template <int RMAX, int U, bool FP32>
__global__ void __launch_bounds__(512)
fused_grad_reduce_adam_kernel(const FusedArgs a) {
  int* my_flags = a.flags.p[a.me];
  const int R = a.nranks;
  // ---- phase A: tell every peer that my bucket is complete, wait for theirs
  if (blockIdx.x == 0 && threadIdx.x < R && threadIdx.x != a.me) {
    __threadfence_system();
    st_release_sys(a.flags.p[threadIdx.x] + a.me, a.epoch);
  }
  bool ok = wait_flags(my_flags, R, a.me, a.epoch, a.status);

  // ---- phase B: reduce my shard over all ranks, step, write the new weights everywhere
  if (ok) {
    const size_t nvec = a.shard_numel >> 3;
    const size_t base = static_cast<size_t>(a.me) * a.shard_numel;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i0 < nvec; i0 += stride * U) {
      if (FP32) {
        uint4 lo[U][RMAX], hi[U][RMAX];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t i = i0 + u * stride;
#pragma unroll
          for (int r = 0; r < RMAX; ++r) {
            if (r < R && i < nvec) {
              const float* src = reinterpret_cast<const float*>(a.grads.p[r]) + base + 8 * i;
              lo[u][r] = ld_peer16(src);
              hi[u][r] = ld_peer16(src + 4);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t i = i0 + u * stride;
          if (i >= nvec) continue;
          float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
          for (int r = 0; r < RMAX; ++r) {      // rank order: the same sum on every run
            if (r < R) {
              const float* l = reinterpret_cast<const float*>(&lo[u][r]);
              const float* h = reinterpret_cast<const float*>(&hi[u][r]);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                g[k] += l[k];
                g[4 + k] += h[k];
              }
            }
          }
          fused_step8(a, i, base, g, R);
        }
      } else {
        uint4 raw[U][RMAX];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t i = i0 + u * stride;
#pragma unroll
          for (int r = 0; r < RMAX; ++r)
            if (r < R && i < nvec)
              raw[u][r] = ld_peer16(reinterpret_cast<const __nv_bfloat16*>(a.grads.p[r]) + base + 8 * i);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t i = i0 + u * stride;
          if (i >= nvec) continue;
          float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
          for (int r = 0; r < RMAX; ++r)
            if (r < R) add8_bf16(g, raw[u][r]);
          fused_step8(a, i, base, g, R);
        }
      }
    }
  }

  // ---- phase C: when the whole grid is through, tell the peers; leave only after every
  // peer has said the same (then nobody reads my bucket or writes my weights any more)
  __threadfence_system();
  __syncthreads();
  __shared__ int last_s;
  if (threadIdx.x == 0) {
    int prev = atomicAdd(my_flags + 2 * R, 1);
    last_s = (prev + 1 == static_cast<int>(gridDim.x) * a.epoch);
  }
  __syncthreads();
  if (last_s) {
    if (threadIdx.x < R && threadIdx.x != a.me) {
      __threadfence_system();
      st_release_sys(a.flags.p[threadIdx.x] + R + a.me, a.epoch);
    }
    __syncthreads();
    wait_flags(my_flags + R, R, a.me, a.epoch, a.status);
  }
}

struct GatherArgs {
  PeerPtrs src;          // every rank's shard (shard_bytes each)
  void* dst;             // local full buffer
  FlagPtrs flags;
  size_t shard_bytes;    // multiple of 16
  int nranks, me, epoch;
  int* status;
};

// dst[r * shard .. ] = src_r for every rank r (own shard copied locally)
__global__ void __launch_bounds__(512)
p2p_all_gather_kernel(const GatherArgs a) {
  int* my_flags = a.flags.p[a.me];
  const int R = a.nranks;
  if (blockIdx.x == 0 && threadIdx.x < R && threadIdx.x != a.me) {
    __threadfence_system();
    st_release_sys(a.flags.p[threadIdx.x] + a.me, a.epoch);
  }
  bool ok = wait_flags(my_flags, R, a.me, a.epoch, a.status);
  if (ok) {
    const size_t nvec = a.shard_bytes >> 4;
    const size_t total = nvec * R;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    constexpr int U = 4;      // loads a thread issues before it stores any of them (NVLink latency is microseconds)
    for (size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i0 < total; i0 += stride * U) {
      uint4 v[U];
      size_t dsti[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t i = i0 + u * stride;
        if (i < total) {
          // start with the next rank's shard so the ranks do not all read the same peer at once
          const size_t k = i / nvec;
          const int r = static_cast<int>((a.me + 1 + k) % R);
          const size_t j = i - k * nvec;
          v[u] = ld_peer16(reinterpret_cast<const uint4*>(a.src.p[r]) + j);
          dsti[u] = static_cast<size_t>(r) * nvec + j;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < total) reinterpret_cast<uint4*>(a.dst)[dsti[u]] = v[u];
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int last_s;
  if (threadIdx.x == 0) {
    int prev = atomicAdd(my_flags + 2 * R, 1);
    last_s = (prev + 1 == static_cast<int>(gridDim.x) * a.epoch);
  }
  __syncthreads();
  if (last_s) {
    if (threadIdx.x < R && threadIdx.x != a.me) st_release_sys(a.flags.p[threadIdx.x] + R + a.me, a.epoch);
    __syncthreads();
    wait_flags(my_flags + R, R, a.me, a.epoch, a.status);
  }
}

struct ReduceScatterArgs {
  PeerPtrs src;          // every rank's full bf16 buffer
  void* dst;             // local shard (bf16 or fp32)
  FlagPtrs flags;
  size_t shard_numel;
  int nranks, me, epoch;
  int dst_is_fp32, accumulate;
  int* status;
};

__global__ void __launch_bounds__(512)
p2p_reduce_scatter_kernel(const ReduceScatterArgs a) {
  int* my_flags = a.flags.p[a.me];
  const int R = a.nranks;
  if (blockIdx.x == 0 && threadIdx.x < R && threadIdx.x != a.me) {
    __threadfence_system();
    st_release_sys(a.flags.p[threadIdx.x] + a.me, a.epoch);
  }
  bool ok = wait_flags(my_flags, R, a.me, a.epoch, a.status);
  if (ok) {
    const size_t nvec = a.shard_numel >> 3;
    const size_t base = static_cast<size_t>(a.me) * a.shard_numel;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
      float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      uint4 raw[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < R) raw[r] = ld_peer16(reinterpret_cast<const __nv_bfloat16*>(a.src.p[r]) + base + 8 * i);
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < R) add8_bf16(g, raw[r]);   // fixed rank order: every run sums in the same order
      if (a.dst_is_fp32) {
        float4* d = reinterpret_cast<float4*>(a.dst) + 2 * i;
        if (a.accumulate) {
          float4 x = d[0], y = d[1];
          g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w;
          g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
        }
        d[0] = make_float4(g[0], g[1], g[2], g[3]);
        d[1] = make_float4(g[4], g[5], g[6], g[7]);
      } else {
        reinterpret_cast<mb::bf16x8*>(a.dst)[i] = mb::pack8(g);
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int last_s;
  if (threadIdx.x == 0) {
    int prev = atomicAdd(my_flags + 2 * R, 1);
    last_s = (prev + 1 == static_cast<int>(gridDim.x) * a.epoch);
  }
  __syncthreads();
  if (last_s) {
    if (threadIdx.x < R && threadIdx.x != a.me) st_release_sys(a.flags.p[threadIdx.x] + R + a.me, a.epoch);
    __syncthreads();
    wait_flags(my_flags + R, R, a.me, a.epoch, a.status);
  }
}

// Sum of the R per-source slots that the store form of the GEMM -> reduce-scatter kernel fills
// (gemm_comm_tcgen05.cu): out = bf16(slot[0] + slot[1] + ... (+ bias) (+ residual)), added in fp32
// in rank order, so the result is the same on every run and for every arrival order.
__global__ void __launch_bounds__(256)
rs_sum_kernel(const __nv_bfloat16* __restrict__ slots, size_t slot_stride, int R, size_t nvec, int ncols,
              const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ residual,
              __nv_bfloat16* __restrict__ out) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    uint4 raw[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < R) raw[r] = *reinterpret_cast<const uint4*>(slots + r * slot_stride + 8 * i);
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < R) add8_bf16(g, raw[r]);
    if (bias) add8_bf16(g, *reinterpret_cast<const uint4*>(bias + (8 * i) % ncols));
    if (residual) add8_bf16(g, *reinterpret_cast<const uint4*>(residual + 8 * i));
    reinterpret_cast<mb::bf16x8*>(out)[i] = mb::pack8(g);
  }
}

// A wait that nothing satisfies: used by the tests of the time limit.
__global__ void wait_on_flag_kernel(const int* flags, int nranks, int epoch, int* status) {
  wait_flags(flags, nranks, -1, epoch, status);
}

}  // namespace

MB_API int* mb_status_device_ptr();

// CTAs of the fused gradient kernel when the caller passes none (mb_set_fused_grad_ctas changes it)
static int g_fused_ctas = 96;
MB_API void mb_set_fused_grad_ctas(int n) { g_fused_ctas = n > 0 ? n : 96; }

MB_API int mb_set_peer_wait_ms(int ms) {
  unsigned long long ns = static_cast<unsigned long long>(ms) * 1000000ull;
  return cudaMemcpyToSymbol(g_peer_wait_ns, &ns, sizeof(ns)) == cudaSuccess ? 0 : -1;
}

// ------------------------------------------------------------ symmetric memory plumbing
MB_API int mb_symm_alloc(size_t bytes, void** out) {
  return cudaMalloc(out, bytes) == cudaSuccess ? 0 : -1;
}
MB_API int mb_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }
MB_API int mb_symm_memset(void* p, int value, size_t bytes, cudaStream_t s) {
  return cudaMemsetAsync(p, value, bytes, s) == cudaSuccess ? 0 : -1;
}
MB_API int mb_ipc_handle_size() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }
MB_API int mb_ipc_get_handle(void* p, void* handle_out) {
  return cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle_out), p) == cudaSuccess ? 0 : -1;
}
MB_API int mb_ipc_open_handle(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
MB_API int mb_ipc_close_handle(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }

// ------------------------------------------------------------------------ launch wrappers
// `ptr_table` layouts are arrays of `nranks` device pointers (index = rank in the group).
MB_API int mb_fused_grad_reduce_adam(void* const* grad_ptrs, void* const* param_ptrs, void* const* flag_ptrs,
                                     float* master, float* exp_avg, float* exp_avg_sq, float* grad_acc,
                                     size_t shard_numel, int nranks, int me, int epoch, int grad_is_fp32,
                                     int do_step, float lr, float beta1, float beta2, float eps,
                                     float weight_decay, int step, float inv_scale, int adamw, int num_ctas,
                                     cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxRanks || (shard_numel & 7)) return -1;
  FusedArgs a;
  memset(&a, 0, sizeof(a));
  for (int r = 0; r < nranks; ++r) {
    a.grads.p[r] = grad_ptrs[r];
    a.params.p[r] = param_ptrs ? param_ptrs[r] : nullptr;
    a.flags.p[r] = reinterpret_cast<int*>(flag_ptrs[r]);
  }
  a.master = master; a.exp_avg = exp_avg; a.exp_avg_sq = exp_avg_sq; a.grad_acc = grad_acc;
  a.shard_numel = shard_numel;
  a.nranks = nranks; a.me = me; a.epoch = epoch;
  a.grad_is_fp32 = grad_is_fp32; a.do_step = do_step;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias_c1 = 1.f - powf(beta1, static_cast<float>(step));
  a.bias_c2 = 1.f - powf(beta2, static_cast<float>(step));
  a.inv_scale = inv_scale; a.adamw = adamw;
  a.status = mb_status_device_ptr();
  if (num_ctas <= 0) num_ctas = g_fused_ctas;
  // the flag counter of a call site assumes the same grid on every launch of that site
  if (grad_is_fp32) {
    if (nranks <= 2) fused_grad_reduce_adam_kernel<2, 2, true><<<num_ctas, 512, 0, stream>>>(a);
    else if (nranks <= 4) fused_grad_reduce_adam_kernel<4, 1, true><<<num_ctas, 512, 0, stream>>>(a);
    else fused_grad_reduce_adam_kernel<8, 1, true><<<num_ctas, 512, 0, stream>>>(a);
  } else {
    if (nranks <= 2) fused_grad_reduce_adam_kernel<2, 4, false><<<num_ctas, 512, 0, stream>>>(a);
    else if (nranks <= 4) fused_grad_reduce_adam_kernel<4, 2, false><<<num_ctas, 512, 0, stream>>>(a);
    else fused_grad_reduce_adam_kernel<8, 1, false><<<num_ctas, 512, 0, stream>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

MB_API int mb_p2p_all_gather(void* const* src_ptrs, void* dst, void* const* flag_ptrs, size_t shard_bytes,
                             int nranks, int me, int epoch, int num_ctas, cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxRanks || (shard_bytes & 15)) return -1;
  GatherArgs a;
  memset(&a, 0, sizeof(a));
  for (int r = 0; r < nranks; ++r) {
    a.src.p[r] = src_ptrs[r];
    a.flags.p[r] = reinterpret_cast<int*>(flag_ptrs[r]);
  }
  a.dst = dst; a.shard_bytes = shard_bytes; a.nranks = nranks; a.me = me; a.epoch = epoch;
  a.status = mb_status_device_ptr();
  if (num_ctas <= 0) num_ctas = 48;
  p2p_all_gather_kernel<<<num_ctas, 512, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

MB_API int mb_p2p_reduce_scatter(void* const* src_ptrs, void* dst, void* const* flag_ptrs, size_t shard_numel,
                                 int nranks, int me, int epoch, int dst_is_fp32, int accumulate, int num_ctas,
                                 cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxRanks || (shard_numel & 7)) return -1;
  ReduceScatterArgs a;
  memset(&a, 0, sizeof(a));
  for (int r = 0; r < nranks; ++r) {
    a.src.p[r] = src_ptrs[r];
    a.flags.p[r] = reinterpret_cast<int*>(flag_ptrs[r]);
  }
  a.dst = dst; a.shard_numel = shard_numel; a.nranks = nranks; a.me = me; a.epoch = epoch;
  a.dst_is_fp32 = dst_is_fp32; a.accumulate = accumulate;
  a.status = mb_status_device_ptr();
  if (num_ctas <= 0) num_ctas = 48;
  p2p_reduce_scatter_kernel<<<num_ctas, 512, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// out[numel] = sum over r < nranks of slots[r * slot_stride + ...] (+ bias[col]) (+ residual), bf16 in and
// out, fp32 sum in rank order.  numel and ncols multiples of 8.
MB_API int mb_rs_sum(const void* slots, size_t slot_stride, int nranks, size_t numel, int ncols, const void* bias,
                     const void* residual, void* out, cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxRanks || (numel & 7) || (ncols & 7) || (slot_stride & 7)) return -1;
  const size_t nvec = numel >> 3;
  int blocks = static_cast<int>((nvec + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  rs_sum_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(slots), slot_stride, nranks, nvec,
                                            ncols, reinterpret_cast<const __nv_bfloat16*>(bias),
                                            reinterpret_cast<const __nv_bfloat16*>(residual),
                                            reinterpret_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Polls `nranks` local flags for `epoch`; with flags that nobody sets this returns after
// the time limit and leaves MB_ERR_TIMEOUT_PEER in the status word.
MB_API int mb_wait_on_flags(const int* flags, int nranks, int epoch, cudaStream_t stream) {
  wait_on_flag_kernel<<<1, 32, 0, stream>>>(flags, nranks, epoch, mb_status_device_ptr());
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
