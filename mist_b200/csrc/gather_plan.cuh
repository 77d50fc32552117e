// Fetch order of the gather CTAs of the fused GEMM kernels (gemm_comm_tcgen05.cu), as plain integer
// arithmetic that compiles for the host as well: the kernel walks it on the device, and
// mb_gather_plan_segment exposes the same code to the tests, which check on the CPU that every remote byte
// is fetched exactly once and that the chunk counters add up.
//
// The remote chunks (the unit a GEMM tile waits for: 128 rows of the gathered activation, or chunk_bytes of
// the flat parameter buffer) are cut into sub-chunks of kGatherSubBytes.  Sub-chunk q of the sequence goes to
// gather CTA q % n_gather, so all gather CTAs work on the chunk that is needed next.
//   activations (AG -> GEMM): the peers in turn, starting with the next rank, so that every rank reads from
//     a different source at any time;
//   weights: the peers' chunks alternate, each peer's in address order (the owner of the first weights of
//     the GEMM starting with the chunk that holds them): every rank needs the same weights first, and one
//     source could not feed all readers at the full rate.
#pragma once
#include <stdint.h>

#ifndef __CUDACC__
#define MB_HD
#else
#define MB_HD __host__ __device__
#endif

constexpr int kGatherSubBytes = 16 * 16384;
constexpr int kGatherRowsPerChunk = 128;      // activation gather: one flag per 128-row block

struct GatherSeg {
  unsigned long long off;     // byte offset in every rank's buffer (source and destination alike)
  uint32_t bytes;
  int flag;                   // index of the chunk's flag and counter
  int expected;               // sub-chunks that make up this chunk
  int r;                      // source rank
};

struct GatherPlan {
  int ag, R, me;
  int cpr;                    // chunks per rank
  int subs;                   // sub-chunks of a full chunk
  int total_subs;             // length of the sequence (entries of a short last chunk may be empty)
  int r0, c0;                 // weights: owner and chunk of the first bytes the GEMM needs
  int rows_per_rank;
  unsigned long long cbytes, row_bytes, shard_bytes, chunk_bytes;

  MB_HD void init_activations(int nranks, int rank, int K, int rows) {
    ag = 1; R = nranks; me = rank; rows_per_rank = rows;
    row_bytes = static_cast<unsigned long long>(K) * 2;
    cbytes = static_cast<unsigned long long>(kGatherRowsPerChunk) * row_bytes;
    cpr = rows / kGatherRowsPerChunk;
    shard_bytes = chunk_bytes = 0;
    r0 = -1; c0 = 0;
    finish();
  }
  // first_byte: offset in the flat buffer of the first weights that the GEMM reads
  MB_HD void init_weights(int nranks, int rank, unsigned long long shard, unsigned long long chunk,
                          unsigned long long first_byte) {
    ag = 0; R = nranks; me = rank; rows_per_rank = 0; row_bytes = 0;
    shard_bytes = shard; chunk_bytes = chunk; cbytes = chunk;
    cpr = static_cast<int>((shard + chunk - 1) / chunk);
    r0 = static_cast<int>(first_byte / shard);
    c0 = static_cast<int>((first_byte - static_cast<unsigned long long>(r0) * shard) / chunk);
    finish();
  }
  MB_HD void finish() {
    subs = static_cast<int>((cbytes + kGatherSubBytes - 1) / kGatherSubBytes);
    total_subs = (R - 1) * cpr * subs;          // < 2^31: a few thousand per GB
  }
  // q-th sub-chunk of the sequence; false when it lies beyond the end of a short last chunk
  MB_HD bool segment(int q, GatherSeg& s) const {
    const int w = q / subs;
    const int sub = q - w * subs;
    int r, c;
    unsigned long long bytes, off;
    if (ag) {
      const int k = w / cpr;
      c = w - k * cpr;
      r = (me + 1 + k) % R;
      off = (static_cast<unsigned long long>(r) * rows_per_rank +
             static_cast<unsigned long long>(c) * kGatherRowsPerChunk) * row_bytes;
      bytes = cbytes;
    } else {
      const int i = w / (R - 1);
      const int k = w - i * (R - 1);
      r = (me + 1 + k) % R;
      c = (r == r0) ? (c0 + i) % cpr : i;
      const unsigned long long in_shard = static_cast<unsigned long long>(c) * chunk_bytes;
      bytes = shard_bytes - in_shard < chunk_bytes ? shard_bytes - in_shard : chunk_bytes;
      off = static_cast<unsigned long long>(r) * shard_bytes + in_shard;
    }
    const unsigned long long lo = static_cast<unsigned long long>(sub) * kGatherSubBytes;
    if (lo >= bytes) return false;
    s.off = off + lo;
    s.bytes = static_cast<uint32_t>(bytes - lo < kGatherSubBytes ? bytes - lo : kGatherSubBytes);
    s.flag = r * cpr + c;
    s.expected = (bytes == cbytes) ? subs : static_cast<int>((bytes + kGatherSubBytes - 1) / kGatherSubBytes);
    s.r = r;
    return true;
  }
};
