// Exact top-k of one row of fp32 logits, ties to the lower position, output in
// ascending position order.
//
// Replaces torch.topk on the logit slab (src/lagged_indexer_dsa/
// attention_core.py:66-91) and the reference's in-kernel select, whose row
// barrier is an unbounded spin on a global counter
// (kernels/cuda_fused_sparse_splitk.py:2017-2154). Here one thread-block
// cluster of 8 CTAs owns a row and its CTAs meet only at hardware cluster
// barriers:
//
//   * every thread keeps ITEMS consecutive logits as order-preserving u32 keys
//     in registers for the whole kernel (the row is read once);
//   * an MSB-first radix select narrows the k-th largest key: per round each
//     CTA histograms the digit of its still-matching keys in shared memory, the
//     cluster sums the eight histograms through distributed shared memory, and
//     every CTA derives the same threshold digit. With the 4096-bin histogram
//     that the scan epilogue already filled, the first round is free;
//   * the last step ranks ties by position with block scans plus one exchange of
//     per-CTA counts, so the kept set and its order are deterministic.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace dsa {
namespace topk {

namespace cg = cooperative_groups;

constexpr int kCluster = 8;
constexpr int kThreads = 1024;
constexpr int kMaxBins = DSA_TOPK_HIST_BINS;  // 4096: first level when the scan supplies it
constexpr int kRoundBins = 2048;              // in-kernel rounds use at most 11-bit digits

struct Params {
  const float* logits;
  const int32_t* seq_lens;
  uint32_t* hist;
  const int32_t* index_map;
  int32_t* out_idx;
  float* out_val;
  int64_t n;
  int64_t slab_stride;
  int topk;
  int32_t pad;
  int32_t index_offset;
};

struct Shared {
  uint32_t tot[kMaxBins];
  uint32_t hist[2][kRoundBins];
  uint32_t warp_tot[32];
  uint32_t sel_bin;
  uint32_t k_next;
  uint32_t block_total;
  uint32_t cta_tot;  // published to the cluster: above | ties << 16
};

// Exclusive prefix of v over the 1024 threads of the block; *total (optional)
// receives the block sum. Two barriers; safe to call back to back.
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, Shared& sh, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += up;
  }
  __syncthreads();  // previous users of warp_tot are done
  if (lane == 31) sh.warp_tot[warp] = inc;
  __syncthreads();
  uint32_t wsum = sh.warp_tot[lane];
  uint32_t winc = wsum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, winc, o);
    if (lane >= o) winc += up;
  }
  const uint32_t before = __shfl_sync(0xffffffffu, winc - wsum, warp);
  if (total) *total = __shfl_sync(0xffffffffu, winc, 31);
  return before + inc - v;
}

// Walks sh.tot[0..nb) from the highest bin down and finds the bin holding the
// k-th largest element; leaves the bin in sh.sel_bin and the rank inside that
// bin in sh.k_next. nb is 1024, 2048 or 4096. Ends with a barrier.
__device__ __forceinline__ void find_threshold_bin(Shared& sh, int nb, uint32_t k) {
  const int per = nb >> 10;
  const int first = nb - 1 - int(threadIdx.x) * per;  // this thread's highest bin
  uint32_t s = 0;
  for (int i = 0; i < per; ++i) s += sh.tot[first - i];
  uint32_t running = block_exclusive_scan(s, sh, nullptr);
  for (int i = 0; i < per; ++i) {
    const uint32_t c = sh.tot[first - i];
    if (running < k && k <= running + c) {
      sh.sel_bin = uint32_t(first - i);
      sh.k_next = k - running;
    }
    running += c;
  }
  __syncthreads();
}

template <int ITEMS>
__global__ void __launch_bounds__(kThreads, 1)
topk_select_kernel(const Params p) {
  __shared__ Shared sh;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned crank = cluster.block_rank();
  const int tid = threadIdx.x;
  const int r = blockIdx.y;
  const float* row = p.logits + int64_t(r) * p.slab_stride;
  int64_t len = p.seq_lens ? int64_t(p.seq_lens[r]) : p.n;
  len = len < 0 ? 0 : (len > p.n ? p.n : len);
  const int64_t base = (int64_t(crank) * kThreads + tid) * ITEMS;

  uint32_t key[ITEMS];
  if (ITEMS % 4 == 0 && base + ITEMS <= len && ((p.slab_stride & 3) == 0)) {
#pragma unroll
    for (int j = 0; j < ITEMS; j += 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + base + j);
      key[j] = ordered_key(v.x);
      key[j + 1] = ordered_key(v.y);
      key[j + 2] = ordered_key(v.z);
      key[j + 3] = ordered_key(v.w);
    }
  } else {
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) key[j] = (base + j < len) ? ordered_key(row[base + j]) : 0u;
  }
  const int n_valid = len - base >= ITEMS ? ITEMS : (len > base ? int(len - base) : 0);

  const bool take_all = len <= p.topk;
  uint32_t prefix = 0, mask = 0, k_rem = uint32_t(p.topk);
  bool hist_pending_reset = false;

  if (!take_all) {
    int shift = 32;
    int round = 0;
    if (p.hist != nullptr) {
      // first level from the histogram the scan filled: top 12 key bits
      const uint32_t* gh = p.hist + size_t(r) * kMaxBins;
      for (int i = tid; i < kMaxBins; i += kThreads) sh.tot[i] = gh[i];
      __syncthreads();
      find_threshold_bin(sh, kMaxBins, k_rem);
      shift = 20;
      prefix = sh.sel_bin << shift;
      mask = 0xFFFu << shift;
      k_rem = sh.k_next;
      hist_pending_reset = true;
    }
    while (shift > 0) {
      const int bits = shift > 21 ? 11 : (shift > 10 ? shift - 10 : shift);
      const int nb = 1 << bits;
      shift -= bits;
      uint32_t* hb = sh.hist[round & 1];
      for (int i = tid; i < nb; i += kThreads) hb[i] = 0;
      __syncthreads();
#pragma unroll
      for (int j = 0; j < ITEMS; ++j)
        if (j < n_valid && (key[j] & mask) == prefix) atomicAdd(&hb[(key[j] >> shift) & (nb - 1)], 1u);
      cluster.sync();
      if (hist_pending_reset) {
        // every CTA of the row has read the scan's histogram: re-arm it for the next launch
        uint32_t* gh = p.hist + size_t(r) * kMaxBins;
        for (int i = crank * kThreads + tid; i < kMaxBins; i += kCluster * kThreads) gh[i] = 0;
        hist_pending_reset = false;
      }
      for (int i = tid; i < nb; i += kThreads) {
        uint32_t t = 0;
#pragma unroll
        for (unsigned c = 0; c < kCluster; ++c) t += cluster.map_shared_rank(hb, c)[i];
        sh.tot[i] = t;
      }
      __syncthreads();
      find_threshold_bin(sh, nb, k_rem);
      prefix |= sh.sel_bin << shift;
      mask |= uint32_t(nb - 1) << shift;
      k_rem = sh.k_next;
      ++round;
    }
  } else if (p.hist != nullptr) {
    uint32_t* gh = p.hist + size_t(r) * kMaxBins;
    for (int i = crank * kThreads + tid; i < kMaxBins; i += kCluster * kThreads) gh[i] = 0;
  }

  // ---- rank ties by position and emit
  uint32_t cnt_above = 0, cnt_tie = 0;
  if (take_all) {
    cnt_above = uint32_t(n_valid);
    k_rem = 0;
  } else {
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
      if (j < n_valid) {
        cnt_above += key[j] > prefix;
        cnt_tie += key[j] == prefix;
      }
    }
  }
  uint32_t block_total = 0;
  const uint32_t excl = block_exclusive_scan(cnt_above | (cnt_tie << 16), sh, &block_total);
  if (tid == 0) sh.cta_tot = block_total;
  cluster.sync();
  // CTAs of lower rank hold lower positions: their kept entries come first
  uint32_t ties_before = 0, sel_before = 0;
#pragma unroll
  for (unsigned c = 0; c < kCluster; ++c) {
    const uint32_t t = *cluster.map_shared_rank(&sh.cta_tot, c);
    if (c < crank) {
      const uint32_t a_c = t & 0xFFFFu, t_c = t >> 16;
      const uint32_t kept = k_rem > ties_before ? min(k_rem - ties_before, t_c) : 0u;
      sel_before += a_c + kept;
      ties_before += t_c;
    }
  }
  const uint32_t my_tie_base = ties_before + (excl >> 16);
  const uint32_t my_kept = k_rem > my_tie_base ? min(k_rem - my_tie_base, cnt_tie) : 0u;
  uint32_t pos = sel_before + block_exclusive_scan(cnt_above + my_kept, sh, nullptr);

  int32_t* out_idx = p.out_idx + int64_t(r) * p.topk;
  float* out_val = p.out_val ? p.out_val + int64_t(r) * p.topk : nullptr;
  const int32_t* imap = p.index_map ? p.index_map + int64_t(r) * p.n : nullptr;
  uint32_t tie_rank = my_tie_base;
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    if (j < n_valid) {
      bool keep;
      if (take_all) {
        keep = true;
      } else if (key[j] > prefix) {
        keep = true;
      } else if (key[j] == prefix) {
        keep = tie_rank < k_rem;
        ++tie_rank;
      } else {
        keep = false;
      }
      if (keep && pos < uint32_t(p.topk)) {
        const uint32_t kk = key[j];
        const uint32_t bits = (kk & 0x80000000u) ? (kk ^ 0x80000000u) : ~kk;
        const bool is_neg_inf = bits == 0xff800000u;
        const int64_t at = base + j;
        int32_t id = imap ? imap[at] : int32_t(at) + p.index_offset;
        out_idx[pos] = is_neg_inf ? p.pad : id;
        if (out_val) out_val[pos] = __uint_as_float(bits);
        ++pos;
      }
    }
  }
  if (take_all && crank == 0) {
    const float neg_inf = __int_as_float(0xff800000);
    for (int64_t i = len + tid; i < p.topk; i += kThreads) {
      out_idx[i] = p.pad;
      if (out_val) out_val[i] = neg_inf;
    }
  }
  cluster.sync();  // nobody leaves while a peer may still read its shared memory
}

}  // namespace topk
}  // namespace dsa
