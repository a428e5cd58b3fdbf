// Exact top-k of each row of fp32 logits, ties to the lower position, output in
// ascending position order.
//
// Replaces torch.topk on the logit slab (src/lagged_indexer_dsa/
// attention_core.py:66-91) and the reference's in-kernel select, which walks a
// 10-bit coarse histogram to a threshold bin and resolves that bin exactly, but
// synchronises a row's blocks with an unbounded spin on a global counter
// (kernels/cuda_fused_sparse_splitk.py:2017-2154). The same two-level idea is
// laid out here as launches in stream order, so no block ever waits for another:
//
//   1. (optional) topk_hist_kernel: 4096-bin histogram of the top 12 bits of the
//      order-preserving key. Skipped when the indexer scan already produced it
//      in its epilogue.
//   2. topk_classify_kernel, all SMs: every CTA finds the threshold bin T from
//      the histogram and classifies its 2048 logits with warp ballots: bin > T
//      goes into a bit mask (certainly kept), bin == T is a candidate whose
//      (key, position) each warp compacts, in position order, into its own slot
//      of a candidate buffer.
//   3. topk_finish_kernel, one CTA per row: gathers the few thousand candidates
//      into shared memory, runs two 10-bit radix rounds on the low 20 key bits,
//      ranks exact ties by position, ORs the kept candidates into the mask and
//      expands the mask into the ascending index list.
//
// Scratch per row (caller-owned): mask of n/32 words, per-warp candidate counts
// and slots, (T, need) header, histogram. Only the histogram must be zero on
// entry; the finish kernel re-zeroes it.
#pragma once

#include "common.cuh"

namespace dsa {
namespace topk {

constexpr int kThreads = 512;                   // classify / histogram CTAs
constexpr int kItems = 4;                       // logits per thread in the classify phase
constexpr int kChunk = kThreads * kItems;       // 2048 logits per CTA
constexpr int kWarpSpan = 32 * kItems;          // 128 consecutive logits per warp = one candidate slot
constexpr int kBins = DSA_TOPK_HIST_BINS;       // 4096 = top 12 key bits
constexpr int kLowBits = 20;
constexpr int kRoundBins = 1024;                // two 10-bit rounds over the low 20 bits
constexpr int kFinThreads = 1024;               // finish CTA
constexpr int kFinWarps = kFinThreads / 32;
constexpr int kCandCap = 8192;                  // candidates held in shared memory (more: re-read from L2)
constexpr int kTinyCap = 1024;                  // candidates sharing the threshold's top 22 key bits
constexpr int64_t kMaxN = 1 << 20;              // the selection mask of one row lives in shared memory

struct Params {
  const float* logits;
  const int32_t* seq_lens;
  uint32_t* hist;        // [R][4096]: from the scan, or the workspace copy filled by topk_hist_kernel
  uint32_t* above_mask;  // [R][words]
  uint32_t* slot_cnt;    // [R][slots]        candidates in each warp slot
  uint2* slot_cand;      // [R][slots][128]   (key, position), position order
  uint32_t* header;      // [R][4]            T, need
  uint32_t* hist2;       // [R][1024]         bits 19..10 of the candidates' keys (filled by classify)
  const int32_t* index_map;
  int32_t* out_idx;
  float* out_val;
  int64_t n;
  int64_t slab_stride;
  int words;             // mask words per row, rounded up to whole chunks
  int slots;             // warp slots per row = words / 4
  int topk;
  int32_t pad;
  int32_t index_offset;
};

// Workspace layout in 32-bit words: [R][words] mask | [R][slots] counts |
// [R][4] header | [R][4096] histogram | [R][1024] second-level histogram |
// [R][slots][128][2] candidates. The two histograms must be zero on entry.
__host__ __device__ inline int64_t mask_words(int64_t n) {
  const int64_t chunks = (n + kChunk - 1) / kChunk;
  return chunks * (kChunk / 32);
}
__host__ __device__ inline int64_t workspace_words(int64_t R, int64_t n) {
  const int64_t words = mask_words(n), slots = words / 4;
  return R * (words + slots + 4 + kBins + kRoundBins + slots * kWarpSpan * 2) + 32;
}

// Exclusive prefix of v over the block's threads (NW warps); *total = block sum.
template <int NW>
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_tot, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += up;
  }
  __syncthreads();  // earlier readers of warp_tot are done
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  const uint32_t wsum = lane < NW ? warp_tot[lane] : 0u;
  uint32_t winc = wsum;
#pragma unroll
  for (int o = 1; o < NW; o <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, winc, o);
    if (lane >= o) winc += up;
  }
  const uint32_t before = __shfl_sync(0xffffffffu, winc - wsum, warp);
  if (total) *total = __shfl_sync(0xffffffffu, winc, NW - 1);
  return before + inc - v;
}

// Given this thread's PER bin counts c[] (thread t owns the PER bins just below
// nb - PER t, highest first), finds the bin holding the k-th largest element.
// res[0] = bin, res[1] = rank inside the bin. Ends with a barrier.
template <int NW, int PER>
__device__ __forceinline__ void find_threshold_bin(const uint32_t (&c)[PER], int nb, uint32_t k,
                                                   uint32_t* warp_tot, uint32_t* res) {
  const int first = nb - 1 - int(threadIdx.x) * PER;
  uint32_t s = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) s += c[i];
  uint32_t running = block_exclusive_scan<NW>(s, warp_tot, nullptr);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    if (running < k && k <= running + c[i]) {
      res[0] = uint32_t(first - i);
      res[1] = k - running;
    }
    running += c[i];
  }
  __syncthreads();
}

// 4096-bin histogram of one row chunk (only needed when the scan did not build it).
__global__ void __launch_bounds__(kThreads)
topk_hist_kernel(const Params p) {
  __shared__ uint32_t s_hist[kBins];
  __shared__ uint32_t s_lo, s_hi;
  const int tid = threadIdx.x, r = blockIdx.y;
  for (int i = tid; i < kBins; i += kThreads) s_hist[i] = 0;
  if (tid == 0) {
    s_lo = kBins;
    s_hi = 0;
  }
  __syncthreads();
  pdl_wait();
  pdl_launch_dependents();
  int64_t len = p.seq_lens ? int64_t(p.seq_lens[r]) : p.n;
  len = len < 0 ? 0 : (len > p.n ? p.n : len);
  const float* row = p.logits + int64_t(r) * p.slab_stride;
  uint32_t lo = kBins, hi = 0;
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const int64_t i = int64_t(blockIdx.x) * kChunk + j * kThreads + tid;
    if (i < len) {
      const uint32_t bin = ordered_key(row[i]) >> kLowBits;
      smem_red_add(&s_hist[bin], 1u);
      lo = min(lo, bin);
      hi = max(hi, bin);
    }
  }
  lo = __reduce_min_sync(0xffffffffu, lo);
  hi = __reduce_max_sync(0xffffffffu, hi);
  if ((tid & 31) == 0) {
    atomicMin(&s_lo, lo);
    atomicMax(&s_hi, hi);
  }
  __syncthreads();
  uint32_t* gh = p.hist + size_t(r) * kBins;
  const int top = int(s_hi);
  for (int i = int(s_lo) + tid; i <= top; i += kThreads) {
    const uint32_t c = s_hist[i];
    if (c) atomicAdd(&gh[i], c);
  }
}

__global__ void __launch_bounds__(kThreads)
topk_classify_kernel(const Params p) {
  __shared__ uint32_t s_warp_tot[kThreads / 32];
  __shared__ uint32_t s_res[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = blockIdx.y;
  DSA_KTIME_BEGIN(1);
  pdl_wait();
  pdl_launch_dependents();
  const float* row = p.logits + int64_t(r) * p.slab_stride;
  int64_t len = p.seq_lens ? int64_t(p.seq_lens[r]) : p.n;
  len = len < 0 ? 0 : (len > p.n ? p.n : len);
  const bool take_all = len <= p.topk;

  // issue the loads of this CTA's 2048 logits, then find the threshold bin
  const int64_t span0 = int64_t(blockIdx.x) * kChunk + warp * kWarpSpan;
  float v[kItems];
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const int64_t i = span0 + j * 32 + lane;
    v[j] = i < len ? row[i] : 0.f;
  }
  uint32_t T = 0;
  if (!take_all) {
    constexpr int PER = kBins / kThreads;  // 8 bins per thread, two 16-byte loads
    const uint4* gh4 = reinterpret_cast<const uint4*>(p.hist + size_t(r) * kBins + (kBins - PER * (tid + 1)));
    const uint4 lo = __ldcg(gh4), hi = __ldcg(gh4 + 1);
    const uint32_t c[PER] = {hi.w, hi.z, hi.y, hi.x, lo.w, lo.z, lo.y, lo.x};  // highest bin first
    find_threshold_bin<kThreads / 32, PER>(c, kBins, uint32_t(p.topk), s_warp_tot, s_res);
    T = s_res[0];
    if (blockIdx.x == 0 && tid == 0) {
      p.header[r * 4 + 0] = T;
      p.header[r * 4 + 1] = s_res[1];  // how many of bin T's elements are kept (>= 1)
    }
  }
  // classify with ballots: mask word for bin > T, compacted (key, position) for bin == T
  const int64_t slot = span0 / kWarpSpan;
  uint2* cand = p.slot_cand + (int64_t(r) * p.slots + slot) * kWarpSpan;
  uint32_t* above_mask = p.above_mask + size_t(r) * p.words;
  uint32_t cnt = 0;
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const int64_t i = span0 + j * 32 + lane;
    const uint32_t key = ordered_key(v[j]);
    const uint32_t bin = key >> kLowBits;
    const bool valid = i < len;
    const bool is_cand = valid && !take_all && bin == T;
    const uint32_t a = __ballot_sync(0xffffffffu, valid && (take_all || bin > T));
    const uint32_t c = __ballot_sync(0xffffffffu, is_cand);
    if (is_cand) cand[cnt + __popc(c & ((1u << lane) - 1u))] = make_uint2(key, uint32_t(i));
    cnt += __popc(c);
    if (c) {  // lanes with the same digit add once (a row of equal logits stays cheap)
      const uint32_t digit = is_cand ? ((key >> 10) & (kRoundBins - 1)) : 0xFFFFFFFFu;
      const uint32_t peers = __match_any_sync(0xffffffffu, digit);
      if (is_cand && lane == __ffs(peers) - 1) atomicAdd(&p.hist2[size_t(r) * kRoundBins + digit], __popc(peers));
    }
    if (lane == 0) above_mask[(span0 >> 5) + j] = a;
  }
  if (lane == 0) p.slot_cnt[int64_t(r) * p.slots + slot] = cnt;
  DSA_KTIME_END(1);
}

struct FinShared {
  uint32_t cand_key[kCandCap];
  uint32_t cand_pos[kCandCap];   // reused as the output position list during emission
  uint32_t hist[kRoundBins];
  uint32_t warp_tot[kFinWarps];
  uint32_t res[2];
  uint32_t tiny_cnt;
  uint32_t sel_mask[1];          // really p.words entries
};
inline size_t fin_smem_bytes(int words) { return sizeof(FinShared) + size_t(words) * 4; }

__global__ void __launch_bounds__(kFinThreads, 1)
topk_finish_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t topk_smem[];
  FinShared& sh = *reinterpret_cast<FinShared*>(topk_smem);
  const int tid = threadIdx.x;
  const int r = blockIdx.x;
  DSA_KTIME_BEGIN(4);
  DSA_STAMP(r, 0);
  pdl_wait();
  pdl_launch_dependents();
  const float* row = p.logits + int64_t(r) * p.slab_stride;
  int64_t len = p.seq_lens ? int64_t(p.seq_lens[r]) : p.n;
  len = len < 0 ? 0 : (len > p.n ? p.n : len);
  const bool take_all = len <= p.topk;
  const int words = p.words, slots = p.slots;
  const uint32_t* above_mask = p.above_mask + size_t(r) * words;
  const uint32_t* slot_cnt = p.slot_cnt + size_t(r) * slots;
  const uint2* slot_cand = p.slot_cand + size_t(r) * slots * kWarpSpan;
  int32_t* out_idx = p.out_idx + int64_t(r) * p.topk;
  float* out_val = p.out_val ? p.out_val + int64_t(r) * p.topk : nullptr;
  const int32_t* imap = p.index_map ? p.index_map + int64_t(r) * p.n : nullptr;
  const uint32_t T = take_all ? 0u : __ldcg(p.header + r * 4 + 0);
  const uint32_t need = take_all ? 0u : __ldcg(p.header + r * 4 + 1);

  // ---- masks into shared memory; candidate counts of this thread's slots (contiguous = position order)
  for (int w = tid; w < words; w += 4 * kFinThreads) {  // batches of independent loads
    uint32_t t[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (w + u * kFinThreads < words) t[u] = __ldcg(above_mask + w + u * kFinThreads);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (w + u * kFinThreads < words) sh.sel_mask[w + u * kFinThreads] = t[u];
  }
  const int sper = (slots + kFinThreads - 1) / kFinThreads;
  const int s0 = min(tid * sper, slots), s1 = min(s0 + sper, slots);
  uint32_t c_cnt = 0;
  if (!take_all)
    for (int s = s0; s < s1; ++s) c_cnt += __ldcg(slot_cnt + s);
  // Prefetch into registers, before any block-wide step: this thread's first
  // kRegCand candidates (its slots are contiguous) and its second-level bin.
  constexpr int kRegCand = 8;
  uint2 rc[kRegCand];
  const bool one_slot = sper == 1 && s0 < s1;  // rows of up to 131072 logits: one slot per thread
  uint32_t cn0 = 0;
  const uint32_t h2 = take_all ? 0u : __ldcg(p.hist2 + size_t(r) * kRoundBins + (kRoundBins - 1 - tid));
  if (!take_all && one_slot) {
    cn0 = c_cnt;
    const uint2* src = slot_cand + size_t(s0) * kWarpSpan;
#pragma unroll
    for (int u = 0; u < kRegCand; ++u)
      if (uint32_t(u) < cn0) rc[u] = __ldcg(src + u);
  }
  // (!take_all implies the threshold bin holds at least one candidate: need >= 1)
  // the histogram has served every classify CTA: clear it for the next scan
  {
    uint4* gh4 = reinterpret_cast<uint4*>(p.hist + size_t(r) * kBins);
    for (int i = tid; i < kBins / 4; i += kFinThreads) gh4[i] = make_uint4(0, 0, 0, 0);
  }
  DSA_STAMP(r, 1);

  uint32_t kstar = 0xFFFFFFFFu;
  bool resolved = false;
  if (!take_all) {
    // ---- fast path: the classify kernel also histogrammed bits 19..10 of the
    // candidates, so the threshold's top 22 bits are one scan away; what shares
    // them (a handful of keys) is ranked by brute force.
    if (tid == 0) sh.tiny_cnt = 0;
    const uint32_t c1[1] = {h2};
    find_threshold_bin<kFinWarps, 1>(c1, kRoundBins, need, sh.warp_tot, sh.res);
    const uint32_t p22 = (T << 10) | sh.res[0];  // top 22 bits of the k-th largest key
    const uint32_t need2 = sh.res[1];            // how many keys with exactly these 22 bits are kept
    p.hist2[size_t(r) * kRoundBins + tid] = 0;   // re-armed (kRoundBins == kFinThreads)
    auto place = [&](uint2 kp) {
      const uint32_t k22 = kp.x >> 10;
      if (k22 > p22) {
        smem_red_or(&sh.sel_mask[kp.y >> 5], 1u << (kp.y & 31));
      } else if (k22 == p22) {
        const uint32_t at = atomicAdd(&sh.tiny_cnt, 1u);
        if (at < uint32_t(kTinyCap)) {
          sh.cand_key[at] = kp.x;
          sh.cand_pos[at] = kp.y;
        }
      }
    };
    if (one_slot) {
#pragma unroll
      for (int u = 0; u < kRegCand; ++u)
        if (uint32_t(u) < cn0) place(rc[u]);
      for (uint32_t e = kRegCand; e < cn0; ++e) place(__ldcg(slot_cand + size_t(s0) * kWarpSpan + e));
    } else {
      for (int s = s0; s < s1; ++s) {
        const uint32_t cn = __ldcg(slot_cnt + s);
        for (uint32_t e = 0; e < cn; ++e) place(__ldcg(slot_cand + size_t(s) * kWarpSpan + e));
      }
    }
    __syncthreads();
    const uint32_t n3 = sh.tiny_cnt;
    if (n3 <= uint32_t(kTinyCap)) {
      if (uint32_t(tid) < n3) {
        const uint32_t k = sh.cand_key[tid], ps = sh.cand_pos[tid];
        uint32_t rank = 0;  // keys that precede this one: larger, or equal at a lower position
        for (uint32_t j = 0; j < n3; ++j) {
          const uint32_t kj = sh.cand_key[j];
          rank += (kj > k) || (kj == k && sh.cand_pos[j] < ps);
        }
        if (rank < need2) smem_red_or(&sh.sel_mask[ps >> 5], 1u << (ps & 31));
        if (rank + 1 == need2) sh.res[0] = k;  // the k-th largest key itself
      }
      __syncthreads();
      kstar = sh.res[0];
      resolved = true;
    } else {
      // too many keys share 22 bits (massive ties): clear what the fast path set and
      // fall through to the general radix path, which handles any multiplicity
      __syncthreads();
      for (int w = tid; w < words; w += kFinThreads) sh.sel_mask[w] = __ldcg(above_mask + w);
      __syncthreads();
    }
  }
  if (!take_all && !resolved) {
    // the general path needs every thread's offset into the candidate list and the total
    uint32_t C = 0;
    const uint32_t c_off = block_exclusive_scan<kFinWarps>(c_cnt, sh.warp_tot, &C);
    const bool listed = C <= uint32_t(kCandCap);
    if (listed) {
      uint32_t at = c_off;
      for (int s = s0; s < s1; ++s) {
        const uint32_t cn = __ldcg(slot_cnt + s);
        const uint2* src = slot_cand + size_t(s) * kWarpSpan;
        for (uint32_t e = 0; e < cn; e += 4) {  // batches of independent loads
          uint2 t[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (e + u < cn) t[u] = __ldcg(src + e + u);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (e + u < cn) {
              sh.cand_key[at] = t[u].x;
              sh.cand_pos[at] = t[u].y;
              ++at;
            }
        }
      }
    }
    __syncthreads();
    DSA_STAMP(r, 2);
    // two 10-bit radix rounds on the low 20 bits of the candidates' keys
    uint32_t prefix = T << kLowBits, pmask = 0xFFFu << kLowBits, k_rem = need;
    for (int shift = 10; shift >= 0; shift -= 10) {
      sh.hist[tid] = 0;  // kRoundBins == kFinThreads
      __syncthreads();
      if (listed) {
        for (uint32_t i = tid; i < C; i += kFinThreads) {
          const uint32_t k = sh.cand_key[i];
          if ((k & pmask) == prefix) smem_red_add(&sh.hist[(k >> shift) & (kRoundBins - 1)], 1u);
        }
        DSA_STAMP(r, shift == 10 ? 10 : 12);
      } else {
        for (int s = s0; s < s1; ++s) {
          const uint32_t cn = __ldcg(slot_cnt + s);
          for (uint32_t e = 0; e < cn; ++e) {
            const uint32_t k = __ldcg(slot_cand + size_t(s) * kWarpSpan + e).x;
            if ((k & pmask) == prefix) smem_red_add(&sh.hist[(k >> shift) & (kRoundBins - 1)], 1u);
          }
        }
      }
      __syncthreads();
      const uint32_t c1[1] = {sh.hist[kRoundBins - 1 - tid]};
      find_threshold_bin<kFinWarps, 1>(c1, kRoundBins, k_rem, sh.warp_tot, sh.res);
      DSA_STAMP(r, shift == 10 ? 11 : 13);
      prefix |= sh.res[0] << shift;
      pmask |= uint32_t(kRoundBins - 1) << shift;
      k_rem = sh.res[1];
    }
    DSA_STAMP(r, 8 + 0);
    kstar = prefix;                    // the k-th largest key of the row
    const uint32_t ties_kept = k_rem;  // elements equal to it that are kept, lowest positions first
    DSA_STAMP(r, 3);
    if (listed) {
      const uint32_t lper = (C + kFinThreads - 1) / kFinThreads;  // contiguous list slice per thread
      const uint32_t l0 = min(uint32_t(tid) * lper, C), l1 = min(l0 + lper, C);
      uint32_t ties = 0;
      for (uint32_t i = l0; i < l1; ++i) ties += sh.cand_key[i] == kstar;
      uint32_t tie_rank = block_exclusive_scan<kFinWarps>(ties, sh.warp_tot, nullptr);
      DSA_STAMP(r, 9);
      for (uint32_t i = l0; i < l1; ++i) {
        const uint32_t k = sh.cand_key[i];
        bool keep = k > kstar;
        if (k == kstar) keep = tie_rank++ < ties_kept;
        if (keep) smem_red_or(&sh.sel_mask[sh.cand_pos[i] >> 5], 1u << (sh.cand_pos[i] & 31));
      }
    } else {
      uint32_t ties = 0;
      for (int s = s0; s < s1; ++s) {
        const uint32_t cn = __ldcg(slot_cnt + s);
        for (uint32_t e = 0; e < cn; ++e) ties += __ldcg(slot_cand + size_t(s) * kWarpSpan + e).x == kstar;
      }
      uint32_t tie_rank = block_exclusive_scan<kFinWarps>(ties, sh.warp_tot, nullptr);
      for (int s = s0; s < s1; ++s) {
        const uint32_t cn = __ldcg(slot_cnt + s);
        for (uint32_t e = 0; e < cn; ++e) {
          const uint2 kp = __ldcg(slot_cand + size_t(s) * kWarpSpan + e);
          bool keep = kp.x > kstar;
          if (kp.x == kstar) keep = tie_rank++ < ties_kept;
          if (keep) smem_red_or(&sh.sel_mask[kp.y >> 5], 1u << (kp.y & 31));
        }
      }
    }
  }
  __syncthreads();
  DSA_STAMP(r, 4);

  // ---- expand the selection mask into ascending positions
  const int per = (words + kFinThreads - 1) / kFinThreads;  // contiguous mask words per thread
  const int w0 = min(tid * per, words), w1 = min(w0 + per, words);
  uint32_t s_cnt = 0;
  for (int w = w0; w < w1; ++w) s_cnt += __popc(sh.sel_mask[w]);
  uint32_t total = 0;
  uint32_t pos_out = block_exclusive_scan<kFinWarps>(s_cnt, sh.warp_tot, &total);
  DSA_STAMP(r, 6);
  // a selected -inf can only appear when the row has fewer than topk finite logits
  const bool check_inf = take_all || kstar <= 0x007FFFFFu;
  const bool simple = !imap && !out_val && !check_inf;
  const bool staged = p.topk <= kCandCap;
  const float neg_inf = __int_as_float(0xff800000);
  for (int w = w0; w < w1; ++w) {
    uint32_t bits = sh.sel_mask[w];
    while (bits) {
      const int b = __ffs(bits) - 1;
      bits &= bits - 1;
      const uint32_t pos = uint32_t(w) * 32 + b;
      if (pos_out < uint32_t(p.topk)) {
        if (simple) {
          out_idx[pos_out] = int32_t(pos) + p.index_offset;
        } else if (staged) {
          sh.cand_pos[pos_out] = pos;
        } else {
          const float val = __ldcg(row + pos);
          const int32_t id = imap ? imap[pos] : int32_t(pos) + p.index_offset;
          out_idx[pos_out] = (val == neg_inf) ? p.pad : id;
          if (out_val) out_val[pos_out] = val;
        }
      }
      ++pos_out;
    }
  }
  DSA_STAMP(r, 7);
  if (!simple && staged) {
    __syncthreads();
    const uint32_t cnt = min(total, uint32_t(p.topk));
    for (uint32_t i = tid; i < cnt; i += kFinThreads) {  // independent loads
      const uint32_t pos = sh.cand_pos[i];
      const float val = __ldcg(row + pos);
      const int32_t id = imap ? imap[pos] : int32_t(pos) + p.index_offset;
      out_idx[i] = (val == neg_inf) ? p.pad : id;
      if (out_val) out_val[i] = val;
    }
  }
  for (uint32_t i = total + tid; i < uint32_t(p.topk); i += kFinThreads) {
    out_idx[i] = p.pad;
    if (out_val) out_val[i] = neg_inf;
  }
  DSA_STAMP(r, 5);
  DSA_KTIME_END(4);
}

// ------------------------------------------------------------------------------
// One launch for rows of up to kClMaxN logits: a thread-block cluster per row.
//
// Every CTA of the cluster keeps its contiguous slice of the row in shared
// memory as order-preserving keys (loaded once, 16-byte coalesced). The k-th
// largest key is found exactly by three radix levels (12 + 10 + 10 bits): a
// level's histogram is built in each CTA's shared memory, its non-zero bins are
// PUSHED into every CTA's copy (distributed-shared-memory reductions), and one
// cluster barrier later each CTA holds the whole row's histogram and finds the
// threshold bin by itself. With the key k* and the number of elements equal to
// k* that are kept, one prefix sum over the pair (larger than k*, equal to k*)
// in position order gives each kept element its slot in the ascending output:
//   slot(x) = larger_before(x) + min(equal_before(x), ties_kept)
// so ties go to the lower positions, and no candidate list, no scratch in
// global memory and no capacity limit is involved. The first level's histogram
// comes from the indexer scan when the caller passes it.
//
// The kernel runs once through its code on a handful of SMs, so its time is
// set by the barriers it crosses and by how much machine code it has to fetch:
// every loop over the keys is a rolled loop with a small body.
constexpr int kClThreads = 1024;
constexpr int kClWarps = kClThreads / 32;
constexpr int kClMaxGroups = 8;                               // 16-byte groups of keys per thread
constexpr int kClMaxCtas = 16;                                // 8 is the portable cluster size, 16 needs an opt-in
constexpr int64_t kClMaxN = int64_t(8) * kClThreads * 4 * kClMaxGroups;  // 262144 (with the portable cluster size)

struct ClShared {
  uint32_t hist1[kBins];        // whole row, complete after the level's cluster barrier
  uint32_t local1[kBins];       // this CTA's part
  uint32_t hist2[kRoundBins];
  uint32_t local2[kRoundBins];
  uint32_t hist3[kRoundBins];
  uint32_t local3[kRoundBins];
  uint32_t warp_tot[kClWarps];
  uint32_t cta_tot[kClMaxCtas];  // (equal << 16 | larger) of every CTA of the cluster
  uint32_t pad_[16];
  uint4 keys[1];                 // really groups * kClThreads entries: this CTA's slice in position order
};
inline size_t cl_smem_bytes(int groups) { return offsetof(ClShared, keys) + size_t(groups) * kClThreads * 16; }

// Adds 1 to h[digit] for the lanes with `pred`. The lanes that share the first such
// lane's digit add once, so a row of equal logits does not serialise on one address.
__device__ __forceinline__ void hist_add_warp(uint32_t* h, bool pred, uint32_t digit) {
  const uint32_t m = __ballot_sync(0xffffffffu, pred);
  if (m == 0) return;
  const int leader = __ffs(m) - 1;
  const uint32_t first = __shfl_sync(0xffffffffu, digit, leader);
  const uint32_t same = __ballot_sync(0xffffffffu, pred && digit == first);
  if (pred) {
    if (digit != first) smem_red_add(&h[digit], 1u);
    else if (int(threadIdx.x & 31) == leader) smem_red_add(&h[digit], __popc(same));
  }
}

// Pushes this CTA's non-zero bins of `local` (one per thread, or four when kWide)
// into `whole` of every CTA of the cluster.
template <bool kWide>
__device__ __forceinline__ void push_bins(const uint32_t* local, uint32_t* whole, uint32_t n_ctas) {
  const int tid = threadIdx.x;
  if (kWide) {
    const uint4 x = reinterpret_cast<const uint4*>(local)[tid];
    if (x.x | x.y | x.z | x.w) {
      const uint32_t a = smem_u32(whole + 4 * tid);
#pragma unroll 1
      for (uint32_t cc = 0; cc < n_ctas; ++cc) {
        const uint32_t ra = cluster_map(a, cc);
        if (x.x) cluster_red_add(ra, x.x);
        if (x.y) cluster_red_add(ra + 4, x.y);
        if (x.z) cluster_red_add(ra + 8, x.z);
        if (x.w) cluster_red_add(ra + 12, x.w);
      }
    }
  } else {
    const uint32_t x = local[tid];
    if (x) {
      const uint32_t a = smem_u32(whole + tid);
#pragma unroll 1
      for (uint32_t cc = 0; cc < n_ctas; ++cc) cluster_red_add(cluster_map(a, cc), x);
    }
  }
}

// Bin holding the k-th largest element of a histogram of NB bins in shared memory
// (searched from the top bin down), and the element's rank inside that bin; the
// result is returned to every thread. `own` are the counts of this thread's
// NB / 1024 bins, highest first: thread t owns the bins just below NB - t * NB / 1024.
// One block barrier: each warp sums its 32 threads' bins, every warp scans the 32
// warp sums, then reads the target warp's bins itself.
template <int NB>
__device__ __forceinline__ void find_kth_bin(const uint32_t* h, const uint32_t (&own)[NB / kClThreads], uint32_t k,
                                             uint32_t* warp_tot, uint32_t& bin, uint32_t& rank) {
  constexpr int PER = NB / kClThreads;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t s = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) s += own[i];
  const uint32_t wsum = __reduce_add_sync(0xffffffffu, s);
  if (lane == 0) warp_tot[warp] = wsum;
  __syncthreads();
  const uint32_t wt = warp_tot[lane];
  uint32_t inc = wt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += up;
  }
  const uint32_t hit = __ballot_sync(0xffffffffu, inc >= k);
  const int W = hit ? __ffs(hit) - 1 : 31;
  const uint32_t k2 = k - __shfl_sync(0xffffffffu, inc - wt, W);
  const int top = NB - 1 - (W * 32 + lane) * PER;  // highest bin of this lane inside warp W's range
  uint32_t c[PER];
  uint32_t s2 = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    c[i] = h[top - i];
    s2 += c[i];
  }
  uint32_t inc2 = s2;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, inc2, o);
    if (lane >= o) inc2 += up;
  }
  const uint32_t hit2 = __ballot_sync(0xffffffffu, inc2 >= k2);
  const int L = hit2 ? __ffs(hit2) - 1 : 31;
  uint32_t running = inc2 - s2, b = uint32_t(top), rk = 1;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    if (running < k2 && k2 <= running + c[i]) {
      b = uint32_t(top - i);
      rk = k2 - running;
    }
    running += c[i];
  }
  bin = __shfl_sync(0xffffffffu, b, L);
  rank = __shfl_sync(0xffffffffu, rk, L);
}

__global__ void __launch_bounds__(kClThreads, 1)
topk_cluster_kernel(const Params p, const int groups) {
  extern __shared__ __align__(16) uint8_t topk_smem[];
  ClShared& sh = *reinterpret_cast<ClShared*>(topk_smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = blockIdx.y;
  const uint32_t c = cluster_cta_rank(), C = cluster_num_ctas();
  const int stamp_cta = 512 + r * int(C) + int(c);
  DSA_KTIME_BEGIN(1);
  DSA_STAMP(stamp_cta, 0);
  // ---- input-free set-up: clear the histograms, then tell the cluster they are clear
  {
    uint4* z = reinterpret_cast<uint4*>(&sh);
    constexpr int kZero16 = int(offsetof(ClShared, keys) / 16);
    for (int i = tid; i < kZero16; i += kClThreads) z[i] = make_uint4(0, 0, 0, 0);
  }
  cluster_arrive();
  pdl_wait();
  pdl_launch_dependents();
  const float* row = p.logits + int64_t(r) * p.slab_stride;
  int64_t len = p.seq_lens ? int64_t(p.seq_lens[r]) : p.n;
  len = len < 0 ? 0 : (len > p.n ? p.n : len);
  const bool take_all = len <= p.topk;
  const bool have_hist = p.hist != nullptr;

  // ---- this CTA's slice as order-preserving keys (0 = not a visible position); thread
  // (warp, lane) owns the 16-byte groups j * 32 + lane of its warp's run of `groups` * 128 positions
  const int64_t base = int64_t(c) * (kClThreads * 4 * groups) + int64_t(warp) * (128 * groups) + lane * 4;
  uint4* my_keys = sh.keys + warp * groups * 32 + lane;
  {
    // every load of the slice is issued before the first key is stored
    const bool vec = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    float4 v[kClMaxGroups];
#pragma unroll
    for (int j = 0; j < kClMaxGroups; ++j) {
      const int64_t p0 = base + j * 128;
      v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < groups && p0 < len) {
        if (vec && p0 + 4 <= p.n) {
          v[j] = *reinterpret_cast<const float4*>(row + p0);
        } else {
          v[j].x = row[p0];
          if (p0 + 1 < len) v[j].y = row[p0 + 1];
          if (p0 + 2 < len) v[j].z = row[p0 + 2];
          if (p0 + 3 < len) v[j].w = row[p0 + 3];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kClMaxGroups; ++j) {
      if (j < groups) {
        const int64_t p0 = base + j * 128;
        uint4 k;
        k.x = p0 + 0 < len ? ordered_key(v[j].x) : 0u;
        k.y = p0 + 1 < len ? ordered_key(v[j].y) : 0u;
        k.z = p0 + 2 < len ? ordered_key(v[j].z) : 0u;
        k.w = p0 + 3 < len ? ordered_key(v[j].w) : 0u;
        my_keys[j * 32] = k;
      }
    }
  }
  DSA_STAMP(stamp_cta, 1);

  uint32_t kstar = 0, ties_kept = 0;  // short rows keep every visible position: all keys exceed 0
  if (!take_all) {
    // ---- level 1: top 12 key bits
    uint32_t own1[4];
    if (have_hist) {  // from the scan: every CTA reads all of it (this thread's bins, highest first)
      const uint4 h1 = __ldcg(reinterpret_cast<const uint4*>(p.hist + size_t(r) * kBins) + (kClThreads - 1 - tid));
      reinterpret_cast<uint4*>(sh.hist1)[kClThreads - 1 - tid] = h1;
      own1[0] = h1.w, own1[1] = h1.z, own1[2] = h1.y, own1[3] = h1.x;
    } else {
#pragma unroll 1
      for (int j = 0; j < groups; ++j) {
        const uint4 k = my_keys[j * 32];
        hist_add_warp(sh.local1, k.x != 0u, k.x >> kLowBits);
        hist_add_warp(sh.local1, k.y != 0u, k.y >> kLowBits);
        hist_add_warp(sh.local1, k.z != 0u, k.z >> kLowBits);
        hist_add_warp(sh.local1, k.w != 0u, k.w >> kLowBits);
      }
      __syncthreads();
      cluster_wait();  // every CTA of the cluster has cleared its histograms: remote adds may start
      push_bins<true>(sh.local1, sh.hist1, C);
      cluster_arrive();
      cluster_wait();
      const uint4 h1 = reinterpret_cast<const uint4*>(sh.hist1)[kClThreads - 1 - tid];
      own1[0] = h1.w, own1[1] = h1.z, own1[2] = h1.y, own1[3] = h1.x;
    }
    uint32_t T, need;
    find_kth_bin<kBins>(sh.hist1, own1, uint32_t(p.topk), sh.warp_tot, T, need);
    DSA_STAMP(stamp_cta, 2);
    // ---- level 2: bits 19..10 of the keys in bin T
#pragma unroll 1
    for (int j = 0; j < groups; ++j) {
      const uint4 k = my_keys[j * 32];
      hist_add_warp(sh.local2, (k.x >> kLowBits) == T && k.x != 0u, (k.x >> 10) & (kRoundBins - 1));
      hist_add_warp(sh.local2, (k.y >> kLowBits) == T && k.y != 0u, (k.y >> 10) & (kRoundBins - 1));
      hist_add_warp(sh.local2, (k.z >> kLowBits) == T && k.z != 0u, (k.z >> 10) & (kRoundBins - 1));
      hist_add_warp(sh.local2, (k.w >> kLowBits) == T && k.w != 0u, (k.w >> 10) & (kRoundBins - 1));
    }
    __syncthreads();
    if (have_hist) cluster_wait();  // (see above; without the scan's histogram it was taken at level 1)
    push_bins<false>(sh.local2, sh.hist2, C);
    cluster_arrive();
    cluster_wait();
    // every CTA has read the scan's histogram by now: re-arm it for the next scan
    if (have_hist && c == 0)
      reinterpret_cast<uint4*>(p.hist + size_t(r) * kBins)[tid] = make_uint4(0, 0, 0, 0);
    uint32_t d2, need2;
    {
      const uint32_t own2[1] = {sh.hist2[kRoundBins - 1 - tid]};
      find_kth_bin<kRoundBins>(sh.hist2, own2, need, sh.warp_tot, d2, need2);
    }
    const uint32_t p22 = (T << 10) | d2;
    DSA_STAMP(stamp_cta, 3);
    // ---- level 3: the low 10 bits of the keys that share those 22 bits
#pragma unroll 1
    for (int j = 0; j < groups; ++j) {
      const uint4 k = my_keys[j * 32];
      hist_add_warp(sh.local3, (k.x >> 10) == p22, k.x & (kRoundBins - 1));
      hist_add_warp(sh.local3, (k.y >> 10) == p22, k.y & (kRoundBins - 1));
      hist_add_warp(sh.local3, (k.z >> 10) == p22, k.z & (kRoundBins - 1));
      hist_add_warp(sh.local3, (k.w >> 10) == p22, k.w & (kRoundBins - 1));
    }
    __syncthreads();
    push_bins<false>(sh.local3, sh.hist3, C);
    cluster_arrive();
    cluster_wait();
    uint32_t d3;
    {
      const uint32_t own3[1] = {sh.hist3[kRoundBins - 1 - tid]};
      find_kth_bin<kRoundBins>(sh.hist3, own3, need2, sh.warp_tot, d3, ties_kept);
    }
    kstar = (p22 << 10) | d3;  // the k-th largest key of the row; ties_kept of its copies are kept
    DSA_STAMP(stamp_cta, 4);
  } else {
    cluster_wait();
    if (have_hist && c == 0)
      reinterpret_cast<uint4*>(p.hist + size_t(r) * kBins)[tid] = make_uint4(0, 0, 0, 0);
  }

  // ---- (larger, equal) counts, packed equal << 16 | larger: this warp's, then the warps and CTAs before it
  auto count4 = [&](const uint4& k) -> uint32_t {
    return (k.x > kstar ? 1u : 0u) + (k.y > kstar ? 1u : 0u) + (k.z > kstar ? 1u : 0u) + (k.w > kstar ? 1u : 0u) +
           (((k.x == kstar ? 1u : 0u) + (k.y == kstar ? 1u : 0u) + (k.z == kstar ? 1u : 0u) + (k.w == kstar ? 1u : 0u)) << 16);
  };
  {
    uint32_t tot = 0;
#pragma unroll 1
    for (int j = 0; j < groups; ++j) tot += count4(my_keys[j * 32]);
    if (take_all) tot &= 0xFFFFu;  // key 0 marks the invisible positions, they are not ties
    const uint32_t wsum = __reduce_add_sync(0xffffffffu, tot);  // at most 1024 of each kind per warp
    __syncthreads();  // earlier readers of warp_tot are done
    if (lane == 0) sh.warp_tot[warp] = wsum;
  }
  __syncthreads();
  uint32_t before_warp, cta_sum;
  {
    const uint32_t w = sh.warp_tot[lane];
    uint32_t inc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += up;
    }
    before_warp = __shfl_sync(0xffffffffu, inc - w, warp);
    cta_sum = __shfl_sync(0xffffffffu, inc, 31);  // at most 32768 of each kind per CTA
  }
  if (tid < int(C)) cluster_st(cluster_map(smem_u32(&sh.cta_tot[c]), uint32_t(tid)), cta_sum);
  cluster_arrive();
  cluster_wait();
  uint32_t gt_before = before_warp & 0xFFFFu, eq_before = before_warp >> 16, gt_total = 0, eq_total = 0;
#pragma unroll 1
  for (uint32_t cc = 0; cc < C; ++cc) {
    const uint32_t t = sh.cta_tot[cc];
    if (cc < c) {
      gt_before += t & 0xFFFFu;
      eq_before += t >> 16;
    }
    gt_total += t & 0xFFFFu;
    eq_total += t >> 16;
  }
  DSA_STAMP(stamp_cta, 5);

  // ---- emit: ascending positions, ties to the lower position
  int32_t* out_idx = p.out_idx + int64_t(r) * p.topk;
  float* out_val = p.out_val ? p.out_val + int64_t(r) * p.topk : nullptr;
  const int32_t* imap = p.index_map ? p.index_map + int64_t(r) * p.n : nullptr;
  const uint32_t kNegInfKey = 0x007FFFFFu;  // ordered_key(-inf)
  const uint32_t topk_u = uint32_t(p.topk);
#pragma unroll 1
  for (int j = 0; j < groups; ++j) {
    const uint4 k4 = my_keys[j * 32];
    uint32_t cnt = count4(k4);
    if (take_all) cnt &= 0xFFFFu;
    if (__ballot_sync(0xffffffffu, cnt != 0u) == 0u) continue;  // nothing of this group is near the cutoff
    uint32_t inc = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += up;
    }
    uint32_t g = gt_before + ((inc - cnt) & 0xFFFFu);
    uint32_t q = eq_before + ((inc - cnt) >> 16);
    const uint32_t ks[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t k = ks[e];
      const bool gt = k > kstar;
      const bool eq = !take_all && k == kstar;
      if (gt || (eq && q < ties_kept)) {
        const uint32_t slot = g + min(q, ties_kept);
        if (slot < topk_u) {
          const int64_t pos = base + j * 128 + e;
          const int32_t id = imap ? imap[pos] : int32_t(pos) + p.index_offset;
          out_idx[slot] = (k == kNegInfKey) ? p.pad : id;
          if (out_val) out_val[slot] = __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
        }
      }
      g += gt ? 1u : 0u;
      q += eq ? 1u : 0u;
    }
    const uint32_t wj = __shfl_sync(0xffffffffu, inc, 31);  // this group's total over the warp
    gt_before += wj & 0xFFFFu;
    eq_before += wj >> 16;
  }
  const uint32_t total = gt_total + min(eq_total, ties_kept);
  const float neg_inf = __int_as_float(0xff800000);
  for (uint32_t i = total + c * kClThreads + tid; i < topk_u; i += C * kClThreads) {
    out_idx[i] = p.pad;
    if (out_val) out_val[i] = neg_inf;
  }
  DSA_STAMP(stamp_cta, 6);
  DSA_KTIME_END(1);
}

}  // namespace topk
}  // namespace dsa
