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
constexpr int kMaxRanks = 8;                    // GPUs of one candidate exchange

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
  // ---- candidate exchange between the GPUs of a sequence-sharded indexer (cluster kernel only)
  // Push side (n_dest > 0): the selection of row r goes, as (index, logit), into slot `src_rank`
  // of every rank's gather buffers [2 parities][R][n_dest][topk], then flag word
  // dest_flag[d][r] of every rank d gets this row's step number.
  int n_dest;
  int src_rank;
  int32_t* dest_idx[kMaxRanks];
  float* dest_val[kMaxRanks];
  uint32_t* dest_flag[kMaxRanks];  // this rank's [R] flag words inside rank d's flag array
  uint32_t* sent;                  // [R] steps pushed so far (local)
  // Merge side (n_src > 0): logits / index_map are this rank's gather buffers; the kernel first
  // waits, bounded, until wait_flags[s * R + r] of every source s reaches this row's next step.
  int n_src;
  const uint32_t* wait_flags;      // [n_src][R], written by the sources
  uint32_t* seen;                  // [R] steps merged so far (local)
  unsigned long long wait_limit_ns;
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
// One launch for rows of up to kClMaxN logits: a thread-block cluster per row (1-8 CTAs up to
// 131072 logits; 16 CTAs, a cluster size the kernel opts into, up to 262144).
//
// Each CTA of the cluster owns a contiguous slice of the row (brought into shared
// memory by one bulk copy) and looks at every logit of it exactly once. With the
// threshold bin T of the 12-bit histogram (the indexer scan's, when the caller
// passes it) one sweep over the slice leaves, per thread, a 32-bit mask of the
// positions that are certainly kept (bin above T) and one of the few candidates
// in bin T. Everything after that touches only mask words and candidates:
//   * the usual case: every CTA sends its candidates as (key, place) pairs, with
//     its 128-bin histogram of their next 7 key bits and its count of certainly
//     kept logits, to every CTA of the cluster (distributed-shared-memory
//     stores). ONE cluster barrier later each CTA holds the whole candidate
//     list: it searches the summed histograms for the level-2 bin, collects the
//     handful of candidates that share the k-th key's top 19 bits, ranks them by
//     comparison (larger key first, lower position first among equal keys), and
//     knows from the tables and the ranks how many candidates every CTA keeps:
//     no further exchange;
//   * a CTA with more candidates than its region of the list holds (8192 / C), or more than kSurvCap candidates
//     sharing the 19 bits (rows with many equal logits): two more radix levels
//     (7 + 13 bits) as histograms PUSHED into every CTA (distributed-shared-
//     memory reductions), a cluster barrier after each, candidates equal to k*
//     in a tie mask, the CTAs' totals exchanged behind a last barrier;
//   * one prefix sum over the pair (kept, tie) in position order gives each
//     element its slot in the ascending output:
//       slot(x) = kept_before(x) + min(ties_before(x), ties_kept)
//     so ties go to the lower positions.
// No scratch in global memory, no wait on another launch.
//
// Cost model that shaped it: the kernel is a chain of short dependent phases, each
// paced by instruction and shared-memory latency, not by throughput. A CTA's
// warps share four issue ports, shared-memory atomics retire about one per cycle
// per SM (so nothing adds per element, only per candidate), a cluster barrier
// costs about 1500 cycles where it stands, a block barrier about 100. Hence 512
// threads, one sweep without warp votes, a single cluster barrier on the usual
// path, warp reductions instead of scans where only a total is needed, and
// whatever needs no data of the previous launch (clearing shared memory, the
// first cluster arrival) ahead of the dependency wait.
constexpr int kClThreads = 512;
constexpr int kClWarps = kClThreads / 32;
constexpr int kClMaxKeys = 32;                                // logits per thread (= mask words per warp)
constexpr int kClMaxCtas = 8;                                 // portable cluster size: rows of up to 131072 logits
constexpr int kClMaxCtasBig = 16;                             // non-portable cluster size (an opt-in of the kernel): up to 262144
constexpr int64_t kClPortableN = int64_t(kClMaxCtas) * kClThreads * kClMaxKeys;   // 131072
constexpr int64_t kClMaxN = int64_t(kClMaxCtasBig) * kClThreads * kClMaxKeys;     // 262144
constexpr int kL2Bits = 7, kL2Bins = 1 << kL2Bits;            // key bits 19..13
constexpr int kL3Bits = 13, kL3Bins = 1 << kL3Bits;           // key bits 12..0
constexpr int kWarpKeys = 32 * kClMaxKeys;                    // 1024: a warp's share of the slice
constexpr int kListTotal = 8192;                              // list entries per CTA image: a region of kListTotal / C per CTA of the cluster (more candidates in one CTA: histograms)
constexpr int kSurvCap = 256;                                 // candidates ranked by comparison (else: histograms)

template <int kMaxC>
struct ClSharedT {
  uint32_t hist1[kBins];         // level 1: whole row (copy of the scan's, or pushed by the CTAs)
  uint32_t hist3[kL3Bins];       // level 3: whole row, pushed; stored as swizzled_bin<kL3Bins> says
  uint32_t hist2[kL2Bins];       // level 2: whole row, pushed
  uint32_t local2[kL2Bins];      // level 2: this CTA's part
  uint32_t cand_kept[kMaxC];  // per CTA of the cluster: its candidates that are kept (list path)
  uint32_t surv_n;               // entries of surv[]
  uint32_t list_n;               // this CTA's candidates (slots handed out in its region of the list)
  uint32_t above_n;              // this CTA's certainly kept logits
  uint32_t pad0;
  uint32_t kept[kClWarps][kClMaxKeys];   // bit (w, i, l): position w * 32 * nk + i * 32 + l of the slice is kept
  uint32_t ties[kClWarps][kClMaxKeys];   // same, for the elements equal to k*
  uint32_t warp_tot[kClWarps];
  uint32_t warp_base[kClWarps];
  uint32_t cta_tot[kMaxC];  // (ties << 16 | kept) of every CTA of the cluster
  uint32_t cnts[kMaxC];     // (certainly kept << 16 | candidates) of every CTA, pushed with the list
  uint32_t res[4];
  uint64_t surv[kSurvCap + 4];   // key << 32 | ~place of the candidates sharing the k-th key's top 19 bits (+ 4 zeros)
  alignas(16) uint32_t tbl[kMaxC][kL2Bins];  // level 2: every CTA's histogram of its candidates, pushed
  uint64_t load_bar;                       // mbarrier of the slice's bulk copy
  uint2 list[kListTotal];                  // (key, place) of every CTA's candidates, region c at c * kListTotal / C, pushed; place =
                                           // CTA << 14 | warp << 10 | word << 5 | bit orders like the position
  alignas(128) uint32_t bits[kClWarps][kWarpKeys];  // (a bulk copy's destination must be 16-byte aligned)      // the slice's raw logits: word (w, i * 32 + l) is thread (w, l)'s i-th
};
using ClShared = ClSharedT<kClMaxCtas>;
using ClSharedBig = ClSharedT<kClMaxCtasBig>;
static_assert(kL3Bins >= kBins, "hist3 doubles as the local level-1 histogram");
static_assert(offsetof(ClShared, bits) % 128 == 0 && offsetof(ClShared, load_bar) % 8 == 0 &&
              offsetof(ClSharedBig, bits) % 128 == 0 && offsetof(ClSharedBig, load_bar) % 8 == 0,
              "alignment of the copy target and its barrier");

// Adds `amount` of 1s to h[digit] for the lanes with `pred`. The lanes that share the first
// such lane's digit add once, so a row of equal logits does not serialise on one address.
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
// The same into `whole` of every CTA of the cluster.
__device__ __forceinline__ void hist_push_warp(uint32_t* whole, bool pred, uint32_t digit, uint32_t n_ctas) {
  const uint32_t m = __ballot_sync(0xffffffffu, pred);
  if (m == 0) return;
  const int leader = __ffs(m) - 1;
  const uint32_t first = __shfl_sync(0xffffffffu, digit, leader);
  const uint32_t same = __ballot_sync(0xffffffffu, pred && digit == first);
  uint32_t add = 0;
  if (pred) add = digit != first ? 1u : (int(threadIdx.x & 31) == leader ? uint32_t(__popc(same)) : 0u);
  if (add) {
    if (n_ctas == 1) {
      smem_red_add(whole + digit, add);
    } else {
      const uint32_t a = smem_u32(whole + digit);
#pragma unroll 1
      for (uint32_t cc = 0; cc < n_ctas; ++cc) cluster_red_add(cluster_map(a, cc), add);
    }
  }
}

// Inclusive prefix sum over the lanes of a warp.
__device__ __forceinline__ uint32_t warp_inclusive_scan(uint32_t v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += up;
  }
  return v;
}

// Bin holding the k-th largest element of the NB-bin histogram h (shared memory, searched
// from the top bin down) and the element's rank inside that bin, left in res[0], res[1] for
// every thread. Thread t owns the PER = NB / kClThreads bins just below NB - PER t (for
// NB < kClThreads: one bin for the first NB threads). All warps prefix-sum their threads' bin
// sums at once; after a barrier every warp prefix-sums the 16 warp totals, the warp that holds
// the k-th element picks its thread by ballot and that thread walks its own bins (registers);
// a second barrier publishes the result. The dependent chain is two warp scans long.
// Where bin b of an NB-bin histogram lives when it is stored for conflict-free reads by
// find_kth_bin<NB, true>: bins are numbered from the top (rb = NB - 1 - b), thread t owns
// rb in [PER t, PER (t + 1)) and its 16-byte chunk j sits at chunk index j * kClThreads + t.
template <int NB>
__device__ __forceinline__ uint32_t swizzled_bin(uint32_t b) {
  constexpr uint32_t PERC = NB / kClThreads / 4;  // 16-byte chunks per thread
  const uint32_t rb = uint32_t(NB - 1) - b, q = rb >> 2;
  return (((q % PERC) * kClThreads + q / PERC) << 2) | (rb & 3u);
}

// The same for a 128-bin histogram (16-byte aligned), by one warp: lane l owns bins
// 127 - 4 l down to 124 - 4 l; one warp scan, one barrier.
template <int NB>
__device__ __forceinline__ void find_kth_bin_warp(const uint32_t* h, uint32_t k, uint32_t* res) {
  static_assert(NB == 128, "four bins per lane");
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const uint4 x = reinterpret_cast<const uint4*>(h)[31 - lane];
    const uint32_t cnt[4] = {x.w, x.z, x.y, x.x};  // highest bin first
    const uint32_t s = cnt[0] + cnt[1] + cnt[2] + cnt[3];
    const uint32_t inc = warp_inclusive_scan(s);
    const uint32_t hit = __ballot_sync(0xffffffffu, inc >= k);
    if (hit == 0u) {
      if (lane == 0) res[0] = 0u, res[1] = 1u;  // k exceeds the total (never with a consistent caller)
    } else if (lane == __ffs(hit) - 1) {
      uint32_t running = inc - s, b = 0, rk = 1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (running < k && k <= running + cnt[i]) {
          b = uint32_t(i);
          rk = k - running;
        }
        running += cnt[i];
      }
      res[0] = uint32_t(NB - 1 - 4 * lane) - b;
      res[1] = rk;
    }
  }
  __syncthreads();
}

// The same over the sum of n_tbl 128-bin tables that lie one after the other; res[2] gets the
// size of the bin found.
template <int kMaxC>
__device__ __forceinline__ void find_kth_bin_tables(const uint32_t* tbl, int n_tbl, uint32_t k, uint32_t* res) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    uint32_t cnt[4] = {0u, 0u, 0u, 0u};  // highest bin first
#pragma unroll
    for (int t = 0; t < kMaxC; ++t) {
      if (t < n_tbl) {
        const uint4 x = reinterpret_cast<const uint4*>(tbl + t * kL2Bins)[31 - lane];
        cnt[0] += x.w, cnt[1] += x.z, cnt[2] += x.y, cnt[3] += x.x;
      }
    }
    const uint32_t s = cnt[0] + cnt[1] + cnt[2] + cnt[3];
    const uint32_t inc = warp_inclusive_scan(s);
    const uint32_t hit = __ballot_sync(0xffffffffu, inc >= k);
    if (hit == 0u) {
      if (lane == 0) res[0] = 0u, res[1] = 1u, res[2] = 0u;  // k exceeds the total (never with a consistent caller)
    } else if (lane == __ffs(hit) - 1) {
      uint32_t running = inc - s, b = 0, rk = 1, size = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (running < k && k <= running + cnt[i]) {
          b = uint32_t(i);
          rk = k - running;
          size = cnt[i];
        }
        running += cnt[i];
      }
      res[0] = uint32_t(kL2Bins - 1 - 4 * lane) - b;
      res[1] = rk;
      res[2] = size;
    }
  }
  __syncthreads();
}

template <int NB, int PER>
__device__ __forceinline__ void find_kth_in_registers(const uint32_t (&cnt)[PER], uint32_t k, uint32_t* warp_tot, uint32_t* res);

template <int NB, bool kSwz = false>
__device__ __forceinline__ void find_kth_bin(const uint32_t* h, uint32_t k, uint32_t* warp_tot, uint32_t* res) {
  constexpr int PER = NB >= kClThreads ? NB / kClThreads : 1;
  const int tid = threadIdx.x;
  uint32_t cnt[PER];  // this thread's bins, highest first
  if (kSwz) {
    static_assert(!kSwz || PER >= 4, "the interleaved layout is for at least one chunk per thread");
#pragma unroll
    for (int i = 0; i < PER / 4; ++i) {
      const uint4 x = reinterpret_cast<const uint4*>(h)[i * kClThreads + tid];
      cnt[4 * i + 0] = x.x, cnt[4 * i + 1] = x.y, cnt[4 * i + 2] = x.z, cnt[4 * i + 3] = x.w;
    }
  } else if (PER >= 4) {
    const uint4* mine = reinterpret_cast<const uint4*>(h + NB - PER * (tid + 1));
#pragma unroll
    for (int i = 0; i < PER / 4; ++i) {
      const uint4 x = mine[PER / 4 - 1 - i];
      cnt[4 * i + 0] = x.w, cnt[4 * i + 1] = x.z, cnt[4 * i + 2] = x.y, cnt[4 * i + 3] = x.x;
    }
  } else {
    cnt[0] = tid < NB ? h[NB - 1 - tid] : 0u;
  }
  find_kth_in_registers<NB, PER>(cnt, k, warp_tot, res);
}

// The search proper: thread t holds its PER bins (highest first) in registers.
template <int NB, int PER>
__device__ __forceinline__ void find_kth_in_registers(const uint32_t (&cnt)[PER], uint32_t k, uint32_t* warp_tot, uint32_t* res) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t s = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) s += cnt[i];
  const uint32_t wsum = __reduce_add_sync(0xffffffffu, s);
  if (lane == 0) warp_tot[warp] = wsum;
  if (tid == 0) res[0] = 0u, res[1] = 1u;  // stays if k exceeds the histogram's total (never with a consistent caller)
  __syncthreads();
  const uint32_t wt = lane < kClWarps ? warp_tot[lane] : 0u;
  const uint32_t before_warp = __reduce_add_sync(0xffffffffu, lane < warp ? wt : 0u);
  if (before_warp < k && k - before_warp <= wsum) {  // this warp holds the k-th element: only it scans
    const uint32_t k2 = k - before_warp;
    const uint32_t inc = warp_inclusive_scan(s);
    const uint32_t hit = __ballot_sync(0xffffffffu, inc >= k2);
    if (lane == __ffs(hit) - 1) {
      uint32_t running = inc - s, b = 0, rk = 1;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        if (running < k2 && k2 <= running + cnt[i]) {
          b = uint32_t(i);
          rk = k2 - running;
        }
        running += cnt[i];
      }
      res[0] = uint32_t(NB - 1 - tid * PER) - b;
      res[1] = rk;
    }
  }
  __syncthreads();
}

// Barrier over the whole cluster (release / acquire), or over the CTA alone when the cluster
// is a single CTA: rows of up to 16384 logits run without any cluster operation.
__device__ __forceinline__ void cluster_sync_all(bool solo) {
  if (solo) {
    __syncthreads();
  } else {
    cluster_arrive();
    cluster_wait();
  }
}

// kPlain = the decode step's call: the scan's histogram is there, no candidate exchange, no index
// map, indices only. It is the same code with those features compiled out, so that the kernel
// every decode step runs is small (it alternates with three other kernels on the same SMs, and
// its time in a step follows its size; alone, both forms take the same time).
template <bool kPlain, int kMaxC = kClMaxCtas>
__global__ void __launch_bounds__(kClThreads, 1)
topk_cluster_kernel(const Params p, const int nk) {
  extern __shared__ __align__(128) uint8_t topk_cl_smem[];
  using Shared = ClSharedT<kMaxC>;
  Shared& sh = *reinterpret_cast<Shared*>(topk_cl_smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = blockIdx.y;
  const uint32_t c = cluster_cta_rank(), C = cluster_num_ctas();
  const bool solo = C == 1;
  const int stamp_cta = 512 + r * int(C) + int(c);
  (void)stamp_cta;  // (used by the tracing build only)
  DSA_KTIME_BEGIN(1);
  DSA_STAMP(stamp_cta, 0);
  const bool have_hist = kPlain || p.hist != nullptr;
  const int n_src = kPlain ? 0 : p.n_src, n_dest = kPlain ? 0 : p.n_dest;
  const int32_t* const index_map = kPlain ? nullptr : p.index_map;
  if (tid == 0) {
    mbar_init(smem_u32(&sh.load_bar), 1);
    mbar_fence_init();
  }
  // ---- before anything of the previous launch is needed: clear what is accumulated into and tell
  // the cluster it is clear (shared memory only, so this runs while the previous launch drains)
  {
    static_assert(offsetof(Shared, warp_tot) % 16 == 0, "the cleared part is whole 16-byte words");
    constexpr int kZero16 = int(offsetof(Shared, warp_tot) / 16);  // the histograms and both masks
    uint4* z = reinterpret_cast<uint4*>(&sh);
    for (int i = (have_hist ? kBins / 4 : 0) + tid; i < kZero16; i += kClThreads)  // (a given hist1 is overwritten)
      z[i] = make_uint4(0, 0, 0, 0);
  }
  if (!solo) cluster_arrive();
  // Dependents are released before the wait: a dependent of the ordinary kind waits for this grid
  // anyway, and one that runs beside this kernel (the lagged schedule's attention, a host copy)
  // can then start while the scan before this kernel is still draining.
  pdl_launch_dependents();
  pdl_wait();
  DSA_STAMP(stamp_cta, 15);
  const int R = int(gridDim.y);
  // ---- loads. The CTA's slice (positions slice_base .. + span) comes into shared memory as it
  // lies in global memory, by one bulk copy when the row is 16-byte aligned. Thread (warp, lane)
  // then owns positions warp_off + i * 32 + lane of the slice, i < nk: conflict-free reads, and
  // (i, lane) is ascending position order. The copy and the histogram loads do not wait for the
  // row's length: what lies past it is overwritten after the copy has landed.
  const int span = kClThreads * nk;
  const int slice_base = int(c) * span;
  const int warp_off = warp * (32 * nk);
  uint32_t* flat = &sh.bits[0][0];
  const int avail = max(0, min(int(p.n), slice_base + span) - slice_base);  // of the slice, inside the buffer
  const float* row = p.logits + int64_t(r) * p.slab_stride;
  // (candidates another GPU wrote are read with plain loads, not by the copy engine)
  const bool bulk = avail > 0 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0 && n_src == 0;
  const int bulk_elems = bulk ? (avail & ~3) : 0;
  const uint32_t bar = smem_u32(&sh.load_bar);
  if (tid == 0 && bulk_elems > 0) {
    mbar_arrive_expect_tx(bar, uint32_t(bulk_elems) * 4u);
    bulk_g2s(smem_u32(flat), row + slice_base, uint32_t(bulk_elems) * 4u, bar);
  }
  uint4 h1a = make_uint4(0, 0, 0, 0), h1b = h1a;
  if (have_hist) {  // this thread's 8 bins of the scan's histogram
    const uint4* gh = reinterpret_cast<const uint4*>(p.hist + size_t(r) * kBins + (kBins - 8 * (tid + 1)));
    h1a = __ldcg(gh);
    h1b = __ldcg(gh + 1);
  }
  // Candidate exchange: this row's step number picks one of the two gather buffers, so that a
  // rank already pushing step e + 1 does not overwrite what a slower rank still merges for step e.
  const uint32_t step = n_dest > 0 ? p.sent[r] + 1u : (n_src > 0 ? p.seen[r] + 1u : 0u);
  const int64_t gather_row = int64_t(step & 1u) * R + r;  // (= r outside an exchange)
  if (n_src > 0) row = p.logits + gather_row * p.slab_stride;
  int64_t len64 = p.seq_lens ? int64_t(p.seq_lens[r]) : p.n;
  len64 = len64 < 0 ? 0 : (len64 > p.n ? p.n : len64);
  const int len = int(len64);
  const bool take_all = len <= p.topk;
  const int live = max(0, min(len - slice_base, span));  // of the slice, visible
  if (n_src > 0) {
    // Merge side: the candidates of every source must have landed. One thread polls the flags the
    // sources set behind their data; the wait is bounded by wall time, and when it runs out the
    // kernel says so in the status word and goes on with whatever is there (the host raises).
    if (tid == 0) {
      const unsigned long long t0 = wall_ns();
      bool ok = false;
      for (uint32_t spin = 0; !ok; ++spin) {
        ok = true;
        for (int src = 0; src < n_src; ++src)
          ok = ok && int32_t(ld_acquire_sys(p.wait_flags + size_t(src) * R + r) - step) >= 0;
        if (!ok && (spin & 63u) == 63u && wall_ns() - t0 > p.wait_limit_ns) break;
      }
      if (!ok) atomicOr(&g_device_status, kStatusExchangeTimeout);
    }
    __syncthreads();
  }
  if (live > 0)
    for (int i = bulk_elems + tid; i < live; i += kClThreads) flat[i] = __float_as_uint(row[slice_base + i]);
  // A short slice leaves room for its part of the index map behind it: the emission then reads
  // shared memory instead of making one trip to global memory per selected element.
  const int32_t* imap = index_map ? index_map + (n_src > 0 ? gather_row : int64_t(r)) * p.n : nullptr;
  const bool imap_staged = imap != nullptr && 2 * span <= kClWarps * kWarpKeys;
  if (imap_staged)
    for (int i = tid; i < live; i += kClThreads) flat[span + i] = uint32_t(imap[slice_base + i]);
  DSA_STAMP(stamp_cta, 1);

  // The slice is in shared memory once the bulk copy has landed; positions past the row's length
  // then get a NaN, which fails every comparison below. Warp 0 waits (bounded), the others at the
  // barrier; if the copy never lands the CTA goes on with an empty slice and the status word says so.
  auto wait_slice = [&]() {
    if (warp == 0 && bulk_elems > 0) {
      if (!mbar_wait(bar, 0)) {
        if (lane == 0) atomicOr(&g_device_status, kStatusSelectOverflow);
        drain_after_timeout();
      }
    }
    __syncthreads();
    for (int i = live + tid; i < span; i += kClThreads) flat[i] = 0xFFFFFFFFu;
    __syncthreads();
  };

  // Thresholds of the sweep as NUMBERS (floating-point compares issue at twice the rate of
  // integer ones): a logit is certainly kept when v >= f_hi (its bin is above T) and a candidate
  // when f_lo <= v < f_hi (its bin is T). Positions past the row's length hold a NaN and fail
  // both. Short rows keep every visible position: f_hi = -inf.
  float f_hi = __int_as_float(0xff800000), f_lo = f_hi;
  uint32_t T = 0, need = 0;
  if (!take_all) {
    // ---- level 1: top 12 key bits
    if (have_hist) {
      const uint32_t cnt[8] = {h1b.w, h1b.z, h1b.y, h1b.x, h1a.w, h1a.z, h1a.y, h1a.x};  // highest bin first
      find_kth_in_registers<kBins, 8>(cnt, uint32_t(p.topk), sh.warp_tot, sh.res);
    } else {
      // this CTA's own histogram, then its non-zero bins pushed into every CTA's hist1. It borrows
      // the (still clear) first half of hist3 and clears it again before anybody pushes there.
      uint32_t* local1 = sh.hist3;
      wait_slice();
#pragma unroll 4
      for (int i = 0; i < nk; ++i) {
        const bool in = i * 32 + lane + warp_off < live;
        const float v = in ? __uint_as_float(flat[warp_off + i * 32 + lane]) : 0.f;
        hist_add_warp(local1, in, ordered_key(v) >> kLowBits);
      }
      DSA_STAMP(stamp_cta, 12);
      __syncthreads();
      if (!solo) cluster_wait();  // every CTA of the cluster runs and has cleared its histograms: remote adds may start
      for (int i = tid; i < kBins; i += kClThreads) {
        const uint32_t x = local1[i];
        if (x) {
          local1[i] = 0;
          if (solo) {
            sh.hist1[i] = x;
          } else {
            const uint32_t a = smem_u32(&sh.hist1[i]);
#pragma unroll 1
            for (uint32_t cc = 0; cc < C; ++cc) cluster_red_add(cluster_map(a, cc), x);
          }
        }
      }
      DSA_STAMP(stamp_cta, 13);
      cluster_sync_all(solo);
      DSA_STAMP(stamp_cta, 5);
      find_kth_bin<kBins>(sh.hist1, uint32_t(p.topk), sh.warp_tot, sh.res);
    }
    T = sh.res[0];
    need = sh.res[1];
    // bin T is [T << 20, (T + 1) << 20) in key space; bins below ordered_key(-inf) hold only NaNs
    const uint32_t key_lo = max(T << kLowBits, 0x007FFFFFu);
    f_lo = key_to_float(key_lo);
    f_hi = T == uint32_t(kBins - 1) ? __int_as_float(0x7fc00000)  // top bin: nothing is above it
                                    : key_to_float(max((T + 1) << kLowBits, 0x007FFFFFu));
  }
  DSA_STAMP(stamp_cta, 2);

  // ---- the sweep: per thread, which of its 32 logits are certainly kept and which are candidates
  if (have_hist || take_all) wait_slice();
  DSA_STAMP(stamp_cta, 4);
  // Lane l of a warp owns word l of the warp's share: 32 consecutive positions, read as eight
  // 16-byte chunks. The lanes start at different chunks ((j + l) mod 8), so that the eight lanes
  // served together touch all 32 banks. Bit b of my_kept / my_cand is position 32 l + b.
  uint32_t my_kept = 0, my_cand = 0;
  const uint32_t* wbits = flat + warp_off;
  if (lane < nk) {
    const uint4* chunks = reinterpret_cast<const uint4*>(wbits + lane * 32);
    uint32_t ge_lo = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int q = (j + lane) & 7;
      const uint4 x = chunks[q];
      const float v0 = __uint_as_float(x.x), v1 = __uint_as_float(x.y), v2 = __uint_as_float(x.z), v3 = __uint_as_float(x.w);
      const uint32_t hi4 = (v0 >= f_hi ? 1u : 0u) | (v1 >= f_hi ? 2u : 0u) | (v2 >= f_hi ? 4u : 0u) | (v3 >= f_hi ? 8u : 0u);
      const uint32_t lo4 = (v0 >= f_lo ? 1u : 0u) | (v1 >= f_lo ? 2u : 0u) | (v2 >= f_lo ? 4u : 0u) | (v3 >= f_lo ? 8u : 0u);
      my_kept |= hi4 << (4 * q);
      ge_lo |= lo4 << (4 * q);
    }
    my_cand = take_all ? 0u : ge_lo & ~my_kept;
    sh.kept[warp][lane] = my_kept;
  }
  __syncwarp();
  DSA_STAMP(stamp_cta, 3);

  // One pass over this warp's candidates: every lane walks the set bits of its own mask, the
  // warp stays converged (a lane that has run out takes part with live = false).
  auto for_each_candidate = [&](auto&& fn) {
    uint32_t rem = my_cand;
    while (__any_sync(0xffffffffu, rem != 0u)) {
      const bool live = rem != 0u;
      const int i = live ? __ffs(rem) - 1 : 0;
      rem &= rem - 1u;
      fn(live, ordered_key(__uint_as_float(wbits[lane * 32 + i])), i);
    }
  };

  uint32_t kstar = 0, ties_kept = 0;
  bool totals_known = false;  // the list path leaves every CTA's kept count in cnts[] / cand_kept[]
  if (!take_all) {
    // ---- the candidates (bin T) of the whole row go to every CTA as a list of (key, position),
    // with the CTA's level-2 histogram of them (key bits 19..13) and its count of certainly kept
    // logits: one cluster barrier, and everything after it is local. A CTA with more than
    // kListTotal / C candidates sends only its counts, and the whole cluster (which sees the same
    // counts) takes the histogram path below instead.
    const uint32_t list_cap = uint32_t(kListTotal) / C;  // entries per CTA's region of the list
    const uint32_t n_cand = uint32_t(__popc(my_cand));
    const uint32_t cinc = warp_inclusive_scan(n_cand);
    const uint32_t wabove = __reduce_add_sync(0xffffffffu, uint32_t(__popc(my_kept)));
    uint32_t slot = 0;
    if (lane == 31) {
      slot = atomicAdd(&sh.list_n, cinc);  // the warp's slots in this CTA's region of the list
      smem_red_add(&sh.above_n, wabove);
    }
    if (have_hist && !solo) cluster_wait();  // every CTA of the cluster runs (without the scan's histogram: taken at level 1)
    slot = __shfl_sync(0xffffffffu, slot, 31);
    if (slot + __shfl_sync(0xffffffffu, cinc, 31) <= list_cap) {  // (else the region overflows: see below)
      slot += cinc - n_cand;
      uint32_t rem = my_cand;
      while (rem) {  // into this CTA's own copy of its region first
        const int i = __ffs(rem) - 1;
        rem &= rem - 1u;
        const uint32_t key = ordered_key(__uint_as_float(wbits[lane * 32 + i]));
        smem_red_add(&sh.local2[(key >> kL3Bits) & (kL2Bins - 1)], 1u);
        // place = (CTA, warp, word, bit): orders like the position
        sh.list[c * list_cap + slot++] = make_uint2(key, (c << 14) | uint32_t((warp << 10) | (lane << 5) | i));
      }
    }
    __syncthreads();
    const uint32_t listed_here = sh.list_n;
    const bool fits = listed_here <= list_cap;
    if (!solo) {
      // ... then one entry per thread to the other CTAs, the level-2 counts and the totals
      if (fits) {
        for (uint32_t j = tid; j < listed_here; j += kClThreads) {
          const uint2 e = sh.list[c * list_cap + j];
          const uint32_t a = smem_u32(&sh.list[c * list_cap + j]);
#pragma unroll
          for (uint32_t cc = 0; cc < uint32_t(kMaxC); ++cc)
            if (cc < C && cc != c) cluster_st2(cluster_map(a, cc), e.x, e.y);
        }
        if (tid >= kClThreads - kL2Bins) {
          const int bin = tid - (kClThreads - kL2Bins);
          const uint32_t x = sh.local2[bin];
          const uint32_t a = smem_u32(&sh.tbl[c][bin]);
#pragma unroll
          for (uint32_t cc = 0; cc < uint32_t(kMaxC); ++cc)
            if (cc < C) cluster_st(cluster_map(a, cc), x);
        }
      }
      if (warp == kClWarps / 2 && lane < int(C))
        cluster_st(cluster_map(smem_u32(&sh.cnts[c]), uint32_t(lane)), listed_here | (sh.above_n << 16));  // at most 16384 of each
    } else {
      if (tid < kL2Bins) sh.tbl[0][tid] = sh.local2[tid];
      if (tid == kL2Bins) sh.cnts[0] = listed_here | (sh.above_n << 16);
    }
    DSA_STAMP(stamp_cta, 8);
    cluster_sync_all(solo);
    DSA_STAMP(stamp_cta, 9);

    bool listed;
    {
      const uint32_t pk = lane < int(C) ? sh.cnts[lane] & 0xFFFFu : 0u;
      listed = !__any_sync(0xffffffffu, pk > list_cap);
    }
    uint32_t p19 = 0, need2 = 0, n_surv = 0, b2 = 0;
    if (listed) {
      // ---- level 2 (key bits 19..13): the sum of the CTAs' tables, searched by one warp
      find_kth_bin_tables<kMaxC>(&sh.tbl[0][0], int(C), need, sh.res);
      b2 = sh.res[0];
      p19 = (T << kL2Bits) | b2;
      need2 = sh.res[1];
      n_surv = sh.res[2];
      listed = n_surv <= uint32_t(kSurvCap);
    }
    DSA_STAMP(stamp_cta, 10);
    if (listed) {
      // ---- (a) this CTA's own candidates above those 19 bits are kept; (b) how many such
      // candidates every CTA has, from its table; (c) the few candidates that share the 19 bits
      // ("survivors") are collected from the whole list: warp w looks at region w % C, 32 entries
      // at a time.
      if (my_cand) {  // (a word has one owner; the survivors' bits come later, behind a barrier)
        uint32_t rem = my_cand;
        while (rem) {
          const int i = __ffs(rem) - 1;
          rem &= rem - 1u;
          if ((ordered_key(__uint_as_float(wbits[lane * 32 + i])) >> kL3Bits) > p19) my_kept |= 1u << i;
        }
        sh.kept[warp][lane] = my_kept;
      }
      if (warp < int(C)) {
        const uint4 x = reinterpret_cast<const uint4*>(sh.tbl[warp])[lane];  // bins 4 lane .. 4 lane + 3
        const uint32_t b0 = uint32_t(4 * lane);
        const uint32_t sum = (b0 > b2 ? x.x : 0u) + (b0 + 1 > b2 ? x.y : 0u) + (b0 + 2 > b2 ? x.z : 0u) + (b0 + 3 > b2 ? x.w : 0u);
        const uint32_t tot = __reduce_add_sync(0xffffffffu, sum);
        if (lane == 0) smem_red_add(&sh.cand_kept[warp], tot);
      }
      {
        const int region = warp & int(C - 1u), chunk_step = (kClWarps / int(C)) * 32;
        const uint2* rlist = sh.list + uint32_t(region) * list_cap;
        const int rcnt = int(sh.cnts[region] & 0xFFFFu);
        for (int j = (warp / int(C)) * 32 + lane; j - lane < rcnt; j += chunk_step) {
          const uint2 e = j < rcnt ? rlist[j] : make_uint2(0u, 0u);
          const bool is = j < rcnt && (e.x >> kL3Bits) == p19;
          const uint32_t m = __ballot_sync(0xffffffffu, is);
          if (m) {
            const int leader = __ffs(m) - 1;
            uint32_t base = 0;
            if (lane == leader) base = atomicAdd(&sh.surv_n, uint32_t(__popc(m)));
            base = __shfl_sync(0xffffffffu, base, leader);
            if (is) sh.surv[base + __popc(m & ((1u << lane) - 1u))] = (uint64_t(e.x) << 32) | uint64_t(~e.y);
          }
        }
      }
      if (tid >= kClThreads - 4) sh.surv[n_surv + uint32_t(tid - (kClThreads - 4))] = 0ull;  // below every survivor
      __syncthreads();
      DSA_STAMP(stamp_cta, 11);
      // ---- a survivor is kept when fewer than need2 survivors come before it (larger key, or the
      // same key at a lower position); k* is the key of the need2-th
      if (warp * 32 < int(n_surv)) {  // (whole warps, for the ballots)
        const bool have = tid < int(n_surv);
        const uint64_t mine = sh.surv[have ? tid : 0];  // larger = earlier in (key descending, position ascending)
        uint32_t before = 0;
#pragma unroll 1
        for (uint32_t j = 0; j < n_surv; j += 4) {
          const uint64_t o0 = sh.surv[j], o1 = sh.surv[j + 1], o2 = sh.surv[j + 2], o3 = sh.surv[j + 3];
          before += uint32_t(o0 > mine) + uint32_t(o1 > mine) + uint32_t(o2 > mine) + uint32_t(o3 > mine);
        }
        const uint32_t key = uint32_t(mine >> 32), place = ~uint32_t(mine);
        if (have && before + 1u == need2) sh.res[3] = key;
        const bool keep = have && before < need2;
        const uint32_t owner = place >> 14;
        // kept survivors per owning CTA: 8-bit counters (at most 32 each), four to a warp sum
        const uint32_t one = keep ? 1u << (8u * (owner & 3u)) : 0u;
        uint32_t mine_n = 0;
#pragma unroll
        for (uint32_t w4 = 0; w4 < uint32_t(kMaxC) / 4; ++w4) {
          if (4 * w4 < C) {
            const uint32_t sum = __reduce_add_sync(0xffffffffu, (owner >> 2) == w4 ? one : 0u);
            if (uint32_t(lane) >> 2 == w4) mine_n = (sum >> (8 * (lane & 3))) & 0xFFu;
          }
        }
        if (lane < int(C) && mine_n) smem_red_add(&sh.cand_kept[lane], mine_n);
        if (keep && owner == c) smem_red_or(&sh.kept[(place >> 10) & 15u][(place >> 5) & 31u], 1u << (place & 31u));
      }
      __syncthreads();
      kstar = sh.res[3];
      totals_known = true;  // (ties_kept stays 0: the ties are already in the kept mask)
    } else {
    // ---- level 2: key bits 19..13 of the candidates
    if (!fits) {  // (a CTA that listed its candidates has counted them already; one that could not starts over)
      if (tid < kL2Bins) sh.local2[tid] = 0u;
      __syncthreads();
      for_each_candidate([&](bool live, uint32_t key, int) {
        hist_add_warp(sh.local2, live, (key >> kL3Bits) & (kL2Bins - 1));
      });
    }
    __syncthreads();
    if (tid < kL2Bins) {
      const uint32_t x = sh.local2[tid];
      if (x && solo) {
        sh.hist2[tid] = x;
      } else if (x) {
        const uint32_t a = smem_u32(&sh.hist2[tid]);
#pragma unroll 1
        for (uint32_t cc = 0; cc < C; ++cc) cluster_red_add(cluster_map(a, cc), x);
      }
    }
    cluster_sync_all(solo);
    find_kth_bin_warp<kL2Bins>(sh.hist2, need, sh.res);
    p19 = (T << kL2Bits) | sh.res[0];
    need2 = sh.res[1];
    // ---- level 3: the low 13 bits of the candidates that share those 19 bits
    for_each_candidate([&](bool live, uint32_t key, int) {
      hist_push_warp(sh.hist3, live && (key >> kL3Bits) == p19, swizzled_bin<kL3Bins>(key & (kL3Bins - 1)), C);
    });
    DSA_STAMP(stamp_cta, 12);
    cluster_sync_all(solo);
    DSA_STAMP(stamp_cta, 13);
    find_kth_bin<kL3Bins, true>(sh.hist3, need2, sh.warp_tot, sh.res);
    kstar = (p19 << kL3Bits) | sh.res[0];  // the k-th largest key of the row
    ties_kept = sh.res[1];                 // elements equal to it that are kept, lowest positions first
    DSA_STAMP(stamp_cta, 5);
    // ---- candidates above k* join the kept mask, those equal to it the tie mask
    for_each_candidate([&](bool live, uint32_t key, int i) {
      if (live && key > kstar) sh.kept[warp][lane] |= 1u << i;  // (a word has one owner)
      else if (live && key == kstar) sh.ties[warp][lane] |= 1u << i;
    });
    __syncwarp();
    }
  } else if (!solo) {
    cluster_wait();
  }

  DSA_STAMP(stamp_cta, 14);
  // ---- (kept, ties) counts in position order, packed ties << 16 | kept: words of a warp, warps, CTAs
  const uint32_t gword = lane < nk ? sh.kept[warp][lane] : 0u;
  const uint32_t qword = lane < nk && !totals_known ? sh.ties[warp][lane] : 0u;
  const uint32_t cnt = uint32_t(__popc(gword)) | (uint32_t(__popc(qword)) << 16);
  const uint32_t inc = warp_inclusive_scan(cnt);  // at most 1024 of each kind per warp
  if (lane == 31) sh.warp_tot[warp] = inc;
  __syncthreads();
  uint32_t g_before, q_before, g_total, q_total;
  {
    const uint32_t wt = lane < kClWarps ? sh.warp_tot[lane] : 0u;  // at most 16384 of each kind per CTA
    const uint32_t wb = __reduce_add_sync(0xffffffffu, lane < warp ? wt : 0u);
    uint32_t t;
    if (totals_known) {
      t = lane < int(C) ? (sh.cnts[lane] >> 16) + sh.cand_kept[lane] : 0u;
    } else {
      const uint32_t cta_sum = __reduce_add_sync(0xffffffffu, wt);
      if (warp == 0) {
        if (solo) {
          if (lane == 0) sh.cta_tot[0] = cta_sum;
        } else if (lane < int(C)) {
          cluster_st(cluster_map(smem_u32(&sh.cta_tot[c]), uint32_t(lane)), cta_sum);
        }
      }
      cluster_sync_all(solo);
      t = lane < int(C) ? sh.cta_tot[lane] : 0u;
    }
    const uint32_t tg = t & 0xFFFFu, tq = t >> 16;
    g_total = __reduce_add_sync(0xffffffffu, tg);
    q_total = __reduce_add_sync(0xffffffffu, tq);
    g_before = __reduce_add_sync(0xffffffffu, lane < int(c) ? tg : 0u);
    q_before = __reduce_add_sync(0xffffffffu, lane < int(c) ? tq : 0u);
    g_before += (wb & 0xFFFFu) + ((inc - cnt) & 0xFFFFu);  // ... and the words before this lane's word
    q_before += (wb >> 16) + ((inc - cnt) >> 16);
  }
  DSA_STAMP(stamp_cta, 6);

  // ---- emit: lane i walks the set bits of its word i in ascending position order
  int32_t* out_idx = p.out_idx ? p.out_idx + int64_t(r) * p.topk : nullptr;
  float* out_val = !kPlain && p.out_val ? p.out_val + int64_t(r) * p.topk : nullptr;
  const uint32_t topk_u = uint32_t(p.topk);
  const float neg_inf = __int_as_float(0xff800000);
  const int64_t dest_off = (gather_row * n_dest + p.src_rank) * int64_t(p.topk);  // this rank's slot of row r
  // a selected -inf can only appear when the row has fewer than topk finite logits
  const bool need_value = out_val != nullptr || n_dest > 0 || take_all || kstar <= 0x007FFFFFu;  // ordered_key(-inf)
  {
    // A short row fills only the first nk words of a warp: each word is then shared by G lanes
    // (G = 32 / nk rounded down to a power of two), every lane taking 32 / G of its bits, so that
    // the emission is spread over all lanes whatever the row's length.
    uint32_t g = gword, q = qword, gb = g_before, qb = q_before;
    int wsel = lane;
    if (2 * nk <= 32) {
      int G = 2;
      while (2 * G * nk <= 32) G *= 2;
      wsel = lane / G;
      const int width = 32 / G, lo = (lane % G) * width;
      const uint32_t gw = __shfl_sync(0xffffffffu, gword, wsel), qw = __shfl_sync(0xffffffffu, qword, wsel);
      gb = __shfl_sync(0xffffffffu, g_before, wsel);
      qb = __shfl_sync(0xffffffffu, q_before, wsel);
      const uint32_t below = (1u << lo) - 1u, mine = ((1u << width) - 1u) << lo;  // (width <= 16)
      gb += uint32_t(__popc(gw & below));
      qb += uint32_t(__popc(qw & below));
      g = gw & mine;
      q = qw & mine;
    }
    const int word_base = slice_base + warp_off + wsel * 32;
    const uint32_t* wvals = wbits + wsel * 32;  // the word's logits (and, staged behind the slice, its index-map entries)
    // next set bit of the word and its output slot (>= topk: a tie that is not kept)
    auto next_bit = [&](int& b, uint32_t& slot) {
      b = __ffs(g | q) - 1;
      const uint32_t bit = 1u << b;
      slot = 0xFFFFFFFFu;
      if (g & bit) {
        slot = gb + min(qb, ties_kept);
        ++gb;
      } else {
        if (qb < ties_kept) slot = gb + qb;
        ++qb;
      }
      g &= ~bit;
      q &= ~bit;
    };
    auto store = [&](int b, uint32_t slot, int32_t id) {
      float v = 0.f;
      if (need_value) {
        v = __uint_as_float(wvals[b]);
        if (v == neg_inf) id = p.pad;
        if (out_val) out_val[slot] = v;
      }
      if (out_idx) out_idx[slot] = id;
      for (int d = 0; d < n_dest; ++d) {  // plain stores into every rank's gather buffers (peer memory)
        p.dest_idx[d][dest_off + slot] = id;
        p.dest_val[d][dest_off + slot] = v;
      }
    };
    if (imap == nullptr || imap_staged) {
      while (g | q) {
        int b;
        uint32_t slot;
        next_bit(b, slot);
        if (slot < topk_u) store(b, slot, imap_staged ? int32_t(wvals[span + b]) : word_base + b + p.index_offset);
      }
    } else {
      // index map in global memory: four set bits at a time, so that their loads travel together
      while (g | q) {
        int bv[4];
        uint32_t sv[4];
        int32_t idv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          bv[u] = 0;
          sv[u] = 0xFFFFFFFFu;
          if (g | q) next_bit(bv[u], sv[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) idv[u] = sv[u] < topk_u ? imap[word_base + bv[u]] : 0;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (sv[u] < topk_u) store(bv[u], sv[u], idv[u]);
      }
    }
  }
  const uint32_t total = g_total + min(q_total, ties_kept);
  for (uint32_t i = total + c * kClThreads + tid; i < topk_u; i += C * kClThreads) {
    if (out_idx) out_idx[i] = p.pad;
    if (out_val) out_val[i] = neg_inf;
    for (int d = 0; d < n_dest; ++d) {
      p.dest_idx[d][dest_off + i] = p.pad;
      p.dest_val[d][dest_off + i] = neg_inf;
    }
  }
  if (n_dest > 0) {
    // Every thread's stores come before the barrier; behind it ONE thread posts the row's step number
    // to every rank behind one fence at system scope (a release). The release is cumulative: it orders the stores
    // that reached this thread through the barrier too, so whoever acquires the flag sees the data
    // (no fence per thread: 4096 system-scope fences cost microseconds per destination).
    cluster_sync_all(solo);
    if (c == 0 && tid == 0) {
      fence_acq_rel_sys();
      for (int d = 0; d < n_dest; ++d) st_relaxed_sys(p.dest_flag[d] + r, step);
      p.sent[r] = step;
    }
  }
  if (n_src > 0 && c == 0 && tid == 0) p.seen[r] = step;
  // every CTA has read the scan's histogram long ago (before the first cluster barrier it
  // passed): re-arm it for the next scan, away from the barriers
  if (have_hist && c == 0) {
    uint4* gh = reinterpret_cast<uint4*>(p.hist + size_t(r) * kBins);
    gh[tid] = make_uint4(0, 0, 0, 0);
    gh[tid + kClThreads] = make_uint4(0, 0, 0, 0);
  }
  DSA_STAMP(stamp_cta, 7);
  DSA_KTIME_END(1);
}

}  // namespace topk
}  // namespace dsa
