// Lightning-indexer scan over an FP8-e4m3 index-key cache.
//
//   logit[r, s] = (sum_h w[r,h] * relu(q[r,h,:] . k[s,:])) * k_scale[s]
//
// Same arithmetic as the reference's indexer blocks
// (kernels/cuda_fused_sparse_splitk.py:531-647 dense, :1677-1903 paged; host
// form ref_indexer_logits_fp8 :2990-2992), laid out for sm_100a:
//
//   * keys stream HBM -> shared memory through a TMA tensor map in 128-key x
//     128-byte tiles with the 128-byte swizzle, into a ring of kStages slots;
//   * one elected thread issues tcgen05.mma kind::f8f6f4 (M = 128 keys,
//     N = 64 heads, K = 4 x 32) per tile, accumulating in tensor memory, two
//     accumulators so the next tile's MMA overlaps this tile's epilogue;
//   * four epilogue warps read the accumulator with tcgen05.ld: one thread owns
//     one key and all 64 head products, so ReLU, the head weights, the head sum
//     and the per-key scale never leave registers, and the logit store (and the
//     optional 4096-bin histogram used by the top-k) is coalesced.
//
// No inter-CTA waits; every mbarrier wait is bounded and reports through
// g_device_status.
#pragma once

#include "common.cuh"

namespace dsa {
namespace scan {

constexpr int kTileKeys = 128;
constexpr int kKeyBytes = DSA_INDEX_DIM;  // 128 e4m3 per key
constexpr int kTileBytes = kTileKeys * kKeyBytes;
constexpr int kStagesTwoPerSm = 4;   // 92 KB of shared memory: two CTAs per SM
constexpr int kMaxHeads = DSA_INDEX_MAX_HEADS;
constexpr int kThreads = 192;    // one epilogue group: warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int kThreads2 = 320;   // two epilogue groups: warps 2..5 take the even tiles, warps 6..9 the odd ones
constexpr int kMaxAcc = 4;       // accumulators (64 fp32 columns each): one per epilogue group, at least two
__host__ __device__ constexpr int tmem_cols(int n_acc) { return n_acc <= 2 ? 128 : 256; }  // allocations are powers of two
constexpr int kHistBins = DSA_TOPK_HIST_BINS;

struct Params {
  const uint8_t* q;
  const float* w;
  const uint8_t* keys;         // dense only (the tcgen05 path reads them through the tensor map)
  const float* k_scale;
  const int32_t* seq_lens;
  float* logits;
  uint32_t* hist;
  const uint8_t* pages;        // paged only
  const int32_t* page_table;   // paged only
  int64_t pt_stride;
  int64_t num_pages;           // paged only: entries of the page table outside [0, num_pages) are not followed
  int64_t ctx;
  int64_t k_seq_stride;
  int64_t scale_seq_stride;
  int64_t slab_stride;
  int rows_per_seq;
  int n_heads;
  int tiles_per_row;
  int paged;
  int balance_rows;  // > 1: the number of rows (<= 32) of a ragged batch on a 1-D grid, see balanced_share
};

template <int kStages>
struct __align__(8) Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[kMaxAcc];
  uint64_t acc_empty[kMaxAcc];
  uint32_t tmem_base;
  uint32_t abort;
  uint32_t bin_lo;  // range of histogram bins this CTA touched
  uint32_t bin_hi;
};

constexpr size_t kSmemQ = size_t(kMaxHeads) * kKeyBytes;
template <int kStages>
constexpr size_t smem_bytes() {
  return 1024 /*alignment slack*/ + size_t(kStages) * kTileBytes + kSmemQ + kHistBins * 4 + kMaxHeads * 4 +
         sizeof(Barriers<kStages>);
}

__device__ __forceinline__ int row_len(const Params& p, int r) {
  int64_t len = p.seq_lens ? static_cast<int64_t>(p.seq_lens[r]) : p.ctx;
  if (len < 0) len = 0;
  if (len > p.ctx) len = p.ctx;
  return static_cast<int>(len);
}

// Ragged batch on a 1-D grid of N CTAs: row j gets one CTA plus its share of the other N - R in
// proportion to its number of key tiles, so that every CTA works through about the same number
// of tiles whatever the rows' lengths (R <= 32: one lane per row; every warp computes the same
// answer by itself). Gives the row of CTA b, its index among the row's CTAs and their count.
__device__ __forceinline__ void balanced_share(const Params& p, int b, int N, int R, int& r, int& bx, int& G, int& len) {
  const int lane = threadIdx.x & 31;
  const int my_len = lane < R ? row_len(p, lane) : 0;
  const int tiles = (my_len + kTileKeys - 1) / kTileKeys;
  int cum = tiles;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, cum, o);
    if (lane >= o) cum += up;
  }
  const int total = __shfl_sync(0xffffffffu, cum, 31), spare = N - R;
  const int start = lane + (total > 0 ? int(int64_t(cum - tiles) * spare / total) : 0);
  const int end = lane + 1 + (total > 0 ? int(int64_t(cum) * spare / total) : 0);
  const uint32_t hit = __ballot_sync(0xffffffffu, lane < R && b >= start && b < end);
  const int j = hit ? __ffs(hit) - 1 : 0;
  r = j;
  bx = b - __shfl_sync(0xffffffffu, start, j);
  G = __shfl_sync(0xffffffffu, end - start, j);
  len = __shfl_sync(0xffffffffu, my_len, j);  // (saves the row's own length a second trip to global memory)
}

// Body of the scan for CTA `bx` of `G` working on row `r` (the kernel below
// passes its block indices; the fused indexer + attention launch passes indices
// of its scan partition). `tmap_ptr` must point at a __grid_constant__ kernel
// parameter; `smem_raw` is the CTA's dynamic shared memory.
template <int kStages, int kEpiGroups = 1, bool kPaged = false>
__device__ __forceinline__ void scan_tc_body(const CUtensorMap* tmap_ptr, const Params& p, const int bx_in,
                                             const int G_in, const int r_grid, uint8_t* smem_raw) {
  int bx = bx_in, G = G_in;  // (a balanced ragged batch settles them after the dependency wait)
  const CUtensorMap& tmap = *tmap_ptr;
  constexpr int kBodyThreads = 64 + 128 * kEpiGroups;  // threads that take part (the caller's CTA may not be larger)
  constexpr int kAcc = kEpiGroups < 2 ? 2 : kEpiGroups;  // tile `it` accumulates in buffer it % kAcc
  constexpr int kTmemCols = tmem_cols(kAcc);
  static_assert(kAcc <= kMaxAcc, "at most four epilogue groups");
  constexpr size_t kSmemStages = size_t(kStages) * kTileBytes;
  // 1024-byte alignment for the swizzled tiles, computed on the shared-window
  // address so the pointer keeps its address space
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* s_tiles = smem;
  uint8_t* s_q = smem + kSmemStages;
  uint32_t* s_hist = reinterpret_cast<uint32_t*>(s_q + kSmemQ);
  float* s_w = reinterpret_cast<float*>(s_hist + kHistBins);
  Barriers<kStages>* bars = reinterpret_cast<Barriers<kStages>*>(s_w + kMaxHeads);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  int r = r_grid, seq = 0, len = 0;  // settled after the dependency wait below
  const bool want_hist = p.hist != nullptr;
  const int stamp_cta = r_grid * G_in + bx_in;
  (void)stamp_cta;  // (used by the tracing build only)
  DSA_STAMP(stamp_cta, 0);
  DSA_KTIME_BEGIN(0);
  if (tid == 0) prefetch_tensor_map(&tmap);

  // One tile's TMA load into ring slot (it % kStages); the caller has made sure the slot is free.
  // (paged layout: the tile's two page ids are read by the caller, ahead of the moment the slot
  // is free, so that the loads from the page table are not on the producer's critical path)
  auto tile_pages = [&](int t) -> int2 {
    if (!kPaged) return make_int2(0, 0);
    const int32_t* pt = p.page_table + int64_t(r) * p.pt_stride + 2 * t;
    const bool second = int64_t(2 * t + 1) * DSA_PAGE_TOKENS < len;
    return make_int2(pt[0], second ? pt[1] : -1);
  };
  auto issue_tile = [&](int it, int t, int2 pages) {
    const int s = it % kStages;
    const uint32_t dst = smem_u32(s_tiles + size_t(s) * kTileBytes);
    const uint32_t bar = smem_u32(&bars->full[s]);
    if (!kPaged) {
      mbar_arrive_expect_tx(bar, kTileBytes);
      tma_load_2d(dst, &tmap, 0, static_cast<int>(int64_t(seq) * p.k_seq_stride + int64_t(t) * kTileKeys), bar);
    } else {
      const bool second = int64_t(2 * t + 1) * DSA_PAGE_TOKENS < len;
      mbar_arrive_expect_tx(bar, second ? kTileBytes : kTileBytes / 2);
      tma_load_3d(dst, &tmap, 0, 0, pages.x, bar);
      if (second) tma_load_3d(dst + kTileBytes / 2, &tmap, 0, 0, pages.y, bar);
    }
  };

  // ---- set-up. What needs no input comes first (barriers, tensor memory,
  // histogram clear) and overlaps the tail of the previous kernel; after the
  // dependency wait thread 0 at once starts the first kStages tile loads, so the
  // HBM latency of the keys overlaps the query-tile and weight loads.
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int b = 0; b < kAcc; ++b) {
      mbar_init(smem_u32(&bars->acc_full[b]), 1);
      mbar_init(smem_u32(&bars->acc_empty[b]), 4);
    }
    bars->abort = 0;
    bars->bin_lo = kHistBins;
    bars->bin_hi = 0;
    mbar_fence_init();
  }
  DSA_STAMP(stamp_cta, 11);
  if (want_hist)
    for (int i = tid; i < kHistBins / 4; i += kBodyThreads)
      reinterpret_cast<uint4*>(s_hist)[i] = make_uint4(0, 0, 0, 0);
  pdl_wait();  // keys, query, weights and lengths may come from the previous kernel
  pdl_launch_dependents();
  DSA_STAMP(stamp_cta, 13);
  bool have_len = false;
  if constexpr (kEpiGroups > 2) {  // (batches run the three-group form)
    if (p.balance_rows > 1) {
      balanced_share(p, bx_in, G_in, p.balance_rows, r, bx, G, len);
      have_len = true;
    }
  }
  seq = r / p.rows_per_seq;
  if (!have_len) len = row_len(p, r);
  // q[r] is [n_heads][128 B]. Its loads (and the head weights') are issued before
  // the key tiles' so they are not queued behind 64 KB of TMA traffic per CTA.
  constexpr int kQChunks = (kMaxHeads * 8 + kBodyThreads - 1) / kBodyThreads;
  uint4 qv[kQChunks];
  {
    const uint4* qsrc = reinterpret_cast<const uint4*>(p.q + size_t(r) * p.n_heads * kKeyBytes);
#pragma unroll
    for (int k = 0; k < kQChunks; ++k) {
      const int i = tid + k * kBodyThreads;
      qv[k] = make_uint4(0, 0, 0, 0);
      if (i < kMaxHeads * 8 && (i >> 3) < p.n_heads) qv[k] = qsrc[i];
    }
  }
  const float wv = tid < p.n_heads ? p.w[size_t(r) * p.n_heads + tid] : 0.f;
  if (warp == 1) {  // tensor-memory allocation overlaps the latency of those loads
    __syncwarp();
    tmem_alloc(smem_u32(&bars->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  DSA_STAMP(stamp_cta, 12);
  // Thread 0 starts the key loads right after its own query loads were issued
  // (the other warps issue theirs within the same few cycles).
  if (tid == 0) {
    if (kPaged) {
      int2 pages[kStages];
#pragma unroll
      for (int i = 0; i < kStages; ++i) {  // all page-table loads first: one latency, not one per tile
        const int t = bx + i * G;
        pages[i] = (t < p.tiles_per_row && int64_t(t) * kTileKeys < len) ? tile_pages(t) : make_int2(0, 0);
      }
#pragma unroll
      for (int i = 0; i < kStages; ++i) {
        const int t = bx + i * G;
        if (t < p.tiles_per_row && int64_t(t) * kTileKeys < len) issue_tile(i, t, pages[i]);
      }
    } else {  // (kept as a short rolled loop: the kernel's time inside a decode step follows its code size)
      int it = 0;
#pragma unroll 1
      for (int t = bx; t < p.tiles_per_row && it < kStages; t += G, ++it) {
        if (int64_t(t) * kTileKeys >= len) break;
        issue_tile(it, t, make_int2(0, 0));
      }
    }
  }
  DSA_STAMP(stamp_cta, 15);
  // shared copy of q: K-major with the 128-B swizzle (16-byte chunk c of row h
  // lands in chunk c ^ (h & 7)); rows past n_heads are zero -> relu(0) * 0.
#pragma unroll
  for (int k = 0; k < kQChunks; ++k) {
    const int i = tid + k * kBodyThreads;
    if (i < kMaxHeads * 8) {
      const int h = i >> 3, c = i & 7;
      *reinterpret_cast<uint4*>(s_q + h * kKeyBytes + ((c ^ (h & 7)) << 4)) = qv[k];
    }
  }
  if (tid < kMaxHeads) s_w[tid] = wv;
  DSA_STAMP(stamp_cta, 14);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile uint32_t* abort_flag = &bars->abort;
  DSA_STAMP(stamp_cta, 1);

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // (tiles beyond the first kStages: wait for the MMA to release a ring slot)
    if (lane == 0) {
      int it = 0;
#pragma unroll 1
      for (int t = bx; t < p.tiles_per_row; t += G, ++it) {
        if (int64_t(t) * kTileKeys >= len || *abort_flag) break;
        if (it < kStages) continue;
        const int2 pages = tile_pages(t);  // (in flight during the wait for the slot)
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(smem_u32(&bars->empty[it % kStages]), ph ^ 1)) {
          atomicOr(&g_device_status, kStatusScanTimeout);
          *abort_flag = 1;
          break;
        }
        issue_tile(it, t, pages);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = idesc_f8_f32(kTileKeys, kMaxHeads);
      const uint64_t b_desc = smem_desc_k128(smem_u32(s_q));
      int it = 0;
#pragma unroll 1
      for (int t = bx; t < p.tiles_per_row; t += G, ++it) {
        if (int64_t(t) * kTileKeys >= len || *abort_flag) break;
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        const int b = it % kAcc;
        const uint32_t bph = (it / kAcc) & 1;
        if (!mbar_wait(smem_u32(&bars->acc_empty[b]), bph ^ 1) ||
            !mbar_wait(smem_u32(&bars->full[s]), ph)) {
          atomicOr(&g_device_status, kStatusScanTimeout);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint64_t a_desc = smem_desc_k128(smem_u32(s_tiles + size_t(s) * kTileBytes));
#pragma unroll
        for (int k = 0; k < kKeyBytes / 32; ++k)  // 32 e4m3 per MMA step = 32 B = 2 x 16-B units
          tc_mma_f8(tmem_base + b * kMaxHeads, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0);
        tc_commit(smem_u32(&bars->empty[s]));
        tc_commit(smem_u32(&bars->acc_full[b]));
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp & 3;  // tcgen05.ld: warp w may touch lanes 32 (w % 4) ..
    // With several epilogue groups, group g (warps 2 + 4 g .. 5 + 4 g) takes the live tiles
    // it = g (mod groups) and their accumulator, so that many tiles are in their epilogue at once.
    const int grp = kEpiGroups > 1 ? (warp - 2) >> 2 : 0;
    const float* kscale_row = p.k_scale;
    float* out_row = p.logits + int64_t(r) * p.slab_stride;
    const float neg_inf = __int_as_float(0xff800000);
    int it = 0;
    bool dead = false;
    uint32_t bin_lo = kHistBins, bin_hi = 0;
    // Per-key scale of this thread's key in tile t (0 past the row's length). The
    // scale of the NEXT tile is requested while the current one is processed, so
    // its latency (two dependent loads in the paged layout) is off the critical path.
    auto load_scale = [&](int t) -> float {
      const int64_t g = int64_t(t) * kTileKeys + quad * 32 + lane;
      if (t >= p.tiles_per_row || g >= len) return 0.f;
      if (!kPaged) return kscale_row[int64_t(seq) * p.scale_seq_stride + g];
      // The tensor-map load of a page outside the pool is zero-filled; this plain load would
      // not be, so a bad entry is not followed: the key's logit becomes -inf (NaN scale marks it).
      const int page = p.page_table[int64_t(r) * p.pt_stride + (g >> 6)];
      if (page < 0 || int64_t(page) >= p.num_pages) {
        atomicOr(&g_device_status, kStatusBadPage);
        return __int_as_float(0x7fc00000);
      }
      return *reinterpret_cast<const float*>(p.pages + int64_t(page) * DSA_INDEX_PAGE_BYTES +
                                             DSA_PAGE_TOKENS * kKeyBytes + (g & 63) * 4);
    };
    float next_scale = load_scale(bx + grp * G);
    {
      // Columns past the row's last live tile are -inf: one pass of 16-byte stores by the epilogue
      // threads of the row's G CTAs, while they would otherwise wait for the first accumulator.
      const int64_t dead0 = (int64_t(len) + kTileKeys - 1) / kTileKeys * kTileKeys;
      const int et = tid - 64, n_epi = 128 * kEpiGroups;
      if ((reinterpret_cast<uintptr_t>(out_row) & 15u) == 0) {
        const float4 ninf4 = make_float4(neg_inf, neg_inf, neg_inf, neg_inf);
        for (int64_t i = dead0 + (int64_t(bx) * n_epi + et) * 4; i < p.ctx; i += int64_t(G) * n_epi * 4) {
          if (i + 3 < p.ctx) {
            *reinterpret_cast<float4*>(out_row + i) = ninf4;
          } else {
            for (int64_t k = i; k < p.ctx; ++k) out_row[k] = neg_inf;
          }
        }
      } else {
        for (int64_t i = dead0 + int64_t(bx) * n_epi + et; i < p.ctx; i += int64_t(G) * n_epi) out_row[i] = neg_inf;
      }
    }
#pragma unroll 1
    for (int t = bx, j = 0; int64_t(t) * kTileKeys < len; t += G, ++j) {
      if ((j % kEpiGroups) != grp) continue;  // the other group's tile
      const int64_t g = int64_t(t) * kTileKeys + quad * 32 + lane;
      if (dead) {  // a wait ran out: what is left of the row's live part reads -inf
        if (g < p.ctx) out_row[g] = neg_inf;
        continue;
      }
      const bool valid = g < len;
      const float scale = next_scale;
      next_scale = load_scale(t + kEpiGroups * G);
      it = j;  // live tiles come first, so the j-th tile of the CTA is its j-th live tile
      const int b = it % kAcc;
      const uint32_t bph = (it / kAcc) & 1;
      ++it;
      if (!mbar_wait(smem_u32(&bars->acc_full[b]), bph)) {
        atomicOr(&g_device_status, kStatusScanTimeout);
        *abort_flag = 1;
        dead = true;
        if (g < p.ctx) out_row[g] = neg_inf;
        continue;
      }
      tc_fence_after();
      DSA_STAMP_IF(tid == 64 && it <= 4, stamp_cta, 2 + it);  // accumulator of live tile it-1 is ready
      const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + b * kMaxHeads;
      float sum = 0.f;
      uint32_t v[32];
      tmem_ld_32x32(taddr, v);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < 32; ++h) sum = fmaf(s_w[h], fmaxf(__uint_as_float(v[h]), 0.f), sum);
      tmem_ld_32x32(taddr + 32, v);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[b]));
#pragma unroll
      for (int h = 0; h < 32; ++h)
        sum = fmaf(s_w[32 + h], fmaxf(__uint_as_float(v[h]), 0.f), sum);
      const float logit = (valid && scale == scale) ? sum * scale : neg_inf;  // scale != scale: bad page
      if (g < p.ctx) out_row[g] = logit;
      if (want_hist) {
        const uint32_t bin = ordered_key(logit) >> 20;
        if (valid) smem_red_add(&s_hist[bin], 1u);  // (a bad page's -inf is counted too: the row keeps len entries)
        bin_lo = min(bin_lo, valid ? bin : uint32_t(kHistBins));
        bin_hi = max(bin_hi, valid ? bin : 0u);
      }
    }
    if (want_hist) {
      bin_lo = __reduce_min_sync(0xffffffffu, bin_lo);
      bin_hi = __reduce_max_sync(0xffffffffu, bin_hi);
      if (lane == 0) {
        smem_red_min(&bars->bin_lo, bin_lo);
        smem_red_max(&bars->bin_hi, bin_hi);
      }
    }
  }

  // ---- teardown
  DSA_STAMP_IF(tid == 64, stamp_cta, 8);
  tc_fence_before();
  __syncthreads();
  DSA_STAMP(stamp_cta, 9);
  if (*abort_flag) {
    // let copies that may still be in flight land before the CTA's shared memory is reused
    drain_after_timeout();
  }
  if (want_hist) {
    // only the bins this CTA touched (a narrow band around the logits' magnitude)
    uint32_t* gh = p.hist + size_t(r) * kHistBins;
    const int hi = int(bars->bin_hi);
    for (int i = int(bars->bin_lo) + tid; i <= hi; i += kBodyThreads) {
      const uint32_t c = s_hist[i];
      if (c) atomicAdd(&gh[i], c);
    }
  }
  DSA_STAMP(stamp_cta, 10);
  DSA_KTIME_END(0);
  if (warp == 1) {  // the warp that allocated it
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// (the dense and the paged cache layout are separate instantiations: what a decode step runs
// carries no code of the other layout)
template <int kStages, int kEpiGroups = 1, bool kPaged = false>
__global__ void __launch_bounds__(64 + 128 * kEpiGroups, kStages <= kStagesTwoPerSm ? 2 : 1)
indexer_scan_tc_kernel(const __grid_constant__ CUtensorMap tmap, const Params p) {
  extern __shared__ uint8_t scan_smem[];
  scan_tc_body<kStages, kEpiGroups, kPaged>(&tmap, p, blockIdx.x, gridDim.x, blockIdx.y, scan_smem);
}

// ------------------------------------------------------------------------------
// Legacy tensor-core path (mma.sync m16n8k32 e4m3), dense caches only. Kept as a
// diagnostic cross-check of the tcgen05 path, like the reference keeps its HMMA
// scan beside wgmma (kernels/cuda_fused_sparse_splitk.py:1851-1880).
constexpr int kLegacyThreads = 128;

__device__ __forceinline__ void mma_e4m3_16832(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kLegacyThreads)
indexer_scan_legacy_kernel(const Params p) {
  __shared__ __align__(16) uint8_t s_q[kMaxHeads * kKeyBytes];
  __shared__ float s_w[kMaxHeads];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = blockIdx.y;
  const int seq = r / p.rows_per_seq;
  const int len = row_len(p, r);
  {
    const uint4* qsrc = reinterpret_cast<const uint4*>(p.q + size_t(r) * p.n_heads * kKeyBytes);
    for (int i = tid; i < kMaxHeads * 8; i += kLegacyThreads) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if ((i >> 3) < p.n_heads) v = qsrc[i];
      reinterpret_cast<uint4*>(s_q)[i] = v;
    }
    for (int i = tid; i < kMaxHeads; i += kLegacyThreads)
      s_w[i] = i < p.n_heads ? p.w[size_t(r) * p.n_heads + i] : 0.f;
  }
  __syncthreads();
  const uint8_t* keys = p.keys + int64_t(seq) * p.k_seq_stride * kKeyBytes;
  const float* kscale = p.k_scale + int64_t(seq) * p.scale_seq_stride;
  float* out_row = p.logits + int64_t(r) * p.slab_stride;
  const float neg_inf = __int_as_float(0xff800000);
  const int gr = lane >> 2, gc = lane & 3;
  const int64_t n_groups = (p.ctx + 15) / 16;
  for (int64_t grp = int64_t(blockIdx.x) * 4 + warp; grp < n_groups; grp += int64_t(gridDim.x) * 4) {
    const int64_t k0 = grp * 16;
    const int64_t ra = k0 + gr, rb = k0 + gr + 8;
    float sa = 0.f, sb = 0.f;
    if (k0 < len) {
      uint32_t a[4][4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int off = kk * 32 + gc * 4;
        a[kk][0] = ra < p.ctx ? *reinterpret_cast<const uint32_t*>(keys + ra * kKeyBytes + off) : 0u;
        a[kk][1] = rb < p.ctx ? *reinterpret_cast<const uint32_t*>(keys + rb * kKeyBytes + off) : 0u;
        a[kk][2] = ra < p.ctx ? *reinterpret_cast<const uint32_t*>(keys + ra * kKeyBytes + off + 16) : 0u;
        a[kk][3] = rb < p.ctx ? *reinterpret_cast<const uint32_t*>(keys + rb * kKeyBytes + off + 16) : 0u;
      }
#pragma unroll
      for (int nt = 0; nt < kMaxHeads / 8; ++nt) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        const uint8_t* qh = s_q + (nt * 8 + gr) * kKeyBytes + gc * 4;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_e4m3_16832(c, a[kk], *reinterpret_cast<const uint32_t*>(qh + kk * 32),
                         *reinterpret_cast<const uint32_t*>(qh + kk * 32 + 16));
        const float w0 = s_w[nt * 8 + gc * 2], w1 = s_w[nt * 8 + gc * 2 + 1];
        sa = fmaf(w0, fmaxf(c[0], 0.f), sa);
        sa = fmaf(w1, fmaxf(c[1], 0.f), sa);
        sb = fmaf(w0, fmaxf(c[2], 0.f), sb);
        sb = fmaf(w1, fmaxf(c[3], 0.f), sb);
      }
      sa += __shfl_xor_sync(0xffffffffu, sa, 1);
      sa += __shfl_xor_sync(0xffffffffu, sa, 2);
      sb += __shfl_xor_sync(0xffffffffu, sb, 1);
      sb += __shfl_xor_sync(0xffffffffu, sb, 2);
    }
    if (gc == 0) {
      if (ra < p.ctx) {
        const float v = ra < len ? sa * kscale[ra] : neg_inf;
        out_row[ra] = v;
        if (p.hist && ra < len) atomicAdd(&p.hist[size_t(r) * kHistBins + (ordered_key(v) >> 20)], 1u);
      }
      if (rb < p.ctx) {
        const float v = rb < len ? sb * kscale[rb] : neg_inf;
        out_row[rb] = v;
        if (p.hist && rb < len) atomicAdd(&p.hist[size_t(r) * kHistBins + (ordered_key(v) >> 20)], 1u);
      }
    }
  }
}

// fp32 scan for any head count / key width: one warp per key, lanes stride the
// key dimension per head. Accuracy path of the full-sequence layer API.
__global__ void __launch_bounds__(256)
indexer_scan_f32_kernel(const float* __restrict__ q, const float* __restrict__ w,
                        const float* __restrict__ k, const int32_t* __restrict__ seq_lens,
                        float* __restrict__ logits, int rows_per_seq, int n_heads, int head_dim,
                        int64_t ctx, int64_t k_seq_stride, int64_t slab_stride) {
  extern __shared__ float s_qf[];  // [n_heads][head_dim] then w[n_heads]
  const int r = blockIdx.y;
  const int seq = r / rows_per_seq;
  float* s_wf = s_qf + size_t(n_heads) * head_dim;
  for (int i = threadIdx.x; i < n_heads * head_dim; i += blockDim.x)
    s_qf[i] = q[size_t(r) * n_heads * head_dim + i];
  for (int i = threadIdx.x; i < n_heads; i += blockDim.x) s_wf[i] = w[size_t(r) * n_heads + i];
  __syncthreads();
  int64_t len = seq_lens ? seq_lens[r] : ctx;
  len = len < 0 ? 0 : (len > ctx ? ctx : len);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const float neg_inf = __int_as_float(0xff800000);
  for (int64_t s = int64_t(blockIdx.x) * wpb + warp; s < ctx; s += int64_t(gridDim.x) * wpb) {
    if (s >= len) {
      if (lane == 0) logits[int64_t(r) * slab_stride + s] = neg_inf;
      continue;
    }
    const float* kr = k + (int64_t(seq) * k_seq_stride + s) * head_dim;
    float total = 0.f;
    for (int h = 0; h < n_heads; ++h) {
      float dot = 0.f;
      for (int d = lane; d < head_dim; d += 32) dot = fmaf(s_qf[h * head_dim + d], kr[d], dot);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      total = fmaf(s_wf[h], fmaxf(dot, 0.f), total);
    }
    if (lane == 0) logits[int64_t(r) * slab_stride + s] = total;
  }
}

}  // namespace scan
}  // namespace dsa
