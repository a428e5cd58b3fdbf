// Split-K sparse MLA decode on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Same contract and the same split-K partials as sparse_mla.cuh (reference:
// kernels/cuda_fused_sparse_splitk.py:282-530 attention warps, :996-1045 merge),
// for head counts that are a multiple of 64. One CTA = (query row, block of 64
// heads, one split of the index list); 64-key tiles:
//
//   S   [64 heads x 64 keys]  = Q K^T      A = Q   (K-major),  B = K tile (K-major)
//   O^T [512 dims x 64 heads] += V^T P^T   A = V^T (MN-major), B = P      (K-major)
//
// Both products read the SAME shared-memory image of the gathered latent rows:
// nine 64-dim chunks of [64 keys][128 B] with the 128-byte swizzle. For Q K^T a
// chunk is a K-major B operand; for V^T P^T the first eight chunks are an
// MN-major A operand (dims contiguous), so no transposed copy is ever made.
// O^T puts the 512 value dims on the 128 TMEM lanes (4 blocks of 64 columns) and
// the heads on columns, which is what lets 64 heads x 512 dims fit in 256 of the
// 512 columns next to two S buffers. S is issued as a 128-row MMA whose rows
// 64..127 read the bytes after the Q chunk and land in TMEM lanes nobody reads
// (a 64-row MMA was measured: it takes the same time and spreads the rows over
// 16 lanes of each lane quadrant, which only costs the softmax half its lanes).
//
// Warp roles (512 threads): a warp reaches the TMEM lane quadrant (warp % 4).
// Warps 0,1 and 4,5 run the softmax on the 64 real S rows (thread = head; warps 0,1
// take key columns 0..31, warps 4,5 columns 32..63); warps 0-3 rescale and write
// O^T; warp 6 allocates TMEM and issues the score MMAs from one lane, warp 7 the value MMAs (one
// issuing thread for both made each product wait behind the other's 36 / 16 instructions: 57.2 -> 55.9 us
// at batch 32; what remains is the instructions' own rate, ~63 cycles per score MMA and ~95 per value MMA
// at N = 64, i.e. ~3800 of a tile's ~4900 cycles); warps 8-15 gather
// rows (eight threads per row; with four gather warps the fp8 conversion paced the
// kernel: 63 us against 56 us at batch 32, bf16 rows unchanged): 16-byte asynchronous copies straight into the swizzled image (bf16 rows)
// or load / dequantise / store (fp8 rows, fp8 -> f32, x group scale, round to
// bf16; :1181-1196).
//
// Softmax reference point: the row maximum of the first visible tile is kept as
// the reference m for the whole split; a later tile only forces a rescale of O^T
// (rare path: all four lane-quadrant warps scale the 64 head columns in TMEM) when
// it exceeds m by more than 2^kRescaleLog2. Probabilities are floating point, so
// a stale reference costs no precision; the split's (m, l, O) stay consistent
// and the merge kernel renormalises them.
//
// Tile size: four 32-key ring slots (the same bytes as two 64-key slots, three
// tiles in flight instead of one) were built and measured 1.5x SLOWER: the
// per-tile fixed latencies (mbarrier hand-offs, tensor-memory load, proxy
// fences, the softmax group barrier) do not shrink with the tile.
#pragma once

#include "sparse_mla.cuh"

#ifndef DSA_MLA_TC_PROD_WARPS
#define DSA_MLA_TC_PROD_WARPS 8
#endif

namespace dsa {
namespace mla_tc {

constexpr int kHG = 64;                        // heads per CTA
constexpr int kBN = 64;                        // keys per tile
constexpr int kChunks = mla::kD / 64;          // 9 chunks of 64 dims (128 B of bf16)
constexpr int kChunkBytes = 64 * 128;          // [64 rows][128 B]
constexpr int kTileBytes = kChunks * kChunkBytes;  // 73,728
constexpr int kProdWarps = DSA_MLA_TC_PROD_WARPS;  // gather warps: 4 or 8
constexpr int kThreads = 256 + 32 * kProdWarps;
constexpr int kSoftThreads = 192;              // warps 0-5: softmax / rescale group
constexpr int kMmaWarp = 6;                    // issues the score products (and owns the tensor-memory allocation)
constexpr int kPvWarp = 7;                     // issues the value products
constexpr int kProducerWarp0 = 8;
constexpr int kProducers = 32 * kProdWarps;
constexpr int kRowsPerPass = 4 * kProdWarps;    // 8 threads per row
constexpr int kPasses = kBN / kRowsPerPass;     // rows of a tile per gather thread
constexpr float kRescaleLog2 = 40.f;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;                  // two S buffers of 64 columns
constexpr uint32_t kColO = 128;                // four O^T blocks of 64 columns
#ifndef DSA_MLA_TC_MIN_TILES
#define DSA_MLA_TC_MIN_TILES 128  // (a build flag, for measuring the crossover)
#endif
constexpr int kMinTiles = DSA_MLA_TC_MIN_TILES;  // fewer 64x64 tiles than this: the mma.sync kernel is faster

struct Smem {
  static constexpr int q_off = 0;
  static constexpr int k_off = q_off + kTileBytes;
  static constexpr int p_off = k_off + 2 * kTileBytes;
  static constexpr int misc_off = p_off + kHG * 128;
  static constexpr int bar_off = misc_off;             // 9 mbarriers
  static constexpr int tmem_off = misc_off + 96;
  static constexpr int flag_off = misc_off + 104;      // int [2]
  static constexpr int valid_off = misc_off + 112;     // uint32 [2 stages][producer warps]
  static constexpr int factor_off = misc_off + 256;    // float [64]
  static constexpr int max_off = misc_off + 512;       // float [2 parities][2 halves][64]
  static constexpr int bytes = misc_off + 1536 + 1024;  // + slack for the 1024-byte alignment
};
static_assert(Smem::bytes <= 232448, "tcgen05 sparse MLA: shared memory over the per-CTA limit");

enum { kBarQ = 0, kBarKFull = 1, kBarKFree = 3, kBarSFull = 5, kBarPFull = 7, kBarOFull = 8, kNumBars = 9 };

// Named barrier 2 over the 192 threads of warps 0-5, plain and with an OR reduction.
__device__ __forceinline__ void group_sync() { asm volatile("bar.sync 2, 192;" ::: "memory"); }
__device__ __forceinline__ bool group_sync_or(bool x) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 2, 192, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(uint32_t(x))
      : "memory");
  return r != 0;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 16-byte unit `u` (0..71) of row `row` inside a swizzled tile image.
__device__ __forceinline__ uint32_t swz(int row, int u) {
  return uint32_t((u >> 3) * kChunkBytes + row * 128 + (((u & 7) ^ (row & 7)) << 4));
}

__global__ void __launch_bounds__(kThreads, 1)
sparse_mla_tc_kernel(const mla::Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t s_q = sbase + Smem::q_off;
  const uint32_t s_k = sbase + Smem::k_off;
  const uint32_t s_p = sbase + Smem::p_off;
  const uint32_t bars = sbase + Smem::bar_off;
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + Smem::tmem_off);
  volatile int* s_flag = reinterpret_cast<volatile int*>(smem + Smem::flag_off);
  volatile uint32_t* s_validw = reinterpret_cast<volatile uint32_t*>(smem + Smem::valid_off);
  volatile float* s_factor = reinterpret_cast<volatile float*>(smem + Smem::factor_off);
  volatile float* s_max = reinterpret_cast<volatile float*>(smem + Smem::max_off);
  auto bar = [&](int i) { return bars + 8u * uint32_t(i); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, hg = blockIdx.y, r = blockIdx.z;
  DSA_KTIME_BEGIN(2);
  const int scta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  (void)scta;

  if (tid == 0) {
    mbar_init(bar(kBarQ), kProducers);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(kBarKFull + s), kProducers);
      mbar_init(bar(kBarKFree + s), 1);
      mbar_init(bar(kBarSFull + s), 1);
      s_flag[s] = 0;
    }
    mbar_init(bar(kBarPFull), 2 * kHG);
    mbar_init(bar(kBarOFull), 1);
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(s_tmem)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  pdl_wait();  // the selection, the queries and the lengths may come from the previous kernel
  pdl_launch_dependents();

  const int seq = r / p.rows_per_seq;
  int64_t len = p.seq_lens ? int64_t(p.seq_lens[r]) : p.ctx;
  len = len < 0 ? 0 : (len > p.ctx ? p.ctx : len);
  const int k_begin = split * p.keys_per_split;
  const int k_end = min(k_begin + p.keys_per_split, p.topk);
  const int n_tiles = (max(k_end - k_begin, 0) + kBN - 1) / kBN;
  bool failed = false;
  DSA_STAMP(scta, 14);

  if (warp >= kProducerWarp0) {
    // ===================================================================== gather
    const int ptid = tid - kProducerWarp0 * 32;
    const int v8 = ptid & 7, rsub = ptid >> 3;  // 8 threads per row, kRowsPerPass rows per pass
    {
      // queries of this head block: [64 heads][1152 B] -> swizzled chunks
      const uint8_t* qsrc = reinterpret_cast<const uint8_t*>(p.q + (int64_t(r) * p.H + hg * kHG) * mla::kD);
#pragma unroll
      for (int k = 0; k < kPasses; ++k) {
        const int row = rsub + kRowsPerPass * k;
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          cp_async16(s_q + swz(row, c * 8 + v8), qsrc + row * mla::kRowBytes + c * 128 + v8 * 16);
      }
      cp_async_commit();
    }
    const int row_bytes = p.kv_fp8 ? mla::kFp8Row : mla::kRowBytes;
    const uint8_t* kv_seq = p.kv + int64_t(seq) * p.kv_seq_stride * row_bytes;
    // selection entries of this thread's four rows of tile t (-1 past the split)
    auto load_idx = [&](int t, int64_t (&idx)[kPasses]) {
#pragma unroll
      for (int k = 0; k < kPasses; ++k) {
        const int j = k_begin + t * kBN + rsub + kRowsPerPass * k;
        idx[k] = -1;
        if (t < n_tiles && j < k_end) idx[k] = p.indices ? int64_t(p.indices[int64_t(r) * p.topk + j]) : int64_t(j);
      }
    };
    int64_t idx_next[kPasses];
    load_idx(0, idx_next);
    bool q_signalled = false;
    // rows of tile t handled by this thread (nullptr: masked key) and the tile's validity bits
    auto resolve = [&](const uint8_t* (&src)[kPasses], uint32_t& vword) {
      vword = 0;
#pragma unroll
      for (int k = 0; k < kPasses; ++k) {
        const bool ok = idx_next[k] >= 0 && idx_next[k] < len;
        src[k] = ok ? kv_seq + idx_next[k] * row_bytes : nullptr;
        const uint32_t b = __ballot_sync(0xffffffffu, ok);
        vword |= (((b >> 0) & 1u) | (((b >> 8) & 1u) << 1) | (((b >> 16) & 1u) << 2) | (((b >> 24) & 1u) << 3)) << (4 * k);
      }
    };
    if (!p.kv_fp8) {
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t & 1;
        const uint32_t stage = s_k + uint32_t(s) * kTileBytes;
        DSA_STAMP_IF(ptid == 0 && t == 4, scta, 0);
        const uint8_t* src[kPasses];
        uint32_t vword;
        resolve(src, vword);
        load_idx(t + 1, idx_next);  // in flight during the waits below
        if (t >= 1) {
          // tile t-1 (and the queries) have landed: publish them before waiting for a free slot
          cp_async_wait_all();
          fence_proxy_async_smem();
          if (!q_signalled) { mbar_arrive(bar(kBarQ)); q_signalled = true; }
          mbar_arrive(bar(kBarKFull + ((t - 1) & 1)));
        }
        DSA_STAMP_IF(ptid == 0 && t == 4, scta, 1);
        // (the outcome of a wait is made warp-uniform: the loop contains warp votes)
        if (__any_sync(0xffffffffu, t >= 2 && !mbar_wait(bar(kBarKFree + s), ((t >> 1) - 1) & 1))) { failed = true; break; }
        DSA_STAMP_IF(ptid == 0 && t == 4, scta, 3);
        if (lane == 0) s_validw[s * kProdWarps + (warp - kProducerWarp0)] = vword;
#pragma unroll
        for (int k = 0; k < kPasses; ++k) {
          const int row = rsub + kRowsPerPass * k;
          if (src[k]) {
#pragma unroll
            for (int c = 0; c < kChunks; ++c) cp_async16(stage + swz(row, c * 8 + v8), src[k] + c * 128 + v8 * 16);
          } else {
            // masked key: its row must be finite because 0 * NaN would poison V^T P^T
#pragma unroll
            for (int c = 0; c < kChunks; ++c) st_shared_v4(stage + swz(row, c * 8 + v8), make_uint4(0, 0, 0, 0));
          }
        }
        cp_async_commit();
        DSA_STAMP_IF(ptid == 0 && t == 4, scta, 4);
      }
    } else {
      // fp8 rows: 512 e4m3 | 4 fp32 group scales | 64 bf16 rope. Unit u = v8 + 8 g of the
      // e4m3 part belongs to scale group g and expands to bf16 units 2u, 2u + 1. The raw
      // bytes of tile t + 1 are requested into registers as soon as tile t is stored, so
      // they travel while the slot of tile t + 1 is still being read by the tensor core.
      uint4 raw[kPasses][4], rope[kPasses], sc4[kPasses];
      uint32_t vword = 0;
      auto request = [&]() {
        const uint8_t* src[kPasses];
        resolve(src, vword);
#pragma unroll
        for (int k = 0; k < kPasses; ++k) {
          if (src[k]) {
#pragma unroll
            for (int g = 0; g < 4; ++g) raw[k][g] = ld_global_nc_v4(src[k] + (v8 + 8 * g) * 16);
            sc4[k] = ld_global_nc_v4(src[k] + 512);
            rope[k] = ld_global_nc_v4(src[k] + 528 + v8 * 16);
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) raw[k][g] = make_uint4(0, 0, 0, 0);
            sc4[k] = make_uint4(0, 0, 0, 0);
            rope[k] = make_uint4(0, 0, 0, 0);
          }
        }
      };
      if (n_tiles > 0) {
        request();
        load_idx(1, idx_next);
      }
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t & 1;
        const uint32_t stage = s_k + uint32_t(s) * kTileBytes;
        DSA_STAMP_IF(ptid == 0 && t == 4, scta, 0);
        if (__any_sync(0xffffffffu, t >= 2 && !mbar_wait(bar(kBarKFree + s), ((t >> 1) - 1) & 1))) { failed = true; break; }
        DSA_STAMP_IF(ptid == 0 && t == 4, scta, 3);
        if (lane == 0) s_validw[s * kProdWarps + (warp - kProducerWarp0)] = vword;
#pragma unroll
        for (int k = 0; k < kPasses; ++k) {
          const int row = rsub + kRowsPerPass * k;
          const float scs[4] = {__uint_as_float(sc4[k].x), __uint_as_float(sc4[k].y),
                                __uint_as_float(sc4[k].z), __uint_as_float(sc4[k].w)};
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint2 d0 = mla::dequant4(raw[k][g].x, scs[g]), d1 = mla::dequant4(raw[k][g].y, scs[g]);
            const uint2 d2 = mla::dequant4(raw[k][g].z, scs[g]), d3 = mla::dequant4(raw[k][g].w, scs[g]);
            const int u = 2 * (v8 + 8 * g);
            st_shared_v4(stage + swz(row, u), make_uint4(d0.x, d0.y, d1.x, d1.y));
            st_shared_v4(stage + swz(row, u + 1), make_uint4(d2.x, d2.y, d3.x, d3.y));
          }
          st_shared_v4(stage + swz(row, 64 + v8), rope[k]);
        }
        if (!q_signalled) {
          cp_async_wait_all();
          q_signalled = true;
          fence_proxy_async_smem();
          mbar_arrive(bar(kBarQ));
        }
        fence_proxy_async_smem();
        mbar_arrive(bar(kBarKFull + s));
        DSA_STAMP_IF(ptid == 0 && t == 4, scta, 4);
        if (t + 1 < n_tiles) {
          request();
          load_idx(t + 2, idx_next);
        }
      }
    }
    cp_async_wait_all();  // never leave with a copy in flight
    if (!failed) {
      fence_proxy_async_smem();
      if (!q_signalled) mbar_arrive(bar(kBarQ));
      if (!p.kv_fp8 && n_tiles > 0) mbar_arrive(bar(kBarKFull + ((n_tiles - 1) & 1)));
    }
  } else if (warp == kMmaWarp) {
    // ===================================================================== MMA issue: scores
    // Two issuing threads, one per product, so that neither waits behind the other's instructions:
    // this one issues S(t) = Q K(t)^T as soon as the rows of tile t have landed. (S(t) reuses the
    // buffer of S(t-2); that tile's softmax has read it, since rows(t) could only be written after
    // the value product of t-2, which needed P(t-2).)
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = idesc_bf16_f32(128, kBN, false, false);
      if (!mbar_wait(bar(kBarQ), 0)) failed = true;
      for (int t = 0; t < n_tiles && !failed; ++t) {
        if (!mbar_wait(bar(kBarKFull + (t & 1)), (t >> 1) & 1)) {
          failed = true;
          break;
        }
        tc_fence_after();
        DSA_STAMP_IF(t == 4, scta, 5);
        const uint32_t stage = s_k + uint32_t(t & 1) * kTileBytes;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t a = smem_desc_k128(s_q + uint32_t(c) * kChunkBytes) + uint64_t(2 * ks);
            const uint64_t b = smem_desc_k128(stage + uint32_t(c) * kChunkBytes) + uint64_t(2 * ks);
            tc_mma_f16(tmem + kColS + 64u * (t & 1), a, b, idesc_qk, (c | ks) ? 1u : 0u);
          }
        }
        tc_commit(bar(kBarSFull + (t & 1)));
        DSA_STAMP_IF(t == 4, scta, 6);
      }
    }
  } else if (warp == kPvWarp) {
    // ===================================================================== MMA issue: values
    // O^T += V(t)^T P(t)^T as soon as P(t) is in shared memory; its completion frees the tile's slot.
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_pv = idesc_bf16_f32(128, kHG, true, false);
      for (int t = 0; t < n_tiles && !failed; ++t) {
        if (!mbar_wait(bar(kBarPFull), t & 1)) {
          failed = true;
          break;
        }
        tc_fence_after();
        const uint32_t stage = s_k + uint32_t(t & 1) * kTileBytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int ks = 0; ks < kBN / 16; ++ks) {
            const uint64_t a = smem_desc_mn128(stage + uint32_t(2 * j) * kChunkBytes + uint32_t(ks) * 2048u,
                                               kChunkBytes, 1024);
            const uint64_t b = smem_desc_k128(s_p) + uint64_t(2 * ks);
            tc_mma_f16(tmem + kColO + 64u * j, a, b, idesc_pv, (t > 0 || ks > 0) ? 1u : 0u);
          }
        }
        tc_commit(bar(kBarKFree + (t & 1)));
        DSA_STAMP_IF(t == 4, scta, 8);
      }
      if (!failed) tc_commit(bar(kBarOFull));
    }
  } else if (warp < 6) {
    // ===================================================================== softmax, rescale, epilogue
    const int quad = warp & 3;                   // TMEM lanes [32 quad, 32 quad + 32)
    const int half = warp >> 2;                  // key columns [32 half, 32 half + 32) of a tile
    const uint32_t tq = tmem + (uint32_t(quad * 32) << 16);
    const bool soft = quad < 2;                  // lanes 0..63 hold the 64 real S rows
    const int head = quad * 32 + lane;
    float m_ref = -INFINITY, l_run = 0.f;
    for (int t = 0; t < n_tiles; ++t) {          // left only through the uniform vote below
      const int s = t & 1;
      float x[32];
      if (soft) {
        // (tcgen05.ld is warp-collective, so the outcome of the wait is made warp-uniform)
        failed = __any_sync(0xffffffffu, failed || !mbar_wait(bar(kBarSFull + s), (t >> 1) & 1));
        tc_fence_after();
        DSA_STAMP_IF(tid == 0 && t == 4, scta, 9);
        float m_loc = -INFINITY;
        if (!failed) {
          uint32_t raw[32];
          tmem_ld_32x32(tq + kColS + 64u * s + 32u * half, raw);
          tmem_ld_wait();
          // key j of the tile was staged by producer warp (j % kRowsPerPass) >> 2 in its pass
          // j / kRowsPerPass: bit 4 pass + (j & 3) of that warp's word
          constexpr int kHalfPasses = kPasses / 2;  // passes that make up 32 keys
          uint32_t vw[kProdWarps], vall = 0xFFFFFFFFu;
#pragma unroll
          for (int w = 0; w < kProdWarps; ++w) {
            vw[w] = s_validw[s * kProdWarps + w] >> (4 * kHalfPasses * half);
            vall &= vw[w];
          }
          // x keeps the raw dot products (-inf for masked keys); the softmax scale (> 0) is
          // applied to the maximum here and folded into the exponent's multiply-add below
          if ((vall & ((1u << (4 * kHalfPasses)) - 1u)) == (1u << (4 * kHalfPasses)) - 1u) {  // every key of the half-tile visible
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] = __uint_as_float(raw[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const bool ok = (vw[(i % kRowsPerPass) >> 2] >> ((i / kRowsPerPass) * 4 + (i & 3))) & 1u;
              x[i] = ok ? __uint_as_float(raw[i]) : -INFINITY;
            }
          }
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], x[i]);
          m_loc = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
          if (m_ref != -INFINITY && m_loc > m_ref + kRescaleLog2) s_flag[s] = 1;
        }
        s_max[(s * 2 + half) * kHG + head] = m_loc;
      }
      if (group_sync_or(failed)) { failed = true; break; }
      DSA_STAMP_IF(tid == 0 && t == 4, scta, 10);
      float m_tile = -INFINITY;
      if (soft) m_tile = fmaxf(s_max[(s * 2) * kHG + head], s_max[(s * 2 + 1) * kHG + head]);
      if (s_flag[s]) {
        // rare: some head's maximum ran away from its reference; scale its O^T column
        if (__any_sync(0xffffffffu, t >= 1 && !mbar_wait(bar(kBarKFree + ((t - 1) & 1)), ((t - 1) >> 1) & 1)))
          failed = true;
        tc_fence_after();
        if (soft) {
          float f = 1.f;
          if (m_ref != -INFINITY && m_tile > m_ref + kRescaleLog2) {
            f = exp2f(m_ref - m_tile);
            l_run *= f;
            m_ref = m_tile;
          }
          if (half == 0) s_factor[head] = f;
        }
        group_sync();
        if (warp < 4 && !failed) {
#pragma unroll 1
          for (int blk = 0; blk < 8; ++blk) {
            uint32_t o[32];
            tmem_ld_32x32(tq + kColO + 32u * blk, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * s_factor[(blk & 1) * 32 + i]);
            tmem_st_32x32(tq + kColO + 32u * blk, o);
          }
          tmem_st_wait();
        }
        tc_fence_before();
        group_sync();
        if (tid == 0) s_flag[s] = 0;
      }
      if (soft && !failed) {
        if (m_ref == -INFINITY) m_ref = m_tile;
        const float mr = m_ref == -INFINITY ? 0.f : m_ref;  // every key so far masked: all p = 0
        // the row sum uses the rounded probabilities that the value product will see
        uint32_t pk[16];
        float psum0 = 0.f, psum1 = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const __nv_bfloat162 b = __floats2bfloat162_rn(ex2_approx(fmaf(x[2 * i], p.scale_log2, -mr)),
                                                         ex2_approx(fmaf(x[2 * i + 1], p.scale_log2, -mr)));
          pk[i] = *reinterpret_cast<const uint32_t*>(&b);
          psum0 += __uint_as_float(pk[i] << 16);
          psum1 += __uint_as_float(pk[i] & 0xFFFF0000u);
        }
        l_run += psum0 + psum1;
        DSA_STAMP_IF(tid == 0 && t == 4, scta, 11);
        // P is single-buffered: the previous tile's value product must have read it
        if (t >= 1 && !mbar_wait(bar(kBarKFree + ((t - 1) & 1)), ((t - 1) >> 1) & 1)) failed = true;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          st_shared_v4(s_p + uint32_t(head * 128 + (((half * 4 + u) ^ (head & 7)) << 4)),
                       make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]));
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(bar(kBarPFull));
        DSA_STAMP_IF(tid == 0 && t == 4, scta, 12);
        DSA_STAMP_IF(tid == 0 && t == 5, scta, 13);
      }
    }
    DSA_STAMP(scta, 2);
    // the two column halves of a head add their sums
    if (soft && half == 1) s_factor[head] = l_run;
    group_sync();
    if (soft && half == 0) l_run += s_factor[head];

    if (warp < 4) {
      // ---- partials of this split: O^T (lane = value dim, column = head), reference m, sum l
      const int64_t pbase = (int64_t(r) * p.nsplit + split) * p.H + hg * kHG;
      bool have = n_tiles > 0 && !__any_sync(0xffffffffu, failed);
      if (__any_sync(0xffffffffu, have && !mbar_wait(bar(kBarOFull), 0))) have = false, failed = true;
      tc_fence_after();
      DSA_STAMP(scta, 7);
#pragma unroll 1
      for (int blk = 0; blk < 8; ++blk) {
        uint32_t o[32];
        if (have) {
          tmem_ld_32x32(tq + kColO + 32u * blk, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        const int dim = (blk >> 1) * 128 + quad * 32 + lane;
        float* dst = p.part_acc + (pbase + (blk & 1) * 32) * mla::kDV + dim;
#pragma unroll
        for (int i = 0; i < 32; ++i) dst[int64_t(i) * mla::kDV] = __uint_as_float(o[i]);
      }
      if (soft) {
        p.part_m[pbase + head] = have ? m_ref : -INFINITY;
        p.part_l[pbase + head] = have ? l_run : 0.f;
      }
    }
  }

  if (failed) {
    atomicOr(&g_device_status, kStatusAttnTimeout);
    drain_after_timeout();  // let outstanding copies and MMAs drain
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, kTmemCols);
  DSA_STAMP(scta, 15);
  DSA_KTIME_END(2);
}

}  // namespace mla_tc
}  // namespace dsa
