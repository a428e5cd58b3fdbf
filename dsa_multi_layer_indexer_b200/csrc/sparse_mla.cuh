// Split-K sparse MLA decode over the selected latent rows, plus the
// log-sum-exp merge of the split partials.
//
//   out[r,h,:] = softmax_j(scale * q[r,h,:] . kv[idx_j,:]) . kv[idx_j,:512]
//
// Same arithmetic as the reference's attention warps and combine kernel
// (kernels/cuda_fused_sparse_splitk.py:282-530, :996-1045; host form
// ref_sparse_mla :2950-2966): bf16 operands, fp32 accumulation, base-2 online
// softmax, probabilities rounded to bf16 before the value product.
//
// One CTA = (query row, block of 16 heads, one split of the index list). The
// 1152-byte latent rows are gathered with one bulk asynchronous copy per row
// (TMA engine, completion counted on an mbarrier) into padded shared-memory
// rows, so the gather costs one instruction per row instead of 72 16-byte
// copies per row. FP8 latent rows (656 B) are staged the same way and
// dequantised into the bf16 tile exactly as the reference does
// (fp8 -> f32, x group scale, round to bf16; :1181-1196).
#pragma once


#include "common.cuh"

namespace dsa {
namespace mla {

constexpr int kD = DSA_LATENT_DIM;       // 576
constexpr int kDV = DSA_VALUE_DIM;       // 512
constexpr int kHB = DSA_HEAD_BLOCK;      // 16 heads per CTA
constexpr int kBN = 64;                  // keys per tile
constexpr int kThreads = 128;            // 4 warps
constexpr int kRowBytes = kD * 2;        // 1152
constexpr int kRowPitch = kRowBytes + 16;  // 1168: 8 consecutive rows hit 8 distinct bank groups
constexpr int kPPitch = (kBN + 8) * 2;   // bf16 probabilities, padded the same way
constexpr int kFp8Row = DSA_FP8_LATENT_ROW;

struct Params {
  const __nv_bfloat16* q;
  const uint8_t* kv;
  const int32_t* indices;
  const int32_t* seq_lens;
  float* part_acc;
  float* part_m;
  float* part_l;
  int64_t kv_seq_stride;  // rows per cached sequence
  int64_t ctx;            // dense mode: key capacity
  int rows_per_seq;
  int H;
  int topk;
  int nsplit;
  int keys_per_split;
  int kv_fp8;
  float scale_log2;       // sm_scale * log2(e)
};

struct SmemLayout {
  static constexpr int q_off = 0;
  static constexpr int k_off = q_off + kHB * kRowPitch;
  static constexpr int p_off = k_off + kBN * kRowPitch;
  static constexpr int red_off = p_off + kHB * kPPitch;         // float [2][4][16]
  static constexpr int valid_off = red_off + 2 * 4 * kHB * 4;   // int [64]
  static constexpr int bar_off = valid_off + kBN * 4;           // 2 mbarriers
  static constexpr int bytes_bf16 = (bar_off + 16 + 15) & ~15;
  static constexpr int bytes_fp8 = bytes_bf16;  // fp8 rows are staged inside their own bf16 slots
};

// Barrier over the 128 attention threads (named barrier 1). The split-K body also
// runs inside a 192-thread CTA of the fused launch, whose two spare warps have
// left, so it must not use the whole-CTA barrier.
__device__ __forceinline__ void cta128_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier of the same 128 threads that also ORs a flag over them: every thread gets the same answer.
__device__ __forceinline__ bool cta128_any(bool flag) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(uint32_t(flag))
      : "memory");
  return r != 0;
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 4 packed e4m3 -> 4 bf16 with one fp32 scale: fp8 -> f16 (exact) -> f32 -> * s -> bf16 RN
__device__ __forceinline__ uint2 dequant4(uint32_t w, float s) {
  const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w & 0xFFFFu), __NV_E4M3);
  const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w >> 16), __NV_E4M3);
  const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&lo));
  const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&hi));
  const __nv_bfloat162 b01 = __floats2bfloat162_rn(f01.x * s, f01.y * s);
  const __nv_bfloat162 b23 = __floats2bfloat162_rn(f23.x * s, f23.y * s);
  uint2 r;
  r.x = *reinterpret_cast<const uint32_t*>(&b01);
  r.y = *reinterpret_cast<const uint32_t*>(&b23);
  return r;
}

// One 64-key tile for the 16 heads of the CTA: S = Q K^T on bf16 tensor cores,
// base-2 online softmax across the four warps, P rounded to bf16, O += P V.
// Warp w owns keys [16 w, 16 w + 16) in S and value columns [128 w, 128 w + 128)
// in O. All 128 threads call it; it contains two block barriers.
__device__ __forceinline__ void attend_tile(const uint8_t* s_q, const uint8_t* s_k, uint8_t* s_p,
                                            float* s_red, const int* s_valid, float scale_log2,
                                            int warp, int lane, float (&m_run)[2], float (&l_run)[2],
                                            float (&acc)[16][4]) {
  const int g = lane >> 2, t4 = lane & 3;
  // ---- S = Q K^T: warp w owns keys [16 w, 16 w + 16) for all 16 heads
  float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  {
    const uint32_t a_base = smem_u32(s_q + (lane & 15) * kRowPitch + (lane >> 4) * 16);
    const uint32_t b_base = smem_u32(s_k + (warp * 16 + (lane & 7) + 8 * (lane >> 4)) * kRowPitch +
                                     ((lane >> 3) & 1) * 16);
#pragma unroll 4
    for (int k0 = 0; k0 < kD; k0 += 16) {
      uint32_t a[4], b[4];
      ldsm_x4(a_base + k0 * 2, a);
      ldsm_x4(b_base + k0 * 2, b);
      mma_bf16(sc[0], a, b[0], b[1]);
      mma_bf16(sc[1], a, b[2], b[3]);
    }
  }
  // scale, mask, tile max per head row (rows g and g + 8)
  float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int col = warp * 16 + nt * 8 + t4 * 2 + (e & 1);
      const float v = s_valid[col] ? sc[nt][e] * scale_log2 : -INFINITY;
      sc[nt][e] = v;
      tmax[e >> 1] = fmaxf(tmax[e >> 1], v);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
    tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
  }
  if (t4 == 0) {
    s_red[warp * kHB + g] = tmax[0];
    s_red[warp * kHB + g + 8] = tmax[1];
  }
  cta128_sync();
  float alpha[2], m_new[2], psum[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = g + 8 * i;
    float m = m_run[i];
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, s_red[w * kHB + row]);
    m_new[i] = m;
    alpha[i] = (m == -INFINITY) ? 1.f : exp2f(m_run[i] - m);
  }
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    float pr[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float m = m_new[e >> 1];
      pr[e] = (m == -INFINITY) ? 0.f : exp2f(sc[nt][e] - m);
    }
    const __nv_bfloat162 p01 = __floats2bfloat162_rn(pr[0], pr[1]);
    const __nv_bfloat162 p23 = __floats2bfloat162_rn(pr[2], pr[3]);
    // the row sum uses the rounded probabilities that P.V will see
    psum[0] += __bfloat162float(p01.x) + __bfloat162float(p01.y);
    psum[1] += __bfloat162float(p23.x) + __bfloat162float(p23.y);
    const int col = warp * 16 + nt * 8 + t4 * 2;
    *reinterpret_cast<__nv_bfloat162*>(s_p + g * kPPitch + col * 2) = p01;
    *reinterpret_cast<__nv_bfloat162*>(s_p + (g + 8) * kPPitch + col * 2) = p23;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    psum[i] += __shfl_xor_sync(0xffffffffu, psum[i], 1);
    psum[i] += __shfl_xor_sync(0xffffffffu, psum[i], 2);
  }
  if (t4 == 0) {
    s_red[4 * kHB + warp * kHB + g] = psum[0];
    s_red[4 * kHB + warp * kHB + g + 8] = psum[1];
  }
  cta128_sync();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = g + 8 * i;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) s += s_red[4 * kHB + w * kHB + row];
    l_run[i] = l_run[i] * alpha[i] + s;
    m_run[i] = m_new[i];
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    acc[i][0] *= alpha[0];
    acc[i][1] *= alpha[0];
    acc[i][2] *= alpha[1];
    acc[i][3] *= alpha[1];
  }

  // ---- O += P V: warp w owns value columns [128 w, 128 w + 128)
  {
    const uint32_t a_base = smem_u32(s_p + (lane & 15) * kPPitch + (lane >> 4) * 16);
    const uint32_t b_base = smem_u32(s_k + ((lane & 7) + 8 * ((lane >> 3) & 1)) * kRowPitch +
                                     (warp * 128 + 8 * (lane >> 4)) * 2);
#pragma unroll
    for (int ks = 0; ks < kBN / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a_base + ks * 32, a);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t b[4];
        ldsm_x4_t(b_base + ks * 16 * kRowPitch + np * 32, b);
        mma_bf16(acc[2 * np], a, b[0], b[1]);
        mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
      }
    }
  }
}

// Dequantises a staged fp8 tile (656-B rows) into the bf16 K tile. Work item =
// one 16-byte chunk of a row: 32 chunks of 16 e4m3 (-> 32 B of bf16) and 8 chunks
// of rope that are copied. Items are independent and the loop is unrolled, so
// each thread keeps several shared-memory loads in flight (the tile is
// latency-bound with four warps per CTA). With zero_invalid the masked rows are
// cleared here (they must be finite: 0 * NaN would poison P.V); otherwise the
// caller has cleared them already.
__device__ __forceinline__ void dequant_tile(const uint8_t* s_stage, uint8_t* s_k, const int* s_valid, int tid,
                                             bool zero_invalid = false) {
  constexpr int kChunks = 40;  // per row
#pragma unroll 4
  for (int i = tid; i < kBN * kChunks; i += kThreads) {
    const int row = i / kChunks, c = i - row * kChunks;
    const uint8_t* src = s_stage + row * kFp8Row;
    uint8_t* dst = s_k + row * kRowPitch;
    const bool ok = s_valid[row] != 0;
    if (!ok && !zero_invalid) continue;
    if (c < 32) {
      uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
      if (ok) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + c * 16);
        const float sc = *reinterpret_cast<const float*>(src + 512 + (c >> 3) * 4);
        const uint2 d0 = dequant4(raw.x, sc), d1 = dequant4(raw.y, sc);
        const uint2 d2 = dequant4(raw.z, sc), d3 = dequant4(raw.w, sc);
        lo = make_uint4(d0.x, d0.y, d1.x, d1.y);
        hi = make_uint4(d2.x, d2.y, d3.x, d3.y);
      }
      *reinterpret_cast<uint4*>(dst + c * 32) = lo;
      *reinterpret_cast<uint4*>(dst + c * 32 + 16) = hi;
    } else {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (ok) v = *reinterpret_cast<const uint4*>(src + 528 + (c - 32) * 16);
      *reinterpret_cast<uint4*>(dst + 1024 + (c - 32) * 16) = v;
    }
  }
}

// In-place variant for the split-K kernel: the 656 staged bytes of a row sit at
// the END of that row's 1152-byte bf16 slot (offset 496), so no separate staging
// buffer is needed and the fp8 path keeps two CTAs per SM. Expanding a chunk
// overwrites bytes other threads may still have to read, so the tile is done in
// three passes of "load into registers, barrier, store", ordered so that a pass
// only overwrites sources of chunks already expanded or loaded:
//   chunks 0..15  read [496,752)   write [0,512)
//   chunks 16..23 read [752,880)   write [512,768)
//   chunks 24..31 + rope read [880,1152) write [768,1152)
// The four group scales sit at [1008,1024) and are read before the last stores.
constexpr int kFp8StageOff = kRowBytes - kFp8Row;  // 496
template <int FIRST, int NDEQ, int NROPE>
__device__ __forceinline__ void dequant_pass(uint8_t* s_k, const int* s_valid, int tid) {
  constexpr int kPerRow = NDEQ + NROPE;
  constexpr int kPer = (kBN * kPerRow) / kThreads;
  static_assert((kBN * kPerRow) % kThreads == 0, "items must divide evenly");
  uint4 raw[kPer];
  float sc[kPer];
#pragma unroll
  for (int u = 0; u < kPer; ++u) {
    const int i = tid + u * kThreads, row = i / kPerRow, k = i - row * kPerRow;
    const uint8_t* src = s_k + row * kRowPitch + kFp8StageOff;
    raw[u] = make_uint4(0, 0, 0, 0);
    sc[u] = 0.f;
    if (s_valid[row]) {
      if (k < NDEQ) {
        raw[u] = *reinterpret_cast<const uint4*>(src + (FIRST + k) * 16);
        sc[u] = *reinterpret_cast<const float*>(src + 512 + ((FIRST + k) >> 3) * 4);
      } else {
        raw[u] = *reinterpret_cast<const uint4*>(src + 528 + (k - NDEQ) * 16);
      }
    }
  }
  cta128_sync();
#pragma unroll
  for (int u = 0; u < kPer; ++u) {
    const int i = tid + u * kThreads, row = i / kPerRow, k = i - row * kPerRow;
    if (!s_valid[row]) continue;  // masked rows were cleared at gather time
    uint8_t* rowp = s_k + row * kRowPitch;
    if (k < NDEQ) {
      const int c = FIRST + k;
      const uint2 d0 = dequant4(raw[u].x, sc[u]), d1 = dequant4(raw[u].y, sc[u]);
      const uint2 d2 = dequant4(raw[u].z, sc[u]), d3 = dequant4(raw[u].w, sc[u]);
      *reinterpret_cast<uint4*>(rowp + c * 32) = make_uint4(d0.x, d0.y, d1.x, d1.y);
      *reinterpret_cast<uint4*>(rowp + c * 32 + 16) = make_uint4(d2.x, d2.y, d3.x, d3.y);
    } else {
      *reinterpret_cast<uint4*>(rowp + 1024 + (k - NDEQ) * 16) = raw[u];
    }
  }
}
__device__ __forceinline__ void dequant_tile_inplace(uint8_t* s_k, const int* s_valid, int tid) {
  dequant_pass<0, 16, 0>(s_k, s_valid, tid);
  dequant_pass<16, 8, 0>(s_k, s_valid, tid);
  dequant_pass<24, 8, 8>(s_k, s_valid, tid);
}

// Body of the split-K partials for CTA (split, hg, r); `smem` is the CTA's
// dynamic shared memory. Threads 0..127 take part.
// kBeside: the launch does not depend on the kernel enqueued just before it (under the lagged
// schedule the attention reads the PREVIOUS layer's selection while this layer's top-k runs), so
// it releases its own dependents and starts at once, beside that kernel, and waits for it only
// before it exits: it still completes after it, and the next kernel's wait covers both.
template <bool kBeside = false>
__device__ __forceinline__ void mla_partials_body(const Params& p, const int split, const int hg, const int r,
                                                  uint8_t* smem) {
  uint8_t* s_q = smem + SmemLayout::q_off;
  uint8_t* s_k = smem + SmemLayout::k_off;
  uint8_t* s_p = smem + SmemLayout::p_off;
  float* s_red = reinterpret_cast<float*>(smem + SmemLayout::red_off);
  int* s_valid = reinterpret_cast<int*>(smem + SmemLayout::valid_off);
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + SmemLayout::bar_off);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  DSA_KTIME_BEGIN(2);
  const int seq = r / p.rows_per_seq;
  const uint32_t bar_q = smem_u32(&s_bar[0]);
  const uint32_t bar_k = smem_u32(&s_bar[1]);
  const int row_bytes = p.kv_fp8 ? kFp8Row : kRowBytes;
  const uint8_t* kv_seq = p.kv + int64_t(seq) * p.kv_seq_stride * row_bytes;

  if (tid == 0) {
    mbar_init(bar_q, kHB);
    mbar_init(bar_k, kBN);
    mbar_fence_init();
  }
  cta128_sync();
  if constexpr (!kBeside) pdl_wait();  // the selection, the queries and the lengths may come from the previous kernel
  pdl_launch_dependents();
  // The first tile's selection entries are requested before the row's length is looked at: two
  // loads in flight together instead of two trips to global memory one after the other.
  const int k_begin = split * p.keys_per_split;
  const int k_end = min(k_begin + p.keys_per_split, p.topk);
  const int n_tiles = (max(k_end - k_begin, 0) + kBN - 1) / kBN;
  int64_t idx_first = -1;
  if (tid < kBN && k_begin + tid < k_end)
    idx_first = p.indices ? int64_t(p.indices[int64_t(r) * p.topk + k_begin + tid]) : int64_t(k_begin + tid);
  int64_t len = p.seq_lens ? int64_t(p.seq_lens[r]) : p.ctx;
  len = len < 0 ? 0 : (len > p.ctx ? p.ctx : len);

  // queries of this head block: 16 rows of 1152 B
  if (tid >= kBN && tid < kBN + kHB) {
    const int h = tid - kBN;
    const __nv_bfloat16* src = p.q + (int64_t(r) * p.H + hg * kHB + h) * kD;
    mbar_arrive_expect_tx(bar_q, kRowBytes);
    bulk_g2s(smem_u32(s_q + h * kRowPitch), src, kRowBytes, bar_q);
  }

  const int g = lane >> 2, t4 = lane & 3;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  bool timed_out = false;

  for (int tile = 0; tile < n_tiles; ++tile) {
    // ---- gather up to 64 latent rows: one bulk copy per valid row. (The copy engine accepts about
    // one such copy per 30 cycles, ~1900 cycles for the tile; 16-byte asynchronous copies by all
    // 128 threads instead were slower still: 4608 of them per tile wait on one another's returns.)
    if (tid < kBN) {
      const int j = k_begin + tile * kBN + tid;
      int64_t idx = idx_first;
      if (tile > 0) {
        idx = -1;
        if (j < k_end) idx = p.indices ? int64_t(p.indices[int64_t(r) * p.topk + j]) : int64_t(j);
      }
      const bool ok = idx >= 0 && idx < len;
      s_valid[tid] = ok;
      uint8_t* dst_row = s_k + tid * kRowPitch;
      if (ok) {
        fence_proxy_async_smem();  // earlier generic reads of this row precede the async write
        mbar_arrive_expect_tx(bar_k, row_bytes);
        if (p.kv_fp8)  // staged at the end of the row's own slot, expanded in place below
          bulk_g2s(smem_u32(dst_row + kFp8StageOff), kv_seq + idx * kFp8Row, kFp8Row, bar_k);
        else
          bulk_g2s(smem_u32(dst_row), kv_seq + idx * kRowBytes, kRowBytes, bar_k);
      } else {
        // masked key: its row must be finite because 0 * NaN would poison P.V
        uint4* z = reinterpret_cast<uint4*>(dst_row);
        for (int i = 0; i < kRowBytes / 16; ++i) z[i] = make_uint4(0, 0, 0, 0);
        mbar_arrive(bar_k);
      }
    }
    if (tile == 0 && !mbar_wait(bar_q, 0)) timed_out = true;
    if (!mbar_wait(bar_k, tile & 1)) timed_out = true;
    // Each thread ran its own clock: the 128 threads agree on leaving here, so nobody is left
    // alone at the barriers below.
    timed_out = cta128_any(timed_out);
    if (timed_out) break;
    if (p.kv_fp8) {
      dequant_tile_inplace(s_k, s_valid, tid);
      cta128_sync();
    }

    attend_tile(s_q, s_k, s_p, s_red, s_valid, p.scale_log2, warp, lane, m_run, l_run, acc);
    cta128_sync();  // the K tile and P are free for the next gather
  }

  if (n_tiles == 0) timed_out = cta128_any(!mbar_wait(bar_q, 0));  // never leave with a copy in flight
  if (timed_out) {
    atomicOr(&g_device_status, kStatusAttnTimeout);
    m_run[0] = m_run[1] = -INFINITY;
    l_run[0] = l_run[1] = 0.f;
    drain_after_timeout();  // let outstanding copies land
  }

  // ---- partials of this split: unnormalised accumulator, running max (base 2), sum
  const int64_t pbase = (int64_t(r) * p.nsplit + split) * p.H + hg * kHB;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int col = warp * 128 + i * 8 + t4 * 2;
    *reinterpret_cast<float2*>(p.part_acc + (pbase + g) * kDV + col) = make_float2(acc[i][0], acc[i][1]);
    *reinterpret_cast<float2*>(p.part_acc + (pbase + g + 8) * kDV + col) = make_float2(acc[i][2], acc[i][3]);
  }
  if (warp == 0 && t4 == 0) {
    p.part_m[pbase + g] = m_run[0];
    p.part_m[pbase + g + 8] = m_run[1];
    p.part_l[pbase + g] = l_run[0];
    p.part_l[pbase + g + 8] = l_run[1];
  }
  if constexpr (kBeside) pdl_wait();
  DSA_KTIME_END(2);
}

__global__ void __launch_bounds__(kThreads)
sparse_mla_partials_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t mla_smem[];
  mla_partials_body<false>(p, blockIdx.x, blockIdx.y, blockIdx.z, mla_smem);
}

__global__ void __launch_bounds__(kThreads)
sparse_mla_partials_beside_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t mla_smem[];
  mla_partials_body<true>(p, blockIdx.x, blockIdx.y, blockIdx.z, mla_smem);
}

// ------------------------------------------------------------------------------
// out = sum_s acc_s 2^(m_s - m) / sum_s l_s 2^(m_s - m); splits with m = -inf
// (no visible key) are skipped, a row with none yields zeros. One CTA per (row,
// head) of 1..4 groups of 128 threads (the launch picks min(nsplit, 4)): group g
// folds splits g, g + ngrp, ... with all loads of a chunk of eight splits in
// flight at once, then group 0 merges the group results in a fixed order.
constexpr int kCombineThreads = 512;
__global__ void __launch_bounds__(kCombineThreads)
sparse_mla_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_m,
                          const float* __restrict__ part_l, __nv_bfloat16* __restrict__ out, int H,
                          int nsplit) {
  __shared__ float s_m[4], s_l[4];
  __shared__ __align__(16) float s_o[4][kDV];
  const int h = blockIdx.x, r = blockIdx.y, tid = threadIdx.x & 127, grp = threadIdx.x >> 7;
  const int ngrp = blockDim.x >> 7;  // 1..4 load groups of 128 threads, each taking every ngrp-th split
  DSA_KTIME_BEGIN(3);
  pdl_wait();
  pdl_launch_dependents();
  const float* pm = part_m + int64_t(r) * nsplit * H + h;
  const float* pl = part_l + int64_t(r) * nsplit * H + h;
  const float* pa = part_acc + (int64_t(r) * nsplit * H + h) * kDV + tid * 4;
  float mg = -INFINITY, lg = 0.f;
  float4 og = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = grp; s0 < nsplit; s0 += 8 * ngrp) {
    float ms[8], ls[8];
    float4 a[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int sp = s0 + ngrp * u;
      const bool ok = sp < nsplit;
      ms[u] = ok ? pm[int64_t(sp) * H] : -INFINITY;
      ls[u] = ok ? pl[int64_t(sp) * H] : 0.f;
      a[u] = ok ? *reinterpret_cast<const float4*>(pa + int64_t(sp) * H * kDV) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float m_new = mg;
#pragma unroll
    for (int u = 0; u < 8; ++u) m_new = fmaxf(m_new, ms[u]);
    if (m_new != -INFINITY) {
      const float keep = (mg == -INFINITY) ? 0.f : exp2f(mg - m_new);
      lg *= keep;
      og.x *= keep;
      og.y *= keep;
      og.z *= keep;
      og.w *= keep;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float e = (ms[u] == -INFINITY) ? 0.f : exp2f(ms[u] - m_new);
        lg = fmaf(ls[u], e, lg);
        og.x = fmaf(a[u].x, e, og.x);
        og.y = fmaf(a[u].y, e, og.y);
        og.z = fmaf(a[u].z, e, og.z);
        og.w = fmaf(a[u].w, e, og.w);
      }
    }
    mg = m_new;
  }
  if (tid == 0) {
    s_m[grp] = mg;
    s_l[grp] = lg;
  }
  *reinterpret_cast<float4*>(&s_o[grp][tid * 4]) = og;
  __syncthreads();
  if (grp == 0) {
    float m = s_m[0];
    for (int gi = 1; gi < ngrp; ++gi) m = fmaxf(m, s_m[gi]);
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    float l = 0.f;
    if (m != -INFINITY) {
      for (int gi = 0; gi < ngrp; ++gi) {
        const float e = (s_m[gi] == -INFINITY) ? 0.f : exp2f(s_m[gi] - m);
        const float4 a = *reinterpret_cast<const float4*>(&s_o[gi][tid * 4]);
        l = fmaf(s_l[gi], e, l);
        o.x = fmaf(a.x, e, o.x);
        o.y = fmaf(a.y, e, o.y);
        o.z = fmaf(a.z, e, o.z);
        o.w = fmaf(a.w, e, o.w);
      }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat162 lo = __floats2bfloat162_rn(o.x * inv, o.y * inv);
    __nv_bfloat162 hi = __floats2bfloat162_rn(o.z * inv, o.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + (int64_t(r) * H + h) * kDV + tid * 4) = pk;
  }
  DSA_KTIME_END(3);
}

// The same merge for many (row, head) pairs with at most eight splits each (large
// batches): one thread per four output columns, every load of a thread in flight
// at once, no shared memory. Splits are folded in ascending order.
constexpr int kFlatMaxSplit = 8;
__global__ void __launch_bounds__(256)
sparse_mla_combine_flat_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_m,
                               const float* __restrict__ part_l, __nv_bfloat16* __restrict__ out, int H,
                               int nsplit, int64_t n_pairs) {
  DSA_KTIME_BEGIN(3);
  pdl_wait();
  pdl_launch_dependents();
  const int64_t gid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t pair = gid >> 7;  // row * H + head
  const int c4 = int(gid & 127);
  if (pair < n_pairs) {
    const int64_t r = pair / H, h = pair % H;
    float ms[kFlatMaxSplit], ls[kFlatMaxSplit];
    float4 a[kFlatMaxSplit];
#pragma unroll
    for (int u = 0; u < kFlatMaxSplit; ++u) {
      const bool ok = u < nsplit;
      const int64_t row = (r * nsplit + u) * H + h;
      ms[u] = ok ? part_m[row] : -INFINITY;
      ls[u] = ok ? part_l[row] : 0.f;
      a[u] = ok ? *reinterpret_cast<const float4*>(part_acc + row * kDV + c4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float m = ms[0];
#pragma unroll
    for (int u = 1; u < kFlatMaxSplit; ++u) m = fmaxf(m, ms[u]);
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    float l = 0.f;
    if (m != -INFINITY) {
#pragma unroll
      for (int u = 0; u < kFlatMaxSplit; ++u) {
        const float e = (ms[u] == -INFINITY) ? 0.f : exp2f(ms[u] - m);
        l = fmaf(ls[u], e, l);
        o.x = fmaf(a[u].x, e, o.x);
        o.y = fmaf(a[u].y, e, o.y);
        o.z = fmaf(a[u].z, e, o.z);
        o.w = fmaf(a[u].w, e, o.w);
      }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat162 lo = __floats2bfloat162_rn(o.x * inv, o.y * inv);
    __nv_bfloat162 hi = __floats2bfloat162_rn(o.z * inv, o.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + pair * kDV + c4 * 4) = pk;
  }
  DSA_KTIME_END(3);
}

// fp32 attention for any head / latent width: one CTA per (row, head), keys in
// chunks of 128 with an online softmax. indices == nullptr attends [0, len).
__global__ void __launch_bounds__(128)
sparse_mla_f32_kernel(const float* __restrict__ q, const float* __restrict__ kv,
                      const int32_t* __restrict__ indices, const int32_t* __restrict__ seq_lens,
                      float* __restrict__ out, int rows_per_seq, int H, int qk_dim, int v_dim,
                      int topk, float sm_scale, int64_t kv_seq_stride, int64_t ctx) {
  extern __shared__ float s_f[];  // q[qk_dim] | p[128] | idx[128] (as int) | red[8]
  float* s_qv = s_f;
  float* s_pv = s_f + qk_dim;
  int* s_idx = reinterpret_cast<int*>(s_pv + 128);
  float* s_r = reinterpret_cast<float*>(s_idx + 128);
  const int h = blockIdx.x, r = blockIdx.y, tid = threadIdx.x;
  const int seq = r / rows_per_seq;
  int64_t len = seq_lens ? int64_t(seq_lens[r]) : ctx;
  len = len < 0 ? 0 : (len > ctx ? ctx : len);
  const float* kvs = kv + int64_t(seq) * kv_seq_stride * qk_dim;
  for (int i = tid; i < qk_dim; i += 128) s_qv[i] = q[(int64_t(r) * H + h) * qk_dim + i];
  const int64_t n_keys = indices ? int64_t(topk) : len;
  float m_run = -INFINITY, l_run = 0.f;
  float o[4] = {0.f, 0.f, 0.f, 0.f};  // value columns tid, tid+128, ...
  __syncthreads();
  for (int64_t c0 = 0; c0 < n_keys; c0 += 128) {
    const int64_t j = c0 + tid;
    int64_t idx = -1;
    if (j < n_keys) idx = indices ? int64_t(indices[int64_t(r) * topk + j]) : j;
    const bool ok = idx >= 0 && idx < len;
    float s = -INFINITY;
    if (ok) {
      const float* kr = kvs + idx * qk_dim;
      float d = 0.f;
      for (int i = 0; i < qk_dim; ++i) d = fmaf(s_qv[i], kr[i], d);
      s = d * sm_scale;
    }
    // chunk max
    float mx = s;
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, of));
    if ((tid & 31) == 0) s_r[tid >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(s_r[0], s_r[1]), fmaxf(s_r[2], s_r[3]));
    const float m_new = fmaxf(m_run, mx);
    const float pj = (ok && m_new != -INFINITY) ? expf(s - m_new) : 0.f;
    s_pv[tid] = pj;
    s_idx[tid] = ok ? int(idx) : -1;
    float ps = pj;
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, of);
    if ((tid & 31) == 0) s_r[4 + (tid >> 5)] = ps;
    __syncthreads();
    ps = s_r[4] + s_r[5] + s_r[6] + s_r[7];
    const float alpha = (m_new == -INFINITY) ? 1.f : expf(m_run - m_new);
    l_run = l_run * alpha + ps;
    m_run = m_new;
#pragma unroll
    for (int c = 0; c < 4; ++c) o[c] *= alpha;
    for (int jj = 0; jj < 128; ++jj) {
      const int id = s_idx[jj];
      if (id < 0) continue;
      const float pw = s_pv[jj];
      const float* vr = kvs + int64_t(id) * qk_dim;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int col = tid + c * 128;
        if (col < v_dim) o[c] = fmaf(pw, vr[col], o[c]);
      }
    }
    __syncthreads();
  }
  const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int col = tid + c * 128;
    if (col < v_dim) out[(int64_t(r) * H + h) * v_dim + col] = o[c] * inv;
  }
}

}  // namespace mla
}  // namespace dsa
