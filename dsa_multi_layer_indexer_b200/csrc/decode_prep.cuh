// Decode-step preparation fused into two small kernels: RMSNorm, and the chain
// that sits between the projection GEMVs and the hot path (RoPE, per-row e4m3
// quantisation with the query scale folded into the head weights, append of the
// new token's index key and latent row to the caches, assembly of the absorbed
// query). In the reference this is a string of small torch launches
// (inference/modeling/transformer.py:1015-1066 stage_fp8_operands, :1137-1144,
// :3268-3276; ~30 us on the indexer branch, sglang_overlay/...patch:3951-3953);
// here each item is one warp's work and all items of a step share one launch.
#pragma once

#include "common.cuh"

namespace dsa {
namespace prep {

// ------------------------------------------------------------------ RMSNorm
// out = x * rsqrt(mean(x^2) + eps) * weight, fp32 math, one rounding
// (src/lagged_indexer_dsa/dsa_layer.py:42-52). One CTA of 256 threads per row.
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ weight, T* __restrict__ out, int dim, float eps) {
  __shared__ float s_part[8];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * dim;
  pdl_wait();
  pdl_launch_dependents();
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += 256) {
    const float v = to_f32<T>(xr[i]);
    ss = fmaf(v, v, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += s_part[w];
  const float inv = rsqrtf(tot / float(dim) + eps);
  for (int i = threadIdx.x; i < dim; i += 256)
    out[row * dim + i] = from_f32<T>(to_f32<T>(xr[i]) * inv * to_f32<T>(weight[i]));
}

// bf16 rows of up to 8192 elements (a multiple of 8): each of the 256 threads keeps its
// 16-byte pieces of the row in registers, so the row is read once. With kAdd the
// kernel first forms s = x + delta (rounded to bf16 as the separate addition would
// be, and written to sum_out) and normalises s: the residual addition and the norm
// that follows it in a decoder layer (src/lagged_indexer_dsa/model.py:137-138,
// dsa_layer.py:42-52) become one launch.
constexpr int kNormVecPerThread = 4;
constexpr int kNormMaxDim = 256 * kNormVecPerThread * 8;
template <bool kAdd>
__global__ void __launch_bounds__(256)
rmsnorm_bf16_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                         const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ sum_out,
                         __nv_bfloat16* __restrict__ out, int dim, float eps) {
  __shared__ float s_part[8];
  const int64_t row = blockIdx.x;
  const int nvec = dim >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
  const uint4* dr = kAdd ? reinterpret_cast<const uint4*>(delta + row * dim) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(weight);
  pdl_wait();
  pdl_launch_dependents();
  uint4 xv[kNormVecPerThread], wv[kNormVecPerThread], dv[kNormVecPerThread];
#pragma unroll
  for (int k = 0; k < kNormVecPerThread; ++k) {
    const int i = threadIdx.x + 256 * k;
    xv[k] = wv[k] = dv[k] = make_uint4(0, 0, 0, 0);
    if (i < nvec) {
      xv[k] = xr[i];
      wv[k] = wr[i];
      if (kAdd) dv[k] = dr[i];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < kNormVecPerThread; ++k) {
    __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&xv[k]);
    if (kAdd) {
      const __nv_bfloat162* dp = reinterpret_cast<const __nv_bfloat162*>(&dv[k]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = __bfloat1622float2(xp[e]), b = __bfloat1622float2(dp[e]);
        xp[e] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
      }
      const int i = threadIdx.x + 256 * k;
      if (i < nvec) reinterpret_cast<uint4*>(sum_out + row * dim)[i] = xv[k];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(xp[e]);
      ss = fmaf(a.x, a.x, ss);
      ss = fmaf(a.y, a.y, ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += s_part[w];
  const float inv = rsqrtf(tot / float(dim) + eps);
#pragma unroll
  for (int k = 0; k < kNormVecPerThread; ++k) {
    const int i = threadIdx.x + 256 * k;
    if (i >= nvec) continue;
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv[k]);
    const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv[k]);
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(xp[e]), w2 = __bfloat1622float2(wp[e]);
      op[e] = __floats2bfloat162_rn(a.x * inv * w2.x, a.y * inv * w2.y);
    }
    reinterpret_cast<uint4*>(out + row * dim)[i] = o;
  }
}

// out = silu(gate) * up, elementwise over bf16 (the SwiGLU between the MLP's GEMVs,
// src/lagged_indexer_dsa/dsa_layer.py:194-196), with the roundings of the two separate
// operations: silu in fp32 rounded to bf16, then the product rounded to bf16.
__global__ void __launch_bounds__(256)
silu_mul_bf16_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                     __nv_bfloat16* __restrict__ out, int64_t n) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t i = (int64_t(blockIdx.x) * 256 + threadIdx.x) * 8;
  if (i + 8 <= n) {
    const uint4 g = *reinterpret_cast<const uint4*>(gate + i), u = *reinterpret_cast<const uint4*>(up + i);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* upp = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(gp[e]), b = __bfloat1622float2(upp[e]);
      const __nv_bfloat162 s2 = __floats2bfloat162_rn(a.x / (1.f + __expf(-a.x)), a.y / (1.f + __expf(-a.y)));
      const float2 sf = __bfloat1622float2(s2);
      op[e] = __floats2bfloat162_rn(sf.x * b.x, sf.y * b.y);
    }
    *reinterpret_cast<uint4*>(out + i) = o;
  } else {
    for (int64_t j = i; j < n; ++j) {
      const float a = __bfloat162float(gate[j]);
      const float sr = __bfloat162float(__float2bfloat16_rn(a / (1.f + __expf(-a))));
      out[j] = __float2bfloat16_rn(sr * __bfloat162float(up[j]));
    }
  }
}

// ------------------------------------------------------------------ small copies
// dst[0, n) = src[0, n) in 16-byte pieces. Either side may be pinned host memory (it is
// mapped into the device's address space): a kernel node starts sooner than a copy-engine
// node inside a CUDA graph, which matters for the few KB a decode step brings from the host.
__global__ void __launch_bounds__(256)
copy16_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int64_t n16) {
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < n16; i += int64_t(gridDim.x) * 256) dst[i] = src[i];
}

// The same copy for data that the kernel enqueued just before it neither produces nor reads
// (a step's queries coming from the host while the selection is still being computed): it
// copies at once, beside that kernel, and only then waits for it, so it still completes after
// it and the kernel enqueued next, whose own wait is for this grid, sees both. A copy in the
// stream's chain of programmatic dependents, where a copy on a forked stream would cost a join.
__global__ void __launch_bounds__(256)
copy16_beside_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int64_t n16) {
  pdl_launch_dependents();
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < n16; i += int64_t(gridDim.x) * 256) dst[i] = src[i];
  pdl_wait();
}

// Completion signal for a host that polls instead of synchronising: bumps a device-side
// epoch counter and posts the new value to a word of pinned host memory, after a
// system-wide fence so that everything the stream wrote to host memory before this
// launch is visible first.
__global__ void post_epoch_kernel(uint32_t* __restrict__ counter, volatile uint32_t* __restrict__ host_flag) {
  pdl_wait();
  const uint32_t e = *counter + 1;
  *counter = e;
  __threadfence_system();
  *host_flag = e;
}

// The same signal with a last small copy in front of it (a step's selection, a few KB, into
// pinned host memory): one node at the end of a step's graph instead of a copy on a forked
// stream, a join and the signal. One CTA; the block barrier orders every thread's copy before
// thread 0's system-wide fence. Launched as a programmatic dependent: it is resident and waiting
// when the kernel before it retires.
// With `beside` the bytes do not come from the kernel enqueued just before (the selection, while
// the merge kernel runs): they are copied first, beside that kernel, and the wait comes after the
// copy, so that by the time of the fence these writes have long left for the host.
__global__ void __launch_bounds__(512)
copy_post_epoch_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int64_t n16,
                       uint32_t* __restrict__ counter, volatile uint32_t* __restrict__ host_flag, int beside) {
  if (!beside) pdl_wait();
  for (int64_t i = threadIdx.x; i < n16; i += 512) dst[i] = src[i];
  if (beside) pdl_wait();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t e = *counter + 1;
    *counter = e;
    __threadfence_system();
    *host_flag = e;
  }
}

// ------------------------------------------------------------------ skinny GEMV
// y[b, n] = sum_k W[n, k] x[b, k] for 1..4 rows of x (decode batch): bf16 operands,
// fp32 accumulation, one rounding. The weight matrix is streamed once with 16-byte
// loads, eight per lane in flight, x staged in shared memory. This is the
// projection GEMV of a decode step (src/lagged_indexer_dsa/dsa_layer.py:87-125) for
// the shapes where the library GEMV is latency-bound (a few thousand output rows).
constexpr int kGemvThreads = 256;
constexpr int kGemvLoads = 8;  // independent 16-byte weight loads per lane per step
// R rows per warp, kGemvLoads / R consecutive 512-byte column blocks per step: the
// launch picks R so that there are enough warps to fill the machine.
template <int B, int R>
__global__ void __launch_bounds__(kGemvThreads)
gemv_bf16_kernel(const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ x,
                 __nv_bfloat16* __restrict__ y, int n, int k, int64_t x_stride, int64_t y_stride) {
  constexpr int UK = kGemvLoads / R;
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  uint4* s_x = reinterpret_cast<uint4*>(gemv_smem);  // [B][k / 8]
  const int kv = k >> 3;
  pdl_wait();
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < B * kv; i += kGemvThreads) {
    const int b = i / kv, c = i - b * kv;
    s_x[i] = *reinterpret_cast<const uint4*>(x + b * x_stride + c * 8);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp_global = (blockIdx.x * kGemvThreads + threadIdx.x) >> 5;
  const int n_warps = (gridDim.x * kGemvThreads) >> 5;
  for (int row0 = warp_global * R; row0 < n; row0 += n_warps * R) {
    float acc[R][B];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
    for (int c0 = lane; c0 < kv; c0 += 32 * UK) {
      uint4 wv[R][UK];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint4* wrow = reinterpret_cast<const uint4*>(w + int64_t(min(row0 + r, n - 1)) * k);
#pragma unroll
        for (int u = 0; u < UK; ++u) {
          const int c = c0 + 32 * u;
          wv[r][u] = c < kv ? __ldcs(wrow + c) : make_uint4(0, 0, 0, 0);  // streamed once
        }
      }
#pragma unroll
      for (int u = 0; u < UK; ++u) {
        const int c = min(c0 + 32 * u, kv - 1);
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const uint4 xv = s_x[b * kv + c];
          const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv[r][u]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 a = __bfloat1622float2(wp[e]), v = __bfloat1622float2(xp[e]);
              acc[r][b] = fmaf(a.x, v.x, acc[r][b]);
              acc[r][b] = fmaf(a.y, v.y, acc[r][b]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int b = 0; b < B; ++b) {
        float v = acc[r][b];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && row0 + r < n) y[b * y_stride + row0 + r] = __float2bfloat16_rn(v);
      }
  }
}

// ------------------------------------------------------------------ decode prep
struct Params {
  // inputs (bf16, outputs of the projection GEMVs), B rows
  const __nv_bfloat16* iq_raw;   // [B, Hidx, 128]  index_q_proj(c_q)
  const __nv_bfloat16* w_raw;    // [B, Hidx]       index_weights_proj(c_q)
  const __nv_bfloat16* ik_raw;   // [B, 128]        index_k_proj(x_norm)
  const __nv_bfloat16* kv_a;     // [B, 576]        kv_a_proj(x_norm): 512 latent | 64 rope
  const __nv_bfloat16* q_abs;    // [B, H, 512]     q_nope absorbed through W_UK
  const __nv_bfloat16* q_pe;     // [B, H, 64] with row stride q_pe_stride (elements): rope part of q_b_proj
  const __nv_bfloat16* kv_norm_w;  // [512] kv_a_layernorm weight
  const __nv_bfloat16* mla_cos;  // [cap, 64]
  const __nv_bfloat16* mla_sin;
  const __nv_bfloat16* idx_cos;  // [cap, 128]
  const __nv_bfloat16* idx_sin;
  const int64_t* positions;      // [B] position of the new token
  // outputs
  uint8_t* index_q;              // [B, Hidx, 128] e4m3
  float* index_w;                // [B, Hidx] = q scale * w_raw
  __nv_bfloat16* q_full;         // [B, H, 576]
  uint8_t* cache_index_k;        // [B, cap, 128] e4m3
  float* cache_k_scale;          // [B, cap]
  __nv_bfloat16* cache_kv;       // [B, cap, 576]
  int64_t cap;
  int64_t q_pe_stride;
  int B, H, Hidx;
  int interleave;                // indexer RoPE pairing (GLM-5) vs half split (DeepSeek)
  float eps;
};

// RoPE of 4 consecutive dims [4 lane, 4 lane + 4) of a 128-wide vector held one
// quad per lane; fp32 in, fp32 out. Half-split pairs dim i with i +- 64 (lane ^ 16).
__device__ __forceinline__ void rope128(float (&v)[4], const __nv_bfloat16* cosr, const __nv_bfloat16* sinr,
                                        int lane, bool interleave) {
  float c[4], s[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    c[j] = __bfloat162float(cosr[4 * lane + j]);
    s[j] = __bfloat162float(sinr[4 * lane + j]);
  }
  float o[4];
  if (interleave) {
    o[0] = v[0] * c[0] - v[1] * s[0];
    o[1] = v[1] * c[1] + v[0] * s[1];
    o[2] = v[2] * c[2] - v[3] * s[2];
    o[3] = v[3] * c[3] + v[2] * s[3];
  } else {
    const float sign = lane < 16 ? -1.f : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float partner = __shfl_xor_sync(0xffffffffu, v[j], 16);
      o[j] = v[j] * c[j] + sign * partner * s[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = o[j];
}

// Per-row absmax e4m3 quantisation of a 128-wide vector (4 per lane): returns
// the packed 4 bytes of this lane and the row scale (same on all lanes).
__device__ __forceinline__ uint32_t quant128(const float (&v)[4], float& scale) {
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  scale = fmaxf(amax, 1e-6f) / 448.0f;
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float q = fminf(fmaxf(v[j] / scale, -448.f), 448.f);
    packed |= uint32_t(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
  }
  return packed;
}

__global__ void __launch_bounds__(128)
decode_prep_kernel(const Params p) {
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int b = blockIdx.y;
  const int n_items = p.Hidx + 2 + p.H;
  if (item >= n_items) return;
  pdl_wait();
  pdl_launch_dependents();
  const int64_t pos = p.positions[b];
  if (pos < 0 || pos >= p.cap) return;

  if (item < p.Hidx) {
    // ---- one indexer query head: RoPE, quantise, fold the scale into the head weight
    const int h = item;
    const __nv_bfloat16* src = p.iq_raw + (int64_t(b) * p.Hidx + h) * 128 + 4 * lane;
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float v[4] = {__bfloat162float(lo.x), __bfloat162float(lo.y), __bfloat162float(hi.x), __bfloat162float(hi.y)};
    rope128(v, p.idx_cos + pos * 128, p.idx_sin + pos * 128, lane, p.interleave != 0);
    float scale;
    const uint32_t q = quant128(v, scale);
    *reinterpret_cast<uint32_t*>(p.index_q + (int64_t(b) * p.Hidx + h) * 128 + 4 * lane) = q;
    if (lane == 0) p.index_w[int64_t(b) * p.Hidx + h] = scale * __bfloat162float(p.w_raw[int64_t(b) * p.Hidx + h]);
  } else if (item == p.Hidx) {
    // ---- the new token's index key: RoPE, quantise, append
    const uint2 raw = *reinterpret_cast<const uint2*>(p.ik_raw + int64_t(b) * 128 + 4 * lane);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float v[4] = {__bfloat162float(lo.x), __bfloat162float(lo.y), __bfloat162float(hi.x), __bfloat162float(hi.y)};
    rope128(v, p.idx_cos + pos * 128, p.idx_sin + pos * 128, lane, p.interleave != 0);
    float scale;
    const uint32_t q = quant128(v, scale);
    *reinterpret_cast<uint32_t*>(p.cache_index_k + (int64_t(b) * p.cap + pos) * 128 + 4 * lane) = q;
    if (lane == 0) p.cache_k_scale[int64_t(b) * p.cap + pos] = scale;
  } else if (item == p.Hidx + 1) {
    // ---- the new token's latent row: RMSNorm(512) | RoPE(64), append
    const __nv_bfloat16* src = p.kv_a + int64_t(b) * 576;
    __nv_bfloat16* dst = p.cache_kv + (int64_t(b) * p.cap + pos) * 576;
    float v[16];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] = __bfloat162float(src[lane + 32 * j]);
      ss = fmaf(v[j], v[j], ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / 512.f + p.eps);
#pragma unroll
    for (int j = 0; j < 16; ++j)
      dst[lane + 32 * j] = __float2bfloat16_rn(v[j] * inv * __bfloat162float(p.kv_norm_w[lane + 32 * j]));
    // rope part: dims 512 + [0, 64), half split pairs i with i +- 32 (lane ^ 16 holds it)
    const float a0 = __bfloat162float(src[512 + 2 * lane]), a1 = __bfloat162float(src[512 + 2 * lane + 1]);
    const float p0 = __shfl_xor_sync(0xffffffffu, a0, 16), p1 = __shfl_xor_sync(0xffffffffu, a1, 16);
    const float sign = lane < 16 ? -1.f : 1.f;
    const __nv_bfloat16* cr = p.mla_cos + pos * 64 + 2 * lane;
    const __nv_bfloat16* sr = p.mla_sin + pos * 64 + 2 * lane;
    dst[512 + 2 * lane] = __float2bfloat16_rn(a0 * __bfloat162float(cr[0]) + sign * p0 * __bfloat162float(sr[0]));
    dst[512 + 2 * lane + 1] = __float2bfloat16_rn(a1 * __bfloat162float(cr[1]) + sign * p1 * __bfloat162float(sr[1]));
  } else {
    // ---- one MLA query head: absorbed 512 dims copied, rope part rotated
    const int h = item - p.Hidx - 2;
    const uint4* src = reinterpret_cast<const uint4*>(p.q_abs + (int64_t(b) * p.H + h) * 512);
    __nv_bfloat16* dst = p.q_full + (int64_t(b) * p.H + h) * 576;
    uint4* dst4 = reinterpret_cast<uint4*>(dst);
    dst4[lane] = src[lane];            // 64 x 16 B = 512 bf16
    dst4[lane + 32] = src[lane + 32];
    const __nv_bfloat16* pe = p.q_pe + (int64_t(b) * p.H + h) * p.q_pe_stride;
    const float a0 = __bfloat162float(pe[2 * lane]), a1 = __bfloat162float(pe[2 * lane + 1]);
    const float p0 = __shfl_xor_sync(0xffffffffu, a0, 16), p1 = __shfl_xor_sync(0xffffffffu, a1, 16);
    const float sign = lane < 16 ? -1.f : 1.f;
    const __nv_bfloat16* cr = p.mla_cos + pos * 64 + 2 * lane;
    const __nv_bfloat16* sr = p.mla_sin + pos * 64 + 2 * lane;
    dst[512 + 2 * lane] = __float2bfloat16_rn(a0 * __bfloat162float(cr[0]) + sign * p0 * __bfloat162float(sr[0]));
    dst[512 + 2 * lane + 1] = __float2bfloat16_rn(a1 * __bfloat162float(cr[1]) + sign * p1 * __bfloat162float(sr[1]));
  }
}

// ------------------------------------------------------------------ serving-form indexer staging
// Everything the serving model's indexer does to the new token between its
// projection GEMVs and the scan (inference/modeling/transformer.py:1015-1066):
//   q = wq_b(qr) [B, heads, 128], k = wk(x) [B, 128], w = weights_proj(x.float())
//   k <- LayerNorm(k) in fp32, rounded to bf16                      (:418-433, :1052)
//   rotary embedding of the first 64 dims in fp32, rounded to bf16  (:525-547),
//     pairs (2i, 2i+1) when interleaved, (i, i+32) otherwise
//   128-point Walsh-Hadamard butterfly in fp32, times 128^-0.5, rounded to bf16
//     (:550-568, :571-592)
//   act_quant over the 128 dims: amax = max(|x|, 1e-4), scale = amax / 448 or, with a
//     scale format, 2^ceil(log2(amax / 448)); e4m3(x / scale)       (kernels.py:19-117)
//   q bytes -> index_q, head weight = w * heads^-0.5 * q_scale * softmax_scale (:1063-1065)
//   k bytes and scale -> the key cache at the token's position (:1062-1063), dense
//     [B, cap, 128] + [B, cap] or 64-token pages of 8448 bytes.
// One warp per 128-wide row (lane l holds dims 4l .. 4l+3); every product and sum is
// rounded on its own (no fused multiply-add) so the arithmetic matches the reference's
// elementwise torch ops.
struct StageParams {
  const __nv_bfloat16* q_raw;
  const __nv_bfloat16* k_raw;
  const float* w_raw;
  const float* norm_w;
  const float* norm_b;
  const float* rope_cos;  // [cap, 32] real part of the rotary table
  const float* rope_sin;  // [cap, 32] imaginary part
  const int64_t* positions;
  uint8_t* index_q;
  float* index_w;
  uint8_t* cache_index_k;
  float* cache_k_scale;
  uint8_t* pages;
  const int32_t* page_table;
  int64_t pt_stride;
  int64_t num_pages;
  int64_t cap;
  int B, n_heads, interleave, round_scale;
  float eps, head_scale, softmax_scale, hadamard_scale;
};

constexpr int kStageWarps = 8;

__global__ void __launch_bounds__(kStageWarps * 32)
indexer_stage_kernel(const StageParams p) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kStageWarps + (threadIdx.x >> 5);
  const int rows_per_b = p.n_heads + 1;
  const int b = row / rows_per_b, item = row % rows_per_b;
  if (b >= p.B) return;
  pdl_wait();
  pdl_launch_dependents();
  const int64_t pos = p.positions[b];
  if (pos < 0 || pos >= p.cap) return;
  const bool is_key = item == p.n_heads;
  const __nv_bfloat16* src = is_key ? p.k_raw + int64_t(b) * 128 : p.q_raw + (int64_t(b) * p.n_heads + item) * 128;
  const uint2 raw = *reinterpret_cast<const uint2*>(src + 4 * lane);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  float v[4] = {__bfloat162float(lo.x), __bfloat162float(lo.y), __bfloat162float(hi.x), __bfloat162float(hi.y)};
  auto round_bf16 = [](float x) { return __bfloat162float(__float2bfloat16_rn(x)); };

  if (is_key) {  // LayerNorm over the 128 dims: biased variance, weight and bias in fp32
    float s = __fadd_rn(__fadd_rn(v[0], v[1]), __fadd_rn(v[2], v[3]));
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
    const float mean = __fdiv_rn(s, 128.f);
    float d[4], ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      d[j] = __fsub_rn(v[j], mean);
      ss = __fadd_rn(ss, __fmul_rn(d[j], d[j]));
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    const float rstd = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.f), p.eps)));
    const float4 w4 = *reinterpret_cast<const float4*>(p.norm_w + 4 * lane);
    const float4 b4 = *reinterpret_cast<const float4*>(p.norm_b + 4 * lane);
    const float w[4] = {w4.x, w4.y, w4.z, w4.w}, bb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = round_bf16(__fadd_rn(__fmul_rn(__fmul_rn(d[j], rstd), w[j]), bb[j]));
  }

  {  // rotary embedding of dims 0..63 (lanes 0..15); complex product (a + bi)(c + si)
    const float* cr = p.rope_cos + pos * 32;
    const float* sr = p.rope_sin + pos * 32;
    float partner[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) partner[j] = __shfl_xor_sync(0xffffffffu, v[j], 8);
    if (lane < 16) {
      if (p.interleave) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const float c = cr[2 * lane + u], s = sr[2 * lane + u];
          const float a = v[2 * u], bi = v[2 * u + 1];
          v[2 * u] = round_bf16(__fsub_rn(__fmul_rn(a, c), __fmul_rn(bi, s)));
          v[2 * u + 1] = round_bf16(__fadd_rn(__fmul_rn(a, s), __fmul_rn(bi, c)));
        }
      } else {
        const bool first = lane < 8;  // dims 0..31 are the real parts, 32..63 the imaginary parts
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i = 4 * (lane & 7) + j;
          const float c = cr[i], s = sr[i];
          const float a = first ? v[j] : partner[j], bi = first ? partner[j] : v[j];
          v[j] = first ? round_bf16(__fsub_rn(__fmul_rn(a, c), __fmul_rn(bi, s)))
                       : round_bf16(__fadd_rn(__fmul_rn(a, s), __fmul_rn(bi, c)));
        }
      }
    }
  }

  {  // Walsh-Hadamard butterfly: strides 1, 2 inside the lane, 4 .. 64 across lanes
    float t0 = __fadd_rn(v[0], v[1]), t1 = __fsub_rn(v[0], v[1]);
    float t2 = __fadd_rn(v[2], v[3]), t3 = __fsub_rn(v[2], v[3]);
    v[0] = __fadd_rn(t0, t2);
    v[2] = __fsub_rn(t0, t2);
    v[1] = __fadd_rn(t1, t3);
    v[3] = __fsub_rn(t1, t3);
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
      const bool upper = (lane & m) != 0;  // this lane holds the element with the stride bit set
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j], m);
        v[j] = upper ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = round_bf16(__fmul_rn(v[j], p.hadamard_scale));
  }

  // act_quant over the row
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax = fmaxf(amax, 1e-4f);
  float scale = __fmul_rn(amax, 1.0f / 448.0f);
  if (p.round_scale) {  // next power of two at or above amax / 448
    const uint32_t bits = __float_as_uint(scale);
    const int e = int((bits >> 23) & 0xFFu) - 127 + ((bits & 0x7FFFFFu) != 0u ? 1 : 0);
    scale = __uint_as_float(uint32_t(e + 127) << 23);
  }
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float q = fminf(fmaxf(__fdiv_rn(v[j], scale), -448.f), 448.f);
    packed |= uint32_t(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
  }
  if (!is_key) {
    *reinterpret_cast<uint32_t*>(p.index_q + (int64_t(b) * p.n_heads + item) * 128 + 4 * lane) = packed;
    if (lane == 0) {
      const float w = p.w_raw[int64_t(b) * p.n_heads + item];
      p.index_w[int64_t(b) * p.n_heads + item] =
          __fmul_rn(__fmul_rn(__fmul_rn(w, p.head_scale), scale), p.softmax_scale);
    }
  } else if (p.pages) {
    // a stale or negative page-table entry must not become a wild write: skip the token and say so
    const int32_t page = (pos >> 6) < p.pt_stride ? p.page_table[int64_t(b) * p.pt_stride + (pos >> 6)] : -1;
    if (page < 0 || int64_t(page) >= p.num_pages) {
      if (lane == 0) atomicOr(&g_device_status, kStatusBadPage);
      return;
    }
    uint8_t* pg = p.pages + int64_t(page) * DSA_INDEX_PAGE_BYTES;
    const int slot = int(pos & 63);
    *reinterpret_cast<uint32_t*>(pg + slot * 128 + 4 * lane) = packed;
    if (lane == 0) *reinterpret_cast<float*>(pg + DSA_PAGE_TOKENS * 128 + slot * 4) = scale;
  } else {
    *reinterpret_cast<uint32_t*>(p.cache_index_k + (int64_t(b) * p.cap + pos) * 128 + 4 * lane) = packed;
    if (lane == 0) p.cache_k_scale[int64_t(b) * p.cap + pos] = scale;
  }
}

// ------------------------------------------------------------------ serving-form latent append
// The new token's latent row between wkv_a and the cache
// (inference/modeling/transformer.py:3264-3276): RMSNorm of the 512 latent dims
// (fp32 weight, :380-410), rotary embedding of the 64 rope dims (:525-547), then one of
//   format 0: the bf16 row [512 | 64] as it is,
//   format 1: the same row with the latent dims passed through act_quant and back
//             (e4m3 with one scale per 128 dims, dequantised and rounded to bf16: the
//             reference's bf16 cache holds these values, :3268-3274),
//   format 2: the serving pool's 656-byte row: 512 e4m3 | 4 fp32 scales | 64 bf16
//             (kernels/cuda_fused_sparse_splitk.py:1098-1104),
// written at slots[b] of the pool. One warp per token; lane l holds dims 4l..4l+3 of
// each 128-dim group, so a group's amax is one warp reduction.
struct LatentParams {
  const __nv_bfloat16* kv_a;  // [B, 576]
  const float* norm_w;        // [512]
  const float* rope_cos;      // [cap, 32]
  const float* rope_sin;
  const int64_t* positions;
  const int64_t* slots;
  uint8_t* pool;
  int64_t cap, n_slots;
  int B, interleave, format, round_scale;
  float eps;
};

__global__ void __launch_bounds__(kStageWarps * 32)
latent_append_kernel(const LatentParams p) {
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.x * kStageWarps + (threadIdx.x >> 5);
  if (b >= p.B) return;
  pdl_wait();
  pdl_launch_dependents();
  const int64_t pos = p.positions[b], slot = p.slots[b];
  if (pos < 0 || pos >= p.cap || slot < 0 || slot >= p.n_slots) return;
  auto round_bf16 = [](float x) { return __bfloat162float(__float2bfloat16_rn(x)); };
  const __nv_bfloat16* src = p.kv_a + int64_t(b) * 576;
  float v[4][4];
  float ss = 0.f;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src + 128 * g + 4 * lane);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    v[g][0] = __bfloat162float(lo.x);
    v[g][1] = __bfloat162float(lo.y);
    v[g][2] = __bfloat162float(hi.x);
    v[g][3] = __bfloat162float(hi.y);
#pragma unroll
    for (int j = 0; j < 4; ++j) ss = __fadd_rn(ss, __fmul_rn(v[g][j], v[g][j]));
  }
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
  const float rstd = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 512.f), p.eps)));
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const float4 w4 = *reinterpret_cast<const float4*>(p.norm_w + 128 * g + 4 * lane);
    const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) v[g][j] = round_bf16(__fmul_rn(w[j], __fmul_rn(v[g][j], rstd)));
  }
  // rope dims: 2 per lane; pair layout as in indexer_stage_kernel
  float r0 = __bfloat162float(src[512 + 2 * lane]), r1 = __bfloat162float(src[512 + 2 * lane + 1]);
  {
    const float* cr = p.rope_cos + pos * 32;
    const float* sr = p.rope_sin + pos * 32;
    const float q0 = __shfl_xor_sync(0xffffffffu, r0, 16), q1 = __shfl_xor_sync(0xffffffffu, r1, 16);
    if (p.interleave) {
      const float c = cr[lane], s = sr[lane];
      const float a = r0, bi = r1;
      r0 = round_bf16(__fsub_rn(__fmul_rn(a, c), __fmul_rn(bi, s)));
      r1 = round_bf16(__fadd_rn(__fmul_rn(a, s), __fmul_rn(bi, c)));
    } else {
      const bool first = lane < 16;  // dims 0..31 real parts, 32..63 imaginary parts
      const int i = 2 * (lane & 15);
      const float a0 = first ? r0 : q0, b0 = first ? q0 : r0, a1 = first ? r1 : q1, b1 = first ? q1 : r1;
      r0 = first ? round_bf16(__fsub_rn(__fmul_rn(a0, cr[i]), __fmul_rn(b0, sr[i])))
                 : round_bf16(__fadd_rn(__fmul_rn(a0, sr[i]), __fmul_rn(b0, cr[i])));
      r1 = first ? round_bf16(__fsub_rn(__fmul_rn(a1, cr[i + 1]), __fmul_rn(b1, sr[i + 1])))
                 : round_bf16(__fadd_rn(__fmul_rn(a1, sr[i + 1]), __fmul_rn(b1, cr[i + 1])));
    }
  }
  const __nv_bfloat162 rope2 = __halves2bfloat162(__float2bfloat16_rn(r0), __float2bfloat16_rn(r1));
  uint32_t packed[4];
  float scale[4];
  if (p.format != 0) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float amax = fmaxf(fmaxf(fabsf(v[g][0]), fabsf(v[g][1])), fmaxf(fabsf(v[g][2]), fabsf(v[g][3])));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      float sc = __fmul_rn(fmaxf(amax, 1e-4f), 1.0f / 448.0f);
      if (p.round_scale) {
        const uint32_t bits = __float_as_uint(sc);
        const int e = int((bits >> 23) & 0xFFu) - 127 + ((bits & 0x7FFFFFu) != 0u ? 1 : 0);
        sc = __uint_as_float(uint32_t(e + 127) << 23);
      }
      scale[g] = sc;
      packed[g] = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float q = fminf(fmaxf(__fdiv_rn(v[g][j], sc), -448.f), 448.f);
        const uint32_t byte = __nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3);
        packed[g] |= byte << (8 * j);
        if (p.format == 1) {
          const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
          v[g][j] = round_bf16(__fmul_rn(__half2float(__half(hr)), sc));
        }
      }
    }
  }
  if (p.format == 2) {
    uint8_t* row = p.pool + slot * int64_t(DSA_FP8_LATENT_ROW);
#pragma unroll
    for (int g = 0; g < 4; ++g) *reinterpret_cast<uint32_t*>(row + 128 * g + 4 * lane) = packed[g];
    if (lane < 4) *reinterpret_cast<float*>(row + 512 + 4 * lane) = scale[lane];
    *reinterpret_cast<__nv_bfloat162*>(row + 528 + 4 * lane) = rope2;
  } else {
    __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(p.pool) + slot * 576;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      __nv_bfloat162 a = __halves2bfloat162(__float2bfloat16_rn(v[g][0]), __float2bfloat16_rn(v[g][1]));
      __nv_bfloat162 c = __halves2bfloat162(__float2bfloat16_rn(v[g][2]), __float2bfloat16_rn(v[g][3]));
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&a);
      o.y = *reinterpret_cast<uint32_t*>(&c);
      *reinterpret_cast<uint2*>(row + 128 * g + 4 * lane) = o;
    }
    *reinterpret_cast<__nv_bfloat162*>(row + 512 + 2 * lane) = rope2;
  }
}

}  // namespace prep
}  // namespace dsa
