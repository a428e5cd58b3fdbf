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

}  // namespace prep
}  // namespace dsa
