// All-reduce of a small activation vector across the GPUs of one node, written
// for the decode step of a tensor-parallel layer: the partial outputs of the
// row-parallel projections (o_proj, down_proj) are [B, hidden] with B a few
// tokens, i.e. tens of kilobytes. The reference sums them with dist.all_reduce
// in fp32 (src/lagged_indexer_dsa/inference/modeling/transformer.py:361-377,
// :3965). Here the sum is two small launches in stream order, so a decode step
// with its collectives is capturable in one CUDA graph and never calls a
// library from inside it:
//
//   push      every rank converts its partial vector to fp32 and STORES it into
//             slot `rank` of every rank's buffer (plain stores through peer-
//             mapped pointers, 16 bytes each), then posts the step number to
//             its flag word on every rank (release, system scope);
//   wait_sum  waits, bounded by wall time, until all flags carry the step
//             number (acquire), adds the world's slots in rank order (the same
//             order on every rank: the result is bit-identical everywhere),
//             optionally adds a residual, and writes fp32 or bf16.
//
// Two step parities of slots, as in the candidate exchange: a rank one step
// ahead cannot overwrite what a slower rank still reads. No loads from peer
// memory, no multicast. When the wait runs out the kernel sets
// DSA_STATUS_EXCHANGE_TIMEOUT, adds what is there and returns.
#pragma once

#include "common.cuh"

namespace dsa {
namespace ar {

constexpr int kThreads = 1024;
constexpr int kMaxRanks = 8;

struct PushParams {
  const void* src;           // [n] bf16 or fp32
  float* dest[kMaxRanks];    // rank d's slots [2][n_dest][n] as this process addresses them
  uint32_t* dest_flag[kMaxRanks];  // this rank's flag word on rank d
  uint32_t* sent;            // local step counter
  int64_t n;
  int n_dest, src_rank, src_bf16;
};

__global__ void __launch_bounds__(kThreads)
allreduce_push_kernel(const PushParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t step = *p.sent + 1u;
  const int64_t off = (int64_t(step & 1u) * p.n_dest + p.src_rank) * p.n;
  for (int64_t i = int64_t(threadIdx.x) * 4; i < p.n; i += int64_t(kThreads) * 4) {
    float4 v;
    if (p.src_bf16) {
      const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.src) + i);
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      v = make_float4(__bfloat162float(lo.x), __bfloat162float(lo.y), __bfloat162float(hi.x), __bfloat162float(hi.y));
    } else {
      v = *reinterpret_cast<const float4*>(static_cast<const float*>(p.src) + i);
    }
    for (int d = 0; d < p.n_dest; ++d) *reinterpret_cast<float4*>(p.dest[d] + off + i) = v;
  }
  // Behind the block barrier ONE thread fences at system scope and posts the step number to every
  // rank: a release that, being cumulative, also orders the stores of the other threads (which
  // reached this thread through the barrier) before the flags.
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    for (int d = 0; d < p.n_dest; ++d) st_relaxed_sys(p.dest_flag[d], step);
    *p.sent = step;
  }
}

struct SumParams {
  const float* slots;        // [2][n_src][n] local
  const uint32_t* flags;     // [n_src] local, written by the sources
  uint32_t* seen;            // local step counter
  const void* residual;      // optional [n], same type as out
  void* out;                 // [n] bf16 or fp32
  int64_t n;
  unsigned long long wait_limit_ns;
  int n_src, out_bf16;
};

__global__ void __launch_bounds__(kThreads)
allreduce_wait_sum_kernel(const SumParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t step = *p.seen + 1u;
  if (threadIdx.x == 0) {
    const unsigned long long t0 = wall_ns();
    bool ok = false;
    for (uint32_t spin = 0; !ok; ++spin) {
      ok = true;
      for (int s = 0; s < p.n_src; ++s) ok = ok && int32_t(ld_acquire_sys(p.flags + s) - step) >= 0;
      if (!ok && (spin & 63u) == 63u && wall_ns() - t0 > p.wait_limit_ns) break;
    }
    if (!ok) atomicOr(&g_device_status, kStatusExchangeTimeout);
  }
  __syncthreads();
  const float* base = p.slots + int64_t(step & 1u) * p.n_src * p.n;
  for (int64_t i = int64_t(threadIdx.x) * 4; i < p.n; i += int64_t(kThreads) * 4) {
    float4 acc = __ldcg(reinterpret_cast<const float4*>(base + i));
    for (int s = 1; s < p.n_src; ++s) {  // rank order: every rank gets the same bits
      const float4 v = __ldcg(reinterpret_cast<const float4*>(base + int64_t(s) * p.n + i));
      acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
    }
    if (p.out_bf16) {
      if (p.residual) {
        const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.residual) + i);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        // the sum is rounded to bf16 first, as the separate all-reduce and addition would round it
        acc.x = __bfloat162float(__float2bfloat16_rn(acc.x)) + __bfloat162float(lo.x);
        acc.y = __bfloat162float(__float2bfloat16_rn(acc.y)) + __bfloat162float(lo.y);
        acc.z = __bfloat162float(__float2bfloat16_rn(acc.z)) + __bfloat162float(hi.x);
        acc.w = __bfloat162float(__float2bfloat16_rn(acc.w)) + __bfloat162float(hi.y);
      }
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + i) = packed;
    } else {
      if (p.residual) {
        const float4 rr = *reinterpret_cast<const float4*>(static_cast<const float*>(p.residual) + i);
        acc.x += rr.x, acc.y += rr.y, acc.z += rr.z, acc.w += rr.w;
      }
      *reinterpret_cast<float4*>(static_cast<float*>(p.out) + i) = acc;
    }
  }
  if (threadIdx.x == 0) *p.seen = step;
}

}  // namespace ar
}  // namespace dsa
