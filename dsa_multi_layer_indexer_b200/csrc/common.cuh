// Shared host/device helpers for the dsa_b200 kernels: error plumbing, the
// per-device status word, and thin wrappers over the sm_100a PTX this library
// uses (mbarrier, bulk/TMA copies, tcgen05 + tensor memory).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/dsa_b200.h"

namespace dsa {

// ---------------------------------------------------------------- host errors
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);

#define DSA_REQUIRE(cond, ...)                                              \
  do {                                                                      \
    if (!(cond)) return ::dsa::fail(DSA_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define DSA_CUDA(expr)                                                          \
  do {                                                                          \
    cudaError_t e__ = (expr);                                                   \
    if (e__ != cudaSuccess)                                                     \
      return ::dsa::fail(DSA_ERR_CUDA, "%s failed: %s", #expr,                  \
                         cudaGetErrorString(e__));                              \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int sm_count();  // multiprocessors of the current device (cached per device)

// Encodes a tiled tensor map through the driver entry point (no libcuda link).
// dims/strides are innermost-first; strides[0] is implied by elem size.
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle);

// ---------------------------------------------------------------- device status
// Bit set by a kernel whose bounded wait ran out; read by dsa_check_device_status.
// (This library is one translation unit, so the word is simply defined here.)
__device__ unsigned int g_device_status = 0;
constexpr unsigned int kStatusScanTimeout = DSA_STATUS_SCAN_TIMEOUT;
constexpr unsigned int kStatusAttnTimeout = DSA_STATUS_ATTN_TIMEOUT;
constexpr unsigned int kStatusSelectOverflow = DSA_STATUS_SELECT_OVERFLOW;
constexpr unsigned int kStatusBadPage = DSA_STATUS_BAD_PAGE;  // a page-table entry outside [0, num_pages): the access was skipped
constexpr unsigned int kStatusExchangeTimeout = DSA_STATUS_EXCHANGE_TIMEOUT;  // a peer's candidates did not arrive in time

#ifdef __CUDACC__
// ---------------------------------------------------------------- device: phase stamps
// Tracing build only (-DDSA_STAMPS): thread 0 of a CTA records its SM cycle
// counter at numbered phases, read back with dsa_debug_read_stamps. The
// reference has the same facility (kernels/cuda_fused_sparse_splitk.py
// :1076-1090 stamps, :2329-2349 read-back). Compiled out of the normal build.
constexpr int kStampSlots = 16;
constexpr int kStampCtas = 1024;
#ifdef DSA_STAMPS
__device__ unsigned long long g_stamps[kStampCtas * kStampSlots];
#define DSA_STAMP_IF(cond, cta, slot)                                                \
  do {                                                                               \
    if ((cond) && (cta) < ::dsa::kStampCtas)                                         \
      ::dsa::g_stamps[(cta) * ::dsa::kStampSlots + (slot)] = clock64();              \
  } while (0)
// Kernel begin / end wall times (global nanosecond timer), min / max over CTAs,
// stored after the per-CTA stamps: words [kStampCtas*kStampSlots + 2*id, +1].
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ unsigned long long g_ktime[32];
#define DSA_KTIME_BEGIN(id)                                                          \
  do {                                                                               \
    if (threadIdx.x == 0) atomicMin(&::dsa::g_ktime[2 * (id)], ::dsa::global_ns());  \
  } while (0)
#define DSA_KTIME_END(id)                                                                \
  do {                                                                                   \
    if (threadIdx.x == 0) atomicMax(&::dsa::g_ktime[2 * (id) + 1], ::dsa::global_ns());  \
  } while (0)
#else
#define DSA_STAMP_IF(cond, cta, slot) do { } while (0)
#define DSA_KTIME_BEGIN(id) do { } while (0)
#define DSA_KTIME_END(id) do { } while (0)
#endif
#define DSA_STAMP(cta, slot) DSA_STAMP_IF(threadIdx.x == 0, cta, slot)

// ---------------------------------------------------------------- device: misc
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// Shared-memory reductions in the explicit .shared state space (no return value).
__device__ __forceinline__ void smem_red_add(uint32_t* p, uint32_t v) {
  asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void smem_red_or(uint32_t* p, uint32_t v) {
  asm volatile("red.shared.or.b32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void smem_red_min(uint32_t* p, uint32_t v) {
  asm volatile("red.shared.min.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void smem_red_max(uint32_t* p, uint32_t v) {
  asm volatile("red.shared.max.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// Programmatic dependent launch: pdl_launch_dependents lets the next kernel in the
// stream be scheduled early; pdl_wait blocks until the previous kernel has
// completed and its writes are visible. Both are no-ops for ordinary launches.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- device: thread-block clusters
// Distributed shared memory is only ever WRITTEN remotely in this library (stores and
// reductions pushed into a peer CTA's window before a cluster barrier both sides
// take part in), so no CTA reads memory of a CTA that may already have exited.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_num_ctas() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// Address of this CTA's shared-memory location `smem_addr` in CTA `cta` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void cluster_red_add(uint32_t cluster_addr, uint32_t v) {
  asm volatile("red.relaxed.cluster.shared::cluster.add.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_st(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_st2(uint32_t cluster_addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared::cluster.v2.u32 [%0], {%1, %2};" ::"r"(cluster_addr), "r"(a), "r"(b) : "memory");
}
// Hardware barrier over every thread of the cluster (the CTAs of a cluster are
// co-scheduled, so this is not a wait on another launch). Split in two so that work
// can sit between the arrival and the wait.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- device: flags between GPUs
// A flag in (possibly another GPU's) global memory that says "the data stored before me is
// there": written with release, read with acquire, both at system scope.
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// One fence, then any number of relaxed flag stores: together a release of everything before the
// fence to whoever acquires one of the flags (a release per flag would repeat the fence, which
// costs about two microseconds at system scope).
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ---------------------------------------------------------------- device: mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Bounded wait on a phase parity. Returns false when the limit ran out: the
// caller records a status bit and leaves its loop instead of spinning forever.
// The limit is wall time (a probe may itself suspend the thread for a while, so an
// iteration count alone would not bound it), checked every 256 probes.
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr unsigned long long kWaitLimitNs = 200ull * 1000 * 1000;
__device__ __forceinline__ unsigned long long wall_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_for(uint32_t bar, uint32_t parity, unsigned long long limit_ns);
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  return mbar_wait_for(bar, parity, kWaitLimitNs);
}
// Waits for the phase with the given parity, at most limit_ns of wall time (and kWaitLimit probes).
__device__ __forceinline__ bool mbar_wait_for(uint32_t bar, uint32_t parity, unsigned long long limit_ns) {
  unsigned long long t0 = 0;
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((i & 255u) == 255u) {
      const unsigned long long now = wall_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
  return false;
}
// After a bounded wait ran out: about two milliseconds for copies that may still be in
// flight to land before the CTA's shared memory is reused. (Kept as a rolled loop: unrolled it is
// 32 KB of machine code in the middle of a kernel.)
__device__ __forceinline__ void drain_after_timeout() {
#pragma unroll 1
  for (int i = 0; i < 2000; ++i) __nanosleep(1000);
}
// Non-blocking probe of a phase parity.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// ---------------------------------------------------------------- device: bulk copies
// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Tiled TMA loads (no cluster multicast anywhere in this library).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensor_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- device: tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_addr, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_result_addr),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// mbarrier arrive once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, 8-bit float operands, fp32 accumulate.
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// This warp's 32 lanes x 32 consecutive fp32 columns of tensor memory.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
        "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
        "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, bf16 / fp16 operands, fp32 accumulate.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Store this warp's 32 lanes x 32 consecutive fp32 columns of tensor memory.
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
        "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
        "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
        "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]),
        "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- device: 16-byte copies
// Asynchronous 16-byte copy global -> shared (L2 only), tracked per thread in groups.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t dst, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_global_nc_v4(const void* src) {
  uint4 v;
  asm volatile("ld.global.nc.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(src));
  return v;
}

// Shared-memory matrix descriptor for a K-major operand whose rows are 128 B
// wide and stored with the 128-byte swizzle (what a SWIZZLE_128B tensor-map
// load produces): 8-row groups are 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);  // start address, 16-B units
  d |= static_cast<uint64_t>(1) << 16;                  // leading byte offset (unused here)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;          // stride between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                  // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                  // SWIZZLE_128B
  return d;
}
// Instruction descriptor: e4m3 x e4m3 -> fp32, both operands K-major.
__host__ __device__ constexpr uint32_t idesc_f8_f32(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// MN-major operand (the M or N index is the contiguous one) with the 128-byte
// swizzle: atoms of [8 k-indices][64 x 16-bit elements = 128 B]; `lbo_bytes` is the
// distance between atoms along M/N, `sbo_bytes` between groups of 8 along K.
__device__ __forceinline__ uint64_t smem_desc_mn128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(sbo_bytes >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32; an operand is K-major unless its flag is set.
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (a_mn_major ? 1u << 15 : 0u) | (b_mn_major ? 1u << 16 : 0u) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------- device: numerics
// Monotone map fp32 -> u32: a > b  <=>  key(a) > key(b), and a == b <=> key(a) == key(b) for
// every pair of numbers: -0.0 is first folded onto +0.0, so ordering by key is exactly the
// ordering of floating-point comparisons (NaNs aside: a positive NaN sorts above +inf).
__device__ __forceinline__ uint32_t ordered_key(float x) {
  uint32_t u = __float_as_uint(x + 0.0f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
// The number whose key is `key` (inverse of the map above).
__device__ __forceinline__ float key_to_float(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}
#endif  // __CUDACC__

}  // namespace dsa
