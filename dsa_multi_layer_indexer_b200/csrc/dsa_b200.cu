// libdsa_b200.so: the C ABI declared in include/dsa_b200.h. One translation
// unit so the kernels share the per-device status word without relocatable
// device code. Host code here only validates arguments, encodes tensor maps
// and launches; it never allocates device memory and never synchronises,
// except dsa_check_device_status which exists to do exactly that.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "decode_prep.cuh"
#include "fused_decode.cuh"
#include "indexer_scan.cuh"
#include "peer_allreduce.cuh"
#include "sparse_mla.cuh"
#include "sparse_mla_tc.cuh"
#include "topk_select.cuh"

namespace dsa {

namespace {
thread_local char tl_error[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
  return status;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(DSA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUresult res = fn(map, dtype, rank, const_cast<void*>(base), gdim, gstr, bx, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    return fail(DSA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(res));
  return DSA_OK;
}

// Raises a kernel's dynamic shared-memory limit, once per device.
template <typename K>
static int opt_in_smem(K kernel, size_t bytes, bool (&done)[64]) {
  int dev = 0;
  DSA_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && done[dev]) return DSA_OK;
  DSA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)));
  if (dev >= 0 && dev < 64) done[dev] = true;
  return DSA_OK;
}
static bool g_opt_fused[64], g_opt_mla[64], g_opt_mla_beside[64], g_opt_mla_tc[64], g_opt_scan_f32[64], g_opt_topk[64], g_opt_gemv[4][64];

// Launch with programmatic dependent launch allowed: the kernel may be scheduled
// while its predecessor in the stream is still draining; it calls
// griddepcontrol.wait (pdl_wait) before it touches anything the predecessor
// wrote.
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace dsa

namespace dsa {
__global__ void __launch_bounds__(128)
quantize_rowwise_kernel(const float* __restrict__ x, uint8_t* __restrict__ q,
                        float* __restrict__ scale, int64_t rows, int cols, float clamp_min) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = int64_t(blockIdx.x) * 4 + warp;
  if (row >= rows) return;
  const float* xr = x + row * cols;
  float amax = 0.f;
  for (int c = lane; c < cols; c += 32) amax = fmaxf(amax, fabsf(xr[c]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = fmaxf(amax, clamp_min) / 448.0f;
  if (lane == 0) scale[row] = s;
  for (int c = lane; c < cols; c += 32) {
    float v = xr[c] / s;
    v = fminf(fmaxf(v, -448.f), 448.f);
    q[row * cols + c] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  }
}
}  // namespace dsa

using namespace dsa;

extern "C" {

int dsa_abi_version(void) { return DSA_ABI_VERSION; }

const char* dsa_last_error(void) { return tl_error; }

const char* dsa_status_string(int status) {
  switch (status) {
    case DSA_OK: return "ok";
    case DSA_ERR_INVALID_ARGUMENT: return "invalid argument";
    case DSA_ERR_UNSUPPORTED: return "unsupported geometry";
    case DSA_ERR_CUDA: return "CUDA error";
    case DSA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    default: return "unknown status";
  }
}

int dsa_check_device_status(uint32_t* detail) {
  unsigned int word = 0, zero = 0;
  DSA_CUDA(cudaDeviceSynchronize());
  DSA_CUDA(cudaMemcpyFromSymbol(&word, g_device_status, sizeof(word)));
  if (word) DSA_CUDA(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero)));
  if (detail) *detail = word;
  if (word & ~kStatusBadPage)
    return fail(DSA_ERR_DEVICE_TIMEOUT, "device status word 0x%x: a bounded device-side wait ran out", word);
  if (word)
    return fail(DSA_ERR_INVALID_ARGUMENT,
                "device status word 0x%x: a page-table entry outside [0, num_pages) was not followed", word);
  return DSA_OK;
}

// One CTA waits on a transaction barrier that nobody completes, for at most limit_ns: the wait
// runs out, the CTA agrees on that (one vote), sets the attention time-out bit and returns.
__global__ void wait_probe_kernel(unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    mbar_fence_init();
  }
  __syncthreads();
  const bool ok = mbar_wait_for(smem_u32(&bar), 0, limit_ns);
  if (__syncthreads_or(!ok) && threadIdx.x == 0) atomicOr(&g_device_status, kStatusAttnTimeout);
}

int dsa_debug_wait_timeout(uint64_t limit_ns, void* stream) {
  DSA_REQUIRE(limit_ns > 0 && limit_ns <= 10ull * 1000 * 1000, "wait probe: limit_ns=%llu outside (0, 10 ms]",
              (unsigned long long)limit_ns);
  wait_probe_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns);
  DSA_CUDA(cudaGetLastError());
  return DSA_OK;
}

int dsa_debug_read_stamps(uint64_t* host_out, int max_words) {
#ifdef DSA_STAMPS
  const int n = max_words < kStampCtas * kStampSlots ? max_words : kStampCtas * kStampSlots;
  DSA_CUDA(cudaDeviceSynchronize());
  DSA_CUDA(cudaMemcpyFromSymbol(host_out, g_stamps, size_t(n) * sizeof(uint64_t)));
  static unsigned long long zeros[kStampCtas * kStampSlots];
  DSA_CUDA(cudaMemcpyToSymbol(g_stamps, zeros, sizeof(zeros)));
  if (max_words >= kStampCtas * kStampSlots + 32) {
    DSA_CUDA(cudaMemcpyFromSymbol(host_out + kStampCtas * kStampSlots, g_ktime, sizeof(g_ktime)));
    unsigned long long init[32];
    for (int i = 0; i < 32; ++i) init[i] = (i & 1) ? 0ull : ~0ull;
    DSA_CUDA(cudaMemcpyToSymbol(g_ktime, init, sizeof(init)));
    return kStampCtas * kStampSlots + 32;
  }
  return n;
#else
  (void)host_out;
  (void)max_words;
  return fail(DSA_ERR_UNSUPPORTED, "this build has no phase stamps (compile with -DDSA_STAMPS)");
#endif
}

// ------------------------------------------------------------------ indexer scan
static int scan_common_checks(const uint8_t* index_q, const float* index_w, const float* logits,
                              int R, int n_heads, int64_t ctx, int64_t slab_stride) {
  DSA_REQUIRE(index_q && index_w && logits, "indexer scan: null pointer");
  DSA_REQUIRE(aligned16(index_q) && aligned16(logits), "indexer scan: pointers must be 16-byte aligned");
  DSA_REQUIRE(R > 0 && R <= 65535, "indexer scan: R=%d out of range [1, 65535]", R);
  DSA_REQUIRE(n_heads > 0 && n_heads <= DSA_INDEX_MAX_HEADS && n_heads % 16 == 0,
              "indexer scan: n_heads=%d must be a multiple of 16 and <= %d", n_heads,
              DSA_INDEX_MAX_HEADS);
  DSA_REQUIRE(ctx > 0 && ctx < (int64_t(1) << 31), "indexer scan: ctx=%lld out of range",
              (long long)ctx);
  DSA_REQUIRE(slab_stride >= ctx, "indexer scan: slab_stride=%lld < ctx=%lld",
              (long long)slab_stride, (long long)ctx);
  return DSA_OK;
}

static int scan_grid_x(int R, int tiles_per_row, int ctas_per_sm) {
  // One resident wave for a single row. A batch gets about 1.75 waves: its rows
  // differ in length, the grid is sized on the host without reading the lengths,
  // and the later CTAs fill the SMs that the short rows' CTAs leave early.
  int per_row = ((R > 1 ? 7 : 4) * ctas_per_sm * sm_count() / 4 + R - 1) / R;
  if (per_row > tiles_per_row) per_row = tiles_per_row;
  if (per_row < 1) per_row = 1;
  return per_row;
}

// Two CTAs per SM with a 4-slot ring. Tiles in their epilogue at once per CTA: three for a
// batch (measured 1.5-2 % faster than two on 32 rows), two for one row (three is 0.15 us
// slower there). A ragged batch is spread so that every CTA gets about the same number of tiles.
extern "C++" {
template <int kEpiGroups, bool kPaged>
static int launch_scan_tc_as(const CUtensorMap& tmap, const scan::Params& p, dim3 grid, cudaStream_t st) {
  static bool done[64];
  constexpr size_t smem = scan::smem_bytes<scan::kStagesTwoPerSm>();
  auto kernel = scan::indexer_scan_tc_kernel<scan::kStagesTwoPerSm, kEpiGroups, kPaged>;
  int rc = opt_in_smem(kernel, smem, done);
  if (rc) return rc;
  DSA_CUDA(launch_pdl(kernel, grid, dim3(64 + 128 * kEpiGroups), smem, st, tmap, p));
  return DSA_OK;
}
}  // extern "C++"

static int launch_scan_tc(const CUtensorMap& tmap, const scan::Params& p_in, int R, cudaStream_t st) {
  scan::Params p = p_in;
  p.balance_rows = (R > 1 && R <= 32 && p.seq_lens) ? R : 0;
  if (R > 1) {
    // a ragged batch of up to 32 rows: one resident wave on a 1-D grid, the rows' CTA counts settled on the device
    const dim3 grid = p.balance_rows ? dim3(std::max(R, 2 * sm_count()), 1) : dim3(scan_grid_x(R, p.tiles_per_row, 2), R);
    return p.paged ? launch_scan_tc_as<3, true>(tmap, p, grid, st) : launch_scan_tc_as<3, false>(tmap, p, grid, st);
  }
  const dim3 grid(scan_grid_x(R, p.tiles_per_row, 2), R);
  return p.paged ? launch_scan_tc_as<2, true>(tmap, p, grid, st) : launch_scan_tc_as<2, false>(tmap, p, grid, st);
}

int dsa_indexer_scan_fp8(const uint8_t* index_q, const float* index_w, const uint8_t* index_k,
                         const float* k_scale, const int32_t* seq_lens, float* logits,
                         uint32_t* hist, int R, int rows_per_seq, int n_heads, int64_t ctx,
                         int64_t n_seq, int64_t k_seq_stride, int64_t scale_seq_stride,
                         int64_t slab_stride, int impl, void* stream) {
  int rc = scan_common_checks(index_q, index_w, logits, R, n_heads, ctx, slab_stride);
  if (rc) return rc;
  DSA_REQUIRE(index_k && k_scale, "indexer scan: null key cache");
  DSA_REQUIRE(aligned16(index_k), "indexer scan: index_k must be 16-byte aligned");
  DSA_REQUIRE(rows_per_seq > 0 && R % rows_per_seq == 0,
              "indexer scan: R=%d is not a multiple of rows_per_seq=%d", R, rows_per_seq);
  DSA_REQUIRE(n_seq == R / rows_per_seq, "indexer scan: n_seq=%lld but R / rows_per_seq = %d",
              (long long)n_seq, R / rows_per_seq);
  DSA_REQUIRE(k_seq_stride >= ctx && scale_seq_stride >= ctx,
              "indexer scan: sequence strides must be >= ctx");
  DSA_REQUIRE(n_seq * k_seq_stride < (int64_t(1) << 31), "indexer scan: key cache too large");
  DSA_REQUIRE(impl == 0 || impl == 1, "indexer scan: impl must be 0 (tcgen05) or 1 (legacy)");

  scan::Params p{};
  p.q = index_q;
  p.w = index_w;
  p.keys = index_k;
  p.k_scale = k_scale;
  p.seq_lens = seq_lens;
  p.logits = logits;
  p.hist = hist;
  p.ctx = ctx;
  p.k_seq_stride = k_seq_stride;
  p.scale_seq_stride = scale_seq_stride;
  p.slab_stride = slab_stride;
  p.rows_per_seq = rows_per_seq;
  p.n_heads = n_heads;
  p.tiles_per_row = int((ctx + scan::kTileKeys - 1) / scan::kTileKeys);
  p.paged = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  if (impl == 1) {
    int gx = int((ctx + 63) / 64);
    int cap = (8 * sm_count() + R - 1) / R;
    if (gx > cap) gx = cap < 1 ? 1 : cap;
    scan::indexer_scan_legacy_kernel<<<dim3(gx, R), scan::kLegacyThreads, 0, st>>>(p);
    DSA_CUDA(cudaGetLastError());
    return DSA_OK;
  }

  CUtensorMap tmap;
  // the map covers exactly the rows the scan may touch, so nothing past them is read
  const uint64_t rows = uint64_t(n_seq - 1) * uint64_t(k_seq_stride) + uint64_t(ctx);
  const uint64_t dims[2] = {uint64_t(scan::kKeyBytes), rows};
  const uint64_t strides[1] = {uint64_t(scan::kKeyBytes)};
  const uint32_t box[2] = {uint32_t(scan::kKeyBytes), uint32_t(scan::kTileKeys)};
  rc = encode_tensor_map(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, index_k, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = launch_scan_tc(tmap, p, R, st);
  if (rc) return rc;
  return DSA_OK;
}

int dsa_indexer_scan_fp8_paged(const uint8_t* index_q, const float* index_w,
                               const uint8_t* index_k_pages, int64_t num_pages,
                               const int32_t* page_table, int64_t pt_stride,
                               const int32_t* seq_lens, float* logits, uint32_t* hist, int R,
                               int n_heads, int64_t ctx, int64_t slab_stride, void* stream) {
  int rc = scan_common_checks(index_q, index_w, logits, R, n_heads, ctx, slab_stride);
  if (rc) return rc;
  DSA_REQUIRE(index_k_pages && page_table && seq_lens, "paged indexer scan: null pointer");
  DSA_REQUIRE(aligned16(index_k_pages), "paged indexer scan: page pool must be 16-byte aligned");
  DSA_REQUIRE(num_pages > 0 && num_pages < (int64_t(1) << 31), "paged indexer scan: bad num_pages");
  DSA_REQUIRE(pt_stride * DSA_PAGE_TOKENS >= ctx,
              "paged indexer scan: pt_stride=%lld pages cannot cover ctx=%lld", (long long)pt_stride,
              (long long)ctx);

  scan::Params p{};
  p.q = index_q;
  p.w = index_w;
  p.seq_lens = seq_lens;
  p.logits = logits;
  p.hist = hist;
  p.pages = index_k_pages;
  p.page_table = page_table;
  p.pt_stride = pt_stride;
  p.num_pages = num_pages;
  p.ctx = ctx;
  p.slab_stride = slab_stride;
  p.rows_per_seq = 1;
  p.n_heads = n_heads;
  p.tiles_per_row = int((ctx + scan::kTileKeys - 1) / scan::kTileKeys);
  p.paged = 1;

  CUtensorMap tmap;
  // a page is 66 rows of 128 B: 64 key rows, then 2 rows holding the 64 fp32 scales
  const uint64_t dims[3] = {uint64_t(scan::kKeyBytes), uint64_t(DSA_INDEX_PAGE_BYTES / scan::kKeyBytes),
                            uint64_t(num_pages)};
  const uint64_t strides[2] = {uint64_t(scan::kKeyBytes), uint64_t(DSA_INDEX_PAGE_BYTES)};
  const uint32_t box[3] = {uint32_t(scan::kKeyBytes), uint32_t(DSA_PAGE_TOKENS), 1u};
  rc = encode_tensor_map(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, index_k_pages, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = launch_scan_tc(tmap, p, R, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return DSA_OK;
}

int dsa_indexer_scan_f32(const float* index_q, const float* index_w, const float* index_k,
                         const int32_t* seq_lens, float* logits, int R, int rows_per_seq,
                         int n_heads, int head_dim, int64_t ctx, int64_t k_seq_stride,
                         int64_t slab_stride, void* stream) {
  DSA_REQUIRE(index_q && index_w && index_k && logits, "f32 indexer scan: null pointer");
  DSA_REQUIRE(R > 0 && R <= 65535 && rows_per_seq > 0 && R % rows_per_seq == 0,
              "f32 indexer scan: bad R=%d / rows_per_seq=%d", R, rows_per_seq);
  DSA_REQUIRE(n_heads > 0 && head_dim > 0 && ctx > 0, "f32 indexer scan: bad geometry");
  DSA_REQUIRE(k_seq_stride >= ctx && slab_stride >= ctx, "f32 indexer scan: strides must be >= ctx");
  const size_t smem = (size_t(n_heads) * head_dim + n_heads) * sizeof(float);
  DSA_REQUIRE(smem <= 200 * 1024, "f32 indexer scan: n_heads * head_dim too large for shared memory");
  if (smem > 48 * 1024) {
    int rc = opt_in_smem(scan::indexer_scan_f32_kernel, 200 * 1024, g_opt_scan_f32);
    if (rc) return rc;
  }
  int gx = int((ctx + 7) / 8);
  int cap = (16 * sm_count() + R - 1) / R;
  if (gx > cap) gx = cap < 1 ? 1 : cap;
  scan::indexer_scan_f32_kernel<<<dim3(gx, R), 256, smem, static_cast<cudaStream_t>(stream)>>>(
      index_q, index_w, index_k, seq_lens, logits, rows_per_seq, n_heads, head_dim, ctx,
      k_seq_stride, slab_stride);
  DSA_CUDA(cudaGetLastError());
  return DSA_OK;
}

// ------------------------------------------------------------------ top-k
// Longest row the one-launch cluster kernel takes on the current device: 262144 logits where a
// cluster of 16 CTAs with its shared memory can be scheduled (asked of the runtime once per
// device), else the portable 8-CTA limit of 131072. Without a device: the portable limit.
static int64_t topk_cluster_max_n() {
  static int state[64];  // 0 unknown, 1 portable only, 2 sixteen CTAs
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return topk::kClPortableN;
  }
  if (state[dev] == 0) {
    auto kernel = topk::topk_cluster_kernel<false, topk::kClMaxCtasBig>;
    constexpr size_t smem = sizeof(topk::ClSharedBig);
    int clusters = 0;
    bool ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) == cudaSuccess &&
              cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
    if (ok) {
      cudaLaunchConfig_t cfg{};
      cudaLaunchAttribute attr[1];
      cfg.gridDim = dim3(topk::kClMaxCtasBig, 1);
      cfg.blockDim = dim3(topk::kClThreads);
      cfg.dynamicSmemBytes = smem;
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = topk::kClMaxCtasBig;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      ok = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters >= 1;
    }
    cudaGetLastError();  // (a refusal is an answer, not an error of the caller)
    state[dev] = ok ? 2 : 1;
  }
  return state[dev] == 2 ? topk::kClMaxN : topk::kClPortableN;
}

int64_t dsa_topk_workspace_bytes(int R, int64_t n) {
  if (R <= 0 || n <= 0) return 0;
  if (n <= topk_cluster_max_n()) return 16;  // the cluster kernel keeps everything in shared memory
  return topk::workspace_words(R, n) * 4;
}

// Rows of up to topk_cluster_max_n() logits: one cluster of 1..8 (or 16) CTAs per row, no scratch.
extern "C++" {
template <bool kPlain, int kMaxC>
static int launch_topk_cluster_as(const topk::Params& p, int R, int ctas, int nk, cudaStream_t st) {
  static bool done[64];
  auto kernel = topk::topk_cluster_kernel<kPlain, kMaxC>;
  constexpr size_t smem = sizeof(topk::ClSharedT<kMaxC>);
  int dev = 0;
  DSA_CUDA(cudaGetDevice(&dev));
  const bool first = !(dev >= 0 && dev < 64 && done[dev]);
  int rc = opt_in_smem(kernel, smem, done);
  if (rc) return rc;
  if (first && kMaxC > 8)  // sixteen CTAs per cluster is not a portable size: the kernel opts in
    DSA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[2];
  cfg.gridDim = dim3(ctas, R);
  cfg.blockDim = dim3(topk::kClThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ctas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  DSA_CUDA(cudaLaunchKernelEx(&cfg, kernel, p, nk));
  return DSA_OK;
}
}  // extern "C++"

static int launch_topk_cluster(const topk::Params& p, int R, int64_t n, cudaStream_t st) {
  const bool plain = p.hist && !p.n_src && !p.n_dest && !p.index_map && !p.out_val;
  // As few CTAs as hold the row at 32 logits per thread: every CTA added costs cluster barriers and
  // remote stores, and a row of up to 16384 logits needs none of either.
  // A row that comes without the scan's histogram counts its own first level with shared-memory
  // atomics, about one per cycle per SM: it is spread over as many SMs as the cluster has (2048 logits
  // per CTA or more).
  int ctas = 1;
  while (ctas < topk::kClMaxCtasBig && int64_t(ctas) * topk::kClThreads * topk::kClMaxKeys < n) ctas *= 2;
  if (!p.hist)  // (as long as the launch still fits the device in one wave)
    while (ctas < topk::kClMaxCtas && int64_t(ctas) * 2048 < n && 2 * ctas * R <= sm_count()) ctas *= 2;
  const int64_t per_key = int64_t(ctas) * topk::kClThreads;
  const int nk = int((n + per_key - 1) / per_key);
  if (ctas > topk::kClMaxCtas)
    return plain ? launch_topk_cluster_as<true, topk::kClMaxCtasBig>(p, R, ctas, nk, st)
                 : launch_topk_cluster_as<false, topk::kClMaxCtasBig>(p, R, ctas, nk, st);
  return plain ? launch_topk_cluster_as<true, topk::kClMaxCtas>(p, R, ctas, nk, st)
               : launch_topk_cluster_as<false, topk::kClMaxCtas>(p, R, ctas, nk, st);
}

int dsa_topk_select(const float* logits, const int32_t* seq_lens, uint32_t* hist,
                    const int32_t* index_map, int32_t* out_idx, float* out_val, void* workspace,
                    int64_t workspace_bytes, int R, int64_t n, int64_t slab_stride, int topk_k,
                    int32_t pad_value, int32_t index_offset, void* stream) {
  DSA_REQUIRE(logits && out_idx && workspace, "topk: null pointer");
  DSA_REQUIRE(aligned16(logits) && aligned16(workspace), "topk: logits / workspace must be 16-byte aligned");
  DSA_REQUIRE(R > 0 && R <= 65535, "topk: R=%d out of range", R);
  DSA_REQUIRE(n > 0 && slab_stride >= n, "topk: need 0 < n <= slab_stride");
  DSA_REQUIRE(topk_k > 0 && topk_k <= 65536, "topk: k=%d out of range [1, 65536]", topk_k);
  if (n > topk::kMaxN)
    return fail(DSA_ERR_UNSUPPORTED, "topk: n=%lld exceeds the %lld-per-row limit", (long long)n,
                (long long)topk::kMaxN);
  DSA_REQUIRE(workspace_bytes >= dsa_topk_workspace_bytes(R, n),
              "topk: workspace of %lld bytes is smaller than dsa_topk_workspace_bytes = %lld",
              (long long)workspace_bytes, (long long)dsa_topk_workspace_bytes(R, n));
  if (n <= topk_cluster_max_n()) {
    topk::Params p{};
    p.logits = logits;
    p.seq_lens = seq_lens;
    p.hist = hist;
    p.index_map = index_map;
    p.out_idx = out_idx;
    p.out_val = out_val;
    p.n = n;
    p.slab_stride = slab_stride;
    p.topk = topk_k;
    p.pad = pad_value;
    p.index_offset = index_offset;
    return launch_topk_cluster(p, R, n, static_cast<cudaStream_t>(stream));
  }
  const int64_t words = topk::mask_words(n), slots = words / 4;
  uint32_t* ws = static_cast<uint32_t*>(workspace);
  topk::Params p{};
  p.logits = logits;
  p.seq_lens = seq_lens;
  p.above_mask = ws;
  p.slot_cnt = p.above_mask + int64_t(R) * words;
  p.header = p.slot_cnt + int64_t(R) * slots;
  uint32_t* ws_hist = p.header + int64_t(R) * 4;
  p.hist2 = ws_hist + int64_t(R) * topk::kBins;
  p.slot_cand = reinterpret_cast<uint2*>(p.hist2 + int64_t(R) * topk::kRoundBins);
  p.hist = hist ? hist : ws_hist;
  p.index_map = index_map;
  p.out_idx = out_idx;
  p.out_val = out_val;
  p.n = n;
  p.slab_stride = slab_stride;
  p.words = int(words);
  p.slots = int(slots);
  p.topk = topk_k;
  p.pad = pad_value;
  p.index_offset = index_offset;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(unsigned(words / (topk::kChunk / 32)), R);
  if (!hist) {
    DSA_CUDA(launch_pdl(topk::topk_hist_kernel, grid, dim3(topk::kThreads), 0, st, p));
  }
  DSA_CUDA(launch_pdl(topk::topk_classify_kernel, grid, dim3(topk::kThreads), 0, st, p));
  int rc = opt_in_smem(topk::topk_finish_kernel,
                       topk::fin_smem_bytes(int(topk::mask_words(topk::kMaxN))), g_opt_topk);
  if (rc) return rc;
  DSA_CUDA(launch_pdl(topk::topk_finish_kernel, dim3(R), dim3(topk::kFinThreads),
                      topk::fin_smem_bytes(p.words), st, p));
  return DSA_OK;
}

// ------------------------------------------------------------------ candidate exchange between GPUs
static int exchange_common(int R, int64_t n, int topk_k, int world) {
  DSA_REQUIRE(R > 0 && R <= 65535, "candidate exchange: R=%d out of range", R);
  DSA_REQUIRE(world >= 1 && world <= topk::kMaxRanks, "candidate exchange: world=%d out of range [1, %d]", world,
              topk::kMaxRanks);
  DSA_REQUIRE(topk_k > 0 && topk_k <= 65536, "candidate exchange: k=%d out of range [1, 65536]", topk_k);
  if (n <= 0 || n > topk_cluster_max_n())
    return fail(DSA_ERR_UNSUPPORTED, "candidate exchange: rows of %lld logits (the limit is %lld)", (long long)n,
                (long long)topk_cluster_max_n());
  return DSA_OK;
}

int dsa_topk_select_push(const float* logits, const int32_t* seq_lens, uint32_t* hist, int R, int64_t n,
                         int64_t slab_stride, int topk_k, int32_t pad_value, int32_t index_offset, int world,
                         int rank, void* const* gather_idx, void* const* gather_val, void* const* flags,
                         uint32_t* sent, void* stream) {
  int rc = exchange_common(R, n, topk_k, world);
  if (rc) return rc;
  DSA_REQUIRE(logits && gather_idx && gather_val && flags && sent, "topk push: null pointer");
  DSA_REQUIRE(aligned16(logits) && slab_stride >= n, "topk push: logits must be 16-byte aligned, slab_stride >= n");
  DSA_REQUIRE(rank >= 0 && rank < world, "topk push: rank=%d outside [0, %d)", rank, world);
  topk::Params p{};
  p.logits = logits;
  p.seq_lens = seq_lens;
  p.hist = hist;
  p.n = n;
  p.slab_stride = slab_stride;
  p.topk = topk_k;
  p.pad = pad_value;
  p.index_offset = index_offset;
  p.n_dest = world;
  p.src_rank = rank;
  for (int d = 0; d < world; ++d) {
    DSA_REQUIRE(gather_idx[d] && gather_val[d] && flags[d], "topk push: null pointer for rank %d", d);
    p.dest_idx[d] = static_cast<int32_t*>(gather_idx[d]);
    p.dest_val[d] = static_cast<float*>(gather_val[d]);
    p.dest_flag[d] = static_cast<uint32_t*>(flags[d]) + size_t(rank) * R;
  }
  p.sent = sent;
  return launch_topk_cluster(p, R, n, static_cast<cudaStream_t>(stream));
}

int dsa_topk_merge_wait(const int32_t* gather_idx, const float* gather_val, const uint32_t* flags, uint32_t* seen,
                        int32_t* out_idx, int R, int world, int topk_k, int32_t pad_value, int64_t wait_limit_ns,
                        void* stream) {
  const int64_t n = int64_t(world) * topk_k;
  int rc = exchange_common(R, n, topk_k, world);
  if (rc) return rc;
  DSA_REQUIRE(gather_idx && gather_val && flags && seen && out_idx, "topk merge: null pointer");
  DSA_REQUIRE(wait_limit_ns > 0, "topk merge: the wait needs a limit");
  topk::Params p{};
  p.logits = gather_val;  // [2][R][world][topk]: the kernel picks the parity of each row's step
  p.index_map = gather_idx;
  p.out_idx = out_idx;
  p.n = n;
  p.slab_stride = n;
  p.topk = topk_k;
  p.pad = pad_value;
  p.n_src = world;
  p.wait_flags = flags;
  p.seen = seen;
  p.wait_limit_ns = static_cast<unsigned long long>(wait_limit_ns);
  return launch_topk_cluster(p, R, n, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------ all-reduce of a decode activation
int dsa_allreduce_push(const void* src, int src_bf16, int64_t n, int world, int rank, void* const* slots,
                       void* const* flags, uint32_t* sent, void* stream) {
  DSA_REQUIRE(src && slots && flags && sent, "all-reduce push: null pointer");
  DSA_REQUIRE(world >= 1 && world <= ar::kMaxRanks && rank >= 0 && rank < world,
              "all-reduce push: world=%d / rank=%d out of range", world, rank);
  DSA_REQUIRE(n > 0 && n % 4 == 0 && n <= (int64_t(1) << 20), "all-reduce push: n=%lld must be a multiple of 4, at most 2^20",
              (long long)n);
  DSA_REQUIRE(aligned16(src), "all-reduce push: src must be 16-byte aligned");
  ar::PushParams p{};
  p.src = src;
  p.src_bf16 = src_bf16 ? 1 : 0;
  p.n = n;
  p.n_dest = world;
  p.src_rank = rank;
  for (int d = 0; d < world; ++d) {
    DSA_REQUIRE(slots[d] && flags[d] && aligned16(slots[d]), "all-reduce push: bad buffer of rank %d", d);
    p.dest[d] = static_cast<float*>(slots[d]);
    p.dest_flag[d] = static_cast<uint32_t*>(flags[d]) + rank;
  }
  p.sent = sent;
  DSA_CUDA(launch_pdl(ar::allreduce_push_kernel, dim3(1), dim3(ar::kThreads), 0, static_cast<cudaStream_t>(stream), p));
  return DSA_OK;
}

int dsa_allreduce_wait_sum(const float* slots, const uint32_t* flags, uint32_t* seen, const void* residual, void* out,
                           int out_bf16, int64_t n, int world, int64_t wait_limit_ns, void* stream) {
  DSA_REQUIRE(slots && flags && seen && out, "all-reduce sum: null pointer");
  DSA_REQUIRE(world >= 1 && world <= ar::kMaxRanks, "all-reduce sum: world=%d out of range", world);
  DSA_REQUIRE(n > 0 && n % 4 == 0 && n <= (int64_t(1) << 20), "all-reduce sum: n=%lld must be a multiple of 4, at most 2^20",
              (long long)n);
  DSA_REQUIRE(aligned16(slots) && aligned16(out) && (!residual || aligned16(residual)),
              "all-reduce sum: pointers must be 16-byte aligned");
  DSA_REQUIRE(wait_limit_ns > 0, "all-reduce sum: the wait needs a limit");
  ar::SumParams p{};
  p.slots = slots;
  p.flags = flags;
  p.seen = seen;
  p.residual = residual;
  p.out = out;
  p.out_bf16 = out_bf16 ? 1 : 0;
  p.n = n;
  p.n_src = world;
  p.wait_limit_ns = static_cast<unsigned long long>(wait_limit_ns);
  DSA_CUDA(launch_pdl(ar::allreduce_wait_sum_kernel, dim3(1), dim3(ar::kThreads), 0, static_cast<cudaStream_t>(stream), p));
  return DSA_OK;
}

// Peer mapping of an exchange buffer (one process per GPU): the owner exports the CUDA IPC handle
// of the allocation that contains `ptr`, every other process opens it and gets an address it can
// store through. Set-up calls, not on any step's path.
typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

int dsa_ipc_export(const void* ptr, void* handle_out, int64_t* offset_out) {
  DSA_REQUIRE(ptr && handle_out && offset_out, "ipc export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == DSA_IPC_HANDLE_BYTES, "handle size");
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  DSA_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &qres));
  if (!sym || qres != cudaDriverEntryPointSuccess) return fail(DSA_ERR_CUDA, "ipc export: cuMemGetAddressRange unavailable");
  CUdeviceptr base = 0;
  size_t size = 0;
  CUresult res = reinterpret_cast<GetAddressRangeFn>(sym)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  if (res != CUDA_SUCCESS) return fail(DSA_ERR_CUDA, "ipc export: cuMemGetAddressRange failed with CUresult %d", int(res));
  cudaIpcMemHandle_t h;
  DSA_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(handle_out, &h, sizeof(h));
  *offset_out = int64_t(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return DSA_OK;
}

int dsa_ipc_open(const void* handle, int64_t offset, void** ptr_out) {
  DSA_REQUIRE(handle && ptr_out && offset >= 0, "ipc open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* base = nullptr;
  DSA_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr_out = static_cast<char*>(base) + offset;
  return DSA_OK;
}

int dsa_ipc_close(void* ptr, int64_t offset) {
  DSA_REQUIRE(ptr && offset >= 0, "ipc close: bad argument");
  DSA_CUDA(cudaIpcCloseMemHandle(static_cast<char*>(ptr) - offset));
  return DSA_OK;
}

// ------------------------------------------------------------------ top-k without caller scratch
}  // extern "C"

// Scratch of dsa_topk_select_static: one fixed array inside the library's device
// image. Every GPU that loads the library carries these 4 MiB until the process
// exits. Host code must not hand this symbol to a kernel: on the host the name is
// only a stand-in, so the device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_topk_static_scratch[DSA_TOPK_STATIC_SCRATCH_BYTES];

// Device address of the array on the current device (looked up on first use;
// host threads making that first call together are serialised by a mutex).
static int topk_static_scratch(void** out) {
  static void* ptr[64];
  static std::mutex mu;
  int dev = 0;
  DSA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(DSA_ERR_UNSUPPORTED, "topk (static scratch): device ordinal %d", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (ptr[dev] == nullptr) {
    void* p = nullptr;
    DSA_CUDA(cudaGetSymbolAddress(&p, g_topk_static_scratch));
    ptr[dev] = p;
  }
  *out = ptr[dev];
  return DSA_OK;
}

extern "C" {

int dsa_topk_select_static(const float* logits, const int32_t* seq_lens, int32_t* out_idx,
                           float* out_val, int R, int64_t n, int64_t slab_stride, int topk_k,
                           int32_t pad_value, int32_t index_offset, void* stream) {
  // every argument is checked before anything is enqueued: a rejected call puts nothing on the stream
  DSA_REQUIRE(logits && out_idx, "topk (static scratch): null pointer");
  DSA_REQUIRE(aligned16(logits), "topk (static scratch): logits must be 16-byte aligned");
  DSA_REQUIRE(R > 0 && R <= 65535, "topk (static scratch): R=%d out of range", R);
  DSA_REQUIRE(n > 0 && slab_stride >= n, "topk (static scratch): need 0 < n <= slab_stride");
  DSA_REQUIRE(topk_k > 0 && topk_k <= 65536, "topk (static scratch): k=%d out of range [1, 65536]", topk_k);
  const int64_t need = dsa_topk_workspace_bytes(R, n);
  if (n > topk::kMaxN || need > int64_t(DSA_TOPK_STATIC_SCRATCH_BYTES))
    return fail(DSA_ERR_UNSUPPORTED,
                "topk (static scratch): R=%d rows of n=%lld logits need %lld bytes of scratch, the built-in "
                "array holds %lld; use dsa_topk_select with caller-owned scratch",
                R, (long long)n, (long long)need, (long long)DSA_TOPK_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  int rc = topk_static_scratch(&scratch);
  if (rc) return rc;
  if (n > topk_cluster_max_n()) {
    // The array still holds whatever the previous call left, possibly laid out for
    // another (R, n): the histograms of this call's layout have to start at zero.
    const int64_t words = topk::mask_words(n), slots = words / 4;
    uint32_t* hist = static_cast<uint32_t*>(scratch) + int64_t(R) * (words + slots + 4);
    DSA_CUDA(cudaMemsetAsync(hist, 0, size_t(R) * (topk::kBins + topk::kRoundBins) * sizeof(uint32_t),
                             static_cast<cudaStream_t>(stream)));  // both histograms, adjacent in the layout
  }
  return dsa_topk_select(logits, seq_lens, nullptr, nullptr, out_idx, out_val, scratch,
                         DSA_TOPK_STATIC_SCRATCH_BYTES, R, n, slab_stride, topk_k, pad_value,
                         index_offset, stream);
}

// ------------------------------------------------------------------ sparse MLA
// Argument checks and parameter block shared by the split and the fused launch.
static int mla_prepare(const void* q, const void* kv, const int32_t* indices, const int32_t* seq_lens,
                       float* part_acc, float* part_m, float* part_l, int R, int rows_per_seq, int H,
                       int topk_k, int nsplit, float sm_scale, int64_t kv_seq_stride, int kv_fp8,
                       bool need_partials, mla::Params* out_p) {
  DSA_REQUIRE(q && kv, "sparse MLA: null pointer");
  DSA_REQUIRE(!need_partials || (part_acc && part_m && part_l), "sparse MLA: null split-K scratch");
  DSA_REQUIRE(aligned16(q) && aligned16(kv) && aligned16(part_acc),
              "sparse MLA: pointers must be 16-byte aligned");
  DSA_REQUIRE(R > 0 && R <= 65535 && rows_per_seq > 0 && R % rows_per_seq == 0,
              "sparse MLA: bad R=%d / rows_per_seq=%d", R, rows_per_seq);
  DSA_REQUIRE(H > 0 && H % DSA_HEAD_BLOCK == 0, "sparse MLA: H=%d must be a multiple of %d", H,
              DSA_HEAD_BLOCK);
  DSA_REQUIRE(topk_k > 0, "sparse MLA: topk must be positive");
  DSA_REQUIRE(nsplit > 0 && nsplit <= 65535, "sparse MLA: nsplit=%d out of range", nsplit);
  DSA_REQUIRE(kv_seq_stride > 0, "sparse MLA: kv_seq_stride must be positive");
  DSA_REQUIRE(kv_fp8 == 0 || kv_fp8 == 1, "sparse MLA: kv_fp8 must be 0 or 1");
  mla::Params& p = *out_p;
  p = mla::Params{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.kv = static_cast<const uint8_t*>(kv);
  p.indices = indices;
  p.seq_lens = seq_lens;
  p.part_acc = part_acc;
  p.part_m = part_m;
  p.part_l = part_l;
  p.kv_seq_stride = kv_seq_stride;
  p.ctx = kv_seq_stride;
  p.rows_per_seq = rows_per_seq;
  p.H = H;
  p.topk = topk_k;
  p.nsplit = nsplit;
  int kps = (topk_k + nsplit - 1) / nsplit;
  kps = (kps + 15) / 16 * 16;
  p.keys_per_split = kps;
  p.kv_fp8 = kv_fp8;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  return DSA_OK;
}

static int mla_partials_launch(const void* q, const void* kv, const int32_t* indices,
                               const int32_t* seq_lens, float* part_acc, float* part_m, float* part_l,
                               int R, int rows_per_seq, int H, int topk_k, int nsplit, float sm_scale,
                               int64_t kv_seq_stride, int kv_fp8, bool beside, void* stream) {
  mla::Params p;
  int rc0 = mla_prepare(q, kv, indices, seq_lens, part_acc, part_m, part_l, R, rows_per_seq, H, topk_k,
                        nsplit, sm_scale, kv_seq_stride, kv_fp8, true, &p);
  if (rc0) return rc0;
  // Head counts that fill 64-row blocks go to the tcgen05 kernel once there are enough
  // 64-head x 64-key tiles to give every SM more than one (a single row of 2048 keys
  // is faster on the mma.sync kernel's 16-head CTAs); its splits are whole 64-key tiles.
  const int64_t tc_tiles = int64_t(R) * (H / mla_tc::kHG) * ((topk_k + mla_tc::kBN - 1) / mla_tc::kBN);
  if (H % mla_tc::kHG == 0 && sm_scale > 0.f && tc_tiles >= mla_tc::kMinTiles) {
    int kps = (topk_k + nsplit - 1) / nsplit;
    p.keys_per_split = (kps + mla_tc::kBN - 1) / mla_tc::kBN * mla_tc::kBN;
    int rc = opt_in_smem(mla_tc::sparse_mla_tc_kernel, mla_tc::Smem::bytes, g_opt_mla_tc);
    if (rc) return rc;
    DSA_CUDA(launch_pdl(mla_tc::sparse_mla_tc_kernel, dim3(nsplit, H / mla_tc::kHG, R), dim3(mla_tc::kThreads),
                        mla_tc::Smem::bytes, static_cast<cudaStream_t>(stream), p));
    return DSA_OK;
  }
  const size_t smem = kv_fp8 ? mla::SmemLayout::bytes_fp8 : mla::SmemLayout::bytes_bf16;
  if (beside) {
    int rc = opt_in_smem(mla::sparse_mla_partials_beside_kernel, mla::SmemLayout::bytes_fp8, g_opt_mla_beside);
    if (rc) return rc;
    DSA_CUDA(launch_pdl(mla::sparse_mla_partials_beside_kernel, dim3(nsplit, H / DSA_HEAD_BLOCK, R),
                        dim3(mla::kThreads), smem, static_cast<cudaStream_t>(stream), p));
    return DSA_OK;
  }
  {
    int rc = opt_in_smem(mla::sparse_mla_partials_kernel, mla::SmemLayout::bytes_fp8, g_opt_mla);
    if (rc) return rc;
  }
  DSA_CUDA(launch_pdl(mla::sparse_mla_partials_kernel, dim3(nsplit, H / DSA_HEAD_BLOCK, R),
                      dim3(mla::kThreads), smem, static_cast<cudaStream_t>(stream), p));
  return DSA_OK;
}

int dsa_sparse_mla_partials(const void* q, const void* kv, const int32_t* indices,
                            const int32_t* seq_lens, float* part_acc, float* part_m, float* part_l,
                            int R, int rows_per_seq, int H, int topk_k, int nsplit, float sm_scale,
                            int64_t kv_seq_stride, int kv_fp8, void* stream) {
  return mla_partials_launch(q, kv, indices, seq_lens, part_acc, part_m, part_l, R, rows_per_seq, H, topk_k,
                             nsplit, sm_scale, kv_seq_stride, kv_fp8, false, stream);
}

int dsa_sparse_mla_combine(const float* part_acc, const float* part_m, const float* part_l,
                           void* out, int R, int H, int nsplit, void* stream) {
  DSA_REQUIRE(part_acc && part_m && part_l && out, "sparse MLA combine: null pointer");
  DSA_REQUIRE(aligned16(part_acc) && aligned16(out), "sparse MLA combine: misaligned pointer");
  DSA_REQUIRE(R > 0 && R <= 65535 && H > 0 && nsplit > 0, "sparse MLA combine: bad geometry");
  if (nsplit <= mla::kFlatMaxSplit && int64_t(R) * H >= 512) {
    // many (row, head) pairs, few splits: one thread per four output columns
    const int64_t n_pairs = int64_t(R) * H;
    DSA_CUDA(launch_pdl(mla::sparse_mla_combine_flat_kernel, dim3(unsigned((n_pairs * 128 + 255) / 256)), dim3(256),
                        0, static_cast<cudaStream_t>(stream), part_acc, part_m, part_l,
                        static_cast<__nv_bfloat16*>(out), H, nsplit, n_pairs));
    return DSA_OK;
  }
  // one load group of 128 threads per split, up to four
  const int combine_threads = 128 * (nsplit < 4 ? nsplit : 4);
  DSA_CUDA(launch_pdl(mla::sparse_mla_combine_kernel, dim3(H, R), dim3(combine_threads), 0,
                      static_cast<cudaStream_t>(stream), part_acc, part_m, part_l,
                      static_cast<__nv_bfloat16*>(out), H, nsplit));
  return DSA_OK;
}

int dsa_sparse_mla_decode(const void* q, const void* kv, const int32_t* indices,
                          const int32_t* seq_lens, float* part_acc, float* part_m, float* part_l,
                          void* out, int R, int rows_per_seq, int H, int topk_k, int nsplit,
                          float sm_scale, int64_t kv_seq_stride, int kv_fp8, void* stream) {
  DSA_REQUIRE(out && aligned16(out), "sparse MLA: out must be a 16-byte aligned pointer");
  int rc = dsa_sparse_mla_partials(q, kv, indices, seq_lens, part_acc, part_m, part_l, R,
                                   rows_per_seq, H, topk_k, nsplit, sm_scale, kv_seq_stride, kv_fp8,
                                   stream);
  if (rc) return rc;
  return dsa_sparse_mla_combine(part_acc, part_m, part_l, out, R, H, nsplit, stream);
}

int dsa_sparse_mla_decode_beside(const void* q, const void* kv, const int32_t* indices,
                                 const int32_t* seq_lens, float* part_acc, float* part_m, float* part_l,
                                 void* out, int R, int rows_per_seq, int H, int topk_k, int nsplit,
                                 float sm_scale, int64_t kv_seq_stride, int kv_fp8, void* stream) {
  DSA_REQUIRE(out && aligned16(out), "sparse MLA: out must be a 16-byte aligned pointer");
  int rc = mla_partials_launch(q, kv, indices, seq_lens, part_acc, part_m, part_l, R, rows_per_seq, H, topk_k,
                               nsplit, sm_scale, kv_seq_stride, kv_fp8, true, stream);
  if (rc) return rc;
  return dsa_sparse_mla_combine(part_acc, part_m, part_l, out, R, H, nsplit, stream);
}

// ------------------------------------------------------------------ decode-step preparation
int dsa_rmsnorm(const void* x, const void* weight, void* out, int64_t rows, int dim, float eps, int dtype,
                void* stream) {
  DSA_REQUIRE(x && weight && out, "rmsnorm: null pointer");
  DSA_REQUIRE(rows > 0 && rows < (int64_t(1) << 31) && dim > 0, "rmsnorm: bad shape");
  DSA_REQUIRE(dtype == 0 || dtype == 1, "rmsnorm: dtype must be 0 (fp32) or 1 (bf16)");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0) {
    DSA_CUDA(launch_pdl(prep::rmsnorm_kernel<float>, dim3(unsigned(rows)), dim3(256), 0, st,
                        static_cast<const float*>(x), static_cast<const float*>(weight), static_cast<float*>(out),
                        dim, eps));
  } else if (dim % 8 == 0 && dim <= prep::kNormMaxDim && aligned16(x) && aligned16(weight) && aligned16(out)) {
    DSA_CUDA(launch_pdl(prep::rmsnorm_bf16_rows_kernel<false>, dim3(unsigned(rows)), dim3(256), 0, st,
                        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(nullptr),
                        static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(nullptr),
                        static_cast<__nv_bfloat16*>(out), dim, eps));
  } else {
    DSA_CUDA(launch_pdl(prep::rmsnorm_kernel<__nv_bfloat16>, dim3(unsigned(rows)), dim3(256), 0, st,
                        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight),
                        static_cast<__nv_bfloat16*>(out), dim, eps));
  }
  return DSA_OK;
}

int dsa_add_rmsnorm_bf16(const void* x, const void* delta, const void* weight, void* sum_out, void* out,
                         int64_t rows, int dim, float eps, void* stream) {
  DSA_REQUIRE(x && delta && weight && sum_out && out, "add + rmsnorm: null pointer");
  DSA_REQUIRE(rows > 0 && rows < (int64_t(1) << 31), "add + rmsnorm: bad row count");
  DSA_REQUIRE(dim > 0 && dim % 8 == 0 && dim <= prep::kNormMaxDim,
              "add + rmsnorm: dim=%d must be a multiple of 8 and at most %d", dim, prep::kNormMaxDim);
  DSA_REQUIRE(aligned16(x) && aligned16(delta) && aligned16(weight) && aligned16(sum_out) && aligned16(out),
              "add + rmsnorm: pointers must be 16-byte aligned");
  DSA_CUDA(launch_pdl(prep::rmsnorm_bf16_rows_kernel<true>, dim3(unsigned(rows)), dim3(256), 0,
                      static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x),
                      static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight),
                      static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(out), dim, eps));
  return DSA_OK;
}

int dsa_copy_bytes(void* dst, const void* src, int64_t bytes, void* stream) {
  DSA_REQUIRE(dst && src, "copy: null pointer");
  DSA_REQUIRE(bytes > 0 && bytes % 16 == 0 && aligned16(dst) && aligned16(src),
              "copy: size and both pointers must be multiples of 16 bytes");
  const int64_t n16 = bytes / 16;
  int64_t blocks = (n16 + 255) / 256;
  if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
  DSA_CUDA(launch_pdl(prep::copy16_kernel, dim3(unsigned(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                      static_cast<uint4*>(dst), static_cast<const uint4*>(src), n16));
  return DSA_OK;
}

int dsa_copy_bytes_beside(void* dst, const void* src, int64_t bytes, void* stream) {
  DSA_REQUIRE(dst && src, "copy: null pointer");
  DSA_REQUIRE(bytes > 0 && bytes % 16 == 0 && aligned16(dst) && aligned16(src),
              "copy: size and both pointers must be multiples of 16 bytes");
  const int64_t n16 = bytes / 16;
  int64_t blocks = (n16 + 255) / 256;
  if (blocks > sm_count()) blocks = sm_count();  // its CTAs stay resident until the kernel before it has completed
  DSA_CUDA(launch_pdl(prep::copy16_beside_kernel, dim3(unsigned(blocks)), dim3(256), 0,
                      static_cast<cudaStream_t>(stream), static_cast<uint4*>(dst), static_cast<const uint4*>(src), n16));
  return DSA_OK;
}

int dsa_post_epoch(uint32_t* counter, uint32_t* host_flag, void* stream) {
  DSA_REQUIRE(counter && host_flag, "post epoch: null pointer");
  // an ordinary launch (no programmatic overlap): it must start after everything before it has completed
  prep::post_epoch_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(counter, host_flag);
  DSA_CUDA(cudaGetLastError());
  return DSA_OK;
}

int dsa_copy_post_epoch(void* dst, const void* src, int64_t bytes, uint32_t* counter, uint32_t* host_flag,
                        int beside, void* stream) {
  DSA_REQUIRE(dst && src && counter && host_flag, "copy + post epoch: null pointer");
  DSA_REQUIRE(bytes > 0 && bytes <= (int64_t(1) << 20) && bytes % 16 == 0 && aligned16(dst) && aligned16(src),
              "copy + post epoch: at most 1 MiB; size and both pointers must be multiples of 16 bytes");
  DSA_CUDA(launch_pdl(prep::copy_post_epoch_kernel, dim3(1), dim3(512), 0, static_cast<cudaStream_t>(stream),
                      static_cast<uint4*>(dst), static_cast<const uint4*>(src), bytes / 16, counter,
                      static_cast<volatile uint32_t*>(host_flag), beside ? 1 : 0));
  return DSA_OK;
}

int dsa_gemv_bf16(const void* w, const void* x, void* y, int batch, int n, int k, int64_t x_stride,
                  int64_t y_stride, void* stream) {
  DSA_REQUIRE(w && x && y, "gemv: null pointer");
  DSA_REQUIRE(batch >= 1 && batch <= 4, "gemv: batch=%d must be 1..4", batch);
  DSA_REQUIRE(n > 0 && k > 0 && k % 8 == 0, "gemv: k=%d must be a positive multiple of 8", k);
  DSA_REQUIRE(int64_t(batch) * k * 2 <= 96 * 1024, "gemv: batch * k too large for the shared-memory copy of x");
  DSA_REQUIRE(x_stride >= k && x_stride % 8 == 0 && y_stride >= n, "gemv: bad row strides");
  DSA_REQUIRE(aligned16(w) && aligned16(x), "gemv: w and x must be 16-byte aligned");
  const size_t smem = size_t(batch) * k * 2;
  // One row per warp with eight 16-byte loads per lane in flight ([32832, 1536]: 18.5 us against
  // 20.9 / 25.6 us with 2 / 4 rows per warp and fewer loads per row; [36864, 7168]: 79 / 84 / 107 us).
  int blocks = (n * 32 + prep::kGemvThreads - 1) / prep::kGemvThreads;
  if (blocks > 8 * sm_count()) blocks = 8 * sm_count();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
#define DSA_GEMV_CASE(BV)                                                                                     \
  case BV: {                                                                                                  \
    if (smem > 48 * 1024) {                                                                                   \
      int rc = opt_in_smem(prep::gemv_bf16_kernel<BV, 1>, 96 * 1024, g_opt_gemv[BV - 1]);                     \
      if (rc) return rc;                                                                                      \
    }                                                                                                         \
    DSA_CUDA(launch_pdl(prep::gemv_bf16_kernel<BV, 1>, dim3(blocks), dim3(prep::kGemvThreads), smem, st, wp,  \
                        xp, yp, n, k, x_stride, y_stride));                                                   \
  } break;
  switch (batch) {
    DSA_GEMV_CASE(1)
    DSA_GEMV_CASE(2)
    DSA_GEMV_CASE(3)
    DSA_GEMV_CASE(4)
  }
#undef DSA_GEMV_CASE
  return DSA_OK;
}

int dsa_silu_mul_bf16(const void* gate, const void* up, void* out, int64_t n, void* stream) {
  DSA_REQUIRE(gate && up && out, "silu * up: null pointer");
  DSA_REQUIRE(n > 0 && n < (int64_t(1) << 40), "silu * up: bad element count");
  DSA_REQUIRE(aligned16(gate) && aligned16(up) && aligned16(out), "silu * up: pointers must be 16-byte aligned");
  const int64_t blocks = (n + 2047) / 2048;
  DSA_CUDA(launch_pdl(prep::silu_mul_bf16_kernel, dim3(unsigned(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
                      static_cast<__nv_bfloat16*>(out), n));
  return DSA_OK;
}

int dsa_indexer_stage_fp8(const void* q_raw, const void* k_raw, const float* w_raw,
                          const float* k_norm_weight, const float* k_norm_bias, float k_norm_eps,
                          const float* rope_cos, const float* rope_sin, const int64_t* positions,
                          uint8_t* index_q, float* index_w, uint8_t* cache_index_k,
                          float* cache_k_scale, uint8_t* pages, int64_t num_pages,
                          const int32_t* page_table, int64_t pt_stride, int B, int n_heads, int64_t cap,
                          int rope_interleave, int round_scale, float head_scale, float softmax_scale,
                          void* stream) {
  DSA_REQUIRE(q_raw && k_raw && w_raw && k_norm_weight && k_norm_bias && rope_cos && rope_sin && positions &&
                  index_q && index_w,
              "indexer stage: null pointer");
  DSA_REQUIRE((pages && page_table && pt_stride > 0) || (!pages && cache_index_k && cache_k_scale),
              "indexer stage: give either the dense key cache or pages + page table");
  DSA_REQUIRE(aligned16(q_raw) && aligned16(index_q) && aligned16(k_norm_weight) && aligned16(k_norm_bias) &&
                  (pages ? aligned16(pages) : aligned16(cache_index_k)) && (uintptr_t(k_raw) & 7) == 0,
              "indexer stage: pointers must be 16-byte aligned (k_raw: 8)");
  DSA_REQUIRE(B > 0 && n_heads > 0 && cap > 0 && int64_t(B) * (n_heads + 1) < (int64_t(1) << 30),
              "indexer stage: bad shape");
  DSA_REQUIRE(!pages || (num_pages > 0 && num_pages < (int64_t(1) << 31)), "indexer stage: bad num_pages");
  DSA_REQUIRE(!pages || pt_stride * DSA_PAGE_TOKENS >= cap,
              "indexer stage: pt_stride=%lld pages cannot cover cap=%lld positions", (long long)pt_stride,
              (long long)cap);
  prep::StageParams p{};
  p.q_raw = static_cast<const __nv_bfloat16*>(q_raw);
  p.k_raw = static_cast<const __nv_bfloat16*>(k_raw);
  p.w_raw = w_raw;
  p.norm_w = k_norm_weight;
  p.norm_b = k_norm_bias;
  p.rope_cos = rope_cos;
  p.rope_sin = rope_sin;
  p.positions = positions;
  p.index_q = index_q;
  p.index_w = index_w;
  p.cache_index_k = cache_index_k;
  p.cache_k_scale = cache_k_scale;
  p.pages = pages;
  p.page_table = page_table;
  p.pt_stride = pt_stride;
  p.num_pages = num_pages;
  p.cap = cap;
  p.B = B;
  p.n_heads = n_heads;
  p.interleave = rope_interleave;
  p.round_scale = round_scale;
  p.eps = k_norm_eps;
  p.head_scale = head_scale;
  p.softmax_scale = softmax_scale;
  p.hadamard_scale = 0.08838834764831845f;  // 128^-0.5
  const int rows = B * (n_heads + 1);
  DSA_CUDA(launch_pdl(prep::indexer_stage_kernel, dim3((rows + prep::kStageWarps - 1) / prep::kStageWarps),
                      dim3(prep::kStageWarps * 32), 0, static_cast<cudaStream_t>(stream), p));
  return DSA_OK;
}

int dsa_latent_append(const void* kv_a, const float* kv_norm_weight, float eps, const float* rope_cos,
                      const float* rope_sin, const int64_t* positions, const int64_t* slots, void* pool,
                      int B, int64_t cap, int64_t n_slots, int rope_interleave, int format,
                      int round_scale, void* stream) {
  DSA_REQUIRE(kv_a && kv_norm_weight && rope_cos && rope_sin && positions && slots && pool,
              "latent append: null pointer");
  DSA_REQUIRE(aligned16(kv_a) && aligned16(kv_norm_weight) && aligned16(pool),
              "latent append: pointers must be 16-byte aligned");
  DSA_REQUIRE(B > 0 && cap > 0 && n_slots > 0, "latent append: bad shape");
  DSA_REQUIRE(format >= 0 && format <= 2, "latent append: format must be 0 (bf16), 1 (bf16, quantised values) or 2 (fp8-packed)");
  prep::LatentParams p{};
  p.kv_a = static_cast<const __nv_bfloat16*>(kv_a);
  p.norm_w = kv_norm_weight;
  p.rope_cos = rope_cos;
  p.rope_sin = rope_sin;
  p.positions = positions;
  p.slots = slots;
  p.pool = static_cast<uint8_t*>(pool);
  p.cap = cap;
  p.n_slots = n_slots;
  p.B = B;
  p.interleave = rope_interleave;
  p.format = format;
  p.round_scale = round_scale;
  p.eps = eps;
  DSA_CUDA(launch_pdl(prep::latent_append_kernel, dim3((B + prep::kStageWarps - 1) / prep::kStageWarps),
                      dim3(prep::kStageWarps * 32), 0, static_cast<cudaStream_t>(stream), p));
  return DSA_OK;
}

int dsa_decode_prep(const void* iq_raw, const void* w_raw, const void* ik_raw, const void* kv_a,
                    const void* q_abs, const void* q_pe, int64_t q_pe_stride, const void* kv_norm_w,
                    const void* mla_cos, const void* mla_sin, const void* idx_cos, const void* idx_sin,
                    const int64_t* positions, uint8_t* index_q, float* index_w, void* q_full,
                    uint8_t* cache_index_k, float* cache_k_scale, void* cache_kv, int B, int H,
                    int n_index_heads, int64_t cap, int interleave, float eps, void* stream) {
  DSA_REQUIRE(iq_raw && w_raw && ik_raw && kv_a && q_abs && q_pe && kv_norm_w && mla_cos && mla_sin && idx_cos &&
                  idx_sin && positions && index_q && index_w && q_full && cache_index_k && cache_k_scale && cache_kv,
              "decode prep: null pointer");
  DSA_REQUIRE(aligned16(iq_raw) && aligned16(ik_raw) && aligned16(q_abs) && aligned16(q_full) && aligned16(index_q) &&
                  aligned16(cache_index_k) && aligned16(cache_kv),
              "decode prep: pointers must be 16-byte aligned");
  DSA_REQUIRE(B > 0 && B <= 65535 && H > 0 && n_index_heads > 0 && cap > 0, "decode prep: bad shape");
  DSA_REQUIRE(q_pe_stride >= 64, "decode prep: q_pe_stride must be >= 64 elements");
  prep::Params p{};
  p.iq_raw = static_cast<const __nv_bfloat16*>(iq_raw);
  p.w_raw = static_cast<const __nv_bfloat16*>(w_raw);
  p.ik_raw = static_cast<const __nv_bfloat16*>(ik_raw);
  p.kv_a = static_cast<const __nv_bfloat16*>(kv_a);
  p.q_abs = static_cast<const __nv_bfloat16*>(q_abs);
  p.q_pe = static_cast<const __nv_bfloat16*>(q_pe);
  p.q_pe_stride = q_pe_stride;
  p.kv_norm_w = static_cast<const __nv_bfloat16*>(kv_norm_w);
  p.mla_cos = static_cast<const __nv_bfloat16*>(mla_cos);
  p.mla_sin = static_cast<const __nv_bfloat16*>(mla_sin);
  p.idx_cos = static_cast<const __nv_bfloat16*>(idx_cos);
  p.idx_sin = static_cast<const __nv_bfloat16*>(idx_sin);
  p.positions = positions;
  p.index_q = index_q;
  p.index_w = index_w;
  p.q_full = static_cast<__nv_bfloat16*>(q_full);
  p.cache_index_k = cache_index_k;
  p.cache_k_scale = cache_k_scale;
  p.cache_kv = static_cast<__nv_bfloat16*>(cache_kv);
  p.cap = cap;
  p.B = B;
  p.H = H;
  p.Hidx = n_index_heads;
  p.interleave = interleave;
  p.eps = eps;
  const int items = n_index_heads + 2 + H;
  DSA_CUDA(launch_pdl(prep::decode_prep_kernel, dim3((items + 3) / 4, B), dim3(128), 0,
                      static_cast<cudaStream_t>(stream), p));
  return DSA_OK;
}

// ------------------------------------------------------------------ fused indexer + attention launch
int dsa_fused_decode(const void* q, const void* kv, const int32_t* attend_indices,
                     const int32_t* attn_seq_lens, float* part_acc, float* part_m, float* part_l, void* out,
                     const uint8_t* index_q, const float* index_w, const uint8_t* index_k,
                     const float* k_scale, const int32_t* index_seq_lens, float* logits, uint32_t* hist,
                     int R, int rows_per_seq, int H, int topk_k, int nsplit, float sm_scale,
                     int64_t kv_seq_stride, int n_index_heads, int64_t ctx, int64_t n_seq,
                     int64_t k_seq_stride, int64_t scale_seq_stride, int64_t slab_stride, void* stream) {
  mla::Params pm;
  int rc = mla_prepare(q, kv, attend_indices, attn_seq_lens, part_acc, part_m, part_l, R, rows_per_seq, H,
                       topk_k, nsplit, sm_scale, kv_seq_stride, 0, true, &pm);
  if (rc) return rc;
  DSA_REQUIRE(out && aligned16(out), "fused decode: out must be a 16-byte aligned pointer");
  rc = scan_common_checks(index_q, index_w, logits, R, n_index_heads, ctx, slab_stride);
  if (rc) return rc;
  DSA_REQUIRE(index_k && k_scale && aligned16(index_k), "fused decode: bad key cache pointers");
  DSA_REQUIRE(n_seq == R / rows_per_seq, "fused decode: n_seq=%lld but R / rows_per_seq = %d", (long long)n_seq,
              R / rows_per_seq);
  DSA_REQUIRE(k_seq_stride >= ctx && scale_seq_stride >= ctx, "fused decode: sequence strides must be >= ctx");
  DSA_REQUIRE(n_seq * k_seq_stride < (int64_t(1) << 31), "fused decode: key cache too large");
  scan::Params ps{};
  ps.q = index_q;
  ps.w = index_w;
  ps.keys = index_k;
  ps.k_scale = k_scale;
  ps.seq_lens = index_seq_lens;
  ps.logits = logits;
  ps.hist = hist;
  ps.ctx = ctx;
  ps.k_seq_stride = k_seq_stride;
  ps.scale_seq_stride = scale_seq_stride;
  ps.slab_stride = slab_stride;
  ps.rows_per_seq = rows_per_seq;
  ps.n_heads = n_index_heads;
  ps.tiles_per_row = int((ctx + scan::kTileKeys - 1) / scan::kTileKeys);
  ps.paged = 0;
  CUtensorMap tmap;
  const uint64_t rows = uint64_t(n_seq - 1) * uint64_t(k_seq_stride) + uint64_t(ctx);
  const uint64_t dims[2] = {uint64_t(scan::kKeyBytes), rows};
  const uint64_t strides[1] = {uint64_t(scan::kKeyBytes)};
  const uint32_t box[2] = {uint32_t(scan::kKeyBytes), uint32_t(scan::kTileKeys)};
  rc = encode_tensor_map(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, index_k, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = opt_in_smem(fused::fused_decode_kernel, fused::kSmemBytes, g_opt_fused);
  if (rc) return rc;
  const int hgs = H / DSA_HEAD_BLOCK;
  const int n_attn = nsplit * hgs * R;
  const int scan_gx = scan_grid_x(R, ps.tiles_per_row, 2);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DSA_CUDA(launch_pdl(fused::fused_decode_kernel, dim3(n_attn + scan_gx * R), dim3(fused::kThreads),
                      fused::kSmemBytes, st, tmap, ps, pm, n_attn, nsplit, hgs, scan_gx));
  return dsa_sparse_mla_combine(part_acc, part_m, part_l, out, R, H, nsplit, stream);
}

int dsa_sparse_mla_f32(const float* q, const float* kv, const int32_t* indices,
                       const int32_t* seq_lens, float* out, int R, int rows_per_seq, int H,
                       int qk_dim, int v_dim, int topk_k, float sm_scale, int64_t kv_seq_stride,
                       void* stream) {
  DSA_REQUIRE(q && kv && out, "f32 sparse MLA: null pointer");
  DSA_REQUIRE(R > 0 && R <= 65535 && rows_per_seq > 0 && R % rows_per_seq == 0,
              "f32 sparse MLA: bad R=%d / rows_per_seq=%d", R, rows_per_seq);
  DSA_REQUIRE(H > 0 && qk_dim > 0 && v_dim > 0 && v_dim <= qk_dim && v_dim <= 512,
              "f32 sparse MLA: need 0 < v_dim <= min(qk_dim, 512)");
  DSA_REQUIRE(indices == nullptr || topk_k > 0, "f32 sparse MLA: topk must be positive");
  const size_t smem = (size_t(qk_dim) + 128 + 128 + 8) * sizeof(float);
  DSA_REQUIRE(smem <= 48 * 1024, "f32 sparse MLA: qk_dim too large");
  mla::sparse_mla_f32_kernel<<<dim3(H, R), 128, smem, static_cast<cudaStream_t>(stream)>>>(
      q, kv, indices, seq_lens, out, rows_per_seq, H, qk_dim, v_dim, topk_k, sm_scale,
      kv_seq_stride, kv_seq_stride);
  DSA_CUDA(cudaGetLastError());
  return DSA_OK;
}

// ------------------------------------------------------------------ quantisation
int dsa_quantize_e4m3_rowwise(const float* x, uint8_t* q_out, float* scale_out, int64_t rows,
                              int cols, float clamp_min, void* stream) {
  DSA_REQUIRE(x && q_out && scale_out, "quantize: null pointer");
  DSA_REQUIRE(rows > 0 && cols > 0, "quantize: bad shape");
  const int64_t blocks = (rows + 3) / 4;
  DSA_REQUIRE(blocks < (int64_t(1) << 31), "quantize: too many rows");
  dsa::quantize_rowwise_kernel<<<unsigned(blocks), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      x, q_out, scale_out, rows, cols, clamp_min);
  DSA_CUDA(cudaGetLastError());
  return DSA_OK;
}

}  // extern "C"
