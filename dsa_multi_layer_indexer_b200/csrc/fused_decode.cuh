// One launch that runs a layer's sparse-MLA split-K partials and its indexer
// scan side by side: the multi-layer-indexer ("lagged") schedule makes the two
// independent (attention reads the PREVIOUS layer's selection), so their CTAs
// can share the machine. Counterpart of the reference's role-split launch
// (kernels/cuda_fused_sparse_splitk.py:178-683: warps 0-3 attention, warps 4-7
// indexer; serving form hide_paged_kernel :2166-2225 assigns roles by
// blockIdx: attention blocks first, then indexer blocks). Here the roles are
// whole CTAs, interleaved by block index: attention CTAs run the split-K partials
// of sparse_mla_partials_kernel, scan CTAs run indexer_scan_tc_kernel's body. No CTA
// waits for another; the LSE merge and the top-k follow as their own launches.
#pragma once

#include "indexer_scan.cuh"
#include "sparse_mla.cuh"

namespace dsa {
namespace fused {

constexpr int kThreads = scan::kThreads;  // 192; an attention CTA uses its first 128 threads
constexpr size_t kSmemBytes =
    scan::smem_bytes<scan::kStagesTwoPerSm>() > size_t(mla::SmemLayout::bytes_bf16)
        ? scan::smem_bytes<scan::kStagesTwoPerSm>()
        : size_t(mla::SmemLayout::bytes_bf16);

__global__ void __launch_bounds__(kThreads, 2)
fused_decode_kernel(const __grid_constant__ CUtensorMap tmap, const scan::Params ps, const mla::Params pm,
                    const int n_attn, const int attn_splits, const int attn_hgs, const int scan_gx) {
  extern __shared__ __align__(16) uint8_t fused_smem[];
  // Roles alternate over the first 2 * min(n_attn, n_scan) block indices so both
  // kinds of work are in flight from the first wave on; the longer list's tail follows.
  const int n_scan = int(gridDim.x) - n_attn;
  const int n_pair = min(n_attn, n_scan);
  const int b = blockIdx.x;
  int attn_id = -1, scan_id = -1;
  if (b < 2 * n_pair) {
    if (b & 1) scan_id = b >> 1; else attn_id = b >> 1;
  } else if (n_attn > n_scan) {
    attn_id = b - n_pair;
  } else {
    scan_id = b - n_pair;
  }
  if (attn_id >= 0) {
    if (threadIdx.x >= mla::kThreads) return;  // two spare warps leave; the rest synchronise among themselves
    const int split = attn_id % attn_splits;
    const int hg = (attn_id / attn_splits) % attn_hgs;
    const int r = attn_id / (attn_splits * attn_hgs);
    mla::mla_partials_body<false>(pm, split, hg, r, fused_smem);
  } else {
    scan::scan_tc_body<scan::kStagesTwoPerSm>(&tmap, ps, scan_id % scan_gx, scan_gx, scan_id / scan_gx, fused_smem);
  }
}

}  // namespace fused
}  // namespace dsa
