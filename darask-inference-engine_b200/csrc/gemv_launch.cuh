// Host side of expert_gemv.cuh: K split selection and launch.
#pragma once
#include "expert_gemv.cuh"
#include "stream_launch.cuh"

namespace dmoe {

// Warps per row slab: the largest divisor of the block count (and of the warps per CTA) that still
// lets every slab x split item start in the first wave of the persistent grid.
inline int gemv_k_split(int nblk, long long slabs, int sms) {
  const long long warps = (long long)sms * kGemvWarps;
  int best = 1;
  for (int ks = 1; ks <= nblk && ks <= 12; ++ks)
    if (nblk % ks == 0 && kGemvWarps % ks == 0 && slabs * ks <= warps) best = ks;
  return best;
}

template <int FMT, int DUAL, bool MINS_TILE, int OUT>
inline cudaError_t launch_gemv(GemvArgs a, cudaStream_t stream) {
  if (a.row_bytes % 16 || a.expert_stride[0] % 16 || a.expert_stride[1] % 16 || a.k % 256 || a.rows < 1 || a.max_groups < 1)
    return cudaErrorInvalidValue;
  constexpr int RPT = DUAL ? 8 : 16;
  const long long slabs = (long long)a.max_groups * ((a.rows + RPT - 1) / RPT);
  a.ks = gemv_k_split(a.nblk, slabs, sm_count());
  if (slabs * a.ks >= (1ll << 31)) return cudaErrorInvalidValue;       // the kernel counts items in 32 bits
  const unsigned tiles_per_group = unsigned((a.rows + RPT - 1) / RPT);
  a.nb_per = a.nblk / a.ks;
  a.ks_inv = 65536 / a.ks + 1;
  a.slab_groups = kGemvWarps / a.ks;
  const unsigned slab_round = unsigned(sm_count()) * unsigned(a.slab_groups);   // slabs all CTAs take per round
  a.group_step = slab_round / tiles_per_group;
  a.slab_step = slab_round % tiles_per_group;
  if (a.out_shared_row == 0) a.out_shared_row = a.tokens * a.topk;
  if (FMT == kGemvNvfp4Tiled && a.rows % 128) return cudaErrorInvalidValue;
  const int smem = gemv_smem_bytes<FMT>();
  auto kernel = expert_gemv_kernel<FMT, DUAL, MINS_TILE, OUT>;
  static bool configured[64] = {};      // one opt-in per instantiation and device
  const int dev = current_device_slot();
  if (dev < 0) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return launch_pdl(kernel, dim3(sm_count()), dim3(kGemvWarps * 32), size_t(smem), stream, a);
}

}  // namespace dmoe
