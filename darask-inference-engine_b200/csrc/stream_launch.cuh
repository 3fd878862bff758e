// Host side of expert_stream.cuh: picks the CTA shape for a matrix shape and launches with the
// programmatic-dependent-launch attribute.
#pragma once
#include "expert_stream.cuh"

namespace dmoe {

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
  return cached[dev];
}

constexpr int kSmemBudget = 227 * 1024;
constexpr int kComputeWarps = 12;

// Chooses row groups / K split / ring depth so that the ring holds at least two stages and as
// many compute warps as fit. Returns false when even one row group does not fit.
inline bool plan_stream(StreamArgs& a, int fmt, int tt, int* smem_bytes) {
  // Row-slot pitch chosen so that the lane pattern of the tile loads (8 rows x 4 lanes) is free of
  // bank conflicts: 8-byte loads (Q4_K) want pitch % 128 in {32, 96}, 4-byte loads pitch % 32 == 16.
  a.pitch = a.row_bytes;
  if (fmt == kFmtQ4K) while (a.pitch % 128 != 32 && a.pitch % 128 != 96) a.pitch += 16;
  else while (a.pitch % 32 != 16) a.pitch += 16;
  a.ks = a.nblk < kComputeWarps ? a.nblk : kComputeWarps;
  for (int rg = kComputeWarps / a.ks > 0 ? kComputeWarps / a.ks : 1; rg >= 1; --rg) {
    for (int stages = kMaxStages; stages >= 2; --stages) {
      const StreamSmem s = stream_smem(fmt, rg, a.ks, stages, a.pitch, a.k, tt);
      if (s.total <= kSmemBudget && (stages >= 3 || rg == 1 || stages * s.stage_bytes >= 128 * 1024)) {
        a.rg = rg;
        a.stages = stages;
        *smem_bytes = s.total;
        return true;
      }
    }
  }
  return false;
}

template <typename Kernel, typename... Args>
inline cudaError_t launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <int FMT, int DUAL, int TT, int ACT>
inline cudaError_t launch_stream_tt(StreamArgs a, cudaStream_t stream) {
  int smem = 0;
  if (!plan_stream(a, FMT, TT, &smem)) return cudaErrorInvalidConfiguration;
  auto kernel = expert_stream_kernel<FMT, DUAL, TT, ACT>;
  static bool configured = false;       // one opt-in per instantiation (and process)
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  return launch_pdl(kernel, dim3(sm_count()), dim3((a.rg * a.ks + 1) * 32), size_t(smem), stream, a);
}

// `max_rows_per_group`: upper bound of tokens that can share one expert in this call.
template <int FMT, int DUAL, int ACT>
inline cudaError_t launch_stream(const StreamArgs& a, int max_rows_per_group, cudaStream_t stream) {
  if (a.row_bytes % 16 || a.expert_stride[0] % 16 || a.expert_stride[1] % 16 || a.k % 256) return cudaErrorInvalidValue;
  if (max_rows_per_group <= 1) return launch_stream_tt<FMT, DUAL, 1, ACT>(a, stream);
  return launch_stream_tt<FMT, DUAL, 2, ACT>(a, stream);
}

}  // namespace dmoe
