// Hayate prefill launchers under the reference's own names and signatures (engines/hayate/crates/kernels/src/glm53.rs:
// 588-650; reference bodies cu/glm53/grouped.cu:28-124): NVFP4 image -> bf16 restore, row gather, weighted scatter,
// device copy, and the ragged grouped bf16 GEMM (here on tcgen05 with TMEM accumulators, see grouped_bf16.cuh).
// Contract as in the reference: enqueue only, no allocation, no synchronisation, cudaErrorInvalidValue for bad
// arguments, otherwise cudaGetLastError().
#include <cuda_fp8.h>
#include "../../include/darask_moe_b200.h"
#include "grouped_bf16.cuh"
#include "grouped_nvfp4.cuh"
#include "stream_launch.cuh"

namespace dmoe {

int hayate_shape_topk();      // hayate.cu: the thread's `topk` (reference literal 8 until hayate_glm_moe_set_shape)

DEVI float e4m3_value(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(__nv_fp8_storage_t(b), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
// value of element (r, c) of an NVFP4 matrix image: the reference's `nvfp4` (cu/glm53/math.cuh:41-49), product
// formed in its order ((e2m1 * e4m3) * global)
DEVI float nvfp4_element(const uint8_t* image, unsigned r, unsigned c, unsigned n, unsigned k, bool scaled) {
  const unsigned code = (image[(size_t(r) * k + c) / 2] >> (4 * (c % 2))) & 15u;
  const unsigned cols = (k / 16 + 3) / 4 * 4, scol = c / 16;
  const size_t tile = size_t((r / 128) * (cols / 4) + scol / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + scol % 4;
  const uint8_t* scales = image + size_t(n) * k / 2;
  const float global = *reinterpret_cast<const float*>(scales + size_t((n + 127) / 128 * 128) * cols);
  const unsigned m = code & 7u;
  const float mag = m < 4 ? 0.5f * float(m) : (m == 4 ? 2.f : m == 5 ? 3.f : m == 6 ? 4.f : 6.f);
  return mag * ((code & 8u) ? -1.f : 1.f) * e4m3_value(scales[tile]) * (scaled ? global : 1.f);
}
__global__ void __launch_bounds__(256) restore_nvfp4_kernel(__nv_bfloat16* out, const uint8_t* image, unsigned n, unsigned k, bool scaled,
                                                            float* global_out) {
  if (global_out && blockIdx.x == 0 && threadIdx.x == 0) {
    const size_t at = size_t(n) * k / 2 + size_t((n + 127) / 128 * 128) * ((k / 16 + 3) / 4 * 4);
    *global_out = *reinterpret_cast<const float*>(image + at);
  }
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i < size_t(n) * k) out[i] = __float2bfloat16_rn(nvfp4_element(image, unsigned(i / k), unsigned(i % k), n, k, scaled));
}
// block-FP8 matrix -> bf16: out = bf16(e4m3(w) * scale[row/128][col/128])   (reference `restore`, cu/glm53/ops.cu:13-16)
__global__ void __launch_bounds__(256) restore_fp8_kernel(__nv_bfloat16* out, const uint8_t* w, const float* scale, unsigned n, unsigned k) {
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i < size_t(n) * k) out[i] = __float2bfloat16_rn(e4m3_value(w[i]) * scale[(i / k / 128) * ((k + 127) / 128) + (i % k) / 128]);
}
// out row i = x row assignments[i] / topk, 16 bytes per thread
__global__ void __launch_bounds__(256) gather_rows_kernel(uint4* out, const uint4* x, const unsigned* assignments, unsigned rows,
                                                          unsigned chunks, unsigned topk) {
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i < size_t(rows) * chunks) out[i] = x[size_t(assignments[i / chunks] / topk) * chunks + i % chunks];
}
__global__ void __launch_bounds__(256) gather_rows_scalar_kernel(__nv_bfloat16* out, const __nv_bfloat16* x, const unsigned* assignments,
                                                                 unsigned rows, unsigned hidden, unsigned topk) {
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i < size_t(rows) * hidden) out[i] = x[size_t(assignments[i / hidden] / topk) * hidden + i % hidden];
}
// out[token] = bf16(out[token] + bf16(x[i] * weights[a])): at most one row per token in a call (the caller enqueues
// experts in ascending id), so there is no race on out
__global__ void __launch_bounds__(256) scatter_rows_kernel(__nv_bfloat16* out, const __nv_bfloat16* x, const float* weights,
                                                           const unsigned* assignments, unsigned rows, unsigned hidden, unsigned topk) {
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= size_t(rows) * hidden) return;
  const unsigned a = assignments[i / hidden];
  const size_t dst = size_t(a / topk) * hidden + i % hidden;
  const float term = __bfloat162float(__float2bfloat16_rn(__bfloat162float(x[i]) * weights[a]));
  out[dst] = __float2bfloat16_rn(__bfloat162float(out[dst]) + term);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// also used by the Tsumuji token-window path (tsumuji.cu)
cudaError_t launch_grouped_bf16(void* out, float* acc, const void* x, const void* w, const void* ranges, unsigned groups,
                                       unsigned n, unsigned k, const float* scales, cudaStream_t st, unsigned w_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return cudaErrorInvalidValue;
  CUtensorMap mw;
  // w_rows: rows the weight array really has (0: groups * n); tiles past it read zeros, never memory
  const cuuint64_t dims[2] = {k, w_rows ? cuuint64_t(w_rows) : cuuint64_t(groups) * n}, strides[1] = {cuuint64_t(k) * 2};
  const cuuint32_t box[2] = {kGbTileK, 128}, estr[2] = {1, 1};
  if (enc(&mw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  GbArgs g = {};
  g.x = static_cast<const __nv_bfloat16*>(x);
  g.ranges = static_cast<const unsigned*>(ranges);
  g.groups = int(groups); g.n = int(n); g.k = int(k);
  g.out = static_cast<__nv_bfloat16*>(out);
  g.acc = acc; g.scales = scales; g.status = nullptr;
  const size_t smem = size_t(kGbFixedSmem) + size_t(groups + 1) * sizeof(int);
  static bool configured[64] = {};      // the opt-in is per device
  const int dev = current_device_slot();
  if (dev < 0) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(grouped_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               int(kGbFixedSmem + 1025 * sizeof(int)));
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return launch_pdl(grouped_bf16_kernel, dim3(sm_count()), dim3(kGbThreads), smem, st, mw, g);
}

static bool grouped_shape_ok(unsigned groups, unsigned n, unsigned k) {
  return groups && groups <= 1024 && n >= 128 && n % 128 == 0 && k >= unsigned(kGbTileK) && k % kGbTileK == 0;
}

// ---- packed NVFP4 images in place (grouped_nvfp4.cuh) ----------------------------------------------------------
// The reference's launchers have no status argument: what the kernels find wrong with an image on the device (a format
// other than NVFP4, a null pointer) goes to this word, which hayate_glm_grouped_packed_status reads and clears.
__device__ unsigned g_packed_status;

template <bool DOWN>
static cudaError_t launch_grouped_packed(void* out, const void* x, const void* images, const void* formats, const void* ranges,
                                         unsigned count, unsigned hidden, unsigned inter, cudaStream_t st) {
  GnArgs g = {};
  g.x = static_cast<const __nv_bfloat16*>(x);
  g.images = static_cast<const void* const*>(images);
  g.formats = static_cast<const HayateExpertFormat*>(formats);
  g.ranges = static_cast<const unsigned*>(ranges);
  g.count = int(count); g.hidden = int(hidden); g.inter = int(inter);
  g.out = static_cast<__nv_bfloat16*>(out);
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&g.status), g_packed_status);
  if (e != cudaSuccess) return e;
  static_assert(kGnFixedSmem + 289 * sizeof(int) <= size_t(kSmemBudget), "stages and staging must fit one CTA");
  const size_t smem = size_t(kGnFixedSmem) + size_t(count + 1) * sizeof(int);
  static bool configured[64][2] = {};   // the opt-in is per device and per kernel
  const int dev = current_device_slot();
  if (dev < 0) return cudaErrorInvalidDevice;
  if (!configured[dev][DOWN]) {
    e = cudaFuncSetAttribute(grouped_nvfp4_kernel<DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kGnFixedSmem + 289 * sizeof(int)));
    if (e != cudaSuccess) return e;
    configured[dev][DOWN] = true;
  }
  return launch_pdl(grouped_nvfp4_kernel<DOWN>, dim3(sm_count()), dim3(kGnThreads), smem, st, g);
}
// the argument checks of the reference (packed_grouped.cu:297-301)
static bool packed_args_ok(const void* out, const void* x, const void* images, const void* formats, const void* ranges, unsigned count,
                           unsigned hidden, unsigned inter) {
  return out && x && out != x && images && formats && ranges && count && count <= 288 && hidden && hidden <= 4096 && hidden % 256 == 0 &&
         inter && inter <= 4096 && inter % 256 == 0;
}

}  // namespace dmoe

using namespace dmoe;

extern "C" int hayate_glm_grouped_packed_gate_up(void* product, const void* x, const void* images, const void* formats, const void* ranges,
                                                 unsigned count, unsigned hidden, unsigned intermediate, cudaStream_t st) {
  if (!packed_args_ok(product, x, images, formats, ranges, count, hidden, intermediate)) return cudaErrorInvalidValue;
  return launch_grouped_packed<false>(product, x, images, formats, ranges, count, hidden, intermediate, st);
}

extern "C" int hayate_glm_grouped_packed_down(void* out, const void* product, const void* images, const void* formats, const void* ranges,
                                              unsigned count, unsigned hidden, unsigned intermediate, cudaStream_t st) {
  if (!packed_args_ok(out, product, images, formats, ranges, count, hidden, intermediate)) return cudaErrorInvalidValue;
  return launch_grouped_packed<true>(out, product, images, formats, ranges, count, hidden, intermediate, st);
}

// The reference picks one of four mma.sync tile shapes here; this library has one tcgen05 tile shape, so a valid id is
// accepted and changes nothing.
extern "C" int hayate_glm_grouped_packed_set_config(unsigned config) {
  return config > 3 ? cudaErrorInvalidValue : cudaSuccess;
}

extern "C" int hayate_glm_grouped_packed_status(unsigned* host_status, cudaStream_t st) {
  if (!host_status) return cudaErrorInvalidValue;
  unsigned* dev = nullptr;
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&dev), g_packed_status);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyAsync(host_status, dev, 4, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(dev, 0, 4, st);
  return e ? e : cudaStreamSynchronize(st);
}

extern "C" int hayate_glm_grouped(void* out, const void* x, const void* w, const void* ranges, unsigned groups, unsigned n, unsigned k,
                                  void* metadata, cudaStream_t st) {
  (void)metadata;           // the reference keeps its CUTLASS problem descriptors there; not needed here
  if (!out || !x || !w || !ranges || !grouped_shape_ok(groups, n, k)) return cudaErrorInvalidValue;
  return launch_grouped_bf16(out, nullptr, x, w, ranges, groups, n, k, nullptr, st, 0);
}

extern "C" int hayate_glm_grouped_nvfp4(void* out, void* accumulator, const void* x, const void* w, const void* ranges, unsigned groups,
                                        unsigned n, unsigned k, void* metadata, const void* scales, unsigned max_rows, cudaStream_t st) {
  (void)metadata;
  if (!out || !accumulator || !x || !w || !ranges || !scales || !max_rows || !grouped_shape_ok(groups, n, k)) return cudaErrorInvalidValue;
  return launch_grouped_bf16(out, static_cast<float*>(accumulator), x, w, ranges, groups, n, k, static_cast<const float*>(scales), st, 0);
}

extern "C" int hayate_glm_nvfp4_restore(void* out, const void* image, unsigned n, unsigned k, cudaStream_t st) {
  if (!out || !image || !n || !k || k % 16) return cudaErrorInvalidValue;
  restore_nvfp4_kernel<<<unsigned((size_t(n) * k + 255) / 256), 256, 0, st>>>(static_cast<__nv_bfloat16*>(out),
                                                                             static_cast<const uint8_t*>(image), n, k, true, nullptr);
  return cudaGetLastError();
}

extern "C" int hayate_glm_nvfp4_restore_unscaled(void* out, void* scale, const void* image, unsigned n, unsigned k, cudaStream_t st) {
  if (!out || !scale || !image || !n || !k || k % 16) return cudaErrorInvalidValue;
  restore_nvfp4_kernel<<<unsigned((size_t(n) * k + 255) / 256), 256, 0, st>>>(static_cast<__nv_bfloat16*>(out),
                                                                             static_cast<const uint8_t*>(image), n, k, false,
                                                                             static_cast<float*>(scale));
  return cudaGetLastError();
}

extern "C" int hayate_glm_restore(void* out, const void* w, const void* scale, unsigned n, unsigned k, cudaStream_t st) {
  if (!out || !w || !scale || !n || !k) return cudaErrorInvalidValue;
  restore_fp8_kernel<<<unsigned((size_t(n) * k + 255) / 256), 256, 0, st>>>(static_cast<__nv_bfloat16*>(out), static_cast<const uint8_t*>(w),
                                                                           static_cast<const float*>(scale), n, k);
  return cudaGetLastError();
}

extern "C" int hayate_glm_gather(void* out, const void* x, const void* assignments, unsigned rows, unsigned hidden, cudaStream_t st) {
  if (!out || !x || !assignments || !rows || !hidden) return cudaErrorInvalidValue;
  const unsigned topk = unsigned(hayate_shape_topk());
  if (hidden % 8 == 0 && !(reinterpret_cast<uintptr_t>(out) & 15) && !(reinterpret_cast<uintptr_t>(x) & 15)) {
    const unsigned chunks = hidden / 8;
    gather_rows_kernel<<<unsigned((size_t(rows) * chunks + 255) / 256), 256, 0, st>>>(static_cast<uint4*>(out), static_cast<const uint4*>(x),
                                                                                     static_cast<const unsigned*>(assignments), rows, chunks, topk);
  } else {
    gather_rows_scalar_kernel<<<unsigned((size_t(rows) * hidden + 255) / 256), 256, 0, st>>>(
        static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(x), static_cast<const unsigned*>(assignments), rows, hidden, topk);
  }
  return cudaGetLastError();
}

extern "C" int hayate_glm_scatter(void* out, const void* x, const void* weights, const void* assignments, unsigned rows, unsigned hidden,
                                  cudaStream_t st) {
  if (!out || !x || !weights || !assignments || !rows || !hidden) return cudaErrorInvalidValue;
  scatter_rows_kernel<<<unsigned((size_t(rows) * hidden + 255) / 256), 256, 0, st>>>(
      static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(weights),
      static_cast<const unsigned*>(assignments), rows, hidden, unsigned(hayate_shape_topk()));
  return cudaGetLastError();
}

extern "C" int hayate_glm_copy(void* out, const void* x, size_t bytes, cudaStream_t st) {
  if (!out || !bytes) return cudaErrorInvalidValue;
  return x ? cudaMemcpyAsync(out, x, bytes, cudaMemcpyDeviceToDevice, st) : cudaMemsetAsync(out, 0, bytes, st);
}
