// Load-time weight quantizers on the device (float32 source -> the byte layouts the expert
// kernels read) and the activation quantizer of the FP8 path.
//   NVFP4 linear  restates tsumuji kernels/decode/quant.cu:77-114 (`nvfp4_amax`, `nvfp4_quant`)
//   NVFP4 tiled   restates hayate python-tools/hayate_tools/quant.py:42-64 with the scale tiling
//                 of common/core/src/dtype.rs:85-105
//   block FP8     e4m3 payload + float32 scale per 128x128 block (hayate cpu/glm53.rs:23-24)
//   Q4_K / Q6_K   written from the block layout that kogarashi kernels/native.cu:26-40 decodes;
//                 the reference has no quantizer for them (its GGUF files arrive quantized)
#include "../../include/darask_moe_b200.h"
#include "common.cuh"
#include <cuda_fp8.h>

namespace dmoe {

DEVI float nearest(float v) { return floorf(v + 0.5f); }
DEVI uint8_t e4m3_rn(float v) { return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); }
DEVI float e4m3_value(uint8_t b) {
  __half_raw r = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&r));
}
// nearest e2m1 magnitude code (0..7) of a >= 0, midpoint ties to the even code
DEVI unsigned e2m1_code(float a) {
  return (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
}
DEVI float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// ---- GGUF Q4_K: one thread per 256-element super-block ----------------------------------------
__global__ void q4k_quant_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst, long long blocks) {
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= blocks) return;
  const float* x = src + b * 256;
  float sub_scale[8], sub_min[8], ms = 0.f, mm = 0.f;
  for (int g = 0; g < 8; ++g) {
    float lo = 0.f, hi = 0.f;
    for (int l = 0; l < 32; ++l) {
      lo = fminf(lo, x[g * 32 + l]);
      hi = fmaxf(hi, x[g * 32 + l]);
    }
    sub_scale[g] = (hi - lo) / 15.f;
    sub_min[g] = 0.f - lo;
    ms = fmaxf(ms, sub_scale[g]);
    mm = fmaxf(mm, sub_min[g]);
  }
  const __half d = __float2half_rn(ms / 63.f), dmin = __float2half_rn(mm / 63.f);
  const float df = __half2float(d), dmf = __half2float(dmin);
  int sc[8], mi[8];
  uint8_t* out = dst + b * 144;
  for (int g = 0; g < 8; ++g) {
    sc[g] = df > 0.f ? (int)fminf(fmaxf(nearest(sub_scale[g] / df), 0.f), 63.f) : 0;
    mi[g] = dmf > 0.f ? (int)fminf(fmaxf(nearest(sub_min[g] / dmf), 0.f), 63.f) : 0;
  }
  *reinterpret_cast<__half*>(out) = d;
  *reinterpret_cast<__half*>(out + 2) = dmin;
  for (int g = 0; g < 4; ++g) {
    out[4 + g] = uint8_t(sc[g] | ((sc[g + 4] >> 4) << 6));
    out[8 + g] = uint8_t(mi[g] | ((mi[g + 4] >> 4) << 6));
    out[12 + g] = uint8_t((sc[g + 4] & 15) | ((mi[g + 4] & 15) << 4));
  }
  for (int p = 0; p < 4; ++p)
    for (int l = 0; l < 32; ++l) {
      unsigned q[2];
      for (int h = 0; h < 2; ++h) {
        const int g = 2 * p + h;
        const float step = df * float(sc[g]), off = dmf * float(mi[g]);
        q[h] = step > 0.f ? (unsigned)fminf(fmaxf(nearest((x[g * 32 + l] + off) / step), 0.f), 15.f) : 0u;
      }
      out[16 + p * 32 + l] = uint8_t(q[0] | (q[1] << 4));
    }
}

// ---- GGUF Q6_K (native 210-byte blocks) ---------------------------------------------------------
__global__ void q6k_quant_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst, long long blocks) {
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= blocks) return;
  const float* x = src + b * 256;
  float sub[16], m = 0.f;
  for (int s = 0; s < 16; ++s) {
    float a = 0.f;
    for (int i = 0; i < 16; ++i) a = fmaxf(a, fabsf(x[s * 16 + i]));
    sub[s] = a / 31.f;
    m = fmaxf(m, sub[s]);
  }
  const __half d = __float2half_rn(m / 127.f);
  const float df = __half2float(d);
  uint8_t* out = dst + b * 210;
  int sc[16];
  for (int s = 0; s < 16; ++s) {
    sc[s] = df > 0.f ? (int)fminf(fmaxf(nearest(sub[s] / df), 0.f), 127.f) : 0;
    out[192 + s] = uint8_t(int8_t(sc[s]));
  }
  *reinterpret_cast<__half*>(out + 208) = d;
  for (int n = 0; n < 2; ++n)
    for (int l = 0; l < 32; ++l) {
      unsigned q[4];
      for (int g = 0; g < 4; ++g) {
        const int j = n * 128 + g * 32 + l;
        const float step = df * float(sc[j / 16]);
        q[g] = step > 0.f ? (unsigned)(fminf(fmaxf(nearest(x[j] / step), -32.f), 31.f) + 32.f) : 32u;
      }
      out[n * 64 + l] = uint8_t((q[0] & 15) | ((q[2] & 15) << 4));
      out[n * 64 + 32 + l] = uint8_t((q[1] & 15) | ((q[3] & 15) << 4));
      out[128 + n * 32 + l] = uint8_t((q[0] >> 4) | ((q[1] >> 4) << 2) | ((q[2] >> 4) << 4) | ((q[3] >> 4) << 6));
    }
}

// ---- NVFP4 ---------------------------------------------------------------------------------------
// Largest magnitude of matrix blockIdx.y, kept as the bit pattern of a non-negative float so that one integer
// atomicMax per thread block combines the blocks (float32 magnitudes and their bit patterns sort alike).
__global__ void __launch_bounds__(256) amax_kernel(const float* __restrict__ src, long long n, long long stride, unsigned* amax, int as_bf16) {
  __shared__ float warp_top[8];
  const float* w = src + blockIdx.y * stride;
  float top = 0.f;
  const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x, step = (long long)gridDim.x * blockDim.x;
  for (long long i = first; i < n; i += step) {
    const float v = as_bf16 ? bf16r(w[i]) : w[i];
    top = fmaxf(top, fabsf(v));
  }
  top = warp_max(top);
  if ((threadIdx.x & 31) == 0) warp_top[threadIdx.x >> 5] = top;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int q = 1; q < int(blockDim.x >> 5); ++q) top = fmaxf(top, warp_top[q]);
    atomicMax(amax + blockIdx.y, __float_as_uint(top));
  }
}

// Tsumuji (ModelOpt) NVFP4 of matrix blockIdx.y, source rounded to bf16 first (the reference quantizes bf16
// checkpoints: tsumuji kernels/decode/quant.cu:77-114). Half a warp owns one 16-element block: lane i of the half holds
// element i, the block maximum travels by shuffles, every lane encodes its own element and the even lanes pair their
// code with the neighbour's into one byte. A warp reads 32 consecutive floats per round.
//   matrix scale g = amax / (6 * 448) (1 for an all-zero matrix); block scale byte = e4m3(max / 6 / g);
//   code = e2m1(element / (e4m3 value * g)) with the sign in bit 3; element 2i in the low nibble of byte i.
__global__ void __launch_bounds__(256) nvfp4_linear_quant_kernel(const float* __restrict__ src, long long src_stride, int rows, int cols,
                                                                 const unsigned* __restrict__ amax, uint8_t* __restrict__ dst,
                                                                 long long dst_stride, long long codes_off, long long scales_off,
                                                                 float* __restrict__ gs, int gs_stride) {
  const int m = blockIdx.y, lane = threadIdx.x & 31, sub = lane & 15;
  float matrix_scale = __uint_as_float(amax[m]) / (6.f * 448.f);
  if (matrix_scale == 0.f) matrix_scale = 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0) gs[m * gs_stride] = matrix_scale;
  const long long blocks = (long long)rows * cols / 16;
  const float* x = src + m * src_stride;
  uint8_t* out = dst + m * dst_stride;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); pair * 2 < blocks; pair += warps) {
    const long long b = pair * 2 + (lane >> 4);                     // this half warp's block
    const bool live = b < blocks;
    const float v = live ? bf16r(x[b * 16 + sub]) : 0.f;
    float top = fabsf(v);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    const uint8_t scale_byte = e4m3_rn(top / 6.f / matrix_scale);
    const float unit = e4m3_value(scale_byte) * matrix_scale;
    const float q = unit > 0.f ? v / unit : 0.f;
    const unsigned code = e2m1_code(fabsf(q)) | (signbit(q) ? 8u : 0u);
    const unsigned neighbour = __shfl_down_sync(0xffffffffu, code, 1);
    if (live && sub == 0) out[scales_off + b] = scale_byte;
    if (live && (sub & 1) == 0) out[codes_off + b * 8 + (sub >> 1)] = uint8_t(code | (neighbour << 4));
  }
}

// Hayate image of one [n, k] matrix: codes | 128x4-tiled e4m3 scales | float32 matrix scale.
__global__ void nvfp4_tiled_quant_kernel(const float* __restrict__ src, int n, int k, const unsigned* __restrict__ amax,
                                         uint8_t* __restrict__ dst) {
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const float maximum = __uint_as_float(amax[0]);
  const float tiny = 1.401298464324817e-45f;       // float32 tiny * eps
  const float ms = maximum == 0.f ? 1.f : fmaxf(maximum / (6.f * 448.f), tiny);
  const int cols = (k / 16 + 3) / 4 * 4;
  uint8_t* scales = dst + (size_t)n * k / 2;
  if (b == 0) *reinterpret_cast<float*>(scales + (size_t)((n + 127) / 128 * 128) * cols) = ms;
  if (b >= (long long)n * k / 16) return;
  const int r = int(b / (k / 16)), sc = int(b % (k / 16));
  const float* x = src + b * 16;
  float a = 0.f;
  for (int i = 0; i < 16; ++i) a = fmaxf(a, fabsf(x[i]));
  const uint8_t s = e4m3_rn(fminf(fmaxf(a / ms / 6.f, 0.f), 448.f));
  float dec = e4m3_value(s);
  if (dec == 0.f) dec = 1.f;
  scales[(size_t)((r / 128) * (cols / 4) + sc / 4) * 512 + (r % 32) * 16 + (r % 128 / 32) * 4 + sc % 4] = s;
  for (int i = 0; i < 8; ++i) {
    const float q0 = fabsf(x[2 * i] / ms / dec), q1 = fabsf(x[2 * i + 1] / ms / dec);
    const unsigned c0 = e2m1_code(q0) | (signbit(x[2 * i]) ? 8u : 0u), c1 = e2m1_code(q1) | (signbit(x[2 * i + 1]) ? 8u : 0u);
    dst[b * 8 + i] = uint8_t(c0 | (c1 << 4));
  }
}

// ---- FP8 ---------------------------------------------------------------------------------------
// Block FP8 weights: one CTA per 128x128 block; scale = absmax / 448 (1 for a zero block).
__global__ void __launch_bounds__(256) fp8_block_quant_kernel(const float* __restrict__ src, int n, int k,
                                                              uint8_t* __restrict__ payload, float* __restrict__ scales) {
  __shared__ float red[8];
  const int kb = blockIdx.x, nb = blockIdx.y, kbs = (k + 127) / 128;
  float a = 0.f;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = nb * 128 + i / 128, c = kb * 128 + i % 128;
    if (r < n && c < k) a = fmaxf(a, fabsf(src[(size_t)r * k + c]));
  }
  a = warp_max(a);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
  __syncthreads();
  a = red[0];
  for (int i = 1; i < 8; ++i) a = fmaxf(a, red[i]);
  const float scale = a == 0.f ? 1.f : a / 448.f;
  if (threadIdx.x == 0) scales[nb * kbs + kb] = scale;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = nb * 128 + i / 128, c = kb * 128 + i % 128;
    if (r < n && c < k) payload[(size_t)r * k + c] = e4m3_rn(fminf(fmaxf(src[(size_t)r * k + c] / scale, -448.f), 448.f));
  }
}

// Activations: one warp per (row, 128-channel group): e4m3 codes + float32 scale = absmax / 448 (1 for zeros);
// code = e4m3(x * (1 / scale)) with the reciprocal rounded to float32 once per group.
template <typename T>
__global__ void __launch_bounds__(256) fp8_act_quant_kernel(const T* __restrict__ x, long long rows, int k,
                                                            uint8_t* __restrict__ q, float* __restrict__ scales) {
  pdl_wait();
  pdl_launch();
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31, groups = k / 128;
  if (w >= rows * groups) return;
  const long long r = w / groups;
  const int g = int(w % groups);
  const T* p = x + r * k + g * 128 + lane * 4;
  float v[4], a = 0.f;
  for (int i = 0; i < 4; ++i) {
    v[i] = float(p[i]);
    a = fmaxf(a, fabsf(v[i]));
  }
  a = warp_max(a);
  const float scale = a == 0.f ? 1.f : a / 448.f;
  if (lane == 0) scales[r * groups + g] = scale;
  uint32_t out = 0;
  const float inv = 1.f / scale;      // codes = e4m3(x * (1 / scale)): one division per group
  for (int i = 0; i < 4; ++i) out |= uint32_t(e4m3_rn(fminf(fmaxf(v[i] * inv, -448.f), 448.f))) << (8 * i);
  *reinterpret_cast<uint32_t*>(q + r * k + g * 128 + lane * 4) = out;
}

}  // namespace dmoe

using namespace dmoe;

extern "C" int darask_quantize_ggml(void* dst, const float* src, int ty, long long elements, cudaStream_t st) {
  if (!dst || !src || elements <= 0 || elements % 256) return cudaErrorInvalidValue;
  const long long blocks = elements / 256;
  const unsigned grid = unsigned((blocks + 127) / 128);
  if (ty == DARASK_GGML_Q4_K) q4k_quant_kernel<<<grid, 128, 0, st>>>(src, static_cast<uint8_t*>(dst), blocks);
  else if (ty == DARASK_GGML_Q6_K) q6k_quant_kernel<<<grid, 128, 0, st>>>(src, static_cast<uint8_t*>(dst), blocks);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

extern "C" int darask_quantize_nvfp4_linear(void* dst, long long dst_stride, long long codes_off, long long scales_off,
                                            float* gs, int gs_stride, const float* src, long long src_stride,
                                            int matrices, int rows, int cols, unsigned* amax_scratch, cudaStream_t st) {
  if (!dst || !gs || !src || !amax_scratch || matrices < 1 || rows < 1 || cols < 16 || cols % 16) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(amax_scratch, 0, size_t(matrices) * 4, st);
  if (e) return e;
  const long long n = (long long)rows * cols;
  amax_kernel<<<dim3(unsigned(n / 4096 > 1024 ? 1024 : (n + 4095) / 4096), matrices), 256, 0, st>>>(src, n, src_stride, amax_scratch, 1);
  const long long warp_rounds = (n / 32 + 7) / 8;                  // thread blocks if every warp took one round
  nvfp4_linear_quant_kernel<<<dim3(unsigned(warp_rounds > 8192 ? 8192 : (warp_rounds < 1 ? 1 : warp_rounds)), matrices), 256, 0, st>>>(
      src, src_stride, rows, cols, amax_scratch, static_cast<uint8_t*>(dst), dst_stride, codes_off, scales_off, gs, gs_stride);
  return cudaGetLastError();
}

extern "C" int darask_quantize_nvfp4_tiled(void* dst, const float* src, int rows, int cols, unsigned* amax_scratch,
                                           cudaStream_t st) {
  if (!dst || !src || !amax_scratch || rows < 1 || cols < 16 || cols % 16) return cudaErrorInvalidValue;
  const long long n = (long long)rows * cols;
  const size_t bytes = size_t(n) / 2 + size_t((rows + 127) / 128 * 128) * ((cols / 16 + 3) / 4 * 4) + 4;
  cudaError_t e = cudaMemsetAsync(amax_scratch, 0, 4, st);
  if (!e) e = cudaMemsetAsync(dst, 0, bytes, st);     // scale-tile padding is zero
  if (e) return e;
  amax_kernel<<<dim3(unsigned(n / 4096 > 1024 ? 1024 : (n + 4095) / 4096), 1), 256, 0, st>>>(src, n, 0, amax_scratch, 0);
  nvfp4_tiled_quant_kernel<<<unsigned((n / 16 + 255) / 256), 256, 0, st>>>(src, rows, cols, amax_scratch, static_cast<uint8_t*>(dst));
  return cudaGetLastError();
}

extern "C" int darask_quantize_fp8_block(void* payload, float* scales, const float* src, int rows, int cols, cudaStream_t st) {
  if (!payload || !scales || !src || rows < 1 || cols < 1) return cudaErrorInvalidValue;
  fp8_block_quant_kernel<<<dim3((cols + 127) / 128, (rows + 127) / 128), 256, 0, st>>>(src, rows, cols, static_cast<uint8_t*>(payload), scales);
  return cudaGetLastError();
}

extern "C" int darask_quantize_fp8_act(void* codes, float* scales, const void* x, int x_is_bf16, long long rows, int cols,
                                       cudaStream_t st) {
  if (!codes || !scales || !x || rows < 1 || cols < 128 || cols % 128) return cudaErrorInvalidValue;
  const long long warps = rows * (cols / 128);
  const unsigned grid = unsigned((warps + 7) / 8);
  if (x_is_bf16) fp8_act_quant_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, cols, static_cast<uint8_t*>(codes), scales);
  else fp8_act_quant_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), rows, cols, static_cast<uint8_t*>(codes), scales);
  return cudaGetLastError();
}
