// Dense bf16 expert matrices (the shared expert of the Tsumuji executor, tsumuji kernels/decode/gemv.cu:
// `dense_dot_part<0>`): the same fp16 tensor-core tiles as expert_gemv.cuh, weight rows loaded straight
// from global memory (16 bytes per lane, eight rows of 64 contiguous bytes per warp instruction).
// bf16 -> fp16 is exact for |w| >= 2^-14 (bf16 keeps 8 significant bits); smaller weights lose at most 2^-25.
#pragma once
#include "expert_gemv.cuh"

namespace dmoe {

struct DenseArgs {
  const __nv_bfloat16* w[2];   // matrix 0 (gate or down) and matrix 1 (up), row-major [rows][k]
  int k, rows, ks;             // ks: warps that split K for one row slab
  const __half* xplanes;       // activation planes, natural order; row of token t = x_row0 + t
  int x_row0, tokens;
  __half* out_planes;          // DUAL: silu(g) * u planes, row out_row0 + t
  float* out;                  // else float rows
  int out_row0;
};

DEVI uint32_t bf16x2_to_f16x2(uint32_t v) {
  const float lo = __uint_as_float(v << 16), hi = __uint_as_float(v & 0xffff0000u);
  return h2_as_u32(__floats2half2_rn(lo, hi));
}

template <int DUAL>
__global__ void __launch_bounds__(kGemvWarps * 32, 1) dense_gemv_kernel(const DenseArgs a) {
  __shared__ float red[kGemvWarps * 4 * 16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g4 = lane >> 2, j = lane & 3;
  pdl_wait();
  pdl_launch();
  constexpr int RPT = DUAL ? 8 : 16;
  const int slabs = (a.rows + RPT - 1) / RPT;
  const int kper = a.k / a.ks;                        // columns per warp (multiple of 32)
  const long long items = (long long)slabs * a.ks;
  for (long long item = (long long)blockIdx.x * kGemvWarps + warp; item < items; item += (long long)gridDim.x * kGemvWarps) {
    const int slab = int(item / a.ks), kpart = int(item % a.ks);
    // MMA rows g4 / g4 + 8: DUAL -> gate row and the up row of the same index, else two rows 8 apart
    const int r0 = slab * RPT + g4, r1 = DUAL ? r0 : r0 + 8;
    const __nv_bfloat16* p0 = a.w[0] + size_t(min(r0, a.rows - 1)) * a.k + kpart * kper + 8 * j;
    const __nv_bfloat16* p1 = (DUAL ? a.w[1] : a.w[0]) + size_t(min(r1, a.rows - 1)) * a.k + kpart * kper + 8 * j;
    for (int c0 = 0; c0 < a.tokens; c0 += 4) {
      const int tcol = c0 + (g4 >> 1);
      const __half* plane = tcol < a.tokens ? a.xplanes + (size_t(a.x_row0 + tcol) * 2 + (g4 & 1)) * a.k + kpart * kper + 8 * j : nullptr;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int col = 0; col < kper; col += 32) {
        const uint4 w0 = __ldg(reinterpret_cast<const uint4*>(p0 + col)), w1 = __ldg(reinterpret_cast<const uint4*>(p1 + col));
        uint4 x = make_uint4(0, 0, 0, 0);
        if (plane) x = __ldg(reinterpret_cast<const uint4*>(plane + col));
        mma_f16(c, bf16x2_to_f16x2(w0.x), bf16x2_to_f16x2(w1.x), bf16x2_to_f16x2(w0.y), bf16x2_to_f16x2(w1.y), x.x, x.y);
        mma_f16(c, bf16x2_to_f16x2(w0.z), bf16x2_to_f16x2(w1.z), bf16x2_to_f16x2(w0.w), bf16x2_to_f16x2(w1.w), x.z, x.w);
      }
      float f0 = c[0] + c[1], f1 = c[2] + c[3];
      if (a.ks > 1) {
        const int bar = 1 + warp / a.ks;
        red[(warp * 4 + j) * 16 + g4] = f0;
        red[(warp * 4 + j) * 16 + 8 + g4] = f1;
        named_barrier(bar, a.ks * 32);
        if (kpart == 0) {
          f0 = f1 = 0.f;
          for (int q = 0; q < a.ks; ++q) {
            f0 += red[((warp + q) * 4 + j) * 16 + g4];
            f1 += red[((warp + q) * 4 + j) * 16 + 8 + g4];
          }
        }
        named_barrier(bar, a.ks * 32);
      }
      const int t = c0 + j;
      if (kpart == 0 && t < a.tokens) {
        const size_t orow = size_t(a.out_row0 + t);
        if (DUAL) {
          if (r0 < a.rows) {
            const float h = silu_mul(f0, f1);
            const __half hi = __float2half_rn(h), lo = __float2half_rn(h - __half2float(hi));
            a.out_planes[orow * 2 * a.rows + r0] = hi;
            a.out_planes[orow * 2 * a.rows + a.rows + r0] = lo;
          }
        } else {
          if (r0 < a.rows) a.out[orow * a.rows + r0] = f0;
          if (r1 < a.rows) a.out[orow * a.rows + r1] = f1;
        }
      }
    }
  }
}

}  // namespace dmoe
