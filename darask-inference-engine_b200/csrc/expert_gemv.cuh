// Decode-path expert products for small token counts (GGUF Q4_K / Q6_K and NVFP4 weights).
//
// Every warp is independent: it owns an 8- or 16-row slab of one expert and a contiguous share of
// the 256-element blocks of K, streams that share HBM -> its private shared-memory ring with
// 16-byte cp.async copies (2-3 blocks in flight per warp, ~100 KB per SM), and multiplies on
// fp16 tensor-core tiles (mma.sync m16n8k16, fp32 accumulate):
//   * A operand = the weight codes as exact fp16 values (Q4_K: q * sc <= 945; Q6_K: q - 32; NVFP4:
//     e2m1 * e4m3, at most six significant bits), built from the packed bytes without int->float
//     conversions;
//   * B operand = the activations split as x = hi + lo (two fp16, error <= 2^-22 |x|), one column
//     pair per token, so one tile serves up to four tokens of the same expert;
//   * fp16 x fp16 products are exact in fp32, the f16/f32 scales are applied to the tile sums.
// The warps that share a row slab (K split) add their partial sums through shared memory in a
// fixed order. No CTA-wide barrier exists after the prologue.
// Activation rows are read as "planes": per row k fp16 hi values then k fp16 lo values; for the GGUF
// formats each aligned group of four is stored as [x0, x2, x1, x3] (the order their tile fragments
// want), for NVFP4 in natural order.
// Replaces kogarashi kernels/native.cu:46-88 (`gemv`) and :97-99 (`activate`), tsumuji kernels/decode/
// gemv.cu:64-158 (`moe_gate_up`, `moe_down`) and hayate cu/glm53/decode.cu:37-54 (`gate_up`, `down`).
#pragma once
#include "common.cuh"
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <type_traits>

namespace dmoe {

enum GemvFormat { kGemvQ4K = 0, kGemvQ6KR = 1, kGemvNvfp4Linear = 2, kGemvNvfp4Tiled = 3, kGemvFp8Block = 4 };
// what the epilogue writes
enum GemvOut {
  kOutSiluPlanes = 0,    // DUAL: silu(g) * u as fp16 hi/lo planes (Kogarashi, Tsumuji)
  kOutFloat = 1,         // rows as float32
  kOutHayateProduct = 2, // DUAL: Hayate SwiGLU (clamps, bf16 roundings) as bf16 rows and as planes
  kOutBf16 = 3           // rows rounded to bf16
};

struct GemvArgs {
  const uint8_t* w[2];          // routed experts: matrix 0 (gate or down) and matrix 1 (up)
  const uint8_t* w_shared[2];   // shared expert matrices (null when there is none)
  unsigned long long expert_stride[2];   // bytes between consecutive experts
  int row_bytes;                // bytes of one row (of codes, for NVFP4) in global memory (multiple of 16)
  const void* const* w_table;   // optional: per group the base pointer of its expert image (replaces w[0] + e * stride)
  unsigned long long matrix_stride;      // w_table / Hayate images: bytes between gate | up | down inside an image
  unsigned long long scale_offset[2];    // NVFP4 / block-FP8: byte offset of the scale area from the matrix base (per matrix)
  const float* scale_shared[2];          // block-FP8: the shared expert's scale arrays when they are not behind its payload (null: scale_offset)
  const uint8_t* gscale;        // per-matrix float32 multiplier: gscale + e * gscale_estride + m * gscale_mstride (null: 1)
  unsigned long long gscale_estride, gscale_mstride;
  const uint8_t* gscale_shared[2];       // the same for the shared expert (null: 1)
  unsigned long long gscale_in_matrix[2]; // non-zero: the multiplier is the float32 at this byte offset of the matrix itself
  int k, rows, nblk;            // columns, rows per matrix, k / 256
  int ks;                       // warps that split K for one row slab (divides nblk and the warps per CTA)
  // derived on the host from ks and the grid (launch_gemv): blocks per item, 65536 / ks + 1, slab groups per CTA, and
  // the slabs all CTAs advance per round as (whole groups, remainder)
  int nb_per, ks_inv, slab_groups;
  unsigned group_step, slab_step;
  const __half* xplanes;        // [x rows][2][k] activation planes
  const __half* xsum_planes;    // [x rows][2][k/32] sums of x over 32 columns as fp16 hi / lo planes (Q4_K mins); null: use tiles
  int x_by_assignment;          // 0: x row = token; 1: x row = assignment index
  const int* counters;          // [0] = number of groups (active experts, plus the shared expert)
  const int4* plan;             // per group {expert (-1: shared), rows, offset into assignments, 0}
  const unsigned* assignments;  // [T*k]
  int tokens, topk, max_groups;
  __half* out_planes;           // DUAL: SwiGLU products as planes [T*k (+T)][2][rows]
  float* out;                   // kOutFloat: [T*k (+T)][rows]
  __nv_bfloat16* out_bf16;      // kOutHayateProduct / kOutBf16: [T*k (+T)][rows]
  int out_shared_row;           // output row of the shared expert's token t is out_shared_row + t (default T*k)
  int shared_x_row0;            // x row of the shared expert's token t when rows are per token (default 0: the token's own row)
  int round_shared;             // NVFP4: the shared expert's weights are rounded to bf16 after scaling (Hayate)
  unsigned* status;
  // 1: counters / plan / assignments were written by a kernel BEFORE the immediate predecessor in the stream (which
  // itself waited for it), only the activation planes come from the predecessor: the dependency wait is then taken after
  // the first weight requests are in flight instead of at kernel entry.
  int late_wait;
};

#ifndef DMOE_GEMV_WARPS
#define DMOE_GEMV_WARPS 16
#endif
constexpr int kGemvWarps = DMOE_GEMV_WARPS;

DEVI void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
DEVI void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> DEVI void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// volatile + memory clobber: the loads must stay behind the cp.async waits that make the data visible
DEVI uint4 lds128(uint32_t a) { uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory"); return v; }
DEVI uint2 lds64(uint32_t a) { uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a) : "memory"); return v; }
DEVI uint32_t lds32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a) : "memory"); return v; }

// D[16x8] += A[16x16] (f16, row) x B[16x8] (f16, col), fp32 accumulate. Thread (g = lane/4, j = lane%4):
// a0/a1: rows g / g+8, k 2j,2j+1; a2/a3: same rows, k 2j+8,2j+9; b0: column g, k 2j,2j+1; b1: k 2j+8,2j+9;
// c0,c1: row g, columns 2j,2j+1; c2,c3: row g+8.
DEVI void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
DEVI uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
DEVI __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
// storage position of logical column e inside a plane
DEVI int plane_pos(int e) { return (e & ~3) | ((e & 1) << 1) | ((e >> 1) & 1); }

// word i of a 16-byte vector (i is a compile-time constant after unrolling)
DEVI uint32_t u4w(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// The block functions below multiply one staged 256-column block of 16 row slots with up to NT groups of four
// tokens: the weight fragments are built once and feed one tile per token group. `bcol[t]`: this lane's B plane
// of group t (column g = lane/4 -> token g/2 of the group, hi or lo) at the block's first column; a column without
// a token gets the plane of another token, its sums are discarded. `facc[t]`: the sums of rows g / g + 8 for token j = lane % 4 of group t.

// ---- Q4_K -------------------------------------------------------------------------------------------
// Row slot pitch PITCH: header 16 B, nibbles 128 B. value = d*sc*q - dmin*m (kogarashi kernels/native.cu:26-34).
// `xsum[t]`: the per-32 sums of this lane's column (hi or lo plane) at the block, or null.
template <int PITCH, bool MINS_TILE, int NT>
DEVI void q4k_block_f16(uint32_t slab, int lane, const __half* const (&bcol)[NT], const __half* const (&xsum)[NT], float (&facc)[NT][2]) {
  const int g = lane >> 2, j = lane & 3;
  const uint32_t r0 = slab + g * PITCH, r1 = slab + (g + 8) * PITCH;
  const uint4 h0 = lds128(r0), h1 = lds128(r1);
  // six-bit scales / mins of the eight sub-blocks, packed four per word
  const uint32_t sc0[2] = {h0.y & 0x3F3F3F3Fu, (h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u)};
  const uint32_t sc1[2] = {h1.y & 0x3F3F3F3Fu, (h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u)};
  const uint32_t mn0[2] = {h0.z & 0x3F3F3F3Fu, ((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u)};
  const uint32_t mn1[2] = {h1.z & 0x3F3F3F3Fu, ((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u)};
  const __half2 k1024 = __float2half2_rn(1024.f);
  float c[NT][4], cm[NT][4];               // sums over the block of sc * q * x and of m * x (rows g, g+8; columns 2j, 2j+1)
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) c[t][i] = cm[t][i] = 0.f;
#pragma unroll
  for (int gp = 0; gp < 4; ++gp) {
    // byte [sc, 0x64] pairs -> half2(1024 + sc) - 1024 = (sc, sc), exact
    const int sel = (gp & 1) ? 0x4342 : 0x4140;        // bytes 2,3 or 0,1 of the scale word: [lo, 0x64, hi, 0x64]
    const uint32_t w0s = sc0[gp >> 1], w1s = sc1[gp >> 1];
    const __half2 p0 = __hsub2(u32_as_h2(__byte_perm(w0s, 0x64646464u, sel)), k1024);   // (sc[2gp], sc[2gp+1]) row g
    const __half2 p1 = __hsub2(u32_as_h2(__byte_perm(w1s, 0x64646464u, sel)), k1024);   // row g+8
    const __half2 sl0 = __low2half2(p0), sh0 = __high2half2(p0), sl1 = __low2half2(p1), sh1 = __high2half2(p1);
    // low nibbles: (1024 + q) * sc - 1024 * sc; high nibbles: (1024 + 16 q) * sc/16 - 64 * sc
    const __half2 bl0 = __hmul2(sl0, __float2half2_rn(-1024.f)), bl1 = __hmul2(sl1, __float2half2_rn(-1024.f));
    const __half2 mh0 = __hmul2(sh0, __float2half2_rn(0.0625f)), mh1 = __hmul2(sh1, __float2half2_rn(0.0625f));
    const __half2 bh0 = __hmul2(sh0, __float2half2_rn(-64.f)), bh1 = __hmul2(sh1, __float2half2_rn(-64.f));
    const uint2 w0 = lds64(r0 + 16 + gp * 32 + 8 * j), w1 = lds64(r1 + 16 + gp * 32 + 8 * j);
    uint4 blo[NT], bhi[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      blo[t] = __ldg(reinterpret_cast<const uint4*>(bcol[t] + gp * 64 + 8 * j));
      bhi[t] = __ldg(reinterpret_cast<const uint4*>(bcol[t] + gp * 64 + 32 + 8 * j));
    }
    const uint32_t words0[2] = {w0.x, w0.y}, words1[2] = {w1.x, w1.y};
#pragma unroll
    for (int s = 0; s < 2; ++s) {          // the two 16-column slabs of a 32-column sub-block
      const uint32_t a = words0[s], b = words1[s];
      // low nibbles -> sub-block 2gp
      uint32_t a0 = h2_as_u32(__hfma2(u32_as_h2((a & 0x000F000Fu) | 0x64006400u), sl0, bl0));
      uint32_t a2 = h2_as_u32(__hfma2(u32_as_h2(((a >> 8) & 0x000F000Fu) | 0x64006400u), sl0, bl0));
      uint32_t a1 = h2_as_u32(__hfma2(u32_as_h2((b & 0x000F000Fu) | 0x64006400u), sl1, bl1));
      uint32_t a3 = h2_as_u32(__hfma2(u32_as_h2(((b >> 8) & 0x000F000Fu) | 0x64006400u), sl1, bl1));
#pragma unroll
      for (int t = 0; t < NT; ++t) mma_f16(c[t], a0, a1, a2, a3, u4w(blo[t], 2 * s), u4w(blo[t], 2 * s + 1));
      // high nibbles -> sub-block 2gp + 1
      a0 = h2_as_u32(__hfma2(u32_as_h2((a & 0x00F000F0u) | 0x64006400u), mh0, bh0));
      a2 = h2_as_u32(__hfma2(u32_as_h2(((a >> 8) & 0x00F000F0u) | 0x64006400u), mh0, bh0));
      a1 = h2_as_u32(__hfma2(u32_as_h2((b & 0x00F000F0u) | 0x64006400u), mh1, bh1));
      a3 = h2_as_u32(__hfma2(u32_as_h2(((b >> 8) & 0x00F000F0u) | 0x64006400u), mh1, bh1));
#pragma unroll
      for (int t = 0; t < NT; ++t) mma_f16(c[t], a0, a1, a2, a3, u4w(bhi[t], 2 * s), u4w(bhi[t], 2 * s + 1));
      if (MINS_TILE) {
        // the min of a sub-block as a constant row of the A operand: the tile sums m * x over the slab
        const int msel = (gp & 1) ? 0x4342 : 0x4140;
        const __half2 q0 = __hsub2(u32_as_h2(__byte_perm(mn0[gp >> 1], 0x64646464u, msel)), k1024);
        const __half2 q1 = __hsub2(u32_as_h2(__byte_perm(mn1[gp >> 1], 0x64646464u, msel)), k1024);
        const uint32_t ml0 = h2_as_u32(__low2half2(q0)), mh0u = h2_as_u32(__high2half2(q0));
        const uint32_t ml1 = h2_as_u32(__low2half2(q1)), mh1u = h2_as_u32(__high2half2(q1));
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          mma_f16(cm[t], ml0, ml1, ml0, ml1, u4w(blo[t], 2 * s), u4w(blo[t], 2 * s + 1));
          mma_f16(cm[t], mh0u, mh1u, mh0u, mh1u, u4w(bhi[t], 2 * s), u4w(bhi[t], 2 * s + 1));
        }
      }
    }
  }
  const float d0 = half_lo(h0.x), dm0 = half_hi(h0.x), d1 = half_lo(h1.x), dm1 = half_hi(h1.x);
  if (!MINS_TILE) {
    // one tile for the mins of the whole block: A = the eight mins of rows g / g + 8 in k slots 0-7 (this lane: slots
    // 2j, 2j + 1), B = the eight per-32 sums of this lane's column
    const __half2 q0 = __hsub2(u32_as_h2(__byte_perm((j & 2) ? mn0[1] : mn0[0], 0x64646464u, (j & 1) ? 0x4342 : 0x4140)), k1024);
    const __half2 q1 = __hsub2(u32_as_h2(__byte_perm((j & 2) ? mn1[1] : mn1[0], 0x64646464u, (j & 1) ? 0x4342 : 0x4140)), k1024);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      uint32_t xs2 = 0;
      if (xsum[t]) xs2 = __ldg(reinterpret_cast<const uint32_t*>(xsum[t]) + j);
      mma_f16(cm[t], h2_as_u32(q0), h2_as_u32(q1), 0u, 0u, xs2, 0u);
    }
  }
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    facc[t][0] += d0 * (c[t][0] + c[t][1]) - dm0 * (cm[t][0] + cm[t][1]);
    facc[t][1] += d1 * (c[t][2] + c[t][3]) - dm1 * (cm[t][2] + cm[t][3]);
  }
}

// ---- Q6_K (row-aligned device layout: per block ql 128 | qh 64 | int8 scales 16; d in a trailing chunk) --
// value = d * scale * (q - 32) (kogarashi kernels/native.cu:35-40). Row slot: 208 data bytes, then the 16-byte
// chunk of the row tail that holds this block's f16 d at byte `doff`.
template <int PITCH, int NT>
DEVI void q6k_block_f16(uint32_t slab, int lane, int doff, const __half* const (&bcol)[NT], float (&facc)[NT][2]) {
  const int g = lane >> 2, j = lane & 3;
  const uint32_t r0 = slab + g * PITCH, r1 = slab + (g + 8) * PITCH;
  const uint4 s0v = lds128(r0 + 192), s1v = lds128(r1 + 192);
  const uint32_t sw0[4] = {s0v.x ^ 0x80808080u, s0v.y ^ 0x80808080u, s0v.z ^ 0x80808080u, s0v.w ^ 0x80808080u};
  const uint32_t sw1[4] = {s1v.x ^ 0x80808080u, s1v.y ^ 0x80808080u, s1v.z ^ 0x80808080u, s1v.w ^ 0x80808080u};
  const uint32_t dw0 = lds32(r0 + 208 + (doff & ~3)), dw1 = lds32(r1 + 208 + (doff & ~3));
  const float d0 = (doff & 2) ? half_hi(dw0) : half_lo(dw0), d1 = (doff & 2) ? half_hi(dw1) : half_lo(dw1);
  const __half2 k1056 = __float2half2_rn(1056.f);      // 1024 (magic) + 32 (code offset)
  float a0[NT], a1[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) a0[t] = a1[t] = 0.f;
#pragma unroll
  for (int n = 0; n < 2; ++n) {
#pragma unroll
    for (int lh = 0; lh < 2; ++lh) {
      const uint32_t q0h = lds32(r0 + 128 + n * 32 + lh * 16 + 4 * j), q1h = lds32(r1 + 128 + n * 32 + lh * 16 + 4 * j);
#pragma unroll
      for (int gb = 0; gb < 2; ++gb) {
        const uint32_t w0 = lds32(r0 + n * 64 + gb * 32 + lh * 16 + 4 * j), w1 = lds32(r1 + n * 64 + gb * 32 + lh * 16 + 4 * j);
        const int col = n * 128 + gb * 32 + lh * 16 + 4 * j;       // columns of the low-nibble group; +64: high nibbles
        uint2 blo[NT], bhi[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          blo[t] = __ldg(reinterpret_cast<const uint2*>(bcol[t] + col));
          bhi[t] = __ldg(reinterpret_cast<const uint2*>(bcol[t] + col + 64));
        }
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
          const uint32_t c0 = hi ? (((w0 >> 4) & 0x0F0F0F0Fu) | ((q0h >> (2 * gb)) & 0x30303030u))
                                 : ((w0 & 0x0F0F0F0Fu) | ((q0h << (4 - 2 * gb)) & 0x30303030u));
          const uint32_t c1 = hi ? (((w1 >> 4) & 0x0F0F0F0Fu) | ((q1h >> (2 * gb)) & 0x30303030u))
                                 : ((w1 & 0x0F0F0F0Fu) | ((q1h << (4 - 2 * gb)) & 0x30303030u));
          // bytes [b0, 0x64, b2, 0x64] = half2(1024 + b0, 1024 + b2); minus 1056 -> q - 32, exact
          const uint32_t f0 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(c0, 0x64646464u, 0x4240)), k1056));
          const uint32_t f2 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(c0, 0x64646464u, 0x4341)), k1056));
          const uint32_t f1 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(c1, 0x64646464u, 0x4240)), k1056));
          const uint32_t f3 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(c1, 0x64646464u, 0x4341)), k1056));
          const int si = 8 * n + 2 * (gb + 2 * hi) + lh;            // scale index of this 16-column group
          const uint32_t wa = sw0[si >> 2], wb = sw1[si >> 2];
          const float fa = ((si & 3) == 0 ? byte_magic<0>(wa) : (si & 3) == 1 ? byte_magic<1>(wa) : (si & 3) == 2 ? byte_magic<2>(wa) : byte_magic<3>(wa)) - (kMagic + 128.f);
          const float fb = ((si & 3) == 0 ? byte_magic<0>(wb) : (si & 3) == 1 ? byte_magic<1>(wb) : (si & 3) == 2 ? byte_magic<2>(wb) : byte_magic<3>(wb)) - (kMagic + 128.f);
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            mma_f16(c, f0, f1, f2, f3, hi ? bhi[t].x : blo[t].x, hi ? bhi[t].y : blo[t].y);
            a0[t] = fmaf(fa, c[0] + c[1], a0[t]);
            a1[t] = fmaf(fb, c[2] + c[3], a1[t]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    facc[t][0] += d0 * a0[t];
    facc[t][1] += d1 * a1[t];
  }
}


// ---- NVFP4 (e2m1 codes, one e4m3 scale per 16 columns) -------------------------------------------------
// Row slot: 128 code bytes of the block (two columns per byte, even column in the low nibble). The scale
// byte of row slot `slot` and 16-column group `c` of the block sits at sbase(slot) + c for the linear
// layout (tsumuji weights.rs:10-12) and inside 16-byte pieces of the 128x4 scale tiles for the tiled one
// (hayate math.cuh:41-49); SCALES tells which.
DEVI uint32_t e4m3x2_to_h2(uint32_t two_bytes) {
  uint32_t out;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(out) : "h"((unsigned short)two_bytes));
  return out;
}
DEVI uint32_t e2m1x2_to_h2(uint32_t byte) {                             // one code byte -> half2(even column, odd column)
  const __half2_raw r = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(byte & 0xffu), __NV_E2M1);
  return uint32_t(r.x) | (uint32_t(r.y) << 16);
}
DEVI void e2m1x4_to_h2(uint32_t w16, uint32_t& lo, uint32_t& hi) {     // two code bytes -> 2 x half2
  lo = e2m1x2_to_h2(w16);
  hi = e2m1x2_to_h2(w16 >> 8);
}
// Address of the 16 scale bytes region helpers. Linear: the slot carries its 16 scale bytes behind the codes.
// Tiled: the stage carries, behind the 16 row slots, pieces[piece][16] where a piece holds the four bytes
// (scale columns 4tc..4tc+3) of the four rows p, p+32, p+64, p+96 of a 128-row tile.
template <int FMT, int DUAL, int PITCH>
DEVI uint32_t nvfp4_scale_addr(uint32_t slab, int slot, int c) {
  if (FMT == kGemvNvfp4Linear) return slab + slot * PITCH + 128 + c;
  // tiled: slot -> (matrix m, local base row pl, quarter q)
  const int s8 = DUAL ? (slot & 7) : slot;
  const int m = DUAL ? (slot >> 3) : 0;
  const int pl = DUAL ? (s8 & 1) : (s8 & 3), q = DUAL ? (s8 >> 1) : (s8 >> 2);
  const int piece = (DUAL ? (m * 2 + pl) : pl) * 4 + (c >> 2);
  return slab + 16 * PITCH + piece * 16 + q * 4 + (c & 3);
}
// weight pair (code * scale, exact) -> fp16 of bf16(code * scale * global) * 2^s, with `rm` = global * 2^s: the
// bf16-rounded weights of the reference's FP8 / shared-expert path (hayate cu/glm53/dense.cuh:61-73), kept inside
// the fp16 range by the power of two (rounding to bf16 commutes with it).
DEVI uint32_t round_bf16_pair(uint32_t v, float rm) {
  const float2 f = __half22float2(u32_as_h2(v));
  const float2 r = __bfloat1622float2(__floats2bfloat162_rn(f.x * rm, f.y * rm));
  return h2_as_u32(__floats2half2_rn(r.x, r.y));
}
template <int FMT, int DUAL, int PITCH, bool ROUNDED, int NT>
DEVI void nvfp4_block_f16(uint32_t slab, int lane, const __half* const (&bcol)[NT], float rm0, float rm1, float (&facc)[NT][2]) {
  const int g = lane >> 2, j = lane & 3;
  const uint32_t r0 = slab + g * PITCH, r1 = slab + (g + 8) * PITCH;
  // the 16 scale bytes of rows g / g + 8 for this block, four per word (word tc = scale columns 4tc .. 4tc + 3)
  uint32_t sw0[4], sw1[4];
  if (FMT == kGemvNvfp4Linear) {
    const uint4 v0 = lds128(r0 + 128), v1 = lds128(r1 + 128);
    sw0[0] = v0.x; sw0[1] = v0.y; sw0[2] = v0.z; sw0[3] = v0.w;
    sw1[0] = v1.x; sw1[1] = v1.y; sw1[2] = v1.z; sw1[3] = v1.w;
  } else {
#pragma unroll
    for (int tc = 0; tc < 4; ++tc) {
      sw0[tc] = lds32(nvfp4_scale_addr<FMT, DUAL, PITCH>(slab, g, 4 * tc));
      sw1[tc] = lds32(nvfp4_scale_addr<FMT, DUAL, PITCH>(slab, g + 8, 4 * tc));
    }
  }
  // step q uses scale column 2q + j/2: byte 2(q & 1) + j/2 of word q/2, duplicated into the low half word
  const uint32_t sel_even = (j >> 1) * 0x11u, sel_odd = sel_even + 0x22u;
  float c[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) c[t][i] = 0.f;
#pragma unroll
  for (int q = 0; q < 8; ++q) {                      // 32 columns per step: this lane owns columns 8j..8j+7 of them
    const uint32_t w0 = lds32(r0 + q * 16 + 4 * j), w1 = lds32(r1 + q * 16 + 4 * j);
    const __half2 s0 = u32_as_h2(e4m3x2_to_h2(__byte_perm(sw0[q >> 1], 0u, (q & 1) ? sel_odd : sel_even)));
    const __half2 s1 = u32_as_h2(e4m3x2_to_h2(__byte_perm(sw1[q >> 1], 0u, (q & 1) ? sel_odd : sel_even)));
    uint32_t a01, a23, a45, a67, b01, b23, b45, b67;
    e2m1x4_to_h2(w0 & 0xffffu, a01, a23);
    e2m1x4_to_h2(w0 >> 16, a45, a67);
    e2m1x4_to_h2(w1 & 0xffffu, b01, b23);
    e2m1x4_to_h2(w1 >> 16, b45, b67);
    uint4 x[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) x[t] = __ldg(reinterpret_cast<const uint4*>(bcol[t] + q * 32 + 8 * j));
    a01 = h2_as_u32(__hmul2(u32_as_h2(a01), s0)); a23 = h2_as_u32(__hmul2(u32_as_h2(a23), s0));
    a45 = h2_as_u32(__hmul2(u32_as_h2(a45), s0)); a67 = h2_as_u32(__hmul2(u32_as_h2(a67), s0));
    b01 = h2_as_u32(__hmul2(u32_as_h2(b01), s1)); b23 = h2_as_u32(__hmul2(u32_as_h2(b23), s1));
    b45 = h2_as_u32(__hmul2(u32_as_h2(b45), s1)); b67 = h2_as_u32(__hmul2(u32_as_h2(b67), s1));
    if (ROUNDED) {
      a01 = round_bf16_pair(a01, rm0); a23 = round_bf16_pair(a23, rm0); a45 = round_bf16_pair(a45, rm0); a67 = round_bf16_pair(a67, rm0);
      b01 = round_bf16_pair(b01, rm1); b23 = round_bf16_pair(b23, rm1); b45 = round_bf16_pair(b45, rm1); b67 = round_bf16_pair(b67, rm1);
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      mma_f16(c[t], a01, b01, a23, b23, x[t].x, x[t].y);
      mma_f16(c[t], a45, b45, a67, b67, x[t].z, x[t].w);
    }
  }
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    facc[t][0] += c[t][0] + c[t][1];
    facc[t][1] += c[t][2] + c[t][3];
  }
}

// ---- block-FP8 (e4m3 payload [rows][k], float32 scale per 128 x 128; hayate `Fp8Block`) ---------------------------
// weight = bf16(e4m3 * scale) (hayate cu/glm53/math.cuh:40 `scaled_fp8`): formed per pair in float32, rounded to
// bf16, kept in fp16 as bf16(..) * 2^s with s chosen per scale so that the values stay normal. One 256-column block =
// two 128-column halves with their own scale. sc0 / sc1: the two scales of rows g / g + 8 for this block.
template <int PITCH, int NT>
DEVI void fp8_block_f16(uint32_t slab, int lane, const __half* const (&bcol)[NT], const float* sc0, const float* sc1, float (&facc)[NT][2]) {
  const int g = lane >> 2, j = lane & 3;
  const uint32_t r0 = slab + g * PITCH, r1 = slab + (g + 8) * PITCH;
#pragma unroll
  for (int hb = 0; hb < 2; ++hb) {                   // 128-column halves
    const float s0 = __ldg(sc0 + hb), s1 = __ldg(sc1 + hb);
    const int e0 = 14 - ilogbf(448.f * s0), e1 = 14 - ilogbf(448.f * s1);
    const float rm0 = scalbnf(s0, e0), rm1 = scalbnf(s1, e1);
    float c[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) c[t][i] = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {                    // 32 columns per step: this lane owns columns 8j..8j+7 of them
      const int col = hb * 128 + q * 32 + 8 * j;
      const uint2 w0 = lds64(r0 + col), w1 = lds64(r1 + col);
      uint4 x[NT];
#pragma unroll
      for (int t = 0; t < NT; ++t) x[t] = __ldg(reinterpret_cast<const uint4*>(bcol[t] + col));
      const uint32_t a01 = round_bf16_pair(e4m3x2_to_h2(w0.x & 0xffffu), rm0), a23 = round_bf16_pair(e4m3x2_to_h2(w0.x >> 16), rm0);
      const uint32_t a45 = round_bf16_pair(e4m3x2_to_h2(w0.y & 0xffffu), rm0), a67 = round_bf16_pair(e4m3x2_to_h2(w0.y >> 16), rm0);
      const uint32_t b01 = round_bf16_pair(e4m3x2_to_h2(w1.x & 0xffffu), rm1), b23 = round_bf16_pair(e4m3x2_to_h2(w1.x >> 16), rm1);
      const uint32_t b45 = round_bf16_pair(e4m3x2_to_h2(w1.y & 0xffffu), rm1), b67 = round_bf16_pair(e4m3x2_to_h2(w1.y >> 16), rm1);
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        mma_f16(c[t], a01, b01, a23, b23, x[t].x, x[t].y);
        mma_f16(c[t], a45, b45, a67, b67, x[t].z, x[t].w);
      }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      facc[t][0] += scalbnf(c[t][0] + c[t][1], -e0);
      facc[t][1] += scalbnf(c[t][2] + c[t][3], -e1);
    }
  }
}

// ring depth of a warp: as many stages of `stage_bytes` as fit beside the other warps' rings (2 to 5)
constexpr int gemv_ring_stages(int stage_bytes) {
  const int s = (208 * 1024) / (kGemvWarps * stage_bytes);
  return s > 5 ? 5 : (s < 2 ? 2 : s);
}
template <int FMT> struct GemvLayout;
// kPitch: bytes of a row slot; kChunks: 16-byte copies per row slot and block that are contiguous in global memory
// (kBlk bytes per block and row); kExtra: bytes per stage behind the 16 row slots (scale tile pieces). Formats with
// one more chunk per row slot that lives elsewhere (the Q6_K block scale d, the linear NVFP4 scales) copy it with
// lanes 0-15 (one row slot each).
template <> struct GemvLayout<kGemvQ4K> { static constexpr int kPitch = 160, kStages = gemv_ring_stages(16 * 160 + 0), kChunks = 9, kBlk = 144, kExtra = 0; };
template <> struct GemvLayout<kGemvQ6KR> { static constexpr int kPitch = 240, kStages = gemv_ring_stages(16 * 240 + 0), kChunks = 13, kBlk = 208, kExtra = 0; };       // + the d chunk at 208
template <> struct GemvLayout<kGemvNvfp4Linear> { static constexpr int kPitch = 144, kStages = gemv_ring_stages(16 * 144 + 0), kChunks = 8, kBlk = 128, kExtra = 0; }; // + the scale chunk at 128
template <> struct GemvLayout<kGemvFp8Block> { static constexpr int kPitch = 272, kStages = gemv_ring_stages(16 * 272 + 0), kChunks = 16, kBlk = 256, kExtra = 0; };   // 256 payload bytes per row slot
template <> struct GemvLayout<kGemvNvfp4Tiled> { static constexpr int kPitch = 144, kStages = gemv_ring_stages(16 * 144 + 256), kChunks = 8, kBlk = 128, kExtra = 256; }; // codes; 16 scale pieces per stage

template <int FMT> __host__ __device__ constexpr int gemv_stage_bytes() { return 16 * GemvLayout<FMT>::kPitch + GemvLayout<FMT>::kExtra; }
template <int FMT> __host__ __device__ constexpr int gemv_smem_bytes() {
  return kGemvWarps * GemvLayout<FMT>::kStages * gemv_stage_bytes<FMT>() + kGemvWarps * 8 * 16 * 4 + 16;
}

// Weight row of matrix-0 row slot `s` of slab `u` = slab_row0(u) + slab_rowc(s). Rows are slabs of RPT consecutive
// rows, except for the tiled NVFP4 layout where a slab takes 16 / RPT... base rows of a 128-row tile in all four
// 32-row quarters, so that the 16-byte pieces of the scale tiles are used completely.
template <int FMT, int DUAL>
DEVI int slab_row0(int u) {
  constexpr int RPT = DUAL ? 8 : 16;
  if (FMT != kGemvNvfp4Tiled) return u * RPT;
  constexpr int per128 = 128 / RPT;                 // slabs per 128-row tile
  return (u / per128) * 128 + (u % per128) * (RPT / 4);
}
template <int FMT, int DUAL>
DEVI int slab_rowc(int s) {
  if (FMT != kGemvNvfp4Tiled) return s;
  const int pl = DUAL ? (s & 1) : (s & 3), q = DUAL ? (s >> 1) : (s >> 2);
  return q * 32 + pl;
}
template <int FMT, int DUAL>
DEVI int slab_row(int u, int s) { return slab_row0<FMT, DUAL>(u) + slab_rowc<FMT, DUAL>(s); }

// Hayate SwiGLU: inputs rounded to bf16, gate <= 10, up in [-10, 10], bf16(bf16(g * sigmoid(g)) * u)
// (hayate cu/glm53/math.cuh:31-34, decode.cu:46).
DEVI float bf16_rn(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
DEVI float hayate_swiglu(float gate, float up) {
  gate = fminf(bf16_rn(gate), 10.f);
  up = fmaxf(-10.f, fminf(10.f, bf16_rn(up)));
  return bf16_rn(bf16_rn(gate * sigmoid_precise(gate)) * up);
}

// All items of one launch for this CTA (blockDim = kGemvWarps * 32, `smem` = gemv_smem_bytes<FMT>() bytes, 128-byte
// aligned). Also called phase by phase from the single-launch decode layer.
template <int FMT, int DUAL, bool MINS_TILE, int OUT>
DEVI void gemv_items(const GemvArgs& a, uint8_t* smem) {
  using LY = GemvLayout<FMT>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int STAGE = gemv_stage_bytes<FMT>();
  const uint32_t ring = smem_u32(smem) + warp * (LY::kStages * STAGE);
  float* red = reinterpret_cast<float*>(smem + kGemvWarps * LY::kStages * STAGE);   // [warp][token 8][row 16]
  constexpr int RPT = DUAL ? 8 : 16;                     // weight rows of matrix 0 per slab
  constexpr bool NV = FMT == kGemvNvfp4Linear || FMT == kGemvNvfp4Tiled;
  constexpr bool NATURAL = NV || FMT == kGemvFp8Block;    // activation planes in natural column order
  const unsigned tiles_per_group = (a.rows + RPT - 1) / RPT;
  const int nb_per = a.nb_per;
  const int groups = __ldcg(a.counters);
  const int g4 = lane >> 2, j = lane & 3;
  const int shared_row0 = a.out_shared_row;
  bool waited = !a.late_wait;
  // ---- this lane's share of a stage: fixed for the whole launch -------------------------------------------
  // The contiguous chunks of a block: LW lanes copy the NR row slots of one matrix (DUAL: lanes 0-15 the gate
  // slots 0-7, lanes 16-31 the up slots 8-15), P lanes per row slot (lane % P = the 16-byte part, parts past the
  // row's chunks idle), copy i of a lane = row slot i * RPI + sub.
  constexpr int LW = DUAL ? 16 : 32, NR = DUAL ? 8 : 16;
  constexpr int P = LY::kChunks <= 8 ? 8 : 16, RPI = LW / P, NI = NR / RPI;
  constexpr int ROW_STEP = FMT == kGemvNvfp4Tiled ? 32 : RPI;       // matrix rows between two copies of a lane
  const int lm = DUAL ? (lane >> 4) : 0, ll = lane & (LW - 1);
  const int part = ll & (P - 1), sub = ll / P;
  const uint32_t lane_dst = (lm * 8 + sub) * LY::kPitch + part * 16;   // + i * RPI * kPitch
  const uint32_t lane_src = uint32_t(sub) * uint32_t(a.row_bytes) + part * 16;
  const uint32_t src_step = uint32_t(ROW_STEP) * uint32_t(a.row_bytes);
  // lanes 0-15: the row slot whose extra chunk (Q6_K d, linear NVFP4 scales) or scale piece (tiled NVFP4) they copy
  const int xm = DUAL ? (lane >> 3) & 1 : 0, xs8 = DUAL ? (lane & 7) : (lane & 15);
  // ---- items: (group, slab, K part); the ks warps of a slab are neighbours in the CTA ------------------------
  const int slab_group = (warp * a.ks_inv) >> 16;             // warp / ks
  const int kpart = warp - slab_group * a.ks;
  const unsigned tile0 = blockIdx.x * unsigned(a.slab_groups) + unsigned(slab_group);
  unsigned grp = tile0 / tiles_per_group, slab_u = tile0 - grp * tiles_per_group;
  const unsigned gstep = a.group_step, sstep = a.slab_step;
  const int b_first = kpart * nb_per;
  auto next_item = [&]() {                   // tile += tstep, without a division
    slab_u += sstep;
    grp += gstep;
    if (slab_u >= tiles_per_group) {
      slab_u -= tiles_per_group;
      ++grp;
    }
  };
  for (; grp < unsigned(a.max_groups); next_item()) {
    const bool live = int(grp) < groups;     // uniform over the ks warps of a slab
    // the plan array holds max_groups entries: the entry is fetched without waiting for the group count (two
    // dependent L2 round trips less before the first weight request), stale entries are masked by `live`
    int4 pl = __ldcg(a.plan + grp);
    if (!live) pl = make_int4(0, 0, 0, 0);
    const int e = pl.x, count = live ? pl.y : 0, offset = pl.z;
    // base of the two matrices of this group's expert
    const uint8_t* mbase[2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      if (e < 0) mbase[m] = a.w_shared[m];
      else if (a.w_table) mbase[m] = reinterpret_cast<const uint8_t*>(__ldcg(reinterpret_cast<const unsigned long long*>(a.w_table) + grp)) + m * a.matrix_stride + (size_t)a.expert_stride[m];
      else mbase[m] = a.w[m] ? a.w[m] + size_t(e) * a.expert_stride[m] : nullptr;
    }
    // ---- weight stream: 16 row slots x one block per stage --------------------------------------------
    const int row0 = slab_row0<FMT, DUAL>(int(slab_u));
    // copies of this lane whose row exists (row slots past the last row of the matrix are not copied)
    int n_copies = part < LY::kChunks ? NI : 0;
    if (FMT != kGemvNvfp4Tiled) n_copies = min(n_copies, max(0, (a.rows - row0 - sub + RPI - 1) / RPI));
    const uint8_t* lane_rows = mbase[lm] + size_t(row0) * a.row_bytes + size_t(b_first) * LY::kBlk + lane_src;
    // extra chunk / scale pieces: source of block b_first (lanes 0-15)
    const uint8_t* extra = nullptr;
    if (lane < 16) {
      if (FMT == kGemvQ6KR) {
        const int r = row0 + xs8;
        if (r < a.rows) extra = mbase[xm] + size_t(r) * a.row_bytes + a.nblk * 208;
      } else if (FMT == kGemvNvfp4Linear) {
        const int r = row0 + xs8;
        if (r < a.rows) extra = mbase[xm] + a.scale_offset[xm] + size_t(r) * (a.k / 16) + b_first * 16;
      } else if (FMT == kGemvNvfp4Tiled) {
        // scale tile pieces: piece = (matrix, local base row) x 4 tile columns; 16 bytes each
        const int piece = lane, tc = piece & 3, pm = piece >> 2;
        const int m = DUAL ? (pm >> 1) : 0, pl_ = DUAL ? (pm & 1) : pm;
        const int r = slab_row<FMT, DUAL>(int(slab_u), pl_);               // quarter 0 row of this base row
        const int cols = (a.k / 16 + 3) / 4 * 4;
        if (r < a.rows) extra = mbase[m] + a.scale_offset[m] + (size_t(r / 128) * (cols / 4) + (b_first * 4 + tc)) * 512 + (r % 32) * 16;
      }
    }
    auto issue = [&](int i_blk, int stage) {              // block b_first + i_blk of this item
      const uint32_t dst = ring + stage * STAGE;
      const uint8_t* src = lane_rows + i_blk * LY::kBlk;
#pragma unroll
      for (int i = 0; i < NI; ++i)
        if (i < n_copies) cp_async16(dst + lane_dst + i * (RPI * LY::kPitch), src + size_t(i) * src_step);
      if (FMT == kGemvQ6KR) {
        if (extra) cp_async16(dst + lane * LY::kPitch + 208, extra + ((2 * (b_first + i_blk)) & ~15));
      } else if (FMT == kGemvNvfp4Linear) {
        if (extra) cp_async16(dst + lane * LY::kPitch + 128, extra + i_blk * 16);
      } else if (FMT == kGemvNvfp4Tiled) {
        if (extra) cp_async16(dst + 16 * LY::kPitch + lane * 16, extra + i_blk * 2048);
      }
    };
    if (count > 0) {
#pragma unroll
      for (int s = 0; s < LY::kStages - 1; ++s) {
        if (s < nb_per) issue(s, s);
        cp_async_commit();
      }
    }
    // per-matrix float multipliers of this expert (global scales of NVFP4)
    float gs0 = 1.f, gs1 = 1.f;
    if (NV && live) {
      if (a.gscale_in_matrix[0]) {
        gs0 = __ldg(reinterpret_cast<const float*>(mbase[0] + a.gscale_in_matrix[0]));
        if (DUAL) gs1 = __ldg(reinterpret_cast<const float*>(mbase[1] + a.gscale_in_matrix[1]));
      } else if (e < 0) {
        if (a.gscale_shared[0]) gs0 = __ldg(reinterpret_cast<const float*>(a.gscale_shared[0]));
        if (DUAL && a.gscale_shared[1]) gs1 = __ldg(reinterpret_cast<const float*>(a.gscale_shared[1]));
      } else if (a.gscale) {
        gs0 = __ldg(reinterpret_cast<const float*>(a.gscale + size_t(e) * a.gscale_estride));
        if (DUAL) gs1 = __ldg(reinterpret_cast<const float*>(a.gscale + size_t(e) * a.gscale_estride + a.gscale_mstride));
      }
    }
    // block-FP8: the scale rows of this lane's two weight rows (rows g and g + 8 of the slab)
    const float *fsc0 = nullptr, *fsc1 = nullptr;
    if (FMT == kGemvFp8Block && live) {
      const int kb128 = a.k / 128;
      const int ra = slab_row<FMT, DUAL>(slab_u, DUAL ? g4 : g4), rb = slab_row<FMT, DUAL>(slab_u, DUAL ? g4 : g4 + 8);
      const int ma = 0, mb = DUAL ? 1 : 0;
      const float* base_a = (e < 0 && a.scale_shared[ma]) ? a.scale_shared[ma] : reinterpret_cast<const float*>(mbase[ma] + a.scale_offset[ma]);
      const float* base_b = (e < 0 && a.scale_shared[mb]) ? a.scale_shared[mb] : reinterpret_cast<const float*>(mbase[mb] + a.scale_offset[mb]);
      fsc0 = base_a + size_t((ra < a.rows ? ra : 0) / 128) * kb128;
      fsc1 = base_b + size_t((rb < a.rows ? rb : 0) / 128) * kb128;
    }
    // shared expert with bf16-rounded weights: A = bf16(code * scale * g) * 2^s, epilogue multiplier 2^-s
    float rm0 = 0.f, rm1 = 0.f;
    const bool rounded = NV && live && e < 0 && a.round_shared;
    if (rounded) {
      const int s0 = 14 - ilogbf(2688.f * gs0), s1 = 14 - ilogbf(2688.f * gs1);
      rm0 = scalbnf(gs0, s0); gs0 = scalbnf(1.f, -s0);
      rm1 = DUAL ? scalbnf(gs1, s1) : rm0;
      if (DUAL) gs1 = scalbnf(1.f, -s1);
    }
    if (!waited) {                                        // the activation planes of the predecessor are read from here on
      pdl_wait();
      waited = true;
    }
    // One pass over the item's blocks for the tokens c0 .. c0 + 4 NT - 1 of the group (NT groups of four: the weight
    // fragments are built once per pass).
    auto pass = [&](auto nt_tag, int c0) {
      constexpr int NT = decltype(nt_tag)::value;
      const __half* plane[NT];
      const __half* xs[NT];
      int ares[NT];
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        // this lane's B column g4 -> token g4/2 of the group, hi (even) or lo (odd) plane
        // (a column without a token reads the rows of token c0: its sums are never stored)
        const int tcol = c0 + 4 * t + (g4 >> 1) < count ? c0 + 4 * t + (g4 >> 1) : c0;
        xs[t] = nullptr;
        {
          const int as = e < 0 ? shared_row0 + tcol : int(__ldcg(a.assignments + offset + tcol));
          const int xrow = a.x_by_assignment ? as : (e < 0 ? a.shared_x_row0 + tcol : as / a.topk);
          plane[t] = a.xplanes + (size_t(xrow) * 2 + (g4 & 1)) * a.k + size_t(b_first) * 256;
          if (FMT == kGemvQ4K && !MINS_TILE && a.xsum_planes) xs[t] = a.xsum_planes + (size_t(xrow) * 2 + (g4 & 1)) * (a.k / 32) + b_first * 8;
        }
        // this lane's result column pair 2j,2j+1 -> token j of the group
        const int tres = c0 + 4 * t + j;
        ares[t] = -1;
        if (tres < count) ares[t] = e < 0 ? shared_row0 + tres : int(__ldcg(a.assignments + offset + tres));
      }
      if (c0 > 0) {                                       // later passes stream the blocks again (L2 hits)
#pragma unroll
        for (int s = 0; s < LY::kStages - 1; ++s) {
          if (s < nb_per) issue(s, s);
          cp_async_commit();
        }
      }
      float facc[NT][2];
#pragma unroll
      for (int t = 0; t < NT; ++t) facc[t][0] = facc[t][1] = 0.f;
      for (int i = 0; i < nb_per; ++i) {
        const int nxt = i + LY::kStages - 1;
        if (nxt < nb_per) issue(nxt, nxt % LY::kStages);
        cp_async_commit();
        cp_async_wait<LY::kStages - 1>();
        __syncwarp();
        const int b = b_first + i;
        const uint32_t slab = ring + (i % LY::kStages) * STAGE;
        const __half* bcol[NT];
        const __half* xsb[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          bcol[t] = plane[t] + i * 256;
          xsb[t] = xs[t] ? xs[t] + i * 8 : nullptr;
        }
        if (FMT == kGemvQ4K) q4k_block_f16<LY::kPitch, MINS_TILE, NT>(slab, lane, bcol, xsb, facc);
        else if (FMT == kGemvQ6KR) q6k_block_f16<LY::kPitch, NT>(slab, lane, (2 * b) & 15, bcol, facc);
        else if (FMT == kGemvFp8Block) fp8_block_f16<LY::kPitch, NT>(slab, lane, bcol, fsc0 + 2 * b, fsc1 + 2 * b, facc);
        else if (rounded) nvfp4_block_f16<FMT, DUAL, LY::kPitch, true, NT>(slab, lane, bcol, rm0, rm1, facc);
        else nvfp4_block_f16<FMT, DUAL, LY::kPitch, false, NT>(slab, lane, bcol, 0.f, 0.f, facc);
        __syncwarp();
      }
      cp_async_wait<0>();
      // ---- sum over the K split (fixed order) and store ------------------------------------------------
      if (a.ks > 1) {
        const int bar = 1 + warp / a.ks;                  // one named barrier per slab group (<= 12)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          red[(warp * 8 + 4 * t + j) * 16 + g4] = facc[t][0];
          red[(warp * 8 + 4 * t + j) * 16 + 8 + g4] = facc[t][1];
        }
        named_barrier(bar, a.ks * 32);
        if (kpart == 0) {
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            facc[t][0] = 0.f;
            facc[t][1] = 0.f;
            for (int q = 0; q < a.ks; ++q) {
              facc[t][0] += red[((warp + q) * 8 + 4 * t + j) * 16 + g4];
              facc[t][1] += red[((warp + q) * 8 + 4 * t + j) * 16 + 8 + g4];
            }
          }
        }
        named_barrier(bar, a.ks * 32);                    // partials are consumed before the next pass overwrites them
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        if (kpart != 0 || ares[t] < 0) continue;
        if (DUAL) {
          const int r = slab_row<FMT, DUAL>(slab_u, g4);
          if (r < a.rows) {
            const float gv = facc[t][0] * gs0, uv = facc[t][1] * gs1;
            const float h = OUT == kOutHayateProduct ? hayate_swiglu(gv, uv) : silu_mul(gv, uv);
            const __half hi = __float2half_rn(h);
            const __half lo = __float2half_rn(h - __half2float(hi));
            if (fabsf(h) > 65504.f && a.status) atomicOr(a.status, 4u);       // does not fit the fp16 planes
            __half* dst = a.out_planes + size_t(ares[t]) * 2 * a.rows + (NATURAL ? r : plane_pos(r));
            dst[0] = hi;
            dst[a.rows] = lo;
            if (OUT == kOutHayateProduct && a.out_bf16) a.out_bf16[size_t(ares[t]) * a.rows + r] = __float2bfloat16_rn(h);
          }
        } else {
          const int r0 = slab_row<FMT, DUAL>(slab_u, g4), r1 = slab_row<FMT, DUAL>(slab_u, g4 + 8);
          if (OUT == kOutBf16) {
            if (r0 < a.rows) a.out_bf16[size_t(ares[t]) * a.rows + r0] = __float2bfloat16_rn(facc[t][0] * gs0);
            if (r1 < a.rows) a.out_bf16[size_t(ares[t]) * a.rows + r1] = __float2bfloat16_rn(facc[t][1] * gs0);
          } else {
            if (r0 < a.rows) a.out[size_t(ares[t]) * a.rows + r0] = facc[t][0] * gs0;
            if (r1 < a.rows) a.out[size_t(ares[t]) * a.rows + r1] = facc[t][1] * gs0;
          }
        }
      }
    };
    for (int c0 = 0; c0 < count;) {
      if (count - c0 > 4) {
        pass(std::integral_constant<int, 2>{}, c0);
        c0 += 8;
      } else {
        pass(std::integral_constant<int, 1>{}, c0);
        c0 += 4;
      }
    }
  }
}

template <int FMT, int DUAL, bool MINS_TILE, int OUT>
__global__ void __launch_bounds__(kGemvWarps * 32, 1) expert_gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  if (!a.late_wait) pdl_wait();
  pdl_launch();
  gemv_items<FMT, DUAL, MINS_TILE, OUT>(a, smem);
  if (a.late_wait) pdl_wait();       // warps without items: the grid must not finish before its predecessor
}

// ---- activation rows -> planes (and per-32 sums) ------------------------------------------------------
// One block per row. planes[row] = k fp16 hi values then k fp16 lo values, groups of four as [x0,x2,x1,x3]
// (or in natural order for the NVFP4 kernels).
template <typename XT>
DEVI void act_planes_row(const XT* x, int k, __half* planes, __half* xsum_planes, bool natural, unsigned* status = nullptr) {
  bool out_of_range = false;        // |value| > 65504 does not fit the fp16 planes: reported in the status word (bit 4)
  for (int base = 0; base < k / 4; base += blockDim.x) {            // uniform trip count: shuffles below
    const int i = base + threadIdx.x;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < k / 4) {
      if (sizeof(XT) == 4) v = __ldcg(reinterpret_cast<const float4*>(x) + i);
      else {
        const uint2 raw = __ldcg(reinterpret_cast<const uint2*>(x) + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 lo2 = __bfloat1622float2(h[0]), hi2 = __bfloat1622float2(h[1]);
        v = make_float4(lo2.x, lo2.y, hi2.x, hi2.y);
      }
    }
    const float vals[4] = {v.x, natural ? v.y : v.z, natural ? v.z : v.y, v.w};   // storage order
    __half hi[4], lo[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      hi[q] = __float2half_rn(vals[q]);
      lo[q] = __float2half_rn(vals[q] - __half2float(hi[q]));
      out_of_range |= fabsf(vals[q]) > 65504.f;
    }
    if (i < k / 4) {
      *reinterpret_cast<uint2*>(planes + 4 * i) = make_uint2(h2_as_u32(__halves2half2(hi[0], hi[1])), h2_as_u32(__halves2half2(hi[2], hi[3])));
      *reinterpret_cast<uint2*>(planes + k + 4 * i) = make_uint2(h2_as_u32(__halves2half2(lo[0], lo[1])), h2_as_u32(__halves2half2(lo[2], lo[3])));
    }
    if (xsum_planes) {
      float p = (v.x + v.y) + (v.z + v.w);
      p += __shfl_xor_sync(0xffffffffu, p, 1);
      p += __shfl_xor_sync(0xffffffffu, p, 2);
      p += __shfl_xor_sync(0xffffffffu, p, 4);
      if (i < k / 4 && (i & 7) == 0) {
        const __half hs = __float2half_rn(p);
        xsum_planes[i >> 3] = hs;
        xsum_planes[k / 32 + (i >> 3)] = __float2half_rn(p - __half2float(hs));
      }
    }
  }
  if (out_of_range && status) atomicOr(status, 4u);
}

}  // namespace dmoe
