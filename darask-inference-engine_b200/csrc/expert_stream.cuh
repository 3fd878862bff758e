// Decode-path expert products: quantized weight rows are streamed HBM -> shared memory by the
// TMA engine (bulk copies completing on mbarriers, a ring of stages per CTA) and multiplied with
// the activations on integer tensor-core tiles, so that the ALUs only unpack bit fields:
//   * the 4/6-bit weight codes go into the A operand of mma.sync (u8) as they are,
//   * an activation row is split once per CTA into three signed 7-bit "digits"
//     x ~ s/127 * (d1 + d2/254 + d3/254^2)   (|error| <= 2^-22 * max|x|),
//     one digit per B column, so the products are exact int32 sums,
//   * per-sub-block integer scales are applied to the int32 tile results, the f16 super-block
//     scale once per block; offsets (Q4_K mins, the -32 of Q6_K) are one more small tile against
//     the digits of the per-sub-block sums of x.
// Work item ("tile") = one group of tokens that chose the same expert x a slab of rows of that
// expert. Persistent CTAs (one per SM) each take a contiguous range of tiles.
//   DUAL = 1: gate and up rows of the same index are streamed together (row slots 0-15 gate,
//             16-31 up of each row group); the epilogue writes silu(g) * u.
//   DUAL = 0: plain rows (down projection).
// Replaces the reference's per-engine GEMV kernels (kogarashi kernels/native.cu:46-88 `gemv` +
// :97-99 `activate`; tsumuji kernels/decode/gemv.cu:64-158; hayate cu/glm53/decode.cu:37-54).
#pragma once
#include "common.cuh"

namespace dmoe {

enum StreamFormat { kFmtQ4K = 0, kFmtQ6KR = 1 };
enum Activation { kActSilu = 0, kActHayate = 1 };

constexpr int kMaxStages = 4;
constexpr int kDigits = 3;

struct StreamArgs {
  const uint8_t* w[2];          // routed experts: matrix 0 (gate or down) and matrix 1 (up)
  const uint8_t* w_shared[2];   // shared expert matrices (null when there is none)
  unsigned long long expert_stride[2];   // bytes between consecutive experts
  int row_bytes;                // bytes of one row in global memory (multiple of 16)
  int pitch;                    // bytes of one row slot in shared memory (multiple of 16)
  int k, rows, nblk;            // columns, rows per matrix, k / 256
  int rg, ks, stages;           // row groups, K split, ring depth; compute warps = rg * ks
  const float* x;               // activations, float32 rows of k
  int x_by_assignment;          // 0: row = token; 1: row = assignment index
  const int* counters;          // [0] = number of active experts
  const int* active;            // ascending ids of experts with at least one row
  const unsigned* ranges;       // [E][2] rows, offset
  const unsigned* assignments;  // [T*k]
  int tokens, topk, has_shared;
  float* out;                   // [T*k (+T)][rows]
  unsigned* status;
};

// ---- tensor-core tiles ---------------------------------------------------------------------------
// C[16x8] (int32) = A[16x32] (u8, row) x B[32x8] (s8, col). Thread (g = lane / 4, j = lane % 4):
// a0/a1: rows g / g+8, k 4j..4j+3; a2/a3: same rows, k 16+4j..; b0/b1: column g, k 4j.. / 16+4j..;
// c0,c1: row g, columns 2j, 2j+1; c2,c3: row g+8.
DEVI void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// C[16x8] = A[16x16] (u8 or s8) x B[16x8] (s8): a0/a1 rows g / g+8, k 4j..4j+3; b0 column g, k 4j..
DEVI void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
DEVI void mma_s8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
template <int I> DEVI int ubyte(uint32_t w) { return int((w >> (8 * I)) & 0xffu); }
template <int I> DEVI int sbyte(uint32_t w) { return int(w << (24 - 8 * I)) >> 24; }

// What a warp needs to know about the activation rows staged in shared memory.
struct XPlanes {
  const uint8_t* dig;     // [TT][kDigits][k]      digits of x
  const uint8_t* sdig;    // [TT][kDigits][nsum]   digits of the sub-block sums of x
  const float* scale;     // [TT][2]               s/127 of x, s'/127 of the sums
  int k, nsum;
};

// Column c of a tile belongs to token c / 4, digit c % 4 (digit 3 is empty). This thread supplies
// B column g = lane / 4 and owns result columns 2j, 2j+1.
template <int TT>
DEVI const uint8_t* b_plane(const XPlanes& xp, int col) {
  const int t = col >> 2, d = col & 3;
  return (t < TT && d < kDigits) ? xp.dig + (size_t(t) * kDigits + d) * xp.k : nullptr;
}
template <int TT>
DEVI const uint8_t* bs_plane(const XPlanes& xp, int col) {
  const int t = col >> 2, d = col & 3;
  return (t < TT && d < kDigits) ? xp.sdig + (size_t(t) * kDigits + d) * xp.nsum : nullptr;
}

// GGUF Q4_K block (144 B: d, dmin f16 | 12 scale bytes | 128 nibble bytes), value = d*sc*q - dmin*m
// (kogarashi kernels/native.cu:26-34). rows[i]: shared-memory row slots of rows g, g+8 of the two
// 16-row tiles. facc[tile][half] accumulates this lane's share (its two result columns).
template <int TT>
DEVI void q4k_block(const uint8_t* const (&rows)[4], int b, const XPlanes& xp, int lane, float (&facc)[4]) {
  const int g = lane >> 2, j = lane & 3;
  const uint8_t* bp = b_plane<TT>(xp, g);
  const uint8_t* bsp = bs_plane<TT>(xp, g);
  uint32_t sc_lo[4], sc_hi[4], mn_lo[4], mn_hi[4];
  float d[4], dmin[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(rows[i] + b * 144);
    d[i] = half_lo(hdr.x);
    dmin[i] = half_hi(hdr.x);
    sc_lo[i] = hdr.y & 0x3F3F3F3Fu;
    mn_lo[i] = hdr.z & 0x3F3F3F3Fu;
    sc_hi[i] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
    mn_hi[i] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
  }
  int iacc[2][4] = {};
#pragma unroll
  for (int gp = 0; gp < 4; ++gp) {
    // B: digits of x for sub-blocks 2gp (low nibbles) and 2gp + 1 (high nibbles), elements 8j..8j+7
    uint2 blo = make_uint2(0, 0), bhi = make_uint2(0, 0);
    if (bp) {
      blo = *reinterpret_cast<const uint2*>(bp + b * 256 + gp * 64 + 8 * j);
      bhi = *reinterpret_cast<const uint2*>(bp + b * 256 + gp * 64 + 32 + 8 * j);
    }
#pragma unroll
    for (int tile = 0; tile < 2; ++tile) {
      const uint2 w0 = *reinterpret_cast<const uint2*>(rows[2 * tile] + b * 144 + 16 + gp * 32 + 8 * j);
      const uint2 w1 = *reinterpret_cast<const uint2*>(rows[2 * tile + 1] + b * 144 + 16 + gp * 32 + 8 * j);
      int c[4];
      mma_u8s8_k32(c, w0.x & 0x0F0F0F0Fu, w1.x & 0x0F0F0F0Fu, w0.y & 0x0F0F0F0Fu, w1.y & 0x0F0F0F0Fu, blo.x, blo.y);
      const uint32_t s0 = gp < 2 ? sc_lo[2 * tile] : sc_hi[2 * tile], s1 = gp < 2 ? sc_lo[2 * tile + 1] : sc_hi[2 * tile + 1];
      int sa, sb, ta, tb;    // scales of sub-blocks 2gp, 2gp+1 for rows g / g+8
      if ((gp & 1) == 0) { sa = ubyte<0>(s0); ta = ubyte<1>(s0); sb = ubyte<0>(s1); tb = ubyte<1>(s1); }
      else { sa = ubyte<2>(s0); ta = ubyte<3>(s0); sb = ubyte<2>(s1); tb = ubyte<3>(s1); }
      iacc[tile][0] += sa * c[0]; iacc[tile][1] += sa * c[1]; iacc[tile][2] += sb * c[2]; iacc[tile][3] += sb * c[3];
      mma_u8s8_k32(c, (w0.x >> 4) & 0x0F0F0F0Fu, (w1.x >> 4) & 0x0F0F0F0Fu, (w0.y >> 4) & 0x0F0F0F0Fu,
                   (w1.y >> 4) & 0x0F0F0F0Fu, bhi.x, bhi.y);
      iacc[tile][0] += ta * c[0]; iacc[tile][1] += ta * c[1]; iacc[tile][2] += tb * c[2]; iacc[tile][3] += tb * c[3];
    }
  }
  // mins: one k16 tile per row tile, A = the eight 6-bit mins of a row, B = digits of the sub-block sums
  const uint32_t bs = (bsp && j < 2) ? *reinterpret_cast<const uint32_t*>(bsp + b * 8 + 4 * j) : 0u;
  const int t = j >> 1;
  const float xs = t < TT ? xp.scale[2 * t] : 0.f, ss = t < TT ? xp.scale[2 * t + 1] : 0.f;
  const float wa = (j & 1) ? 1.f / (254.f * 254.f) : 1.f, wb = (j & 1) ? 0.f : 1.f / 254.f;
#pragma unroll
  for (int tile = 0; tile < 2; ++tile) {
    int cm[4];
    const uint32_t m0 = j == 0 ? mn_lo[2 * tile] : j == 1 ? mn_hi[2 * tile] : 0u;
    const uint32_t m1 = j == 0 ? mn_lo[2 * tile + 1] : j == 1 ? mn_hi[2 * tile + 1] : 0u;
    mma_u8s8_k16(cm, m0, m1, bs);
    const float p0 = fmaf(float(iacc[tile][0]), wa, float(iacc[tile][1]) * wb) * xs;
    const float p1 = fmaf(float(iacc[tile][2]), wa, float(iacc[tile][3]) * wb) * xs;
    const float q0 = fmaf(float(cm[0]), wa, float(cm[1]) * wb) * ss;
    const float q1 = fmaf(float(cm[2]), wa, float(cm[3]) * wb) * ss;
    facc[2 * tile] += d[2 * tile] * p0 - dmin[2 * tile] * q0;
    facc[2 * tile + 1] += d[2 * tile + 1] * p1 - dmin[2 * tile + 1] * q1;
  }
}

// GGUF Q6_K in the row-aligned device layout ("Q6_K-R16"): a row is nblk x [ql 128 | qh 64 |
// int8 scales 16] followed by nblk f16 `d` (padded to 16 bytes); the same bits as the 210-byte
// GGUF blocks, regrouped so that every block starts on a 16-byte boundary.
// value = d * scale * (q - 32)  (kogarashi kernels/native.cu:35-40); scale groups are 16 wide, so
// the tiles are k16; the -32 is applied as 32 * sum_s scale_s * (sum of x over group s).
template <int TT>
DEVI void q6k_block(const uint8_t* const (&rows)[4], int b, int nblk, const XPlanes& xp, int lane, float (&facc)[4]) {
  const int g = lane >> 2, j = lane & 3;
  const uint8_t* bp = b_plane<TT>(xp, g);
  const uint8_t* bsp = bs_plane<TT>(xp, g);
  uint32_t sc[4][4];
  float d[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 v = *reinterpret_cast<const uint4*>(rows[i] + b * 208 + 192);
    sc[i][0] = v.x; sc[i][1] = v.y; sc[i][2] = v.z; sc[i][3] = v.w;
    d[i] = __half2float(*reinterpret_cast<const __half*>(rows[i] + nblk * 208 + 2 * b));
  }
  int iacc[2][4] = {};
#pragma unroll
  for (int n = 0; n < 2; ++n) {
#pragma unroll
    for (int lh = 0; lh < 2; ++lh) {
      uint32_t h[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = *reinterpret_cast<const uint32_t*>(rows[i] + b * 208 + 128 + n * 32 + lh * 16 + 4 * j);
#pragma unroll
      for (int gb = 0; gb < 2; ++gb) {
        const int col_lo = n * 128 + gb * 32 + lh * 16 + 4 * j;        // elements of the low-nibble group
        const uint32_t blo = bp ? *reinterpret_cast<const uint32_t*>(bp + b * 256 + col_lo) : 0u;
        const uint32_t bhi = bp ? *reinterpret_cast<const uint32_t*>(bp + b * 256 + col_lo + 64) : 0u;
        const int s_lo = 8 * n + 2 * gb + lh, s_hi = s_lo + 4;         // scale index of the two groups
#pragma unroll
        for (int tile = 0; tile < 2; ++tile) {
          uint32_t lo[2], hi[2];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(rows[2 * tile + r] + b * 208 + n * 64 + gb * 32 + lh * 16 + 4 * j);
            const uint32_t hh = h[2 * tile + r];
            lo[r] = (w & 0x0F0F0F0Fu) | ((hh << (4 - 2 * gb)) & 0x30303030u);
            hi[r] = ((w >> 4) & 0x0F0F0F0Fu) | ((hh >> (2 * gb)) & 0x30303030u);
          }
          const uint32_t(&s0)[4] = sc[2 * tile];
          const uint32_t(&s1)[4] = sc[2 * tile + 1];
          auto pick = [](const uint32_t(&s)[4], int idx) {             // idx is a compile-time constant after unrolling
            const uint32_t w = s[idx >> 2];
            return (idx & 3) == 0 ? sbyte<0>(w) : (idx & 3) == 1 ? sbyte<1>(w) : (idx & 3) == 2 ? sbyte<2>(w) : sbyte<3>(w);
          };
          int c[4];
          mma_u8s8_k16(c, lo[0], lo[1], blo);
          int sa = pick(s0, s_lo), sb = pick(s1, s_lo);
          iacc[tile][0] += sa * c[0]; iacc[tile][1] += sa * c[1]; iacc[tile][2] += sb * c[2]; iacc[tile][3] += sb * c[3];
          mma_u8s8_k16(c, hi[0], hi[1], bhi);
          sa = pick(s0, s_hi); sb = pick(s1, s_hi);
          iacc[tile][0] += sa * c[0]; iacc[tile][1] += sa * c[1]; iacc[tile][2] += sb * c[2]; iacc[tile][3] += sb * c[3];
        }
      }
    }
  }
  // offset: 32 * sum_s scale_s * xsum16_s, A = the sixteen int8 scales of a row, B = digits of the sums
  const uint32_t bs = bsp ? *reinterpret_cast<const uint32_t*>(bsp + b * 16 + 4 * j) : 0u;
  const int t = j >> 1;
  const float xs = t < TT ? xp.scale[2 * t] : 0.f, ss = t < TT ? xp.scale[2 * t + 1] : 0.f;
  const float wa = (j & 1) ? 1.f / (254.f * 254.f) : 1.f, wb = (j & 1) ? 0.f : 1.f / 254.f;
#pragma unroll
  for (int tile = 0; tile < 2; ++tile) {
    int cm[4];
    const uint32_t a0 = j == 0 ? sc[2 * tile][0] : j == 1 ? sc[2 * tile][1] : j == 2 ? sc[2 * tile][2] : sc[2 * tile][3];
    const uint32_t a1 = j == 0 ? sc[2 * tile + 1][0] : j == 1 ? sc[2 * tile + 1][1] : j == 2 ? sc[2 * tile + 1][2] : sc[2 * tile + 1][3];
    mma_s8s8_k16(cm, a0, a1, bs);
    const float p0 = fmaf(float(iacc[tile][0]), wa, float(iacc[tile][1]) * wb) * xs;
    const float p1 = fmaf(float(iacc[tile][2]), wa, float(iacc[tile][3]) * wb) * xs;
    const float q0 = fmaf(float(cm[0]), wa, float(cm[1]) * wb) * ss * 32.f;
    const float q1 = fmaf(float(cm[2]), wa, float(cm[3]) * wb) * ss * 32.f;
    facc[2 * tile] += d[2 * tile] * (p0 - q0);
    facc[2 * tile + 1] += d[2 * tile + 1] * (p1 - q1);
  }
}

// Shared-memory carve-up, shared by host (size) and device (offsets).
struct StreamSmem {
  int stage_bytes, dig_off, sdig_off, scale_off, sums_off, red_off, bar_off, total;
};
__host__ __device__ inline int stream_nsum(int fmt, int k) { return fmt == kFmtQ4K ? k / 32 : k / 16; }
__host__ __device__ inline StreamSmem stream_smem(int fmt, int rg, int ks, int stages, int pitch, int k, int tt) {
  StreamSmem s;
  const int nsum = stream_nsum(fmt, k);
  s.stage_bytes = 32 * rg * pitch;
  s.dig_off = stages * s.stage_bytes;
  s.sdig_off = s.dig_off + tt * kDigits * k;
  s.scale_off = s.sdig_off + (tt * kDigits * nsum + 15) / 16 * 16;
  s.sums_off = s.scale_off + 16 * tt;
  s.red_off = s.sums_off + nsum * 4 + 64 * 4;                 // float sums of one row + block-max scratch
  s.bar_off = s.red_off + 2 * rg * ks * tt * 32 * 4;
  s.total = s.bar_off + 2 * kMaxStages * 8 + 16;
  return s;
}

// x -> three signed 7-bit digits: x ~ (s/127) * (d1 + d2/254 + d3/254^2) with inv = 127 / s.
DEVI void digits3(float x, float inv, int (&d)[3]) {
  const float r0 = x * inv;
  const float d1 = rintf(r0);
  const float r1 = (r0 - d1) * 254.f;
  const float d2 = rintf(r1);
  const float d3 = rintf((r1 - d2) * 254.f);
  d[0] = int(d1); d[1] = int(d2); d[2] = int(d3);
}

template <int FMT, int DUAL, int TT, int ACT>
__global__ void __launch_bounds__(544, 1) expert_stream_kernel(const StreamArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int NW = a.rg * a.ks;                       // compute warps; warp NW is the producer
  const StreamSmem L = stream_smem(FMT, a.rg, a.ks, a.stages, a.pitch, a.k, TT);
  const int nsum = stream_nsum(FMT, a.k);
  uint8_t* dig = smem + L.dig_off;
  uint8_t* sdig = smem + L.sdig_off;
  float* xscale = reinterpret_cast<float*>(smem + L.scale_off);
  float* sums = reinterpret_cast<float*>(smem + L.sums_off);
  float* bmax = sums + nsum;
  float* red = reinterpret_cast<float*>(smem + L.red_off);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bar_off);
  uint64_t* empty = full + kMaxStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kMaxStages);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, NW);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait();          // routing metadata and activations come from the previous kernels
  pdl_launch();
  const int n_active = __ldcg(a.counters);
  const int groups = n_active + (a.has_shared ? 1 : 0);
  const int rows_per_tile = (DUAL ? 16 : 32) * a.rg;
  const int tiles_per_group = (a.rows + rows_per_tile - 1) / rows_per_tile;
  const long long total = (long long)groups * tiles_per_group;
  const int t_begin = int(total * blockIdx.x / gridDim.x), t_end = int(total * (blockIdx.x + 1) / gridDim.x);
  const int routed = a.tokens * a.topk;

  if (warp == NW) {
    // ---- producer: one bulk copy per row slot -------------------------------------------------
    for (int tile = t_begin, it = 0; tile < t_end; ++tile, ++it) {
      const int s = it % a.stages;
      if (it >= a.stages) {
        int ok = 1;
        if (lane == 0) ok = mbar_wait(empty + s, ((it / a.stages) & 1) ^ 1, a.status) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      const int g = tile / tiles_per_group, row0 = (tile % tiles_per_group) * rows_per_tile;
      const bool sh = g >= n_active;
      const int e = sh ? 0 : __ldcg(a.active + g);
      const int valid = min(rows_per_tile, a.rows - row0);
      if (lane == 0) mbar_arrive_expect_tx(full + s, uint32_t(valid) * (DUAL ? 2u : 1u) * uint32_t(a.row_bytes));
      __syncwarp();
      uint8_t* stage = smem + s * L.stage_bytes;
      for (int slot = lane; slot < 32 * a.rg; slot += 32) {
        const int rgi = slot >> 5, l = slot & 31;
        const int m = DUAL ? (l >> 4) : 0;
        const int r = DUAL ? rgi * 16 + (l & 15) : slot;
        if (r < valid) {
          const uint8_t* base = sh ? a.w_shared[m] : a.w[m] + size_t(e) * a.expert_stride[m];
          bulk_g2s(stage + size_t(slot) * a.pitch, base + size_t(row0 + r) * a.row_bytes, a.row_bytes, full + s);
        }
      }
    }
    return;
  }

  // ---- consumers ---------------------------------------------------------------------------------
  const int rgi = warp / a.ks, kw = warp % a.ks;
  const int nthr = NW * 32, tid = threadIdx.x;
  XPlanes xp{dig, sdig, xscale, a.k, nsum};
  long long loaded_key = -1;       // which activation rows sit in the digit planes
  int red_flip = 0;
  for (int tile = t_begin, it = 0; tile < t_end; ++tile, ++it) {
    const int s = it % a.stages;
    const int g = tile / tiles_per_group, row0 = (tile % tiles_per_group) * rows_per_tile;
    const bool sh = g >= n_active;
    const int e = sh ? 0 : __ldcg(a.active + g);
    const int count = sh ? a.tokens : int(__ldcg(a.ranges + 2 * e));
    const int offset = sh ? 0 : int(__ldcg(a.ranges + 2 * e + 1));
    const uint8_t* slab = smem + s * L.stage_bytes + size_t(rgi * 32) * a.pitch;
    const uint8_t* const rows[4] = {slab + size_t(lane >> 2) * a.pitch, slab + size_t((lane >> 2) + 8) * a.pitch,
                                    slab + size_t((lane >> 2) + 16) * a.pitch, slab + size_t((lane >> 2) + 24) * a.pitch};
    bool waited = false;
    for (int c0 = 0; c0 < count; c0 += TT) {
      const int nt = min(TT, count - c0);
      int arow[TT], xrow[TT];       // assignment index and activation row of each token of this chunk
#pragma unroll
      for (int t = 0; t < TT; ++t) {
        const int i = c0 + (t < nt ? t : 0);
        const int as = sh ? routed + i : int(__ldcg(a.assignments + offset + i));
        arow[t] = as;
        xrow[t] = a.x_by_assignment ? as : (sh ? i : as / a.topk);
      }
      long long key = 0;
#pragma unroll
      for (int t = 0; t < TT; ++t) key = key * 1000003ll + xrow[t] + 1;
      if (key != loaded_key) {          // uniform over the CTA: every warp computes the same key
        // ---- stage the activation rows as digit planes --------------------------------------------
#pragma unroll
        for (int t = 0; t < TT; ++t) {
          const float4* src = reinterpret_cast<const float4*>(a.x + size_t(xrow[t]) * a.k);
          const int n4 = a.k / 4;
          float m = 0.f;
          for (int i = tid; i < n4; i += nthr) {
            const float4 v = __ldcg(src + i);
            m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
          }
          m = warp_max(m);
          named_barrier(1, nthr);         // previous planes / bmax are no longer read
          if (lane == 0) bmax[warp] = m;
          named_barrier(1, nthr);
          float smax = 0.f;
          for (int w = 0; w < NW; ++w) smax = fmaxf(smax, bmax[w]);
          if (!(smax > 0.f)) smax = 1.f;
          const float inv = 127.f / smax;
          constexpr int GROUP = FMT == kFmtQ4K ? 8 : 4;          // float4 chunks per sub-block sum
          for (int base = 0; base < n4; base += nthr) {          // uniform trip count: shuffles below
            const int i = base + tid;
            const float4 v = i < n4 ? __ldcg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            int d0[3], d1[3], d2[3], d3[3];
            digits3(v.x, inv, d0); digits3(v.y, inv, d1); digits3(v.z, inv, d2); digits3(v.w, inv, d3);
            if (i < n4) {
#pragma unroll
              for (int p = 0; p < kDigits; ++p)
                *reinterpret_cast<uint32_t*>(dig + (size_t(t) * kDigits + p) * a.k + 4 * i) =
                    (uint32_t(d0[p]) & 0xffu) | ((uint32_t(d1[p]) & 0xffu) << 8) | ((uint32_t(d2[p]) & 0xffu) << 16) |
                    ((uint32_t(d3[p]) & 0xffu) << 24);
            }
            float p = (v.x + v.y) + (v.z + v.w);
            p += __shfl_xor_sync(0xffffffffu, p, 1);
            p += __shfl_xor_sync(0xffffffffu, p, 2);
            if (GROUP == 8) p += __shfl_xor_sync(0xffffffffu, p, 4);
            if (i < n4 && (i % GROUP) == 0) sums[i / GROUP] = p;
          }
          named_barrier(1, nthr);
          // the sums are bounded by (32 or 16) * smax: digits against that bound
          const float sbound = smax * float(GROUP * 4);
          const float sinv = 127.f / sbound;
          for (int i = tid; i < nsum; i += nthr) {
            int ds[3];
            digits3(sums[i], sinv, ds);
#pragma unroll
            for (int p = 0; p < kDigits; ++p) sdig[(size_t(t) * kDigits + p) * nsum + i] = uint8_t(ds[p]);
          }
          if (tid == 0) {
            xscale[2 * t] = smax / 127.f;
            xscale[2 * t + 1] = sbound / 127.f;
          }
        }
        named_barrier(1, nthr);
        loaded_key = key;
      }
      if (!waited) {
        if (lane == 0 && !mbar_wait(full + s, (it / a.stages) & 1, a.status)) *abort_flag = 1;
        __syncwarp();
        waited = true;
      }
      float facc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int b = kw; b < a.nblk; b += a.ks) {
        if (FMT == kFmtQ4K) q4k_block<TT>(rows, b, xp, lane, facc);
        else q6k_block<TT>(rows, b, a.nblk, xp, lane, facc);
      }
      // lanes j and j^1 hold the two column pairs of one token: add them; lane j = 2t then owns token t
#pragma unroll
      for (int i = 0; i < 4; ++i) facc[i] += __shfl_xor_sync(0xffffffffu, facc[i], 1);
      float* rbuf = red + red_flip * (NW * TT * 32);
      {
        const int j = lane & 3, t = j >> 1, gq = lane >> 2;
        if ((j & 1) == 0 && t < TT) {
#pragma unroll
          for (int i = 0; i < 4; ++i) rbuf[(warp * TT + t) * 32 + (i >> 1) * 16 + (i & 1) * 8 + gq] = facc[i];
        }
      }
      if (c0 + TT >= count) {           // last use of this stage: hand it back to the producer
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
      }
      named_barrier(2, nthr);
      if (*abort_flag) return;          // a wait ran out somewhere: every warp leaves here together
      if (kw == 0) {
#pragma unroll
        for (int t = 0; t < TT; ++t) {
          float v = 0.f;
          for (int q = 0; q < a.ks; ++q) v += rbuf[((rgi * a.ks + q) * TT + t) * 32 + lane];
          if (DUAL) {
            const float u = __shfl_down_sync(0xffffffffu, v, 16);
            const int r = row0 + rgi * 16 + lane;
            if (lane < 16 && r < a.rows && t < nt) a.out[size_t(arow[t]) * a.rows + r] = ACT == kActSilu ? silu_mul(v, u) : 0.f;
          } else {
            const int r = row0 + rgi * 32 + lane;
            if (r < a.rows && t < nt) a.out[size_t(arow[t]) * a.rows + r] = v;
          }
        }
      }
      red_flip ^= 1;
    }
    if (count == 0) {                   // an empty group still has to hand its stage back
      if (lane == 0) {
        if (!mbar_wait(full + s, (it / a.stages) & 1, a.status)) *abort_flag = 1;
        mbar_arrive(empty + s);
      }
      __syncwarp();
    }
  }
}

}  // namespace dmoe
