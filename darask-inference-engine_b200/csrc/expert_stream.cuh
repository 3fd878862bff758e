// Decode-path expert products: quantized weight rows are streamed HBM -> shared memory by the
// TMA engine (bulk copies completing on mbarriers, a ring of stages per CTA) and dequantized in
// registers. One lane owns one weight row (so a row's scales are unpacked once and no cross-lane
// shuffle is needed), the warps of a row group split the 256-element blocks of K, activations
// sit in shared memory and are read as warp broadcasts.
//
// Work item ("tile") = one group of tokens that chose the same expert x a slab of rows of that
// expert. Persistent CTAs (one per SM) each take a contiguous range of tiles.
//   DUAL = 1: gate and up rows of the same index are streamed together, lanes 0-15 hold gate
//             rows and lanes 16-31 the matching up rows; the epilogue writes silu(g) * u.
//   DUAL = 0: plain rows (down projection).
// Replaces the reference's per-engine GEMV kernels (kogarashi kernels/native.cu:46-88 `gemv` +
// :97-99 `activate`; tsumuji kernels/decode/gemv.cu:64-158; hayate cu/glm53/decode.cu:37-54).
#pragma once
#include "common.cuh"

namespace dmoe {

enum StreamFormat { kFmtQ4K = 0, kFmtQ6KR = 1, kFmtNvfp4Linear = 2, kFmtNvfp4Tiled = 3, kFmtFp8Block = 4, kFmtBf16 = 5 };
enum Activation { kActSilu = 0, kActHayate = 1 };

constexpr int kMaxStages = 4;

struct StreamArgs {
  const uint8_t* w[2];          // routed experts: matrix 0 (gate or down) and matrix 1 (up)
  const uint8_t* w_shared[2];   // shared expert matrices (null when there is none)
  unsigned long long expert_stride[2];   // bytes between consecutive experts
  int row_bytes;                // bytes of one row in global memory (multiple of 16)
  int pitch;                    // bytes of one row slot in shared memory (odd multiple of 16)
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

// ---- per-format block dot products -------------------------------------------------------------
// All take a pointer to this lane's row slot in shared memory and accumulate the dot product of
// block `b` (256 columns) with TT activation rows `xs[t * kx + column]`.

DEVI float2 f2(float a, float b) { return make_float2(a, b); }

// GGUF Q4_K, 144 bytes per block: d, dmin (f16), twelve 6-bit scale/min bytes, 128 nibble bytes.
// value = (d * sc) * q - dmin * m  (kogarashi kernels/native.cu:26-34). The mins are applied to
// per-32 sums of x (`xsum`), the nibbles through exact small-integer floats.
template <int TT>
DEVI void q4k_block(const uint8_t* row, int b, const float* xs, int kx, const float* xsum, int sx, float (&acc)[TT]) {
  const uint8_t* blk = row + b * 144;
  const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
  const float d = half_lo(hdr.x), dmin = half_hi(hdr.x);
  const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, mn_lo = hdr.z & 0x3F3F3F3Fu;
  const uint32_t sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
  const uint32_t mn_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
  float dsc[8], dm[8];
  dsc[0] = (byte_magic<0>(sc_lo) - kMagic) * d; dsc[1] = (byte_magic<1>(sc_lo) - kMagic) * d;
  dsc[2] = (byte_magic<2>(sc_lo) - kMagic) * d; dsc[3] = (byte_magic<3>(sc_lo) - kMagic) * d;
  dsc[4] = (byte_magic<0>(sc_hi) - kMagic) * d; dsc[5] = (byte_magic<1>(sc_hi) - kMagic) * d;
  dsc[6] = (byte_magic<2>(sc_hi) - kMagic) * d; dsc[7] = (byte_magic<3>(sc_hi) - kMagic) * d;
  dm[0] = (byte_magic<0>(mn_lo) - kMagic) * dmin; dm[1] = (byte_magic<1>(mn_lo) - kMagic) * dmin;
  dm[2] = (byte_magic<2>(mn_lo) - kMagic) * dmin; dm[3] = (byte_magic<3>(mn_lo) - kMagic) * dmin;
  dm[4] = (byte_magic<0>(mn_hi) - kMagic) * dmin; dm[5] = (byte_magic<1>(mn_hi) - kMagic) * dmin;
  dm[6] = (byte_magic<2>(mn_hi) - kMagic) * dmin; dm[7] = (byte_magic<3>(mn_hi) - kMagic) * dmin;
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    const float4 s0 = *reinterpret_cast<const float4*>(xsum + t * sx + b * 8);
    const float4 s1 = *reinterpret_cast<const float4*>(xsum + t * sx + b * 8 + 4);
    float m = dm[0] * s0.x;
    m = fmaf(dm[1], s0.y, m); m = fmaf(dm[2], s0.z, m); m = fmaf(dm[3], s0.w, m);
    m = fmaf(dm[4], s1.x, m); m = fmaf(dm[5], s1.y, m); m = fmaf(dm[6], s1.z, m); m = fmaf(dm[7], s1.w, m);
    acc[t] -= m;
  }
  const float2 neg = f2(-kMagic, -kMagic);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 q = *reinterpret_cast<const uint4*>(blk + 16 + 16 * c);
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
    const int gp = c >> 1;
    const float* xl = xs + b * 256 + gp * 64 + (c & 1) * 16;
    float2 slo[TT], shi[TT];
#pragma unroll
    for (int t = 0; t < TT; ++t) slo[t] = shi[t] = f2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lo = words[i] & 0x0F0F0F0Fu, hi = words[i] & 0xF0F0F0F0u;   // hi holds 16 * q
      const float2 l01 = __fadd2_rn(f2(byte_magic<0>(lo), byte_magic<1>(lo)), neg);
      const float2 l23 = __fadd2_rn(f2(byte_magic<2>(lo), byte_magic<3>(lo)), neg);
      const float2 h01 = __fadd2_rn(f2(byte_magic<0>(hi), byte_magic<1>(hi)), neg);
      const float2 h23 = __fadd2_rn(f2(byte_magic<2>(hi), byte_magic<3>(hi)), neg);
#pragma unroll
      for (int t = 0; t < TT; ++t) {
        const float4 a = *reinterpret_cast<const float4*>(xl + t * kx + 4 * i);
        const float4 e = *reinterpret_cast<const float4*>(xl + t * kx + 32 + 4 * i);
        slo[t] = __ffma2_rn(l01, f2(a.x, a.y), slo[t]);
        slo[t] = __ffma2_rn(l23, f2(a.z, a.w), slo[t]);
        shi[t] = __ffma2_rn(h01, f2(e.x, e.y), shi[t]);
        shi[t] = __ffma2_rn(h23, f2(e.z, e.w), shi[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      acc[t] = fmaf(dsc[2 * gp], slo[t].x + slo[t].y, acc[t]);
      acc[t] = fmaf(dsc[2 * gp + 1] * 0.0625f, shi[t].x + shi[t].y, acc[t]);
    }
  }
}

// GGUF Q6_K in the row-aligned device layout ("Q6_K-R16"): a row is nblk x [ql 128 | qh 64 |
// int8 scales 16] followed by nblk f16 `d` (padded to 16 bytes); the same bits as the 210-byte
// GGUF blocks, regrouped so that every block starts on a 16-byte boundary.
// value = (d * scale) * (q - 32)  (kogarashi kernels/native.cu:35-40).
template <int TT>
DEVI void q6k_block(const uint8_t* row, int b, int nblk, const float* xs, int kx, float (&acc)[TT]) {
  const uint8_t* blk = row + b * 208;
  const float d = __half2float(*reinterpret_cast<const __half*>(row + nblk * 208 + 2 * b));
  const uint4 sv = *reinterpret_cast<const uint4*>(blk + 192);
  const uint32_t sw[4] = {sv.x ^ 0x80808080u, sv.y ^ 0x80808080u, sv.z ^ 0x80808080u, sv.w ^ 0x80808080u};
  float dsc[16];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    dsc[4 * i + 0] = (byte_magic<0>(sw[i]) - (kMagic + 128.f)) * d;
    dsc[4 * i + 1] = (byte_magic<1>(sw[i]) - (kMagic + 128.f)) * d;
    dsc[4 * i + 2] = (byte_magic<2>(sw[i]) - (kMagic + 128.f)) * d;
    dsc[4 * i + 3] = (byte_magic<3>(sw[i]) - (kMagic + 128.f)) * d;
  }
  const float2 neg = f2(-(kMagic + 32.f), -(kMagic + 32.f));
#pragma unroll
  for (int n = 0; n < 2; ++n) {
#pragma unroll
    for (int lh = 0; lh < 2; ++lh) {        // columns l = 16 * lh .. + 15 of each 32-group
      const uint4 hq = *reinterpret_cast<const uint4*>(blk + 128 + 16 * (2 * n + lh));
      const uint32_t hw[4] = {hq.x, hq.y, hq.z, hq.w};
#pragma unroll
      for (int gb = 0; gb < 2; ++gb) {      // low nibbles: group gb, high nibbles: group gb + 2
        const uint4 lq = *reinterpret_cast<const uint4*>(blk + 16 * (4 * n + 2 * gb + lh));
        const uint32_t lw[4] = {lq.x, lq.y, lq.z, lq.w};
        const float* xl = xs + b * 256 + n * 128 + gb * 32 + lh * 16;
        float2 slo[TT], shi[TT];
#pragma unroll
        for (int t = 0; t < TT; ++t) slo[t] = shi[t] = f2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t lo = (lw[i] & 0x0F0F0F0Fu) | ((hw[i] << (4 - 2 * gb)) & 0x30303030u);
          const uint32_t hi = ((lw[i] >> 4) & 0x0F0F0F0Fu) | ((hw[i] >> (2 * gb)) & 0x30303030u);
          const float2 l01 = __fadd2_rn(f2(byte_magic<0>(lo), byte_magic<1>(lo)), neg);
          const float2 l23 = __fadd2_rn(f2(byte_magic<2>(lo), byte_magic<3>(lo)), neg);
          const float2 h01 = __fadd2_rn(f2(byte_magic<0>(hi), byte_magic<1>(hi)), neg);
          const float2 h23 = __fadd2_rn(f2(byte_magic<2>(hi), byte_magic<3>(hi)), neg);
#pragma unroll
          for (int t = 0; t < TT; ++t) {
            const float4 a = *reinterpret_cast<const float4*>(xl + t * kx + 4 * i);
            const float4 e = *reinterpret_cast<const float4*>(xl + t * kx + 64 + 4 * i);
            slo[t] = __ffma2_rn(l01, f2(a.x, a.y), slo[t]);
            slo[t] = __ffma2_rn(l23, f2(a.z, a.w), slo[t]);
            shi[t] = __ffma2_rn(h01, f2(e.x, e.y), shi[t]);
            shi[t] = __ffma2_rn(h23, f2(e.z, e.w), shi[t]);
          }
        }
#pragma unroll
        for (int t = 0; t < TT; ++t) {
          acc[t] = fmaf(dsc[8 * n + 2 * gb + lh], slo[t].x + slo[t].y, acc[t]);
          acc[t] = fmaf(dsc[8 * n + 2 * (gb + 2) + lh], shi[t].x + shi[t].y, acc[t]);
        }
      }
    }
  }
}

template <int FMT, int TT>
DEVI void block_dot(const uint8_t* row, int b, const StreamArgs& a, const float* xs, const float* xsum, float (&acc)[TT]) {
  if (FMT == kFmtQ4K) q4k_block<TT>(row, b, xs, a.k, xsum, a.k / 32, acc);
  else if (FMT == kFmtQ6KR) q6k_block<TT>(row, b, a.nblk, xs, a.k, acc);
}

// Shared-memory carve-up, shared by host (size) and device (offsets).
struct StreamSmem {
  int stage_bytes, x_off, xsum_off, red_off, bar_off, total;
};
__host__ __device__ inline StreamSmem stream_smem(int rg, int ks, int stages, int pitch, int k, int tt, bool xsum) {
  StreamSmem s;
  s.stage_bytes = 32 * rg * pitch;
  s.x_off = stages * s.stage_bytes;
  s.xsum_off = s.x_off + tt * k * 4;
  s.red_off = s.xsum_off + (xsum ? tt * (k / 32) * 4 : 0);
  s.bar_off = s.red_off + 2 * rg * ks * tt * 32 * 4;
  s.total = s.bar_off + 2 * kMaxStages * 8 + 16;
  return s;
}

template <int FMT, int DUAL, int TT, int ACT>
__global__ void __launch_bounds__(544, 1) expert_stream_kernel(const StreamArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int NW = a.rg * a.ks;                       // compute warps; warp NW is the producer
  const StreamSmem L = stream_smem(a.rg, a.ks, a.stages, a.pitch, a.k, TT, FMT == kFmtQ4K);
  float* xs = reinterpret_cast<float*>(smem + L.x_off);
  float* xsum = reinterpret_cast<float*>(smem + L.xsum_off);
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
      for (int j = lane; j < 32 * a.rg; j += 32) {
        const int rgi = j >> 5, l = j & 31;
        const int m = DUAL ? (l >> 4) : 0;
        const int r = DUAL ? rgi * 16 + (l & 15) : j;
        if (r < valid) {
          const uint8_t* base = sh ? a.w_shared[m] : a.w[m] + size_t(e) * a.expert_stride[m];
          bulk_g2s(stage + size_t(j) * a.pitch, base + size_t(row0 + r) * a.row_bytes, a.row_bytes, full + s);
        }
      }
    }
    return;
  }

  // ---- consumers ---------------------------------------------------------------------------------
  const int rgi = warp / a.ks, kw = warp % a.ks;
  const int nthr = NW * 32, tid = threadIdx.x;
  long long loaded_key = -1;       // which activation rows sit in xs
  int red_flip = 0;
  for (int tile = t_begin, it = 0; tile < t_end; ++tile, ++it) {
    const int s = it % a.stages;
    const int g = tile / tiles_per_group, row0 = (tile % tiles_per_group) * rows_per_tile;
    const bool sh = g >= n_active;
    const int e = sh ? 0 : __ldcg(a.active + g);
    const int count = sh ? a.tokens : int(__ldcg(a.ranges + 2 * e));
    const int offset = sh ? 0 : int(__ldcg(a.ranges + 2 * e + 1));
    const uint8_t* rowp = smem + s * L.stage_bytes + size_t(rgi * 32 + lane) * a.pitch;
    bool waited = false;
    for (int c0 = 0; c0 < count; c0 += TT) {
      const int nt = min(TT, count - c0);
      // assignment index and activation row of each token of this chunk
      int arow[TT], xrow[TT];
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
        named_barrier(1, nthr);         // everyone is done reading the previous rows
#pragma unroll
        for (int t = 0; t < TT; ++t) {
          const float4* src = reinterpret_cast<const float4*>(a.x + size_t(xrow[t]) * a.k);
          float4* dst = reinterpret_cast<float4*>(xs + t * a.k);
          const int n4 = a.k / 4;
          for (int base = 0; base < n4; base += nthr) {     // uniform trip count: shuffles below
            const int i = base + tid;
            const float4 v = i < n4 ? __ldcg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < n4) dst[i] = v;
            if (FMT == kFmtQ4K) {
              // 8 consecutive lanes cover 32 columns: their sum is the per-sub-block sum of x
              float p = (v.x + v.y) + (v.z + v.w);
              p += __shfl_xor_sync(0xffffffffu, p, 1);
              p += __shfl_xor_sync(0xffffffffu, p, 2);
              p += __shfl_xor_sync(0xffffffffu, p, 4);
              if (i < n4 && (i & 7) == 0) xsum[t * (a.k / 32) + (i >> 3)] = p;
            }
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
      float acc[TT];
#pragma unroll
      for (int t = 0; t < TT; ++t) acc[t] = 0.f;
      for (int b = kw; b < a.nblk; b += a.ks) block_dot<FMT, TT>(rowp, b, a, xs, xsum, acc);
      float* rbuf = red + red_flip * (NW * TT * 32);
#pragma unroll
      for (int t = 0; t < TT; ++t) rbuf[(warp * TT + t) * 32 + lane] = acc[t];
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
          for (int j = 0; j < a.ks; ++j) v += rbuf[((rgi * a.ks + j) * TT + t) * 32 + lane];
          if (DUAL) {
            const float u = __shfl_down_sync(0xffffffffu, v, 16);
            const int r = row0 + rgi * 16 + lane;
            if (lane < 16 && r < a.rows && t < nt) {
              float h;
              if (ACT == kActSilu) h = silu_mul(v, u);
              else h = 0.f;
              a.out[size_t(arow[t]) * a.rows + r] = h;
            }
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
