// Ragged grouped GEMM that reads the experts' packed NVFP4 images in place, on the 5th-generation tensor cores.
//   gate/up: product[row][c] = swiglu(bf16(x[row] . gate[c] * s_gate), bf16(x[row] . up[c] * s_up))    (bf16)
//   down:    out[row][c]     = bf16(product[row] . down[c] * s_down)                                   (bf16)
// for the rows of every expert, float32 accumulation in TMEM over the whole K extent. No bf16 copy of the weights ever
// exists in HBM: four warps read the e2m1 codes (32 bytes per row and 64-column K block) and the e4m3 block scales
// (one 32-bit word per row and K block: the tiled scale layout keeps the four scales of 64 columns together) of the
// tile's 256 weight rows straight from the image, multiply code by scale (exact in bf16: 3 x 4 significant bits) and
// write bf16 into the 128-byte-swizzled shared-memory tile the MMA descriptor expects; the per-matrix float32 scale is
// applied in the epilogue, as the reference does. Roles and tile scheduler as in grouped_bf16.cuh:
//   warp 1      MMA issuer (one elected lane): tcgen05.mma kind::f16, 128 x 256 x 16 per instruction
//   warps 2-3   activation loaders (16-byte cp.async copies of the valid rows into the swizzled tile)
//   warps 4-11  epilogue, once per tile, overlapping the next tile's MMAs through the second TMEM buffer
//   warps 0, 12-14  weight expanders (global -> registers one K block ahead -> bf16 -> shared memory)
// A gate/up tile holds 128 gate rows and the 128 matching up rows, so the SwiGLU runs in the epilogue on one thread's
// registers. Image layout (hayate cu/glm53/lowbit.cuh:9-13, packed_grouped.cu:13-36): per matrix [n][k/2] codes, then
// 128 x 64 scale tiles, then the float32 tensor scale; gate, up, down follow each other at a 256-byte-aligned stride.
// Replaces hayate cu/glm53/packed_grouped.cu:177-318 (`grouped<DOWN,C>`: cp.async + mma.sync.m16n8k16).
#pragma once
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "expert_gemv.cuh"
#include "grouped_bf16.cuh"

namespace dmoe {

constexpr int kGnThreads = 480;                                // 15 warps
constexpr int kGnExpanders = 4;
constexpr int kGnPitch = 80;                                   // epilogue staging row: 64 bytes of bf16 + 16 (bank phase)
constexpr int kGnStoreBytes = 8 * 32 * kGnPitch;               // 8 warps x 32 rows
constexpr int kGnFixedSmem = 1024 + kGbStages * kGbStageBytes + kGnStoreBytes;   // + (groups + 1) ints

struct HayateMatrixFormat { unsigned char format, grid, group, reserved; };     // lowbit.cuh:5
struct HayateExpertFormat { HayateMatrixFormat gate_up, down; };                 // lowbit.cuh:6

constexpr unsigned kStatusBadFormat = 8u;     // an expert image is not NVFP4 (or its pointer is null): its rows are zero

struct GnArgs {
  const __nv_bfloat16* x;            // [rows][k]
  const void* const* images;         // device array: one image per expert
  const HayateExpertFormat* formats; // device array
  const unsigned* ranges;            // [count][2] rows, offset
  int count, hidden, inter;
  __nv_bfloat16* out;                // [rows][n]
  unsigned* status;                  // optional device status word
};

// bytes of one NVFP4 matrix image and the stride between the matrices of an expert (lowbit.cuh:9-13)
DEVI size_t nvfp4_storage(unsigned n, unsigned k) { return size_t(n) * k / 2 + size_t((n + 127) / 128 * 128) * (k / 16) + 4; }
DEVI size_t nvfp4_stride(unsigned n, unsigned k) { return (nvfp4_storage(n, k) + 255) / 256 * 256; }

// eight e2m1 codes (one 32-bit word, low nibble first) times one e4m3 scale -> eight bf16 values
DEVI uint4 expand8(uint32_t codes, __half2 scale) {
  uint32_t w[4];
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const __half2_raw raw = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>((codes >> (8 * b)) & 255u), __NV_E2M1);
    const __half2 v = __hmul2(static_cast<__half2>(raw), scale);          // exact
    const __nv_bfloat162 p = __float22bfloat162_rn(__half22float2(v));     // exact
    w[b] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
DEVI __half2 e4m3_to_half2(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte & 255u), __NV_E4M3);
  return __half2half2(static_cast<__half>(h));
}

template <bool DOWN>
__global__ void __launch_bounds__(kGnThreads, 1) grouped_nvfp4_kernel(const GnArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* store_stage = smem + kGbStages * kGbStageBytes;
  int* ends = reinterpret_cast<int*>(store_stage + kGnStoreBytes);
  __shared__ uint64_t full[kGbStages], empty[kGbStages], tfull[2], tempty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ unsigned local_status;
  __shared__ volatile int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = DOWN ? a.hidden : a.inter, k = DOWN ? a.inter : a.hidden;
  constexpr int TN = DOWN ? 256 : 128;                           // output columns per tile
  const int ntile_n = n / TN;
  unsigned* status = a.status ? a.status : &local_status;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    local_status = 0;
    for (int s = 0; s < kGbStages; ++s) { mbar_init(full + s, 2 + kGnExpanders); mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull + b, 1); mbar_init(tempty + b, 8); }
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();
  pdl_launch();
  if (threadIdx.x == 0) {
    int sum = 0;
    for (int g = 0; g < a.count; ++g) { sum += int((__ldcg(a.ranges + 2 * g) + 127u) / 128u) * ntile_n; ends[g] = sum; }
    ends[a.count] = sum;
  }
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const int total = ends[a.count];
  const int kblocks = k / kGbTileK;
  auto locate = [&](int tile) {
    int g = 0;
    while (g < a.count - 1 && tile >= ends[g]) ++g;
    const int local = tile - (g ? ends[g - 1] : 0);
    G8Tile t;
    t.expert = g;
    t.rows = int(__ldcg(a.ranges + 2 * g));
    t.offset = int(__ldcg(a.ranges + 2 * g + 1));
    t.m0 = (local / ntile_n) * 128;
    t.n0 = (local % ntile_n) * TN;
    return t;
  };
  // the matrix this kernel multiplies with, inside an expert's image: [gate | up | down] at one stride
  const size_t step = nvfp4_stride(unsigned(a.inter), unsigned(a.hidden));
  const size_t scales_at = size_t(n) * k / 2;                    // scale tiles follow the codes

  if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer: all K blocks of a tile accumulate in one TMEM buffer ------------------------------------
      int it = 0, tile_it = 0;
      for (int tile = blockIdx.x; tile < total && !abort_flag; tile += gridDim.x, ++tile_it) {
        const int buf = tile_it & 1;
        if (tile_it >= 2 && !mbar_wait_suspend(tempty + buf, ((tile_it >> 1) & 1) ^ 1, status)) { abort_flag = 1; break; }
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kGbStages;
          if (!mbar_wait_suspend(full + s, (it / kGbStages) & 1, status)) { abort_flag = 1; break; }
          tmem_fence_after();
          const uint32_t sa = smem_u32(smem + s * kGbStageBytes), sb = sa + 128 * 128;
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sb);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem_base + buf * 256, da + 2 * kk, db + 2 * kk, (kb | kk) ? 1u : 0u);
          umma_commit(empty + s);
        }
        if (abort_flag) break;
        umma_commit(tfull + buf);
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ---- activation loaders: 64 rows each, 16-byte cp.async copies into the swizzled tile, two stages in flight ----
    const int lw = warp - 2;
    int it = 0, signalled = 0;
    bool ok = true;
    auto signal_oldest = [&](int pending_allowed) {
      if (pending_allowed == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(full + (signalled % kGbStages));
      ++signalled;
    };
    for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
      const G8Tile t = locate(tile);
      for (int kb = 0; kb < kblocks && ok; ++kb, ++it) {
        const int s = it % kGbStages;
        int got = 1;
        if (it >= kGbStages && lane == 0) got = mbar_wait_suspend(empty + s, ((it / kGbStages) & 1) ^ 1, status) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) { abort_flag = 1; ok = false; break; }
        const uint32_t tile_smem = smem_u32(smem + s * kGbStageBytes);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int idx = j * 32 + lane, r = lw * 64 + (idx >> 3), c = idx & 7;      // row of the tile, 16-byte chunk
          const bool valid = t.m0 + r < t.rows;
          const __nv_bfloat16* src = a.x + size_t(t.offset + t.m0 + (valid ? r : 0)) * k + kb * kGbTileK + c * 8;
          cp_async16_zfill(tile_smem + r * 128 + ((c ^ (r & 7)) << 4), src, valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (it >= 1) signal_oldest(1);
      }
    }
    while (signalled < it) signal_oldest(0);
  } else if (warp == 0 || warp >= 12) {
    // ---- weight expanders: 128 threads, four half rows (32 columns) of the 256-row tile each per K block ----------
    const int et = (warp == 0 ? 0 : warp - 11) * 32 + lane;               // 0 .. 127
    struct Piece { uint4 codes; uint32_t scales; };
    Piece cur[4], nxt[4];
    int tile = blockIdx.x, kb = 0;
    G8Tile t = {};
    const uint8_t* image = nullptr;
    bool bad_format = false;
    auto open_tile = [&]() {
      t = locate(tile);
      image = reinterpret_cast<const uint8_t*>(__ldcg(reinterpret_cast<const unsigned long long*>(a.images) + t.expert));
      const HayateExpertFormat ef = a.formats[t.expert];
      bad_format = (DOWN ? ef.down.format : ef.gate_up.format) != 0 || image == nullptr;     // only NVFP4 images
      if (bad_format && lane == 0) atomicOr(status, kStatusBadFormat);
    };
    auto fetch = [&](Piece (&p)[4]) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int hidx = j * 128 + et, r = hidx >> 1, half = hidx & 1;
        // rows 0-127 of a gate/up tile are gate rows, rows 128-255 the matching up rows
        const uint8_t* mat = image + (DOWN ? 2 * step : (r >= 128 ? step : 0));
        const unsigned row = unsigned(t.n0 + (DOWN ? r : (r & 127)));
        if (bad_format) {
          p[j].codes = make_uint4(0u, 0u, 0u, 0u);
          p[j].scales = 0u;
        } else {
          p[j].codes = __ldg(reinterpret_cast<const uint4*>(mat + (size_t(row) * k + kb * kGbTileK + half * 32) / 2));
          p[j].scales = __ldg(reinterpret_cast<const uint32_t*>(mat + scales_at + (size_t(row / 128) * (k / 64) + kb) * 512 + (row % 32) * 16 +
                                                                 (row % 128 / 32) * 4));
        }
      }
    };
    bool ok = tile < total;
    if (ok) {
      open_tile();
      fetch(cur);
    }
    for (int it = 0; ok; ++it) {
      // the next K block's bytes are requested before this one is expanded
      int ntile = tile, nkb = kb + 1;
      if (nkb == kblocks) { nkb = 0; ntile += gridDim.x; }
      const bool more = ntile < total;
      if (more) {
        if (ntile != tile) { tile = ntile; kb = 0; open_tile(); } else { kb = nkb; }
        fetch(nxt);
      }
      const int s = it % kGbStages;
      int got = 1;
      if (it >= kGbStages && lane == 0) got = mbar_wait_suspend(empty + s, ((it / kGbStages) & 1) ^ 1, status) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got || abort_flag) { abort_flag = 1; break; }
      const uint32_t wt = smem_u32(smem + s * kGbStageBytes) + 128 * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int hidx = j * 128 + et, r = hidx >> 1, half = hidx & 1;
        const uint32_t sc = cur[j].scales >> (16 * half);
        const __half2 s0 = e4m3_to_half2(sc), s1 = e4m3_to_half2(sc >> 8);
        const uint32_t cw[4] = {cur[j].codes.x, cur[j].codes.y, cur[j].codes.z, cur[j].codes.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 v = expand8(cw[q], q < 2 ? s0 : s1);
          const int c = half * 4 + q;
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(wt + r * 128 + ((c ^ (r & 7)) << 4)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                       : "memory");
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(full + s);
      if (!more) break;
#pragma unroll
      for (int j = 0; j < 4; ++j) cur[j] = nxt[j];
    }
  } else {
    // ---- epilogue: thread = one row of the tile; warps 4-7 take the first half of the output columns, 8-11 the second ----
    const int quarter = warp & 3, half = (warp - 4) >> 2;
    uint8_t* my_stage = store_stage + (warp - 4) * 32 * kGnPitch;
    const uint32_t tlane = tmem_base + (uint32_t(quarter * 32) << 16);
    int tile_it = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++tile_it) {
      const G8Tile t = locate(tile);
      const int buf = tile_it & 1;
      int got = 1;
      if (lane == 0) got = mbar_wait_suspend(tfull + buf, (tile_it >> 1) & 1, status) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) { abort_flag = 1; break; }
      tmem_fence_after();
      const uint8_t* image = reinterpret_cast<const uint8_t*>(__ldcg(reinterpret_cast<const unsigned long long*>(a.images) + t.expert));
      const size_t tail = nvfp4_storage(unsigned(n), unsigned(k)) - 4;                  // the float32 tensor scale ends a matrix
      float s_main = 0.f, s_up = 0.f;
      if (image) {
        s_main = __ldg(reinterpret_cast<const float*>(image + (DOWN ? 2 * step : 0) + tail));
        if (!DOWN) s_up = __ldg(reinterpret_cast<const float*>(image + step + tail));
      }
      const int grow0 = t.offset + t.m0 + quarter * 32;
      constexpr int PIECES = TN / 2 / 32;                          // pieces of 32 output columns per thread: 4 (down) or 2 (gate/up)
#pragma unroll 1
      for (int c = 0; c < PIECES; ++c) {
        const int col_in_tile = (TN / 2) * half + 32 * c;         // first output column of the piece inside the tile
        uint4* mine = reinterpret_cast<uint4*>(my_stage + lane * kGnPitch);
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {                           // 16 columns at a time
          uint32_t v0[16], v1[16];
          tmem_ld16(tlane + buf * 256 + col_in_tile + 16 * h2, v0);
          if (!DOWN) tmem_ld16(tlane + buf * 256 + 128 + col_in_tile + 16 * h2, v1);
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float r0 = bf16_rn(__uint_as_float(v0[2 * j]) * s_main), r1 = bf16_rn(__uint_as_float(v0[2 * j + 1]) * s_main);
            if (!DOWN) {
              r0 = hayate_swiglu(r0, bf16_rn(__uint_as_float(v1[2 * j]) * s_up));
              r1 = hayate_swiglu(r1, bf16_rn(__uint_as_float(v1[2 * j + 1]) * s_up));
            }
            const __nv_bfloat162 p = __floats2bfloat162_rn(r0, r1);
            w[j] = *reinterpret_cast<const uint32_t*>(&p);
          }
          mine[2 * h2] = make_uint4(w[0], w[1], w[2], w[3]);
          mine[2 * h2 + 1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
        __syncwarp();
        const int col = t.n0 + col_in_tile;
#pragma unroll
        for (int i = 0; i < 4; ++i) {                              // 32 rows x 64 bytes leave as 16-byte pieces, four lanes per row
          const int r = i * 8 + (lane >> 2), part = lane & 3;
          if (t.m0 + quarter * 32 + r < t.rows)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.out) + (size_t(grow0 + r) * n + col) * 2 + part * 16) =
                *reinterpret_cast<const uint4*>(my_stage + r * kGnPitch + part * 16);
        }
        __syncwarp();
      }
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty + buf);
    }
  }
  tmem_fence_before();
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}

}  // namespace dmoe
