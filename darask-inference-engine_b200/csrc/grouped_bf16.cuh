// Ragged grouped GEMM over bf16 operands on the 5th-generation tensor cores: out[row][n] = x[row][:] . w_g[n][:]
// for the rows of every group g, float32 accumulation in TMEM over the whole K extent.
// Same tile scheduler and roles as grouped_fp8.cuh, with two differences:
//   * the accumulator stays in TMEM for all K blocks of a tile (no per-block scales), so the epilogue runs once
//     per tile and overlaps the next tile's MMAs through the second TMEM buffer;
//   * the caller's interface gives no bound on the total number of rows, so the activation tile is not loaded
//     by TMA (a box may not run past the end of the allocation): warps 2-3 fetch the valid rows with 16-byte
//     cp.async copies into the 128-byte-swizzled layout the MMA descriptor expects; the weight tile is a TMA box.
// Replaces hayate cu/glm53/grouped.cu:59-124 (`hayate_glm_grouped`, `hayate_glm_grouped_nvfp4`: CUTLASS Sm80
// grouped GEMM, bf16 mma.sync).
#pragma once
#include "grouped_fp8.cuh"

namespace dmoe {

constexpr int kGbStages = 4;
constexpr int kGbTileK = 64;                                   // bf16 elements = 128 bytes per row
constexpr int kGbStageBytes = 128 * 128 + 256 * 128;           // A 128 rows + W 256 rows of 128 bytes
constexpr int kGbThreads = 384;
constexpr int kGbStoreBytes = 8 * 32 * kG8StagePitch;
constexpr int kGbFixedSmem = 1024 + kGbStages * kGbStageBytes + kGbStoreBytes;   // + (groups + 1) ints

struct GbArgs {
  const __nv_bfloat16* x;      // [rows][k], rows of group g at ranges[g][1]
  const unsigned* ranges;      // [groups][2] rows, offset
  int groups, n, k;
  __nv_bfloat16* out;          // [rows][n]
  float* acc;                  // optional: the float32 products before scaling, [rows][n]
  const float* scales;         // optional: out = bf16(acc * scales[g])
  unsigned* status;            // optional device status word
};

// kind::f16, bf16 x bf16 -> f32, both K-major, M = 128, N = 256
constexpr uint32_t kIdescBf16 = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(256 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
DEVI void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(kIdescBf16), "r"(accumulate), "r"(0u) : "memory");
}
DEVI void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16u : 0u) : "memory");
}

__global__ void __launch_bounds__(kGbThreads, 1)
grouped_bf16_kernel(const __grid_constant__ CUtensorMap map_w, const GbArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* store_stage = smem + kGbStages * kGbStageBytes;
  int* ends = reinterpret_cast<int*>(store_stage + kGbStoreBytes);
  __shared__ uint64_t full[kGbStages], empty[kGbStages], tfull[2], tempty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ unsigned local_status;
  __shared__ volatile int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntile_n = (a.n + 255) / 256;
  unsigned* status = a.status ? a.status : &local_status;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    local_status = 0;
    for (int s = 0; s < kGbStages; ++s) { mbar_init(full + s, 3); mbar_init(empty + s, 1); }   // full: TMA thread + two loader warps
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
    for (int g = 0; g < a.groups; ++g) { sum += int((__ldcg(a.ranges + 2 * g) + 127u) / 128u) * ntile_n; ends[g] = sum; }
    ends[a.groups] = sum;
  }
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const int total = ends[a.groups];
  const int kblocks = a.k / kGbTileK;
  auto locate = [&](int tile) {
    int g = 0;
    while (g < a.groups - 1 && tile >= ends[g]) ++g;
    const int local = tile - (g ? ends[g - 1] : 0);
    G8Tile t;
    t.expert = g;
    t.rows = int(__ldcg(a.ranges + 2 * g));
    t.offset = int(__ldcg(a.ranges + 2 * g + 1));
    t.m0 = (local / ntile_n) * 128;
    t.n0 = (local % ntile_n) * 256;
    return t;
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer: the weight tile (two boxes of 128 rows) ---------------------------------------------
      int it = 0;
      for (int tile = blockIdx.x; tile < total && !abort_flag; tile += gridDim.x) {
        const G8Tile t = locate(tile);
        const int wrow = t.expert * a.n + t.n0;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kGbStages;
          if (it >= kGbStages && !mbar_wait_suspend(empty + s, ((it / kGbStages) & 1) ^ 1, status)) { abort_flag = 1; break; }
          const uint32_t dst = smem_u32(smem + s * kGbStageBytes) + 128 * 128;
          mbar_arrive_expect_tx(full + s, 256 * 128);
          tma_load_2d(dst, &map_w, kb * kGbTileK, wrow, full + s);
          tma_load_2d(dst + 128 * 128, &map_w, kb * kGbTileK, wrow + 128, full + s);
        }
      }
    }
  } else if (warp == 1) {
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
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_base + buf * 256, da + 2 * k, db + 2 * k, (kb | k) ? 1u : 0u);
          umma_commit(empty + s);
        }
        if (abort_flag) break;
        umma_commit(tfull + buf);
      }
    }
  } else if (warp < 4) {
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
          const __nv_bfloat16* src = a.x + size_t(t.offset + t.m0 + (valid ? r : 0)) * a.k + kb * kGbTileK + c * 8;
          cp_async16_zfill(tile_smem + r * 128 + ((c ^ (r & 7)) << 4), src, valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (it >= 1) signal_oldest(1);
      }
    }
    while (signalled < it) signal_oldest(0);
  } else {
    // ---- epilogue: thread = one row of the tile, 128 of its 256 columns, once per tile ----------------------------
    const int quarter = warp & 3, half = (warp - 4) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    uint8_t* my_stage = store_stage + (warp - 4) * 32 * kG8StagePitch;
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
      const int grow0 = t.offset + t.m0 + quarter * 32;
      const bool cols = t.n0 + 128 * half < a.n;
      const float scale = a.scales ? __ldg(a.scales + t.expert) : 1.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {                      // 4 pieces of 32 columns: 64 bytes of bf16 per row
        uint32_t v0[16], v1[16];
        tmem_ld16(tlane + buf * 256 + 128 * half + 32 * c, v0);
        tmem_ld16(tlane + buf * 256 + 128 * half + 32 * c + 16, v1);
        if (!cols) continue;
        const int col = t.n0 + 128 * half + 32 * c;
        if (a.acc && t.m0 + row_in_tile < t.rows) {
          float4* dst = reinterpret_cast<float4*>(a.acc + size_t(grow0 + lane) * a.n + col);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            dst[i] = make_float4(__uint_as_float(v0[4 * i]), __uint_as_float(v0[4 * i + 1]), __uint_as_float(v0[4 * i + 2]), __uint_as_float(v0[4 * i + 3]));
            dst[4 + i] = make_float4(__uint_as_float(v1[4 * i]), __uint_as_float(v1[4 * i + 1]), __uint_as_float(v1[4 * i + 2]), __uint_as_float(v1[4 * i + 3]));
          }
        }
        uint4* mine = reinterpret_cast<uint4*>(my_stage + lane * kG8StagePitch);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          uint32_t w[4], u[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(v0[8 * i + 2 * j]) * scale, __uint_as_float(v0[8 * i + 2 * j + 1]) * scale);
            const __nv_bfloat162 q = __floats2bfloat162_rn(__uint_as_float(v1[8 * i + 2 * j]) * scale, __uint_as_float(v1[8 * i + 2 * j + 1]) * scale);
            w[j] = *reinterpret_cast<const uint32_t*>(&p);
            u[j] = *reinterpret_cast<const uint32_t*>(&q);
          }
          mine[i] = make_uint4(w[0], w[1], w[2], w[3]);
          mine[2 + i] = make_uint4(u[0], u[1], u[2], u[3]);
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = i * 8 + (lane >> 2), part = lane & 3;
          if (t.m0 + quarter * 32 + r < t.rows)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.out) + (size_t(grow0 + r) * a.n + col) * 2 + part * 16) =
                *reinterpret_cast<const uint4*>(my_stage + r * kG8StagePitch + part * 16);
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
