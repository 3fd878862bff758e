// Prefill / large-batch expert products: ragged grouped GEMM over block-scaled FP8 (e4m3) operands on the
// 5th-generation tensor cores.
//   out[row][n] = sum_kb (A[row][kb*128 .. +128] . W_e[n][kb*128 .. +128]) * sa[row][kb] * sw_e[n/128][kb]
// A: the token rows of every expert, gathered in dispatch order, e4m3 with one float32 scale per row and 128
// columns; W: e4m3 with one float32 scale per 128x128 block (hayate `Fp8Block`, cpu/glm53.rs:23-24).
// One CTA computes a 128-row x 128-column output tile of one expert:
//   warp 0    TMA producer: cp.async.bulk.tensor 2D loads (128B swizzle) of the A and W tiles of one 128-wide
//             K block per stage into a 6-stage shared-memory ring (mbarrier full/empty)
//   warp 1    issues tcgen05.mma kind::f8f6f4 (M128 N128 K32, four per K block) into one of four TMEM
//             accumulator buffers and commits to the ring / accumulator barriers
//   warps 2-9 epilogue: two warps per TMEM lane quarter, 64 columns each; tcgen05.ld the K block's partial tile
//             (one TMEM lane = one row per thread), multiply by the block scales and add into float32 registers
//             (packed f32x2 fma); after the last K block apply SwiGLU (gate/up mode: columns 0-63 are gate rows,
//             64-127 the matching up rows; a warp owns 32 gate columns and their 32 up columns) and store
// Every wait is bounded; a timeout sets a status bit, the CTA drains, frees its TMEM and returns.
// Replaces hayate cu/glm53/grouped.cu:59-124 (CUTLASS Sm80 grouped GEMM on restored bf16 weights) and
// packed_grouped.cu:177-266 (mma.sync grouped GEMM); the FP8 activation path has no reference counterpart.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace dmoe {

constexpr int kG8Stages = 6;
constexpr int kG8TileM = 128, kG8TileN = 128, kG8TileK = 128;
constexpr int kG8StageBytes = kG8TileM * kG8TileK + kG8TileN * kG8TileK;     // A tile + W tile, one byte per element
constexpr int kG8Threads = 320;          // TMA warp, MMA warp, 8 epilogue warps
constexpr int kG8AccBufs = 4;            // TMEM accumulator buffers of 128 columns

struct G8Args {
  const float* sa;             // [rows_total][K/128]
  const float* sw[2];          // per expert [N_w/128][K/128]; [1]: the up matrix in gate/up mode
  unsigned long long sw_expert_stride;   // floats
  const unsigned* ranges;      // [E][2] rows, offset (in dispatch order)
  int experts, n, k;           // n: output columns of the tile grid (gate/up: inter, i.e. 64 gate + 64 up rows per tile)
  int gate_up;                 // 1: W tile = 64 gate rows + 64 up rows, output silu(g)*u [rows][n] bf16
  __nv_bfloat16* out_bf16;     // gate/up mode
  float* out_f32;              // plain mode [rows_total][n]
  unsigned* status;
};

DEVI void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
// K-major operand tile, rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
DEVI uint64_t umma_desc_k128(uint32_t smem_addr) {
  return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f8f6f4, e4m3 x e4m3 -> f32, both K-major, M = 128, N = 128
constexpr uint32_t kIdescE4m3M128N128 = (1u << 4) | (uint32_t(kG8TileN >> 3) << 17) | (uint32_t(kG8TileM >> 4) << 24);
DEVI void umma_f8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(kIdescE4m3M128N128), "r"(accumulate), "r"(0u) : "memory");
}
DEVI void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
DEVI void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DEVI void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
DEVI void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
DEVI void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// tile index -> (expert, first row of the tile inside the expert, first output column)
struct G8Tile { int expert, m0, n0, rows, offset; };

__global__ void __launch_bounds__(kG8Threads, 1)
grouped_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w0,
                   const __grid_constant__ CUtensorMap map_w1, const G8Args a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full[kG8Stages], empty[kG8Stages], tfull[kG8AccBufs], tempty[kG8AccBufs];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int ends[1025];
  __shared__ volatile int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntile_n = a.n / (a.gate_up ? 64 : 128);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kG8Stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < kG8AccBufs; ++b) { mbar_init(tfull + b, 1); mbar_init(tempty + b, 256); }
    mbar_fence_init();
  }
  if (warp == 1) {       // TMEM: all 512 columns = four accumulator buffers
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();
  pdl_launch();
  // cumulative tile counts per expert
  if (threadIdx.x == 0) {
    int sum = 0;
    for (int e = 0; e < a.experts; ++e) {
      sum += int((__ldcg(a.ranges + 2 * e) + 127u) / 128u) * ntile_n;
      ends[e] = sum;
    }
    ends[a.experts] = sum;
  }
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const int total = ends[a.experts];
  const int kblocks = a.k / 128;
  auto locate = [&](int tile) {
    int lo = 0, hi = a.experts;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (tile < ends[mid]) hi = mid; else lo = mid + 1; }
    const int local = tile - (lo ? ends[lo - 1] : 0);
    G8Tile t;
    t.expert = lo;
    t.rows = int(__ldcg(a.ranges + 2 * lo));
    t.offset = int(__ldcg(a.ranges + 2 * lo + 1));
    t.m0 = (local / ntile_n) * 128;
    t.n0 = (local % ntile_n) * (a.gate_up ? 64 : 128);
    return t;
  };

  if (warp == 0) {
    // ---- TMA producer ------------------------------------------------------------------------------------
    if (lane == 0) {
      int it = 0;
      for (int tile = blockIdx.x; tile < total && !abort_flag; tile += gridDim.x) {
        const G8Tile t = locate(tile);
        const int wrow = t.expert * (a.gate_up ? a.n : a.n) + t.n0;       // row of the weight tensor [E*N][K]
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kG8Stages;
          if (it >= kG8Stages && !mbar_wait(empty + s, ((it / kG8Stages) & 1) ^ 1, a.status)) { abort_flag = 1; break; }
          const uint32_t dst = smem_u32(smem + s * kG8StageBytes);
          mbar_arrive_expect_tx(full + s, kG8StageBytes);
          tma_load_2d(dst, &map_a, kb * 128, t.offset + t.m0, full + s);
          if (a.gate_up) {
            tma_load_2d(dst + kG8TileM * kG8TileK, &map_w0, kb * 128, wrow, full + s);
            tma_load_2d(dst + kG8TileM * kG8TileK + 64 * kG8TileK, &map_w1, kb * 128, wrow, full + s);
          } else {
            tma_load_2d(dst + kG8TileM * kG8TileK, &map_w0, kb * 128, wrow, full + s);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----------------------------------------------------------------------------------------
    if (lane == 0) {
      int it = 0, acc_it = 0;
      for (int tile = blockIdx.x; tile < total && !abort_flag; tile += gridDim.x) {
        for (int kb = 0; kb < kblocks; ++kb, ++it, ++acc_it) {
          const int s = it % kG8Stages, buf = acc_it & (kG8AccBufs - 1);
          if (acc_it >= kG8AccBufs && !mbar_wait(tempty + buf, ((acc_it / kG8AccBufs) & 1) ^ 1, a.status)) { abort_flag = 1; break; }
          if (!mbar_wait(full + s, (it / kG8Stages) & 1, a.status)) { abort_flag = 1; break; }
          tmem_fence_after();
          const uint32_t sa = smem_u32(smem + s * kG8StageBytes), sb = sa + kG8TileM * kG8TileK;
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sb);
#pragma unroll
          for (int k = 0; k < kG8TileK / 32; ++k) umma_f8(tmem_base + buf * 128, da + 2 * k, db + 2 * k, k > 0 ? 1u : 0u);
          umma_commit(empty + s);          // the ring stage is free once these MMAs have read it
          umma_commit(tfull + buf);        // and the partial tile is complete
        }
        if (abort_flag) break;
      }
    }
  } else {
    // ---- epilogue: thread = one row of the tile, 64 of its 128 columns -----------------------------------------
    const int quarter = warp & 3;                       // TMEM lanes 32*quarter .. +31 belong to this warp
    const int half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const int col0 = a.gate_up ? 32 * half : 64 * half, col1 = a.gate_up ? 64 + 32 * half : 64 * half + 32;
    int acc_it = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      const G8Tile t = locate(tile);
      const int grow = t.offset + t.m0 + row_in_tile;   // row in the gathered activation / output arrays
      const bool valid = t.m0 + row_in_tile < t.rows;
      const float* sa_row = a.sa + size_t(grow) * kblocks;
      const float* sw0 = a.sw[0] + size_t(t.expert) * a.sw_expert_stride + size_t(t.n0 / 128) * kblocks;
      const float* sw1 = a.gate_up ? a.sw[1] + size_t(t.expert) * a.sw_expert_stride + size_t(t.n0 / 128) * kblocks : sw0;
      float2 acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = make_float2(0.f, 0.f);
      bool ok = true;
      for (int kb = 0; kb < kblocks; ++kb, ++acc_it) {
        const int buf = acc_it & (kG8AccBufs - 1);
        const float s_row = valid ? __ldg(sa_row + kb) : 0.f;
        const float f0 = s_row * __ldg(sw0 + kb), f1 = s_row * __ldg(sw1 + kb);
        if (ok && !mbar_wait(tfull + buf, (acc_it / kG8AccBufs) & 1, a.status)) { abort_flag = 1; ok = false; }
        if (!ok) continue;
        tmem_fence_after();
        const uint32_t taddr = tmem_base + buf * 128 + (uint32_t(quarter * 32) << 16);
        uint32_t v0[32], v1[32];
        tmem_ld32_issue(taddr + col0, v0);
        tmem_ld32_issue(taddr + col1, v1);
        tmem_ld_wait();
        tmem_fence_before();
        mbar_arrive(tempty + buf);                      // the values are in registers: the buffer may be overwritten
        const float2 p0 = make_float2(f0, f0), p1 = make_float2(f1, f1);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          acc[i] = __ffma2_rn(make_float2(__uint_as_float(v0[2 * i]), __uint_as_float(v0[2 * i + 1])), p0, acc[i]);
          acc[16 + i] = __ffma2_rn(make_float2(__uint_as_float(v1[2 * i]), __uint_as_float(v1[2 * i + 1])), p1, acc[16 + i]);
        }
      }
      if (ok && valid) {
        if (a.gate_up) {
          __nv_bfloat16* dst = a.out_bf16 + size_t(grow) * a.n + t.n0 + 32 * half;
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            uint4 o;
            uint32_t* w = &o.x;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(silu_mul(acc[i + j].x, acc[16 + i + j].x), silu_mul(acc[i + j].y, acc[16 + i + j].y));
              w[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(dst + 2 * i) = o;
          }
        } else {
          float* dst = a.out_f32 + size_t(grow) * a.n + t.n0 + 64 * half;
#pragma unroll
          for (int i = 0; i < 32; i += 2) *reinterpret_cast<float4*>(dst + 2 * i) = make_float4(acc[i].x, acc[i].y, acc[i + 1].x, acc[i + 1].y);
        }
      }
      if (!ok) break;
    }
  }
  tmem_fence_before();
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}

}  // namespace dmoe
