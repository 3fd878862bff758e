// Prefill / large-batch expert products: ragged grouped GEMM over block-scaled FP8 (e4m3) operands on the
// 5th-generation tensor cores.
//   out[row][n] = sum_kb (A[row][kb*128 .. +128] . W_e[n][kb*128 .. +128]) * sa[row][kb] * sw_e[n/128][kb]
// A: the token rows of every expert, gathered in dispatch order, e4m3 with one float32 scale per row and 128
// columns; W: e4m3 with one float32 scale per 128x128 block (hayate `Fp8Block`, cpu/glm53.rs:23-24).
// One CTA computes a tile of 128 token rows x 256 weight rows of one expert (gate/up modes: 128 gate rows and the
// 128 matching up rows, i.e. 128 columns of the SwiGLU product):
//   warp 0     TMA producer: cp.async.bulk.tensor 2D loads (128B swizzle) of the A tile and the two W half tiles
//              of one 128-wide K block per stage into a 4-stage shared-memory ring (mbarrier full/empty)
//   warp 1     issues tcgen05.mma kind::f8f6f4 (M128 N256 K32, four per K block; N = 256 is the shape that keeps
//              the tensor pipe fed from shared memory) into one of two TMEM accumulator buffers of 256 columns and
//              commits to the ring / accumulator barriers
//   warps 4-11 epilogue, two warps per TMEM lane quarter with 128 columns each: tcgen05.ld the K block's partial
//              tile (one TMEM lane = one row per thread) 16 columns at a time, multiply by the block scales and add
//              into float32 registers ; after the last K block SwiGLU and one of three stores (float32, bf16, or e4m3 codes +
//              scale per row and 128 columns), staged through shared memory so that rows leave in 64-byte pieces
// The producer/MMA warpgroup gives registers to the two epilogue warpgroups (setmaxnreg).
// Every wait is bounded; a timeout sets a status bit, the CTA drains, frees its TMEM and returns.
// Replaces hayate cu/glm53/grouped.cu:59-124 (CUTLASS Sm80 grouped GEMM on restored bf16 weights) and
// packed_grouped.cu:177-266 (mma.sync grouped GEMM); the FP8 activation path has no reference counterpart.
#pragma once
#include <cuda.h>
#include <cuda_fp8.h>
#include "common.cuh"

namespace dmoe {

constexpr int kG8Stages = 4;
constexpr int kG8TileM = 128, kG8TileN = 256, kG8TileK = 128;
constexpr int kG8StageBytes = kG8TileM * kG8TileK + kG8TileN * kG8TileK;     // A tile + W tile, one byte per element
constexpr int kG8Threads = 384;          // warpgroup 0: TMA warp, MMA warp, two idle warps; warpgroups 1-2: epilogue
constexpr int kG8AccBufs = 2;            // TMEM accumulator buffers of 256 columns
constexpr int kG8StagePitch = 80;        // bytes per row of a warp's store staging (64 + 16: conflict-free 16-byte rows)
constexpr int kG8StoreBytes = 8 * 32 * kG8StagePitch;
constexpr int kG8MaxExperts = 1024;
constexpr int kG8MaxStagedK = 64;        // K blocks whose weight scales a warp keeps in shared memory (K <= 8192)
constexpr int kG8FixedSmem = 1024 + kG8Stages * kG8StageBytes + kG8StoreBytes + 8 * 2 * kG8MaxStagedK * 4;   // + (experts + 1) ints

enum G8Mode { kG8Plain = 0, kG8GateUpBf16 = 1, kG8GateUpFp8 = 2 };

struct G8Args {
  const float* sa;             // [rows_total][K/128]
  const float* sw[2];          // per expert [N_w/128][K/128]; [1]: the up matrix in gate/up modes
  unsigned long long sw_expert_stride;   // floats
  const unsigned* ranges;      // [E][2] rows, offset (in dispatch order)
  int experts, n, k;           // n: output columns (gate/up modes: the intermediate width)
  int mode;                    // G8Mode
  float* out_f32;              // plain: [rows_total][n]
  __nv_bfloat16* out_bf16;     // gate/up bf16: silu(g)*u [rows_total][n]
  uint8_t* out_codes;          // gate/up fp8: e4m3(bf16(silu(g)*u) / scale) [rows_total][n]
  float* out_scales;           //              scale [rows_total][n/128] = absmax/448 (1 for a zero group)
  const unsigned* out_row_map; // optional (plain): output row of dispatch row i is out_row_map[i]
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
// kind::f8f6f4, e4m3 x e4m3 -> f32, both K-major, M = 128, N = 256
constexpr uint32_t kIdescE4m3 = (1u << 4) | (uint32_t(kG8TileN >> 3) << 17) | (uint32_t(kG8TileM >> 4) << 24);
DEVI void umma_f8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(kIdescE4m3), "r"(accumulate), "r"(0u) : "memory");
}
DEVI void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
DEVI void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DEVI void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 16 columns of this warp's 32 TMEM lanes -> registers, complete on return (load and wait in one statement, so
// that no use of the registers can be scheduled between them)
DEVI void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
struct G8Tile { int expert, m0, n0, rows, offset; };

template <int MODE>
__global__ void __launch_bounds__(kG8Threads, 1)
grouped_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w0,
                   const __grid_constant__ CUtensorMap map_w1, const G8Args a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* store_stage = smem + kG8Stages * kG8StageBytes;
  float* sw_stage = reinterpret_cast<float*>(store_stage + kG8StoreBytes);  // per epilogue warp 2 x kG8MaxStagedK weight scales
  int* ends = reinterpret_cast<int*>(sw_stage + 8 * 2 * kG8MaxStagedK);     // [experts + 1] cumulative tile counts
  __shared__ uint64_t full[kG8Stages], empty[kG8Stages], tfull[kG8AccBufs], tempty[kG8AccBufs], xbar[4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ float row_amax[2][128];
  __shared__ volatile int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr bool gate_up = MODE != kG8Plain;
  const int ntile_n = gate_up ? a.n / 128 : (a.n + 255) / 256;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kG8Stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < kG8AccBufs; ++b) { mbar_init(tfull + b, 1); mbar_init(tempty + b, 8); }   // tempty: one arrival per epilogue warp
    for (int q = 0; q < 4; ++q) mbar_init(xbar + q, 2);
    mbar_fence_init();
  }
  if (warp == 1) {       // TMEM: all 512 columns = two accumulator buffers
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();
  pdl_launch();
  // cumulative tile counts per expert: per-thread counts, then an inclusive scan (32 experts per lane of warp 0)
  for (int e = threadIdx.x; e < a.experts; e += kG8Threads) ends[e] = int((__ldcg(a.ranges + 2 * e) + 127u) / 128u) * ntile_n;
  __syncthreads();
  if (warp == 0) {
    const int per = (a.experts + 31) / 32;
    int sum = 0;
    for (int i = 0; i < per; ++i) { const int e = lane * per + i; if (e < a.experts) sum += ends[e]; }
    int run = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, run, o); if (lane >= o) run += t; }
    int off = run - sum;
    for (int i = 0; i < per; ++i) { const int e = lane * per + i; if (e < a.experts) { off += ends[e]; ends[e] = off; } }
    if (lane == 31) ends[a.experts] = run;
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
    t.n0 = (local % ntile_n) * (gate_up ? 128 : 256);
    return t;
  };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0 && lane == 0) {
      // ---- TMA producer ------------------------------------------------------------------------------------
      int it = 0;
      for (int tile = blockIdx.x; tile < total && !abort_flag; tile += gridDim.x) {
        const G8Tile t = locate(tile);
        const int wrow = t.expert * a.n + t.n0;                              // row of the weight tensor [E*N][K]
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kG8Stages;
          if (it >= kG8Stages && !mbar_wait_suspend(empty + s, ((it / kG8Stages) & 1) ^ 1, a.status)) { abort_flag = 1; break; }
          const uint32_t dst = smem_u32(smem + s * kG8StageBytes);
          mbar_arrive_expect_tx(full + s, kG8StageBytes);
          tma_load_2d(dst, &map_a, kb * 128, t.offset + t.m0, full + s);
          tma_load_2d(dst + kG8TileM * kG8TileK, &map_w0, kb * 128, wrow, full + s);
          if (gate_up) tma_load_2d(dst + kG8TileM * kG8TileK + 128 * kG8TileK, &map_w1, kb * 128, wrow, full + s);
          else tma_load_2d(dst + kG8TileM * kG8TileK + 128 * kG8TileK, &map_w0, kb * 128, wrow + 128, full + s);
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ---- MMA issuer ----------------------------------------------------------------------------------------
      int it = 0;
      for (int tile = blockIdx.x; tile < total && !abort_flag; tile += gridDim.x) {
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kG8Stages, buf = it & (kG8AccBufs - 1);
          if (it >= kG8AccBufs && !mbar_wait_suspend(tempty + buf, ((it / kG8AccBufs) & 1) ^ 1, a.status)) { abort_flag = 1; break; }
          if (!mbar_wait_suspend(full + s, (it / kG8Stages) & 1, a.status)) { abort_flag = 1; break; }
          tmem_fence_after();
          const uint32_t sa = smem_u32(smem + s * kG8StageBytes), sb = sa + kG8TileM * kG8TileK;
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sb);
#pragma unroll
          for (int k = 0; k < kG8TileK / 32; ++k) umma_f8(tmem_base + buf * 256, da + 2 * k, db + 2 * k, k > 0 ? 1u : 0u);
          umma_commit(empty + s);          // the ring stage is free once these MMAs have read it
          umma_commit(tfull + buf);        // and the partial tile is complete
        }
        if (abort_flag) break;
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ---- epilogue: thread = one row of the tile, 128 of its 256 accumulator columns ---------------------------------
    const int quarter = warp & 3;                       // TMEM lanes 32*quarter .. +31 belong to this warp
    const int half = (warp - 4) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    // accumulator columns of the four 32-column loads of a step
    const int colA = gate_up ? 64 * half : 128 * half;              // loads 0, 1: colA, colA + 32
    const int colB = gate_up ? 128 + 64 * half : 128 * half + 64;   // loads 2, 3: colB, colB + 32
    uint8_t* my_stage = store_stage + (warp - 4) * 32 * kG8StagePitch;
    // Steps = (tile, K block) pairs of this CTA in order.
    const int my_tiles = total > int(blockIdx.x) ? (total - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    const int steps = my_tiles * kblocks;
    const uint32_t tlane = tmem_base + (uint32_t(quarter * 32) << 16);
    bool ok = true;
    uint32_t va[16];
    auto await_step = [&](int step) {                   // the MMAs of this step have written their TMEM buffer
      const int buf = step & (kG8AccBufs - 1);
      // one lane watches the barrier (many threads probing one barrier word serialise in shared memory)
      int got = 1;
      if (lane == 0) got = mbar_wait_suspend(tfull + buf, (step / kG8AccBufs) & 1, a.status) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) { abort_flag = 1; ok = false; return; }
      tmem_fence_after();
    };
    int tile = blockIdx.x, kb = 0, tile_it = 0;
    G8Tile t = {};
    int grow0 = 0;                                      // dispatch row of this warp's first TMEM lane
    bool valid = false;
    bool cols = true;                                   // this thread's columns exist (plain mode, n not a multiple of 256)
    float2 acc[64];
    // Row scales: the 32 lanes read 32 different cache lines and the first touch of a line comes from HBM, so they
    // are fetched four K blocks at a time, one group ahead of their use. Weight scales (the same for the whole
    // warp): lanes fetch the next tile's values while this tile runs and park them in shared memory when it opens.
    const bool vec = (kblocks & 3) == 0, sw_staged = kblocks <= kG8MaxStagedK;
    float* my_sw = sw_stage + (warp - 4) * 2 * kG8MaxStagedK;
    float4 cur_r = make_float4(0.f, 0.f, 0.f, 0.f), nxt_r = cur_r;
    float pend_a[2] = {0.f, 0.f}, pend_b[2] = {0.f, 0.f};
    auto sw_ptr = [&](const G8Tile& tt, int which) {
      const float* base = a.sw[gate_up ? which : 0] + size_t(tt.expert) * a.sw_expert_stride;
      const int block = gate_up ? tt.n0 / 128 : (tt.n0 + 128 * half < a.n ? tt.n0 / 128 + half : 0);
      return base + size_t(block) * kblocks;
    };
    auto fetch_row4 = [&](const G8Tile& tt, int kb0) {
      const float* p = a.sa + size_t(tt.offset + tt.m0 + row_in_tile) * kblocks;
      if (vec) { nxt_r = __ldg(reinterpret_cast<const float4*>(p + kb0)); return; }
      nxt_r = make_float4(0.f, 0.f, 0.f, 0.f);
      if (kb0 < kblocks) nxt_r.x = __ldg(p + kb0);
      if (kb0 + 1 < kblocks) nxt_r.y = __ldg(p + kb0 + 1);
      if (kb0 + 2 < kblocks) nxt_r.z = __ldg(p + kb0 + 2);
      if (kb0 + 3 < kblocks) nxt_r.w = __ldg(p + kb0 + 3);
    };
    auto fetch_sw = [&](const G8Tile& tt) {
      if (!sw_staged) return;
      const float *pa = sw_ptr(tt, 0), *pb = sw_ptr(tt, 1);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (lane + 32 * j < kblocks) { pend_a[j] = __ldg(pa + lane + 32 * j); pend_b[j] = __ldg(pb + lane + 32 * j); }
    };
    auto pick = [&](const float4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; };
    auto open_tile = [&]() {                             // `t` holds the tile; its scales were fetched ahead
      grow0 = t.offset + t.m0 + quarter * 32;
      valid = t.m0 + row_in_tile < t.rows;
      cols = gate_up || t.n0 + 128 * half < a.n;
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = make_float2(0.f, 0.f);
      if (sw_staged) {
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 2; ++j)
          if (lane + 32 * j < kblocks) { my_sw[lane + 32 * j] = pend_a[j]; my_sw[kG8MaxStagedK + lane + 32 * j] = pend_b[j]; }
        __syncwarp();
      }
    };
    // Writes 64 bytes per row of this warp's 32 rows: every lane puts its row's piece into the staging area, then
    // the rows leave as four 16-byte parts, 8 rows per store instruction.
    auto store_rows = [&](uint8_t* out_base, size_t row_bytes, size_t col_byte, const uint4 (&piece)[4]) {
      uint4* mine = reinterpret_cast<uint4*>(my_stage + lane * kG8StagePitch);
#pragma unroll
      for (int j = 0; j < 4; ++j) mine[j] = piece[j];
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i * 8 + (lane >> 2), part = lane & 3;
        if (t.m0 + quarter * 32 + r < t.rows) {
          const size_t orow = a.out_row_map ? size_t(__ldg(a.out_row_map + grow0 + r)) : size_t(grow0 + r);
          *reinterpret_cast<uint4*>(out_base + orow * row_bytes + col_byte + part * 16) =
              *reinterpret_cast<const uint4*>(my_stage + r * kG8StagePitch + part * 16);
        }
      }
      __syncwarp();
    };
    auto close_tile = [&]() {
      if (MODE == kG8Plain) {
        if (!cols) return;
#pragma unroll
        for (int c = 0; c < 8; ++c) {                    // 8 pieces of 16 float32
          uint4 piece[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            piece[j] = make_uint4(__float_as_uint(acc[c * 8 + 2 * j].x), __float_as_uint(acc[c * 8 + 2 * j].y),
                                  __float_as_uint(acc[c * 8 + 2 * j + 1].x), __float_as_uint(acc[c * 8 + 2 * j + 1].y));
          store_rows(reinterpret_cast<uint8_t*>(a.out_f32), size_t(a.n) * 4, size_t(t.n0 + 128 * half) * 4 + c * 64, piece);
        }
        return;
      }
      // SwiGLU product of this thread's 64 columns, rounded to bf16 (acc[i]: gate, acc[32 + i]: up)
      // two bf16 per word, kept as bits in acc[i].x (low half: even column)
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const uint32_t lo = __float_as_uint(__bfloat162float(__float2bfloat16_rn(silu_mul_fast(acc[i].x, acc[32 + i].x))));
        const uint32_t hi = __float_as_uint(__bfloat162float(__float2bfloat16_rn(silu_mul_fast(acc[i].y, acc[32 + i].y))));
        acc[i].x = __uint_as_float((lo >> 16) | (hi & 0xffff0000u));
        amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(lo)), fabsf(__uint_as_float(hi))));
      }
      auto h = [&](int i) { return __float_as_uint(acc[i].x); };
      if (MODE == kG8GateUpBf16) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint4 piece[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) piece[j] = make_uint4(h(c * 16 + 4 * j), h(c * 16 + 4 * j + 1), h(c * 16 + 4 * j + 2), h(c * 16 + 4 * j + 3));
          store_rows(reinterpret_cast<uint8_t*>(a.out_bf16), size_t(a.n) * 2, size_t(t.n0 + 64 * half) * 2 + c * 64, piece);
        }
        return;
      }
      // e4m3 codes with one scale per row and 128 columns: the row's other 64 columns are in the partner warp
      row_amax[half][row_in_tile] = amax;
      __syncwarp();
      int got = 1;
      if (lane == 0) {
        mbar_arrive(xbar + quarter);
        got = mbar_wait_suspend(xbar + quarter, tile_it & 1, a.status) ? 1 : 0;
      }
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) { abort_flag = 1; ok = false; return; }
      amax = fmaxf(amax, row_amax[half ^ 1][row_in_tile]);
      const float scale = amax == 0.f ? 1.f : amax / 448.f;
      const float inv = 1.f / scale;
      uint4 piece[4];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint32_t bits = h(2 * i + j);
          const float q0 = fminf(fmaxf(__uint_as_float(bits << 16) * inv, -448.f), 448.f);
          const float q1 = fminf(fmaxf(__uint_as_float(bits & 0xffff0000u) * inv, -448.f), 448.f);
          w |= uint32_t((uint8_t)__nv_cvt_float_to_fp8(q0, __NV_SATFINITE, __NV_E4M3)) << (16 * j);
          w |= uint32_t((uint8_t)__nv_cvt_float_to_fp8(q1, __NV_SATFINITE, __NV_E4M3)) << (16 * j + 8);
        }
        if ((i & 3) == 0) piece[i >> 2].x = w;
        else if ((i & 3) == 1) piece[i >> 2].y = w;
        else if ((i & 3) == 2) piece[i >> 2].z = w;
        else piece[i >> 2].w = w;
      }
      if (half == 0 && valid) a.out_scales[size_t(grow0 + lane) * (a.n / 128) + t.n0 / 128] = scale;
      store_rows(a.out_codes, size_t(a.n), size_t(t.n0 + 64 * half), piece);
    };
    auto fma16 = [&](float f, int base) {                // acc[base .. base + 8) += va * f
#pragma unroll
      for (int i = 0; i < 8; ++i) {     // scalar fma: the packed f32x2 form measured slower here (operand pairing moves)
        acc[base + i].x = fmaf(__uint_as_float(va[2 * i]), f, acc[base + i].x);
        acc[base + i].y = fmaf(__uint_as_float(va[2 * i + 1]), f, acc[base + i].y);
      }
    };
    if (steps > 0) {
      t = locate(tile);
      fetch_row4(t, 0);
      fetch_sw(t);
      open_tile();
      await_step(0);
      for (int step = 0; step < steps && ok; ++step) {
        const uint32_t tbuf = tlane + (step & (kG8AccBufs - 1)) * 256;
        if ((kb & 3) == 0) {
          cur_r = nxt_r;
          if (kb + 4 < kblocks) {
            fetch_row4(t, kb + 4);
          } else if (tile + int(gridDim.x) < total) {    // the last group of this tile: look the next tile up
            const G8Tile nx = locate(tile + gridDim.x);
            fetch_row4(nx, 0);
            fetch_sw(nx);
          }
        }
        const float s_row = (valid && cols) ? pick(cur_r, kb & 3) : 0.f;
        const float wa = sw_staged ? my_sw[kb] : __ldg(sw_ptr(t, 0) + kb), wb = sw_staged ? my_sw[kG8MaxStagedK + kb] : __ldg(sw_ptr(t, 1) + kb);
        const float fA = s_row * wa, fB = s_row * wb;
        // eight 16-column loads (columns colA .. +64, colB .. +64); the partner warp of this scheduler partition
        // covers a load's latency with its adds. (Measured: 32-column loads into two alternating register sets, one
        // in flight while the other is consumed, made the kernel a fifth slower: 232 registers do not hold both sets
        // and the 128 accumulators.)
#pragma unroll
        for (int j = 0; j < 7; ++j) {
          tmem_ld16(tbuf + (j < 4 ? colA + 16 * j : colB + 16 * (j - 4)), va);
          fma16(j < 4 ? fA : fB, 8 * j);
        }
        tmem_ld16(tbuf + colB + 48, va);
        tmem_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty + (step & (kG8AccBufs - 1)));   // the values are in registers: the buffer may be overwritten
        fma16(fB, 56);
        if (step + 1 < steps) await_step(step + 1);
        if (++kb == kblocks) {
          close_tile();
          kb = 0;
          ++tile_it;
          tile += gridDim.x;
          if (tile < total) { t = locate(tile); open_tile(); }
        }
      }
    }
  }
  tmem_fence_before();
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}

}  // namespace dmoe
