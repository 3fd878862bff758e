// One-token Kogarashi MoE FFN layer as ONE persistent launch (one CTA per SM), without grid-wide barriers.
//
//   phase R   every CTA projects its one or two router rows (fetched before the dependency wait) and publishes the
//             logits; a producer warp of every CTA collects all logits and selects the top-k itself (same result
//             everywhere), so no CTA waits for a routing block and no plan travels through global memory
//   phase 1   gate/up tiles (8 gate rows + the 8 matching up rows of one expert), SwiGLU products published as float32
//   phase 2   down tiles (16 rows of one expert), expert-major: a quad of warps stages the product vector of the
//             tile's expert (16-bit fixed point) and publishes the tile's rows as float32
//   combine   every CTA adds the weighted experts (slot order) and the gated shared expert into its share of the
//             residual stream
//
// What one CTA publishes for the others (logits, products, down rows) travels as 8-byte words {float, tag}, written
// with one 64-bit store each and read by polling (the scheme of low-latency collectives): the tag is derived from a
// call counter kept in the workspace, which every CTA reads at the start and CTA 0 advances at the end, so a word is
// valid exactly when its tag is this call's. A consumer therefore waits only for the values it needs: the experts'
// products become complete one after the other during phase 1 and the down tiles take the experts in the same
// order, so only the last tiles of a CTA can meet a product that is still being computed, and the weight stream runs
// through from the first gate row to the last down row. (Grid-wide barriers cost three L2 round trips each, about
// 2 us, three times per layer.)
//
// Producer threads issue ONE `cp.async.bulk` copy per chunk of
// whole, consecutive weight rows (8 gate rows, the 8 matching up rows, or 16 down rows: about 14 KB at the benchmark
// shape, contiguous in global memory; the copies of one thread are carried out one after the other at about half a
// microsecond each whatever their size, so two issuing threads are needed to keep HBM busy with chunks of this size)
// into a ring of chunk slots in a fixed order (shared expert first, then the routed experts, then the down tiles);
// while the gate/up tiles are being multiplied the ring refills with down weights, which depend on the routing only.
// A tile is multiplied by a quad of warps that take its 256-column blocks in turn (warp k: blocks k, k + 4, ...) and
// add their partial sums through shared memory. Inside the block loop the half-rate integer pipe that unpacks the codes
// is the busy one, not the tensor pipe: the activation fragments of a block are loaded once into registers, and the
// zero halves of the block-diagonal operand never travel through shared memory. (Measured on the whole kernel the
// block loop is a small part: with it compiled out the launch is 1.3 us shorter of 24; the time from the dependency
// wait to the first routed weight byte, about 6 us, and the per-tile hand-offs inside a quad are the larger parts.)
//
// Optionally the layer entry of the reference (`residual` + `rms_native`, native.cu:89-96) is part of phase R: every
// CTA forms u = (x + attn_out) * norm_w and the sum of squares of x + attn_out itself, multiplies the router rows with
// u and applies the norm's scale to logits and activations afterwards; CTA 0 writes n back.
//
// Arithmetic per 256-column block, `mma.sync.m16n8k32` on 8-bit integers (u8 weight codes x s8 activations, s32
// accumulate; the legacy tensor path issues one such instruction per 8 cycles and scheduler, twice the weights of the
// f16 shape, and the codes need no float conversion: the block loop is bound by the half-rate integer pipe that
// unpacks the codes, so instructions per weight are what counts). The activations are held as 16-bit fixed point of
// the largest magnitude inside their own scale group (32 columns for Q4_K, 16 for Q6_K): x ~ (256 hi + lo) / S with two
// signed bytes per value, error <= max|x over the group| / 64000 per value, so an outlier costs precision only among
// its own 15 or 31 neighbours; hi and lo are two columns of the B operand. B is block diagonal: the
// 32 k slots of an MMA belong to four different scale groups of the block and column pair s of the tile holds the
// activation bytes only in the eight slots of group s, so that column pair s of the accumulator is the exact integer
// code sum of scale group s; 1 / S of the group, the group scales, the Q4_K minimum (through per-group float sums of
// the activations) and the Q6_K code offset 32 (through per-group integer sums) are applied once per block and lane
// in float32.
//
// Replaces kogarashi kernels/native.cu:46-117 (`gemv`, `activate`, `route`, `combine`) for one token; formulas of the
// formats: native.cu:26-40 and :52-82.
#pragma once
#include "common.cuh"
#include "expert_gemv.cuh"
#include "route_impl.cuh"

namespace dmoe {

// Build-time knobs of the one-token kernel (measured: inlining everything is fastest; the waits neither gain nor lose
// from suspend hints or sleeps between probes).
#ifndef DMOE_HOT
#define DMOE_HOT DEVI
#endif
#ifndef DMOE_COLD
#define DMOE_COLD DEVI
#endif
#ifndef DMOE_ROUTE
#define DMOE_ROUTE DEVI
#endif
#ifndef DMOE_WAIT_HINT_NS
#define DMOE_WAIT_HINT_NS 10000
#endif
#ifndef DMOE_WAIT_SLEEP_NS
#define DMOE_WAIT_SLEEP_NS 64
#endif
#ifndef DMOE_FILL_SLEEP_NS
#define DMOE_FILL_SLEEP_NS 32
#endif

constexpr float kFixedPointRange = 32000.f;     // the largest magnitude of a scale group maps to this integer
constexpr unsigned kStatusActRange = 4u;   // an activation is not finite (the staged kernels: does not fit fp16 planes)

constexpr int kFusedConsumers = 16;                          // consumer warps
#ifndef DMOE_FUSED_PRODUCERS
#define DMOE_FUSED_PRODUCERS 2
#endif
constexpr int kFusedProducers = DMOE_FUSED_PRODUCERS;                           // warps that issue bulk copies (one thread each)
constexpr int kFusedThreads = (kFusedConsumers + kFusedProducers) * 32;
constexpr int kFusedSlots = 16;                              // partial-sum slots: a slot is reused 16 tiles later, further than the ring reaches
constexpr int kFusedMaxStages = 14;
constexpr int kFusedQuad = 4;                                // warps that share a tile
constexpr int kFusedPasses = 1;                              // 16-row MMA passes per tile: a tile is 8 gate + 8 up rows, or 16 down rows, per pass

struct FusedArgs {
  const float* router_w; const float* router_bias; const float* sh_inp;
  const uint8_t* gate_w; const uint8_t* up_w; const uint8_t* down_w;
  const uint8_t* sh_gate; const uint8_t* sh_up; const uint8_t* sh_down;
  const float* n; float* x; float* logits; int* ids; float* prob;
  // optional layer entry: x += attn_out, n = x * rsqrt(mean(x^2) + norm_eps) * norm_w, written to n_out by CTA 0
  const float* attn_out; const float* norm_w; float* n_out; float norm_eps;
  int H, F, E, K, G, has_shared, ldlog;
  int nblk1, row_bytes1, tps;                     // gate/up: 256-column blocks per row, bytes per row, tiles per group
  int nblk2, row_bytes2, rt2, down_q6;            // down: the same, row tiles of the output
  int stage_bytes, nstage;                        // chunk slot size and number of slots of the ring
  int off_bars, off_psum, off_log, off_act, off_ring;    // shared-memory offsets
  int act_lo1, act_xs1, act_rows;                 // phase R/1 inside the activation area: lo-plane offset, (sum, 1/S) pairs, router rows
  int act_q, act_qs, act_lo2, act_xs2;            // phase 2: first quad area, bytes per quad area; inside its planes: lo-plane offset, (sum, 1/S) pairs
  unsigned* status; unsigned* epoch; unsigned* seen;    // call counter of the workspace; CTAs of this call that have read it
  unsigned long long* tlog; unsigned long long* th; unsigned long long* ty;   // tagged: logits [CTA][ldlog], products [G][F], down rows [G][H]
};

// ---- small pieces -----------------------------------------------------------------------------------------
DEVI unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// ---- tagged words: {float value, 32-bit tag} in one 64-bit store --------------------------------------------------
DEVI unsigned make_tag(unsigned epoch) { return 0x80000001u + epoch % 0x7FFFFFFEu; }     // never 0, never the bits of -0.0f
DEVI void st_tagged(unsigned long long* p, float v, unsigned tag) {
  const unsigned long long w = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
DEVI unsigned long long ld_tagged(const unsigned long long* p) {
  unsigned long long w;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}
DEVI uint4 ld_tagged2(const unsigned long long* p) {          // two words: (value, tag, value, tag)
  unsigned long long w0, w1;
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(p) : "memory");
  return make_uint4(unsigned(w0), unsigned(w0 >> 32), unsigned(w1), unsigned(w1 >> 32));
}
// One poll site gives up after the time limit or when another role of the CTA has: status bit, abort flag, false.
struct PollClock {
  uint64_t start;
  uint32_t spin;
  DEVI PollClock() : start(0), spin(0) {}
  DMOE_COLD bool expired(unsigned* status, volatile int* abort_flag) {
    if ((++spin & 15u) != 0) return false;
    if (*abort_flag) return true;
    const uint64_t now = global_timer_ns();
    if (start == 0) start = now;
    else if (now - start > kWaitLimitNs) {
      atomicOr(status, kStatusWaitTimeout);
      *abort_flag = 1;
      return true;
    }
    __nanosleep(64);
    return false;
  }
};
// A warp collects entries lane, lane + 32, ... (< n <= 320) of a tagged array into `dst`. Uniform result.
DMOE_COLD bool gather_tagged(const unsigned long long* src, int n, unsigned tag, float* dst, int lane, unsigned* status, volatile int* abort_flag) {
  constexpr int MAXQ = 10;
  unsigned pend = 0;
#pragma unroll
  for (int q = 0; q < MAXQ; ++q)
    if (lane + 32 * q < n) pend |= 1u << q;
  PollClock clk;
  for (;;) {
    unsigned long long w[MAXQ];
#pragma unroll
    for (int q = 0; q < MAXQ; ++q)                    // all loads first: they are in flight together
      if (pend >> q & 1) w[q] = ld_tagged(src + lane + 32 * q);
#pragma unroll
    for (int q = 0; q < MAXQ; ++q)
      if ((pend >> q & 1) && unsigned(w[q] >> 32) == tag) {
        dst[lane + 32 * q] = __uint_as_float(unsigned(w[q]));
        pend &= ~(1u << q);
      }
    if (!__any_sync(0xffffffffu, pend != 0)) return true;
    int quit = (lane == 0 && clk.expired(status, abort_flag)) ? 1 : 0;
    quit = __shfl_sync(0xffffffffu, quit, 0);
    if (quit) return false;
  }
}
// One thread: up to eight entries base[q * stride], q < n, all in flight together.
DMOE_COLD bool poll_strided(const unsigned long long* base, size_t stride, int n, unsigned tag, float (&out)[8], unsigned* status, volatile int* abort_flag) {
  unsigned pend = (1u << n) - 1u;
  PollClock clk;
  for (;;) {
    unsigned long long w[8];
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (pend >> q & 1) w[q] = ld_tagged(base + q * stride);
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if ((pend >> q & 1) && unsigned(w[q] >> 32) == tag) {
        out[q] = __uint_as_float(unsigned(w[q]));
        pend &= ~(1u << q);
      }
    if (!pend) return true;
    if (clk.expired(status, abort_flag)) return false;
  }
}
// One thread: four consecutive entries as (v, t, v, t) x 2.
DMOE_COLD bool poll_four(const unsigned long long* p, unsigned tag, uint4& r0, uint4& r1, unsigned* status, volatile int* abort_flag) {
  PollClock clk;
  for (;;) {
    r0 = ld_tagged2(p);
    r1 = ld_tagged2(p + 2);
    if (r0.y == tag && r0.w == tag && r1.y == tag && r1.w == tag) return true;
    if (clk.expired(status, abort_flag)) return false;
  }
}
// mbarrier wait that also leaves when another role gave up
DMOE_HOT bool mbar_wait_abortable(uint64_t* bar, uint32_t parity, unsigned* status, volatile int* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  uint64_t start = 0;
  for (uint32_t spin = 0;; ++spin) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity), "r"(unsigned(DMOE_WAIT_HINT_NS))
        : "memory");
    if (ok) return true;
    if (*abort_flag) return false;
    if (DMOE_WAIT_SLEEP_NS) __nanosleep(DMOE_WAIT_SLEEP_NS);     // waiting warps leave the issue slots to the warps that have data
    if ((spin & 15u) == 0) {
      const uint64_t now = global_timer_ns();
      if (spin == 0) start = now;
      else if (now - start > kWaitLimitNs) {
        atomicOr(status, kStatusWaitTimeout);
        *abort_flag = 1;
        return false;
      }
    }
  }
}
DEVI float magic_u8(uint32_t v) { return __uint_as_float(0x4B000000u | v) - kMagic; }   // small unsigned integer -> float
DEVI float quad_sum(float v) {            // over the four lanes that share g = lane / 4
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

// Lane constants of the block-diagonal tiles. Lane = (g, j), g = lane / 4, j = lane % 4.
//   A side: lanes j = 0,1 supply k slots 0-3 (a0/a1) and 8-11 (a2/a3), lanes j = 2,3 slots 4-7 and 12-15.
//   B side: column g of the tile belongs to column pair s = g / 2 (plane g % 2); of this lane's two B registers only
//           the one whose slots lie in slot group s is non-zero, and only when j / 2 == s % 2.
//   D side: this lane holds columns 2j, 2j+1 = (hi, lo) sums of slot group j for rows g and g + 8.
struct DiagLane {
  int g, j;
  bool active, second;     // B: this lane carries activations; in b1 (slot groups 2, 3) instead of b0
  int plane;               // B: 0 hi, 1 lo
};
DEVI DiagLane diag_lane(int lane) {
  DiagLane d;
  d.g = lane >> 2; d.j = lane & 3;
  const int s = d.g >> 1;
  d.plane = d.g & 1;
  d.active = (d.j >> 1) == (s & 1);
  d.second = s >= 2;
  return d;
}

// The activation side of one 256-column block for this lane. pair[i] = the (b0, b1) operand registers of MMA i of
// the block. A lane carries real values in at most one of the two registers of a pair (always the same one) and zero
// in the other; which one is a property of the lane. The pairs are zeroed once per launch and a block load writes only
// the live half, straight into the register the MMA reads (predicated 32-bit loads: no zero fragments in shared
// memory, no register moves to assemble the operand).
//   xs[i]: the sum of the activations over the scale group this lane owns in tile i (Q4_K: float sum of x over a
//   sub-block; Q6_K: the integer sum of the fixed-point values over 16 columns, as a float); inv[i]: 1 / S of that group.
struct BlockFrags {
  uint2 pair[8];
  float xs[4], inv[4];
};
DEVI void frags_clear(BlockFrags& f) {
#pragma unroll
  for (int i = 0; i < 8; ++i) f.pair[i] = make_uint2(0u, 0u);
#pragma unroll
  for (int i = 0; i < 4; ++i) f.xs[i] = f.inv[i] = 0.f;
}
// Q4_K: tile t of a block covers sub-blocks 4t .. 4t+3; this lane's fragments of tile t are 16 activation bytes at
// xb + 128 t (natural column order); xs_addr: the eight (sum, 1 / S) pairs of the block.
DEVI void q4k_load_frags(BlockFrags& f, uint32_t xb, bool first, bool second, uint32_t xs_addr, int sbl) {
#pragma unroll
  for (int t = 0; t < 2; ++t) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (first) f.pair[4 * t + i].x = lds32(xb + 128 * t + 4 * i);
      if (second) f.pair[4 * t + i].y = lds32(xb + 128 * t + 4 * i);
    }
    const uint2 v = lds64(xs_addr + 8 * (4 * t + sbl));
    f.xs[t] = __uint_as_float(v.x);
    f.inv[t] = __uint_as_float(v.y);
  }
}
// Q6_K: tile (n, A) covers the scale groups 8n + 2A + {0, 1, 4, 5}; this lane's fragments of it are 8 activation bytes at
// xb + 128 n + 32 A; xs_addr: the sixteen (sum, 1 / S) pairs of the block.
DEVI void q6k_load_frags(BlockFrags& f, uint32_t xb, bool first, bool second, uint32_t xs_addr, int sl) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int n = t >> 1, A = t & 1;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (first) f.pair[2 * t + i].x = lds32(xb + 128 * n + 32 * A + 4 * i);
      if (second) f.pair[2 * t + i].y = lds32(xb + 128 * n + 32 * A + 4 * i);
    }
    const uint2 v = lds64(xs_addr + 8 * (8 * n + 2 * A + sl));
    f.xs[t] = __uint_as_float(v.x);
    f.inv[t] = __uint_as_float(v.y);
  }
}
// D[16x8] (+)= A[16x32] (u8, row) x B[32x8] (s8, col), s32 accumulate. Thread (g = lane/4, j = lane%4):
// a0/a1: rows g / g+8, k 4j..4j+3; a2/a3: same rows, k 16+4j..; b0: column g, k 4j..4j+3; b1: k 16+4j..;
// c0,c1: row g, columns 2j,2j+1; c2,c3: row g+8.
DEVI void mma_i8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the first MMA of a tile: the zero accumulator is one register that is never written
DEVI void mma_i8_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, int zero) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(zero));
}
// byte `sel & 3` of `word` as a float (the byte is the low mantissa byte of 2^23, minus 2^23)
DEVI float byte_to_float(uint32_t word, uint32_t sel) { return __uint_as_float(__byte_perm(word, 0x4B000000u, sel)) - kMagic; }

// ---- Q4_K: 16 row slots x one 256-column block against the block's fragments ----------------------------------------
// Tile t covers sub-blocks 4t .. 4t+3: slot group 0 = low nibbles of bytes 64t .. 64t+31 (sub-block 4t), group 1 = low
// nibbles of bytes 64t+32 .. (sub-block 4t+2), groups 2 / 3 = the high nibbles of the same bytes (sub-blocks 4t+1 /
// 4t+3). Lane j reads bytes 64t + 16j .. +15 of rows g and g + 8 (rA / rB: shared-memory address of the block in them);
// word q of them feeds MMA q of the tile: its low nibbles are four k slots of a0 / a1, its high nibbles of a2 / a3.
DEVI void q4k_rows(uint32_t rA, uint32_t rB, int j, const BlockFrags& f, float& acc0, float& acc1) {
  const uint4 hA = lds128(rA), hB = lds128(rB);
  const int sbl = 2 * (j & 1) + (j >> 1);         // this lane's sub-block inside a tile (slot group j)
  const uint32_t pick = 0x7650u + sbl;            // byte sbl of a word into the low byte of a magic float
  const float dA = half_lo(hA.x), mA = half_hi(hA.x), dB = half_lo(hB.x), mB = half_hi(hB.x);
  // the six-bit scales and minimums of the eight sub-blocks, four per word (kogarashi kernels/native.cu:59-60):
  // sub-blocks 0-3: bytes of y / z & 63; sub-blocks 4-7: (w & 15) | ((y >> 6) << 4) and (w >> 4) | ((z >> 6) << 4)
  const uint32_t scA[2] = {hA.y & 0x3F3F3F3Fu, (hA.w & 0x0F0F0F0Fu) | ((hA.y >> 2) & 0x30303030u)};
  const uint32_t mnA[2] = {hA.z & 0x3F3F3F3Fu, ((hA.w >> 4) & 0x0F0F0F0Fu) | ((hA.z >> 2) & 0x30303030u)};
  const uint32_t scB[2] = {hB.y & 0x3F3F3F3Fu, (hB.w & 0x0F0F0F0Fu) | ((hB.y >> 2) & 0x30303030u)};
  const uint32_t mnB[2] = {hB.z & 0x3F3F3F3Fu, ((hB.w >> 4) & 0x0F0F0F0Fu) | ((hB.z >> 2) & 0x30303030u)};
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const uint4 wA = lds128(rA + 16 + 64 * t + 16 * j), wB = lds128(rB + 16 + 64 * t + 16 * j);
    int c[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t a = u4w(wA, q), b = u4w(wB, q);
      const uint2 e = f.pair[4 * t + q];
      if (q == 0) mma_i8_first(c, a & 0x0F0F0F0Fu, b & 0x0F0F0F0Fu, (a >> 4) & 0x0F0F0F0Fu, (b >> 4) & 0x0F0F0F0Fu, e.x, e.y, 0);
      else mma_i8(c, a & 0x0F0F0F0Fu, b & 0x0F0F0F0Fu, (a >> 4) & 0x0F0F0F0Fu, (b >> 4) & 0x0F0F0F0Fu, e.x, e.y);
    }
    // sum of q x = (256 c_hi + c_lo) / S; value = d sc sum(q x) - dmin m sum(x)
    const float rawA = __int2float_rn(256 * c[0] + c[1]) * f.inv[t], rawB = __int2float_rn(256 * c[2] + c[3]) * f.inv[t];
    const float xsv = f.xs[t];
    acc0 = fmaf(dA * byte_to_float(scA[t], pick), rawA, acc0);
    acc0 = fmaf(-(mA * byte_to_float(mnA[t], pick)), xsv, acc0);
    acc1 = fmaf(dB * byte_to_float(scB[t], pick), rawB, acc1);
    acc1 = fmaf(-(mB * byte_to_float(mnB[t], pick)), xsv, acc1);
  }
}

// ---- Q6_K (row-aligned device layout: ql 128 | qh 64 | int8 scales 16 per block) ------------------------------------
// Tile (n, A) covers the scale groups 8n + 2A + {0, 1, 4, 5}: slot groups 0 / 1 = low nibbles of ql bytes
// 64n + 32A + [0,16) / [16,32) with qh bit pair A, groups 2 / 3 = the high nibbles with bit pair A + 2. Lane j reads ql
// bytes 64n + 32A + 8j .. +7 and qh bytes 32n + 8j .. +7 of rows g and g + 8; word u of them feeds MMA u of the tile.
// The codes enter unsigned (value + 32); the offset comes back through the integer group sums.
// dA / dB: the float block scales of the two rows.
DEVI void q6k_rows(uint32_t rA, uint32_t rB, int j, float dA, float dB, const BlockFrags& f, float& acc0, float& acc1) {
  const uint4 sA4 = lds128(rA + 192), sB4 = lds128(rB + 192);
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const uint2 hA = lds64(rA + 128 + 32 * n + 8 * j), hB = lds64(rB + 128 + 32 * n + 8 * j);
    // int8 scales of groups 8n + 4 (j / 2) .. + 3 as biased bytes
    const uint32_t swA = ((j >> 1) ? (n ? sA4.w : sA4.y) : (n ? sA4.z : sA4.x)) ^ 0x80808080u;
    const uint32_t swB = ((j >> 1) ? (n ? sB4.w : sB4.y) : (n ? sB4.z : sB4.x)) ^ 0x80808080u;
#pragma unroll
    for (int A = 0; A < 2; ++A) {
      const uint2 lA = lds64(rA + 64 * n + 32 * A + 8 * j), lB = lds64(rB + 64 * n + 32 * A + 8 * j);
      int c[4];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t wa = u ? lA.y : lA.x, wb = u ? lB.y : lB.x, ha = u ? hA.y : hA.x, hb = u ? hB.y : hB.x;
        // six-bit codes, four per word: low nibbles with qh bit pair A, high nibbles with bit pair A + 2
        const uint32_t loa = (wa & 0x0F0F0F0Fu) | ((A ? ha << 2 : ha << 4) & 0x30303030u);
        const uint32_t lob = (wb & 0x0F0F0F0Fu) | ((A ? hb << 2 : hb << 4) & 0x30303030u);
        const uint32_t hia = ((wa >> 4) & 0x0F0F0F0Fu) | ((A ? ha >> 2 : ha) & 0x30303030u);
        const uint32_t hib = ((wb >> 4) & 0x0F0F0F0Fu) | ((A ? hb >> 2 : hb) & 0x30303030u);
        const uint2 e = f.pair[2 * (2 * n + A) + u];
        if (u == 0) mma_i8_first(c, loa, lob, hia, hib, e.x, e.y, 0);
        else mma_i8(c, loa, lob, hia, hib, e.x, e.y);
      }
      const uint32_t sel = 0x7650u + 2 * A + (j & 1);
      const float dinvA = dA * f.inv[2 * n + A], dinvB = dB * f.inv[2 * n + A];
      const float sA = dinvA * (__uint_as_float(__byte_perm(swA, 0x4B000000u, sel)) - (kMagic + 128.f));
      const float sB = dinvB * (__uint_as_float(__byte_perm(swB, 0x4B000000u, sel)) - (kMagic + 128.f));
      // sum of (code - 32) x = (256 c_hi + c_lo - 32 sum(x_int)) / S
      const float xsv = f.xs[2 * n + A];
      acc0 = fmaf(sA, fmaf(-32.f, xsv, __int2float_rn(256 * c[0] + c[1])), acc0);
      acc1 = fmaf(sB, fmaf(-32.f, xsv, __int2float_rn(256 * c[2] + c[3])), acc1);
    }
  }
}

// Fixed-point scale of a scale group whose largest magnitude is `top`; `inv` = 1 / S.
DEVI float group_scale(float top, float& inv) {
  inv = top * (1.f / kFixedPointRange);
  return top > 0.f ? kFixedPointRange / top : 0.f;
}
DEVI float max4(float4 v) { return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))); }
DEVI bool finite4(float4 v) { return fabsf(v.x) <= 3.0e38f && fabsf(v.y) <= 3.0e38f && fabsf(v.z) <= 3.0e38f && fabsf(v.w) <= 3.0e38f; }
// Four consecutive activations times S -> 16-bit fixed point, split into two signed bytes each (value = 256 hi + lo,
// lo in [-128, 127]); returns the integer sum of the four fixed-point values.
DEVI int split_bytes4(float4 v, float S, uint32_t& hi, uint32_t& lo) {
  const float vals[4] = {v.x, v.y, v.z, v.w};
  int sum = 0;
  hi = lo = 0u;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int xi = __float2int_rn(vals[q] * S);
    const int l = ((xi + 128) & 255) - 128;
    const int h = (xi - l) >> 8;
    sum += xi;
    hi |= uint32_t(h & 255) << (8 * q);
    lo |= uint32_t(l & 255) << (8 * q);
  }
  return sum;
}

DEVI void sts32(uint32_t a, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
DEVI void sts64(uint32_t a, uint2 v) { asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a), "r"(v.x), "r"(v.y) : "memory"); }
DEVI void sts32f(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }

// The selection of one token by one warp, as a function of its own: the kernel calls it twice (rehearsal and
// selection) and both calls run the same instructions.
DMOE_ROUTE void fused_route(const float* logits, int experts, int topk, int lane, int* ids, float* prob) {
  RouteArgs r{logits, experts, experts, topk, 1, nullptr, 1.f, nullptr, nullptr, nullptr};
  if (experts <= 128) route_token<kRouteKogarashi, 4>(r, 0, lane, ids, prob);
  else if (experts <= 256) route_token<kRouteKogarashi, 8>(r, 0, lane, ids, prob);
  else route_token<kRouteKogarashi, 16>(r, 0, lane, ids, prob);
}
// Waits until fill `use` of a ring slot has been requested (`fill` counts the requests) and has landed.
DMOE_HOT bool wait_fill(volatile int* fill, uint64_t* full_bar, int use, unsigned* status, volatile int* abort_flag) {
  if (use > 0 && *fill <= use) {
    const uint64_t start = global_timer_ns();
    while (*fill <= use) {
      if (DMOE_FILL_SLEEP_NS) __nanosleep(DMOE_FILL_SLEEP_NS);
      if (*abort_flag) return false;
      if (global_timer_ns() - start > kWaitLimitNs) {
        atomicOr(status, kStatusWaitTimeout);
        *abort_flag = 1;
        return false;
      }
    }
  }
  return mbar_wait_abortable(full_bar, use & 1, status, abort_flag);
}

// ---- the kernel ----------------------------------------------------------------------------------------------
template <int DOWN_Q6>
__global__ void __launch_bounds__(kFusedThreads, 1) kogarashi_decode1_kernel(const FusedArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, grid = gridDim.x;
  // ---- shared memory ----
  int* sm_ids = reinterpret_cast<int*>(smem);                       // [32]
  float* sm_prob = reinterpret_cast<float*>(smem + 128);             // [32]
  float* sm_misc = reinterpret_cast<float*>(smem + 256);             // [0] sigmoid of the shared gate logit
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 272);
  float* pss = reinterpret_cast<float*>(smem + 384);                 // [16] per-warp sums of squares (layer entry)
  float* part = reinterpret_cast<float*>(smem + 448);                // [16][2] router partial sums
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + a.off_bars);   // [nstage]
  uint64_t* empty = full + a.nstage;                                 // [nstage]
  uint64_t* routed = empty + a.nstage;                               // routing published
  uint64_t* qbar = routed + 1;                                       // [4] one per quad: partial sums of a tile written
  volatile int* fill_id = reinterpret_cast<volatile int*>(smem + 576);   // [nstage] how many times a slot has been filled (requests issued)
  float* psum = reinterpret_cast<float*>(smem + a.off_psum);         // [slot][warp of the quad][16]
  float* sm_log = reinterpret_cast<float*>(smem + a.off_log);        // [E + 1] the logits as collected by the selecting warp
  const uint32_t act = smem_u32(smem + a.off_act);
  const uint32_t ring = smem_u32(smem + a.off_ring);
  const int NS = a.nstage;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, kFusedQuad);           // the four warps of the quad that owns a fill hand it back
    }
    mbar_init(routed, 1);
    for (int q = 0; q < 4; ++q) mbar_init(qbar + q, kFusedQuad);
    for (int s2 = 0; s2 < NS; ++s2) fill_id[s2] = 0;
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  // ---- the work lists of this CTA (same arithmetic in producer and consumers) ----
  // gate/up tiles sigma = cta, cta + grid, ... of G * tps (group-major, shared expert first; a tile = 16 rows of the gate
  // matrix and the same 16 rows of the up matrix); down tiles likewise of G * rt2 (also group-major: the products of
  // the groups become complete in this order). Chunks of the ring, in order: (gate rows, up rows) per gate/up tile,
  // then one per down tile.
  const int tiles1 = a.G * a.tps;
  const int n1 = cta < tiles1 ? (tiles1 - cta + grid - 1) / grid : 0;
  const int tiles2 = a.rt2 * a.G;
  const int n2 = cta < tiles2 ? (tiles2 - cta + grid - 1) / grid : 0;
  const int chunks = 2 * n1 + n2;
  const int R = a.E + a.has_shared;                                  // router rows incl. the shared gate projection

  if (warp >= kFusedConsumers) {
    // =========================== producer warps ===========================
    // Lane 0 of producer warp p issues the bulk copies of chunks p, p + 4, ... (the copies one thread issues are
    // carried out one after the other, about half a microsecond each whatever their size up to ~28 KB; four issuing
    // threads keep the HBM stream at its full rate). Producer warp 0 also selects the top-k, as a whole warp.
    const int prod = warp - kFusedConsumers;
    auto issue = [&](int c) -> bool {
      const int stage = c % NS, use = c / NS;
      if (use > 0 && !mbar_wait_abortable(empty + stage, (use - 1) & 1, a.status, abort_flag)) return false;
      const uint8_t* src;
      uint32_t bytes;
      if (c < 2 * n1) {
        const int lt = c >> 1, m = c & 1;
        const int sigma = cta + lt * grid, gi = sigma / a.tps, tile = sigma - gi * a.tps;
        const uint8_t* base;
        if (a.has_shared && gi == 0) base = m ? a.sh_up : a.sh_gate;
        else base = (m ? a.up_w : a.gate_w) + size_t(sm_ids[gi - a.has_shared]) * a.F * a.row_bytes1;
        src = base + size_t(tile) * (8 * kFusedPasses) * a.row_bytes1;
        bytes = uint32_t(8 * kFusedPasses) * a.row_bytes1;
      } else {
        const int u2 = cta + (c - 2 * n1) * grid, gi = u2 / a.rt2, rt = u2 - gi * a.rt2;
        const uint8_t* base = (a.has_shared && gi == 0) ? a.sh_down : a.down_w + size_t(sm_ids[gi - a.has_shared]) * a.H * a.row_bytes2;
        src = base + size_t(rt) * (16 * kFusedPasses) * a.row_bytes2;
        bytes = uint32_t(16 * kFusedPasses) * a.row_bytes2;
      }
      fill_id[stage] = use + 1;                  // consumers of fill `use` wait for this before they trust the parity
      mbar_arrive_expect_tx(full + stage, bytes);
      bulk_g2s(smem + a.off_ring + stage * a.stage_bytes, src, bytes, full + stage);
      return true;
    };
    int c = prod;
    int ok = 1;
    // the shared expert's first tile does not depend on anything: its weights are requested before the dependency wait
    if (lane == 0 && a.has_shared && n1 > 0 && cta < a.tps && c < 2 && c < NS) {
      ok = issue(c) ? 1 : 0;
      c += kFusedProducers;
    }
    if (prod == 0) {
      __syncwarp();
      {
        // Rehearsal: the selection below runs once per launch on the critical path between the two halves of the weight
        // stream, where every instruction-cache line it touches for the first time is a miss. The time before the
        // dependency wait is idle, so the same code runs here once on stand-in values (a router row); what it writes
        // to shared memory is overwritten by the real selection.
        fused_route(a.router_w, a.E, a.K, lane, sm_ids, sm_prob);
        __syncwarp();
      }
      pdl_wait();
      const unsigned tag = make_tag(__ldcg(a.epoch));
      ok = __shfl_sync(0xffffffffu, ok, 0);
      // every router row of this call, as the CTAs publish them
      if (ok) ok = gather_tagged(a.tlog + size_t(cta) * a.ldlog, R, tag, sm_log, lane, a.status, abort_flag) ? 1 : 0;
      __syncwarp();
      if (ok) {
        fused_route(sm_log, a.E, a.K, lane, sm_ids, sm_prob);
        if (lane == 0 && a.has_shared) sm_misc[0] = sigmoid_precise(sm_log[a.E]);
        __syncwarp();
        if (cta == 0 && lane < a.K) {
          a.ids[lane] = sm_ids[lane];
          a.prob[lane] = sm_prob[lane];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(routed);
      }
    }
    if (lane != 0) return;
    if (ok && prod != 0) ok = mbar_wait_abortable(routed, 0, a.status, abort_flag) ? 1 : 0;
    for (; ok && c < chunks; c += kFusedProducers) ok = issue(c) ? 1 : 0;
    if (!ok) {
      // gave up: let the copies this thread requested land before the CTA's shared memory goes away
      const uint64_t start = global_timer_ns();
      for (int q = prod; q < c && q < chunks; q += kFusedProducers)
        if (q + NS >= c)               // only the last ring's worth of chunks can still be in flight
          while (!mbar_test(full + q % NS, (q / NS) & 1) && global_timer_ns() - start < kWaitLimitNs) __nanosleep(256);
    }
    return;
  }

  // =========================== consumer warps ===========================
  const DiagLane dl = diag_lane(lane);
  const int g = dl.g, j = dl.j;
  const int quad = warp >> 2, kq = warp & 3;                          // tiles go to quads in turn; warp kq takes blocks kq, kq + 4, ...
  // ---- phase R: router rows of this CTA: row cta and row cta + grid ----
  const int chunks4 = a.H / 4;                                       // float4 per row
  const uint32_t rows_sm = act + a.act_rows;
  int my_rows = 0;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int row = cta + q * grid;
    if (row < R) {
      my_rows = q + 1;
      const float* src = row < a.E ? a.router_w + size_t(row) * a.H : a.sh_inp;
      for (int i = tid; i < chunks4; i += kFusedConsumers * 32) cp_async16(rows_sm + (q * chunks4 + i) * 16, src + 4 * i);
    }
  }
  cp_async_commit();
  constexpr int MAXC = 4;                                            // hidden <= 8192
  unsigned epoch_now, tag;
  {
    pdl_wait();
    epoch_now = __ldcg(a.epoch);
    tag = make_tag(epoch_now);
    if (tid == 0) atomicAdd(a.seen, 1u);            // CTA 0 advances the counter only when every CTA has read it
    // the token's activations: this thread's chunks stay in registers for the planes below. With the layer entry the
    // kernel forms them itself: u = (x + attn_out) * norm_w here, times the norm's scale once the sum of squares of the
    // whole vector is known (the logits are linear in that scale, so the router rows are multiplied with u meanwhile).
    float4 nv[MAXC];
    float sumsq = 0.f;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int i = tid + c * kFusedConsumers * 32;
      nv[c] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < chunks4) {
        if (a.norm_w) {
          float4 xv = __ldcg(reinterpret_cast<const float4*>(a.x) + i);
          if (a.attn_out) {
            const float4 o = __ldcg(reinterpret_cast<const float4*>(a.attn_out) + i);
            xv = make_float4(xv.x + o.x, xv.y + o.y, xv.z + o.z, xv.w + o.w);
          }
          const float4 wv = __ldg(reinterpret_cast<const float4*>(a.norm_w) + i);
          sumsq = fmaf(xv.x, xv.x, fmaf(xv.y, xv.y, fmaf(xv.z, xv.z, fmaf(xv.w, xv.w, sumsq))));
          nv[c] = make_float4(xv.x * wv.x, xv.y * wv.y, xv.z * wv.z, xv.w * wv.w);
        } else {
          nv[c] = __ldcg(reinterpret_cast<const float4*>(a.n) + i);
        }
      }
    }
    cp_async_wait<0>();
    float dot[2] = {0.f, 0.f};
#pragma unroll
    for (int q = 0; q < 2; ++q)
      if (q < my_rows) {
#pragma unroll
        for (int c = 0; c < MAXC; ++c) {
          const int i = tid + c * kFusedConsumers * 32;
          if (i < chunks4) {
            const uint4 w = lds128(rows_sm + (q * chunks4 + i) * 16);
            dot[q] = fmaf(__uint_as_float(w.x), nv[c].x, dot[q]);
            dot[q] = fmaf(__uint_as_float(w.y), nv[c].y, dot[q]);
            dot[q] = fmaf(__uint_as_float(w.z), nv[c].z, dot[q]);
            dot[q] = fmaf(__uint_as_float(w.w), nv[c].w, dot[q]);
          }
        }
      }
    dot[0] = warp_sum(dot[0]);
    dot[1] = warp_sum(dot[1]);
    sumsq = warp_sum(sumsq);
    if (lane == 0) {
      part[warp * 2] = dot[0];
      part[warp * 2 + 1] = dot[1];
      pss[warp] = sumsq;
    }
    named_barrier(1, kFusedConsumers * 32);
    float nscale = 1.f;
    if (a.norm_w) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kFusedConsumers; ++w) total += pss[w];        // the same order in every thread and CTA
      nscale = rsqrtf(total / float(a.H) + a.norm_eps);
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        nv[c] = make_float4(nv[c].x * nscale, nv[c].y * nscale, nv[c].z * nscale, nv[c].w * nscale);
        const int i = tid + c * kFusedConsumers * 32;
        if (cta == 0 && i < chunks4) reinterpret_cast<float4*>(a.n_out)[i] = nv[c];
      }
    }
    if (warp == 0) {
      // lanes 0-15 hold the partial sums of row 0, lanes 16-31 those of row 1; summed in a fixed tree
      float v = part[(lane & 15) * 2 + (lane >> 4)];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v *= nscale;
      const int q = lane >> 4, row = cta + q * grid;
      if ((lane & 15) == 0 && q < my_rows && row < a.E) {
        if (a.router_bias) v += a.router_bias[row];
        a.logits[row] = v;
      }
      // one copy of the logits per CTA, each polled by its owner only (148 CTAs polling the same lines would queue
      // up at those lines' L2 slices); row E: the shared expert's gate logit
      const float v0 = __shfl_sync(0xffffffffu, v, 0), v1 = __shfl_sync(0xffffffffu, v, 16);
      for (int d = lane; d < grid; d += 32) {
        unsigned long long* copy = a.tlog + size_t(d) * a.ldlog;
        if (my_rows > 0) st_tagged(copy + cta, v0, tag);
        if (my_rows > 1) st_tagged(copy + cta + grid, v1, tag);
      }
    }
    // ---- the token as 16-bit fixed point per 32 columns: two byte planes, and (float sum, 1 / S) per 32 columns ----
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int i = tid + c * kFusedConsumers * 32;
      float top = max4(nv[c]);
      top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
      top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
      top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 4));
      float inv;
      const float S = group_scale(top, inv);
      uint32_t hi, lo;
      int sum = split_bytes4(nv[c], S, hi, lo);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      if (i < chunks4) {
        if (!finite4(nv[c])) atomicOr(a.status, kStatusActRange);
        sts32(act + 4 * i, hi);
        sts32(act + a.act_lo1 + 4 * i, lo);
        if ((i & 7) == 0) sts64(act + a.act_xs1 + 8 * (i >> 3), make_uint2(__float_as_uint(inv * __int2float_rn(sum)), __float_as_uint(inv)));
      }
    }
    named_barrier(1, kFusedConsumers * 32);
  }

  // This lane's B fragments: offset inside a plane pair (bytes) from the first column of a block; which of its two B
  // register sets carries values (neither for half of the lanes)
  const uint32_t lane_x4 = (dl.plane ? uint32_t(a.act_lo1) : 0u) + 32u * (2 * ((g >> 1) & 1) + (g >> 2)) + 16u * (j & 1);
  const bool first = dl.active && !dl.second, second = dl.active && dl.second;
  const int sbl = 2 * (j & 1) + (j >> 1), sl = 4 * (j >> 1) + (j & 1);     // this lane's scale group inside a tile (Q4_K / Q6_K)
  BlockFrags fr;
  frags_clear(fr);
  bool ok = true;

  // Sum of the quad's partial rows: every warp writes its rows, the quad meets at its mbarrier (arrive = release,
  // wait = acquire: no fence), and warp 0 of the quad gets all rows (lane l: pass l / 16, row l % 16) and owns the
  // epilogue while the other three go on to their next tile. `slot`: partial-sum slot of the tile (tiles of one quad that may be pending
  // at the same time have different slots). Returns false when the wait was given up.
  int quad_syncs = 0;
  // The four warps of a quad meet (arrive = release, wait = acquire: what they wrote to shared memory before is visible
  // after). Every warp waits: a warp that ran ahead would arrive for the next meeting inside this one's phase. The wait
  // can be given up, unlike a `bar.sync`: false then.
  auto quad_sync = [&]() -> bool {
    __syncwarp();
    if (lane == 0) mbar_arrive(qbar + quad);
    const int parity = quad_syncs++ & 1;
    return mbar_wait_abortable(qbar + quad, parity, a.status, abort_flag);
  };
  auto quad_reduce = [&](int slot, float (&acc)[kFusedPasses][2], float& row_sum) -> bool {
    float* ps = psum + (slot * kFusedQuad + kq) * (16 * kFusedPasses);
#pragma unroll
    for (int p = 0; p < kFusedPasses; ++p) {
      const float r0 = quad_sum(acc[p][0]), r1 = quad_sum(acc[p][1]);
      if (j == 0) {
        ps[p * 16 + g] = r0;
        ps[p * 16 + 8 + g] = r1;
      }
    }
    if (!quad_sync()) return false;
    if (kq != 0) return true;
    row_sum = 0.f;
    if (lane < 16 * kFusedPasses) {
#pragma unroll
      for (int q = 0; q < kFusedQuad; ++q) row_sum += psum[(slot * kFusedQuad + q) * (16 * kFusedPasses) + lane];
    }
    return true;
  };

  // Waits until chunk c has landed in its slot. A parity wait can only tell the current fill of a slot from the one
  // before it, and a quad does not see every fill of a slot (other quads consume some): so the producer publishes the
  // number of fills it has requested per slot, and a consumer first waits until its fill has been requested (the
  // barrier is then in that fill's phase or just past it) and only then for the parity.
  auto wait_chunk = [&](int c) -> bool { return wait_fill(fill_id + c % NS, full + c % NS, c / NS, a.status, abort_flag); };

  // ---- the product vector of one expert group for this quad's down tiles ----
  // Raw tagged words are copied asynchronously (every thread copies, and later reads, its own 32 bytes: four values)
  // into the quad's area ahead of time; staging checks the tags (a word that was not there yet is polled from global
  // memory), converts to fixed point per scale group of the down format: byte planes, and per 16 (Q6_K: integer sum) or
  // 32 (Q4_K: float sum) columns the pair (sum, 1 / S); then the quad meets. False when a wait was given up.
  const int qt = tid & (32 * kFusedQuad - 1);
  const uint32_t qraw = act + a.act_q + quad * a.act_qs, qpl = qraw + 8u * a.F, qxs = qpl + a.act_xs2;
  int pre = -1;                                                          // group whose raw words are on their way
  auto prefetch_group = [&](int gi) {
    const unsigned long long* src = a.th + size_t(gi) * a.F;
    for (int i = qt; i < a.F / 4; i += 32 * kFusedQuad) {
      cp_async16(qraw + 32u * i, src + 4 * i);
      cp_async16(qraw + 32u * i + 16u, src + 4 * i + 2);
    }
    cp_async_commit();
  };
  auto stage_group = [&](int gi) -> bool {
    cp_async_wait<0>();
    for (int base = 0; base < a.F / 4; base += 32 * kFusedQuad) {        // uniform trip count: shuffles below
      const int i = base + qt;
      const bool live = i < a.F / 4;
      float4 hv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live) {
        uint4 r0 = lds128(qraw + 32u * i), r1 = lds128(qraw + 32u * i + 16u);
        bool have = r0.y == tag && r0.w == tag && r1.y == tag && r1.w == tag;
        if (!have) have = poll_four(a.th + size_t(gi) * a.F + 4 * i, tag, r0, r1, a.status, abort_flag);
        if (have) hv = make_float4(__uint_as_float(r0.x), __uint_as_float(r0.z), __uint_as_float(r1.x), __uint_as_float(r1.z));
      }
      __syncwarp();
      float top = max4(hv);
      top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
      top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
      if (!DOWN_Q6) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 4));
      float inv;
      const float S = group_scale(top, inv);
      uint32_t hi, lo;
      int sum = split_bytes4(hv, S, hi, lo);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (!DOWN_Q6) sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      if (live) {
        sts32(qpl + 4 * i, hi);
        sts32(qpl + a.act_lo2 + 4 * i, lo);
        if (DOWN_Q6) {
          if ((i & 3) == 0) sts64(qxs + 8 * (i >> 2), make_uint2(__float_as_uint(__int2float_rn(sum)), __float_as_uint(inv)));
        } else {
          if ((i & 7) == 0) sts64(qxs + 8 * (i >> 3), make_uint2(__float_as_uint(inv * __int2float_rn(sum)), __float_as_uint(inv)));
        }
      }
    }
    return quad_sync() && !*abort_flag;
  };

  // The tiles start only when the selection is done, the shared expert's (whose weights are already here) included:
  // a consumer warp that multiplies while the producer warp selects slows the selection down several times (they
  // share a scheduler), and the selection, not the shared expert, is on the critical path.
  if (!mbar_wait_abortable(routed, 0, a.status, abort_flag)) ok = false;

  // ---- phase 1: gate/up tiles ----
  for (int lt = quad; lt < n1 && ok; lt += kFusedConsumers / kFusedQuad) {
    const int cg = 2 * lt, cu = cg + 1;
    if (lt + kFusedConsumers / kFusedQuad >= n1 && quad < n2) {       // the quad's last gate/up tile: its first down tile's products
      pre = (cta + quad * grid) / a.rt2;
      prefetch_group(pre);
    }
    if (!wait_chunk(cg) || !wait_chunk(cu)) { ok = false; break; }
    const int sigma = cta + lt * grid, gi = sigma / a.tps, tile = sigma - gi * a.tps;
    float acc[kFusedPasses][2] = {};
    if (kq < a.nblk1) {
      const uint32_t gate_rows = ring + (cg % NS) * a.stage_bytes + g * a.row_bytes1;    // row g of the tile's gate rows
      const uint32_t up_rows = ring + (cu % NS) * a.stage_bytes + g * a.row_bytes1;
      for (int b = kq; b < a.nblk1; b += kFusedQuad) {
        q4k_load_frags(fr, act + lane_x4 + 256u * b, first, second, act + a.act_xs1 + 64u * b, sbl);
#pragma unroll
        for (int p = 0; p < kFusedPasses; ++p)       // eight rows of the tile per pass: gate row in MMA row g, up row in MMA row g + 8
          q4k_rows(gate_rows + 8 * p * a.row_bytes1 + b * 144, up_rows + 8 * p * a.row_bytes1 + b * 144, j, fr, acc[p][0], acc[p][1]);
      }
    }
    // the weights of the tile are not needed any more: the slots go back before the sums meet
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(empty + cg % NS);
      mbar_arrive(empty + cu % NS);
    }
    float rows = 0.f;
    if (!quad_reduce(lt % kFusedSlots, acc, rows)) { ok = false; break; }
    if (kq == 0) {
      // lane l: pass l / 16; lanes 0-7 of a pass hold its gate rows, lanes 8-15 its up rows
      const float up = __shfl_down_sync(0xffffffffu, rows, 8);
      float h = 0.f;
      if (lane < 16 * kFusedPasses && (lane & 15) < 8) {
        h = silu_mul(rows, up);
        st_tagged(a.th + size_t(gi) * a.F + tile * (8 * kFusedPasses) + 8 * (lane >> 4) + (lane & 7), h, tag);
      }
      if (!(fabsf(h) <= 3.0e38f)) atomicOr(a.status, kStatusActRange);
    }
  }

  // ---- phase 2: down tiles ----
  const uint32_t lane_x6 = (dl.plane ? uint32_t(a.act_lo2) : 0u) + 64u * (g >> 2) + 16u * ((g >> 1) & 1) + 8u * (j & 1);
  const uint32_t lane_x4d = (dl.plane ? uint32_t(a.act_lo2) : 0u) + 32u * (2 * ((g >> 1) & 1) + (g >> 2)) + 16u * (j & 1);
  int staged = -1;                                                       // group whose planes the quad holds
  for (int t2 = quad; t2 < n2 && ok; t2 += kFusedConsumers / kFusedQuad) {
    const int c = 2 * n1 + t2, stage = c % NS;
    const int u2 = cta + t2 * grid, gi = u2 / a.rt2, rt = u2 - gi * a.rt2;
    if (gi != staged) {
      if (pre != gi) prefetch_group(gi);
      pre = -1;
      if (!stage_group(gi)) { ok = false; break; }
      staged = gi;
    }
    if (pre < 0 && t2 + kFusedConsumers / kFusedQuad < n2) {             // the next tile's products, while this tile is multiplied
      const int gn = (u2 + (kFusedConsumers / kFusedQuad) * grid) / a.rt2;
      if (gn != staged) {
        pre = gn;
        prefetch_group(gn);
      }
    }
    if (!wait_chunk(c)) { ok = false; break; }
    float acc[kFusedPasses][2] = {};
    if (kq < a.nblk2) {
      const uint32_t rowg = ring + stage * a.stage_bytes + g * a.row_bytes2;            // row g of the tile
      const uint32_t xreal = qpl + (DOWN_Q6 ? lane_x6 : lane_x4d);
      for (int b = kq; b < a.nblk2; b += kFusedQuad) {
        if (DOWN_Q6) {
          q6k_load_frags(fr, xreal + 256u * b, first, second, qxs + 128u * b, sl);
#pragma unroll
          for (int p = 0; p < kFusedPasses; ++p) {     // sixteen rows of the tile per pass
            const uint32_t rA = rowg + 16 * p * a.row_bytes2, rB = rA + 8 * a.row_bytes2;
            // the f16 block scales follow the blocks of a row
            const uint32_t dwA = lds32(rA + a.nblk2 * 208 + ((2 * b) & ~3)), dwB = lds32(rB + a.nblk2 * 208 + ((2 * b) & ~3));
            const float dA = (b & 1) ? half_hi(dwA) : half_lo(dwA), dB = (b & 1) ? half_hi(dwB) : half_lo(dwB);
            q6k_rows(rA + b * 208, rB + b * 208, j, dA, dB, fr, acc[p][0], acc[p][1]);
          }
        } else {
          q4k_load_frags(fr, xreal + 256u * b, first, second, qxs + 64u * b, sbl);
#pragma unroll
          for (int p = 0; p < kFusedPasses; ++p) {
            const uint32_t rA = rowg + 16 * p * a.row_bytes2, rB = rA + 8 * a.row_bytes2;
            q4k_rows(rA + b * 144, rB + b * 144, j, fr, acc[p][0], acc[p][1]);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty + stage);
    float rows = 0.f;
    if (!quad_reduce(t2 % kFusedSlots, acc, rows)) { ok = false; break; }
    // the finished rows of this expert: lane l holds row 16 (l / 16) + (l % 16) of the tile
    if (kq == 0 && lane < 16 * kFusedPasses) st_tagged(a.ty + size_t(gi) * a.H + rt * (16 * kFusedPasses) + lane, rows, tag);
  }
  if (!ok) *abort_flag = 1;
  cp_async_wait<0>();                            // a prefetch that was never used must not outlive the CTA

  // ---- combine: x[i] += sum_s fma(p_s, down_s[i]) + sigmoid(sg) * shared[i]   (kogarashi kernels/native.cu:113-117);
  //      row i = tid * grid + cta; the down rows arrive tagged ----
  const int row = tid * grid + cta;
  if (ok && row < a.H) {
    const float xin = a.x[row] + (a.attn_out ? a.attn_out[row] : 0.f);
    bool good = true;
    float ysh[8] = {};
    if (a.has_shared) good = poll_strided(a.ty + row, 0, 1, tag, ysh, a.status, abort_flag);
    float v = 0.f;
    for (int s0 = 0; s0 < a.K && good; s0 += 8) {          // eight loads in flight at a time; the sum itself stays in slot order
      float ys[8] = {};
      const int nq = a.K - s0 < 8 ? a.K - s0 : 8;
      good = poll_strided(a.ty + size_t(s0 + a.has_shared) * a.H + row, size_t(a.H), nq, tag, ys, a.status, abort_flag);
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < nq) v = fmaf(sm_prob[s0 + q], ys[q], v);
    }
    if (a.has_shared) v += sm_misc[0] * ysh[0];
    if (good) a.x[row] = xin + v;
  }
  // ---- the call counter moves on (also after a failure: the next call must not take this call's words for its own) ----
  if (cta == 0 && tid == 0) {
    PollClock clk;
    while (ld_acquire_u32(a.seen) < unsigned(grid) && !clk.expired(a.status, abort_flag)) {}
    *a.seen = 0u;
    *a.epoch = epoch_now + 1u;
  }
}

}  // namespace dmoe
