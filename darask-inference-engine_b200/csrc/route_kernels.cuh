// Kernels around route_impl.cuh: stand-alone top-k, the router projection (logits) fused with
// top-k and the dispatch permutation through a "last block finishes" counter, and the
// stand-alone permutation. Included by kogarashi.cu and tsumuji.cu (precise math) and by
// hayate.cu (compiled with --use_fast_math, as the reference builds its GLM kernels).
#pragma once
#include "route_impl.cuh"
#include "expert_gemv.cuh"

namespace dmoe {

template <int MODE>
__global__ void __launch_bounds__(128) route_topk_kernel(RouteArgs a) {
  pdl_wait();
  pdl_launch();
  const int token = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (token < a.tokens) route_token_any<MODE>(a, token, threadIdx.x & 31);
}

template <int UNUSED = 0>
__global__ void __launch_bounds__(1024) permute_kernel(PermuteArgs p) {
  extern __shared__ int hist[];
  pdl_wait();
  pdl_launch();
  permute_block(p, hist, p.ids);
}

// ---- router projection -----------------------------------------------------------------------
// logits[t][row] = sum_k W[row][k] x[t][k], one block per row, the four warps split k.
// Rows [0, experts) come from `w`; row `experts` (optional) from `extra` : the shared-expert gate
// projection (kogarashi engine.rs:610-618 ffn_gate_inp_shexp; tsumuji keeps it as row E of the
// router matrix, weights.rs:937-947).
template <typename T> DEVI float to_f32(T v);
template <> DEVI float to_f32<float>(float v) { return v; }
template <> DEVI float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> DEVI float to_f32<__half>(__half v) { return __half2float(v); }

constexpr int kRouteIdCache = 2048;   // routes the fused kernel keeps in shared memory for the permutation

struct RouterArgs {
  const void* w;        // [rows][hidden]
  const void* extra;    // [hidden] or null
  const void* x;        // [T][hidden]
  const float* row_bias; // [rows] added to the logits of rows < `rows` (null: none)
  float* logits;        // [T][ld]
  float* extra_out;     // [T] raw logit of the extra row when it is not stored in `logits`
  int hidden, rows, ld, tokens;
  RouteArgs route;      // routing of the finished logits (route.logits == logits)
  PermuteArgs perm;
  unsigned* done;       // counter, zero before the launch; reset to zero by the last block
  __half* planes;       // optional (float x only): blocks past the router rows write the activation planes
  __half* xsum_planes;  //   [T][2][hidden] and the per-32 sums as hi / lo planes [T][2][hidden/32] read by the expert kernels
  int planes_natural;   // plane element order: 0 GGUF fragment order, 1 natural (NVFP4)
  int fuse;             // 1: last block routes and permutes
};

template <typename WT, typename XT, int MODE>
__global__ void __launch_bounds__(128) router_kernel(RouterArgs a) {
  extern __shared__ int hist[];
  __shared__ float part[4][16];
  __shared__ unsigned last;
  constexpr int VEC = 16 / sizeof(WT);          // weights per 16-byte load
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int router_rows = a.rows + (a.extra ? 1 : 0);
  if (row >= router_rows) {          // activation planes of token row - router_rows
    pdl_wait();
    pdl_launch();
    if (a.planes) {
      const int t = row - router_rows;
      act_planes_row(static_cast<const XT*>(a.x) + size_t(t) * a.hidden, a.hidden, a.planes + size_t(t) * 2 * a.hidden,
                     a.xsum_planes ? a.xsum_planes + size_t(t) * 2 * (a.hidden / 32) : nullptr, a.planes_natural != 0, a.perm.status);
    }
    return;                            // not counted: only the router rows gate the routing below
  }
  const bool is_extra = row >= a.rows;
  const WT* wr = is_extra ? static_cast<const WT*>(a.extra) : static_cast<const WT*>(a.w) + size_t(row) * a.hidden;
  // weights do not depend on earlier kernels: fetch them before the dependency wait
  constexpr int MAXC = 8;                        // 16-byte chunks per thread kept in registers
  uint4 wv[MAXC];
  const int chunks = a.hidden / VEC;
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = tid + i * 128;
    wv[i] = c < chunks ? __ldg(reinterpret_cast<const uint4*>(wr) + c) : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();
  pdl_launch();
  for (int t0 = 0; t0 < a.tokens; t0 += 16) {
    const int nt = min(16, a.tokens - t0);
    for (int t = 0; t < nt; ++t) {
      const XT* xt = static_cast<const XT*>(a.x) + size_t(t0 + t) * a.hidden;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < MAXC; ++i) {
        const int c = tid + i * 128;
        if (c < chunks) {
          const WT* wp = reinterpret_cast<const WT*>(&wv[i]);
#pragma unroll
          for (int j = 0; j < VEC; ++j) acc = fmaf(to_f32(wp[j]), to_f32(xt[c * VEC + j]), acc);
        }
      }
      for (int c = tid + MAXC * 128; c < chunks; c += 128) {   // rows longer than the register window
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(wr) + c);
        const WT* wp = reinterpret_cast<const WT*>(&q);
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc = fmaf(to_f32(wp[j]), to_f32(xt[c * VEC + j]), acc);
      }
      acc = warp_sum(acc);
      if (lane == 0) part[warp][t] = acc;
    }
    __syncthreads();
    if (tid < nt) {
      float v = (part[0][tid] + part[1][tid]) + (part[2][tid] + part[3][tid]);
      if (!is_extra && a.row_bias) v += a.row_bias[row];
      if (is_extra && a.extra_out) a.extra_out[t0 + tid] = v;
      if (!is_extra || a.ld > a.rows) a.logits[size_t(t0 + tid) * a.ld + row] = v;
    }
    __syncthreads();
  }
  if (!a.fuse) return;
  // Last block to finish routes every token and builds the permutation.
  __threadfence();
  if (tid == 0) last = atomicAdd(a.done, 1u) == unsigned(router_rows) - 1 ? 1u : 0u;
  __syncthreads();
  if (!last) return;
  __threadfence();
  for (int token = warp; token < a.tokens; token += 4) route_token_any<MODE>(a.route, token, lane);
  __threadfence_block();
  __syncthreads();
  if (a.perm.assignments) {
    // the routes of this block, copied once into shared memory (after the E + 1 histogram words)
    const int n = a.tokens * a.route.topk;
    const int* ids = a.perm.ids;
    if (n <= kRouteIdCache) {
      int* cache = hist + a.route.experts + 1;
      for (int i = tid; i < n; i += 128) cache[i] = __ldcg(a.perm.ids + i);
      __syncthreads();
      ids = cache;
    }
    permute_block(a.perm, hist, ids);
  }
  if (tid == 0) *a.done = 0u;
}

}  // namespace dmoe
