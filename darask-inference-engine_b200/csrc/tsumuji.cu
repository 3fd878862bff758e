// Tsumuji (Qwen-Next, NVFP4 routed experts + dense bf16 shared expert) MoE FFN for a window of N tokens.
// Reference call site: tsumuji crates/tsumuji-engine/src/engine.rs:1586-1683 (`mlp_half`): router GEMV,
// `router_topk`, `moe_gate_up`, `moe_down`, `moe_combine`; kernels tsumuji kernels/decode/ops.cu:148-230,
// decode/gemv.cu:64-158. Expert block layout: tsumuji crates/tsumuji-engine/src/weights.rs:10-12.
#include "../../include/darask_moe_b200.h"
#include "dense_gemv.cuh"
#include "gemv_launch.cuh"
#include "route_kernels.cuh"
#include "permute_large.cuh"

namespace dmoe {

// Residual-stream write-back of the reference's `moe_combine` (tsumuji kernels/decode/ops.cu:76-94, 202-230), optional.
struct TsumujiWriteback {
  float* R;            // [N][HC][H] residual streams, R[n][i] += inj_i * out[n]
  const float* di;     // [Sd][N][ld] partial sums of the stream-gate projection; inj_i = 2 sigmoid(sum_s di[s][n][rank + i] / HC)
  int Sd, ld, rank, HC;
  float* ss;           // [N][blocks of 256 columns][HC]: sum of squares of the new R over the block's columns
};

// out[n][i] = sum_s fma(w[n][s], y[n*k+s][i]) then fma(shared_gate[n], y[N*k+n][i])   (ops.cu:217-223);
// with a write-back: the HC streams of token n take inj_i * out and every block leaves its share of their
// sums of squares (one block = 256 columns of one token, as in the reference, so `ss` has the same layout).
__global__ void __launch_bounds__(256) tsumuji_combine_kernel(float* out, const float* y, const float* w, const float* sgate,
                                                              int hidden, int topk, int tokens, int accumulate, TsumujiWriteback wb) {
  __shared__ float gate_of_stream[8];
  __shared__ float warp_part[8][8];
  pdl_wait();
  pdl_launch();
  const int i = blockIdx.x * 256 + threadIdx.x, n = blockIdx.y;
  float o = 0.f;
  if (i < hidden) {
    for (int s = 0; s < topk; ++s) o = fmaf(__ldcg(w + n * topk + s), __ldcg(y + size_t(n * topk + s) * hidden + i), o);
    o = fmaf(__ldcg(sgate + n), __ldcg(y + size_t(tokens * topk + n) * hidden + i), o);
    if (out) out[size_t(n) * hidden + i] = accumulate ? out[size_t(n) * hidden + i] + o : o;
  }
  if (!wb.R) return;
  if (threadIdx.x < wb.HC) {
    float a = 0.f;
    for (int s = 0; s < wb.Sd; ++s) a += __ldcg(wb.di + size_t(s * tokens + n) * wb.ld + wb.rank + threadIdx.x);
    gate_of_stream[threadIdx.x] = 2.f * (1.f / (1.f + expf(-(a / float(wb.HC)))));
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int st = 0; st < wb.HC; ++st) {
    float v = 0.f;
    if (i < hidden) {
      float* r = wb.R + (size_t(n) * wb.HC + st) * hidden + i;
      v = *r + gate_of_stream[st] * o;
      *r = v;
    }
    const float sq = warp_sum(v * v);
    if (lane == 0) warp_part[st][warp] = sq;
  }
  __syncthreads();
  if (threadIdx.x < wb.HC) {
    float total = 0.f;
    for (int q = 0; q < 8; ++q) total += warp_part[threadIdx.x][q];      // fixed order
    wb.ss[(size_t(n) * gridDim.x + blockIdx.x) * wb.HC + threadIdx.x] = total;
  }
}

// stand-alone routing of given logits followed by the permutation, one block
template <int MODE>
__global__ void __launch_bounds__(128) route_permute_kernel(RouteArgs r, PermuteArgs p) {
  extern __shared__ int hist[];
  pdl_wait();
  pdl_launch();
  for (int token = threadIdx.x >> 5; token < r.tokens; token += 4) route_token_any<MODE>(r, token, threadIdx.x & 31);
  __threadfence_block();
  __syncthreads();
  permute_block(p, hist, p.ids);
}

template <typename XT>
__global__ void __launch_bounds__(128) act_planes_kernel(const XT* x, int k, __half* planes, __half* xsum_planes, int natural) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  act_planes_row(x + size_t(t) * k, k, planes + size_t(t) * 2 * k, xsum_planes ? xsum_planes + size_t(t) * 2 * (k / 32) : nullptr, natural != 0);
}

// ---- expert-parallel pieces ---------------------------------------------------------------------------------------
// send rows in dispatch order: row i = x[assignments[i] / topk]; position[a] = i
__global__ void __launch_bounds__(256) tsumuji_gather_kernel(const float* x, const unsigned* assignments, const int* counters, int topk,
                                                             int hidden, float* send, unsigned* position) {
  pdl_wait();
  pdl_launch();
  const int i = blockIdx.x;
  if (i >= __ldcg(counters + 1)) return;
  const unsigned a = __ldcg(assignments + i);
  if (threadIdx.x == 0) position[a] = i;
  const float4* src = reinterpret_cast<const float4*>(x + size_t(a / topk) * hidden);
  float4* dst = reinterpret_cast<float4*>(send + size_t(i) * hidden);
  for (int c = threadIdx.x; c < hidden / 4; c += 256) dst[c] = __ldg(src + c);
}
// received rows come grouped by source rank, then by ascending local expert: ids[row] = that expert
__global__ void __launch_bounds__(128) ep_row_experts_kernel(const int* counts, int ranks, int local, int* ids) {
  pdl_wait();
  pdl_launch();
  __shared__ int start;
  const int seg = blockIdx.x;                 // = rank * local + expert
  if (threadIdx.x == 0) {
    int s = 0;
    for (int i = 0; i < seg; ++i) s += counts[i];
    start = s;
  }
  __syncthreads();
  const int n = counts[seg];
  for (int i = threadIdx.x; i < n; i += 128) ids[start + i] = seg % local;
}
// out[n][i] = sum_s fma(w[n][s], y[position[n*k+s]][i]) then fma(shared_gate[n], y_shared[n][i])
__global__ void __launch_bounds__(256) tsumuji_ep_combine_kernel(float* out, const float* y, const float* w, const unsigned* position,
                                                                 const float* sgate, const float* y_shared, int hidden, int topk,
                                                                 int accumulate) {
  pdl_wait();
  pdl_launch();
  const int i = blockIdx.x * 256 + threadIdx.x, n = blockIdx.y;
  if (i >= hidden) return;
  float o = 0.f;
  for (int s = 0; s < topk; ++s) o = fmaf(__ldcg(w + n * topk + s), __ldcg(y + size_t(__ldcg(position + n * topk + s)) * hidden + i), o);
  o = fmaf(__ldcg(sgate + n), __ldcg(y_shared + size_t(n) * hidden + i), o);
  out[size_t(n) * hidden + i] = accumulate ? out[size_t(n) * hidden + i] + o : o;
}

// ---- shared expert of a token window on the tensor cores ---------------------------------------------------------
// hayate_prefill.cu: ragged grouped bf16 GEMM (tcgen05), float32 accumulator output
cudaError_t launch_grouped_bf16(void* out, float* acc, const void* x, const void* w, const void* ranges, unsigned groups,
                                unsigned n, unsigned k, const float* scales, cudaStream_t st, unsigned w_rows);
// float32 rows -> bf16 "hi" rows [0, N) and bf16 "lo" rows [N, 2N) with x = hi + lo up to 2^-17 |x|; one group of 2N rows
__global__ void __launch_bounds__(256) split_rows_kernel(const float* x, int rows, int k, __nv_bfloat16* hl, unsigned* ranges) {
  pdl_wait();
  pdl_launch();
  if (blockIdx.x == 0 && threadIdx.x == 0) { ranges[0] = 2u * unsigned(rows); ranges[1] = 0u; }
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x, total = size_t(rows) * k;
  if (i >= total) return;
  const float v = x[i];
  const __nv_bfloat16 hi = __float2bfloat16_rn(v);
  hl[i] = hi;
  hl[total + i] = __float2bfloat16_rn(v - __bfloat162float(hi));
}
// acc [2N][2F] (hi rows then lo rows; gate columns then up columns) -> h = silu(g) * u as bf16 hi/lo rows [2N][F]
__global__ void __launch_bounds__(256) shared_swiglu_kernel(const float* acc, int rows, int inter, __nv_bfloat16* hl) {
  pdl_wait();
  pdl_launch();
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x, total = size_t(rows) * inter;
  if (i >= total) return;
  const size_t t = i / inter, c = i % inter;
  const float* a0 = acc + t * 2 * inter;
  const float* a1 = acc + (t + rows) * 2 * inter;
  const float g = a0[c] + a1[c], u = a0[inter + c] + a1[inter + c];
  const float h = silu_mul(g, u);
  const __nv_bfloat16 hi = __float2bfloat16_rn(h);
  hl[i] = hi;
  hl[total + i] = __float2bfloat16_rn(h - __bfloat162float(hi));
}
// y[t] = acc[t] + acc[N + t]
__global__ void __launch_bounds__(256) add_halves_kernel(const float* acc, int rows, int hidden, float* y) {
  pdl_wait();
  pdl_launch();
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x, total = size_t(rows) * hidden;
  if (i < total) y[i] = acc[i] + acc[total + i];
}

// acc [2N][ld_acc] (hi rows then lo rows of the router products) -> logits [N][rows]
__global__ void __launch_bounds__(256) add_logits_kernel(const float* acc, int tokens, int ld_acc, int rows, float* logits) {
  pdl_wait();
  pdl_launch();
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x, total = size_t(tokens) * rows;
  if (i >= total) return;
  const size_t t = i / rows, c = i % rows;
  logits[i] = acc[t * ld_acc + c] + acc[(t + tokens) * ld_acc + c];
}

constexpr int kWindowTokens = 16;      // more tokens than this: the batched front end and the tensor-core shared expert
static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
struct TsumujiWs {
  int* counters; unsigned* done; unsigned* status; int* active; unsigned* ranges; unsigned* assignments; int4* plan;
  __half* xplanes; __half* hplanes; float* y; int* perm_scratch;
  // token windows: operands of the shared expert's tensor-core products
  unsigned* sh_ranges; __nv_bfloat16* sh_x; float* sh_acc; __nv_bfloat16* sh_out; __nv_bfloat16* sh_h;
  size_t bytes;
};
static TsumujiWs carve(void* base, int hidden, int inter, int experts, int topk, int tokens) {
  TsumujiWs w;
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) { uint8_t* q = p ? p + off : nullptr; off = align_up(off + bytes, 256); return q; };
  w.counters = reinterpret_cast<int*>(take(16));
  w.done = reinterpret_cast<unsigned*>(take(4));
  w.status = reinterpret_cast<unsigned*>(take(4));
  w.active = reinterpret_cast<int*>(take(size_t(experts) * 4));
  w.ranges = reinterpret_cast<unsigned*>(take(size_t(experts) * 8));
  w.assignments = reinterpret_cast<unsigned*>(take(size_t(tokens) * topk * 4));
  w.plan = reinterpret_cast<int4*>(take(size_t(experts + 1) * 16));
  w.xplanes = reinterpret_cast<__half*>(take(size_t(tokens) * 2 * hidden * 2));
  const size_t rows = size_t(tokens) * topk + tokens;
  w.hplanes = reinterpret_cast<__half*>(take(rows * 2 * inter * 2));
  w.y = reinterpret_cast<float*>(take(rows * hidden * 4));
  w.perm_scratch = reinterpret_cast<int*>(take(permute_scratch_bytes(tokens, topk, experts)));
  const size_t router_pad = (size_t(experts) + 1 + 127) / 128 * 128;     // router rows as a multiple of the 128-row weight tiles
  size_t wide = size_t(hidden > 2 * inter ? hidden : 2 * inter);
  if (router_pad > wide) wide = router_pad;
  const size_t win = tokens > kWindowTokens ? size_t(tokens) : 0;
  w.sh_ranges = reinterpret_cast<unsigned*>(take(8));
  w.sh_x = reinterpret_cast<__nv_bfloat16*>(take(2 * win * hidden * 2));
  w.sh_acc = reinterpret_cast<float*>(take(2 * win * wide * 4));
  w.sh_out = reinterpret_cast<__nv_bfloat16*>(take(2 * win * wide * 2));
  w.sh_h = reinterpret_cast<__nv_bfloat16*>(take(2 * win * inter * 2));
  w.bytes = off;
  return w;
}

// token windows: projection, routing, permutation and planes as separate launches that scale with N
static cudaError_t route_window(const void* router_w, const float* x, const RouteArgs& route, const PermuteArgs& perm, const TsumujiWs& w,
                                int H, int E, int N, cudaStream_t st) {
  cudaError_t e;
  const unsigned blocks_x = unsigned((size_t(N) * H + 255) / 256);
  // the float32 rows as bf16 hi + lo rows (also the shared expert's operand); H is a multiple of 256 here
  if ((e = launch_pdl(split_rows_kernel, dim3(blocks_x), dim3(256), 0, st, x, N, H, w.sh_x, w.sh_ranges))) return e;
  if (router_w) {
    // logits = W x on the tcgen05 bf16 grouped GEMM: one group of 2N rows against the E + 1 router rows (padded to
    // 128-row tiles that read zeros), then hi + lo
    const unsigned npad = unsigned((E + 1 + 127) / 128 * 128);
    if ((e = launch_grouped_bf16(w.sh_out, w.sh_acc, w.sh_x, router_w, w.sh_ranges, 1, npad, unsigned(H), nullptr, st, unsigned(E + 1)))) return e;
    if ((e = launch_pdl(add_logits_kernel, dim3(unsigned((size_t(N) * (E + 1) + 255) / 256)), dim3(256), 0, st, (const float*)w.sh_acc, N,
                        int(npad), E + 1, const_cast<float*>(route.logits)))) return e;
  }
  if ((e = launch_pdl(route_topk_kernel<kRouteTsumuji>, dim3((N + 3) / 4), dim3(128), 0, st, route))) return e;
  if ((e = launch_permute_large(perm, w.perm_scratch, st))) return e;
  return launch_pdl(act_planes_kernel<float>, dim3(N), dim3(128), 0, st, x, H, w.xplanes, (__half*)nullptr, 1);
}

// shared expert of a window: y_out[t] = W_down . silu(W_gate . x[t]) * (W_up . x[t]), two tcgen05 bf16 GEMMs over the
// hi / lo split of the float32 operands (exact bf16 weights, float32 accumulation)
static cudaError_t shared_expert_window(const TsumujiMoe* d, const TsumujiWs& w, int N, int H, int F, float* y_out, cudaStream_t st) {
  cudaError_t e;
  // w.sh_x / w.sh_ranges: the hi / lo split of x, written by route_window
  const unsigned blocks_x = unsigned((size_t(N) * H + 255) / 256), blocks_h = unsigned((size_t(N) * F + 255) / 256);
  if ((e = launch_grouped_bf16(w.sh_out, w.sh_acc, w.sh_x, d->shared_gu, w.sh_ranges, 1, unsigned(2 * F), unsigned(H), nullptr, st, 0))) return e;
  if ((e = launch_pdl(shared_swiglu_kernel, dim3(blocks_h), dim3(256), 0, st, (const float*)w.sh_acc, N, F, w.sh_h))) return e;
  if ((e = launch_grouped_bf16(w.sh_out, w.sh_acc, w.sh_h, d->shared_down, w.sh_ranges, 1, unsigned(H), unsigned(F), nullptr, st, 0))) return e;
  return launch_pdl(add_halves_kernel, dim3(blocks_x), dim3(256), 0, st, (const float*)w.sh_acc, N, H, y_out);
}

static int dense_k_split(int k, long long slabs) {
  const long long warps = (long long)sm_count() * kGemvWarps;
  int best = 1;
  for (int ks = 1; ks <= 12; ++ks)
    if (kGemvWarps % ks == 0 && k % (32 * ks) == 0 && slabs * ks <= warps) best = ks;
  return best;
}

}  // namespace dmoe

using namespace dmoe;

extern "C" size_t tsumuji_moe_workspace_bytes(int hidden, int inter, int experts, int topk, int tokens) {
  return carve(nullptr, hidden, inter, experts, topk, tokens).bytes;
}

extern "C" int tsumuji_moe_workspace_init(void* workspace, size_t bytes, cudaStream_t st) {
  if (!workspace || !bytes) return cudaErrorInvalidValue;
  return cudaMemsetAsync(workspace, 0, bytes < 4096 ? bytes : 4096, st);
}

extern "C" int tsumuji_moe_layer(const TsumujiMoe* d, cudaStream_t st) {
  if (!d || !d->experts_w || !d->gs || !d->shared_gu || !d->shared_down || !d->x || (!d->out && !d->R) || !d->rlogits || !d->sel ||
      !d->rw || !d->shared_gate || !d->workspace)
    return cudaErrorInvalidValue;
  const int H = d->hidden, F = d->inter, E = d->experts, K = d->topk, N = d->tokens;
  // the reference limits: E <= 1024, top-k <= 32, H and F multiples of 32 (tsumuji-engine/src/config.rs:185-195);
  // the tiles here want multiples of 256
  if (H <= 0 || F <= 0 || H % 256 || F % 256 || E < K || E > 1024 || K < 1 || K > 32 || N < 1) return cudaErrorInvalidValue;
  if (d->workspace_bytes < tsumuji_moe_workspace_bytes(H, F, E, K, N)) return cudaErrorInvalidValue;
  const TsumujiWs w = carve(d->workspace, H, F, E, K, N);
  const RouteArgs route{d->rlogits, E + 1, E, K, N, nullptr, 1.f, d->sel, d->rw, d->shared_gate};
  const PermuteArgs perm{d->sel, N, K, E, w.assignments, w.ranges, w.active, w.counters, w.status, w.plan, 0};
  cudaError_t e;
  if (N > kWindowTokens) {
    if ((e = cudaMemsetAsync(w.counters, 0, 16, st))) return e;
    if ((e = route_window(d->router_w, d->x, route, perm, w, H, E, N, st))) return e;
  } else if (d->router_w) {
    // router projection (bf16 [E+1][H], row E = shared-expert gate), top-k, permutation, activation planes
    RouterArgs r = {};
    r.w = d->router_w; r.x = d->x; r.logits = d->rlogits; r.hidden = H; r.rows = E + 1; r.ld = E + 1; r.tokens = N;
    r.route = route; r.perm = perm; r.done = w.done; r.fuse = 1;
    r.planes = w.xplanes; r.xsum_planes = nullptr; r.planes_natural = 1;
    const size_t hist = size_t(E + 1) * 4 + size_t(N * K <= kRouteIdCache ? N * K : 0) * 4;
    if ((e = launch_pdl(router_kernel<__nv_bfloat16, float, kRouteTsumuji>, dim3(E + 1 + N), dim3(128), hist, st, r))) return e;
  } else {
    // logits supplied by the caller (the reference computes them with its dense GEMV, engine.rs:1589)
    if ((e = launch_pdl(route_permute_kernel<kRouteTsumuji>, dim3(1), dim3(128), size_t(E + 1) * 4, st, route, perm))) return e;
    if ((e = launch_pdl(act_planes_kernel<float>, dim3(N), dim3(128), 0, st, d->x, H, w.xplanes, (__half*)nullptr, 1))) return e;
  }
  const unsigned long long fh = (unsigned long long)F * H;
  const uint8_t* base = static_cast<const uint8_t*>(d->experts_w);
  // routed gate/up
  GemvArgs a = {};
  a.w[0] = base; a.w[1] = base + fh / 2;
  a.expert_stride[0] = a.expert_stride[1] = fh * 27 / 16;
  a.scale_offset[0] = fh * 3 / 2; a.scale_offset[1] = fh * 3 / 2 + fh / 16 - fh / 2;
  a.row_bytes = H / 2; a.k = H; a.rows = F; a.nblk = H / 256;
  a.gscale = reinterpret_cast<const uint8_t*>(d->gs); a.gscale_estride = 12; a.gscale_mstride = 4;
  a.xplanes = w.xplanes; a.x_by_assignment = 0;
  a.counters = w.counters + 2; a.plan = w.plan; a.assignments = w.assignments;
  a.tokens = N; a.topk = K; a.max_groups = N * K < E ? N * K : E;
  a.out_planes = w.hplanes; a.status = w.status;
  if ((e = launch_gemv<kGemvNvfp4Linear, 1, false, kOutSiluPlanes>(a, st))) return e;
  const bool window = N > kWindowTokens && H % 64 == 0 && F % 64 == 0;
  if (window) {
    if ((e = shared_expert_window(d, w, N, H, F, w.y + size_t(N) * K * H, st))) return e;
  } else {
    // shared gate/up (dense bf16 [2F][H])
    DenseArgs s = {};
    s.w[0] = static_cast<const __nv_bfloat16*>(d->shared_gu); s.w[1] = s.w[0] + size_t(F) * H;
    s.k = H; s.rows = F; s.ks = dense_k_split(H, (F + 7) / 8);
    s.xplanes = w.xplanes; s.x_row0 = 0; s.tokens = N; s.out_planes = w.hplanes; s.out_row0 = N * K;
    if ((e = launch_pdl(dense_gemv_kernel<1>, dim3(sm_count()), dim3(kGemvWarps * 32), 0, st, s))) return e;
  }
  // routed down
  GemvArgs b = a;
  b.w[0] = base + fh; b.w[1] = nullptr;
  b.scale_offset[0] = fh * 3 / 2 + fh / 8 - fh; b.scale_offset[1] = 0;
  b.row_bytes = F / 2; b.k = F; b.rows = H; b.nblk = F / 256;
  b.gscale = reinterpret_cast<const uint8_t*>(d->gs) + 8;
  b.xplanes = w.hplanes; b.x_by_assignment = 1; b.out_planes = nullptr; b.out = w.y;
  b.late_wait = 1;           // the plan is the router's; the predecessor (shared gate/up) only adds product rows
  if ((e = launch_gemv<kGemvNvfp4Linear, 0, false, kOutFloat>(b, st))) return e;
  if (!window) {
    // shared down (dense bf16 [H][F])
    DenseArgs t = {};
    t.w[0] = static_cast<const __nv_bfloat16*>(d->shared_down); t.w[1] = nullptr;
    t.k = F; t.rows = H; t.ks = dense_k_split(F, (H + 15) / 16);
    t.xplanes = w.hplanes; t.x_row0 = N * K; t.tokens = N; t.out = w.y; t.out_row0 = N * K;
    if ((e = launch_pdl(dense_gemv_kernel<0>, dim3(sm_count()), dim3(kGemvWarps * 32), 0, st, t))) return e;
  }
  TsumujiWriteback wb = {};
  if (d->R) {
    if (!d->di || !d->ss || d->HC < 1 || d->HC > 8 || d->Sd < 1 || d->ld < d->rank + d->HC || d->rank < 0) return cudaErrorInvalidValue;
    wb = TsumujiWriteback{d->R, d->di, d->Sd, d->ld, d->rank, d->HC, d->ss};
  }
  return launch_pdl(tsumuji_combine_kernel, dim3((H + 255) / 256, N), dim3(256), 0, st, d->out, (const float*)w.y,
                    (const float*)d->rw, (const float*)d->shared_gate, H, K, N, d->accumulate, wb);
}

// ---- expert-parallel entry points (rank g holds experts [g*E/G, (g+1)*E/G) and its own tokens) ---------------------------
static void routed_args(GemvArgs& a, GemvArgs& b, const void* experts_w, const float* gs, int H, int F) {
  const unsigned long long fh = (unsigned long long)F * H;
  const uint8_t* base = static_cast<const uint8_t*>(experts_w);
  a = GemvArgs{};
  a.w[0] = base; a.w[1] = base + fh / 2;
  a.expert_stride[0] = a.expert_stride[1] = fh * 27 / 16;
  a.scale_offset[0] = fh * 3 / 2; a.scale_offset[1] = fh * 3 / 2 + fh / 16 - fh / 2;
  a.row_bytes = H / 2; a.k = H; a.rows = F; a.nblk = H / 256;
  a.gscale = reinterpret_cast<const uint8_t*>(gs); a.gscale_estride = 12; a.gscale_mstride = 4;
  b = a;
  b.w[0] = base + fh; b.w[1] = nullptr;
  b.scale_offset[0] = fh * 3 / 2 + fh / 8 - fh; b.scale_offset[1] = 0;
  b.row_bytes = F / 2; b.k = F; b.rows = H; b.nblk = F / 256;
  b.gscale = reinterpret_cast<const uint8_t*>(gs) + 8;
}

extern "C" int tsumuji_ep_dispatch(const TsumujiMoe* d, float* send_x, unsigned* ranges, unsigned* position, float* y_shared,
                                   cudaStream_t st) {
  if (!d || !d->router_w || !d->shared_gu || !d->shared_down || !d->x || !d->rlogits || !d->sel || !d->rw || !d->shared_gate ||
      !d->workspace || !send_x || !ranges || !position || !y_shared)
    return cudaErrorInvalidValue;
  const int H = d->hidden, F = d->inter, E = d->experts, K = d->topk, N = d->tokens;
  if (H <= 0 || F <= 0 || H % 256 || F % 256 || E < K || E > 1024 || K < 1 || K > 32 || N < 1) return cudaErrorInvalidValue;
  if (d->workspace_bytes < tsumuji_moe_workspace_bytes(H, F, E, K, N)) return cudaErrorInvalidValue;
  const TsumujiWs w = carve(d->workspace, H, F, E, K, N);
  cudaError_t e;
  const RouteArgs route{d->rlogits, E + 1, E, K, N, nullptr, 1.f, d->sel, d->rw, d->shared_gate};
  const PermuteArgs perm{d->sel, N, K, E, w.assignments, ranges, w.active, w.counters, w.status, w.plan, 0};
  if (N > kWindowTokens) {
    if ((e = cudaMemsetAsync(w.counters, 0, 16, st))) return e;
    if ((e = route_window(d->router_w, d->x, route, perm, w, H, E, N, st))) return e;
  } else {
    RouterArgs r = {};
    r.w = d->router_w; r.x = d->x; r.logits = d->rlogits; r.hidden = H; r.rows = E + 1; r.ld = E + 1; r.tokens = N;
    r.route = route; r.perm = perm;
    r.done = w.done; r.fuse = 1;
    r.planes = w.xplanes; r.xsum_planes = nullptr; r.planes_natural = 1;
    const size_t hist = size_t(E + 1) * 4 + size_t(N * K <= kRouteIdCache ? N * K : 0) * 4;
    if ((e = launch_pdl(router_kernel<__nv_bfloat16, float, kRouteTsumuji>, dim3(E + 1 + N), dim3(128), hist, st, r))) return e;
  }
  if ((e = launch_pdl(tsumuji_gather_kernel, dim3(N * K), dim3(256), 0, st, d->x, (const unsigned*)w.assignments, (const int*)w.counters, K,
                      H, send_x, position))) return e;
  // the shared expert stays on the home rank (dense bf16), its rows go straight to y_shared
  if (N > kWindowTokens && H % 64 == 0 && F % 64 == 0) return shared_expert_window(d, w, N, H, F, y_shared, st);
  DenseArgs s = {};
  s.w[0] = static_cast<const __nv_bfloat16*>(d->shared_gu); s.w[1] = s.w[0] + size_t(F) * H;
  s.k = H; s.rows = F; s.ks = dense_k_split(H, (F + 7) / 8);
  s.xplanes = w.xplanes; s.x_row0 = 0; s.tokens = N; s.out_planes = w.hplanes; s.out_row0 = 0;
  if ((e = launch_pdl(dense_gemv_kernel<1>, dim3(sm_count()), dim3(kGemvWarps * 32), 0, st, s))) return e;
  DenseArgs t = {};
  t.w[0] = static_cast<const __nv_bfloat16*>(d->shared_down); t.w[1] = nullptr;
  t.k = F; t.rows = H; t.ks = dense_k_split(F, (H + 15) / 16);
  t.xplanes = w.hplanes; t.x_row0 = 0; t.tokens = N; t.out = y_shared; t.out_row0 = 0;
  return launch_pdl(dense_gemv_kernel<0>, dim3(sm_count()), dim3(kGemvWarps * 32), 0, st, t);
}

extern "C" size_t tsumuji_ep_experts_workspace_bytes(int hidden, int inter, int local_experts, int rows) {
  if (hidden < 1 || inter < 1 || local_experts < 1 || rows < 1) return 0;
  return carve(nullptr, hidden, inter, local_experts, 1, rows).bytes + align_up(size_t(rows) * 4, 256) +
         align_up(permute_scratch_bytes(rows, 1, local_experts), 256);
}

extern "C" int tsumuji_ep_experts(const void* experts_w, const float* gs, int hidden, int inter, int local_experts, int ranks,
                                  const int* recv_counts, const float* x_rows, int rows, float* y_rows, void* workspace,
                                  size_t workspace_bytes, cudaStream_t st) {
  if (!experts_w || !gs || !recv_counts || !x_rows || !y_rows || !workspace || hidden <= 0 || inter <= 0 || hidden % 256 ||
      inter % 256 || local_experts < 1 || local_experts > 1024 || ranks < 1 || rows < 1 ||
      workspace_bytes < tsumuji_ep_experts_workspace_bytes(hidden, inter, local_experts, rows))
    return cudaErrorInvalidValue;
  const TsumujiWs w = carve(workspace, hidden, inter, local_experts, 1, rows);
  int* ids = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + w.bytes);
  void* perm_scratch = reinterpret_cast<uint8_t*>(ids) + align_up(size_t(rows) * 4, 256);
  cudaError_t e;
  if ((e = cudaMemsetAsync(w.counters, 0, 16, st))) return e;
  if ((e = launch_pdl(ep_row_experts_kernel, dim3(ranks * local_experts), dim3(128), 0, st, recv_counts, ranks, local_experts, ids))) return e;
  const PermuteArgs perm{ids, rows, 1, local_experts, w.assignments, w.ranges, w.active, w.counters, w.status, w.plan, 0};
  if (rows > 2048) {
    if ((e = launch_permute_large(perm, perm_scratch, st))) return e;
  } else if ((e = launch_pdl(permute_kernel<0>, dim3(1), dim3(1024), size_t(local_experts + 1) * 4, st, perm))) return e;
  if ((e = launch_pdl(act_planes_kernel<float>, dim3(rows), dim3(128), 0, st, x_rows, hidden, w.xplanes, (__half*)nullptr, 1))) return e;
  GemvArgs a, b;
  routed_args(a, b, experts_w, gs, hidden, inter);
  a.xplanes = w.xplanes; a.x_by_assignment = 0;
  a.counters = w.counters + 2; a.plan = w.plan; a.assignments = w.assignments;
  a.tokens = rows; a.topk = 1; a.max_groups = rows < local_experts ? rows : local_experts;
  a.out_planes = w.hplanes; a.status = w.status;
  if ((e = launch_gemv<kGemvNvfp4Linear, 1, false, kOutSiluPlanes>(a, st))) return e;
  b.counters = a.counters; b.plan = a.plan; b.assignments = a.assignments; b.tokens = rows; b.topk = 1; b.max_groups = a.max_groups;
  b.status = w.status;
  b.xplanes = w.hplanes; b.x_by_assignment = 1; b.out_planes = nullptr; b.out = y_rows;
  return launch_gemv<kGemvNvfp4Linear, 0, false, kOutFloat>(b, st);
}

extern "C" int tsumuji_ep_combine(float* out, const float* y_home, const float* rw, const unsigned* position, const float* shared_gate,
                                  const float* y_shared, int tokens, int hidden, int topk, int accumulate, cudaStream_t st) {
  if (!out || !y_home || !rw || !position || !shared_gate || !y_shared || tokens < 1 || hidden < 1 || topk < 1) return cudaErrorInvalidValue;
  return launch_pdl(tsumuji_ep_combine_kernel, dim3((hidden + 255) / 256, tokens), dim3(256), 0, st, out, y_home, rw, position, shared_gate,
                    y_shared, hidden, topk, accumulate);
}
