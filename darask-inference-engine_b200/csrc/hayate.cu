// Hayate (GLM) MoE FFN: sigmoid + bias router, NVFP4 expert images in the tiled-scale layout, bf16
// activations, bf16-rounded products and an expert-id-ordered bf16 reduction.
// Reference: hayate crates/kernels/cu/glm53/decode.cu:18-88 (router_project, router_select, gate_up, down,
// sum and their launchers), ops.cu:100-114 (prefill router), math.cuh:31-49; call sites hayate
// crates/models/src/glm53/gpu.rs:1612-1905.
// This translation unit is compiled with --use_fast_math, as the reference builds its GLM kernels
// (hayate crates/kernels/build.rs:59), so that sigmoid(logit) + bias is formed with the same approximate
// exp / reciprocal and selects the same experts.
#include "../../include/darask_moe_b200.h"
#include "gemv_launch.cuh"
#include "route_kernels.cuh"

namespace dmoe {

// reference literals (hayate crates/models/src/glm53/mod.rs:15-18); changed by hayate_glm_moe_set_shape
struct HayateShape { int hidden = 4096, inter = 2048, experts = 288, topk = 8; float scale = 2.5f; void* ws = nullptr; size_t ws_bytes = 0; };
static thread_local HayateShape g_shape;

template <typename XT>
__global__ void __launch_bounds__(128) hayate_planes_kernel(const XT* x0, const XT* x1, int rows0, int k, __half* planes) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  const XT* src = t < rows0 ? x0 + size_t(t) * k : x1 + size_t(t - rows0) * k;
  act_planes_row(src, k, planes + size_t(t) * 2 * k, nullptr, true);
}

// plan for one token whose experts are given as an image pointer table in top-k order: group g = slot g,
// plus the shared expert; rows of empty (null) images are zeroed in `zero_rows`.
__global__ void hayate_slot_plan_kernel(const void* const* images, int topk, int4* plan, unsigned* assignments, int* counters,
                                        __nv_bfloat16* zero_rows, int row_len) {
  pdl_wait();
  pdl_launch();
  for (int g = threadIdx.x; g < topk; g += blockDim.x) {
    const bool present = images[g] != nullptr;
    plan[g] = make_int4(g, present ? 1 : 0, g, 0);
    assignments[g] = g;
    if (!present && zero_rows)
      for (int i = 0; i < row_len; ++i) zero_rows[size_t(g) * row_len + i] = __float2bfloat16_rn(0.f);
  }
  if (threadIdx.x == 0) {
    plan[topk] = make_int4(-1, 1, 0, 0);
    counters[0] = topk;
    counters[1] = topk;
    counters[2] = topk + 1;
  }
}

// out[t][c] = sum over the token's experts in ascending expert id of bf16(sum + bf16(y * w)), then + shared
// (decode.cu:55-59, math.cuh:35-39). y: bf16 [T*k + T][hidden].
__global__ void __launch_bounds__(256) hayate_reduce_kernel(__nv_bfloat16* out, const __nv_bfloat16* y, const int* ids,
                                                            const float* weights, int hidden, int topk, int tokens,
                                                            int shared_row0) {
  pdl_wait();
  pdl_launch();
  const int c = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
  if (c >= hidden) return;
  int order[32];
  for (int i = 0; i < topk; ++i) order[i] = i;
  for (int i = 1; i < topk; ++i) {                 // stable insertion sort by expert id (route_order)
    const int v = order[i];
    int j = i;
    while (j && ids[t * topk + order[j - 1]] > ids[t * topk + v]) {
      order[j] = order[j - 1];
      --j;
    }
    order[j] = v;
  }
  float value = 0.f;
  for (int g = 0; g < topk; ++g) {
    const int s = order[g];
    value = bf16_rn(value + bf16_rn(__bfloat162float(y[size_t(t * topk + s) * hidden + c]) * weights[t * topk + s]));
  }
  out[size_t(t) * hidden + c] = __float2bfloat16_rn(value + __bfloat162float(y[size_t(shared_row0 + t) * hidden + c]));
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
struct HayateWs {
  int* counters; unsigned* done; unsigned* status; int* active; unsigned* ranges; unsigned* assignments; int4* plan;
  __half* xplanes; __half* hplanes; __nv_bfloat16* product; __nv_bfloat16* y; size_t bytes;
};
static HayateWs carve(void* base, int hidden, int inter, int experts, int topk, int tokens) {
  HayateWs w;
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
  const size_t rows = size_t(tokens) * topk + tokens;
  const size_t widest = hidden > inter ? hidden : inter;
  w.xplanes = reinterpret_cast<__half*>(take((rows > 2 * size_t(tokens) ? rows : 2 * size_t(tokens)) * 2 * widest * 2));
  w.hplanes = reinterpret_cast<__half*>(take(rows * 2 * inter * 2));
  w.product = reinterpret_cast<__nv_bfloat16*>(take(rows * inter * 2));
  w.y = reinterpret_cast<__nv_bfloat16*>(take(rows * hidden * 2));
  w.bytes = off;
  return w;
}

static unsigned long long tiled_scale_offset(int n, int k) { return (unsigned long long)n * k / 2; }
static unsigned long long tiled_global_offset(int n, int k) {
  return (unsigned long long)n * k / 2 + (unsigned long long)((n + 127) / 128 * 128) * ((k / 16 + 3) / 4 * 4);
}

// gate/up (DUAL) or down launch over NVFP4 tiled images
static cudaError_t launch_hayate_gemv(bool dual, GemvArgs a, int n, int k, cudaStream_t st) {
  a.row_bytes = k / 2; a.k = k; a.rows = n; a.nblk = k / 256;
  a.scale_offset[0] = a.scale_offset[1] = tiled_scale_offset(n, k);
  a.gscale_in_matrix[0] = a.gscale_in_matrix[1] = tiled_global_offset(n, k);
  a.round_shared = 1;      // the shared expert's weights are bf16-rounded (decode.cu:44-45,52: `rounded` = g==8)
  return dual ? launch_gemv<kGemvNvfp4Tiled, 1, false, kOutHayateProduct>(a, st) : launch_gemv<kGemvNvfp4Tiled, 0, false, kOutBf16>(a, st);
}

// the same over block-FP8 images: payload [n][k] e4m3, float32 scales [n/128][k/128] right behind it
// (decode.cu:32-36 `routed`: scale = w + n*k); the shared expert's scales come with its DenseWeight
static cudaError_t launch_hayate_gemv_fp8(bool dual, GemvArgs a, int n, int k, cudaStream_t st) {
  a.row_bytes = k; a.k = k; a.rows = n; a.nblk = k / 256;
  a.scale_offset[0] = a.scale_offset[1] = (unsigned long long)n * k;
  return dual ? launch_gemv<kGemvFp8Block, 1, false, kOutHayateProduct>(a, st) : launch_gemv<kGemvFp8Block, 0, false, kOutBf16>(a, st);
}

}  // namespace dmoe

using namespace dmoe;

extern "C" int darask_route_topk_hayate(const float* logits, int ld, int experts, int topk, int tokens,
                                        const float* bias, float scale, int* ids, float* weights, cudaStream_t st) {
  if (!logits || !bias || !ids || !weights || experts < 1 || experts > 1024 || topk < 1 || topk > 32 ||
      topk > experts || tokens < 1 || ld < experts)
    return cudaErrorInvalidValue;
  RouteArgs a{logits, ld, experts, topk, tokens, bias, scale, ids, weights, nullptr};
  return launch_pdl(route_topk_kernel<kRouteHayate>, dim3((tokens + 3) / 4), dim3(128), 0, st, a);
}

extern "C" int hayate_glm_moe_set_shape(unsigned hidden, unsigned inter, unsigned experts, unsigned topk, float scale) {
  if (!hidden || !inter || hidden % 256 || inter % 256 || hidden % 128 || inter % 128 || !experts || experts > 1024 ||
      !topk || topk > 32 || topk > experts)
    return cudaErrorInvalidValue;
  g_shape.hidden = int(hidden); g_shape.inter = int(inter); g_shape.experts = int(experts); g_shape.topk = int(topk);
  g_shape.scale = scale;
  return cudaSuccess;
}

namespace dmoe { int hayate_shape_topk() { return g_shape.topk; } }

extern "C" size_t hayate_glm_moe_workspace_bytes(unsigned hidden, unsigned inter, unsigned experts, unsigned topk, unsigned tokens) {
  return carve(nullptr, int(hidden), int(inter), int(experts), int(topk), int(tokens)).bytes;
}

extern "C" int hayate_glm_moe_set_workspace(void* workspace, size_t bytes, cudaStream_t st) {
  if (workspace && bytes < 4096) return cudaErrorInvalidValue;
  g_shape.ws = workspace;
  g_shape.ws_bytes = bytes;
  return workspace ? cudaMemsetAsync(workspace, 0, 4096, st) : cudaSuccess;
}

// ---- router ---------------------------------------------------------------------------------------------
static cudaError_t hayate_route_impl(float* logits, float* weights, int* ids, const void* x, const void* w, const float* bias,
                                     int tokens, int hidden, int experts, int topk, float scale, unsigned* done,
                                     const PermuteArgs* perm, __half* planes, cudaStream_t st) {
  RouterArgs r = {};
  r.w = w; r.x = x; r.logits = logits; r.hidden = hidden; r.rows = experts; r.ld = experts; r.tokens = tokens;
  r.route = RouteArgs{logits, experts, experts, topk, tokens, bias, scale, ids, weights, nullptr};
  if (perm) r.perm = *perm;
  r.done = done; r.fuse = 1; r.planes = planes; r.planes_natural = 1;
  const size_t hist = size_t(experts + 1) * 4 + size_t(tokens * topk <= kRouteIdCache ? tokens * topk : 0) * 4;
  return launch_pdl(router_kernel<__nv_bfloat16, __nv_bfloat16, kRouteHayate>, dim3(experts + (planes ? tokens : 0)), dim3(128), hist, st, r);
}

extern "C" int hayate_glm_route(void* logits, void* weights, void* ids, const void* x, const void* w, const void* bias,
                                unsigned tokens, unsigned hidden, unsigned experts, unsigned topk, cudaStream_t st) {
  if (!logits || !weights || !ids || !x || !w || !bias || !tokens || !hidden || hidden % 8 || !experts || experts > 1024 ||
      !topk || topk > 32 || topk > experts)
    return cudaErrorInvalidValue;
  if (g_shape.ws) {      // fused: the last block of the projection selects
    const HayateWs ws = carve(g_shape.ws, g_shape.hidden, g_shape.inter, g_shape.experts, g_shape.topk, 1);
    return hayate_route_impl((float*)logits, (float*)weights, (int*)ids, x, w, (const float*)bias, int(tokens), int(hidden),
                             int(experts), int(topk), g_shape.scale, ws.done, nullptr, nullptr, st);
  }
  RouterArgs r = {};     // no workspace registered: projection and selection as two launches
  r.w = w; r.x = x; r.logits = (float*)logits; r.hidden = int(hidden); r.rows = int(experts); r.ld = int(experts); r.tokens = int(tokens);
  cudaError_t e = launch_pdl(router_kernel<__nv_bfloat16, __nv_bfloat16, kRouteHayate>, dim3(experts), dim3(128), size_t(experts + 1) * 4, st, r);
  if (e) return e;
  return darask_route_topk_hayate((const float*)logits, int(experts), int(experts), int(topk), int(tokens), (const float*)bias,
                                  g_shape.scale, (int*)ids, (float*)weights, st);
}

extern "C" int hayate_glm_route_decode(void* logits, void* weights, void* ids, const void* x, const void* w, const void* bias,
                                       cudaStream_t st) {
  return hayate_glm_route(logits, weights, ids, x, w, bias, 1, unsigned(g_shape.hidden), unsigned(g_shape.experts),
                          unsigned(g_shape.topk), st);
}

extern "C" int hayate_glm_route_batch(void* logits, void* weights, void* ids, const void* x, const void* w, const void* bias,
                                      unsigned m, cudaStream_t st) {
  if (m < 1 || m > 4) return cudaErrorInvalidValue;
  return hayate_glm_route(logits, weights, ids, x, w, bias, m, unsigned(g_shape.hidden), unsigned(g_shape.experts),
                          unsigned(g_shape.topk), st);
}

// ---- one-token expert products with the reference's signatures ---------------------------------------------
extern "C" int hayate_glm_moe_gate_up(void* out, const void* x, const void* original, const void* images,
                                      HayateDenseWeight gate, HayateDenseWeight up, int nv, int down_fp8, size_t stride,
                                      cudaStream_t st) {
  if (!out || !x || !original || !images || !gate.data || !up.data || !stride || !g_shape.ws) return cudaErrorInvalidValue;
  // routed and shared expert in one launch: both NVFP4 (nv, format 3) or both block-FP8 (!nv, format 1 with scales)
  const bool fp8 = !nv;
  if (fp8 ? (gate.format != 1 || up.format != 1 || !gate.scale || !up.scale) : (gate.format != 3 || up.format != 3)) return cudaErrorInvalidValue;
  (void)down_fp8;
  const int H = g_shape.hidden, F = g_shape.inter, K = g_shape.topk;
  const HayateWs ws = carve(g_shape.ws, H, F, g_shape.experts, K, 1);
  cudaError_t e;
  if ((e = launch_pdl(hayate_slot_plan_kernel, dim3(1), dim3(32), 0, st, (const void* const*)images, K, ws.plan, ws.assignments,
                      ws.counters, (__nv_bfloat16*)out, F))) return e;
  if ((e = launch_pdl(hayate_planes_kernel<__nv_bfloat16>, dim3(2), dim3(128), 0, st, (const __nv_bfloat16*)x,
                      (const __nv_bfloat16*)original, 1, H, ws.xplanes))) return e;
  GemvArgs a = {};
  a.w_table = (const void* const*)images; a.matrix_stride = stride;
  a.w_shared[0] = static_cast<const uint8_t*>(gate.data); a.w_shared[1] = static_cast<const uint8_t*>(up.data);
  a.xplanes = ws.xplanes; a.x_by_assignment = 0; a.shared_x_row0 = 1;
  a.counters = ws.counters + 2; a.plan = ws.plan; a.assignments = ws.assignments;
  a.tokens = 1; a.topk = K; a.max_groups = K + 1;
  a.out_planes = ws.hplanes; a.out_bf16 = (__nv_bfloat16*)out; a.status = ws.status;
  if (fp8) {
    a.scale_shared[0] = static_cast<const float*>(gate.scale); a.scale_shared[1] = static_cast<const float*>(up.scale);
    return launch_hayate_gemv_fp8(true, a, F, H, st);
  }
  return launch_hayate_gemv(true, a, F, H, st);
}

extern "C" int hayate_glm_moe_down(void* out, const void* x, const void* images, HayateDenseWeight shared, int nv, int down_fp8,
                                   size_t stride, cudaStream_t st) {
  if (!out || !x || !images || !shared.data || !stride || !g_shape.ws) return cudaErrorInvalidValue;
  const bool fp8 = !nv || down_fp8;     // the down matrices are block-FP8 (decode.cu:32-36)
  if (fp8 ? (shared.format != 1 || !shared.scale) : shared.format != 3) return cudaErrorInvalidValue;
  const int H = g_shape.hidden, F = g_shape.inter, K = g_shape.topk;
  const HayateWs ws = carve(g_shape.ws, H, F, g_shape.experts, K, 1);
  cudaError_t e;
  if ((e = launch_pdl(hayate_slot_plan_kernel, dim3(1), dim3(32), 0, st, (const void* const*)images, K, ws.plan, ws.assignments,
                      ws.counters, (__nv_bfloat16*)nullptr, 0))) return e;
  // the products may have been changed by the caller (rotation): planes are rebuilt from the bf16 rows
  if ((e = launch_pdl(hayate_planes_kernel<__nv_bfloat16>, dim3(K + 1), dim3(128), 0, st, (const __nv_bfloat16*)x,
                      (const __nv_bfloat16*)x, K + 1, F, ws.xplanes))) return e;
  GemvArgs a = {};
  a.w_table = (const void* const*)images; a.matrix_stride = 0; a.expert_stride[0] = 2 * stride;   // down is the third matrix
  a.w_shared[0] = static_cast<const uint8_t*>(shared.data);
  a.xplanes = ws.xplanes; a.x_by_assignment = 1;
  a.counters = ws.counters + 2; a.plan = ws.plan; a.assignments = ws.assignments;
  a.tokens = 1; a.topk = K; a.max_groups = K + 1;
  a.out_bf16 = (__nv_bfloat16*)out; a.status = ws.status;
  if (fp8) {
    a.scale_shared[0] = static_cast<const float*>(shared.scale);
    return launch_hayate_gemv_fp8(false, a, H, F, st);
  }
  return launch_hayate_gemv(false, a, H, F, st);
}

extern "C" int hayate_glm_moe_reduce(void* out, const void* x, const void* ids, const void* weights, cudaStream_t st) {
  if (!out || !x || !ids || !weights) return cudaErrorInvalidValue;
  return launch_pdl(hayate_reduce_kernel, dim3((g_shape.hidden + 255) / 256, 1), dim3(256), 0, st, (__nv_bfloat16*)out,
                    (const __nv_bfloat16*)x, (const int*)ids, (const float*)weights, g_shape.hidden, g_shape.topk, 1, g_shape.topk);
}

// ---- whole layer for `tokens` tokens, all expert images resident in one slab ---------------------------------
extern "C" size_t hayate_moe_workspace_bytes(int hidden, int inter, int experts, int topk, int tokens) {
  return carve(nullptr, hidden, inter, experts, topk, tokens).bytes;
}
extern "C" int hayate_moe_workspace_init(void* workspace, size_t bytes, cudaStream_t st) {
  if (!workspace || !bytes) return cudaErrorInvalidValue;
  return cudaMemsetAsync(workspace, 0, bytes < 4096 ? bytes : 4096, st);
}

extern "C" int hayate_moe_layer(const HayateMoe* d, cudaStream_t st) {
  if (!d || !d->router_w || !d->bias || !d->images || !d->shared_image || !d->x || !d->out || !d->logits || !d->ids ||
      !d->weights || !d->workspace)
    return cudaErrorInvalidValue;
  const int H = d->hidden, F = d->inter, E = d->experts, K = d->topk, T = d->tokens;
  if (H <= 0 || F <= 0 || H % 256 || F % 256 || E < K || E > 1024 || K < 1 || K > 32 || T < 1 || !d->stride || d->stride % 16)
    return cudaErrorInvalidValue;
  if (d->workspace_bytes < hayate_moe_workspace_bytes(H, F, E, K, T)) return cudaErrorInvalidValue;
  const HayateWs w = carve(d->workspace, H, F, E, K, T);
  const PermuteArgs perm{d->ids, T, K, E, w.assignments, w.ranges, w.active, w.counters, w.status, w.plan, T};
  cudaError_t e;
  if ((e = hayate_route_impl(d->logits, d->weights, d->ids, d->x, d->router_w, d->bias, T, H, E, K, d->scale, w.done, &perm,
                             w.xplanes, st))) return e;
  const uint8_t* images = static_cast<const uint8_t*>(d->images);
  const uint8_t* shared = static_cast<const uint8_t*>(d->shared_image);
  GemvArgs a = {};
  a.w[0] = images; a.w[1] = images + d->stride;
  a.expert_stride[0] = a.expert_stride[1] = 3ull * d->stride;
  a.w_shared[0] = shared; a.w_shared[1] = shared + d->stride;
  a.xplanes = w.xplanes; a.x_by_assignment = 0;
  a.counters = w.counters + 2; a.plan = w.plan; a.assignments = w.assignments;
  a.tokens = T; a.topk = K; a.max_groups = (T * K < E ? T * K : E) + 1;
  a.out_planes = w.hplanes; a.out_bf16 = w.product; a.status = w.status;
  if ((e = launch_hayate_gemv(true, a, F, H, st))) return e;
  GemvArgs b = a;
  b.w[0] = images + 2 * d->stride; b.w[1] = nullptr;
  b.w_shared[0] = shared + 2 * d->stride; b.w_shared[1] = nullptr;
  b.xplanes = w.hplanes; b.x_by_assignment = 1; b.out_planes = nullptr; b.out_bf16 = w.y;
  b.late_wait = 1;           // the plan is the router's (two launches back); only the products come from gate/up
  if ((e = launch_hayate_gemv(false, b, H, F, st))) return e;
  return launch_pdl(hayate_reduce_kernel, dim3((H + 255) / 256, T), dim3(256), 0, st, static_cast<__nv_bfloat16*>(d->out),
                    (const __nv_bfloat16*)w.y, (const int*)d->ids, (const float*)d->weights, H, K, T, T * K);
}
