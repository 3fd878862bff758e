// Kogarashi (Qwen3.5-MoE, GGUF Q4_K / Q6_K) MoE FFN layer for 1..N tokens as four launches:
//   router projection + top-k + dispatch permutation + activation planes  (reference: `gemv` on ffn_gate_inp, `route`)
//   gate/up products with SwiGLU                        (`gemv` x2, `activate`, also the shared expert)
//   down products                                       (`gemv`, also the shared expert)
//   weighted combine into the residual stream           (`combine`)
// Reference call site: kogarashi crates/kogarashi-engine/src/engine.rs:530-632; kernels
// kogarashi kernels/native.cu:46-117. The reference runs 12 launches per layer for one token.
#include "../../include/darask_moe_b200.h"
#include "route_kernels.cuh"
#include "stream_launch.cuh"
#include "gemv_launch.cuh"
#include "decode_fused.cuh"
#include <cstdio>

namespace dmoe {

// x[t][i] += sum_s fma(p[t][s], y[t*k+s][i]) + sigmoid(sg[t]) * y[T*k+t][i]   (native.cu:113-117)
__global__ void __launch_bounds__(256) kogarashi_combine_kernel(float* x, const float* y, const float* prob,
                                                                const float* sg, int hidden, int topk, int tokens,
                                                                int has_shared) {
  pdl_wait();
  pdl_launch();
  const int i = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
  if (i >= hidden) return;
  float v = 0.f;
  for (int s = 0; s < topk; ++s) v = fmaf(__ldcg(prob + t * topk + s), __ldcg(y + size_t(t * topk + s) * hidden + i), v);
  if (has_shared) v += sigmoid_precise(__ldcg(sg + t)) * __ldcg(y + size_t(tokens * topk + t) * hidden + i);
  const float out = x[size_t(t) * hidden + i] + v;
  x[size_t(t) * hidden + i] = out;
}

// GGUF Q6_K rows (nblk x 210 bytes) <-> the row-aligned device layout read by q6k_block.
__global__ void q6k_repack_kernel(const uint8_t* src, uint8_t* dst, long long rows, int nblk, int inverse) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = nblk * 105;                 // 16-bit units of payload per row
  if (idx >= rows * per_row) return;
  const long long r = idx / per_row;
  const int u = int(idx % per_row), b = u / 105, o = (u % 105) * 2;   // byte o of block b
  const int rbytes = nblk * 208 + ((2 * nblk + 15) / 16) * 16;
  const uint8_t* g = src + (inverse ? 0 : r * (long long)nblk * 210 + b * 210 + o);
  uint8_t* d = dst + (inverse ? r * (long long)nblk * 210 + b * 210 + o : 0);
  const long long packed = r * rbytes + (o < 208 ? b * 208 + o : nblk * 208 + 2 * b);
  if (inverse) {
    d[0] = src[packed];
    d[1] = src[packed + 1];
  } else {
    dst[packed] = g[0];
    dst[packed + 1] = g[1];
  }
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct KogarashiWs {
  int* counters; unsigned* done; unsigned* status; unsigned* gbar; unsigned* tile_cnt; int* active; unsigned* ranges;
  unsigned* assignments; int4* plan; float* sg; __half* xplanes; __half* xsum_planes; __half* hplanes; float* y;
  unsigned* epoch; unsigned long long* tlog; unsigned long long* th; unsigned long long* ty;    // the one-token kernel's tagged words
  size_t bytes;
};
constexpr int kHeadKept = 256;              // bytes at the start of a workspace that only `kogarashi_moe_workspace_init` clears
constexpr int kFusedMaxRowTiles = 512;
constexpr int kFusedMaxCtas = 160;          // CTAs (SMs) the one-token kernel can run on
constexpr int kFusedMaxLogits = 320;        // router rows it can route (shared gate row included)
static int fused_logit_stride(int experts) { return ((experts + 1 < kFusedMaxLogits ? experts + 1 : kFusedMaxLogits) + 15) / 16 * 16; }      // 16-row output tiles with a completion counter (hidden <= 8192)
static KogarashiWs carve(void* base, int hidden, int inter, int experts, int topk, int tokens) {
  KogarashiWs w;
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) { uint8_t* q = p ? p + off : nullptr; off = align_up(off + bytes, 256); return q; };
  // first, at an offset that no shape moves: the call counter of the one-token kernel and the count of CTAs that have
  // read it. The built-in workspace clears the rest of the head on every call but not these: the counter has to
  // outlive a call, whatever shapes share the array, for a stale tagged word never to carry the current tag.
  w.epoch = reinterpret_cast<unsigned*>(take(8));
  w.counters = reinterpret_cast<int*>(take(16));
  w.done = reinterpret_cast<unsigned*>(take(4));
  w.status = reinterpret_cast<unsigned*>(take(4));
  w.gbar = reinterpret_cast<unsigned*>(take(16));                                   // unused (kept: the layout of the head is part of the status accessor)
  w.tile_cnt = reinterpret_cast<unsigned*>(take(size_t(kFusedMaxRowTiles) * 4));    // unused; ends at byte 3072: inside the zeroed head
  w.active = reinterpret_cast<int*>(take(size_t(experts) * 4));
  w.ranges = reinterpret_cast<unsigned*>(take(size_t(experts) * 8));
  w.assignments = reinterpret_cast<unsigned*>(take(size_t(tokens) * topk * 4));
  w.plan = reinterpret_cast<int4*>(take(size_t(experts + 1) * 16));
  w.sg = reinterpret_cast<float*>(take(size_t(tokens) * 4));
  w.xplanes = reinterpret_cast<__half*>(take(size_t(tokens) * 2 * hidden * 2));
  w.xsum_planes = reinterpret_cast<__half*>(take(size_t(tokens) * (hidden / 32) * 4));
  const size_t rows = size_t(tokens) * topk + tokens;
  w.hplanes = reinterpret_cast<__half*>(take(rows * 2 * inter * 2));
  w.y = reinterpret_cast<float*>(take(rows * hidden * 4));
  // one-token kernel: {float, tag} words
  w.tlog = reinterpret_cast<unsigned long long*>(take(size_t(kFusedMaxCtas) * fused_logit_stride(experts) * 8));   // one copy per CTA
  w.th = reinterpret_cast<unsigned long long*>(take(size_t(topk + 1) * inter * 8));
  w.ty = reinterpret_cast<unsigned long long*>(take(size_t(topk + 1) * hidden * 8));
  w.bytes = off;
  return w;
}

static int q6k_r16_row_bytes(int k) { return k / 256 * 208 + ((2 * (k / 256) + 15) / 16) * 16; }
static int row_bytes_of(int ty, int k) {
  return ty == DARASK_GGML_Q4_K ? k / 256 * 144 : ty == DARASK_GGML_Q6_K ? q6k_r16_row_bytes(k) : 0;
}

template <int DUAL>
static cudaError_t launch_gemv_ggml(int ty, const GemvArgs& a, cudaStream_t st) {
  // gate/up read per-32 sums of x written with the planes; the down projection has no such sums and
  // lets the tensor-core tiles form the Q4_K min term instead
  constexpr int OUT = DUAL ? kOutSiluPlanes : kOutFloat;
  if (ty == DARASK_GGML_Q4_K) return DUAL ? launch_gemv<kGemvQ4K, DUAL, false, OUT>(a, st) : launch_gemv<kGemvQ4K, DUAL, true, OUT>(a, st);
  if (ty == DARASK_GGML_Q6_K) return launch_gemv<kGemvQ6KR, DUAL, false, OUT>(a, st);
  return cudaErrorInvalidValue;
}

// ---- layer entry for the staged launches: `residual` and `rms_native` of the reference as one launch --------------
// One block of 256 threads per token, sums taken in the reference's order (native.cu:8-17, 89-96: thread t adds
// elements t, t + 256, ... with fused multiply-adds, warps by xor shuffles 16 .. 1, then the eight warp sums the same
// way), so that x and n come out bit for bit as from the reference's two kernels.
__global__ void __launch_bounds__(256) kogarashi_entry_kernel(float* x, const float* attn_out, const float* w, float* n, int h, float eps) {
  __shared__ float partial[8];
  pdl_wait();
  pdl_launch();
  float* xr = x + size_t(blockIdx.x) * h;
  float* nr = n + size_t(blockIdx.x) * h;
  const float* ar = attn_out ? attn_out + size_t(blockIdx.x) * h : nullptr;
  float v = 0.f;
  for (int i = threadIdx.x; i < h; i += 256) {
    float xv = xr[i];
    if (ar) {
      xv += ar[i];
      xr[i] = xv;
    }
    v = fmaf(xv, xv, v);
  }
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = v;
  __syncthreads();
  v = warp_sum((threadIdx.x & 31) < 8 ? partial[threadIdx.x & 31] : 0.f);      // every warp forms the same total, as warp 0 of the reference does
  const float scale = rsqrtf(v / h + eps);
  for (int i = threadIdx.x; i < h; i += 256) nr[i] = xr[i] * scale * w[i];
}

// ---- the one-token layer as one launch (decode_fused.cuh) ---------------------------------------------------
// Fills `f` and returns true when the shape can take the single-launch path.
static bool fused_plan(const KogarashiMoe* d, const KogarashiWs& w, FusedArgs* f, int* smem_bytes) {
  const int H = d->hidden, F = d->inter, E = d->experts, K = d->topk;
  if (d->tokens != 1 || d->router_ty != DARASK_GGML_F32 || d->gate_ty != DARASK_GGML_Q4_K) return false;
  if (d->down_ty != DARASK_GGML_Q4_K && d->down_ty != DARASK_GGML_Q6_K) return false;
  const bool shared = d->sh_gate_w != nullptr;
  const int grid = sm_count();
  if (E + (shared ? 1 : 0) > 2 * grid || E + (shared ? 1 : 0) > kFusedMaxLogits || grid > kFusedMaxCtas || H > 8192 || H % (16 * kFusedPasses) || F % (8 * kFusedPasses)) return false;
  FusedArgs a = {};
  a.H = H; a.F = F; a.E = E; a.K = K; a.has_shared = shared ? 1 : 0; a.G = K + a.has_shared;
  a.down_q6 = d->down_ty == DARASK_GGML_Q6_K;
  a.ldlog = fused_logit_stride(E);
  a.nblk1 = H / 256; a.nblk2 = F / 256;
  a.row_bytes1 = row_bytes_of(DARASK_GGML_Q4_K, H);
  a.row_bytes2 = row_bytes_of(d->down_ty, F);
  a.tps = F / (8 * kFusedPasses);
  a.rt2 = H / (16 * kFusedPasses);
  // a chunk = the gate rows or the up rows of a tile, or the rows of a down tile: whole rows, one bulk copy
  const int c1 = 8 * kFusedPasses * a.row_bytes1, c2 = 16 * kFusedPasses * a.row_bytes2;
  const int chunk = c1 > c2 ? c1 : c2;
  a.stage_bytes = (chunk + 127) / 128 * 128;
  // shared memory: control words | barriers | partial sums | activation area | ring
  a.off_bars = 640;
  a.off_psum = (a.off_bars + (2 * kFusedMaxStages + 1 + 4) * 8 + 127) / 128 * 128;
  a.off_log = (a.off_psum + kFusedSlots * kFusedQuad * 16 * kFusedPasses * 4 + 127) / 128 * 128;
  a.off_act = (a.off_log + (E + 1) * 4 + 127) / 128 * 128;
  // the token's two byte planes (the second 32 bytes off the bank phase of the first), (sum, 1 / S) per 32 columns; then
  // the router rows (phase R) and in the same place one area per quad (phase 2): the raw tagged products of one expert,
  // their two byte planes, their (sum, 1 / S) pairs
  a.act_lo1 = H + 32;
  a.act_xs1 = (2 * a.act_lo1 + 15) / 16 * 16;
  a.act_rows = (a.act_xs1 + H / 32 * 8 + 127) / 128 * 128;
  a.act_lo2 = F + 32;
  a.act_xs2 = (2 * a.act_lo2 + 15) / 16 * 16;
  a.act_q = a.act_rows;
  a.act_qs = (8 * F + a.act_xs2 + F / 16 * 8 + 127) / 128 * 128;
  const int rows_bytes = 2 * H * 4, quads_bytes = kFusedQuad * a.act_qs;
  a.off_ring = (a.off_act + a.act_rows + (rows_bytes > quads_bytes ? rows_bytes : quads_bytes) + 127) / 128 * 128;
  a.nstage = (kSmemBudget - a.off_ring) / a.stage_bytes;
  if (a.nstage > kFusedMaxStages) a.nstage = kFusedMaxStages;
  if (a.nstage < 3) return false;
  *smem_bytes = a.off_ring + a.nstage * a.stage_bytes;
  a.router_w = static_cast<const float*>(d->router_w); a.router_bias = d->router_bias; a.sh_inp = static_cast<const float*>(d->sh_inp_w);
  a.gate_w = static_cast<const uint8_t*>(d->gate_w); a.up_w = static_cast<const uint8_t*>(d->up_w); a.down_w = static_cast<const uint8_t*>(d->down_w);
  a.sh_gate = static_cast<const uint8_t*>(d->sh_gate_w); a.sh_up = static_cast<const uint8_t*>(d->sh_up_w); a.sh_down = static_cast<const uint8_t*>(d->sh_down_w);
  a.n = d->n; a.n_out = d->norm_w ? d->n : nullptr; a.attn_out = d->attn_out; a.norm_w = d->norm_w; a.norm_eps = d->norm_eps; a.x = d->x; a.logits = d->logits; a.ids = d->ids; a.prob = d->prob;
  a.status = w.status; a.epoch = w.epoch; a.seen = w.epoch + 1; a.tlog = w.tlog; a.th = w.th; a.ty = w.ty;
  *f = a;
  return true;
}

static cudaError_t launch_fused(const FusedArgs& a, int smem_bytes, cudaStream_t st) {
  static bool configured[64][2] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  auto k6 = kogarashi_decode1_kernel<1>;
  auto k4 = kogarashi_decode1_kernel<0>;
  if (!configured[dev][a.down_q6]) {
    e = a.down_q6 ? cudaFuncSetAttribute(k6, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget)
                  : cudaFuncSetAttribute(k4, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e != cudaSuccess) return e;
    configured[dev][a.down_q6] = true;
  }
  return a.down_q6 ? launch_pdl(k6, dim3(sm_count()), dim3(kFusedThreads), size_t(smem_bytes), st, a)
                   : launch_pdl(k4, dim3(sm_count()), dim3(kFusedThreads), size_t(smem_bytes), st, a);
}

static thread_local bool g_force_staged = false;    // host-thread-local: take the staged launches for one token too

}  // namespace dmoe

using namespace dmoe;

extern "C" int kogarashi_moe_set_single_launch(int enabled) {
  g_force_staged = !enabled;
  return cudaSuccess;
}

extern "C" size_t kogarashi_moe_workspace_bytes(int hidden, int inter, int experts, int topk, int tokens) {
  return carve(nullptr, hidden, inter, experts, topk, tokens).bytes;
}

extern "C" int kogarashi_moe_workspace_init(void* workspace, size_t bytes, cudaStream_t st) {
  if (!workspace || !bytes) return cudaErrorInvalidValue;
  return cudaMemsetAsync(workspace, 0, bytes, st);     // once per workspace: also the tagged words of the one-token kernel
}

extern "C" int kogarashi_moe_status(const void* workspace, unsigned* host_status, cudaStream_t st) {
  if (!workspace || !host_status) return cudaErrorInvalidValue;
  const KogarashiWs w = carve(const_cast<void*>(workspace), 256, 256, 1, 1, 1);
  cudaError_t e = cudaMemcpyAsync(host_status, w.status, 4, cudaMemcpyDeviceToHost, st);
  return e ? e : cudaStreamSynchronize(st);
}

extern "C" int darask_q6k_repack(void* dst, const void* src, long long rows, int k, int inverse, cudaStream_t st) {
  if (!dst || !src || rows <= 0 || k <= 0 || k % 256) return cudaErrorInvalidValue;
  const long long n = rows * (k / 256) * 105;
  if (!inverse) {
    cudaError_t e = cudaMemsetAsync(dst, 0, size_t(rows) * q6k_r16_row_bytes(k), st);
    if (e) return e;
  }
  q6k_repack_kernel<<<unsigned((n + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst),
                                                             rows, k / 256, inverse);
  return cudaGetLastError();
}

extern "C" size_t darask_q6k_repacked_bytes(long long rows, int k) { return size_t(rows) * q6k_r16_row_bytes(k); }

// Everything about a descriptor that can be checked without its workspace.
static bool descriptor_ok(const KogarashiMoe* d) {
  if (!d || !d->router_w || !d->gate_w || !d->up_w || !d->down_w || !d->n || !d->x || !d->logits || !d->ids || !d->prob) return false;
  const int H = d->hidden, F = d->inter, E = d->experts, K = d->topk, T = d->tokens;
  if (H <= 0 || F <= 0 || H % 256 || F % 256 || E < K || E > 1024 || K < 1 || K > 32 || T < 1) return false;
  if (d->gate_ty != d->up_ty || d->reserved) return false;
  if (d->router_ty != DARASK_GGML_F32 && d->router_ty != DARASK_GGML_BF16 && d->router_ty != DARASK_GGML_F16) return false;
  if (row_bytes_of(d->gate_ty, H) == 0 || row_bytes_of(d->down_ty, F) == 0) return false;
  if (d->sh_gate_w && (!d->sh_up_w || !d->sh_down_w || !d->sh_inp_w)) return false;
  if (d->attn_out && !d->norm_w) return false;
  if (d->norm_w && !(d->norm_eps >= 0.f)) return false;
  return true;
}

extern "C" int kogarashi_moe_layer(const KogarashiMoe* d, cudaStream_t st) {
  if (!descriptor_ok(d) || !d->workspace) return cudaErrorInvalidValue;
  const int H = d->hidden, F = d->inter, E = d->experts, K = d->topk, T = d->tokens;
  const bool shared = d->sh_gate_w != nullptr;
  if (d->workspace_bytes < kogarashi_moe_workspace_bytes(H, F, E, K, T)) return cudaErrorInvalidValue;
  const KogarashiWs w = carve(d->workspace, H, F, E, K, T);

  // one token: the whole layer is one persistent launch
  {
    FusedArgs f;
    int smem_bytes = 0;
    if (!g_force_staged && fused_plan(d, w, &f, &smem_bytes)) return launch_fused(f, smem_bytes, st);
  }

  // 0. layer entry (optional): x += attn_out, n = rms_norm(x) * norm_w
  if (d->norm_w) {
    const cudaError_t e0 = launch_pdl(kogarashi_entry_kernel, dim3(T), dim3(256), size_t(0), st, d->x, d->attn_out, d->norm_w, d->n, H, d->norm_eps);
    if (e0) return e0;
  }
  // 1. router projection, top-k, permutation
  RouterArgs r = {};
  r.w = d->router_w; r.extra = shared ? d->sh_inp_w : nullptr; r.x = d->n; r.row_bias = d->router_bias; r.logits = d->logits; r.extra_out = w.sg;
  r.hidden = H; r.rows = E; r.ld = E; r.tokens = T;
  r.route = RouteArgs{d->logits, E, E, K, T, nullptr, 1.f, d->ids, d->prob, nullptr};
  r.perm = PermuteArgs{d->ids, T, K, E, w.assignments, w.ranges, w.active, w.counters, w.status, w.plan, shared ? T : 0};
  r.done = w.done; r.fuse = 1;
  r.planes = w.xplanes; r.xsum_planes = w.xsum_planes;
  const int rblocks = E + (shared ? 1 : 0) + T;
  const size_t hist = size_t(E + 1) * 4 + size_t(T * K <= kRouteIdCache ? T * K : 0) * 4;
  cudaError_t e = cudaSuccess;
  if (d->router_ty == DARASK_GGML_F32) e = launch_pdl(router_kernel<float, float, kRouteKogarashi>, dim3(rblocks), dim3(128), hist, st, r);
  else if (d->router_ty == DARASK_GGML_BF16) e = launch_pdl(router_kernel<__nv_bfloat16, float, kRouteKogarashi>, dim3(rblocks), dim3(128), hist, st, r);
  else if (d->router_ty == DARASK_GGML_F16) e = launch_pdl(router_kernel<__half, float, kRouteKogarashi>, dim3(rblocks), dim3(128), hist, st, r);
  else return cudaErrorInvalidValue;
  if (e) return e;

  // 2. gate/up + SwiGLU for every (token, slot) and the shared expert
  const int max_groups = (T * K < E ? T * K : E) + (shared ? 1 : 0);
  GemvArgs a = {};
  a.w[0] = static_cast<const uint8_t*>(d->gate_w); a.w[1] = static_cast<const uint8_t*>(d->up_w);
  a.w_shared[0] = static_cast<const uint8_t*>(d->sh_gate_w); a.w_shared[1] = static_cast<const uint8_t*>(d->sh_up_w);
  a.row_bytes = row_bytes_of(d->gate_ty, H);
  a.expert_stride[0] = a.expert_stride[1] = (unsigned long long)a.row_bytes * F;
  a.k = H; a.rows = F; a.nblk = H / 256;
  a.xplanes = w.xplanes; a.xsum_planes = w.xsum_planes; a.x_by_assignment = 0;
  a.counters = w.counters + 2; a.plan = w.plan; a.assignments = w.assignments;
  a.tokens = T; a.topk = K; a.max_groups = max_groups;
  a.out_planes = w.hplanes; a.out = nullptr; a.status = w.status;
  if ((e = launch_gemv_ggml<1>(d->gate_ty, a, st))) return e;

  // 3. down
  GemvArgs b = a;
  b.w[0] = static_cast<const uint8_t*>(d->down_w); b.w[1] = nullptr;
  b.w_shared[0] = static_cast<const uint8_t*>(d->sh_down_w); b.w_shared[1] = nullptr;
  b.row_bytes = row_bytes_of(d->down_ty, F);
  b.expert_stride[0] = (unsigned long long)b.row_bytes * H; b.expert_stride[1] = 0;
  b.k = F; b.rows = H; b.nblk = F / 256;
  b.xplanes = w.hplanes; b.xsum_planes = nullptr; b.x_by_assignment = 1;
  b.out_planes = nullptr; b.out = w.y;
  b.late_wait = 1;                       // the plan is the router's, two launches back; only the products come from gate/up
  if ((e = launch_gemv_ggml<0>(d->down_ty, b, st))) return e;

  // 4. combine
  return launch_pdl(kogarashi_combine_kernel, dim3((H + 255) / 256, T), dim3(256), 0, st, d->x, (const float*)w.y,
                    (const float*)d->prob, (const float*)w.sg, H, K, T, shared ? 1 : 0);
}

// ---- stand-alone pieces (also used by the parity tests) ------------------------------------------

extern "C" int darask_route_topk(int mode, const float* logits, int ld, int experts, int topk, int tokens,
                                 const float* bias, float scale, int* ids, float* weights, float* shared_gate,
                                 cudaStream_t st) {
  if (!logits || !ids || !weights || experts < 1 || experts > 1024 || topk < 1 || topk > 32 || topk > experts ||
      tokens < 1 || ld < experts)
    return cudaErrorInvalidValue;
  RouteArgs a{logits, ld, experts, topk, tokens, bias, scale, ids, weights, shared_gate};
  const dim3 grid((tokens + 3) / 4), block(128);
  if (mode == DARASK_ROUTE_KOGARASHI) return launch_pdl(route_topk_kernel<kRouteKogarashi>, grid, block, 0, st, a);
  if (mode == DARASK_ROUTE_TSUMUJI) {
    if (shared_gate && ld < experts + 1) return cudaErrorInvalidValue;
    return launch_pdl(route_topk_kernel<kRouteTsumuji>, grid, block, 0, st, a);
  }
  if (mode == DARASK_ROUTE_HAYATE) {
    if (!bias) return cudaErrorInvalidValue;
    return darask_route_topk_hayate(logits, ld, experts, topk, tokens, bias, scale, ids, weights, st);
  }
  return cudaErrorInvalidValue;
}

extern "C" int darask_moe_permute(const int* ids, int tokens, int topk, int experts, unsigned* assignments,
                                  unsigned* ranges, int* active, int* counters, unsigned* status, cudaStream_t st) {
  if (!ids || !assignments || !ranges || !active || !counters || !status || tokens < 1 || topk < 1 || experts < 1 ||
      experts > 1024)
    return cudaErrorInvalidValue;
  PermuteArgs p{ids, tokens, topk, experts, assignments, ranges, active, counters, status};
  return launch_pdl(permute_kernel<0>, dim3(1), dim3(1024), size_t(experts + 1) * 4, st, p);
}

// ---- entry point that needs no caller-provided workspace -----------------------------------------
// Scratch of the layer lives in this fixed device array instead of `KogarashiMoe::workspace`.
// Every GPU that loads the library holds these bytes until the process exits.
#define KOGARASHI_STATIC_SCRATCH_BYTES (1u << 20)
static __device__ __align__(256) unsigned char g_kogarashi_static_scratch[KOGARASHI_STATIC_SCRATCH_BYTES];

extern "C" size_t kogarashi_moe_static_scratch_bytes(void) { return KOGARASHI_STATIC_SCRATCH_BYTES; }

// Device address of the built-in array on the current device (looked up once per device, with that device current:
// the array's name is only a host-side handle), or null with *err set.
static void* static_scratch_address(cudaError_t* err) {
  static void* address[64] = {nullptr};
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
  if (!address[dev]) {
    void* p = nullptr;
    *err = cudaGetSymbolAddress(&p, g_kogarashi_static_scratch);
    if (*err != cudaSuccess) return nullptr;
    address[dev] = p;
  }
  return address[dev];
}

extern "C" int kogarashi_moe_layer_static(const KogarashiMoe* d, cudaStream_t st) {
  if (!descriptor_ok(d)) return cudaErrorInvalidValue;        // nothing is enqueued for a descriptor that is refused
  const size_t need = kogarashi_moe_workspace_bytes(d->hidden, d->inter, d->experts, d->topk, d->tokens);
  if (need > KOGARASHI_STATIC_SCRATCH_BYTES) {
    fprintf(stderr,
            "kogarashi_moe_layer_static: this shape needs %zu bytes of scratch, the built-in array holds %u; "
            "use kogarashi_moe_layer with a caller-provided workspace\n",
            need, KOGARASHI_STATIC_SCRATCH_BYTES);
    return cudaErrorInvalidValue;
  }
  cudaError_t e = cudaSuccess;
  void* scratch = static_scratch_address(&e);
  if (!scratch) return e;
  // The array keeps whatever the previous call left: the control words (counters, barrier words, status) start at zero.
  e = cudaMemsetAsync(static_cast<uint8_t*>(scratch) + kHeadKept, 0, 4096 - kHeadKept, st);
  if (e != cudaSuccess) return e;
  KogarashiMoe copy = *d;
  copy.workspace = scratch;
  copy.workspace_bytes = KOGARASHI_STATIC_SCRATCH_BYTES;
  return kogarashi_moe_layer(&copy, st);
}

extern "C" int kogarashi_moe_static_status(unsigned* host_status, cudaStream_t st) {
  if (!host_status) return cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
  void* scratch = static_scratch_address(&e);
  if (!scratch) return e;
  return kogarashi_moe_status(scratch, host_status, st);
}
