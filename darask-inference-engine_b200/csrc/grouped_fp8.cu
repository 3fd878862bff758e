// FP8 prefill MoE layer: routing -> activation quantization -> dispatch gather -> grouped FP8 GEMM (gate/up with
// SwiGLU) -> quantization of the products -> grouped FP8 GEMM (down) -> weighted combine.
// The grouped GEMM kernel is in grouped_fp8.cuh. Reference orchestration: hayate crates/models/src/glm53/gpu.rs:
// 2068-2566 (`prefill_experts`: route, host-side `group_routes`, gather, grouped GEMMs, scatter).
#include "../../include/darask_moe_b200.h"
#include "grouped_fp8.cuh"
#include "route_kernels.cuh"
#include "permute_large.cuh"
#include "stream_launch.cuh"

namespace dmoe {

// rows in dispatch order: out row i = token assignments[i] / topk; also the inverse map position[a] = i
__global__ void __launch_bounds__(256) gather_fp8_kernel(const uint8_t* codes, const float* scales, const unsigned* assignments,
                                                         const int* counters, int topk, int k, uint8_t* out_codes,
                                                         float* out_scales, unsigned* position) {
  pdl_wait();
  pdl_launch();
  const int i = blockIdx.x;
  if (i >= __ldcg(counters + 1)) return;
  const unsigned asg = __ldcg(assignments + i);
  const size_t src = size_t(asg / topk), dst = size_t(i);
  if (threadIdx.x == 0) position[asg] = i;
  for (int c = threadIdx.x; c < k / 16; c += 256)
    reinterpret_cast<uint4*>(out_codes + dst * k)[c] = __ldg(reinterpret_cast<const uint4*>(codes + src * k) + c);
  for (int c = threadIdx.x; c < k / 128; c += 256) out_scales[dst * (k / 128) + c] = __ldg(scales + src * (k / 128) + c);
}

// out[t][i] = sum_s prob[t][s] * y[position[t*k+s]][i]  (fp32 fma in slot order), stored as float32
__global__ void __launch_bounds__(256) combine_rows_kernel(float* out, const float* y, const float* prob, const unsigned* position,
                                                           int hidden, int topk) {
  pdl_wait();
  pdl_launch();
  const int i = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
  if (i >= hidden) return;
  float v = 0.f;
  for (int s = 0; s < topk; ++s) v = fmaf(__ldg(prob + t * topk + s), __ldg(y + size_t(__ldg(position + t * topk + s)) * hidden + i), v);
  out[size_t(t) * hidden + i] = v;
}

// ---- expert-parallel regrouping ----------------------------------------------------------------------------------
// Rows received from `ranks` peers arrive grouped by source rank and, inside a source, by ascending local expert.
// plan: per local expert the range {rows, offset} of the regrouped order (expert-major, then source rank, then
// arrival order) and per (source, expert) segment its first received row and its first regrouped row.
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int* counts, int ranks, int local, unsigned* ranges, int* seg_src, int* seg_dst,
                                                       int slab /* rows per source slab; 0: sources follow each other without gaps */) {
  __shared__ int expert_off[1025];
  __shared__ int rank_off[65];
  pdl_wait();
  pdl_launch();
  const int tid = threadIdx.x;
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < local; ++e) {
      int rows = 0;
      for (int r = 0; r < ranks; ++r) rows += counts[r * local + e];
      ranges[2 * e] = rows;
      ranges[2 * e + 1] = run;
      expert_off[e] = run;
      run += rows;
    }
  }
  if (tid == 32) {
    int run = 0;
    for (int r = 0; r < ranks; ++r) {
      rank_off[r] = slab ? r * slab : run;
      for (int e = 0; e < local; ++e) run += counts[r * local + e];
    }
  }
  __syncthreads();
  for (int e = tid; e < local; e += 1024) {
    int dst = expert_off[e];
    for (int r = 0; r < ranks; ++r) { seg_dst[r * local + e] = dst; dst += counts[r * local + e]; }
  }
  for (int r = tid; r < ranks; r += 1024) {
    int src = rank_off[r];
    for (int e = 0; e < local; ++e) { seg_src[r * local + e] = src; src += counts[r * local + e]; }
  }
}
// row_map[regrouped row] = received row
__global__ void __launch_bounds__(128) ep_row_map_kernel(const int* counts, const int* seg_src, const int* seg_dst, unsigned* row_map) {
  pdl_wait();
  pdl_launch();
  const int seg = blockIdx.x, n = counts[seg], src = seg_src[seg], dst = seg_dst[seg];
  for (int i = threadIdx.x; i < n; i += 128) row_map[dst + i] = src + i;
}
__global__ void __launch_bounds__(256) ep_regroup_rows_kernel(const uint8_t* in_codes, const float* in_scales, const unsigned* row_map,
                                                              int k, uint8_t* codes, float* scales) {
  pdl_wait();
  pdl_launch();
  const size_t dst = blockIdx.x, src = __ldcg(row_map + dst);
  for (int c = threadIdx.x; c < k / 16; c += 256)
    reinterpret_cast<uint4*>(codes + dst * k)[c] = __ldg(reinterpret_cast<const uint4*>(in_codes + src * k) + c);
  for (int c = threadIdx.x; c < k / 128; c += 256) scales[dst * (k / 128) + c] = __ldg(in_scales + src * (k / 128) + c);
}

// ---- expert-parallel exchange without split sizes on the host ---------------------------------------------------
// Rows travel in slabs of fixed capacity, one per (source, destination) pair, as packed rows
//   [hidden e4m3 codes | hidden/128 float32 scales | float32 routing weight | int32 token of the source rank | pad to 16]
// so that both exchanges are equal-split all-to-alls and no device->host copy sits between the launches; the expert
// rank adds each token's rows (weight * row, ascending local expert) before they return, so what comes back is one
// float32 row per (token, expert rank), dense by token.
constexpr unsigned kStatusEpOverflow = 16u;     // more rows for one destination rank than a slab holds: rows were dropped
DEVI int packed_row_bytes(int k) { return (k + 4 * (k / 128) + 8 + 15) / 16 * 16; }

// dispatch row i (ascending expert order) -> slab of its expert's rank, at the row's index among that rank's rows
__global__ void __launch_bounds__(256) gather_packed_kernel(const uint8_t* codes, const float* scales, const unsigned* assignments,
                                                            const int* counters, const int* ids, const float* prob, const unsigned* ranges,
                                                            int topk, int k, int local, int cap, uint8_t* send, unsigned* position,
                                                            unsigned* overflow) {
  pdl_wait();
  pdl_launch();
  const int i = blockIdx.x;
  if (i >= __ldcg(counters + 1)) return;
  const unsigned asg = __ldcg(assignments + i);
  const int tok = int(asg / topk), r = __ldcg(ids + asg) / local;
  const int first = int(__ldcg(ranges + 2 * (r * local) + 1));            // first dispatch row that goes to rank r
  if (i - first >= cap) {                                                 // the slab is full: the row is dropped and reported
    if (threadIdx.x == 0) atomicOr(overflow, kStatusEpOverflow);
    return;
  }
  uint8_t* row = send + (size_t(r) * cap + size_t(i - first)) * packed_row_bytes(k);
  if (threadIdx.x == 0) {
    position[asg] = i;
    *reinterpret_cast<float*>(row + k + 4 * (k / 128)) = __ldg(prob + asg);
    *reinterpret_cast<int*>(row + k + 4 * (k / 128) + 4) = tok;
  }
  for (int c = threadIdx.x; c < k / 16; c += 256) reinterpret_cast<uint4*>(row)[c] = __ldg(reinterpret_cast<const uint4*>(codes + size_t(tok) * k) + c);
  for (int c = threadIdx.x; c < k / 128; c += 256) reinterpret_cast<float*>(row + k)[c] = __ldg(scales + size_t(tok) * (k / 128) + c);
}
// counts[e] = rows of expert e that fit its rank's slab (all of them unless the slab overflowed)
__global__ void __launch_bounds__(64) ep_slab_counts_kernel(const unsigned* ranges, int ranks, int local, int cap, int* counts) {
  pdl_wait();
  pdl_launch();
  const int r = threadIdx.x;
  if (r >= ranks) return;
  int run = 0;
  for (int e = r * local; e < (r + 1) * local; ++e) {
    const int c = min(int(__ldcg(ranges + 2 * e)), cap - run);
    counts[e] = c;
    run += c;
  }
}
// regrouped row <- packed row of its slab; also the row's source rank, token and routing weight
__global__ void __launch_bounds__(256) ep_unpack_rows_kernel(const uint8_t* recv, const unsigned* row_map, const unsigned* ranges, int local,
                                                             int k, int cap, uint8_t* codes, float* scales, int* meta_src, int* meta_tok,
                                                             float* meta_prob) {
  pdl_wait();
  pdl_launch();
  const unsigned total = __ldcg(ranges + 2 * (local - 1)) + __ldcg(ranges + 2 * (local - 1) + 1);
  const size_t dst = blockIdx.x;
  if (dst >= total) return;
  const size_t src = __ldcg(row_map + dst);
  const uint8_t* row = recv + src * packed_row_bytes(k);
  for (int c = threadIdx.x; c < k / 16; c += 256) reinterpret_cast<uint4*>(codes + dst * k)[c] = __ldg(reinterpret_cast<const uint4*>(row) + c);
  for (int c = threadIdx.x; c < k / 128; c += 256) scales[dst * (k / 128) + c] = __ldg(reinterpret_cast<const float*>(row + k) + c);
  if (threadIdx.x == 0) {
    meta_src[dst] = int(src / size_t(cap));
    meta_prob[dst] = __ldg(reinterpret_cast<const float*>(row + k + 4 * (k / 128)));
    meta_tok[dst] = __ldg(reinterpret_cast<const int*>(row + k + 4 * (k / 128) + 4));
  }
}
// the rows of every (source rank, token): list[(s * tcap + t) * topk + j]; count[] must be zero on entry
__global__ void __launch_bounds__(256) ep_index_kernel(const unsigned* ranges, int local, const int* meta_src, const int* meta_tok, int tcap,
                                                       int topk, int* count, int* list, unsigned* status) {
  pdl_wait();
  pdl_launch();
  const unsigned total = __ldcg(ranges + 2 * (local - 1)) + __ldcg(ranges + 2 * (local - 1) + 1);
  const unsigned i = blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  const int t = meta_tok[i], slot_of = meta_src[i] * tcap + t;
  if (t < 0 || t >= tcap) { atomicOr(status, kStatusBadRoute); return; }
  const int j = atomicAdd(count + slot_of, 1);
  if (j < topk) list[size_t(slot_of) * topk + j] = int(i);
  else atomicOr(status, kStatusBadRoute);
}
// z[s][t] = sum over the rows of (s, t), ascending row (= ascending local expert), of weight * y[row]; zero without rows
__global__ void __launch_bounds__(256) ep_reduce_kernel(const float* y, const float* meta_prob, const int* count, const int* list, int topk,
                                                        int hidden, float* z) {
  __shared__ int rows[32];
  __shared__ float w[32];
  pdl_wait();
  pdl_launch();
  const size_t slot_of = blockIdx.x;
  const int n = min(__ldcg(count + slot_of), topk);
  if (threadIdx.x == 0) {
    for (int j = 0; j < n; ++j) {                       // insertion sort: the order in which the rows were indexed is arbitrary
      const int v = __ldcg(list + slot_of * topk + j);
      int q = j;
      while (q > 0 && rows[q - 1] > v) { rows[q] = rows[q - 1]; --q; }
      rows[q] = v;
    }
    for (int j = 0; j < n; ++j) w[j] = __ldg(meta_prob + rows[j]);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < hidden / 4; c += 256) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < n; ++j) {
      const float4 a = __ldcs(reinterpret_cast<const float4*>(y + size_t(rows[j]) * hidden) + c);
      v.x = fmaf(w[j], a.x, v.x); v.y = fmaf(w[j], a.y, v.y); v.z = fmaf(w[j], a.z, v.z); v.w = fmaf(w[j], a.w, v.w);
    }
    reinterpret_cast<float4*>(z + slot_of * hidden)[c] = v;
  }
}
// out[t] = sum over the expert ranks, ascending, of their partial rows
__global__ void __launch_bounds__(256) ep_sum_kernel(float* out, const float* zr, int ranks, int tcap, int hidden) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
  if (c >= hidden / 4) return;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = 0; r < ranks; ++r) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(zr + (size_t(r) * tcap + t) * hidden) + c);
    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
  }
  reinterpret_cast<float4*>(out + size_t(t) * hidden)[c] = v;
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(p);
  }
  return fn;
}
// 2D byte tensor [rows][k], box [box_rows][128], 128-byte swizzle
static bool make_map(CUtensorMap* m, const void* base, unsigned long long rows, unsigned long long k, unsigned box_rows) {
  EncodeTiled enc = encode_tiled();
  if (!enc) return false;
  const cuuint64_t dims[2] = {k, rows}, strides[1] = {k};
  const cuuint32_t box[2] = {128, box_rows}, estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static cudaError_t launch_grouped(const void* a_codes, const float* a_scales, unsigned long long a_rows, const void* w0,
                                  const void* w1, const float* sw0, const float* sw1, int experts, int n, int k, int mode,
                                  const unsigned* ranges, void* out, float* out_scales, const unsigned* out_row_map,
                                  unsigned* status, cudaStream_t st) {
  CUtensorMap ma, mw0, mw1;
  const bool gate_up = mode != kG8Plain;
  if (!make_map(&ma, a_codes, a_rows, k, 128)) return cudaErrorInvalidValue;
  if (!make_map(&mw0, w0, (unsigned long long)experts * n, k, 128)) return cudaErrorInvalidValue;
  if (!make_map(&mw1, gate_up ? w1 : w0, (unsigned long long)experts * n, k, 128)) return cudaErrorInvalidValue;
  G8Args g = {};
  g.sa = a_scales; g.sw[0] = sw0; g.sw[1] = sw1;
  g.sw_expert_stride = (unsigned long long)(n / 128) * (k / 128);
  g.ranges = ranges; g.experts = experts; g.n = n; g.k = k; g.mode = mode;
  g.out_f32 = mode == kG8Plain ? static_cast<float*>(out) : nullptr;
  g.out_bf16 = mode == kG8GateUpBf16 ? static_cast<__nv_bfloat16*>(out) : nullptr;
  g.out_codes = mode == kG8GateUpFp8 ? static_cast<uint8_t*>(out) : nullptr;
  g.out_scales = out_scales; g.out_row_map = out_row_map; g.status = status;
  const size_t smem = size_t(kG8FixedSmem) + size_t(experts + 1) * sizeof(int);
  static bool configured[64] = {};      // the opt-in is per device
  const int dev = current_device_slot();
  if (dev < 0) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    const int most = int(size_t(kG8FixedSmem) + size_t(kG8MaxExperts + 1) * sizeof(int));
    cudaError_t e = cudaFuncSetAttribute(grouped_fp8_kernel<kG8Plain>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (!e) e = cudaFuncSetAttribute(grouped_fp8_kernel<kG8GateUpBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (!e) e = cudaFuncSetAttribute(grouped_fp8_kernel<kG8GateUpFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const dim3 grid(sm_count()), block(kG8Threads);
  if (mode == kG8Plain) return launch_pdl(grouped_fp8_kernel<kG8Plain>, grid, block, smem, st, ma, mw0, mw1, g);
  if (mode == kG8GateUpBf16) return launch_pdl(grouped_fp8_kernel<kG8GateUpBf16>, grid, block, smem, st, ma, mw0, mw1, g);
  return launch_pdl(grouped_fp8_kernel<kG8GateUpFp8>, grid, block, smem, st, ma, mw0, mw1, g);
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
struct Fp8Ws {
  int* counters; unsigned* status; int* active; unsigned* ranges; unsigned* assignments; unsigned* position; int* perm_scratch;
  uint8_t* xq; float* xs; uint8_t* aq; float* as; uint8_t* pq; float* ps; float* y; size_t bytes;
};
static Fp8Ws carve(void* base, int hidden, int inter, int experts, int topk, int tokens) {
  Fp8Ws w;
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) { uint8_t* q = p ? p + off : nullptr; off = align_up(off + bytes, 1024); return q; };
  const size_t rows = size_t(tokens) * topk + 128;          // + one tile of slack for the last tile's tail loads
  w.counters = reinterpret_cast<int*>(take(16));
  w.status = reinterpret_cast<unsigned*>(take(4));
  w.active = reinterpret_cast<int*>(take(size_t(experts) * 4));
  w.ranges = reinterpret_cast<unsigned*>(take(size_t(experts) * 8));
  w.assignments = reinterpret_cast<unsigned*>(take(size_t(tokens) * topk * 4));
  w.position = reinterpret_cast<unsigned*>(take(size_t(tokens) * topk * 4));
  w.perm_scratch = reinterpret_cast<int*>(take(permute_scratch_bytes(tokens, topk, experts)));
  w.xq = take(size_t(tokens) * hidden);
  w.xs = reinterpret_cast<float*>(take(size_t(tokens) * (hidden / 128) * 4));
  w.aq = take(rows * hidden);
  w.as = reinterpret_cast<float*>(take(rows * (hidden / 128) * 4));
  w.pq = take(rows * inter);
  w.ps = reinterpret_cast<float*>(take(rows * (inter / 128) * 4));
  w.y = reinterpret_cast<float*>(take(rows * hidden * 4));
  w.bytes = off;
  return w;
}

}  // namespace dmoe

using namespace dmoe;

extern "C" int darask_fp8_grouped_gemm(const void* a_codes, const float* a_scales, unsigned long long a_rows, const void* w0,
                                       const void* w1, const float* sw0, const float* sw1, int experts, int n, int k, int mode,
                                       const unsigned* ranges, void* out, float* out_scales, const unsigned* out_row_map,
                                       unsigned* status, cudaStream_t st) {
  if (!a_codes || !a_scales || !w0 || !sw0 || !ranges || !out || !status || experts < 1 || experts > kG8MaxExperts || n < 128 ||
      n % 128 || k < 128 || k % 128 || mode < kG8Plain || mode > kG8GateUpFp8 || (mode != kG8Plain && (!w1 || !sw1 || out_row_map)) ||
      (mode == kG8GateUpFp8 && !out_scales))
    return cudaErrorInvalidValue;
  return launch_grouped(a_codes, a_scales, a_rows, w0, w1, sw0, sw1, experts, n, k, mode, ranges, out, out_scales, out_row_map, status, st);
}

extern "C" size_t darask_moe_permute_scratch_bytes(int tokens, int topk, int experts) {
  return tokens < 1 || topk < 1 || experts < 1 ? 0 : permute_scratch_bytes(tokens, topk, experts);
}

extern "C" int darask_moe_permute_large(const int* ids, int tokens, int topk, int experts, unsigned* assignments, unsigned* ranges,
                                        int* active, int* counters, unsigned* status, void* scratch, size_t scratch_bytes,
                                        cudaStream_t st) {
  if (!ids || !assignments || !ranges || !active || !counters || !status || !scratch || tokens < 1 || topk < 1 || experts < 1 ||
      experts > 1024 || scratch_bytes < permute_scratch_bytes(tokens, topk, experts))
    return cudaErrorInvalidValue;
  const PermuteArgs p{ids, tokens, topk, experts, assignments, ranges, active, counters, status, nullptr, 0};
  return launch_permute_large(p, scratch, st);
}

extern "C" size_t darask_fp8_moe_workspace_bytes(int hidden, int inter, int experts, int topk, int tokens) {
  return carve(nullptr, hidden, inter, experts, topk, tokens).bytes;
}

extern "C" int darask_fp8_moe_layer(const DaraskFp8Moe* d, cudaStream_t st) {
  if (!d || !d->x || !d->logits || !d->gate_w || !d->up_w || !d->down_w || !d->gate_s || !d->up_s || !d->down_s || !d->out ||
      !d->ids || !d->prob || !d->workspace)
    return cudaErrorInvalidValue;
  const int H = d->hidden, F = d->inter, E = d->experts, K = d->topk, T = d->tokens;
  if (H < 128 || F < 128 || H % 128 || F % 128 || E < K || E > 1024 || K < 1 || K > 32 || T < 1) return cudaErrorInvalidValue;
  if (d->workspace_bytes < darask_fp8_moe_workspace_bytes(H, F, E, K, T)) return cudaErrorInvalidValue;
  const Fp8Ws w = carve(d->workspace, H, F, E, K, T);
  cudaError_t e;
  if ((e = cudaMemsetAsync(w.counters, 0, 2048, st))) return e;       // counters and the status word
  const RouteArgs route{d->logits, E, E, K, T, nullptr, 1.f, d->ids, d->prob, nullptr};
  const PermuteArgs perm{d->ids, T, K, E, w.assignments, w.ranges, w.active, w.counters, w.status, nullptr, 0};
  if ((e = launch_pdl(route_topk_kernel<kRouteKogarashi>, dim3((T + 3) / 4), dim3(128), 0, st, route))) return e;
  if (T * K > 2048) {
    if ((e = launch_permute_large(perm, w.perm_scratch, st))) return e;
  } else if ((e = launch_pdl(permute_kernel<0>, dim3(1), dim3(1024), size_t(E + 1) * 4, st, perm))) return e;
  if ((e = (cudaError_t)darask_quantize_fp8_act(w.xq, w.xs, d->x, 1, T, H, st))) return e;
  if ((e = launch_pdl(gather_fp8_kernel, dim3(T * K), dim3(256), 0, st, (const uint8_t*)w.xq, (const float*)w.xs,
                      (const unsigned*)w.assignments, (const int*)w.counters, K, H, w.aq, w.as, w.position))) return e;
  const unsigned long long rows = (unsigned long long)T * K + 128;
  if ((e = launch_grouped(w.aq, w.as, rows, d->gate_w, d->up_w, d->gate_s, d->up_s, E, F, H, kG8GateUpFp8, w.ranges, w.pq, w.ps, nullptr,
                          w.status, st))) return e;
  if ((e = launch_grouped(w.pq, w.ps, rows, d->down_w, nullptr, d->down_s, nullptr, E, H, F, kG8Plain, w.ranges, w.y, nullptr, nullptr,
                          w.status, st))) return e;
  return launch_pdl(combine_rows_kernel, dim3((H + 255) / 256, T), dim3(256), 0, st, d->out, (const float*)w.y, (const float*)d->prob,
                    (const unsigned*)w.position, H, K);
}

// ---- expert-parallel entry points ------------------------------------------------------------------------------
extern "C" size_t darask_fp8_ep_dispatch_scratch_bytes(int hidden, int experts, int topk, int tokens) {
  if (hidden < 128 || experts < 1 || topk < 1 || tokens < 1) return 0;
  return 4096 + align_up(size_t(experts) * 4, 1024) + align_up(size_t(tokens) * topk * 4, 1024) +
         align_up(permute_scratch_bytes(tokens, topk, experts), 1024) + align_up(size_t(tokens) * hidden, 1024) +
         align_up(size_t(tokens) * (hidden / 128) * 4, 1024);
}

// ranks > 0: packed slabs of `cap` rows per destination rank into send_codes (send_scales unused)
static int ep_dispatch(const void* x, const float* logits, int hidden, int experts, int topk, int tokens, int* ids, float* prob,
                       void* send_codes, float* send_scales, unsigned* ranges, unsigned* position, void* scratch, size_t scratch_bytes,
                       int ranks, int cap, int* counts, unsigned* overflow, cudaStream_t st) {
  if (!x || !logits || !ids || !prob || !send_codes || (!send_scales && !ranks) || !ranges || !position || !scratch || hidden < 128 ||
      hidden % 128 || experts < topk || experts > 1024 || topk < 1 || topk > 32 || tokens < 1 ||
      scratch_bytes < darask_fp8_ep_dispatch_scratch_bytes(hidden, experts, topk, tokens))
    return cudaErrorInvalidValue;
  uint8_t* p = static_cast<uint8_t*>(scratch);
  size_t off = 0;
  auto take = [&](size_t bytes) { uint8_t* q = p + off; off = align_up(off + bytes, 1024); return q; };
  int* counters = reinterpret_cast<int*>(take(2048));
  unsigned* status = reinterpret_cast<unsigned*>(take(2048));
  int* active = reinterpret_cast<int*>(take(size_t(experts) * 4));
  unsigned* assignments = reinterpret_cast<unsigned*>(take(size_t(tokens) * topk * 4));
  int* perm_scratch = reinterpret_cast<int*>(take(permute_scratch_bytes(tokens, topk, experts)));
  uint8_t* xq = take(size_t(tokens) * hidden);
  float* xs = reinterpret_cast<float*>(take(size_t(tokens) * (hidden / 128) * 4));
  cudaError_t e;
  if ((e = cudaMemsetAsync(counters, 0, 4096, st))) return e;
  const RouteArgs route{logits, experts, experts, topk, tokens, nullptr, 1.f, ids, prob, nullptr};
  const PermuteArgs perm{ids, tokens, topk, experts, assignments, ranges, active, counters, status, nullptr, 0};
  if ((e = launch_pdl(route_topk_kernel<kRouteKogarashi>, dim3((tokens + 3) / 4), dim3(128), 0, st, route))) return e;
  if (tokens * topk > 2048) {
    if ((e = launch_permute_large(perm, perm_scratch, st))) return e;
  } else if ((e = launch_pdl(permute_kernel<0>, dim3(1), dim3(1024), size_t(experts + 1) * 4, st, perm))) return e;
  if ((e = (cudaError_t)darask_quantize_fp8_act(xq, xs, x, 1, tokens, hidden, st))) return e;
  if (ranks) {
    if ((e = launch_pdl(gather_packed_kernel, dim3(tokens * topk), dim3(256), 0, st, (const uint8_t*)xq, (const float*)xs,
                        (const unsigned*)assignments, (const int*)counters, (const int*)ids, (const float*)prob, (const unsigned*)ranges, topk,
                        hidden, experts / ranks, cap, static_cast<uint8_t*>(send_codes), position, overflow))) return e;
    return launch_pdl(ep_slab_counts_kernel, dim3(1), dim3(64), 0, st, (const unsigned*)ranges, ranks, experts / ranks, cap, counts);
  }
  return launch_pdl(gather_fp8_kernel, dim3(tokens * topk), dim3(256), 0, st, (const uint8_t*)xq, (const float*)xs,
                    (const unsigned*)assignments, (const int*)counters, topk, hidden, static_cast<uint8_t*>(send_codes), send_scales,
                    position);
}

extern "C" int darask_fp8_ep_dispatch(const void* x, const float* logits, int hidden, int experts, int topk, int tokens, int* ids,
                                      float* prob, void* send_codes, float* send_scales, unsigned* ranges, unsigned* position,
                                      void* scratch, size_t scratch_bytes, cudaStream_t st) {
  return ep_dispatch(x, logits, hidden, experts, topk, tokens, ids, prob, send_codes, send_scales, ranges, position, scratch, scratch_bytes,
                     0, 0, nullptr, nullptr, st);
}

extern "C" size_t darask_fp8_ep_packed_row_bytes(int hidden) { return hidden >= 128 && hidden % 128 == 0 ? size_t((hidden + 4 * (hidden / 128) + 8 + 15) / 16 * 16) : 0; }

extern "C" int darask_fp8_ep_dispatch_packed(const void* x, const float* logits, int hidden, int experts, int topk, int tokens, int ranks,
                                             int cap, int* ids, float* prob, void* send, int* counts, unsigned* ranges,
                                             unsigned* position, unsigned* status, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (ranks < 1 || ranks > 64 || experts % ranks || cap < 1 || !counts || !status) return cudaErrorInvalidValue;
  return ep_dispatch(x, logits, hidden, experts, topk, tokens, ids, prob, send, nullptr, ranges, position, scratch, scratch_bytes, ranks,
                     cap, counts, status, st);
}

extern "C" int darask_fp8_ep_regroup_packed(const int* recv_counts, int ranks, int local_experts, const void* recv, int cap, int hidden,
                                            void* codes, float* scales, unsigned* ranges, unsigned* row_map, int* meta_src, int* meta_tok,
                                            float* meta_prob, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (!recv_counts || !recv || !codes || !scales || !ranges || !row_map || !meta_src || !meta_tok || !meta_prob || !scratch || ranks < 1 ||
      ranks > 64 || local_experts < 1 || local_experts > 1024 || hidden < 128 || hidden % 128 || cap < 1 ||
      scratch_bytes < size_t(ranks) * local_experts * 8)
    return cudaErrorInvalidValue;
  int* seg_src = static_cast<int*>(scratch);
  int* seg_dst = seg_src + size_t(ranks) * local_experts;
  cudaError_t e;
  if ((e = launch_pdl(ep_plan_kernel, dim3(1), dim3(1024), 0, st, recv_counts, ranks, local_experts, ranges, seg_src, seg_dst, cap))) return e;
  if ((e = launch_pdl(ep_row_map_kernel, dim3(ranks * local_experts), dim3(128), 0, st, recv_counts, (const int*)seg_src,
                      (const int*)seg_dst, row_map))) return e;
  // the number of rows is known on the device only: one block per row a rank can receive, the surplus returns at once
  return launch_pdl(ep_unpack_rows_kernel, dim3(unsigned(ranks) * unsigned(cap)), dim3(256), 0, st, static_cast<const uint8_t*>(recv),
                    (const unsigned*)row_map, (const unsigned*)ranges, local_experts, hidden, cap, static_cast<uint8_t*>(codes), scales,
                    meta_src, meta_tok, meta_prob);
}

extern "C" int darask_fp8_ep_reduce(const float* y, const unsigned* ranges, int local_experts, const int* meta_src, const int* meta_tok,
                                    const float* meta_prob, int ranks, int cap, int tcap, int topk, int hidden, float* z, int* count,
                                    int* list, unsigned* status, cudaStream_t st) {
  if (!y || !ranges || !meta_src || !meta_tok || !meta_prob || !z || !count || !list || !status || ranks < 1 || cap < 1 || tcap < 1 ||
      topk < 1 || topk > 32 || hidden < 4 || hidden % 4 || local_experts < 1)
    return cudaErrorInvalidValue;
  cudaError_t e;
  if ((e = cudaMemsetAsync(count, 0, size_t(ranks) * tcap * 4, st))) return e;
  const unsigned max_rows = unsigned(ranks) * unsigned(cap);
  if ((e = launch_pdl(ep_index_kernel, dim3((max_rows + 255) / 256), dim3(256), 0, st, ranges, local_experts, meta_src, meta_tok, tcap, topk,
                      count, list, status))) return e;
  return launch_pdl(ep_reduce_kernel, dim3(unsigned(ranks) * unsigned(tcap)), dim3(256), 0, st, y, meta_prob, (const int*)count,
                    (const int*)list, topk, hidden, z);
}

extern "C" int darask_fp8_ep_sum(float* out, const float* zr, int ranks, int tokens, int tcap, int hidden, cudaStream_t st) {
  if (!out || !zr || ranks < 1 || tokens < 1 || tokens > tcap || hidden < 4 || hidden % 4) return cudaErrorInvalidValue;
  return launch_pdl(ep_sum_kernel, dim3((hidden / 4 + 255) / 256, tokens), dim3(256), 0, st, out, zr, ranks, tcap, hidden);
}

extern "C" int darask_fp8_ep_regroup(const int* recv_counts, int ranks, int local_experts, const void* recv_codes,
                                     const float* recv_scales, int hidden, long long recv_rows, void* codes, float* scales,
                                     unsigned* ranges, unsigned* row_map, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (!recv_counts || !codes || !scales || !ranges || !row_map || !scratch || ranks < 1 || ranks > 64 || local_experts < 1 ||
      local_experts > 1024 || hidden < 128 || hidden % 128 || recv_rows < 0 || (recv_rows > 0 && (!recv_codes || !recv_scales)) ||
      scratch_bytes < size_t(ranks) * local_experts * 8)
    return cudaErrorInvalidValue;
  int* seg_src = static_cast<int*>(scratch);
  int* seg_dst = seg_src + size_t(ranks) * local_experts;
  cudaError_t e;
  if ((e = launch_pdl(ep_plan_kernel, dim3(1), dim3(1024), 0, st, recv_counts, ranks, local_experts, ranges, seg_src, seg_dst, 0))) return e;
  if (recv_rows == 0) return cudaSuccess;
  if ((e = launch_pdl(ep_row_map_kernel, dim3(ranks * local_experts), dim3(128), 0, st, recv_counts, (const int*)seg_src,
                      (const int*)seg_dst, row_map))) return e;
  return launch_pdl(ep_regroup_rows_kernel, dim3((unsigned)recv_rows), dim3(256), 0, st, static_cast<const uint8_t*>(recv_codes),
                    recv_scales, (const unsigned*)row_map, hidden, static_cast<uint8_t*>(codes), scales);
}

extern "C" int darask_fp8_ep_experts(const void* codes, const float* scales, unsigned long long rows_alloc, const unsigned* ranges,
                                     int local_experts, int hidden, int inter, const void* gate_w, const void* up_w,
                                     const void* down_w, const float* gate_s, const float* up_s, const float* down_s,
                                     const unsigned* row_map, float* y, void* prod_codes, float* prod_scales, unsigned* status,
                                     cudaStream_t st) {
  if (!codes || !scales || !ranges || !gate_w || !up_w || !down_w || !gate_s || !up_s || !down_s || !y || !prod_codes ||
      !prod_scales || !status || local_experts < 1 || local_experts > kG8MaxExperts || hidden < 128 || hidden % 128 || inter < 128 ||
      inter % 128 || rows_alloc < 128)
    return cudaErrorInvalidValue;
  cudaError_t e;
  if ((e = launch_grouped(codes, scales, rows_alloc, gate_w, up_w, gate_s, up_s, local_experts, inter, hidden, kG8GateUpFp8, ranges,
                          prod_codes, prod_scales, nullptr, status, st))) return e;
  return launch_grouped(prod_codes, prod_scales, rows_alloc, down_w, nullptr, down_s, nullptr, local_experts, hidden, inter, kG8Plain,
                        ranges, y, nullptr, row_map, status, st);
}

extern "C" int darask_fp8_ep_combine(float* out, const float* y, const float* prob, const unsigned* position, int tokens, int hidden,
                                     int topk, cudaStream_t st) {
  if (!out || !y || !prob || !position || tokens < 1 || hidden < 1 || topk < 1) return cudaErrorInvalidValue;
  return launch_pdl(combine_rows_kernel, dim3((hidden + 255) / 256, tokens), dim3(256), 0, st, out, y, prob, position, hidden, topk);
}

extern "C" int darask_fp8_moe_status(const void* workspace, unsigned* host_status, cudaStream_t st) {
  if (!workspace || !host_status) return cudaErrorInvalidValue;
  const Fp8Ws w = carve(const_cast<void*>(workspace), 128, 128, 1, 1, 1);
  cudaError_t e = cudaMemcpyAsync(host_status, w.status, 4, cudaMemcpyDeviceToHost, st);
  return e ? e : cudaStreamSynchronize(st);
}
