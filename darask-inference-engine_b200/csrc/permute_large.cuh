// Dispatch permutation for prefill-sized batches: the same stable counting sort as permute_block, spread over
// many thread blocks.  Assignments are cut into chunks of 1024; (1) every chunk counts its rows per expert,
// (2) one block turns the counts into per-expert ranges and per-(chunk, expert) start offsets, (3) every chunk
// places its assignments: rank inside the chunk = rows of the same expert in earlier warps + earlier lanes.
// (The kernels are templates only so that several translation units may include this file.)
// Replaces the host loop `groups` (hayate models/src/glm53/prefill.rs:12-26) for batches where one block is slow.
#pragma once
#include "route_impl.cuh"
#include "stream_launch.cuh"

namespace dmoe {

constexpr int kPermChunk = 1024;

DEVI bool route_ok(const int* ids, int a, int n, int E, int K, int& e) {
  if (a >= n) return false;
  e = __ldg(ids + a);
  bool ok = e >= 0 && e < E;
  for (int j = a - a % K; ok && j < a; ++j) ok = __ldg(ids + j) != e;
  return ok;
}

// chunk_counts [chunks][E]
template <int UNUSED = 0>
__global__ void __launch_bounds__(kPermChunk) permute_count_kernel(PermuteArgs p, int* chunk_counts) {
  extern __shared__ int hist[];
  pdl_wait();
  pdl_launch();
  const int n = p.tokens * p.topk, E = p.experts;
  for (int e = threadIdx.x; e < E; e += kPermChunk) hist[e] = 0;
  __syncthreads();
  const int a = blockIdx.x * kPermChunk + threadIdx.x;
  int e;
  if (route_ok(p.ids, a, n, E, p.topk, e)) atomicAdd(&hist[e], 1);
  else if (a < n) atomicOr(p.status, kStatusBadRoute);
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += kPermChunk) chunk_counts[size_t(blockIdx.x) * E + i] = hist[i];
}

// chunk_counts -> in place: rows of the expert in earlier chunks; ranges / active / plan / counters as permute_block
template <int UNUSED = 0>
__global__ void __launch_bounds__(1024) permute_scan_kernel(PermuteArgs p, int* chunk_counts, int chunks) {
  extern __shared__ int hist[];
  pdl_wait();
  pdl_launch();
  const int E = p.experts, tid = threadIdx.x;
  for (int e = tid; e < E; e += 1024) {
    int run = 0;
    for (int c = 0; c < chunks; ++c) {
      const int v = chunk_counts[size_t(c) * E + e];
      chunk_counts[size_t(c) * E + e] = run;
      run += v;
    }
    hist[e] = run;
  }
  __syncthreads();
  if (tid < 32) {
    const int per = (E + 31) / 32;
    int sum = 0, act = 0;
    for (int i = 0; i < per; ++i) {
      const int e = tid * per + i;
      if (e < E) { sum += hist[e]; act += hist[e] > 0; }
    }
    int run = sum, arun = act;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, run, o), u = __shfl_up_sync(0xffffffffu, arun, o);
      if (tid >= o) { run += t; arun += u; }
    }
    int off = run - sum, aoff = arun - act;
    for (int i = 0; i < per; ++i) {
      const int e = tid * per + i;
      if (e < E) {
        const int c = hist[e];
        p.ranges[2 * e] = c;
        p.ranges[2 * e + 1] = off;
        if (c) {
          if (p.plan) p.plan[aoff] = make_int4(e, c, off, 0);
          p.active[aoff++] = e;
        }
        off += c;
      }
    }
    if (tid == 31) {
      p.counters[0] = arun;
      p.counters[1] = run;
      p.counters[2] = arun + (p.shared_rows > 0 ? 1 : 0);
      if (p.plan && p.shared_rows > 0) p.plan[arun] = make_int4(-1, p.shared_rows, 0, 0);
    }
  }
}

template <int UNUSED = 0>
__global__ void __launch_bounds__(kPermChunk) permute_place_kernel(PermuteArgs p, const int* chunk_base) {
  extern __shared__ unsigned short warp_rows[];        // [32 warps][E]
  pdl_wait();
  pdl_launch();
  const int n = p.tokens * p.topk, E = p.experts, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < 32 * E; i += kPermChunk) warp_rows[i] = 0;
  __syncthreads();
  const int a = blockIdx.x * kPermChunk + tid;
  int e = 0;
  const bool ok = route_ok(p.ids, a, n, E, p.topk, e);
  const unsigned same = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);
  const int rank = __popc(same & ((1u << lane) - 1u));
  if (ok && rank == 0) warp_rows[warp * E + e] = (unsigned short)__popc(same);
  __syncthreads();
  for (int x = tid; x < E; x += kPermChunk) {          // exclusive prefix over the warps, per expert
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int v = warp_rows[w * E + x];
      warp_rows[w * E + x] = (unsigned short)run;
      run += v;
    }
  }
  __syncthreads();
  if (ok) p.assignments[__ldcg(p.ranges + 2 * e + 1) + __ldcg(chunk_base + size_t(blockIdx.x) * E + e) + warp_rows[warp * E + e] + rank] = a;
}

inline size_t permute_scratch_bytes(int tokens, int topk, int experts) {
  const long long n = (long long)tokens * topk;
  return size_t((n + kPermChunk - 1) / kPermChunk) * experts * sizeof(int);
}

// The three launches above; `scratch` holds permute_scratch_bytes().
inline cudaError_t launch_permute_large(const PermuteArgs& p, void* scratch, cudaStream_t st) {
  const int chunks = int(((long long)p.tokens * p.topk + kPermChunk - 1) / kPermChunk);
  int* counts = static_cast<int*>(scratch);
  const size_t place_smem = size_t(32) * p.experts * sizeof(unsigned short);
  static bool configured[64] = {};      // the opt-in is per device
  const int dev = current_device_slot();
  if (dev < 0) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(permute_place_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 1024 * 2);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  cudaError_t e;
  if ((e = launch_pdl(permute_count_kernel<0>, dim3(chunks), dim3(kPermChunk), size_t(p.experts) * 4, st, p, counts))) return e;
  if ((e = launch_pdl(permute_scan_kernel<0>, dim3(1), dim3(1024), size_t(p.experts) * 4, st, p, counts, chunks))) return e;
  return launch_pdl(permute_place_kernel<0>, dim3(chunks), dim3(kPermChunk), place_smem, st, p, (const int*)counts);
}

}  // namespace dmoe
