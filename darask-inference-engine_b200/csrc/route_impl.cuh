// Router top-k for the three executors and the dispatch permutation (device code).
//
// Selection is bit-exact with the reference kernels given identical float32 logits: the same
// float32 key, k rounds of arg-max ordered by (key descending, expert id ascending), and the
// same math functions (this header is compiled twice: with precise math for the Kogarashi and
// Tsumuji routers, and with --use_fast_math for the Hayate router, as the reference builds are).
//   Kogarashi  key = logit;               w = softmax over the k selected   (kogarashi kernels/native.cu:100-112)
//   Tsumuji    key = expf(logit - max);   w = p / sum of selected p         (tsumuji kernels/decode/ops.cu:148-200)
//   Hayate     key = sigmoid(logit)+bias; w = score/(sum+1e-20)*scale       (hayate cu/glm53/ops.cu:100-114, decode.cu:23-31)
#pragma once
#include "common.cuh"

namespace dmoe {

enum RouteMode { kRouteKogarashi = 0, kRouteTsumuji = 1, kRouteHayate = 2 };

struct RouteArgs {
  const float* logits;   // [T][ld]
  int ld;                // row stride of logits (E, or E + 1 when the shared gate logit follows)
  int experts, topk, tokens;
  const float* bias;     // Hayate: [E]
  float scale;           // Hayate: routed scaling factor
  int* ids;              // [T][k], selection order
  float* weights;        // [T][k]
  float* shared_gate;    // Tsumuji: [T] = sigmoid(logits[E]); may be null
};

// One warp routes one token. MAXV * 32 >= experts.
template <int MODE, int MAXV>
DEVI void route_token(const RouteArgs& a, int token, int lane) {
  const float* lg = a.logits + size_t(token) * a.ld;
  const int E = a.experts, K = a.topk;
  float v[MAXV];
  float score[MODE == kRouteHayate ? MAXV : 1];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? __ldcg(lg + e) : -INFINITY;   // L2 read: another block may just have written it
    m = fmaxf(m, v[i]);
  }
  float s = 0.f;
  if (MODE == kRouteTsumuji) {
    m = warp_max(m);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      v[i] = lane + 32 * i < E ? expf(v[i] - m) : -1.f;   // -1: not a candidate
      s += fmaxf(v[i], 0.f);
    }
    s = warp_sum(s);
  } else if (MODE == kRouteHayate) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int e = lane + 32 * i;
      score[i] = e < E ? 1.f / (1.f + expf(-v[i])) : 0.f;
      v[i] = e < E ? score[i] + a.bias[e] : -INFINITY;
    }
  }
  const float floor_value = MODE == kRouteTsumuji ? -1.f : -INFINITY;
  const float taken_value = MODE == kRouteTsumuji ? -2.f : -INFINITY;
  float mine = 0.f;     // lane t keeps what slot t needs for the weights
  float total = 0.f;    // Tsumuji / Hayate: running sum in selection order
  float first = 0.f;    // Kogarashi: the largest logit
  for (int t = 0; t < K; ++t) {
    float bv = floor_value;
    int bi = MODE == kRouteTsumuji ? 0x7fffffff : 0;   // defaults of the reference kernels
    float bs = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i)
      if (v[i] > bv) {      // ascending index inside a lane: the first maximum wins
        bv = v[i];
        bi = lane + 32 * i;
        if (MODE == kRouteHayate) bs = score[i];
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      const float os = MODE == kRouteHayate ? __shfl_xor_sync(0xffffffffu, bs, o) : 0.f;
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
        bs = os;
      }
    }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int i = 0; i < MAXV; ++i)
        if (lane + 32 * i == bi) v[i] = taken_value;
    }
    if (lane == 0) a.ids[token * K + t] = bi;
    if (MODE == kRouteKogarashi) {
      if (t == 0) first = bv;
      if (lane == t) mine = bv;
    } else if (MODE == kRouteTsumuji) {
      if (lane == t) mine = bv / s;
      total += bv / s;
    } else {
      if (lane == t) mine = bs;
      total += bs;
    }
  }
  float* w = a.weights + size_t(token) * K;
  if (MODE == kRouteKogarashi) {
    // softmax over the selected logits; K <= 32, lane s holds logit s
    float z = lane < K ? expf(mine - first) : 0.f;
    const float denom = warp_sum(z);
    if (lane < K) w[lane] = z / denom;
  } else if (MODE == kRouteTsumuji) {
    if (lane < K) w[lane] = mine / total;
    if (lane == 0 && a.shared_gate) a.shared_gate[token] = 1.f / (1.f + expf(-__ldcg(lg + E)));
  } else {
    if (lane < K) w[lane] = mine / (total + 1.e-20f) * a.scale;
  }
}

template <int MODE>
DEVI void route_token_any(const RouteArgs& a, int token, int lane) {
  if (a.experts <= 128) route_token<MODE, 4>(a, token, lane);
  else if (a.experts <= 256) route_token<MODE, 8>(a, token, lane);
  else if (a.experts <= 512) route_token<MODE, 16>(a, token, lane);
  else route_token<MODE, 32>(a, token, lane);
}

// ---- dispatch permutation -------------------------------------------------------------------
// Stable counting sort of the assignment index a = token * k + slot by expert id: experts in
// ascending id, inside an expert ascending a (hayate crates/models/src/glm53/prefill.rs:12-26,
// gpu.rs:29-80). Outputs, all indexed by expert id unless noted:
//   ranges[e] = {rows, offset}   (offset = rows of all smaller ids)
//   assignments[offset .. offset + rows) = the a of expert e
//   active[0 .. n_active) = ids with rows > 0, ascending;  counters[0] = n_active
// Ids outside [0, E) or repeated inside a token set kStatusBadRoute and are dropped.
struct PermuteArgs {
  const int* ids;          // [T*k]
  int tokens, topk, experts;
  unsigned* assignments;   // [T*k]
  unsigned* ranges;        // [E][2]
  int* active;             // [E]
  int* counters;           // [4]: n_active, total rows, number of plan entries, 0
  unsigned* status;
  int4* plan;              // optional: per active expert {id, rows, offset, 0}, then (shared_rows > 0) {-1, shared_rows, 0, 0}
  int shared_rows;
};

// Runs in one thread block (any size that is a multiple of 32, >= 64). `hist` : E + 1 ints of
// shared memory. `ids`: the routes, p.ids or a copy of them in shared memory.
DEVI void permute_block(const PermuteArgs& p, int* hist, const int* ids) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int n = p.tokens * p.topk, E = p.experts, K = p.topk;
  for (int e = tid; e <= E; e += nthr) hist[e] = 0;
  __syncthreads();
  for (int a = tid; a < n; a += nthr) {
    const int e = ids[a];
    bool ok = e >= 0 && e < E;
    for (int j = a - a % K; ok && j < a; ++j) ok = ids[j] != e;
    if (ok) atomicAdd(&hist[e], 1);
    else atomicOr(p.status, kStatusBadRoute);
  }
  __syncthreads();
  // exclusive scan + active list by warp 0 (E <= 1024: 32 values per lane, then a lane scan)
  if (tid < 32) {
    const int per = (E + 31) / 32;
    int sum = 0, act = 0;
    for (int i = 0; i < per; ++i) {
      const int e = tid * per + i;
      if (e < E) {
        sum += hist[e];
        act += hist[e] > 0;
      }
    }
    int run = sum, arun = act;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, run, o), u = __shfl_up_sync(0xffffffffu, arun, o);
      if (tid >= o) {
        run += t;
        arun += u;
      }
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
        hist[e] = off;          // becomes the write cursor
        off += c;
      }
    }
    if (tid == 31) {
      p.counters[0] = arun;
      p.counters[1] = run;
      p.counters[2] = arun + (p.shared_rows > 0 ? 1 : 0);
      if (p.plan && p.shared_rows > 0) p.plan[arun] = make_int4(-1, p.shared_rows, 0, 0);
    }
    __syncwarp();
    // stable placement, 32 assignments per round
    for (int base = 0; base < n; base += 32) {
      const int a = base + tid;
      int e = a < n ? ids[a] : -1;
      bool ok = e >= 0 && e < E;
      for (int j = a - a % K; ok && j < a; ++j) ok = ids[j] != e;
      if (!ok) e = -1 - tid;    // unique key: never matches another lane
      const unsigned same = __match_any_sync(0xffffffffu, e);
      const int rank = __popc(same & ((1u << tid) - 1u));
      if (ok) p.assignments[hist[e] + rank] = a;
      __syncwarp();
      if (ok && rank == 0) hist[e] += __popc(same);
      __syncwarp();
    }
  }
}

}  // namespace dmoe
