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

// ---- selection as an arg-max over packed 64-bit words -------------------------------------------
// A candidate is one word: the float32 key mapped to an unsigned integer of the same order in the
// high half, (2^32 - 1 - expert id) in the low half. The largest word is the largest key and, among
// equal keys, the lowest id; a taken or absent candidate is the word 0. Results equal k rounds of
// "first maximum wins" over the float keys, which is what the three reference routers do.
DEVI uint32_t ordered_bits(float key) {
  if (!(key == key)) key = -INFINITY;          // a NaN key never wins against a number
  const uint32_t b = __float_as_uint(key + 0.f);   // -0 and +0 are the same key
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
DEVI float ordered_value(uint32_t o) { return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o); }
DEVI unsigned long long pack_candidate(float key, int expert) {
  return (static_cast<unsigned long long>(ordered_bits(key)) << 32) | (0xffffffffu - static_cast<uint32_t>(expert));
}
// Largest packed candidate of the warp: the largest key by one hardware reduction, then among the lanes that hold
// it the largest low half (= the lowest expert id) by a second one.
DEVI unsigned long long warp_max_u64(unsigned long long v) {
  const uint32_t hi = static_cast<uint32_t>(v >> 32), lo = static_cast<uint32_t>(v);
  const uint32_t top = __reduce_max_sync(0xffffffffu, hi);
  const uint32_t low = __reduce_max_sync(0xffffffffu, hi == top ? lo : 0u);
  return (static_cast<unsigned long long>(top) << 32) | low;
}

// Compare-exchange of two candidates, larger first.
DEVI void order_pair(unsigned long long& x, unsigned long long& y) {
  const unsigned long long hi = x > y ? x : y, lo = x > y ? y : x;
  x = hi;
  y = lo;
}
// This lane's candidates in descending order (sorting networks of 3 / 19 exchanges).
template <int PER>
DEVI void sort_candidates(unsigned long long (&c)[PER]) {
  static_assert(PER == 4 || PER == 8, "networks for 4 and 8 candidates");
  if (PER == 4) {
    order_pair(c[0], c[1]); order_pair(c[2], c[3]);
    order_pair(c[0], c[2]); order_pair(c[1], c[3]);
    order_pair(c[1], c[2]);
  } else {
    order_pair(c[0], c[1]); order_pair(c[2], c[3]); order_pair(c[4 % PER], c[5 % PER]); order_pair(c[6 % PER], c[7 % PER]);
    order_pair(c[0], c[2]); order_pair(c[1], c[3]); order_pair(c[4 % PER], c[6 % PER]); order_pair(c[5 % PER], c[7 % PER]);
    order_pair(c[1], c[2]); order_pair(c[5 % PER], c[6 % PER]);
    order_pair(c[0], c[4 % PER]); order_pair(c[1], c[5 % PER]); order_pair(c[2], c[6 % PER]); order_pair(c[3], c[7 % PER]);
    order_pair(c[2], c[4 % PER]); order_pair(c[3], c[5 % PER]);
    order_pair(c[1], c[2]); order_pair(c[3], c[4 % PER]); order_pair(c[5 % PER], c[6 % PER]);
  }
}

// A logit from global memory (through L2: another block may have written it) or from the caller's shared memory.
DEVI float load_logit(const float* p) { return __isGlobal(p) ? __ldcg(p) : *p; }
// One warp routes one token; lane l owns experts l, l + 32, ... (PER * 32 >= experts). `ids_out` / `w_out`
// (k entries each) may point to global or shared memory, and so may the logits.
template <int MODE, int PER>
DEVI void route_token(const RouteArgs& a, int token, int lane, int* ids_out, float* w_out) {
  const float* row = a.logits + size_t(token) * a.ld;
  const int E = a.experts, K = a.topk;
  float logit[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) logit[i] = lane + 32 * i < E ? load_logit(row + lane + 32 * i) : -INFINITY;
  unsigned long long cand[PER];
  float score[MODE == kRouteHayate ? PER : 1];
  float norm = 1.f;                          // Tsumuji: sum over all experts of exp(logit - max)
  if (MODE == kRouteKogarashi) {
#pragma unroll
    for (int i = 0; i < PER; ++i) cand[i] = lane + 32 * i < E ? pack_candidate(logit[i], lane + 32 * i) : 0ull;
  } else if (MODE == kRouteTsumuji) {
    float top = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) top = fmaxf(top, logit[i]);
    top = warp_max(top);
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const bool live = lane + 32 * i < E;
      const float key = live ? expf(logit[i] - top) : 0.f;
      part += key;
      cand[i] = live ? pack_candidate(key, lane + 32 * i) : 0ull;
    }
    norm = warp_sum(part);
  } else {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      score[i] = e < E ? 1.f / (1.f + expf(-logit[i])) : 0.f;
      cand[i] = e < E ? pack_candidate(score[i] + a.bias[e], e) : 0ull;
    }
  }
  // Few candidates per lane and no per-candidate side value: each lane sorts its own once, its best is then the
  // first, and the lane that wins a round shifts its list. (Same words, same order of winners.)
  constexpr bool SORTED = PER <= 8 && MODE != kRouteHayate;
  if constexpr (SORTED) sort_candidates(cand);
  float keep = 0.f;       // lane t keeps the quantity slot t's weight is made from
  float running = 0.f;    // Tsumuji / Hayate: sum over the selected, in selection order
  float lead = 0.f;       // Kogarashi: the first (largest) selected logit
  for (int t = 0; t < K; ++t) {
    unsigned long long best = 0ull;
    if (SORTED) {
      best = cand[0];
    } else {
#pragma unroll
      for (int i = 0; i < PER; ++i) best = cand[i] > best ? cand[i] : best;
    }
    best = warp_max_u64(best);
    const int winner = int(0xffffffffu - static_cast<uint32_t>(best));
    const float key = ordered_value(static_cast<uint32_t>(best >> 32));
    float won_score = 0.f;
    if (SORTED) {
      if ((winner & 31) == lane) {
#pragma unroll
        for (int i = 0; i + 1 < PER; ++i) cand[i] = cand[i + 1];
        cand[PER - 1] = 0ull;
      }
    } else {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const bool hit = (winner & 31) == lane && (winner >> 5) == i;
        if (MODE == kRouteHayate && hit) won_score = score[i];
        if (hit) cand[i] = 0ull;
      }
    }
    if (lane == 0) ids_out[t] = winner;
    if (MODE == kRouteKogarashi) {
      if (t == 0) lead = key;
      if (lane == t) keep = key;
    } else if (MODE == kRouteTsumuji) {
      const float p = key / norm;
      if (lane == t) keep = p;
      running += p;
    } else {
      won_score = __shfl_sync(0xffffffffu, won_score, winner & 31);
      if (lane == t) keep = won_score;
      running += won_score;
    }
  }
  if (MODE == kRouteKogarashi) {       // softmax over the selected logits (K <= 32: lane s holds logit s)
    const float z = lane < K ? expf(keep - lead) : 0.f;
    const float denom = warp_sum(z);
    if (lane < K) w_out[lane] = z / denom;
  } else if (MODE == kRouteTsumuji) {
    if (lane < K) w_out[lane] = keep / running;
    if (lane == 0 && a.shared_gate) a.shared_gate[token] = 1.f / (1.f + expf(-load_logit(row + E)));
  } else {
    if (lane < K) w_out[lane] = keep / (running + 1.e-20f) * a.scale;
  }
}

template <int MODE>
DEVI void route_token_to(const RouteArgs& a, int token, int lane, int* ids_out, float* w_out) {
  if (a.experts <= 128) route_token<MODE, 4>(a, token, lane, ids_out, w_out);
  else if (a.experts <= 256) route_token<MODE, 8>(a, token, lane, ids_out, w_out);
  else if (a.experts <= 512) route_token<MODE, 16>(a, token, lane, ids_out, w_out);
  else route_token<MODE, 32>(a, token, lane, ids_out, w_out);
}

template <int MODE>
DEVI void route_token_any(const RouteArgs& a, int token, int lane) {
  route_token_to<MODE>(a, token, lane, a.ids + size_t(token) * a.topk, a.weights + size_t(token) * a.topk);
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
