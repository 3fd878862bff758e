// Hayate router top-k. This translation unit is compiled with --use_fast_math, as the reference
// builds its GLM kernels (hayate crates/kernels/build.rs:59), so that sigmoid(logit) + bias is
// formed with the same approximate exp / reciprocal and selects the same experts.
#include "../../include/darask_moe_b200.h"
#include "route_kernels.cuh"
#include "stream_launch.cuh"

using namespace dmoe;

extern "C" int darask_route_topk_hayate(const float* logits, int ld, int experts, int topk, int tokens,
                                        const float* bias, float scale, int* ids, float* weights, cudaStream_t st) {
  if (!logits || !bias || !ids || !weights || experts < 1 || experts > 1024 || topk < 1 || topk > 32 ||
      topk > experts || tokens < 1 || ld < experts)
    return cudaErrorInvalidValue;
  RouteArgs a{logits, ld, experts, topk, tokens, bias, scale, ids, weights, nullptr};
  return launch_pdl(route_topk_kernel<kRouteHayate>, dim3((tokens + 3) / 4), dim3(128), 0, st, a);
}
