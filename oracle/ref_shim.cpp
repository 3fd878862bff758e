// Thin C wrapper around the reference engine's host-compilable arithmetic headers.
// TEST INFRASTRUCTURE: compiled by oracle/build_ref.py with -I pointing at the reference
// checkout (engines/hayate/crates/kernels/cu/glm53); the reference sources are included from
// where they lie and are never copied.  The resulting library validates oracle/*.py.
#include "packed_grouped.cu"   // host half: lowbit.cuh + math.cuh + weight_pair/find_expert
#include "async_math.cuh"
extern "C" {
float ref_fp8(unsigned char b) { return glm53::fp8(b); }
float ref_bf16(float x) { return glm53::bf16(x); }
float ref_sigmoid(float x) { return glm53::sigmoid(x); }
float ref_swiglu(float g, float u) { return glm53::swiglu(g, u); }
void ref_route_order(int* order, const int* ids) { glm53::route_order(order, ids); }
float ref_expert_add(float s, float v, float w) { return glm53::expert_add(s, v, w); }
float ref_scaled_fp8(unsigned char v, float s) { return glm53::scaled_fp8(v, s); }
float ref_nvfp4(const unsigned char* image, unsigned r, unsigned c, unsigned n, unsigned k, int scaled) {
  return glm53::nvfp4(image, r, c, n, k, scaled != 0);
}
unsigned ref_weight_pair(const unsigned char* image, unsigned r, unsigned c, unsigned n, unsigned k) {
  return glm53::packed_grouped::weight_pair(image, r, c, n, k, glm53::lowbit::MatrixFormat{0, 0, 0, 0});
}
unsigned long long ref_storage(unsigned n, unsigned k) { return glm53::lowbit::storage(n, k, {0, 0, 0, 0}); }
unsigned long long ref_stride(unsigned n, unsigned k) { return glm53::lowbit::stride(n, k, {0, 0, 0, 0}); }
unsigned ref_tile_count(unsigned rows, unsigned n, unsigned tm, unsigned tn) {
  return glm53::packed_grouped::tile_count(rows, n, tm, tn);
}
unsigned ref_find_expert(const unsigned* ends, unsigned count, unsigned tile) {
  return glm53::packed_grouped::find_expert(ends, count, tile);
}
}
