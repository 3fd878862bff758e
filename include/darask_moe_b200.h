/* C ABI of the B200 (sm_100a) MoE FFN library, libdarask_moe_b200.so.
 *
 * Conventions, the same as the reference engine's kernel launchers
 * (engines/hayate/crates/kernels/src/cuda.rs:29-36): every call only enqueues work on the
 * given stream, never allocates and never synchronizes (the two *_status calls, which copy one
 * word back, are the exception); device pointers must stay valid until the stream has passed
 * the launch; the return value is a cudaError_t as int, cudaErrorInvalidValue (1) for
 * arguments that fail validation.  All pointers are device pointers unless a comment says
 * "host".  `stream` is a cudaStream_t / CUstream.
 */
#ifndef DARASK_MOE_B200_H
#define DARASK_MOE_B200_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* darask_stream_t;

/* GGML tensor type ids as the reference reads them (engines/kogarashi/crates/kogarashi-engine/
 * src/config.rs:86-105). */
enum { DARASK_GGML_F32 = 0, DARASK_GGML_F16 = 1, DARASK_GGML_Q4_K = 12, DARASK_GGML_Q6_K = 14, DARASK_GGML_BF16 = 30 };
enum { DARASK_ROUTE_KOGARASHI = 0, DARASK_ROUTE_TSUMUJI = 1, DARASK_ROUTE_HAYATE = 2 };
/* bits of the status word kept in every workspace */
enum {
  DARASK_STATUS_WAIT_TIMEOUT = 1,  /* a bounded device-side wait ran out; re-initialise the workspace before the next call */
  DARASK_STATUS_BAD_ROUTE = 2,     /* an expert id out of range or repeated inside a token was dropped */
  DARASK_STATUS_EP_OVERFLOW = 16,  /* expert-parallel slab capacity exceeded: rows were dropped, the layer's result is wrong */
  DARASK_STATUS_ACT_RANGE = 4      /* an activation or SwiGLU product exceeds 65504 in magnitude: the decode kernels hold
                                      activations as two fp16 planes (the reference reads float32), the result is not finite */
};

/* ---- routing ------------------------------------------------------------------------------
 * Top-k and gate weights from float32 logits [tokens][ld], bit-exact in ids and order with
 *   mode 0: kernel `route`        engines/kogarashi/kernels/native.cu:100-112
 *   mode 1: kernel `router_topk`  engines/tsumuji/kernels/decode/ops.cu:148-200 (shared_gate = sigmoid(logits[t][experts]))
 *   mode 2: `router_select`/`route` engines/hayate/crates/kernels/cu/glm53/decode.cu:23-31, ops.cu:100-114
 * but for any experts <= 1024 and topk <= 32 (the reference kernels hard-code 256/8 and 288/8). */
int darask_route_topk(int mode, const float* logits, int ld, int experts, int topk, int tokens,
                      const float* bias, float scale, int* ids, float* weights, float* shared_gate,
                      darask_stream_t stream);
int darask_route_topk_hayate(const float* logits, int ld, int experts, int topk, int tokens, const float* bias,
                             float scale, int* ids, float* weights, darask_stream_t stream);

/* Dispatch permutation on the device: replaces the host function `groups`
 * (engines/hayate/crates/models/src/glm53/prefill.rs:12-26) and `PackedMeta::push`
 * (models/src/glm53/gpu.rs:29-80).  ids [tokens*topk] -> assignments [tokens*topk] (assignment
 * index token*topk+slot, grouped by ascending expert id, ascending inside a group),
 * ranges [experts][2] = {rows, offset}, active [experts] = ids with rows > 0, counters[0] = their
 * number, counters[1] = total rows.  Ids out of range or repeated inside a token are dropped and
 * set DARASK_STATUS_BAD_ROUTE in *status. */
int darask_moe_permute(const int* ids, int tokens, int topk, int experts, unsigned* assignments, unsigned* ranges,
                       int* active, int* counters, unsigned* status, darask_stream_t stream);
/* The same permutation for prefill-sized batches, spread over many thread blocks (three launches);
 * `scratch`: darask_moe_permute_scratch_bytes(tokens, topk, experts) bytes of device memory. */
size_t darask_moe_permute_scratch_bytes(int tokens, int topk, int experts);
int darask_moe_permute_large(const int* ids, int tokens, int topk, int experts, unsigned* assignments, unsigned* ranges,
                             int* active, int* counters, unsigned* status, void* scratch, size_t scratch_bytes,
                             darask_stream_t stream);

/* ---- GGUF Q6_K device layout ------------------------------------------------------------------
 * Lossless regrouping of Q6_K rows (k/256 blocks of 210 bytes, never 16-byte aligned) into
 * rows of k/256 x 208 bytes [ql|qh|scales] followed by the k/256 f16 block scales, padded to
 * 16 bytes, which the TMA engine can stream.  Done once after the upload that replaces
 * engines/kogarashi/crates/kogarashi-engine/src/engine.rs:73-107.  inverse != 0 restores GGUF. */
size_t darask_q6k_repacked_bytes(long long rows, int k);
int darask_q6k_repack(void* dst, const void* src, long long rows, int k, int inverse, darask_stream_t stream);

/* ---- load-time quantizers ------------------------------------------------------------------------
 * float32 source on the device -> the byte layouts the expert kernels read.
 *   darask_quantize_nvfp4_linear  replaces kernels `nvfp4_amax` + `nvfp4_quant`
 *       (engines/tsumuji/kernels/decode/quant.cu:77-114): `matrices` matrices of rows x cols, matrix m read
 *       at src + m*src_stride (elements, rounded to bf16 first), codes written to dst + m*dst_stride +
 *       codes_off, e4m3 scales to dst + m*dst_stride + scales_off, global scale to gs[m*gs_stride].
 *   darask_quantize_nvfp4_tiled   one Hayate NVFP4 matrix image (codes | 128x4 tiled scales | f32), the
 *       arithmetic of engines/hayate/python-tools/hayate_tools/quant.py:42-64.
 *   darask_quantize_fp8_block     e4m3 payload [rows][cols] + float32 scale per 128x128 block
 *       (format `Fp8Block`, engines/hayate/crates/kernels/src/cpu/glm53.rs:23-24).
 *   darask_quantize_fp8_act       activations [rows][cols] (float32 or bf16) -> e4m3 codes + float32 scale per
 *       row and 128 channels; no counterpart in the reference (its activations stay bf16 / float32).
 *   darask_quantize_ggml          GGUF Q4_K (12) / Q6_K (14) blocks; the reference ships no quantizer for these
 *       (it decodes them: engines/kogarashi/kernels/native.cu:26-40), this one is this library's own.
 * amax_scratch: `matrices` (or 1) unsigned words of device scratch. */
int darask_quantize_ggml(void* dst, const float* src, int ty, long long elements, darask_stream_t stream);
int darask_quantize_nvfp4_linear(void* dst, long long dst_stride, long long codes_off, long long scales_off, float* gs,
                                 int gs_stride, const float* src, long long src_stride, int matrices, int rows, int cols,
                                 unsigned* amax_scratch, darask_stream_t stream);
int darask_quantize_nvfp4_tiled(void* dst, const float* src, int rows, int cols, unsigned* amax_scratch,
                                darask_stream_t stream);
int darask_quantize_fp8_block(void* payload, float* scales, const float* src, int rows, int cols, darask_stream_t stream);
int darask_quantize_fp8_act(void* codes, float* scales, const void* x, int x_is_bf16, long long rows, int cols,
                            darask_stream_t stream);

/* ---- Kogarashi MoE FFN layer -----------------------------------------------------------------
 * One call replaces the 12 launches of engines/kogarashi/crates/kogarashi-engine/src/engine.rs:
 * 530-632 (router `gemv`, `route`, expert `gemv` x3, `activate`, shared expert `gemv` x4,
 * `activate`, `combine`; kernels engines/kogarashi/kernels/native.cu:46-117) for `tokens` >= 1.
 * Weight tensors are the GGUF tensors of that call site in GGML order [k, rows, experts];
 * Q4_K tensors as uploaded, Q6_K tensors after darask_q6k_repack. */
typedef struct {
  int hidden, inter, experts, topk, tokens;
  const void* router_w; int router_ty;                 /* ffn_gate_inp        [hidden, experts]     */
  const float* router_bias;                            /* [experts] added to the logits; NULL as in the reference */
  const void* gate_w; int gate_ty;                     /* ffn_gate_exps       [hidden, inter, E]    */
  const void* up_w; int up_ty;                         /* ffn_up_exps                               */
  const void* down_w; int down_ty;                     /* ffn_down_exps       [inter, hidden, E]    */
  const void* sh_gate_w; const void* sh_up_w;          /* ffn_{gate,up}_shexp, same types; NULL: no shared expert */
  const void* sh_down_w;                               /* ffn_down_shexp                            */
  const void* sh_inp_w;                                /* ffn_gate_inp_shexp  [hidden], type router_ty */
  float* n;                                            /* [tokens][hidden] normalised input (buffer "n"); written when norm_w is set */
  float* x;                                            /* [tokens][hidden] residual stream, updated in place ("x") */
  float* logits;                                       /* [tokens][experts]   ("router")            */
  int* ids;                                            /* [tokens][topk]      ("ids")               */
  float* prob;                                         /* [tokens][topk]      ("prob")              */
  void* workspace; size_t workspace_bytes;
  /* Optional layer entry, the reference's `residual` and `rms_native` launches in front of the MoE block
   * (engines/kogarashi/kernels/native.cu:89-96, engine.rs:507-526).  norm_w != NULL: first x += attn_out (skipped when
   * attn_out is NULL), then n = x * rsqrt(mean(x^2) + norm_eps) * norm_w is formed by the layer itself and written to
   * `n`, which is then an output buffer.  norm_w == NULL: `n` is an input and attn_out must be NULL. */
  const float* attn_out;                               /* [tokens][hidden] ("out") */
  const float* norm_w;                                 /* post_attention_norm.weight [hidden] */
  float norm_eps;
  int reserved;                                        /* must be 0 */
} KogarashiMoe;
size_t kogarashi_moe_workspace_bytes(int hidden, int inter, int experts, int topk, int tokens);
/* zeroes the whole workspace, once after allocation (the control words, and the tagged words through which the
 * CTAs of the one-token launch hand values to each other: a workspace that was never cleared may hold a stale tag) */
int kogarashi_moe_workspace_init(void* workspace, size_t bytes, darask_stream_t stream);
int kogarashi_moe_layer(const KogarashiMoe* desc /* host */, darask_stream_t stream);
/* One token with an F32 router and Q4_K gate/up runs as ONE persistent launch (router rows, top-k in every CTA,
 * gate/up, down and combine; the CTAs hand logits, products and rows to each other as tagged words with bounded
 * polling, the weight stream running through); other shapes take four launches.  enabled = 0 makes the calling host thread take the four launches for one token as well
 * (no counterpart in the reference; used to compare the two paths). */
int kogarashi_moe_set_single_launch(int enabled);
/* copies the status word to *host_status and synchronizes the stream */
int kogarashi_moe_status(const void* workspace, unsigned* host_status /* host */, darask_stream_t stream);

/* Same layer, for callers that cannot hand over a workspace.  No counterpart in the reference.
 * Meant for hosts that have no device allocator at the call site: an FFI embedder that gave all
 * device memory to its own arena at start-up, or plugin code running after the point where its
 * engine forbids cudaMalloc.  The scratch is a fixed array inside the library
 * (kogarashi_moe_static_scratch_bytes() = 1 MiB per GPU, held from library load to process exit);
 * desc->workspace and desc->workspace_bytes are ignored.  Shapes whose scratch need
 * (kogarashi_moe_workspace_bytes) exceeds the array are refused with cudaErrorInvalidValue and a
 * message on stderr.  The call itself allocates nothing.  The first call on each device looks up
 * the array's device address (with that device current); make that first call before any stream
 * capture.  All calls on a device share the one array: calls whose kernels can overlap on the
 * GPU (different streams) race; serialize them.  Every call first clears the array's control
 * words (all but the call counter of the one-token launch), the status word among them: read the status of a call (kogarashi_moe_static_status,
 * which synchronizes the stream) before the next call if it matters.  A descriptor that fails
 * validation is refused before anything is enqueued. */
size_t kogarashi_moe_static_scratch_bytes(void);
int kogarashi_moe_layer_static(const KogarashiMoe* desc /* host */, darask_stream_t stream);
int kogarashi_moe_static_status(unsigned* host_status /* host */, darask_stream_t stream);

/* ---- Tsumuji MoE FFN layer ----------------------------------------------------------------------------
 * One call replaces `router_topk`, `moe_gate_up`, `moe_down` and the expert part of `moe_combine`
 * (engines/tsumuji/crates/tsumuji-engine/src/engine.rs:1586-1683; kernels engines/tsumuji/kernels/decode/ops.cu:148-230,
 * decode/gemv.cu:64-158) for a window of `tokens` tokens (the reference kernels stop at 8).
 * experts_w: routed experts, per expert one block of 27/16*F*H bytes
 *   [gate codes | up codes | down codes | gate sf | up sf | down sf] (engines/tsumuji/crates/tsumuji-engine/src/weights.rs:10-12),
 * gs: float32 [experts][3] global scales; shared_gu bf16 [2F][H] (gate rows, then up rows), shared_down bf16 [H][F].
 * router_w: bf16 [experts+1][H] (row `experts` = shared-expert gate) or NULL when rlogits already holds the
 * logits.  out[n] = sum_s w_s y_s + shared_gate y_shared (accumulate != 0: added to out; out may be NULL when R is
 * given).  R != NULL adds the rest of `moe_combine` (ops.cu:76-94, 202-230) to the same launch: the write-back
 * R[n][i] += inj_i * out[n] into the HC residual streams with inj_i = 2 sigmoid(sum_s di[s][n][rank+i] / HC), and
 * ss[n][b][i] = sum over the 256 columns of block b of the new R[n][i]^2 (the statistics the next norm reads). */
typedef struct {
  int hidden, inter, experts, topk, tokens;
  const void* router_w;
  const void* experts_w; const float* gs;
  const void* shared_gu; const void* shared_down;
  const float* x;                 /* [tokens][hidden] float32 ("inp")                          */
  float* out;                     /* [tokens][hidden]                                          */
  float* rlogits;                 /* [tokens][experts+1]                                       */
  int* sel; float* rw;            /* [tokens][topk]                                            */
  float* shared_gate;             /* [tokens]                                                  */
  int accumulate;
  void* workspace; size_t workspace_bytes;
  float* R;                       /* [tokens][HC][hidden] residual streams, updated in place; NULL: no write-back */
  const float* di;                /* [Sd][tokens][ld] partial sums of the stream-gate projection                  */
  int Sd, ld, rank, HC;           /* HC <= 8 streams; their gate logits are di[..][rank .. rank+HC)               */
  float* ss;                      /* [tokens][ceil(hidden/256)][HC]                                               */
} TsumujiMoe;
size_t tsumuji_moe_workspace_bytes(int hidden, int inter, int experts, int topk, int tokens);
/* zeroes the control words once after allocation (same as kogarashi_moe_workspace_init) */
int tsumuji_moe_workspace_init(void* workspace, size_t bytes, darask_stream_t stream);
int tsumuji_moe_layer(const TsumujiMoe* desc /* host */, darask_stream_t stream);
/* The same layer cut at the two exchange steps of expert parallelism (rank g holds experts [g*E/G, (g+1)*E/G) and its
 * own tokens; the reference has no multi-GPU path).  Home rank: tsumuji_ep_dispatch = router projection, router_topk,
 * permutation over all E experts, the token rows gathered in ascending expert order (send_x float32
 * [tokens*topk][hidden], ranges [E][2], position[a] = dispatch row of assignment a) and the shared expert
 * (y_shared [tokens][hidden]).  Expert rank: tsumuji_ep_experts = gate/up + SwiGLU + down over the received rows
 * (grouped by source rank, then local expert; recv_counts int32 [ranks][local_experts]) -> y_rows in received order.
 * Home rank: tsumuji_ep_combine = sum_s rw*y[position] in slot order, then the gated shared expert (ops.cu:217-223). */
int tsumuji_ep_dispatch(const TsumujiMoe* desc /* host; out unused */, float* send_x, unsigned* ranges, unsigned* position,
                        float* y_shared, darask_stream_t stream);
size_t tsumuji_ep_experts_workspace_bytes(int hidden, int inter, int local_experts, int rows);
int tsumuji_ep_experts(const void* experts_w, const float* gs, int hidden, int inter, int local_experts, int ranks,
                       const int* recv_counts, const float* x_rows, int rows, float* y_rows, void* workspace,
                       size_t workspace_bytes, darask_stream_t stream);
int tsumuji_ep_combine(float* out, const float* y_home, const float* rw, const unsigned* position, const float* shared_gate,
                       const float* y_shared, int tokens, int hidden, int topk, int accumulate, darask_stream_t stream);


/* ---- Hayate (GLM) ------------------------------------------------------------------------------------------
 * Same names, argument order and error behaviour as the reference launchers
 * (engines/hayate/crates/kernels/cu/glm53/decode.cu:69-88, ops.cu:308-311; Rust declarations
 * engines/hayate/crates/kernels/src/glm53.rs:539-577, 847-860).  The reference hard-codes hidden 4096,
 * intermediate 2048, 288 experts, top-8 and scale 2.5; here those are the defaults of a host-thread-local shape
 * that hayate_glm_moe_set_shape changes (the reference already keeps one such thread-local knob,
 * hayate_glm_grouped_packed_set_config, packed_grouped.cu:269,315-318).  The expert launchers need scratch for the
 * fp16 activation planes and the routing plan: register it once per host thread with hayate_glm_moe_set_workspace
 * (hayate_glm_moe_workspace_bytes(hidden, inter, experts, topk, 1) bytes); the router calls work without it.
 * NVFP4 and block-FP8 images are implemented; the combinations are listed in front of hayate_glm_moe_gate_up. */
typedef struct { const void* data; const void* scale; unsigned format; } HayateDenseWeight;
int hayate_glm_moe_set_shape(unsigned hidden, unsigned inter, unsigned experts, unsigned topk, float scale);
size_t hayate_glm_moe_workspace_bytes(unsigned hidden, unsigned inter, unsigned experts, unsigned topk, unsigned tokens);
int hayate_glm_moe_set_workspace(void* workspace, size_t bytes, darask_stream_t stream);
int hayate_glm_route_decode(void* logits, void* weights, void* ids, const void* x, const void* w, const void* bias, darask_stream_t stream);
int hayate_glm_route(void* logits, void* weights, void* ids, const void* x, const void* w, const void* bias, unsigned tokens,
                     unsigned hidden, unsigned experts, unsigned topk, darask_stream_t stream);
int hayate_glm_route_batch(void* logits, void* weights, void* ids, const void* x, const void* w, const void* bias, unsigned m,
                           darask_stream_t stream);
/* images: device array of top-k image pointers in route order; a null pointer leaves a zero row (the reference's
 * "computed on the CPU" slot).  out: bf16 [topk+1][inter], row topk = shared expert. */
/* Image formats of the expert launchers: nv != 0: NVFP4 tiled images with the shared expert's DenseWeight.format == 3;
 * nv == 0 (gate/up and down) or down_fp8 != 0 (down only): block-FP8 images (payload [n][k], float32 scales [n/128][k/128]
 * right behind it, decode.cu:32-36) with the shared expert as format 1 {data, scale}.  Other combinations: cudaErrorInvalidValue. */
int hayate_glm_moe_gate_up(void* out, const void* x, const void* original, const void* images, HayateDenseWeight gate,
                           HayateDenseWeight up, int nv, int down_fp8, size_t stride, darask_stream_t stream);
int hayate_glm_moe_down(void* out, const void* x, const void* images, HayateDenseWeight shared, int nv, int down_fp8,
                        size_t stride, darask_stream_t stream);
int hayate_glm_moe_reduce(void* out, const void* x, const void* ids, const void* weights, darask_stream_t stream);

/* Whole Hayate MoE layer for `tokens` tokens with every expert image resident in one slab (images + e * 3 * stride:
 * gate | up | down at `stride`), replacing the route -> host lookup -> gate_up -> down -> reduce sequence of
 * engines/hayate/crates/models/src/glm53/gpu.rs:1612-1757 including its device->host copy of the ids. */
typedef struct {
  int hidden, inter, experts, topk, tokens;
  float scale;                          /* routed scaling factor (2.5 in the reference)           */
  const void* router_w;                 /* bf16 [experts][hidden]                                 */
  const float* bias;                    /* [experts], selection only                              */
  const void* images; size_t stride;    /* NVFP4 expert images                                    */
  const void* shared_image;             /* gate | up | down of the shared expert at `stride`      */
  const void* x;                        /* bf16 [tokens][hidden]                                  */
  void* out;                            /* bf16 [tokens][hidden]                                  */
  float* logits; int* ids; float* weights;
  void* workspace; size_t workspace_bytes;
} HayateMoe;
size_t hayate_moe_workspace_bytes(int hidden, int inter, int experts, int topk, int tokens);
int hayate_moe_workspace_init(void* workspace, size_t bytes, darask_stream_t stream);
int hayate_moe_layer(const HayateMoe* desc /* host */, darask_stream_t stream);

/* Hayate prefill launchers, the reference's names and signatures (engines/hayate/crates/kernels/src/glm53.rs:588-650,
 * bodies cu/glm53/grouped.cu:28-124).  x / out / w are bf16; ranges u32 [groups][2] = {rows, offset}; assignments
 * index [token][topk] routes (topk from hayate_glm_moe_set_shape, 8 by default as in the reference).  The grouped
 * GEMM accepts any n % 128 == 0, k % 64 == 0 and up to 1024 groups (the reference: two fixed shapes, 8 groups) and
 * ignores `metadata`.  hayate_glm_grouped_nvfp4: accumulator = float32 x.w^T, out = bf16(accumulator * scales[g]). */
int hayate_glm_grouped(void* out, const void* x, const void* w, const void* ranges, unsigned groups, unsigned n, unsigned k,
                       void* metadata, darask_stream_t stream);
int hayate_glm_grouped_nvfp4(void* out, void* accumulator, const void* x, const void* w, const void* ranges, unsigned groups,
                             unsigned n, unsigned k, void* metadata, const void* scales, unsigned max_rows, darask_stream_t stream);
/* block-FP8 matrix (e4m3 payload, float32 scale per 128x128) -> bf16 (glm53.rs:746-753) */
int hayate_glm_restore(void* out, const void* w, const void* scale, unsigned n, unsigned k, darask_stream_t stream);
int hayate_glm_nvfp4_restore(void* out, const void* image, unsigned n, unsigned k, darask_stream_t stream);
int hayate_glm_nvfp4_restore_unscaled(void* out, void* scale, const void* image, unsigned n, unsigned k, darask_stream_t stream);
int hayate_glm_gather(void* out, const void* x, const void* assignments, unsigned rows, unsigned hidden, darask_stream_t stream);
int hayate_glm_scatter(void* out, const void* x, const void* weights, const void* assignments, unsigned rows, unsigned hidden,
                       darask_stream_t stream);
int hayate_glm_copy(void* out, const void* x, size_t bytes, darask_stream_t stream);
/* Ragged grouped GEMM on the experts' packed NVFP4 images, read in place: the reference's names and signatures
 * (engines/hayate/crates/kernels/src/glm53.rs:2843-2870, bodies cu/glm53/packed_grouped.cu:302-318).  images: device
 * array of `count` image pointers ([gate | up | down] at the 256-byte-aligned stride of lowbit.cuh:9-13); formats:
 * device array of `count` ExpertFormat (8 bytes: gate_up and down {format, grid, group, reserved}); ranges u32
 * [count][2] = {rows, offset}.  gate_up: x [rows][hidden] bf16 -> product [rows][intermediate] bf16 =
 * swiglu(bf16(x.gate * s_gate), bf16(x.up * s_up)); down: product -> out [rows][hidden] bf16 = bf16(product.down * s_down).
 * count <= 288, hidden and intermediate multiples of 256 up to 4096, out != x (the reference's checks).  Only format 0
 * (NVFP4) images are multiplied: the LOWBIT grids are outside this library, an expert with another format or a null
 * image gets zero rows and bit 8 in the word hayate_glm_grouped_packed_status returns (and clears; synchronizes the
 * stream; no counterpart in the reference, whose launchers have no status either).  set_config accepts the
 * reference's ids 0-3 and changes nothing: there is one tcgen05 tile shape. */
int hayate_glm_grouped_packed_set_config(unsigned config);
int hayate_glm_grouped_packed_gate_up(void* product, const void* x, const void* images, const void* formats, const void* ranges,
                                      unsigned count, unsigned hidden, unsigned intermediate, darask_stream_t stream);
int hayate_glm_grouped_packed_down(void* out, const void* product, const void* images, const void* formats, const void* ranges,
                                   unsigned count, unsigned hidden, unsigned intermediate, darask_stream_t stream);
int hayate_glm_grouped_packed_status(unsigned* host_status /* host */, darask_stream_t stream);

/* ---- FP8 prefill path -----------------------------------------------------------------------------------------
 * Ragged grouped GEMM on tcgen05 tensor cores over block-scaled e4m3 operands.  Replaces hayate_glm_grouped /
 * hayate_glm_grouped_nvfp4 (engines/hayate/crates/kernels/cu/glm53/grouped.cu:59-124: CUTLASS Sm80 grouped GEMM on
 * weights restored to bf16) and hayate_glm_grouped_packed_{gate_up,down} (packed_grouped.cu:177-318) for the
 * FP8 format: a_codes e4m3 [a_rows][k] with a_scales float32 [a_rows][k/128] (rows in dispatch order; the buffer
 * must reach one 128-row tile past the last expert's rows), w e4m3 [experts][n][k] with sw float32
 * [experts][n/128][k/128], ranges [experts][2] = {rows, offset}.  n and k multiples of 128.
 *   mode 0: out = a.w0^T as float32 [a_rows][n]; with out_row_map, dispatch row i is written to row out_row_map[i]
 *   mode 1: out = silu(a.w0^T) * (a.w1^T) as bf16 [a_rows][n]
 *   mode 2: the same product rounded to bf16, then quantized: out = e4m3 codes [a_rows][n], out_scales float32
 *           [a_rows][n/128] = absmax/448 of each 128 columns (1 where they are all zero) */
int darask_fp8_grouped_gemm(const void* a_codes, const float* a_scales, unsigned long long a_rows, const void* w0,
                            const void* w1, const float* sw0, const float* sw1, int experts, int n, int k, int mode,
                            const unsigned* ranges, void* out, float* out_scales, const unsigned* out_row_map,
                            unsigned* status, darask_stream_t stream);
/* Whole FP8 MoE layer for a prefill batch: softmax top-k (renormalised) on the given logits, activations
 * quantized to e4m3 per token and 128 channels, dispatch gather, grouped gate/up GEMM with SwiGLU, products
 * quantized the same way, grouped down GEMM, combine.  Mirrors `prefill_experts`
 * (engines/hayate/crates/models/src/glm53/gpu.rs:2068-2566) without its device->host copy of the routes. */
typedef struct {
  int hidden, inter, experts, topk, tokens;
  const void* x;                        /* bf16 [tokens][hidden]                                         */
  const float* logits;                  /* [tokens][experts]                                             */
  const void* gate_w; const void* up_w; const void* down_w;     /* e4m3 [E][inter][hidden] x2, [E][hidden][inter] */
  const float* gate_s; const float* up_s; const float* down_s;  /* float32 per 128x128 block              */
  float* out;                           /* float32 [tokens][hidden]                                      */
  int* ids; float* prob;                /* [tokens][topk]                                                */
  void* workspace; size_t workspace_bytes;
} DaraskFp8Moe;
size_t darask_fp8_moe_workspace_bytes(int hidden, int inter, int experts, int topk, int tokens);
int darask_fp8_moe_layer(const DaraskFp8Moe* desc /* host */, darask_stream_t stream);
int darask_fp8_moe_status(const void* workspace, unsigned* host_status /* host */, darask_stream_t stream);

/* ---- expert-parallel FP8 prefill: the same layer cut at its two exchange steps ---------------------------------
 * Rank g of G holds experts [g*E/G, (g+1)*E/G) and its own tokens.  Per layer and rank:
 *   1. darask_fp8_ep_dispatch   route (softmax top-k, renormalised), permutation over all E experts, activation
 *                               quantization, gather: send_codes / send_scales hold the token rows in ascending
 *                               expert order (so already grouped by destination rank), ranges [E][2] their
 *                               {rows, offset}, position[a] the dispatch row of assignment a = token*topk+slot.
 *   2. host: all-to-all of the per-expert counts, then all-to-all-v of rows and scales (NCCL).
 *   3. darask_fp8_ep_regroup    received rows (by source rank, then local expert) -> local expert order;
 *                               ranges [E/G][2], row_map[regrouped row] = received row.
 *   4. darask_fp8_ep_experts    grouped gate/up GEMM + SwiGLU + quantization, grouped down GEMM; y float32
 *                               [received rows][hidden] written back in RECEIVED order through row_map.
 *   5. host: all-to-all-v of y back (splits swapped): rows return in the sender's dispatch order.
 *   6. darask_fp8_ep_combine    out[t] = sum_s prob[t][s] * y[position[t*topk+s]]  (slot order, fp32 fma).
 * These replace the host-side `group_routes` + gather/scatter of `prefill_experts`
 * (engines/hayate/crates/models/src/glm53/gpu.rs:2068-2566); the reference has no multi-GPU path.
 * Buffers holding rows that feed a grouped GEMM (send_codes at G = 1, codes, prod_codes and their scales) must reach
 * 128 rows past the last used row.  recv_counts: int32 [G][E/G], row r = the counts rank r sends here. */
size_t darask_fp8_ep_dispatch_scratch_bytes(int hidden, int experts, int topk, int tokens);
int darask_fp8_ep_dispatch(const void* x /* bf16 [tokens][hidden] */, const float* logits, int hidden, int experts, int topk,
                           int tokens, int* ids, float* prob, void* send_codes, float* send_scales, unsigned* ranges,
                           unsigned* position, void* scratch, size_t scratch_bytes, darask_stream_t stream);
int darask_fp8_ep_regroup(const int* recv_counts, int ranks, int local_experts, const void* recv_codes,
                          const float* recv_scales, int hidden, long long recv_rows, void* codes, float* scales,
                          unsigned* ranges, unsigned* row_map, void* scratch /* ranks*local_experts*8 bytes */,
                          size_t scratch_bytes, darask_stream_t stream);
int darask_fp8_ep_experts(const void* codes, const float* scales, unsigned long long rows_alloc, const unsigned* ranges,
                          int local_experts, int hidden, int inter, const void* gate_w, const void* up_w, const void* down_w,
                          const float* gate_s, const float* up_s, const float* down_s, const unsigned* row_map, float* y,
                          void* prod_codes /* [rows_alloc][inter] */, float* prod_scales /* [rows_alloc][inter/128] */,
                          unsigned* status, darask_stream_t stream);
int darask_fp8_ep_combine(float* out, const float* y, const float* prob, const unsigned* position, int tokens, int hidden,
                          int topk, darask_stream_t stream);
/* The same layer with exchanges whose sizes the host never needs ("packed"): rows travel in slabs of `cap` rows per
 * (source, destination) pair (cap = tokens*topk is a rank's worst case; with a smaller cap the rows that do not fit are
 * dropped, bit 16 is set in *status and the result is wrong: raise the capacity) as packed rows of darask_fp8_ep_packed_row_bytes
 * bytes [codes | scales | routing weight | token], so both exchanges and the counts are equal-split all-to-alls and no
 * device->host copy sits between the launches; the expert rank adds a token's rows (weight * row, ascending local expert)
 * before they return, so one float32 row per (token, expert rank) comes back, dense by token, and the home rank adds the
 * ranks' partial rows in ascending rank order (P2's pre-reduction; the summation order differs from the single-GPU slot
 * order, inside the layer tolerance).
 *   1. darask_fp8_ep_dispatch_packed  send [ranks][cap] packed rows; counts [E] = rows per expert that are in the slabs
 *   2. all-to-all of counts [ranks][E/ranks] and of the slabs
 *   3. darask_fp8_ep_regroup_packed   slabs -> codes / scales in local expert order, ranges [E/ranks][2], per row its
 *                                     source rank, token and weight
 *   4. darask_fp8_ep_experts          with row_map = NULL and rows_alloc = ranks*cap + 128: y in regrouped order
 *   5. darask_fp8_ep_reduce           z [ranks][tcap][hidden] (count: ranks*tcap ints, list: ranks*tcap*topk ints)
 *   6. all-to-all of z; darask_fp8_ep_sum  out[t] = sum_r zr[r][t] */
size_t darask_fp8_ep_packed_row_bytes(int hidden);
int darask_fp8_ep_dispatch_packed(const void* x, const float* logits, int hidden, int experts, int topk, int tokens, int ranks,
                                  int cap, int* ids, float* prob, void* send, int* counts /* [experts] */, unsigned* ranges,
                                  unsigned* position, unsigned* status, void* scratch, size_t scratch_bytes, darask_stream_t stream);
int darask_fp8_ep_regroup_packed(const int* recv_counts, int ranks, int local_experts, const void* recv, int cap, int hidden,
                                 void* codes, float* scales, unsigned* ranges, unsigned* row_map, int* meta_src, int* meta_tok,
                                 float* meta_prob, void* scratch /* ranks*local_experts*8 bytes */, size_t scratch_bytes,
                                 darask_stream_t stream);
int darask_fp8_ep_reduce(const float* y, const unsigned* ranges, int local_experts, const int* meta_src, const int* meta_tok,
                         const float* meta_prob, int ranks, int cap, int tcap, int topk, int hidden, float* z, int* count, int* list,
                         unsigned* status, darask_stream_t stream);
int darask_fp8_ep_sum(float* out, const float* zr, int ranks, int tokens, int tcap, int hidden, darask_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
