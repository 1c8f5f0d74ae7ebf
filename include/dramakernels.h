/* C ABI of libdramakernels.so — the sm_100a (B200) implementation of drama-rs's routed-expert MoE
 * path and the dense weight-streaming GEMVs around it.
 *
 * Every function below has the name, argument order and argument meaning of the launcher it
 * replaces in the reference's kernels/drama.cu, as bound by the reference's src/ffi.rs; each
 * declaration cites both. A host that links the reference's libdramakernels.a can link this
 * library for these symbols without source changes.
 *
 * Conventions (reference: src/gpu.rs:9-26, kernels/drama.cu:1-8):
 *   - launchers return 0, -1 for a shape they do not support, or -2 when the per-device setup
 *     has not run and cannot run now (first call made inside a stream capture without any of
 *     dr_stream_create / dr_malloc / dr_cublas_create / dr_sample_init / drb_init before it);
 *   - runtime wrappers return the cudaError_t as int;
 *   - the stream is the last argument; nothing synchronises, allocates or reads device values
 *     on the host inside a launcher, so every launcher can be captured in a CUDA graph;
 *   - all buffers are owned by the caller; weight pointers must be 16-byte aligned.
 *
 * Weight formats (reference: src/model.rs:16-43, tools/convert.py:33-41, 92-101):
 *   Q8: int8 [N, K] row-major + f16 scale [N, K/128];             w = q * scale
 *   Q4: u8 [E, N, K/2], low nibble = even k, nibble 0..15
 *       + f16 [E, N, K/64, 2] = (scale, min) per 64 inputs;       w = q * scale + min
 */
#ifndef DRAMAKERNELS_H
#define DRAMAKERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* dr_stream;     /* cudaStream_t */
typedef void* dr_graph_exec; /* cudaGraphExec_t */
typedef uint16_t dr_bf16;    /* bfloat16 bit pattern */
typedef uint16_t dr_half;    /* IEEE binary16 bit pattern */

/* ---- runtime wrappers: kernels/drama.cu:1991-2037, src/ffi.rs:13-30 ------------------------ */
const char* dr_error_string(int e);                             /* drama.cu:1998, ffi.rs:13 */
int dr_last_error(void);                                        /* drama.cu:1991, ffi.rs:14 */
int dr_malloc(void** p, size_t n);                              /* drama.cu:1999, ffi.rs:15 */
int dr_free(void* p);                                           /* drama.cu:2000, ffi.rs:16 */
int dr_host_alloc(void** p, size_t n);                          /* drama.cu:2001, ffi.rs:17 */
int dr_host_free(void* p);                                      /* drama.cu:2002, ffi.rs:18 */
int dr_h2d(void* d, const void* h, size_t n, dr_stream st);     /* drama.cu:2003, ffi.rs:19 */
int dr_d2h(void* h, const void* d, size_t n, dr_stream st);     /* drama.cu:2006, ffi.rs:20 */
int dr_d2d(void* d, const void* s, size_t n, dr_stream st);     /* drama.cu:2009, ffi.rs:21 */
int dr_memset(void* d, int v, size_t n, dr_stream st);          /* drama.cu:2012, ffi.rs:22 */
int dr_stream_create(dr_stream* s);                             /* drama.cu:2013, ffi.rs:23 */
int dr_stream_sync(dr_stream s);                                /* drama.cu:2014, ffi.rs:24 */
int dr_device_sync(void);                                       /* drama.cu:2015 */
int dr_mem_info(size_t* free_b, size_t* total_b);               /* drama.cu:2016, ffi.rs:25 */
int dr_graph_begin(dr_stream s);                                /* drama.cu:2018, ffi.rs:26 */
int dr_graph_end(dr_stream s, dr_graph_exec* exec);             /* drama.cu:2019, ffi.rs:27 */
int dr_graph_launch(dr_graph_exec exec, dr_stream s);           /* drama.cu:2027, ffi.rs:28 */
int dr_graph_destroy(dr_graph_exec exec);                       /* drama.cu:2028, ffi.rs:29 */
int dr_cublas_create(void** h, dr_stream s);                    /* drama.cu:2030, ffi.rs:30 */
int dr_sample_init(void);                                       /* ffi.rs:105 (pre-capture hook only) */

/* C[M,N] f32 = A[M,K] bf16 . W[N,K]^T bf16 + beta*C (cuBLAS). drama.cu:2040-2044, ffi.rs:31 */
int dr_gemm(void* h, const dr_bf16* a, const dr_bf16* w, float* c, int m, int n, int k, float beta);

/* ---- dense GEMVs, batch 1 ----------------------------------------------------------------- */

/* y[n] = W[n] . x' (+ res[n]);  x' = rmsnorm(x, nw, eps) when nw != NULL, else x. y may alias res.
 * K in {512, 2048, 4096, 6144, 8192}. pf/pf_bytes: a region to prefetch into L2 (the next kernel's
 * weights), or NULL. drama.cu:222-240, 283-294; ffi.rs:33-36 */
int dr_gemv_q8(const int8_t* w, const dr_half* s, const float* x, const float* res, float* y, int n, int k,
               const float* nw, float eps, const char* pf, size_t pf_bytes, dr_stream st);

/* y[j] = silu(W[j] . x') * (W[i + j] . x'), W is [2i, k]. K in {2048, 4096}.
 * drama.cu:242-261, 296-305; ffi.rs:37-39 */
int dr_gemv_q8_swiglu(const int8_t* w, const dr_half* s, const float* x, float* y, int i, int k, const float* nw,
                      float eps, const char* pf, size_t pf_bytes, dr_stream st);

/* y[n] = W[n] . x' for bf16 weights. K == 2048. drama.cu:263-279, 307-315; ffi.rs:40 */
int dr_gemv_bf16(const dr_bf16* w, const float* x, float* y, int n, int k, const float* nw, float eps,
                 const char* pf, size_t pf_bytes, dr_stream st);

/* ---- routing ------------------------------------------------------------------------------ */

/* Decode router: logits[0..e] = W[e+1, k] . rmsnorm(x); softmax over the first e, top-k in
 * descending probability (ties to the lower index), wts renormalised, sgate = logits[e].
 * counter: one zeroed u32 that is left zero. gu_q != NULL asks for an L2 prefetch of the chosen
 * experts (sizes in bytes per expert). k == 2048, e <= 256, topk <= 32.
 * drama.cu:371-461; ffi.rs:56-60 */
int dr_router_topk(const dr_bf16* w, const float* x, const float* nw, float eps, float* logits, int e, int topk,
                   int k, int* idx, float* wts, float* sgate, unsigned* counter, const char* gu_q, const char* gu_sm,
                   const char* d_q, const char* d_sm, size_t gu_q_b, size_t gu_sm_b, size_t d_q_b, size_t d_sm_b,
                   dr_stream st);

/* Prefill routing over precomputed logits [rows, stride] (column e = shared gate).
 * drama.cu:322-367, 463-468; ffi.rs:41 */
int dr_moe_topk(const float* logits, int rows, int e, int topk, int stride, int* idx, float* wts, float* sgate,
                dr_stream st);

/* ---- MoE decode, batch 1 ------------------------------------------------------------------ */

/* y = res + sigmoid(sgate) * shared(x') + sum_k wts[k] * expert_{idx[k]}(x'), x' = rmsnorm(x, nw, eps).
 * act: scratch of (topk + 1) * i floats. x, res and y may be the same buffer.
 * h == 2048, i == 512, topk == 8. drama.cu:470-599; ffi.rs:42-46 */
int dr_moe_decode(const uint8_t* gu_q, const dr_half* gu_sm, const uint8_t* d_q, const dr_half* d_sm,
                  const int8_t* sgu_q, const dr_half* sgu_s, const int8_t* sd_q, const dr_half* sd_s, const float* x,
                  const int* idx, const float* wts, const float* sgate, const float* res, float* act, float* y, int h,
                  int i, int topk, const float* nw, float eps, const char* pf, size_t pf_bytes, dr_stream st);

/* The same layer with block-FP8 routed experts (the checkpoint's own format): gu_w E4M3 [E, 2i, h] (gate rows, then
 * up rows) with gu_s f32 [E, 2i/128, h/128], d_w E4M3 [E, h, i] with d_s f32 [E, h/128, i/128];
 * weight = e4m3(byte) * scale of its 128 x 128 block. The shared expert stays int8. Same limits.
 * drama.cu:602-742; ffi.rs:47-51 */
int dr_moe_decode_fp8(const uint8_t* gu_w, const float* gu_s, const uint8_t* d_w, const float* d_s,
                      const int8_t* sgu_q, const dr_half* sgu_s, const int8_t* sd_q, const dr_half* sd_s, const float* x,
                      const int* idx, const float* wts, const float* sgate, const float* res, float* act, float* y, int h,
                      int i, int topk, const float* nw, float eps, const char* pf, size_t pf_bytes, dr_stream st);

/* ---- MoE prefill -------------------------------------------------------------------------- */

int dr_moe_count(const int* idx, int n, int* counts, dr_stream st); /* drama.cu:745-753; ffi.rs:65 */
/* drama.cu:755-778; ffi.rs:66-69 */
int dr_moe_permute(const int* idx, int rows, int topk, const int* offsets, int* fill, int* slot_of, const dr_bf16* x,
                   dr_bf16* xp, int h, dr_stream st);
/* Rows of xp sorted by expert (offsets/counts). act: scratch, 16 bits per (slot, j), contents
 * unspecified. y[slot, :] = down_e(silu(gate_e . x) * (up_e . x)). h == 2048, i == 512.
 * drama.cu:799-968; ffi.rs:61-64 */
int dr_moe_prefill(const uint8_t* gu_q, const dr_half* gu_sm, const uint8_t* d_q, const dr_half* d_sm,
                   const dr_bf16* xp, const int* offsets, const int* counts, dr_bf16* act, float* y, int e, int h, int i,
                   dr_stream st);
/* dr_moe_prefill over block-FP8 experts (layouts as dr_moe_decode_fp8). drama.cu:971-1109; ffi.rs:52-55 */
int dr_moe_prefill_fp8(const uint8_t* gu_w, const float* gu_s, const uint8_t* d_w, const float* d_s, const dr_bf16* xp,
                       const int* offsets, const int* counts, dr_bf16* act, float* y, int e, int h, int i, dr_stream st);
/* drama.cu:780-797; ffi.rs:70-73 */
int dr_moe_combine(float* x, const float* y, const int* slot_of, const float* wts, const float* sgate,
                   const float* shared, int rows, int topk, int h, dr_stream st);

/* ---- elementwise helpers of the prefill path ------------------------------------------------ */
int dr_dequant_q8(const int8_t* w, const dr_half* s, dr_bf16* out, int n, int k, dr_stream st); /* drama.cu:1114-1134; ffi.rs:74 */
int dr_f32_to_bf16(const float* x, dr_bf16* y, size_t n, dr_stream st);                         /* drama.cu:1158-1166; ffi.rs:75 */
int dr_swiglu_rows(const float* h, dr_bf16* y, int rows, int i, dr_stream st);                  /* drama.cu:1168-1180; ffi.rs:76 */
int dr_rmsnorm(const float* x, const float* w, float* y, dr_bf16* yb, int rows, int d, float eps,
               dr_stream st);                                                                   /* drama.cu:1182-1202; ffi.rs:77 */

/* dr_moe_decode for callers that have no scratch to pass and may not allocate any (memory budget fixed at
 * start-up, allocator owned by another component, a capture running on another thread). It has no
 * counterpart in the reference. The (topk + 1) * i floats live in a fixed 18 KB device array inside the
 * library, so: shapes beyond h = 2048, i = 512, topk = 8 return -1; calls that overlap on the GPU race on
 * that array (same-stream calls are fine); the first call per device does a one-time set-up without
 * allocating and should be made outside stream capture. */
int dr_moe_decode_static(const uint8_t* gu_q, const dr_half* gu_sm, const uint8_t* d_q, const dr_half* d_sm,
                         const int8_t* sgu_q, const dr_half* sgu_s, const int8_t* sd_q, const dr_half* sd_s,
                         const float* x, const int* idx, const float* wts, const float* sgate, const float* res,
                         float* y, int h, int i, int topk, const float* nw, float eps, const char* pf, size_t pf_bytes,
                         dr_stream st);

/* ---- additions of this library; no counterpart in the reference ----------------------------- */
/* One layer's weights for drb_moe_stack_decode: device pointers in the layouts above. */
typedef struct {
  const void *router, *post_norm, *gu_q, *gu_sm, *d_q, *d_sm, *sgu_q, *sgu_s, *sd_q, *sd_s;
} drb_moe_layer;
/* x <- x + moe_l(rmsnorm(x, post_norm_l)) for l = 0 .. n_layers-1, in place, as ONE persistent cooperative
 * kernel (the benchmark's 40-layer decode step without per-layer launches). layers: device array.
 * workspace: drb_moe_stack_workspace_bytes() bytes of device memory. idx_trace / wts_trace: optional
 * [n_layers, topk] device arrays receiving each layer's routing. h == 2048, i == 512, topk == 8, e <= 256,
 * >= 148 multiprocessors; -1 otherwise. The per-layer dr_router_topk + dr_moe_decode compute the same. */
int drb_moe_stack_workspace_bytes(void);
int drb_moe_stack_decode(const drb_moe_layer* layers, int n_layers, float* x, void* workspace, int e, int topk, int h,
                         int i, float eps, int* idx_trace, float* wts_trace, dr_stream st);
/* offsets[e] = counts[0] + ... + counts[e-1] on the device: replaces the reference's host-side scan between
 * dr_moe_count and dr_moe_permute (src/engine.rs:567-574), so the prefill sequence needs no host round trip. */
int drb_moe_offsets(const int* counts, int e, int* offsets, dr_stream st);
/* logits [rows, e1] = xb [rows, h] . w [e1, h]^T + beta * logits (bf16 inputs, fp32 sums in a fixed order), such that a
 * row's logits do not depend on how many rows are computed together. The reference uses cublasGemmEx for these
 * logits (src/engine.rs:554), whose kernel choice, and with it the last bits of a row, changes with the batch size;
 * a host that spreads rows over several GPUs uses this call so that the routing is the same at every split.
 * h == 2048, else -1. */
int drb_router_logits(const dr_bf16* xb, const dr_bf16* w, float* logits, int rows, int e1, int h, float beta, dr_stream st);
/* Chained decode: dr_moe_decode as one link of a chain over consecutive MoE layers, on a caller-owned workspace of
 * drb_moe_chain_workspace_bytes() bytes (zeroed once by the caller, private to one stream of launches).
 *   next_router != NULL: the down kernel also computes the NEXT layer's routing. Every block adds its share of
 *     next_router . (y * next_nw) and of sum(y^2) to fixed-point accumulators in the workspace (integer atomics: the
 *     totals do not depend on the order of arrival); the last block to arrive applies rsqrt(mean(y^2) + eps), runs
 *     softmax + top-k and OVERWRITES idx / wts / sgate (and logits [e_next + 1], if not NULL) with the next layer's
 *     routing: what dr_router_topk(next_router, y, next_nw, eps, ...) would write. The router rows are fetched while
 *     the kernel waits for its activations, so the next layer needs no router launch.
 *   next_router == NULL ends the chain: idx / wts / sgate are left as they are.
 *   have_prev != 0: this layer's routing was produced by the previous chained call on the same workspace and x is that
 *     call's y; both are then read from replicas in the workspace (one per group of blocks, so that 148 blocks do not
 *     read the same cache lines at once). idx / wts / sgate / x are still passed and hold the same values.
 * topk == 8, 8 <= e_next <= 256, h == 2048; other limits and return codes as dr_moe_decode. In the reference's engine
 * the call replaces dr_moe_decode(layer l) and dr_router_topk(layer l + 1) (src/engine.rs:959-1042). */
int drb_moe_decode_chained(const uint8_t* gu_q, const dr_half* gu_sm, const uint8_t* d_q, const dr_half* d_sm,
                           const int8_t* sgu_q, const dr_half* sgu_s, const int8_t* sd_q, const dr_half* sd_s,
                           const float* x, int* idx, float* wts, float* sgate, const float* res, float* act, float* y,
                           int h, int i, int topk, const float* nw, float eps, const dr_bf16* next_router,
                           const float* next_nw, int e_next, float* logits, float* workspace, int have_prev,
                           dr_stream st);
size_t drb_moe_chain_workspace_bytes(void);
/* The checkpoint quantisers of the reference's converter on the GPU (tools/convert.py:33-41 `quant_q8`, 44-101
 * `quant_q4_groups` / `quant_q4`: 24-step clipping search with a least-squares refit). w: `groups` x 64 (q4) or
 * 128 (q8) consecutive floats, i.e. a row-major weight whose last dimension is a multiple of the group; outputs in
 * the layouts above (q4: 32 bytes per group, low nibble = even k, and f16 (scale, min); q8: codes and f16 scale). */
int drb_quant_q4(const float* w, size_t groups, uint8_t* q, dr_half* sm, dr_stream st);
int drb_quant_q8(const float* w, size_t groups, int8_t* q, dr_half* s, dr_stream st);
int dr_stream_destroy(dr_stream s);
int dr_cublas_destroy(void* h);
int drb_init(void);                    /* per-device setup; also run by the pre-capture hooks above */
int drb_device_error(unsigned* out);   /* reads and clears the bounded-wait error word; synchronises */
int drb_grid_blocks(void);             /* blocks of the persistent kernels on the current device */

#ifdef __cplusplus
}
#endif
#endif /* DRAMAKERNELS_H */
