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
/* dr_moe_prefill over block-FP8 experts (layouts as dr_moe_decode_fp8). The weight bytes reach the tensor cores as
 * E4M3 (tiled TMA, tcgen05 kind::f8f6f4); the block scales ride on the token operand. Until its rows are written, y is
 * scratch (its first floats hold every token row's largest magnitude), as act is. gu_w and d_w 16-byte aligned.
 * Returns -3 if a tensor map cannot be encoded. e > 256, or DRB_FP8_DEQUANT=1 in the environment: the kernels that turn
 * the weights into fp16 first. drama.cu:971-1109; ffi.rs:52-55 */
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
 * kernel (the benchmark's 40-layer decode step without per-layer launches; what src/engine.rs:946-1042 issues as
 * dr_router_topk + dr_moe_decode per layer). layers: device array. workspace: drb_moe_stack_workspace_bytes() bytes
 * of device memory, 256-byte aligned, any contents (every call clears it first, on `st`); calls that share a
 * workspace must not overlap on the GPU. idx_trace / wts_trace: optional [n_layers, topk] device arrays receiving
 * each layer's routing. Blocks hand the hidden state, the router logits and the activations to one another as
 * tagged 64-bit words; every wait on such a word is bounded and reports through drb_device_error().
 * The top-k is chosen on the logits (softmax is monotonic), ties towards the lower index as dr_moe_topk does; the
 * weights are the softmax over all e logits, renormalised over the chosen k.
 * h == 2048, i == 512, topk == 8, topk <= e <= 256, at least 144 multiprocessors (one block each, all resident);
 * -1 otherwise. Capturable in a graph. */
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
/* ---- prefill without a library GEMM, a permuted copy or a host round trip -------------------- */
/* dr_rmsnorm / drb_router_logits for rows kept in fp16 (the reference rounds the normalised rows to bf16,
 * src/engine.rs:499): yh [rows, d] = fp16(rmsnorm(x) * w), clamped to +-65504; logits as drb_router_logits. With
 * drb_moe_prefill_block(x_f16 = 1) the whole block then works on rows with eleven significant bits instead of eight. */
int drb_rmsnorm_f16(const float* x, const float* w, dr_half* yh, int rows, int d, float eps, dr_stream st);
int drb_router_logits_f16(const dr_half* xh, const dr_bf16* w, float* logits, int rows, int e1, int h, float beta, dr_stream st);
/* Count, exclusive scan and slot assignment of the (row, k) pairs in one launch: counts [e_n], offsets [e_n],
 * slot_of [rows * topk] (-1 for a pair whose expert lies outside [e_lo, e_lo + e_n)), row_of [slot] = row.
 * Replaces dr_moe_count + the host scan + dr_moe_permute (src/engine.rs:565-580) when the grouped GEMM is
 * drb_moe_prefill_block, which reads its rows through row_of. The order of the slots inside an expert is
 * arbitrary, as dr_moe_permute's is (both assign them by atomics); no result depends on it. e_n <= 1024, else -1. */
int drb_moe_group(const int* idx, int rows, int topk, int e_lo, int e_n, int* counts, int* offsets, int* slot_of,
                  int* row_of, dr_stream st);
/* The routed experts AND the int8 shared expert of one prefill block in two launches: dr_moe_prefill with
 * (a) the operand rows read in place through row_of (xb: the normalised rows in row order, [rows_sh, h], bf16 or with
 *     x_f16 != 0 fp16; row_of == NULL: slot s reads row s, as dr_moe_prefill does), and
 * (b) the shared expert as one more expert that owns every row, its int8 weights dequantised into the same
 *     tensor-core tiles (sh_act: 16-bit scratch [rows_sh, i]; sh_out: f32 [rows_sh, h]). The reference runs it through
 *     cuBLAS on weights dequantised to bf16 (src/engine.rs:351-355, 560-562).
 * y [slots, h] f32; y_row_of (or NULL): slot -> row of y. rows_sh = 0 skips the shared expert, e = 0 the routed
 * ones. Every pointer except row_of / y_row_of must be a valid device address even for a part that does not run
 * (any buffer will do): NULL returns -1. Intermediates are fp16: SwiGLU values beyond +-65504 are clamped.
 * h == 2048, i == 512, else -1. With x_f16 != 0 and e <= 256 the weights are addressed through TMA tensor maps built
 * from the pointers given (gu_q / d_q: e experts from the pointer on); -3 when the driver refuses a map. */
int drb_moe_prefill_block(const uint8_t* gu_q, const dr_half* gu_sm, const uint8_t* d_q, const dr_half* d_sm,
                          const int8_t* sgu_q, const dr_half* sgu_s, const int8_t* sd_q, const dr_half* sd_s,
                          const dr_bf16* xb, const int* row_of, const int* offsets, const int* counts, dr_bf16* act,
                          float* y, dr_bf16* sh_act, float* sh_out, int rows_sh, int e, int h, int i, int x_f16,
                          const int* y_row_of, dr_stream st);
/* ---- expert parallelism (the reference is single-GPU) ---------------------------------------- */
/* Rows travel between ranks in a buffer of `world` blocks; a block is drb_ep_block_rows(cap, row_bytes) rows of
 * row_bytes bytes: cap row slots, then the cap local expert ids of those rows (int32, `per` = empty slot), padded
 * to whole rows, so that ONE fixed-size all-to-all moves rows and ids together and no sizes are exchanged first.
 *   drb_ep_pack   sender: places this rank's (row, k) pairs (idx [n_rows, topk]; `per` experts per rank) into `send`;
 *                 slot_of [n_rows * topk] = owner * cap + slot, for dr_moe_combine on the returned rows;
 *                 dst_row [n_rows * topk]: scratch. *overflow (device word, zeroed by the caller) is set when a
 *                 block was full: the step's result is void then, and the caller repeats it with a larger cap.
 *   drb_ep_group  owner: groups the received world * cap pairs by local expert: counts / offsets [per],
 *                 slot_of [world * cap] scratch, row_of [slot] = row of `recv` (operand gather of
 *                 drb_moe_prefill_block), pair_of [slot] = position of the pair in receive order (its y_row_of).
 * row_bytes % 16 == 0, world <= 64, per <= 1024; -1 otherwise. */
int drb_ep_block_rows(int cap, int row_bytes);
int drb_ep_pack(const void* rows, const int* idx, int n_rows, int topk, int per, int world, int cap, int row_bytes,
                void* send, int* slot_of, int* dst_row, unsigned* overflow, dr_stream st);
int drb_ep_group(const void* recv, int world, int cap, int row_bytes, int per, int* counts, int* offsets, int* slot_of,
                 int* row_of, int* pair_of, dr_stream st);
/* The exchange itself over NVLink peer stores instead of a library collective. peer_recv / peer_flags: device arrays
 * of `world` pointers, entry p = rank p's receive buffer / flag array (memory every rank can store to, e.g. symmetric
 * memory), this rank's own included.
 *   drb_ep_put     block p (block_bytes each) of `send` -> peer p's receive buffer at slot `rank`, 16-byte stores
 *   drb_ep_signal  ++*step (device word, zero at start on every rank); peer p's flag [rank] = *step
 *   drb_ep_wait    ++*step (another device word, zero at start); returns once flags [0, world) have all reached it, or
 *                  after poll_limit polls (drb_device_error() then reads non-zero and the step's result is void)
 * One exchange = put + signal on the sender, wait on the receiver before it reads. A rank may start its next
 * exchange into a peer's buffer only after that peer's reply to the current one (the combine step's wait).
 * block_bytes % 16 == 0, world <= 64, else -1. */
int drb_ep_put(const void* send, void* const* peer_recv, int world, int rank, size_t block_bytes, dr_stream st);
/* drb_ep_pack with the blocks stored straight into the owners' receive buffers (this rank's block in peer o's buffer is
 * block `rank`; no local send buffer, no drb_ep_put), and drb_moe_prefill_block (fp16 rows, e <= 256) with the routed
 * results stored straight into the home ranks' result buffers from the down GEMM's epilogue: y_row_of[slot] = s * cap + j
 * names the token's source rank s and its slot j in this rank's receive order (drb_ep_group's pair_of); the row goes to
 * peer_y[s] ([world * cap, h] f32 on rank s) at row rank * cap + j. y must be a valid address and is not written.
 * Either call is followed by drb_ep_signal on this rank and awaited with drb_ep_wait on the peers. */
int drb_ep_pack_peers(const void* rows, const int* idx, int n_rows, int topk, int per, int world, int cap, int row_bytes,
                      void* const* peer_recv, int rank, int* slot_of, int* dst_row, unsigned* overflow, dr_stream st);
int drb_moe_prefill_block_peers(const uint8_t* gu_q, const dr_half* gu_sm, const uint8_t* d_q, const dr_half* d_sm,
                                const int8_t* sgu_q, const dr_half* sgu_s, const int8_t* sd_q, const dr_half* sd_s,
                                const dr_bf16* xb, const int* row_of, const int* offsets, const int* counts, dr_bf16* act,
                                float* y, dr_bf16* sh_act, float* sh_out, int rows_sh, int e, int h, int i,
                                const int* y_row_of, float* const* peer_y, int cap, int rank, dr_stream st);
int drb_ep_signal(unsigned* const* peer_flags, int world, int rank, unsigned* step, dr_stream st);
int drb_ep_wait(const unsigned* flags, int world, unsigned* step, unsigned poll_limit, dr_stream st);
/* drb_ep_signal followed by drb_ep_wait in one launch; steps: two device words (signalled, awaited), zero at start. */
int drb_ep_sync(unsigned* const* peer_flags, const unsigned* flags, int world, int rank, unsigned* steps, unsigned poll_limit,
                dr_stream st);
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
/* Test hook: one block whose bounded wait runs out after `limit` polls (which: 1 = copy wait of the per-layer
 * kernels, 2 = copy wait of the persistent kernel, 3 = its tagged-word polls; word: 512 zeroed device bytes; clocks:
 * device word or NULL). The launch completes normally and the code is read with drb_device_error().
 * limit <= 65536 (milliseconds at most), else -1. */
int drb_test_wait_runs_out(int which, unsigned limit, const void* word, unsigned* clocks, dr_stream st);

#ifdef __cplusplus
}
#endif
#endif /* DRAMAKERNELS_H */
