/*
 * lmoe.h -- C ABI of the B200 (sm_100a) backend for the quantized indexed
 * mixture-of-experts path of the "laguna" engine: on-GPU routing, the indexed
 * Q4_K / Q6_K expert matmuls (decode mat-vec and prefill grouped GEMM), SwiGLU,
 * weighted combine and the shared expert.
 *
 * Every entry point mirrors one function of the reference's `src/ops` dispatch
 * layer or of `src/moe.rs`; the comment above each declaration names the
 * reference interface it replaces (path:line inside the reference project).
 *
 * Conventions
 *   - All data pointers are DEVICE pointers on the current CUDA device unless
 *     the parameter name ends in `_host`.  Tensors are dense row-major f32
 *     (activations, weights of the router) or u32 (expert ids), exactly the
 *     dtypes the reference validates (src/ops/dispatch.rs:812-833).
 *   - `stream` is a `cudaStream_t` passed as `void *` (NULL = default stream).
 *     Like the reference (src/ops/dispatch.rs:891-917) every op is
 *     asynchronous: it is enqueued on the stream and returns.
 *   - Return value: 0 on success, a negative `lmoe_status` otherwise; the
 *     message is available from `lmoe_last_error()` (thread-local).  Shape or
 *     dtype mismatches are reported as errors before anything is launched --
 *     never as a GPU fault (src/ops/mv_id.rs:137-145).
 *   - No entry point allocates device memory on the hot path except the
 *     `*_create` functions.  Scratch is supplied by the caller; its size comes
 *     from the `*_workspace_bytes` queries.
 *   - There is no CPU fallback.  Without a CUDA device every compute entry
 *     point fails with LMOE_ERR_CUDA.
 */
#ifndef LMOE_H
#define LMOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t lmoe_status;

enum {
    LMOE_OK = 0,
    LMOE_ERR_INVALID = -1,     /* shape / dtype / argument mismatch */
    LMOE_ERR_UNSUPPORTED = -2, /* valid request this build has no kernel for */
    LMOE_ERR_CUDA = -3,        /* CUDA runtime error (message has the detail) */
    LMOE_ERR_WORKSPACE = -4,   /* workspace missing, too small or misaligned */
    LMOE_ERR_DEVICE_FLAG = -5  /* a kernel recorded a bounded-wait timeout or index-guard trip */
};

/* ggml type ids of the two expert formats (src/gguf.rs:244-276 keeps the GGUF
 * dtype on the stack; the official checkpoint uses Q4_K gate/up, Q6_K down). */
enum {
    LMOE_Q4_K = 12, /* 144-byte super-block, 256 weights (src/ops/mv.metal:55-60) */
    LMOE_Q6_K = 14  /* 210-byte super-block, 256 weights (src/ops/mv.metal:70-75) */
};

/* The reference's own switch from the indexed mat-vec to the grouped GEMM:
 * `MM_ID_MIN_SEQ`, src/ops/mod.rs:31 (kept for documentation; see lmoe_mm_id_min_seq). */
#define LMOE_MM_ID_MIN_SEQ 32
/* Tokens one launch of the fused mat-vec (decode) kernel serves.  On B200 that kernel, which takes all 64
 * tokens in one launch and streams each of their distinct experts once, is ahead of the grouped GEMM up to
 * here (535 against 901 us per layer at 64 tokens). */
#define LMOE_DECODE_MAX_SEQ 64

const char *lmoe_version(void);
/* Token count from which every entry that picks a path itself (lmoe_moe_forward_host,
 * lmoe_moe_layer_forward, lmoe_experts_forward, and the host mirrors above this ABI) uses the grouped
 * GEMM; below it the mat-vec kernel.  LMOE_DECODE_MAX_SEQ + 1 unless the reference's process-wide switches
 * are set (src/ops/mod.rs:24-60): LAGUNA_MM_ID_MIN_SEQ=<n> moves it, LAGUNA_NO_MM_ID (presence) forces the
 * mat-vec path everywhere.  Read once per process. */
int64_t lmoe_mm_id_min_seq(void);
/* Message of the last failing call made by this thread ("" if none). */
const char *lmoe_last_error(void);

/* ------------------------------------------------------------------ stack --
 * `ExpertStack`, src/gguf.rs:247-276: `[n_expert][n_out][k/256]` super-blocks,
 * expert-major, contiguous, byte-identical to the GGUF tensor data.
 * `base_off` (bytes, multiple of 16) is the offset of the first block inside
 * the device allocation, kept for signature compatibility with the reference's
 * page-floored mmap views (src/gguf.rs:617-658). */
typedef struct lmoe_expert_stack lmoe_expert_stack;

/* `Weights::expert_stack` (src/gguf.rs:554-607): one upload of the raw
 * super-blocks into device memory, layout unchanged. `nbytes` must equal
 * n_expert * n_out * (k/256) * type_size. */
lmoe_status lmoe_expert_stack_create(int32_t dtype, int64_t n_expert, int64_t n_out, int64_t k,
                                     const void *bytes_host, size_t nbytes, size_t base_off,
                                     lmoe_expert_stack **out);
/* Zero-copy view over super-blocks already resident in device memory (the
 * counterpart of `expert_stack_mmap`, src/gguf.rs:617-658). The caller keeps
 * the allocation alive; `device_base + base_off` must be 16-byte aligned. */
lmoe_status lmoe_expert_stack_wrap(int32_t dtype, int64_t n_expert, int64_t n_out, int64_t k,
                                   const void *device_base, size_t nbytes, size_t base_off,
                                   lmoe_expert_stack **out);
void lmoe_expert_stack_destroy(lmoe_expert_stack *stack);
/* First super-block on the device (base + base_off). */
const void *lmoe_expert_stack_device_ptr(const lmoe_expert_stack *stack);
/* Shape query: any out pointer may be NULL. */
lmoe_status lmoe_expert_stack_info(const lmoe_expert_stack *stack, int32_t *dtype, int64_t *n_expert,
                                   int64_t *n_out, int64_t *k, size_t *nbytes);

/* Encode f32 rows into Q4_K / Q6_K super-blocks on the device (a deterministic
 * encoder used to build synthetic stacks; the reference calls candle's
 * `QTensor::quantize` for this in its tests, src/ops/dispatch.rs:2234).
 * `src` holds nblocks*256 floats, `dst` nblocks*type_size bytes. */
lmoe_status lmoe_quantize(int32_t dtype, const float *src, int64_t nblocks, void *dst, void *stream);
/* Decode super-blocks to f32 on the device (`QTensor::dequantize`). */
lmoe_status lmoe_dequantize(int32_t dtype, const void *src, int64_t nblocks, float *dst, void *stream);

/* ---------------------------------------------------------------- routing --
 * `MoeBlock::route` = `route_logits` + `route_from_logits`, src/moe.rs:62-119:
 * logits = x . router^T; p = sigmoid(logits); selection = p + bias; ids = the
 * first top_k of the stable descending order of `selection` (ties -> lower
 * expert index); weights = p[ids], divided by max(sum, 2^-14) when `norm`,
 * times `scale` unless scale is 0 or 1.
 *   router [n_expert, hidden] f32 (GGUF `ffn_gate_inp` orientation),
 *   bias [n_expert] f32 or NULL, x [t, hidden] f32,
 *   ids_out [t, top_k] u32, weights_out [t, top_k] f32.
 * Workspace: lmoe_route_workspace_bytes(t, n_expert). */
size_t lmoe_route_workspace_bytes(int64_t t, int64_t n_expert);
lmoe_status lmoe_route(const float *router, const float *bias, const float *x, int64_t t, int64_t hidden,
                       int64_t n_expert, int64_t top_k, float scale, int32_t norm, uint32_t *ids_out,
                       float *weights_out, void *workspace, size_t workspace_bytes, void *stream);
/* `lmoe_route` for callers that cannot allocate device memory when they route (a host engine
 * whose pool owns the device, a loop under a fixed memory budget, code inside a stream
 * capture): same arguments and results, but the logits scratch is a fixed array inside the
 * library instead of a workspace.  It has no counterpart in the reference.
 *   - limit: t * n_expert <= 32768 (128 KB of scratch held by every GPU that loads the
 *     library, until exit); larger requests are rejected with LMOE_ERR_INVALID;
 *   - the first call on each device looks up the array's device address, and the first call with
 *     more than 64 tokens and hidden = 3072 also sets a kernel attribute (cudaFuncSetAttribute):
 *     make one call of each kind you will use before starting any stream capture;
 *   - all calls share the one array (it keeps the previous call's logits; nothing needs
 *     clearing because each call overwrites what it reads): calls that overlap on the GPU,
 *     e.g. on two streams, race.
 * No cudaMalloc / cudaFree or allocating library routine is called. */
lmoe_status lmoe_route_noalloc(const float *router, const float *bias, const float *x, int64_t t, int64_t hidden,
                               int64_t n_expert, int64_t top_k, float scale, int32_t norm, uint32_t *ids_out,
                               float *weights_out, void *stream);
/* `route_from_logits` alone, src/moe.rs:94-119 (logits [t, n_expert] f32). */
lmoe_status lmoe_route_from_logits(const float *logits, const float *bias, int64_t t, int64_t n_expert,
                                   int64_t top_k, float scale, int32_t norm, uint32_t *ids_out,
                                   float *weights_out, void *stream);

/* -------------------------------------------------------- indexed mat-vec --
 * `ops::mul_mv_id`, src/ops/mv_id.rs:37-45 -> `run_inner`,
 * src/ops/dispatch.rs:799-918 -> kernel_mul_mv_id_q{4,6}_K_f32_v,
 * src/ops/mv.metal:181-290, 413-504, 638-717.
 *   out[t, s, :] = W[ids[t, s]] . x[t, (x_per_row == 1 ? 0 : s), :]
 *   x [t, x_per_row, k] f32, ids [t_ids, top_k] u32, out [t, top_k, n_out] f32.
 * Errors (not faults): k != stack k, t_ids != t, x_per_row not in {1, top_k},
 * k % 256 != 0, top_k > 65535. An id >= n_expert yields a zero row (this op has no
 * workspace and therefore no device flag; the whole-block entries record one). */
lmoe_status lmoe_mul_mv_id(const lmoe_expert_stack *stack, const float *x, int64_t t, int64_t x_per_row,
                           int64_t k, const uint32_t *ids, int64_t t_ids, int64_t top_k, float *out,
                           void *stream);

/* `ops::mul_mv`, src/ops/mv_id.rs:54-56 -> `run_plain_mv`,
 * src/ops/dispatch.rs:964-1057: plain quantized mat-vec (the lm_head bypass).
 *   weight: raw [n_out, k/256] super-blocks on the device, x [t, k] -> out [t, n_out]. */
lmoe_status lmoe_mul_mv(const void *weight, int32_t dtype, int64_t n_out, int64_t k, const float *x,
                        int64_t t, float *out, void *stream);

/* ------------------------------------------------------ grouped GEMM path --
 * `Map0Scratch`, src/ops/dispatch.rs:547-549, 752-757: `tpe` (n_expert u32 at
 * byte 0) followed by `ids_map` (n_expert * t i32 at byte n_expert*4): for each
 * expert the flat `token*top_k + slot` ids routed to it, tokens ascending. */
size_t lmoe_map0_scratch_bytes(int64_t n_expert, int64_t t);
/* `ops::mm_id::prepare_map0`, src/ops/mm_id.rs:27-29 -> `prepare_mm_id_map0`,
 * src/ops/dispatch.rs:927-956 -> kernel_mul_mm_id_map0, src/ops/mm_id.metal:207-269.
 * Experts must be distinct within a token (src/ops/dispatch.rs:2341-2346). */
lmoe_status lmoe_prepare_map0(const uint32_t *ids, int64_t t, int64_t top_k, int64_t n_expert,
                              void *scratch, size_t scratch_bytes, void *stream);
/* `ops::mm_id::supported`, src/ops/mm_id.rs:48-50. Returns 1 or 0. */
int32_t lmoe_mm_id_supported(int32_t dtype, int64_t top_k);
/* Workspace of one grouped-GEMM projection over `stack` (staged f16 activations,
 * tile list, device flag). */
size_t lmoe_mm_id_workspace_bytes(const lmoe_expert_stack *stack, int64_t t, int64_t top_k, int64_t x_per_row);
/* `ops::mm_id::mul_mm_id_shared`, src/ops/mm_id.rs:32-39 -> `run_mm_shared`,
 * src/ops/dispatch.rs:789-797 -> kernel_mul_mm_id_q{4,6}_K_f32_t,
 * src/ops/mm_id.metal:492-647.  Same shapes and errors as lmoe_mul_mv_id.  The
 * scratch geometry (`map_n_expert`, `map_t`, `map_top_k`: what prepare_map0 was
 * called with) is re-validated against this projection, src/ops/dispatch.rs:903-909.
 * Operands are staged as f16 tiles with f32 accumulation, like the reference's
 * default variant (`MmVariant::Tensor`, src/ops/mod.rs:205-215). */
lmoe_status lmoe_mul_mm_id_shared(const lmoe_expert_stack *stack, const float *x, int64_t t,
                                  int64_t x_per_row, int64_t k, const uint32_t *ids, int64_t t_ids,
                                  int64_t top_k, const void *map0_scratch, int64_t map_n_expert,
                                  int64_t map_t, int64_t map_top_k, float *out, void *workspace,
                                  size_t workspace_bytes, void *stream);
/* `ops::mm_id::mul_mm_id`, src/ops/mm_id.rs:16-18: self-contained (runs its own
 * map0 pass). Workspace: lmoe_mm_id_workspace_bytes(...) + lmoe_map0_scratch_bytes(n_expert, t). */
lmoe_status lmoe_mul_mm_id(const lmoe_expert_stack *stack, const float *x, int64_t t, int64_t x_per_row,
                           int64_t k, const uint32_t *ids, int64_t t_ids, int64_t top_k, float *out,
                           void *workspace, size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------- glue --
 * `ops::silu_mul`, src/ops/silu_mul.rs:14 -> kernel_moe_silu_mul,
 * src/ops/silu_mul.metal:57-72: out[i] = (g / (1 + exp(-g))) * u, the two
 * roundings kept separate. n <= INT32_MAX. */
lmoe_status lmoe_silu_mul(const float *gate, const float *up, int64_t n, float *out, void *stream);
/* `ops::combine`, src/ops/combine.rs:16 -> `run_combine`, src/ops/dispatch.rs:1366-1506
 * -> kernel_moe_combine{,_rescale}, src/ops/combine.metal:70-133:
 *   out[s, c] = sum_k down[s, k, c] * (col_l2[s, k] * 2^-15) * w[s, k]
 * (col_l2 may be NULL: plain weighted sum). Fixed summation order: k strided
 * over next_pow2(top_k/2) lanes, lanes folded by a butterfly. Errors:
 * next_pow2(top_k/2) > 32; seq*top_k*n_out > INT32_MAX (src/ops/dispatch.rs:294-305). */
lmoe_status lmoe_combine(const float *down, const float *col_l2, const float *weights, int64_t seq,
                         int64_t top_k, int64_t n_out, float *out, void *stream);

/* ------------------------------------------------------------ whole block --
 * `MoeBlock`, src/moe.rs:28-79, with `FusedExperts` (src/moe.rs:194-324) and
 * `SharedExpert` (src/moe.rs:327-345) behind it.  The layer borrows the stacks
 * and the router/bias device buffers; they must outlive it. Shared stacks are
 * `[1, n_out, k]` stacks or all NULL (no shared expert). */
typedef struct lmoe_layer lmoe_layer;

lmoe_status lmoe_layer_create(int64_t hidden, int64_t expert_ff, int64_t n_expert, int64_t top_k,
                              float scale, int32_t norm, const float *router, const float *bias,
                              const lmoe_expert_stack *gate, const lmoe_expert_stack *up,
                              const lmoe_expert_stack *down, const lmoe_expert_stack *shared_gate,
                              const lmoe_expert_stack *shared_up, const lmoe_expert_stack *shared_down,
                              lmoe_layer **out);
void lmoe_layer_destroy(lmoe_layer *layer);

/* Bytes of scratch `lmoe_moe_forward*` needs for up to `max_tokens` tokens. */
size_t lmoe_layer_workspace_bytes(const lmoe_layer *layer, int64_t max_tokens);

/* `MoeBlock::forward` on the decode path (t < LMOE_MM_ID_MIN_SEQ in the
 * reference; any t here: LMOE_DECODE_MAX_SEQ tokens per launch), src/moe.rs:73-78 with the mv_id branch of
 * src/moe.rs:221-323 fused: route, stream each DISTINCT selected expert and the
 * shared expert once, SwiGLU and the weighted combine in the same kernels.
 *   x [t, hidden] f32 -> out [t, hidden] f32; ids_out [t, top_k] / weights_out
 * [t, top_k] receive the routing decision when non-NULL.
 * The workspace needs no initialisation.  The kernel's CTAs synchronise through
 * device words owned by `layer`: at most one decode call in flight per layer
 * handle (create a second handle over the same stacks for a second stream).  A call
 * on another stream while the previous one is still running fails with LMOE_ERR_INVALID. */
lmoe_status lmoe_moe_forward_decode(const lmoe_layer *layer, const float *x, int64_t t, float *out,
                                    uint32_t *ids_out, float *weights_out, void *workspace,
                                    size_t workspace_bytes, void *stream);

/* `ExpertFfn::forward`, src/moe.rs:19-21 (the seam `FusedExperts`, src/moe.rs:194-324, implements and
 * `MoeBlock::forward` calls after routing, src/moe.rs:73-78): the routed experts on a routing decision the
 * CALLER made.
 *   x [t, hidden] f32, ids [t, top_k] u32, weights [t, top_k] f32 (top_k = the layer's), all on the device
 *   -> out [t, hidden] f32 = sum over slots, in slot order, of weights[t,k] * FFN_{ids[t,k]}(x[t]);
 *   add_shared != 0 adds the layer's shared expert (src/moe.rs:76-77), 0 is the bare trait.
 * An id >= the layer's expert count is an empty slot (contributes nothing).  Below lmoe_mm_id_min_seq()
 * tokens the fused mat-vec kernel runs with its routing phase skipped and accepts the same expert more
 * than once in a row (src/ops/mv_id.rs:100-203); from there on the grouped GEMM runs, which, like the
 * reference's (src/ops/dispatch.rs:2341-2346), needs the experts of a token to be distinct.
 * The one-call-in-flight rule of lmoe_moe_forward_decode applies on the mat-vec path.
 * Workspace: lmoe_experts_workspace_bytes(layer, t); needs no initialisation. */
size_t lmoe_experts_workspace_bytes(const lmoe_layer *layer, int64_t max_tokens);
lmoe_status lmoe_experts_forward(const lmoe_layer *layer, const float *x, const uint32_t *ids, const float *weights,
                                 int64_t t, int32_t add_shared, float *out, void *workspace, size_t workspace_bytes,
                                 void *stream);

/* The same for one rank of an expert-parallel decode step (no counterpart in the single-GPU reference): x / ids
 * / weights cover ALL tokens of the batch, with the slots of experts that live on other ranks set empty; the
 * replicated shared expert is added only for the tokens [shared_first, shared_first + shared_count), this
 * rank's own.  out [t, hidden] holds this rank's partial rows; the ranks' rows of a token are summed by its
 * owner.  A partial shared range needs t < lmoe_mm_id_min_seq(). */
lmoe_status lmoe_experts_forward_ep(const lmoe_layer *layer, const float *x, const uint32_t *ids, const float *weights,
                                    int64_t t, int64_t shared_first, int64_t shared_count, float *out, void *workspace,
                                    size_t workspace_bytes, void *stream);

/* `MoeBlock::forward` on the prefill path (the mm_id branch of src/moe.rs:236-323):
 * route, sort token-slots by expert, grouped GEMM on tensor cores with f16
 * operand tiles dequantized in shared memory and f32 accumulation, SwiGLU in
 * the gate/up epilogue, routing weight in the down epilogue, fixed-order
 * combine plus the shared expert. */
lmoe_status lmoe_moe_forward_prefill(const lmoe_layer *layer, const float *x, int64_t t, float *out,
                                     uint32_t *ids_out, float *weights_out, void *workspace,
                                     size_t workspace_bytes, void *stream);

/* `MoeBlock::forward` with HOST buffers: copies x to the device, runs the decode
 * or prefill path (t >= lmoe_mm_id_min_seq() -> prefill; the reference's own switch, src/moe.rs:236-240, is at 32),
 * copies the result back and synchronises the stream. `x_host` / `out_host`
 * should be pinned for full copy bandwidth; on the decode path a pinned, device-mapped `out_host` is written by
 * the kernel itself (no device-to-host copy), pageable memory goes through a copy. */
lmoe_status lmoe_moe_forward_host(const lmoe_layer *layer, const float *x_host, int64_t t, float *out_host,
                                  uint32_t *ids_out_host, float *weights_out_host, void *workspace,
                                  size_t workspace_bytes, void *stream);

/* The same without the final synchronisation, like every other entry of this header (the reference's ops return
 * before the GPU has run them, src/ops/dispatch.rs `run_inner`): the copies and the kernels are enqueued on `stream`
 * and the call returns; `out_host` holds the result once the stream has been synchronised.  Calls that share a
 * workspace must share the stream.  Both buffers must be pinned for the copies to be asynchronous.  With both
 * pinned, a decode call's input is copied on a stream of the layer's own (into staging buffers of the layer), so
 * that the copy runs beside the previous call's kernel: x_host is read without regard to earlier work on `stream`
 * and must be complete when the call is made.  Not for use inside a stream capture (host addresses). */
lmoe_status lmoe_moe_forward_host_async(const lmoe_layer *layer, const float *x_host, int64_t t, float *out_host,
                                  uint32_t *ids_out_host, float *weights_out_host, void *workspace,
                                  size_t workspace_bytes, void *stream);

/* The FFN half of a transformer layer around the block, src/model.rs:340-350:
 *   ffn_normed = rms_norm(ffn_inp) * norm_weight;  out = ffn_inp + MoeBlock::forward(ffn_normed).
 * rms_norm is candle's `RmsNorm` (x * 1/sqrt(mean(x^2) + eps) * weight, f32); its sum of squares runs in
 * the same fixed order as the router logits (128 fmaf chains, lane fold, warp butterfly), so the expert
 * selection downstream is reproducible.  ffn_inp / out [t, hidden] f32 (out must not alias ffn_inp),
 * norm_weight [hidden] f32; ids_out / weights_out as in lmoe_moe_forward_*; t < lmoe_mm_id_min_seq() runs the
 * decode kernel, larger t the grouped-GEMM path.  Workspace: lmoe_moe_layer_workspace_bytes(layer, t). */
lmoe_status lmoe_rms_norm(const float *x, const float *weight, float eps, int64_t t, int64_t hidden,
                          float *out, void *stream);
size_t lmoe_moe_layer_workspace_bytes(const lmoe_layer *layer, int64_t max_tokens);
lmoe_status lmoe_moe_layer_forward(const lmoe_layer *layer, const float *ffn_inp, const float *norm_weight,
                                   float eps, int64_t t, float *out, uint32_t *ids_out, float *weights_out,
                                   void *workspace, size_t workspace_bytes, void *stream);

/* Expert-parallel pieces (experts [first, first + n_local) of the layer are
 * resident on this GPU; the reference has no multi-GPU path, this is new):
 * run the routed experts of pre-routed, pre-dispatched rows.
 *   x [rows, hidden] f32, local_ids [rows] u32 (expert id relative to the
 *   layer's first expert), row_weights [rows] f32 -> out [rows, hidden] f32
 *   = row_weights[r] * FFN_{local_ids[r]}(x[r]). */
lmoe_status lmoe_experts_forward_rows(const lmoe_layer *layer, const float *x, const uint32_t *local_ids,
                                      const float *row_weights, int64_t rows, float *out, void *workspace,
                                      size_t workspace_bytes, void *stream);
/* The same with x [rows, hidden] in IEEE half precision (16-byte aligned): the wire format of the token
 * dispatch.  The grouped GEMM rounds its activation operand to half anyway, so results are identical to
 * passing the same values as f32. */
lmoe_status lmoe_experts_forward_rows_f16(const lmoe_layer *layer, const void *x_f16, const uint32_t *local_ids,
                                          const float *row_weights, int64_t rows, float *out, void *workspace,
                                          size_t workspace_bytes, void *stream);
/* Token-level form of the same: one half-precision activation row per token and up to top_k local experts
 * for it.  x_f16 [t, hidden], ids / weights [t, top_k]; a slot whose id is >= the layer's expert count is
 * empty.  out [t, hidden] f32 = sum over the non-empty slots, in slot order, of weights * FFN_{ids}(x[token]).
 * A token travels to a rank once, however many of its experts live there, and one summed row comes back.
 * Needs the fused Q4_K gate/up and Q6_K down kernels (LMOE_ERR_UNSUPPORTED otherwise).
 * Workspace: lmoe_tokens_workspace_bytes(layer, t, top_k). */
size_t lmoe_tokens_workspace_bytes(const lmoe_layer *layer, int64_t t, int64_t top_k);
lmoe_status lmoe_experts_forward_tokens_f16(const lmoe_layer *layer, const void *x_f16, const uint32_t *ids,
                                            const float *weights, int64_t t, int64_t top_k, float *out,
                                            void *workspace, size_t workspace_bytes, void *stream);
/* Token dispatch of the expert-parallel path, packed on the device: rank r owns experts
 * [r * n_expert / world, (r + 1) * n_expert / world).  From x [t, hidden] f32 and the routing decision
 * ids / weights [t, top_k], writes the t * top_k routed rows grouped by destination rank (by expert inside a
 * rank): rows_f16 [t*top_k, hidden] half, local_ids [t*top_k] (expert id relative to the destination's first
 * expert), row_weights [t*top_k], row_pos [t*top_k] = position of flat id (token * top_k + slot) in that order,
 * and send_counts [world] (int64, device).  Workspace: lmoe_ep_pack_workspace_bytes(n_expert, t). */
size_t lmoe_ep_pack_workspace_bytes(int64_t n_expert, int64_t t);
lmoe_status lmoe_ep_pack(const float *x, const uint32_t *ids, const float *weights, int64_t t, int64_t hidden,
                         int64_t top_k, int64_t n_expert, int64_t world, void *rows_f16, uint32_t *local_ids,
                         float *row_weights, int32_t *row_pos, int64_t *send_counts, void *workspace,
                         size_t workspace_bytes, void *stream);
/* Expert ids of the whole block -> ids relative to the experts [first, first + count) of one rank; every other
 * id becomes the empty-slot id `count` (what lmoe_experts_forward{,_ep,_tokens_f16} skip).  n = number of ids. */
lmoe_status lmoe_ep_localize_ids(const uint32_t *ids, int64_t n, int64_t first, int64_t count, uint32_t *out, void *stream);
/* The return leg: out [t, hidden] = sum over slots, in slot order, of rows[row_pos[token * top_k + slot]]
 * (the weighted expert outputs, back in the order they were sent), then + shared [t, hidden] when non-NULL.
 * A negative row_pos entry is skipped (with the token-level dispatch: top_k = ranks, one slot per rank). */
lmoe_status lmoe_ep_combine(const float *rows, const int32_t *row_pos, const float *shared, int64_t t,
                            int64_t top_k, int64_t hidden, float *out, void *stream);
/* Bytes of scratch `lmoe_experts_forward_rows` / `lmoe_shared_forward` need for `rows` rows. */
size_t lmoe_rows_workspace_bytes(const lmoe_layer *layer, int64_t rows);
/* The shared expert alone: out [t, hidden] = FFN_shared(x [t, hidden]). */
lmoe_status lmoe_shared_forward(const lmoe_layer *layer, const float *x, int64_t t, float *out,
                                void *workspace, size_t workspace_bytes, void *stream);

/* Reads (and clears) the device error word kept in the first bytes of a
 * workspace after the stream has been synchronised by the caller: 0 = clean.
 * Non-zero: LMOE_ERR_DEVICE_FLAG with the cause in lmoe_last_error(). */
lmoe_status lmoe_check_device_flag(void *workspace, void *stream);

/* ---- exchanges of an expert-parallel decode step over peer memory (no counterpart in the reference: one GPU) ----
 * One process per GPU.  Every rank allocates a receive buffer and a control block with lmoe_peer_alloc, sends the
 * 64-byte handles to the other ranks by whatever channel the host has, and maps theirs with lmoe_peer_open.
 * lmoe_peer_put stores this rank's rows into slot `rank` of the other ranks' buffers and raises its flag there;
 * lmoe_peer_wait holds the stream until the flags of all ranks have arrived (bounded: a time-out sets word 40 of the
 * control block, bit 0x2 plus one bit per missing rank, and the stream goes on).  direction 0 / 1: two independent
 * exchanges (gather, return) share one control block.  All ranks must issue the same sequence of puts. */
lmoe_status lmoe_peer_alloc(size_t bytes, void **ptr, void *handle64);   /* zero-filled; handle64: 64 bytes out */
lmoe_status lmoe_peer_open(const void *handle64, void **ptr);
lmoe_status lmoe_peer_close(void *ptr);
lmoe_status lmoe_peer_free(void *ptr);
size_t lmoe_peer_ctrl_bytes(void);
/* src: `world` chunks of chunk_bytes (per_rank_src = 1: chunk s goes to rank s, an all-to-all) or one chunk that goes to
 * every rank (per_rank_src = 0, an all-gather).  peer_bufs[s] / peer_flags[s]: rank s's receive buffer and control block
 * as mapped in this process (entry `rank`: this rank's own).  chunk_bytes a multiple of 16. */
lmoe_status lmoe_peer_put(const void *src, int64_t chunk_bytes, int32_t world, int32_t rank, int32_t per_rank_src,
                          void *const *peer_bufs, void *const *peer_flags, void *local_ctrl, int32_t direction,
                          void *stream);
lmoe_status lmoe_peer_wait(void *local_ctrl, int32_t world, int32_t direction, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LMOE_H */
