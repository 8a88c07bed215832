// Shared declarations of the sm_100a MoE library: error plumbing, handle
// structs, launch prototypes of every kernel file.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/lmoe.h"

#define QK_K 256
#define Q4K_BYTES 144
#define Q6K_BYTES 210

// ---- error plumbing (thread-local message, status code) --------------------
lmoe_status lmoe_fail(lmoe_status code, const char *fmt, ...);
void lmoe_clear_error();

#define LMOE_CUDA(expr)                                                                            \
    do {                                                                                           \
        cudaError_t e__ = (expr);                                                                  \
        if (e__ != cudaSuccess)                                                                    \
            return lmoe_fail(LMOE_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));      \
    } while (0)

#define LMOE_LAUNCH_CHECK(name)                                                                    \
    do {                                                                                           \
        cudaError_t e__ = cudaGetLastError();                                                      \
        if (e__ != cudaSuccess)                                                                    \
            return lmoe_fail(LMOE_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

// ---- handles ----------------------------------------------------------------
struct lmoe_expert_stack {
    int32_t dtype;
    int64_t n_expert, n_out, k;
    const uint8_t *base; // device allocation (or caller's buffer for wrapped stacks)
    size_t base_off;     // first super-block = base + base_off
    size_t nbytes;       // bytes of super-blocks
    bool owned;
    int device;
    const uint8_t *blocks() const { return base + base_off; }
    int type_size() const { return dtype == LMOE_Q4_K ? Q4K_BYTES : Q6K_BYTES; }
    int64_t row_bytes() const { return k / QK_K * type_size(); }
    int64_t expert_bytes() const { return n_out * row_bytes(); }
};

struct lmoe_layer {
    int64_t hidden, expert_ff, n_expert, top_k;
    float scale;
    int32_t norm;
    const float *router, *bias;
    const lmoe_expert_stack *gate, *up, *down, *sh_gate, *sh_up, *sh_down;
    // device words the fused decode kernel synchronises its CTAs through; zero between launches,
    // so one decode call at a time per layer
    uint32_t *sync;
    // guard of that rule: the stream and completion event of the latest decode call.  A call on a
    // different stream while the event is still pending is refused instead of corrupting `sync`.
    mutable std::mutex dec_mutex;
    mutable cudaEvent_t dec_event = nullptr;
    mutable cudaStream_t dec_stream = nullptr;
    mutable bool dec_pending = false;
    // Host-buffer decode calls: two device staging rows-buffers, filled by a copy stream of the layer's own, so that
    // the host-to-device copy of a call runs while the previous call's kernel does (created at the first such call).
    mutable std::mutex host_mutex;
    mutable float *host_x[2] = {nullptr, nullptr};
    mutable cudaStream_t host_copy_stream = nullptr;
    mutable cudaEvent_t host_copied[2] = {nullptr, nullptr}, host_slot_free[2] = {nullptr, nullptr};
    mutable int host_slot = 0;
    mutable bool host_failed = false;
};

static inline int lmoe_type_size(int32_t dtype) {
    return dtype == LMOE_Q4_K ? Q4K_BYTES : dtype == LMOE_Q6_K ? Q6K_BYTES : 0;
}

static inline size_t lmoe_align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- kernel launchers (one per .cu file) -----------------------------------
// route.cu
cudaError_t launch_route_logits(const float *router, const float *x, int t, int hidden, int n_expert,
                                float *logits, cudaStream_t s);
cudaError_t launch_route_select(const float *logits, const float *bias, int t, int n_expert, int top_k,
                                float scale, int norm, uint32_t *ids, float *weights, cudaStream_t s);
// mv_id.cu
// Streamed Q6_K mat-vec (mv_stream.cu): rows [0, n_out - n_out % 16) of one activation row.
bool mv_q6k_stream_available(int64_t n_out, int64_t k);
cudaError_t launch_mv_q6k_stream(const uint8_t *w, int n_out, int k, const float *x, float *out, cudaStream_t s);
cudaError_t launch_mul_mv_id(int dtype, const uint8_t *w, int64_t expert_bytes, int n_expert, int n_out, int k,
                             const float *x, int t, int x_per_row, const uint32_t *ids, int top_k, float *out,
                             cudaStream_t s);
// glue.cu
cudaError_t launch_silu_mul(const float *g, const float *u, int64_t n, float *out, cudaStream_t s);
cudaError_t launch_combine(const float *down, const float *col_l2, const float *w, int seq, int top_k,
                           int n_out, float *out, cudaStream_t s);
cudaError_t launch_add_inplace(float *out, const float *b, int64_t n, cudaStream_t s);
cudaError_t launch_ep_localize_ids(const uint32_t *ids, int64_t n, uint32_t first, uint32_t count, uint32_t *out,
                                   cudaStream_t s);
cudaError_t launch_rms_norm(const float *x, const float *w, float eps, int64_t t, int hidden, float *out, cudaStream_t s);
cudaError_t launch_map0(const uint32_t *ids, int t, int top_k, int n_expert, uint32_t *tpe, int32_t *ids_map,
                        cudaStream_t s);
// codec.cu
cudaError_t launch_quantize(int dtype, const float *src, int64_t nblocks, uint8_t *dst, cudaStream_t s);
cudaError_t launch_dequantize(int dtype, const uint8_t *src, int64_t nblocks, float *dst, cudaStream_t s);
