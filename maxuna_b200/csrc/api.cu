// C ABI: argument validation (every check of the reference's `run_inner`,
// src/ops/dispatch.rs:812-847, `prepare_mm_id_map0` :927-939 and `run_combine`
// :1366-1420 comes back as an error code, never a GPU fault), handles, and the
// glue between entry points and kernel launchers.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <new>

#include "common.cuh"

size_t decode_sync_bytes(); // decode.cu
#include "fused.cuh"

// ---------------------------------------------------------------- errors ----
static thread_local char g_err[512] = "";

lmoe_status lmoe_fail(lmoe_status code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

void lmoe_clear_error() { g_err[0] = 0; }

extern "C" const char *lmoe_last_error(void) { return g_err; }
extern "C" const char *lmoe_version(void) { return "lmoe 0.1 (sm_100a)"; }

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define REQUIRE(cond, ...)                                                                         \
    do {                                                                                           \
        if (!(cond)) return lmoe_fail(LMOE_ERR_INVALID, __VA_ARGS__);                              \
    } while (0)

// ----------------------------------------------------------------- stack ----
static lmoe_status stack_check(int32_t dtype, int64_t n_expert, int64_t n_out, int64_t k, size_t nbytes,
                               size_t base_off) {
    const int ts = lmoe_type_size(dtype);
    REQUIRE(ts != 0, "unsupported expert dtype %d (Q4_K=12 and Q6_K=14 are built)", dtype);
    REQUIRE(n_expert > 0 && n_out > 0 && k > 0, "expert stack dims must be positive, got [%lld, %lld, %lld]",
            (long long)n_expert, (long long)n_out, (long long)k);
    REQUIRE(k % QK_K == 0, "expert stack k (%lld) is not a multiple of the block size %d", (long long)k, QK_K);
    REQUIRE(n_expert <= INT32_MAX && n_out <= INT32_MAX && k <= INT32_MAX, "expert stack dims exceed int32");
    const size_t want = (size_t)n_expert * (size_t)n_out * (size_t)(k / QK_K) * (size_t)ts;
    REQUIRE(nbytes == want, "expert stack byte size %zu does not match [%lld, %lld, %lld] (%zu bytes)", nbytes,
            (long long)n_expert, (long long)n_out, (long long)k, want);
    REQUIRE(base_off % 16 == 0, "base_off (%zu) must be a multiple of 16", base_off);
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_expert_stack_create(int32_t dtype, int64_t n_expert, int64_t n_out, int64_t k,
                                                const void *bytes_host, size_t nbytes, size_t base_off,
                                                lmoe_expert_stack **out) {
    lmoe_clear_error();
    REQUIRE(out != nullptr, "out handle pointer is NULL");
    *out = nullptr;
    lmoe_status st = stack_check(dtype, n_expert, n_out, k, nbytes, base_off);
    if (st) return st;
    REQUIRE(bytes_host != nullptr, "bytes_host is NULL");
    int dev = 0;
    LMOE_CUDA(cudaGetDevice(&dev));
    uint8_t *buf = nullptr;
    // 128 spare bytes: the decode kernel moves whole 16-byte pieces and may touch the tail
    LMOE_CUDA(cudaMalloc(&buf, base_off + nbytes + 128));
    cudaError_t e = cudaMemcpy(buf + base_off, bytes_host, nbytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(buf);
        return lmoe_fail(LMOE_ERR_CUDA, "expert stack upload failed: %s", cudaGetErrorString(e));
    }
    cudaMemset(buf + base_off + nbytes, 0, 128);
    *out = new (std::nothrow) lmoe_expert_stack{dtype, n_expert, n_out, k, buf, base_off, nbytes, true, dev};
    if (!*out) {
        cudaFree(buf);
        return lmoe_fail(LMOE_ERR_INVALID, "out of host memory");
    }
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_expert_stack_wrap(int32_t dtype, int64_t n_expert, int64_t n_out, int64_t k,
                                              const void *device_base, size_t nbytes, size_t base_off,
                                              lmoe_expert_stack **out) {
    lmoe_clear_error();
    REQUIRE(out != nullptr, "out handle pointer is NULL");
    *out = nullptr;
    lmoe_status st = stack_check(dtype, n_expert, n_out, k, nbytes, base_off);
    if (st) return st;
    REQUIRE(device_base != nullptr, "device_base is NULL");
    REQUIRE(aligned16(static_cast<const uint8_t *>(device_base) + base_off),
            "first super-block (device_base + base_off) must be 16-byte aligned");
    int dev = 0;
    cudaGetDevice(&dev);
    *out = new (std::nothrow) lmoe_expert_stack{dtype, n_expert, n_out, k, static_cast<const uint8_t *>(device_base),
                                                base_off, nbytes, false, dev};
    REQUIRE(*out != nullptr, "out of host memory");
    return LMOE_OK;
}

extern "C" void lmoe_expert_stack_destroy(lmoe_expert_stack *stack) {
    if (!stack) return;
    if (stack->owned) cudaFree(const_cast<uint8_t *>(stack->base));
    delete stack;
}

extern "C" const void *lmoe_expert_stack_device_ptr(const lmoe_expert_stack *stack) {
    return stack ? stack->blocks() : nullptr;
}

extern "C" lmoe_status lmoe_expert_stack_info(const lmoe_expert_stack *stack, int32_t *dtype, int64_t *n_expert,
                                              int64_t *n_out, int64_t *k, size_t *nbytes) {
    lmoe_clear_error();
    REQUIRE(stack != nullptr, "stack is NULL");
    if (dtype) *dtype = stack->dtype;
    if (n_expert) *n_expert = stack->n_expert;
    if (n_out) *n_out = stack->n_out;
    if (k) *k = stack->k;
    if (nbytes) *nbytes = stack->nbytes;
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_quantize(int32_t dtype, const float *src, int64_t nblocks, void *dst, void *stream) {
    lmoe_clear_error();
    REQUIRE(lmoe_type_size(dtype) != 0, "unsupported dtype %d", dtype);
    REQUIRE(nblocks >= 0, "nblocks must be >= 0");
    REQUIRE(src && dst, "src/dst is NULL");
    REQUIRE(aligned16(src), "src must be 16-byte aligned");
    LMOE_CUDA(launch_quantize(dtype, src, nblocks, static_cast<uint8_t *>(dst), (cudaStream_t)stream));
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_dequantize(int32_t dtype, const void *src, int64_t nblocks, float *dst, void *stream) {
    lmoe_clear_error();
    REQUIRE(lmoe_type_size(dtype) != 0, "unsupported dtype %d", dtype);
    REQUIRE(nblocks >= 0, "nblocks must be >= 0");
    REQUIRE(src && dst, "src/dst is NULL");
    REQUIRE((reinterpret_cast<uintptr_t>(src) & 1u) == 0, "src must be 2-byte aligned");
    LMOE_CUDA(launch_dequantize(dtype, static_cast<const uint8_t *>(src), nblocks, dst, (cudaStream_t)stream));
    return LMOE_OK;
}

// --------------------------------------------------------------- routing ----
static lmoe_status route_check(int64_t t, int64_t n_expert, int64_t top_k) {
    REQUIRE(t >= 0 && t <= (1 << 24), "t (%lld) out of range", (long long)t);
    REQUIRE(n_expert >= 1 && n_expert <= 512, "n_expert (%lld) must be in [1, 512]", (long long)n_expert);
    REQUIRE(top_k >= 1 && top_k <= 32 && top_k <= n_expert, "top_k (%lld) must be in [1, min(32, n_expert)]",
            (long long)top_k);
    return LMOE_OK;
}

extern "C" size_t lmoe_route_workspace_bytes(int64_t t, int64_t n_expert) {
    if (t < 0 || n_expert < 0) return 0;
    return lmoe_align_up((size_t)t * (size_t)n_expert * sizeof(float), 256);
}

extern "C" lmoe_status lmoe_route_from_logits(const float *logits, const float *bias, int64_t t, int64_t n_expert,
                                              int64_t top_k, float scale, int32_t norm, uint32_t *ids_out,
                                              float *weights_out, void *stream) {
    lmoe_clear_error();
    lmoe_status st = route_check(t, n_expert, top_k);
    if (st) return st;
    REQUIRE(logits && ids_out && weights_out, "logits/ids_out/weights_out is NULL");
    LMOE_CUDA(launch_route_select(logits, bias, (int)t, (int)n_expert, (int)top_k, scale, norm, ids_out, weights_out,
                                  (cudaStream_t)stream));
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_route(const float *router, const float *bias, const float *x, int64_t t, int64_t hidden,
                                  int64_t n_expert, int64_t top_k, float scale, int32_t norm, uint32_t *ids_out,
                                  float *weights_out, void *workspace, size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    lmoe_status st = route_check(t, n_expert, top_k);
    if (st) return st;
    REQUIRE(hidden >= 1 && hidden <= (1 << 20), "hidden (%lld) out of range", (long long)hidden);
    REQUIRE(router && x && ids_out && weights_out, "router/x/ids_out/weights_out is NULL");
    if (hidden % 4 == 0) REQUIRE(aligned16(router) && aligned16(x), "router and x must be 16-byte aligned");
    if (workspace_bytes < lmoe_route_workspace_bytes(t, n_expert) || (t > 0 && !workspace))
        return lmoe_fail(LMOE_ERR_WORKSPACE, "route workspace needs %zu bytes, got %zu",
                         lmoe_route_workspace_bytes(t, n_expert), workspace_bytes);
    float *logits = static_cast<float *>(workspace);
    LMOE_CUDA(launch_route_logits(router, x, (int)t, (int)hidden, (int)n_expert, logits, (cudaStream_t)stream));
    LMOE_CUDA(launch_route_select(logits, bias, (int)t, (int)n_expert, (int)top_k, scale, norm, ids_out, weights_out,
                                  (cudaStream_t)stream));
    return LMOE_OK;
}

// ------------------------------------------------------- indexed mat-vec ----
// The seam checks of `run_inner`, src/ops/dispatch.rs:812-847.
lmoe_status lmoe_id_shape_check(const lmoe_expert_stack *stack, const void *x, int64_t t, int64_t x_per_row,
                                int64_t k, const void *ids, int64_t t_ids, int64_t top_k, const void *out) {
    REQUIRE(stack != nullptr, "expert stack is NULL");
    REQUIRE(x && ids && out, "x/ids/out is NULL");
    REQUIRE(t >= 0 && top_k >= 1 && top_k <= 65535, "t must be >= 0 and top_k in [1, 65535]");
    REQUIRE(k == stack->k, "x k (%lld) does not match expert stack k (%lld)", (long long)k, (long long)stack->k);
    REQUIRE(t_ids == t, "ids t (%lld) does not match x t (%lld)", (long long)t_ids, (long long)t);
    REQUIRE(x_per_row == 1 || x_per_row == top_k,
            "x_per_row (%lld) must be 1 (shared row) or top_k (%lld) (per-slot row)", (long long)x_per_row,
            (long long)top_k);
    REQUIRE(stack->k % QK_K == 0, "expert stack k (%lld) is not a multiple of the block size %d",
            (long long)stack->k, QK_K);
    REQUIRE(t * top_k <= INT32_MAX && t * top_k * stack->n_out <= ((int64_t)1 << 40), "problem too large");
    REQUIRE(aligned16(x), "x must be 16-byte aligned");
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_mul_mv_id(const lmoe_expert_stack *stack, const float *x, int64_t t, int64_t x_per_row,
                                      int64_t k, const uint32_t *ids, int64_t t_ids, int64_t top_k, float *out,
                                      void *stream) {
    lmoe_clear_error();
    lmoe_status st = lmoe_id_shape_check(stack, x, t, x_per_row, k, ids, t_ids, top_k, out);
    if (st) return st;
    LMOE_CUDA(launch_mul_mv_id(stack->dtype, stack->blocks(), stack->expert_bytes(), (int)stack->n_expert,
                               (int)stack->n_out, (int)stack->k, x, (int)t, (int)x_per_row, ids, (int)top_k, out,
                               (cudaStream_t)stream));
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_mul_mv(const void *weight, int32_t dtype, int64_t n_out, int64_t k, const float *x,
                                   int64_t t, float *out, void *stream) {
    lmoe_clear_error();
    const int ts = lmoe_type_size(dtype);
    REQUIRE(ts != 0, "unsupported dtype %d", dtype);
    REQUIRE(weight && x && out, "weight/x/out is NULL");
    REQUIRE(n_out >= 1 && n_out <= INT32_MAX && t >= 0 && t <= INT32_MAX, "n_out/t out of range");
    REQUIRE(k > 0 && k % QK_K == 0 && k <= INT32_MAX, "k (%lld) is not a positive multiple of %d", (long long)k, QK_K);
    REQUIRE(aligned16(weight) && aligned16(x), "weight and x must be 16-byte aligned");
    const uint8_t *wb = static_cast<const uint8_t *>(weight);
    if (dtype == LMOE_Q6_K && t >= 1 && t <= 4 && n_out >= 4096 && mv_q6k_stream_available(n_out, k)) {
        // the vocabulary projection of a decode step: every weight byte is read once per token, through the
        // streamed kernel; the rows past the last whole 16-row chunk go to the row-per-warp kernel below
        const int64_t body = n_out / 16 * 16, row_bytes = (k / QK_K) * ts;
        for (int64_t i = 0; i < t; i++) {
            LMOE_CUDA(launch_mv_q6k_stream(wb, (int)n_out, (int)k, x + i * k, out + i * n_out, (cudaStream_t)stream));
            if (body < n_out)
                LMOE_CUDA(launch_mul_mv_id(dtype, wb + body * row_bytes, (n_out - body) * row_bytes, 1, (int)(n_out - body),
                                           (int)k, x + i * k, 1, 1, nullptr, 1, out + i * n_out + body, (cudaStream_t)stream));
        }
        return LMOE_OK;
    }
    LMOE_CUDA(launch_mul_mv_id(dtype, wb, n_out * (k / QK_K) * ts, 1, (int)n_out,
                               (int)k, x, (int)t, 1, nullptr, 1, out, (cudaStream_t)stream));
    return LMOE_OK;
}

// ------------------------------------------------------------------ glue ----
extern "C" lmoe_status lmoe_silu_mul(const float *gate, const float *up, int64_t n, float *out, void *stream) {
    lmoe_clear_error();
    REQUIRE(gate && up && out, "gate/up/out is NULL");
    REQUIRE(n >= 0 && n <= INT32_MAX, "silu_mul n (%lld) must be in [0, i32::MAX]", (long long)n);
    LMOE_CUDA(launch_silu_mul(gate, up, n, out, (cudaStream_t)stream));
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_combine(const float *down, const float *col_l2, const float *weights, int64_t seq,
                                    int64_t top_k, int64_t n_out, float *out, void *stream) {
    lmoe_clear_error();
    REQUIRE(down && weights && out, "down/weights/out is NULL");
    REQUIRE(seq >= 0 && top_k >= 1 && n_out >= 1, "combine dims must be positive");
    int64_t width = 1;
    while (width < top_k / 2) width <<= 1;
    REQUIRE(width <= 32, "combine top_k (%lld) needs a reduction width %lld > 32", (long long)top_k, (long long)width);
    REQUIRE(seq * top_k * n_out <= INT32_MAX, "combine seq*top_k*n_out (%lld) exceeds i32::MAX",
            (long long)(seq * top_k * n_out));
    LMOE_CUDA(launch_combine(down, col_l2, weights, (int)seq, (int)top_k, (int)n_out, out, (cudaStream_t)stream));
    return LMOE_OK;
}

// ------------------------------------------------------------------ map0 ----
extern "C" size_t lmoe_map0_scratch_bytes(int64_t n_expert, int64_t t) {
    if (n_expert < 0 || t < 0) return 0;
    return lmoe_align_up((size_t)n_expert * 4 + (size_t)n_expert * (size_t)t * 4, 256);
}

extern "C" lmoe_status lmoe_prepare_map0(const uint32_t *ids, int64_t t, int64_t top_k, int64_t n_expert,
                                         void *scratch, size_t scratch_bytes, void *stream) {
    lmoe_clear_error();
    REQUIRE(ids != nullptr, "ids is NULL");
    REQUIRE(t >= 0 && top_k >= 1 && n_expert >= 1, "map0 dims must be positive");
    REQUIRE(t * top_k <= INT32_MAX && n_expert <= 65535, "map0 problem too large");
    if (!scratch || scratch_bytes < lmoe_map0_scratch_bytes(n_expert, t))
        return lmoe_fail(LMOE_ERR_WORKSPACE, "map0 scratch needs %zu bytes, got %zu",
                         lmoe_map0_scratch_bytes(n_expert, t), scratch_bytes);
    uint32_t *tpe = static_cast<uint32_t *>(scratch);
    int32_t *ids_map = reinterpret_cast<int32_t *>(static_cast<uint8_t *>(scratch) + n_expert * 4);
    LMOE_CUDA(launch_map0(ids, (int)t, (int)top_k, (int)n_expert, tpe, ids_map, (cudaStream_t)stream));
    return LMOE_OK;
}

// ----------------------------------------------------------------- layer ----
extern "C" lmoe_status lmoe_layer_create(int64_t hidden, int64_t expert_ff, int64_t n_expert, int64_t top_k,
                                         float scale, int32_t norm, const float *router, const float *bias,
                                         const lmoe_expert_stack *gate, const lmoe_expert_stack *up,
                                         const lmoe_expert_stack *down, const lmoe_expert_stack *shared_gate,
                                         const lmoe_expert_stack *shared_up, const lmoe_expert_stack *shared_down,
                                         lmoe_layer **out) {
    lmoe_clear_error();
    REQUIRE(out != nullptr, "out handle pointer is NULL");
    *out = nullptr;
    REQUIRE(gate && up && down, "gate/up/down stack is NULL");
    lmoe_status st = route_check(0, n_expert, top_k);
    if (st) return st;
    // `FusedExperts::new`, src/moe.rs:205-213: the three stacks must agree on n_expert
    REQUIRE(gate->n_expert == up->n_expert && gate->n_expert == down->n_expert,
            "MoE expert stacks disagree on n_expert: gate=%lld, up=%lld, down=%lld", (long long)gate->n_expert,
            (long long)up->n_expert, (long long)down->n_expert);
    REQUIRE(gate->n_expert == n_expert, "stacks hold %lld experts, layer says %lld", (long long)gate->n_expert,
            (long long)n_expert);
    REQUIRE(gate->k == hidden && up->k == hidden && gate->n_out == expert_ff && up->n_out == expert_ff,
            "gate/up stacks must be [n_expert, expert_ff=%lld, hidden=%lld]", (long long)expert_ff, (long long)hidden);
    REQUIRE(down->k == expert_ff && down->n_out == hidden, "down stack must be [n_expert, hidden=%lld, expert_ff=%lld]",
            (long long)hidden, (long long)expert_ff);
    REQUIRE(gate->dtype == up->dtype, "gate and up stacks must share a dtype");
    REQUIRE(router != nullptr, "router is NULL");
    REQUIRE(hidden % QK_K == 0 && expert_ff % QK_K == 0, "hidden and expert_ff must be multiples of %d", QK_K);
    const bool any_sh = shared_gate || shared_up || shared_down;
    if (any_sh) {
        REQUIRE(shared_gate && shared_up && shared_down, "shared expert needs all of gate/up/down");
        REQUIRE(shared_gate->n_expert == 1 && shared_up->n_expert == 1 && shared_down->n_expert == 1,
                "shared stacks must hold exactly one expert");
        REQUIRE(shared_gate->k == hidden && shared_up->k == hidden && shared_gate->n_out == expert_ff &&
                    shared_up->n_out == expert_ff && shared_down->k == expert_ff && shared_down->n_out == hidden,
                "shared expert shapes must match the routed experts'");
        REQUIRE(shared_gate->dtype == gate->dtype && shared_up->dtype == gate->dtype &&
                    shared_down->dtype == down->dtype,
                "shared expert dtypes must match the routed experts'");
    }
    uint32_t *sync = nullptr;
    LMOE_CUDA(cudaMalloc(&sync, decode_sync_bytes()));
    if (cudaMemset(sync, 0, decode_sync_bytes()) != cudaSuccess) {
        cudaFree(sync);
        return lmoe_fail(LMOE_ERR_CUDA, "could not clear the layer's synchronisation words");
    }
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
        cudaFree(sync);
        return lmoe_fail(LMOE_ERR_CUDA, "could not create the layer's completion event");
    }
    lmoe_layer *ly = new (std::nothrow) lmoe_layer;
    if (ly == nullptr) {
        cudaFree(sync);
        cudaEventDestroy(ev);
    }
    REQUIRE(ly != nullptr, "out of host memory");
    ly->hidden = hidden; ly->expert_ff = expert_ff; ly->n_expert = n_expert; ly->top_k = top_k;
    ly->scale = scale; ly->norm = norm; ly->router = router; ly->bias = bias;
    ly->gate = gate; ly->up = up; ly->down = down;
    ly->sh_gate = shared_gate; ly->sh_up = shared_up; ly->sh_down = shared_down;
    ly->sync = sync;
    ly->dec_event = ev;
    *out = ly;
    return LMOE_OK;
}

extern "C" void lmoe_layer_destroy(lmoe_layer *layer) {
    if (!layer) return;
    cudaFree(layer->sync);
    if (layer->dec_event) cudaEventDestroy(layer->dec_event);
    for (int i = 0; i < 2; i++) {
        if (layer->host_x[i]) cudaFree(layer->host_x[i]);
        if (layer->host_copied[i]) cudaEventDestroy(layer->host_copied[i]);
        if (layer->host_slot_free[i]) cudaEventDestroy(layer->host_slot_free[i]);
    }
    if (layer->host_copy_stream) cudaStreamDestroy(layer->host_copy_stream);
    delete layer;
}

extern "C" lmoe_status lmoe_check_device_flag(void *workspace, void *stream) {
    lmoe_clear_error();
    if (!workspace) return lmoe_fail(LMOE_ERR_WORKSPACE, "workspace is NULL");
    uint32_t flag[4] = {0, 0, 0, 0};
    LMOE_CUDA(cudaMemcpyAsync(flag, workspace, sizeof flag, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    LMOE_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (flag[0] == 0) return LMOE_OK;
    LMOE_CUDA(cudaMemsetAsync(workspace, 0, sizeof flag, (cudaStream_t)stream));
    return lmoe_fail(LMOE_ERR_DEVICE_FLAG, "device flag 0x%x (detail %u, %u, %u): %s", flag[0], flag[1], flag[2],
                     flag[3],
                     flag[0] == LMOE_FLAG_BAD_EXPERT_ID ? "expert id out of range"
                     : flag[0] == LMOE_FLAG_WAIT_TIMEOUT ? "bounded wait ran out"
                     : flag[0] == LMOE_FLAG_BAD_INDEX    ? "index guard tripped"
                                                         : "unknown");
}
