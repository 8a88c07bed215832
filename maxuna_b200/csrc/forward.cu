// Whole-block entry points (`MoeBlock::forward`, src/moe.rs:73-78).
#include <stdlib.h>

#include "fused.cuh"

// decode.cu
size_t decode_workspace_bytes(int t, int hidden, int ff, int n_expert, int top_k);
int decode_max_tokens();
lmoe_status launch_moe_decode(const lmoe_layer *Ly, const float *x, int t, float *out, uint32_t *ids_out,
                              float *w_out, const uint32_t *ext_ids, const float *ext_w, int shared_first, int shared_count,
                              void *workspace, size_t workspace_bytes, int first_launch, cudaStream_t stream);
// prefill.cu
size_t prefill_workspace_bytes(const lmoe_layer *Ly, int64_t t);
lmoe_status launch_moe_prefill(const lmoe_layer *Ly, const float *x, int64_t t, float *out, uint32_t *ids_out,
                               float *w_out, void *workspace, size_t workspace_bytes, cudaStream_t stream);

size_t experts_prefill_workspace_bytes(const lmoe_layer *L, int64_t t);
lmoe_status launch_experts_prefill(const lmoe_layer *L, const float *x, const uint32_t *ids, const float *w, int64_t t,
                                   int add_shared, float *out, void *workspace, size_t workspace_bytes, cudaStream_t s);

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The one place that decides mat-vec or grouped GEMM for the entries that pick a path themselves.
// Process-wide and read once, like the reference's `OnceLock` switches (src/ops/mod.rs:24-60).
extern "C" int64_t lmoe_mm_id_min_seq(void) {
    static const int64_t v = [] {
        if (getenv("LAGUNA_NO_MM_ID")) return (int64_t)INT64_MAX; // presence-based: mat-vec everywhere
        const char *e = getenv("LAGUNA_MM_ID_MIN_SEQ");
        if (e && *e) {
            char *end = nullptr;
            const long long n = strtoll(e, &end, 10);
            if (end != e && n >= 1) return (int64_t)n;
        }
        return (int64_t)LMOE_DECODE_MAX_SEQ + 1;
    }();
    return v;
}

extern "C" size_t lmoe_layer_workspace_bytes(const lmoe_layer *layer, int64_t max_tokens) {
    if (!layer || max_tokens < 0) return 0;
    const int tdec = (int)(max_tokens < decode_max_tokens() ? (max_tokens < 1 ? 1 : max_tokens) : decode_max_tokens());
    size_t dec = decode_workspace_bytes(tdec, (int)layer->hidden, (int)layer->expert_ff, (int)layer->n_expert,
                                        (int)layer->top_k);
    size_t pre = prefill_workspace_bytes(layer, max_tokens);
    // host-buffer calls stage x and out behind the kernel scratch
    size_t host = 2 * lmoe_align_up((size_t)max_tokens * layer->hidden * 4, 256) +
                  2 * lmoe_align_up((size_t)max_tokens * layer->top_k * 4, 256);
    return lmoe_align_up(dec > pre ? dec : pre, 256) + host;
}

static lmoe_status forward_check(const lmoe_layer *layer, const float *x, int64_t t, float *out) {
    if (!layer) return lmoe_fail(LMOE_ERR_INVALID, "layer is NULL");
    if (!x || !out) return lmoe_fail(LMOE_ERR_INVALID, "x/out is NULL");
    if (t < 0 || t > (1 << 22)) return lmoe_fail(LMOE_ERR_INVALID, "t (%lld) out of range", (long long)t);
    if (!aligned16(x) || !aligned16(out)) return lmoe_fail(LMOE_ERR_INVALID, "x and out must be 16-byte aligned");
    return LMOE_OK;
}

// The mat-vec kernel over any token count, 64 tokens per launch, with the one-call-per-handle guard.
// ext_ids / ext_w: NULL = route inside the kernel, else the caller's decision [t, top_k].
// The shared expert is added for tokens [sh_first, sh_first + sh_count) of the call.
static lmoe_status decode_run(const lmoe_layer *layer, const float *x, int64_t t, float *out, uint32_t *ids_out,
                              float *weights_out, const uint32_t *ext_ids, const float *ext_w, int64_t sh_first, int64_t sh_count,
                              void *workspace, size_t workspace_bytes, cudaStream_t s) {
    // The kernel's CTAs meet through words owned by the layer: a second call may only start once the
    // previous one has finished.  Calls on one stream are ordered; a call on another stream is refused
    // while the previous call's completion event is still pending.
    std::lock_guard<std::mutex> lock(layer->dec_mutex);
    if (layer->dec_pending && layer->dec_stream != s) {
        const cudaError_t q = cudaEventQuery(layer->dec_event);
        if (q == cudaErrorNotReady)
            return lmoe_fail(LMOE_ERR_INVALID,
                             "a decode call on this layer handle is still in flight on another stream; one call at a "
                             "time per handle (create a second handle over the same stacks for a second stream)");
        if (q != cudaSuccess) (void)cudaGetLastError(); // e.g. an event recorded inside a capture: not decidable here
    }
    // more than 64 tokens: several launches, 64 tokens each, through the same workspace
    const int step = decode_max_tokens();
    const int64_t K = layer->top_k;
    for (int64_t t0 = 0; t0 < t; t0 += step) {
        const int n = (int)(t - t0 < step ? t - t0 : step);
        // the part of the shared-expert range that falls into this launch
        const int64_t a = sh_first > t0 ? sh_first : t0, b = sh_first + sh_count < t0 + n ? sh_first + sh_count : t0 + n;
        lmoe_status st = launch_moe_decode(layer, x + t0 * layer->hidden, n, out + t0 * layer->hidden,
                                           ids_out ? ids_out + t0 * K : nullptr, weights_out ? weights_out + t0 * K : nullptr,
                                           ext_ids ? ext_ids + t0 * K : nullptr, ext_w ? ext_w + t0 * K : nullptr,
                                           b > a ? (int)(a - t0) : 0, b > a ? (int)(b - a) : 0, workspace, workspace_bytes, t0 == 0, s);
        if (st) return st;
    }
    if (cudaEventRecord(layer->dec_event, s) == cudaSuccess) {
        layer->dec_stream = s;
        layer->dec_pending = true;
    } else {
        (void)cudaGetLastError();
    }
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_moe_forward_decode(const lmoe_layer *layer, const float *x, int64_t t, float *out,
                                               uint32_t *ids_out, float *weights_out, void *workspace,
                                               size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    lmoe_status st = forward_check(layer, x, t, out);
    if (st) return st;
    if (t == 0) return LMOE_OK;
    return decode_run(layer, x, t, out, ids_out, weights_out, nullptr, nullptr, 0, t, workspace, workspace_bytes,
                      (cudaStream_t)stream);
}

// `ExpertFfn::forward`, src/moe.rs:19-21: the caller routed (ids / weights on the device).
extern "C" size_t lmoe_experts_workspace_bytes(const lmoe_layer *layer, int64_t max_tokens) {
    if (!layer || max_tokens < 0) return 0;
    const int tdec = (int)(max_tokens < decode_max_tokens() ? (max_tokens < 1 ? 1 : max_tokens) : decode_max_tokens());
    const size_t dec = decode_workspace_bytes(tdec, (int)layer->hidden, (int)layer->expert_ff, (int)layer->n_expert,
                                              (int)layer->top_k);
    const size_t pre = experts_prefill_workspace_bytes(layer, max_tokens);
    return lmoe_align_up(dec > pre ? dec : pre, 256);
}

extern "C" lmoe_status lmoe_experts_forward(const lmoe_layer *layer, const float *x, const uint32_t *ids,
                                            const float *weights, int64_t t, int32_t add_shared, float *out,
                                            void *workspace, size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    lmoe_status st = forward_check(layer, x, t, out);
    if (st) return st;
    if (!ids || !weights) return lmoe_fail(LMOE_ERR_INVALID, "ids/weights is NULL");
    if (t == 0) return LMOE_OK;
    if (!workspace || workspace_bytes < lmoe_experts_workspace_bytes(layer, t))
        return lmoe_fail(LMOE_ERR_WORKSPACE, "workspace needs %zu bytes for %lld tokens, got %zu",
                         lmoe_experts_workspace_bytes(layer, t), (long long)t, workspace_bytes);
    if (t >= lmoe_mm_id_min_seq())
        return launch_experts_prefill(layer, x, ids, weights, t, add_shared, out, workspace, workspace_bytes, (cudaStream_t)stream);
    return decode_run(layer, x, t, out, nullptr, nullptr, ids, weights, 0, add_shared ? t : 0, workspace, workspace_bytes,
                      (cudaStream_t)stream);
}

// The expert-parallel decode step of one rank: the routed experts resident here for ALL tokens of the batch
// (slots of other ranks' experts arrive as empty), the replicated shared expert only for this rank's own tokens.
extern "C" lmoe_status lmoe_experts_forward_ep(const lmoe_layer *layer, const float *x, const uint32_t *ids,
                                               const float *weights, int64_t t, int64_t shared_first, int64_t shared_count,
                                               float *out, void *workspace, size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    lmoe_status st = forward_check(layer, x, t, out);
    if (st) return st;
    if (!ids || !weights) return lmoe_fail(LMOE_ERR_INVALID, "ids/weights is NULL");
    if (shared_first < 0 || shared_count < 0 || shared_first + shared_count > t)
        return lmoe_fail(LMOE_ERR_INVALID, "shared-expert token range [%lld, %lld) lies outside the %lld tokens", (long long)shared_first,
                         (long long)(shared_first + shared_count), (long long)t);
    if (t == 0) return LMOE_OK;
    if (t >= lmoe_mm_id_min_seq() && shared_count != 0 && shared_count != t)
        return lmoe_fail(LMOE_ERR_UNSUPPORTED, "a partial shared-expert range needs the mat-vec path (fewer than %lld tokens)",
                         (long long)lmoe_mm_id_min_seq());
    if (!workspace || workspace_bytes < lmoe_experts_workspace_bytes(layer, t))
        return lmoe_fail(LMOE_ERR_WORKSPACE, "workspace needs %zu bytes for %lld tokens, got %zu",
                         lmoe_experts_workspace_bytes(layer, t), (long long)t, workspace_bytes);
    if (t >= lmoe_mm_id_min_seq())
        return launch_experts_prefill(layer, x, ids, weights, t, shared_count == t, out, workspace, workspace_bytes,
                                      (cudaStream_t)stream);
    return decode_run(layer, x, t, out, nullptr, nullptr, ids, weights, shared_first, shared_count, workspace, workspace_bytes,
                      (cudaStream_t)stream);
}

extern "C" lmoe_status lmoe_moe_forward_prefill(const lmoe_layer *layer, const float *x, int64_t t, float *out,
                                                uint32_t *ids_out, float *weights_out, void *workspace,
                                                size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    lmoe_status st = forward_check(layer, x, t, out);
    if (st) return st;
    if (t == 0) return LMOE_OK;
    return launch_moe_prefill(layer, x, t, out, ids_out, weights_out, workspace, workspace_bytes, (cudaStream_t)stream);
}

// The device-side address of a page-locked, device-mapped host buffer; NULL for pageable or unknown memory
// (those go through a copy).
static float *host_buffer_device_alias(float *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    if (a.type != cudaMemoryTypeHost || a.devicePointer == nullptr) return nullptr;
    if ((reinterpret_cast<uintptr_t>(a.devicePointer) & 15u) != 0) return nullptr; // the kernel stores 16-byte vectors
    return static_cast<float *>(a.devicePointer);
}

// True for page-locked host memory (a copy from it is asynchronous).
static bool host_buffer_is_pinned(const void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeHost;
}

// The staging buffers, copy stream and events of the host-buffer decode path; false when they cannot be had
// (the call then copies on the caller's stream).
static bool host_staging_ready(const lmoe_layer *L) {
    if (L->host_failed) return false;
    if (L->host_copy_stream) return true;
    const size_t bytes = (size_t)decode_max_tokens() * L->hidden * 4;
    bool ok = cudaMalloc(&L->host_x[0], bytes) == cudaSuccess && cudaMalloc(&L->host_x[1], bytes) == cudaSuccess;
    for (int i = 0; i < 2 && ok; i++)
        ok = cudaEventCreateWithFlags(&L->host_copied[i], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&L->host_slot_free[i], cudaEventDisableTiming) == cudaSuccess;
    cudaStream_t cs = nullptr;
    ok = ok && cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        L->host_failed = true; // what was created is released with the layer
        return false;
    }
    L->host_copy_stream = cs;
    return true;
}

static lmoe_status forward_host_enqueue(const lmoe_layer *layer, const float *x_host, int64_t t, float *out_host,
                                        uint32_t *ids_out_host, float *weights_out_host, void *workspace,
                                        size_t workspace_bytes, void *stream) {
    if (!layer) return lmoe_fail(LMOE_ERR_INVALID, "layer is NULL");
    if (!x_host || !out_host) return lmoe_fail(LMOE_ERR_INVALID, "x_host/out_host is NULL");
    if (t < 0 || t > (1 << 22)) return lmoe_fail(LMOE_ERR_INVALID, "t (%lld) out of range", (long long)t);
    if (t == 0) return LMOE_OK;
    const size_t need = lmoe_layer_workspace_bytes(layer, t);
    if (!workspace || workspace_bytes < need)
        return lmoe_fail(LMOE_ERR_WORKSPACE, "workspace needs %zu bytes for %lld tokens, got %zu", need, (long long)t,
                         workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t xb = lmoe_align_up((size_t)t * layer->hidden * 4, 256);
    const size_t ib = lmoe_align_up((size_t)t * layer->top_k * 4, 256);
    const size_t kernel_ws = need - 2 * xb - 2 * ib;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    float *xd = reinterpret_cast<float *>(ws + kernel_ws);
    float *od = reinterpret_cast<float *>(ws + kernel_ws + xb);
    uint32_t *idd = reinterpret_cast<uint32_t *>(ws + kernel_ws + 2 * xb);
    float *wd = reinterpret_cast<float *>(ws + kernel_ws + 2 * xb + ib);
    lmoe_status st;
    // the reference switches to its grouped GEMM at 32 tokens (`use_mm`, src/moe.rs:236-240); here the mat-vec
    // kernel, which streams each distinct expert once per launch, stays ahead up to 64 tokens
    const bool decode = t < lmoe_mm_id_min_seq();
    // Decode: when the result buffer is page-locked host memory that the device can address, the kernel's last
    // phase stores the rows there itself (a few KB of posted writes) and the device-to-host copy, whose fixed
    // cost is a tenth of a one-token call, is not needed.
    float *out_direct = decode ? host_buffer_device_alias(out_host) : nullptr;
    if (decode && out_direct && t <= decode_max_tokens() && host_buffer_is_pinned(x_host)) {
        // Both buffers pinned: the input goes through one of two staging buffers of the layer on the layer's own
        // copy stream, so this call's copy overlaps the previous call's kernel; `stream` waits for the copy, the
        // copy waits for the kernel that last read the staging buffer.  x_host is read without regard to earlier
        // work on `stream`: it must be complete when the call is made.
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(s, &cap) != cudaSuccess) (void)cudaGetLastError();
        std::unique_lock<std::mutex> lock(layer->host_mutex);
        if (cap == cudaStreamCaptureStatusNone && host_staging_ready(layer)) {
            const int slot = layer->host_slot;
            layer->host_slot ^= 1;
            cudaStream_t cs = layer->host_copy_stream;
            LMOE_CUDA(cudaStreamWaitEvent(cs, layer->host_slot_free[slot], 0));
            LMOE_CUDA(cudaMemcpyAsync(layer->host_x[slot], x_host, (size_t)t * layer->hidden * 4, cudaMemcpyHostToDevice, cs));
            LMOE_CUDA(cudaEventRecord(layer->host_copied[slot], cs));
            LMOE_CUDA(cudaStreamWaitEvent(s, layer->host_copied[slot], 0));
            st = lmoe_moe_forward_decode(layer, layer->host_x[slot], t, out_direct, ids_out_host ? idd : nullptr,
                                         weights_out_host ? wd : nullptr, workspace, kernel_ws, stream);
            if (st) return st;
            LMOE_CUDA(cudaEventRecord(layer->host_slot_free[slot], s));
            lock.unlock();
            if (ids_out_host) LMOE_CUDA(cudaMemcpyAsync(ids_out_host, idd, (size_t)t * layer->top_k * 4, cudaMemcpyDeviceToHost, s));
            if (weights_out_host)
                LMOE_CUDA(cudaMemcpyAsync(weights_out_host, wd, (size_t)t * layer->top_k * 4, cudaMemcpyDeviceToHost, s));
            return LMOE_OK;
        }
    }
    LMOE_CUDA(cudaMemcpyAsync(xd, x_host, (size_t)t * layer->hidden * 4, cudaMemcpyHostToDevice, s));
    if (!decode)
        st = lmoe_moe_forward_prefill(layer, xd, t, od, ids_out_host ? idd : nullptr, weights_out_host ? wd : nullptr,
                                      workspace, kernel_ws, stream);
    else
        st = lmoe_moe_forward_decode(layer, xd, t, out_direct ? out_direct : od, ids_out_host ? idd : nullptr,
                                     weights_out_host ? wd : nullptr, workspace, kernel_ws, stream);
    if (st) return st;
    if (!out_direct) LMOE_CUDA(cudaMemcpyAsync(out_host, od, (size_t)t * layer->hidden * 4, cudaMemcpyDeviceToHost, s));
    if (ids_out_host) LMOE_CUDA(cudaMemcpyAsync(ids_out_host, idd, (size_t)t * layer->top_k * 4, cudaMemcpyDeviceToHost, s));
    if (weights_out_host)
        LMOE_CUDA(cudaMemcpyAsync(weights_out_host, wd, (size_t)t * layer->top_k * 4, cudaMemcpyDeviceToHost, s));
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_moe_forward_host(const lmoe_layer *layer, const float *x_host, int64_t t, float *out_host,
                                             uint32_t *ids_out_host, float *weights_out_host, void *workspace,
                                             size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    lmoe_status st = forward_host_enqueue(layer, x_host, t, out_host, ids_out_host, weights_out_host, workspace,
                                          workspace_bytes, stream);
    if (st) return st;
    LMOE_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_moe_forward_host_async(const lmoe_layer *layer, const float *x_host, int64_t t, float *out_host,
                                                   uint32_t *ids_out_host, float *weights_out_host, void *workspace,
                                                   size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    return forward_host_enqueue(layer, x_host, t, out_host, ids_out_host, weights_out_host, workspace, workspace_bytes,
                                stream);
}

// ---- the transformer layer's FFN half around the block (src/model.rs:340-350) -------------
extern "C" lmoe_status lmoe_rms_norm(const float *x, const float *weight, float eps, int64_t t, int64_t hidden,
                                     float *out, void *stream) {
    lmoe_clear_error();
    if (!x || !weight || !out) return lmoe_fail(LMOE_ERR_INVALID, "x/weight/out is NULL");
    if (t < 0 || t > (1 << 22) || hidden < 4 || hidden % 4 || hidden > (1 << 20))
        return lmoe_fail(LMOE_ERR_INVALID, "rms_norm: t >= 0 and hidden a multiple of 4 required (t=%lld, hidden=%lld)",
                         (long long)t, (long long)hidden);
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15u)
        return lmoe_fail(LMOE_ERR_INVALID, "rms_norm: x, weight and out must be 16-byte aligned");
    LMOE_CUDA(launch_rms_norm(x, weight, eps, t, (int)hidden, out, (cudaStream_t)stream));
    return LMOE_OK;
}

extern "C" size_t lmoe_moe_layer_workspace_bytes(const lmoe_layer *layer, int64_t max_tokens) {
    if (!layer || max_tokens < 0) return 0;
    return lmoe_layer_workspace_bytes(layer, max_tokens) + lmoe_align_up((size_t)(max_tokens < 1 ? 1 : max_tokens) * layer->hidden * 4, 256);
}

extern "C" lmoe_status lmoe_moe_layer_forward(const lmoe_layer *layer, const float *ffn_inp, const float *norm_weight,
                                              float eps, int64_t t, float *out, uint32_t *ids_out, float *weights_out,
                                              void *workspace, size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    lmoe_status st = forward_check(layer, ffn_inp, t, out);
    if (st) return st;
    if (!norm_weight) return lmoe_fail(LMOE_ERR_INVALID, "norm_weight is NULL");
    if (ffn_inp == out) return lmoe_fail(LMOE_ERR_INVALID, "out must not alias ffn_inp (the residual is read after the block)");
    if (t == 0) return LMOE_OK;
    const size_t need = lmoe_moe_layer_workspace_bytes(layer, t);
    if (!workspace || workspace_bytes < need)
        return lmoe_fail(LMOE_ERR_WORKSPACE, "workspace needs %zu bytes for %lld tokens, got %zu", need, (long long)t,
                         workspace_bytes);
    const size_t block_ws = lmoe_layer_workspace_bytes(layer, t);
    float *normed = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + block_ws);
    if ((st = lmoe_rms_norm(ffn_inp, norm_weight, eps, t, layer->hidden, normed, stream))) return st;
    // mat-vec kernel up to 64 tokens, grouped GEMM beyond (measured crossover; the reference's own is 32)
    if (t >= lmoe_mm_id_min_seq())
        st = lmoe_moe_forward_prefill(layer, normed, t, out, ids_out, weights_out, workspace, block_ws, stream);
    else
        st = lmoe_moe_forward_decode(layer, normed, t, out, ids_out, weights_out, workspace, block_ws, stream);
    if (st) return st;
    // x = ffn_inp + ffn_out
    LMOE_CUDA(launch_add_inplace(out, ffn_inp, t * layer->hidden, (cudaStream_t)stream));
    return LMOE_OK;
}
