// Prefill path: routing, per-expert row lists, grouped tensor-core GEMMs for
// gate / up / down, SwiGLU with the f16 range guard, fixed-order combine, shared expert.
// Reference: the mm_id branch of `FusedExperts::forward`, src/moe.rs:236-323, and
// `MoeBlock::forward`, src/moe.rs:73-78.
#include "fused.cuh"

// mm_id.cu
int64_t mm_max_tiles(int64_t rows, int64_t n_expert, int64_t n_out);
bool mm_id_kernel_available(int dtype, int64_t n_out, int64_t k);
size_t mm_tiles_bytes(int64_t rows, int64_t n_expert, int64_t n_out);
size_t mm_tiled_bytes(int64_t rows, int64_t n_expert, int64_t k);
cudaError_t launch_gather_tiles(const void *x, int x_f16, int x_per_row, int top_k, int k, const uint32_t *tpe,
                                const int32_t *ids_map, int map_stride, int n_expert, void *xt, int32_t *pos,
                                int32_t *spos, int32_t *sfid, cudaStream_t s);
lmoe_status launch_mm_gateup(const lmoe_expert_stack *gate, const lmoe_expert_stack *up, const void *xt,
                             const uint32_t *tpe, const int32_t *ids_map, int64_t map_stride, int64_t list_rows,
                             float *act, int sorted, void *tiles_ws, uint32_t *flag, cudaStream_t stream);
bool mm_down_available(const lmoe_expert_stack *down);
lmoe_status launch_mm_down(const lmoe_expert_stack *down, const void *xt, const uint32_t *tpe, const int32_t *ids_map,
                           int64_t map_stride, int64_t list_rows, const float *row_scale, float *out, int sorted,
                           void *tiles_ws, uint32_t *flag, cudaStream_t stream);
lmoe_status launch_mm_id(const lmoe_expert_stack *st, const void *xt, const uint32_t *tpe, const int32_t *ids_map,
                         int64_t map_stride, int64_t list_rows, const float *row_scale, float *out, void *tiles_ws,
                         uint32_t *flag, cudaStream_t stream);

namespace {

// One warp per row: act = silu(g) * u; l2 = clamp(||act||, 1e-8, 1e30); the f16 operand of the
// down projection is act * 32768 / l2 (src/moe.rs:292-302), written in the grouped GEMM's tile
// order (row tile pos / LMOE_MM_N, row pos % LMOE_MM_N, 128-byte swizzle, groups of 8 as [0 2 1 3 4 6 5 7]);
// scale[row] = l2 * 2^-15 * weight[row] undoes it in the down epilogue together with the
// routing weight (src/ops/combine.metal:102-133).
__global__ void __launch_bounds__(256) swiglu_rows_kernel(const float *__restrict__ g, const float *__restrict__ u,
                                                          const float *__restrict__ w, const int32_t *__restrict__ pos,
                                                          int64_t rows, int ff, uint8_t *__restrict__ act,
                                                          float *__restrict__ scale) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float *gr = g + row * ff, *ur = u + row * ff;
    float ss = 0.f;
    for (int i = lane * 8; i < ff; i += 256) {
        const float4 g0 = *reinterpret_cast<const float4 *>(gr + i), g1 = *reinterpret_cast<const float4 *>(gr + i + 4);
        const float4 u0 = *reinterpret_cast<const float4 *>(ur + i), u1 = *reinterpret_cast<const float4 *>(ur + i + 4);
        const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float a = __fmul_rn(__fdiv_rn(gv[j], __fadd_rn(1.0f, expf(-gv[j]))), uv[j]);
            ss += a * a;
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float l2 = fminf(fmaxf(sqrtf(ss), 1e-8f), 1e30f);
    const float k = 32768.0f / l2;
    const int p = pos[row];
    for (int i = lane * 8; i < ff; i += 256) {
        const float4 g0 = *reinterpret_cast<const float4 *>(gr + i), g1 = *reinterpret_cast<const float4 *>(gr + i + 4);
        const float4 u0 = *reinterpret_cast<const float4 *>(ur + i), u1 = *reinterpret_cast<const float4 *>(ur + i + 4);
        const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = __fmul_rn(__fdiv_rn(gv[j], __fadd_rn(1.0f, expf(-gv[j]))), uv[j]) * k;
        __align__(16) __half2 h[4] = {__floats2half2_rn(a[0], a[2]), __floats2half2_rn(a[1], a[3]),
                                      __floats2half2_rn(a[4], a[6]), __floats2half2_rn(a[5], a[7])};
        const int ci = i >> 3;
        const size_t off = (((size_t)(p / LMOE_MM_N) * (ff / 64) + (ci >> 3)) * LMOE_MM_N + (p % LMOE_MM_N)) * 128 +
                           ((size_t)((ci & 7) ^ (p & 7)) << 4);
        *reinterpret_cast<uint4 *>(act + off) = *reinterpret_cast<const uint4 *>(h);
    }
    if (lane == 0) scale[row] = l2 * 0x1p-15f * (w ? w[row] : 1.0f);
}

// Same range guard for an activation that is already silu(g)*u (f32): l2, rescale, f16, tile order.
// With `sfid` the rows of `a` (and of `scale`) are in expert-sorted order and sfid[row] is the flat id.
__global__ void __launch_bounds__(256) rescale_rows_kernel(const float *__restrict__ a, const float *__restrict__ w,
                                                           const int32_t *__restrict__ pos, const int32_t *__restrict__ sfid,
                                                           int64_t rows, int ff, uint8_t *__restrict__ act,
                                                           float *__restrict__ scale) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int64_t fid = sfid ? sfid[row] : row;
    if (fid < 0) return;                                   // no routed row here (masked slots leave a tail unused)
    const float *ar = a + row * ff;
    float ss = 0.f;
    for (int i = lane * 8; i < ff; i += 256) {
        const float4 a0 = *reinterpret_cast<const float4 *>(ar + i), a1 = *reinterpret_cast<const float4 *>(ar + i + 4);
        ss += a0.x * a0.x + a0.y * a0.y + a0.z * a0.z + a0.w * a0.w + a1.x * a1.x + a1.y * a1.y + a1.z * a1.z + a1.w * a1.w;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float l2 = fminf(fmaxf(sqrtf(ss), 1e-8f), 1e30f);
    const float k = 32768.0f / l2;
    const int p = pos[fid];
    for (int i = lane * 8; i < ff; i += 256) {
        const float4 a0 = *reinterpret_cast<const float4 *>(ar + i), a1 = *reinterpret_cast<const float4 *>(ar + i + 4);
        __align__(16) __half2 h[4] = {__floats2half2_rn(a0.x * k, a0.z * k), __floats2half2_rn(a0.y * k, a0.w * k),
                                      __floats2half2_rn(a1.x * k, a1.z * k), __floats2half2_rn(a1.y * k, a1.w * k)};
        const int ci = i >> 3;
        const size_t off = (((size_t)(p / LMOE_MM_N) * (ff / 64) + (ci >> 3)) * LMOE_MM_N + (p % LMOE_MM_N)) * 128 +
                           ((size_t)((ci & 7) ^ (p & 7)) << 4);
        *reinterpret_cast<uint4 *>(act + off) = *reinterpret_cast<const uint4 *>(h);
    }
    if (lane == 0) scale[row] = l2 * 0x1p-15f * (w ? w[fid] : 1.0f);
}

// out[t, c] = sum over slots (in slot order) of y[t, s, c], then + shared[t, c].
__global__ void sum_slots_kernel(const float *__restrict__ y, const float *__restrict__ shared, int64_t t, int top_k,
                                 int n4, float *__restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= t * n4) return;
    const int64_t tok = i / n4, c = i - tok * n4;
    const float4 *yp = reinterpret_cast<const float4 *>(y) + tok * top_k * n4 + c;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < top_k; k++) {
        const float4 v = yp[(int64_t)k * n4];
        s.x = __fadd_rn(s.x, v.x); s.y = __fadd_rn(s.y, v.y); s.z = __fadd_rn(s.z, v.z); s.w = __fadd_rn(s.w, v.w);
    }
    if (shared) {
        const float4 v = reinterpret_cast<const float4 *>(shared)[i];
        s.x = __fadd_rn(s.x, v.x); s.y = __fadd_rn(s.y, v.y); s.z = __fadd_rn(s.z, v.z); s.w = __fadd_rn(s.w, v.w);
    }
    reinterpret_cast<float4 *>(out)[i] = s;
}

// Same sum when the partial rows are unscaled and in expert-sorted order: row spos[flat id] of `y`
// times scale[that row]; likewise for the shared expert's rows.  A negative position marks an empty slot.
__global__ void sum_sorted_kernel(const float *__restrict__ y, const float *__restrict__ scale,
                                  const int32_t *__restrict__ spos, const float *__restrict__ shared,
                                  const float *__restrict__ sh_scale, const int32_t *__restrict__ sh_spos, int64_t t,
                                  int top_k, int n4, float *__restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= t * n4) return;
    const int64_t tok = i / n4, c = i - tok * n4;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < top_k; k++) {
        const int64_t r = spos[tok * top_k + k];
        if (r < 0) continue;                               // empty slot
        const float sc = scale ? scale[r] : 1.0f;
        const float4 v = reinterpret_cast<const float4 *>(y)[r * n4 + c];
        s.x = __fadd_rn(s.x, __fmul_rn(v.x, sc)); s.y = __fadd_rn(s.y, __fmul_rn(v.y, sc));
        s.z = __fadd_rn(s.z, __fmul_rn(v.z, sc)); s.w = __fadd_rn(s.w, __fmul_rn(v.w, sc));
    }
    if (shared) {
        const int64_t r = sh_spos ? sh_spos[tok] : tok;
        const float sc = sh_scale ? sh_scale[r] : 1.0f;
        const float4 v = reinterpret_cast<const float4 *>(shared)[r * n4 + c];
        s.x = __fadd_rn(s.x, __fmul_rn(v.x, sc)); s.y = __fadd_rn(s.y, __fmul_rn(v.y, sc));
        s.z = __fadd_rn(s.z, __fmul_rn(v.z, sc)); s.w = __fadd_rn(s.w, __fmul_rn(v.w, sc));
    }
    reinterpret_cast<float4 *>(out)[i] = s;
}

// Expert-parallel dispatch packing: the routed rows of expert e (list `ids_map[e]`) go to positions
// [prefix(e), prefix(e) + tpe[e]) of the send buffers, as f16; experts are contiguous per destination rank,
// so the buffer is grouped by rank.  row_pos[flat id] remembers where each row went.
__global__ void __launch_bounds__(256) ep_pack_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                      const uint32_t *__restrict__ tpe, const int32_t *__restrict__ ids_map,
                                                      int map_stride, int top_k, int hidden, int e_local,
                                                      __half *__restrict__ rows, uint32_t *__restrict__ local_ids,
                                                      float *__restrict__ row_w, int32_t *__restrict__ row_pos) {
    __shared__ int warp_rows[8];
    __shared__ int row0_s;
    const int e = blockIdx.x;
    int rpart = 0;
    for (int i = threadIdx.x; i < e; i += 256) rpart += (int)tpe[i];
    for (int o = 16; o; o >>= 1) rpart += __shfl_xor_sync(0xffffffffu, rpart, o);
    if ((threadIdx.x & 31) == 0) warp_rows[threadIdx.x >> 5] = rpart;
    __syncthreads();
    if (threadIdx.x == 0) {
        int r = 0;
        for (int i = 0; i < 8; i++) r += warp_rows[i];
        row0_s = r;
    }
    __syncthreads();
    const int row0 = row0_s, n = (int)tpe[e], chunks = hidden / 8;
    for (int i = blockIdx.y; i < n; i += gridDim.y) {
        const int fid = ids_map[(size_t)e * map_stride + i];
        const int p = row0 + i;
        const float *src = x + (size_t)(fid / top_k) * hidden;
        __half *dst = rows + (size_t)p * hidden;
        for (int ci = threadIdx.x; ci < chunks; ci += 256) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(src) + 2 * ci);
            const float4 b = __ldg(reinterpret_cast<const float4 *>(src) + 2 * ci + 1);
            __align__(16) __half2 h[4] = {__floats2half2_rn(a.x, a.y), __floats2half2_rn(a.z, a.w),
                                          __floats2half2_rn(b.x, b.y), __floats2half2_rn(b.z, b.w)};
            reinterpret_cast<uint4 *>(dst)[ci] = *reinterpret_cast<const uint4 *>(h);
        }
        if (threadIdx.x == 0) {
            local_ids[p] = (uint32_t)(e % e_local);
            row_w[p] = w[fid];
            row_pos[fid] = p;
        }
    }
}

// send_counts[r] = rows routed to the experts of rank r
__global__ void ep_counts_kernel(const uint32_t *__restrict__ tpe, int n_expert, int e_local, long long *__restrict__ counts) {
    const int r = blockIdx.x;
    int c = 0;
    for (int e = r * e_local + threadIdx.x; e < (r + 1) * e_local && e < n_expert; e += 32) c += (int)tpe[e];
    for (int o = 16; o; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if (threadIdx.x == 0) counts[r] = c;
}

// identity row list for a one-expert stack: tpe[0] = t, ids_map[i] = i
__global__ void iota_list_kernel(int64_t t, uint32_t *tpe, int32_t *ids_map) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0) tpe[0] = (uint32_t)t;
    if (i < t) ids_map[i] = (int32_t)i;
}

struct Carver {
    uint8_t *base;
    size_t off;
    template <typename T>
    T *take(size_t count) {
        T *p = reinterpret_cast<T *>(base + off);
        off += lmoe_align_up(count * sizeof(T), 256);
        return p;
    }
};

// Scratch of one grouped SwiGLU FFN over `rows` routed rows.
size_t ffn_bytes(int64_t rows, int64_t hidden, int64_t ff, int64_t n_expert) {
    size_t o = 0;
    o += mm_tiled_bytes(rows, n_expert, hidden);             // x in tile order
    o += lmoe_align_up((size_t)rows * 4, 256);               // position of every flat id
    o += 2 * lmoe_align_up((size_t)rows * ff * 4, 256);      // gate, up
    o += mm_tiled_bytes(rows, n_expert, ff);                 // f16 activation in tile order
    o += lmoe_align_up((size_t)rows * 4, 256);               // row scale
    o += lmoe_align_up((size_t)rows * 4, 256);               // flat id of every sorted row
    const size_t t1 = mm_tiles_bytes(rows, n_expert, ff), t2 = mm_tiles_bytes(rows, n_expert, hidden);
    o += t1 > t2 ? t1 : t2;
    return o;
}

// y[rows, hidden] = row_weight * FFN_{expert of row}(x[row / top_k]); lists as produced by map0.
// With `spos` / `scale_out` (both [rows], caller-owned) and the fused kernels available, y instead holds the
// UNSCALED rows in expert-sorted order: row spos[flat id], to be multiplied by scale_out[that row]; the
// tensor-core epilogues then store whole tile columns side by side instead of scattering by flat id.
// *sorted_used tells which form was produced.  `masked`: ids >= n_expert were left out of the lists.
lmoe_status ffn_grouped(const lmoe_expert_stack *gate, const lmoe_expert_stack *up, const lmoe_expert_stack *down,
                        const void *x, int top_k, int64_t t, const uint32_t *tpe, const int32_t *ids_map,
                        int64_t map_stride, const float *row_w, float *y, uint8_t *ws, uint32_t *flag,
                        cudaStream_t s, int32_t *spos = nullptr, float *scale_out = nullptr, bool *sorted_used = nullptr,
                        int x_f16 = 0, int masked = 0) {
    const int64_t rows = t * top_k, ff = gate->n_out, hidden = gate->k, ne = gate->n_expert;
    Carver c{ws, 0};
    uint8_t *xt = c.take<uint8_t>(mm_tiled_bytes(rows, ne, hidden));
    int32_t *pos = c.take<int32_t>((size_t)rows);
    float *g = c.take<float>((size_t)rows * ff), *u = c.take<float>((size_t)rows * ff);
    uint8_t *act = c.take<uint8_t>(mm_tiled_bytes(rows, ne, ff));
    float *rs = c.take<float>((size_t)rows);
    int32_t *sfid = c.take<int32_t>((size_t)rows);
    void *tiles = ws + c.off;
    lmoe_status st;
    const bool fused_gu = gate->dtype == LMOE_Q4_K && up->dtype == LMOE_Q4_K;
    const bool fused_dn = mm_down_available(down);
    const bool sorted = spos && scale_out && fused_gu && fused_dn;
    if (sorted_used) *sorted_used = sorted;
    if (masked) {
        // some (token, slot) pairs name no expert: the lists skip them, and the per-row arrays mark them
        if (!sorted) return lmoe_fail(LMOE_ERR_UNSUPPORTED, "masked slots need the fused Q4_K / Q6_K kernels");
        LMOE_CUDA(cudaMemsetAsync(spos, 0xFF, (size_t)rows * 4, s));
        LMOE_CUDA(cudaMemsetAsync(sfid, 0xFF, (size_t)rows * 4, s));
    }
    LMOE_CUDA(launch_gather_tiles(x, x_f16, 1, top_k, (int)hidden, tpe, ids_map, (int)map_stride, (int)ne, xt, pos,
                                  sorted ? spos : nullptr, sorted ? sfid : nullptr, s));
    if (fused_gu) {
        // both projections in one pass over the activations, SwiGLU in the epilogue
        if ((st = launch_mm_gateup(gate, up, xt, tpe, ids_map, map_stride, rows, g, sorted, tiles, flag, s))) return st;
        rescale_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(g, row_w, pos, sorted ? sfid : nullptr, rows, (int)ff,
                                                                       act, sorted ? scale_out : rs);
        LMOE_LAUNCH_CHECK("rescale_rows_kernel");
    } else {
        if ((st = launch_mm_id(gate, xt, tpe, ids_map, map_stride, rows, nullptr, g, tiles, flag, s))) return st;
        if ((st = launch_mm_id(up, xt, tpe, ids_map, map_stride, rows, nullptr, u, tiles, flag, s))) return st;
        swiglu_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(g, u, row_w, pos, rows, (int)ff, act, rs);
        LMOE_LAUNCH_CHECK("swiglu_rows_kernel");
    }
    if (fused_dn)
        st = launch_mm_down(down, act, tpe, ids_map, map_stride, rows, sorted ? nullptr : rs, y, sorted, tiles, flag, s);
    else
        st = launch_mm_id(down, act, tpe, ids_map, map_stride, rows, rs, y, tiles, flag, s);
    return st;
}

bool layer_mm_ok(const lmoe_layer *L) {
    return mm_id_kernel_available(L->gate->dtype, L->expert_ff, L->hidden) &&
           mm_id_kernel_available(L->down->dtype, L->hidden, L->expert_ff) && L->expert_ff % 256 == 0 &&
           L->hidden % 8 == 0;
}

} // namespace

// Scratch of the routed (+ shared) experts of `t` tokens with `top_k` slots each, after the routing decision.
static size_t experts_ws_bytes(const lmoe_layer *L, int64_t t, int64_t top_k) {
    const int64_t rows = t * top_k;
    size_t o = 0;
    o += lmoe_map0_scratch_bytes(L->n_expert, t);
    o += lmoe_align_up((size_t)rows * L->hidden * 4, 256);           // routed partial rows
    o += lmoe_align_up((size_t)t * L->hidden * 4, 256);              // shared expert rows
    o += lmoe_align_up((size_t)(t + 64) * 4, 256);                   // identity list
    o += 2 * lmoe_align_up((size_t)rows * 4, 256);                   // sorted position and scale of every routed row
    o += 2 * lmoe_align_up((size_t)t * 4, 256);                      // the same for the shared expert's rows
    o += ffn_bytes(rows, L->hidden, L->expert_ff, L->n_expert);
    return o;
}

// The experts of a block on a routing decision that is already on the device: per-expert row lists, grouped
// GEMMs, slot-order sum, optionally the shared expert.  x: [t, hidden] f32 or f16; ids / w: [t, top_k]
// (`masked`: ids >= n_expert are empty slots).  `ws` holds experts_ws_bytes(); `flag` is the device flag.
static lmoe_status experts_prefill(const lmoe_layer *L, const void *x, int x_f16, const uint32_t *ids, const float *w,
                                   int64_t t, int64_t top_k, int masked, int add_shared, float *out, uint8_t *ws,
                                   uint32_t *flag, cudaStream_t s) {
    const int64_t rows = t * top_k, H = L->hidden;
    Carver c{ws, 0};
    uint8_t *map0 = c.take<uint8_t>(lmoe_map0_scratch_bytes(L->n_expert, t));
    float *y = c.take<float>((size_t)rows * H);
    float *ysh = c.take<float>((size_t)t * H);
    uint32_t *sh_list = c.take<uint32_t>((size_t)t + 64);
    int32_t *spos = c.take<int32_t>((size_t)rows);
    float *rscale = c.take<float>((size_t)rows);
    int32_t *sh_spos = c.take<int32_t>((size_t)t);
    float *sh_scale = c.take<float>((size_t)t);
    uint8_t *ffn_ws = ws + c.off;
    uint32_t *tpe = reinterpret_cast<uint32_t *>(map0);
    int32_t *ids_map = reinterpret_cast<int32_t *>(map0 + L->n_expert * 4);
    // ids >= n_expert match no expert's list: those slots stay empty
    LMOE_CUDA(launch_map0(ids, (int)t, (int)top_k, (int)L->n_expert, tpe, ids_map, s));
    bool sorted = false, sh_sorted = false;
    lmoe_status st = ffn_grouped(L->gate, L->up, L->down, x, (int)top_k, t, tpe, ids_map, t, w, y, ffn_ws, flag, s, spos,
                                 rscale, &sorted, x_f16, masked);
    if (st) return st;
    const float *shared = nullptr;
    if (add_shared && L->sh_gate) {
        iota_list_kernel<<<(unsigned)((t + 255) / 256), 256, 0, s>>>(t, sh_list, reinterpret_cast<int32_t *>(sh_list + 64));
        LMOE_LAUNCH_CHECK("iota_list_kernel");
        // the shared expert's rows take the same form as the routed ones, so one kernel sums both
        st = ffn_grouped(L->sh_gate, L->sh_up, L->sh_down, x, 1, t, sh_list, reinterpret_cast<int32_t *>(sh_list + 64), t,
                         nullptr, ysh, ffn_ws, flag, s, sorted ? sh_spos : nullptr, sorted ? sh_scale : nullptr, &sh_sorted,
                         x_f16);
        if (st) return st;
        shared = ysh;
    }
    const int64_t n = t * (H / 4);
    if (sorted && (!shared || sh_sorted))
        sum_sorted_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(y, rscale, spos, shared, sh_scale, sh_spos, t,
                                                                      (int)top_k, (int)(H / 4), out);
    else
        sum_slots_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(y, shared, t, (int)top_k, (int)(H / 4), out);
    LMOE_LAUNCH_CHECK("sum_slots_kernel");
    return LMOE_OK;
}

size_t prefill_workspace_bytes(const lmoe_layer *L, int64_t t) {
    if (t < 1) t = 1;
    const int64_t rows = t * L->top_k;
    size_t o = 65536;
    o += lmoe_align_up((size_t)t * L->n_expert * 4, 256);            // logits
    o += 2 * lmoe_align_up((size_t)rows * 4, 256);                   // ids, weights
    o += experts_ws_bytes(L, t, L->top_k);
    return o;
}

lmoe_status launch_moe_prefill(const lmoe_layer *L, const float *x, int64_t t, float *out, uint32_t *ids_out,
                               float *w_out, void *workspace, size_t workspace_bytes, cudaStream_t s) {
    if (!layer_mm_ok(L)) return lmoe_fail(LMOE_ERR_UNSUPPORTED, "no grouped-GEMM kernel for this layer's shapes / dtypes");
    if (!workspace || workspace_bytes < prefill_workspace_bytes(L, t))
        return lmoe_fail(LMOE_ERR_WORKSPACE, "prefill workspace needs %zu bytes, got %zu", prefill_workspace_bytes(L, t),
                         workspace_bytes);
    if (t * L->top_k > INT32_MAX / 2) return lmoe_fail(LMOE_ERR_INVALID, "too many routed rows");
    const int64_t rows = t * L->top_k, H = L->hidden;
    Carver c{static_cast<uint8_t *>(workspace), 65536};
    uint32_t *flag = reinterpret_cast<uint32_t *>(workspace);
    float *logits = c.take<float>((size_t)t * L->n_expert);
    uint32_t *ids = c.take<uint32_t>((size_t)rows);
    float *w = c.take<float>((size_t)rows);
    uint8_t *ex_ws = static_cast<uint8_t *>(workspace) + c.off;

    LMOE_CUDA(cudaMemsetAsync(flag, 0, 16, s)); // a fresh device flag: the workspace needs no initialisation
    LMOE_CUDA(launch_route_logits(L->router, x, (int)t, (int)H, (int)L->n_expert, logits, s));
    LMOE_CUDA(launch_route_select(logits, L->bias, (int)t, (int)L->n_expert, (int)L->top_k, L->scale, L->norm, ids, w, s));
    lmoe_status st = experts_prefill(L, x, 0, ids, w, t, L->top_k, 0, 1, out, ex_ws, flag, s);
    if (st) return st;
    if (ids_out) LMOE_CUDA(cudaMemcpyAsync(ids_out, ids, (size_t)rows * 4, cudaMemcpyDeviceToDevice, s));
    if (w_out) LMOE_CUDA(cudaMemcpyAsync(w_out, w, (size_t)rows * 4, cudaMemcpyDeviceToDevice, s));
    return LMOE_OK;
}

// `ExpertFfn::forward` on the grouped-GEMM path (see lmoe_experts_forward): the caller's routing decision.
size_t experts_prefill_workspace_bytes(const lmoe_layer *L, int64_t t) {
    return 65536 + experts_ws_bytes(L, t < 1 ? 1 : t, L->top_k);
}
lmoe_status launch_experts_prefill(const lmoe_layer *L, const float *x, const uint32_t *ids, const float *w, int64_t t,
                                   int add_shared, float *out, void *workspace, size_t workspace_bytes, cudaStream_t s) {
    if (!layer_mm_ok(L)) return lmoe_fail(LMOE_ERR_UNSUPPORTED, "no grouped-GEMM kernel for this layer's shapes / dtypes");
    if (!workspace || workspace_bytes < experts_prefill_workspace_bytes(L, t))
        return lmoe_fail(LMOE_ERR_WORKSPACE, "workspace needs %zu bytes, got %zu", experts_prefill_workspace_bytes(L, t),
                         workspace_bytes);
    if (t * L->top_k > INT32_MAX / 2) return lmoe_fail(LMOE_ERR_INVALID, "too many routed rows");
    uint32_t *flag = reinterpret_cast<uint32_t *>(workspace);
    LMOE_CUDA(cudaMemsetAsync(flag, 0, 16, s));
    return experts_prefill(L, x, 0, ids, w, t, L->top_k, 1, add_shared, out, static_cast<uint8_t *>(workspace) + 65536, flag, s);
}

// ---- op-level entry points ------------------------------------------------------------
extern "C" int32_t lmoe_mm_id_supported(int32_t dtype, int64_t top_k) {
    return (dtype == LMOE_Q4_K || dtype == LMOE_Q6_K) && top_k >= 1 ? 1 : 0;
}

extern "C" size_t lmoe_mm_id_workspace_bytes(const lmoe_expert_stack *stack, int64_t t, int64_t top_k, int64_t x_per_row) {
    if (!stack || t < 0 || top_k < 1 || x_per_row < 1) return 0;
    return 256 + mm_tiled_bytes(t * top_k, stack->n_expert, stack->k) +
           mm_tiles_bytes(t * top_k, stack->n_expert, stack->n_out);
}

static lmoe_status mm_id_run(const lmoe_expert_stack *stack, const float *x, int64_t t, int64_t x_per_row, int64_t k,
                             const uint32_t *ids, int64_t t_ids, int64_t top_k, const void *map0, float *out,
                             void *workspace, size_t workspace_bytes, cudaStream_t s) {
    lmoe_status st = lmoe_id_shape_check(stack, x, t, x_per_row, k, ids, t_ids, top_k, out);
    if (st) return st;
    if (!mm_id_kernel_available(stack->dtype, stack->n_out, stack->k))
        return lmoe_fail(LMOE_ERR_UNSUPPORTED, "no grouped-GEMM kernel for dtype %d, n_out %lld, k %lld", stack->dtype,
                         (long long)stack->n_out, (long long)stack->k);
    const size_t need = lmoe_mm_id_workspace_bytes(stack, t, top_k, x_per_row);
    if (!workspace || workspace_bytes < need)
        return lmoe_fail(LMOE_ERR_WORKSPACE, "mul_mm_id workspace needs %zu bytes, got %zu", need, workspace_bytes);
    if (t == 0) return LMOE_OK;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    uint32_t *flag = reinterpret_cast<uint32_t *>(ws);
    uint8_t *xt = ws + 256;
    void *tiles = ws + 256 + mm_tiled_bytes(t * top_k, stack->n_expert, k);
    LMOE_CUDA(cudaMemsetAsync(flag, 0, 16, s));
    const uint32_t *tpe = static_cast<const uint32_t *>(map0);
    const int32_t *ids_map = reinterpret_cast<const int32_t *>(static_cast<const uint8_t *>(map0) + stack->n_expert * 4);
    LMOE_CUDA(launch_gather_tiles(x, 0, (int)x_per_row, (int)top_k, (int)k, tpe, ids_map, (int)t, (int)stack->n_expert, xt,
                                  nullptr, nullptr, nullptr, s));
    return launch_mm_id(stack, xt, tpe, ids_map, t, t * top_k, nullptr, out, tiles, flag, s);
}

extern "C" lmoe_status lmoe_mul_mm_id_shared(const lmoe_expert_stack *stack, const float *x, int64_t t, int64_t x_per_row,
                                             int64_t k, const uint32_t *ids, int64_t t_ids, int64_t top_k,
                                             const void *map0_scratch, int64_t map_n_expert, int64_t map_t,
                                             int64_t map_top_k, float *out, void *workspace, size_t workspace_bytes,
                                             void *stream) {
    lmoe_clear_error();
    if (!stack) return lmoe_fail(LMOE_ERR_INVALID, "expert stack is NULL");
    if (!map0_scratch) return lmoe_fail(LMOE_ERR_INVALID, "map0 scratch is NULL");
    // the consumer re-validates the producer's geometry, src/ops/dispatch.rs:903-909
    if (map_n_expert != stack->n_expert || map_t != t || map_top_k != top_k)
        return lmoe_fail(LMOE_ERR_INVALID,
                         "shared map0 scratch geometry (n_expert=%lld, t=%lld, top_k=%lld) does not match this projection "
                         "(n_expert=%lld, t=%lld, top_k=%lld); the ids-map offset would be wrong",
                         (long long)map_n_expert, (long long)map_t, (long long)map_top_k, (long long)stack->n_expert,
                         (long long)t, (long long)top_k);
    return mm_id_run(stack, x, t, x_per_row, k, ids, t_ids, top_k, map0_scratch, out, workspace, workspace_bytes,
                     (cudaStream_t)stream);
}

extern "C" lmoe_status lmoe_mul_mm_id(const lmoe_expert_stack *stack, const float *x, int64_t t, int64_t x_per_row,
                                      int64_t k, const uint32_t *ids, int64_t t_ids, int64_t top_k, float *out,
                                      void *workspace, size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    if (!stack) return lmoe_fail(LMOE_ERR_INVALID, "expert stack is NULL");
    lmoe_status st = lmoe_id_shape_check(stack, x, t, x_per_row, k, ids, t_ids, top_k, out);
    if (st) return st;
    const size_t mm = lmoe_mm_id_workspace_bytes(stack, t, top_k, x_per_row), mp = lmoe_map0_scratch_bytes(stack->n_expert, t);
    if (!workspace || workspace_bytes < mm + mp)
        return lmoe_fail(LMOE_ERR_WORKSPACE, "mul_mm_id workspace needs %zu bytes, got %zu", mm + mp, workspace_bytes);
    uint8_t *map0 = static_cast<uint8_t *>(workspace) + mm;
    LMOE_CUDA(launch_map0(ids, (int)t, (int)top_k, (int)stack->n_expert, reinterpret_cast<uint32_t *>(map0),
                          reinterpret_cast<int32_t *>(map0 + stack->n_expert * 4), (cudaStream_t)stream));
    return mm_id_run(stack, x, t, x_per_row, k, ids, t_ids, top_k, map0, out, workspace, mm, (cudaStream_t)stream);
}

// ---- expert-parallel pieces -------------------------------------------------------------
static size_t rows_ws_bytes(const lmoe_layer *L, int64_t rows) {
    return 65536 + lmoe_map0_scratch_bytes(L->n_expert, rows) + lmoe_align_up((size_t)(rows + 64) * 4, 256) +
           ffn_bytes(rows, L->hidden, L->expert_ff, L->n_expert);
}

static lmoe_status experts_rows_run(const lmoe_layer *L, const void *x, int x_f16, const uint32_t *local_ids,
                                    const float *row_weights, int64_t rows, float *out, void *workspace,
                                    size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    if (!L || !x || !local_ids || !out) return lmoe_fail(LMOE_ERR_INVALID, "layer/x/local_ids/out is NULL");
    if (rows < 0 || rows > INT32_MAX / 2) return lmoe_fail(LMOE_ERR_INVALID, "rows out of range");
    if (rows == 0) return LMOE_OK;
    if (reinterpret_cast<uintptr_t>(x) & 15u) return lmoe_fail(LMOE_ERR_INVALID, "x must be 16-byte aligned");
    if (!layer_mm_ok(L)) return lmoe_fail(LMOE_ERR_UNSUPPORTED, "no grouped-GEMM kernel for this layer's shapes / dtypes");
    if (!workspace || workspace_bytes < rows_ws_bytes(L, rows))
        return lmoe_fail(LMOE_ERR_WORKSPACE, "workspace needs %zu bytes, got %zu", rows_ws_bytes(L, rows), workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    Carver c{static_cast<uint8_t *>(workspace), 65536};
    uint32_t *flag = reinterpret_cast<uint32_t *>(workspace);
    uint8_t *map0 = c.take<uint8_t>(lmoe_map0_scratch_bytes(L->n_expert, rows));
    uint8_t *ffn_ws = static_cast<uint8_t *>(workspace) + c.off;
    uint32_t *tpe = reinterpret_cast<uint32_t *>(map0);
    int32_t *ids_map = reinterpret_cast<int32_t *>(map0 + L->n_expert * 4);
    LMOE_CUDA(cudaMemsetAsync(flag, 0, 16, s));
    LMOE_CUDA(launch_map0(local_ids, (int)rows, 1, (int)L->n_expert, tpe, ids_map, s));
    return ffn_grouped(L->gate, L->up, L->down, x, 1, rows, tpe, ids_map, rows, row_weights, out, ffn_ws, flag, s, nullptr,
                       nullptr, nullptr, x_f16);
}

extern "C" lmoe_status lmoe_experts_forward_rows(const lmoe_layer *L, const float *x, const uint32_t *local_ids,
                                                 const float *row_weights, int64_t rows, float *out, void *workspace,
                                                 size_t workspace_bytes, void *stream) {
    return experts_rows_run(L, x, 0, local_ids, row_weights, rows, out, workspace, workspace_bytes, stream);
}

extern "C" lmoe_status lmoe_experts_forward_rows_f16(const lmoe_layer *L, const void *x_f16, const uint32_t *local_ids,
                                                     const float *row_weights, int64_t rows, float *out, void *workspace,
                                                     size_t workspace_bytes, void *stream) {
    return experts_rows_run(L, x_f16, 1, local_ids, row_weights, rows, out, workspace, workspace_bytes, stream);
}

// Token-level form for the expert-parallel exchange: one activation row per token, up to top_k experts each.
static size_t tokens_ws_bytes(const lmoe_layer *L, int64_t t, int64_t top_k) {
    return 65536 + experts_ws_bytes(L, t, top_k);
}

extern "C" size_t lmoe_tokens_workspace_bytes(const lmoe_layer *L, int64_t t, int64_t top_k) {
    return L && top_k >= 1 ? tokens_ws_bytes(L, t < 1 ? 1 : t, top_k) : 0;
}

extern "C" lmoe_status lmoe_experts_forward_tokens_f16(const lmoe_layer *L, const void *x_f16, const uint32_t *ids,
                                                       const float *weights, int64_t t, int64_t top_k, float *out,
                                                       void *workspace, size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    if (!L || !x_f16 || !ids || !weights || !out) return lmoe_fail(LMOE_ERR_INVALID, "layer/x/ids/weights/out is NULL");
    if (top_k < 1 || t < 0 || t * top_k > INT32_MAX / 2) return lmoe_fail(LMOE_ERR_INVALID, "t / top_k out of range");
    if (t == 0) return LMOE_OK;
    if ((reinterpret_cast<uintptr_t>(x_f16) | reinterpret_cast<uintptr_t>(out)) & 15u)
        return lmoe_fail(LMOE_ERR_INVALID, "x and out must be 16-byte aligned");
    if (!layer_mm_ok(L)) return lmoe_fail(LMOE_ERR_UNSUPPORTED, "no grouped-GEMM kernel for this layer's shapes / dtypes");
    if (!workspace || workspace_bytes < tokens_ws_bytes(L, t, top_k))
        return lmoe_fail(LMOE_ERR_WORKSPACE, "workspace needs %zu bytes, got %zu", tokens_ws_bytes(L, t, top_k), workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    uint32_t *flag = reinterpret_cast<uint32_t *>(workspace);
    LMOE_CUDA(cudaMemsetAsync(flag, 0, 16, s));
    return experts_prefill(L, x_f16, 1, ids, weights, t, top_k, 1, 0, out, static_cast<uint8_t *>(workspace) + 65536, flag, s);
}

extern "C" lmoe_status lmoe_shared_forward(const lmoe_layer *L, const float *x, int64_t t, float *out, void *workspace,
                                           size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    if (!L || !x || !out) return lmoe_fail(LMOE_ERR_INVALID, "layer/x/out is NULL");
    if (!L->sh_gate) return lmoe_fail(LMOE_ERR_INVALID, "the layer has no shared expert");
    if (t < 0 || t > INT32_MAX / 2) return lmoe_fail(LMOE_ERR_INVALID, "t out of range");
    if (t == 0) return LMOE_OK;
    if (!layer_mm_ok(L)) return lmoe_fail(LMOE_ERR_UNSUPPORTED, "no grouped-GEMM kernel for this layer's shapes / dtypes");
    if (!workspace || workspace_bytes < rows_ws_bytes(L, t))
        return lmoe_fail(LMOE_ERR_WORKSPACE, "workspace needs %zu bytes, got %zu", rows_ws_bytes(L, t), workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    Carver c{static_cast<uint8_t *>(workspace), 65536};
    uint32_t *flag = reinterpret_cast<uint32_t *>(workspace);
    uint32_t *list = c.take<uint32_t>((size_t)t + 64);
    uint8_t *ffn_ws = static_cast<uint8_t *>(workspace) + c.off;
    LMOE_CUDA(cudaMemsetAsync(flag, 0, 16, s));
    iota_list_kernel<<<(unsigned)((t + 255) / 256), 256, 0, s>>>(t, list, reinterpret_cast<int32_t *>(list + 64));
    LMOE_LAUNCH_CHECK("iota_list_kernel");
    return ffn_grouped(L->sh_gate, L->sh_up, L->sh_down, x, 1, t, list, reinterpret_cast<int32_t *>(list + 64), t, nullptr,
                       out, ffn_ws, flag, s);
}

extern "C" size_t lmoe_rows_workspace_bytes(const lmoe_layer *L, int64_t rows) {
    return L ? rows_ws_bytes(L, rows < 1 ? 1 : rows) : 0;
}

// Expert-parallel exchange helpers (no counterpart in the single-GPU reference).
extern "C" size_t lmoe_ep_pack_workspace_bytes(int64_t n_expert, int64_t t) { return lmoe_map0_scratch_bytes(n_expert, t); }

extern "C" lmoe_status lmoe_ep_pack(const float *x, const uint32_t *ids, const float *weights, int64_t t, int64_t hidden,
                                    int64_t top_k, int64_t n_expert, int64_t world, void *rows_f16, uint32_t *local_ids,
                                    float *row_weights, int32_t *row_pos, int64_t *send_counts, void *workspace,
                                    size_t workspace_bytes, void *stream) {
    lmoe_clear_error();
    if (!x || !ids || !weights || !rows_f16 || !local_ids || !row_weights || !row_pos || !send_counts)
        return lmoe_fail(LMOE_ERR_INVALID, "ep_pack: a buffer is NULL");
    if (t < 0 || top_k < 1 || n_expert < 1 || world < 1 || n_expert % world || hidden < 8 || hidden % 8)
        return lmoe_fail(LMOE_ERR_INVALID, "ep_pack: t >= 0, top_k >= 1, n_expert divisible by world, hidden a multiple of 8 required");
    if (t * top_k > INT32_MAX / 2 || n_expert > 65535) return lmoe_fail(LMOE_ERR_INVALID, "ep_pack: problem too large");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(rows_f16)) & 15u)
        return lmoe_fail(LMOE_ERR_INVALID, "ep_pack: x and rows_f16 must be 16-byte aligned");
    if (!workspace || workspace_bytes < lmoe_map0_scratch_bytes(n_expert, t))
        return lmoe_fail(LMOE_ERR_WORKSPACE, "ep_pack workspace needs %zu bytes, got %zu", lmoe_map0_scratch_bytes(n_expert, t),
                         workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    uint32_t *tpe = static_cast<uint32_t *>(workspace);
    int32_t *ids_map = reinterpret_cast<int32_t *>(static_cast<uint8_t *>(workspace) + n_expert * 4);
    LMOE_CUDA(launch_map0(ids, (int)t, (int)top_k, (int)n_expert, tpe, ids_map, s));
    const int e_local = (int)(n_expert / world);
    ep_counts_kernel<<<(unsigned)world, 32, 0, s>>>(tpe, (int)n_expert, e_local, reinterpret_cast<long long *>(send_counts));
    LMOE_LAUNCH_CHECK("ep_counts_kernel");
    if (t > 0) {
        const int gy = n_expert >= 64 ? 16 : (n_expert >= 8 ? 128 : 1024);
        ep_pack_kernel<<<dim3((unsigned)n_expert, gy), 256, 0, s>>>(x, weights, tpe, ids_map, (int)t, (int)top_k, (int)hidden, e_local,
                                                                static_cast<__half *>(rows_f16), local_ids, row_weights, row_pos);
        LMOE_LAUNCH_CHECK("ep_pack_kernel");
    }
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_ep_localize_ids(const uint32_t *ids, int64_t n, int64_t first, int64_t count, uint32_t *out,
                                            void *stream) {
    lmoe_clear_error();
    if (!ids || !out) return lmoe_fail(LMOE_ERR_INVALID, "ep_localize_ids: ids/out is NULL");
    if (n < 0 || first < 0 || count < 1 || first + count > (int64_t)UINT32_MAX)
        return lmoe_fail(LMOE_ERR_INVALID, "ep_localize_ids: n >= 0, first >= 0, count >= 1 required");
    LMOE_CUDA(launch_ep_localize_ids(ids, n, (uint32_t)first, (uint32_t)count, out, (cudaStream_t)stream));
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_ep_combine(const float *rows, const int32_t *row_pos, const float *shared, int64_t t,
                                       int64_t top_k, int64_t hidden, float *out, void *stream) {
    lmoe_clear_error();
    if (!rows || !row_pos || !out) return lmoe_fail(LMOE_ERR_INVALID, "ep_combine: rows/row_pos/out is NULL");
    if (t < 0 || top_k < 1 || hidden < 4 || hidden % 4) return lmoe_fail(LMOE_ERR_INVALID, "ep_combine: bad dimensions");
    if ((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(shared)) & 15u)
        return lmoe_fail(LMOE_ERR_INVALID, "ep_combine: rows, shared and out must be 16-byte aligned");
    if (t == 0) return LMOE_OK;
    const int64_t n = t * (hidden / 4);
    sum_sorted_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(rows, nullptr, row_pos, shared, nullptr, nullptr,
                                                                               t, (int)top_k, (int)(hidden / 4), out);
    LMOE_LAUNCH_CHECK("sum_sorted_kernel");
    return LMOE_OK;
}
