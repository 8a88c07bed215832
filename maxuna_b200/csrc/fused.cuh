// Whole-block entry points: workspace layout and device flag codes.
#pragma once

#include "common.cuh"

// Device flag word (first 16 bytes of every workspace): [0] code, [1..3] detail.
enum {
    LMOE_FLAG_BAD_EXPERT_ID = 0x1,
    LMOE_FLAG_WAIT_TIMEOUT = 0x2,
    LMOE_FLAG_BAD_INDEX = 0x4,
};

// seam checks shared by the mat-vec and grouped-GEMM entry points (api.cu)
lmoe_status lmoe_id_shape_check(const lmoe_expert_stack *stack, const void *x, int64_t t, int64_t x_per_row,
                                int64_t k, const void *ids, int64_t t_ids, int64_t top_k, const void *out);

// Routed rows per tile of the grouped GEMMs (the N extent of one tensor-core tile).  192, not 256: the gate/up
// kernel keeps its dequantised weight operand in tensor memory beside the two accumulators, and
// 2 x 192 accumulator columns + 128 operand columns fill the 512 columns of an SM.  The tile-ordered
// activation operand in global memory is laid out in row tiles of this size.
constexpr int LMOE_MM_N = 192;
