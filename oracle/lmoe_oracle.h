/*
 * Declarations shared by the two units of the CPU oracle -- TEST INFRASTRUCTURE ONLY
 * (see lmoe_oracle.c for what may use it).
 */
#ifndef LMOE_ORACLE_H
#define LMOE_ORACLE_H

#include <stdint.h>

#define QK_K 256
#define Q4K_BYTES 144
#define Q6K_BYTES 210

enum { LMO_Q4_K = 12, LMO_Q6_K = 14 }; /* ggml type ids */

typedef struct {
    int hidden, expert_ff, n_expert, top_k;
    float scale;
    int norm;
    const float *router;   /* [n_expert, hidden] */
    const float *bias;     /* [n_expert] */
    const uint8_t *gate;   /* Q4_K [n_expert, expert_ff, hidden] */
    const uint8_t *up;     /* Q4_K [n_expert, expert_ff, hidden] */
    const uint8_t *down;   /* Q6_K [n_expert, hidden, expert_ff] */
    const uint8_t *sh_gate; /* Q4_K [expert_ff, hidden] or NULL */
    const uint8_t *sh_up;
    const uint8_t *sh_down; /* Q6_K [hidden, expert_ff] */
    int gate_dtype, down_dtype;
} lmo_layer;

/* 6-bit (scale, min) pair j of a Q4_K super-block; src/ops/mm_id.metal:89-92
 * decodes the same packing two at a time. */
static inline void q4k_scale_min(const uint8_t *s, int j, int *sc, int *mn) {
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (s[j + 4] & 0x0f) | ((s[j - 4] >> 6) << 4);
        *mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

float lmo_h2f(uint16_t h);
int lmo_type_size(int dtype);
void lmo_route(const float *router, const float *bias, const float *x, int t, int hidden, int n_expert,
               int top_k, float scale, int norm, uint32_t *ids, float *weights);

#endif /* LMOE_ORACLE_H */
