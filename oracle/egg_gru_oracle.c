/*
 * egg_gru_oracle.c — CPU restatement of the reference's CPU trainer full_trained_egg.c (the
 * recurrent GRU + MLP model), run-time sized.  TEST INFRASTRUCTURE ONLY: the checker the CUDA
 * path of this model is compared against; never linked into or called by the library.
 *
 * Pinned against the reference itself: oracle/_ref/ref_cpu_gru is full_trained_egg.c lines 1-476
 * compiled unmodified; tests/test_gru_cpu.py runs both on the same seeded case and compares
 * losses, fitness, recurrent states and post-update weights bit for bit.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "egg_oracle.h"

/* full_trained_egg.c:70-82 */
static inline uint32_t gru_xorshift32(uint32_t *st) {
    uint32_t x = *st;
    x ^= x << 13; x ^= x >> 17; x ^= x << 5;
    *st = x;
    return x;
}
static inline int gru_noise_val(uint32_t *st) {
    uint32_t r = gru_xorshift32(st);
    int mag = (int)((r >> 1) & 31u);
    return (r & 1u) ? mag : -mag;
}
/* full_trained_egg.c:88-104: four draws are thrown away in front of every block of 16 values */
static void gru_noise_vector(uint32_t *st, int8_t *out, int count) {
    for (int i = 0; i < count; i += 16) {
        for (int b = 0; b < 4; b++) (void)gru_xorshift32(st);
        for (int j = i; j < i + 16 && j < count; j++) out[j] = (int8_t)gru_noise_val(st);
    }
}

static inline int gru_clip(int v) { return v > 127 ? 127 : (v < -127 ? -127 : v); }

typedef struct {
    int64_t embedding, gru_w, gru_b, mlp_w, head, ln_w, ln_out, total;
} gru_layout;

/* EggModel, full_trained_egg.c:42-50 */
static gru_layout gru_layout_of(const egg_gru_config *c) {
    gru_layout L;
    int64_t H = c->hidden_dim, V = c->vocab_size, NL = c->n_layers, o = 0;
    L.embedding = o; o += V * H;
    L.gru_w = o;     o += NL * 4 * H * H;
    L.gru_b = o;     o += NL * 2 * H;
    L.mlp_w = o;     o += NL * 2 * 4 * H * H;
    L.head = o;      o += H * V;
    L.ln_w = o;      o += NL * 2 * H;
    L.ln_out = o;    o += H;
    L.total = o;
    return L;
}

int64_t oracle_gru_model_bytes(const egg_gru_config *c) { return gru_layout_of(c).total; }

/* main(), full_trained_egg.c:491-515: the reference's own initial weights */
void oracle_gru_init_model(const egg_gru_config *c, int8_t *model, uint32_t seed) {
    gru_layout L = gru_layout_of(c);
    int64_t H = c->hidden_dim, V = c->vocab_size;
    memset(model, 0, (size_t)L.total);
    uint32_t rng = seed;
    for (int64_t i = 0; i < V * H; i++) model[L.embedding + i] = (int8_t)gru_noise_val(&rng);
    for (int64_t i = 0; i < V * H; i++) model[L.head + i] = (int8_t)gru_noise_val(&rng);
    for (int l = 0; l < c->n_layers; l++) {
        for (int64_t i = 0; i < 4 * H * H; i++) model[L.gru_w + (int64_t)l * 4 * H * H + i] = (int8_t)gru_noise_val(&rng);
        for (int64_t i = 0; i < 8 * H * H; i++) model[L.mlp_w + (int64_t)l * 8 * H * H + i] = (int8_t)gru_noise_val(&rng);
    }
    for (int64_t i = 0; i < 2 * H * c->n_layers; i++) model[L.ln_w + i] = 16;
    for (int64_t i = 0; i < H; i++) model[L.ln_out + i] = 16;
}

/* matmul_perturbed, full_trained_egg.c:108-177: out[r] = clip((in·w[r] + ((xB*A[r]*sign) >> (FP+SS))) >> shift),
 * A (rows) then B (cols) drawn from one stream seeded with layer_seed */
static void gru_matmul(const egg_gru_config *c, const int8_t *in, const int8_t *w, int8_t *out, int rows, int cols,
                       uint32_t seed, int sign, int shift) {
    int8_t *A = (int8_t *)malloc((size_t)rows), *B = (int8_t *)malloc((size_t)cols);
    uint32_t rng = seed;
    gru_noise_vector(&rng, A, rows);
    gru_noise_vector(&rng, B, cols);
    int32_t xB = 0;
    for (int k = 0; k < cols; k++) xB += (int32_t)in[k] * B[k];
    for (int r = 0; r < rows; r++) {
        int32_t acc = 0;
        const int8_t *wr = w + (int64_t)r * cols;
        for (int k = 0; k < cols; k++) acc += (int32_t)in[k] * wr[k];
        if (sign != 0) acc += ((xB * (int32_t)A[r]) * sign) >> (c->fixed_point + c->sigma_shift);
        out[r] = (int8_t)gru_clip(acc >> shift);
    }
    free(A); free(B);
}

/* egg_ln, full_trained_egg.c:180-210 (no noise, no bias) */
static void gru_ln(const int8_t *x, const int8_t *w, int8_t *out, int H) {
    int32_t sum = 0;
    for (int i = 0; i < H; i++) sum += abs((int)x[i]);
    if (sum == 0) sum = 1;
    int32_t mean = sum / H;
    if (mean == 0) mean = 1;
    for (int i = 0; i < H; i++) out[i] = (int8_t)gru_clip(((int32_t)x[i] * w[i]) / mean);
}

/* compute_loss / log2_fixed, full_trained_egg.c:298-330 */
static int32_t gru_loss(const int32_t *exp2_table, const int8_t *logits, int V, int target) {
    int32_t sum_exp = 0;
    for (int i = 0; i < V; i++) sum_exp += exp2_table[(int)logits[i] + 128];
    int32_t log_sum = 0;
    if (sum_exp > 0) {
        int k = 31 - __builtin_clz((uint32_t)sum_exp);
        int32_t frac = k >= 4 ? (sum_exp - (1 << k)) >> (k - 4) : (sum_exp - (1 << k)) << (4 - k);
        log_sum = (k << 4) + frac - 64;
    }
    return log_sum - ((int32_t)logits[target] + 128);
}

void oracle_gru_exp2_table(const egg_gru_config *c, int32_t *table256) {     /* init_tables, :58-61 */
    for (int i = 0; i < 256; i++)
        table256[i] = (int32_t)(pow(2.0, (double)i / (1 << c->fixed_point)) * (1 << c->fixed_point));
}

/* forward_pass, full_trained_egg.c:212-296; state = h[n_layers][H] of this member, carried over */
static int32_t gru_forward(const egg_gru_config *c, const gru_layout *L, const int8_t *M, const int32_t *exp2_table,
                           const uint8_t *inputs, const uint8_t *targets, int tokens, uint32_t p_seed, int sign,
                           int8_t *state, int8_t *logits_out) {
    const int H = c->hidden_dim, V = c->vocab_size;
    int8_t *x = malloc((size_t)H), *res = malloc((size_t)H), *b1 = malloc((size_t)4 * H), *b2 = malloc((size_t)H),
           *ft = malloc((size_t)H), *gp = malloc((size_t)H), *ht = malloc((size_t)H), *lg = malloc((size_t)V);
    int32_t loss = 0;
    for (int t = 0; t < tokens; t++) {
        memcpy(x, M + L->embedding + (int64_t)inputs[t] * H, (size_t)H);
        for (int l = 0; l < c->n_layers; l++) {
            uint32_t ls = p_seed + (uint32_t)(l * 100);
            const int8_t *gw = M + L->gru_w + (int64_t)l * 4 * H * H, *gb = M + L->gru_b + (int64_t)l * 2 * H;
            const int8_t *mw = M + L->mlp_w + (int64_t)l * 8 * H * H, *lw = M + L->ln_w + (int64_t)l * 2 * H;
            int8_t *h = state + (int64_t)l * H;
            memcpy(res, x, (size_t)H);
            gru_ln(x, lw, x, H);
            gru_matmul(c, x, gw, b1, H, H, ls + 1, sign, 8);
            gru_matmul(c, h, gw + (int64_t)H * H, b2, H, H, ls + 2, sign, 8);
            for (int i = 0; i < H; i++) ft[i] = (int8_t)gru_clip(gru_clip(b1[i] + b2[i]) + gb[i]);
            for (int i = 0; i < H; i++) gp[i] = (int8_t)((((int32_t)ft[i] + 127) * h[i]) >> 8);
            gru_matmul(c, x, gw + 2 * (int64_t)H * H, b1, H, H, ls + 3, sign, 8);
            gru_matmul(c, gp, gw + 3 * (int64_t)H * H, b2, H, H, ls + 4, sign, 8);
            for (int i = 0; i < H; i++) ht[i] = (int8_t)gru_clip(gru_clip(b1[i] + b2[i]) + gb[H + i]);
            for (int i = 0; i < H; i++) {
                int32_t upd = (((int32_t)ft[i] + 127) * ((int32_t)ht[i] - h[i])) >> 8;
                h[i] = (int8_t)gru_clip(h[i] + upd);
                x[i] = (int8_t)gru_clip(h[i] + res[i]);
            }
            memcpy(res, x, (size_t)H);
            gru_ln(x, lw + H, x, H);
            gru_matmul(c, x, mw, b1, 4 * H, H, ls + 5, sign, 8);
            gru_matmul(c, b1, mw + 4 * (int64_t)H * H, x, H, 4 * H, ls + 6, sign, 9);
            for (int i = 0; i < H; i++) x[i] = (int8_t)gru_clip(x[i] + res[i]);
        }
        gru_ln(x, M + L->ln_out, x, H);
        gru_matmul(c, x, M + L->head, lg, V, H, p_seed + 999, sign, 8);
        if (targets) loss += gru_loss(exp2_table, lg, V, targets[t]);
    }
    if (logits_out) memcpy(logits_out, lg, (size_t)V);
    free(x); free(res); free(b1); free(b2); free(ft); free(gp); free(ht); free(lg);
    return loss;
}

/* update_matrix, full_trained_egg.c:332-409: vote = Σ_p (int8)(A_p[r]*f_p) * B_p[c]; one step of ±1 beyond the
 * threshold.  Pairs with f = 0 contribute nothing (their A column is zero; their B column is left stale, which
 * cannot matter because it is multiplied by zero). */
static void gru_update_matrix(const egg_gru_config *c, int8_t *W, int rows, int cols, uint32_t seed, const int32_t *fit) {
    const int pairs = c->population_size / 2;
    int8_t *At = calloc((size_t)rows * pairs, 1), *Bt = calloc((size_t)cols * pairs, 1);
    int8_t *a = malloc((size_t)rows), *b = malloc((size_t)cols);
    for (int p = 0; p < pairs; p++) {
        uint32_t rng = seed + (uint32_t)p;
        gru_noise_vector(&rng, a, rows);
        gru_noise_vector(&rng, b, cols);
        if (fit[p] == 0) continue;
        for (int r = 0; r < rows; r++) At[(int64_t)r * pairs + p] = (int8_t)(a[r] * fit[p]);
        for (int k = 0; k < cols; k++) Bt[(int64_t)k * pairs + p] = b[k];
    }
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++)
        for (int k = 0; k < cols; k++) {
            int32_t vote = 0;
            for (int p = 0; p < pairs; p++) vote += (int32_t)At[(int64_t)r * pairs + p] * Bt[(int64_t)k * pairs + p];
            int8_t *w = &W[(int64_t)r * cols + k];
            if (vote > c->update_threshold && *w < 127) (*w)++;
            else if (vote < -c->update_threshold && *w > -127) (*w)--;
        }
    free(At); free(Bt); free(a); free(b);
}

/* One iteration of the training loop, full_trained_egg.c:529-575.  states: [population][n_layers][H], carried. */
void oracle_gru_generation(const egg_gru_config *c, int8_t *model, int8_t *states, const uint8_t *data, int64_t data_len,
                           uint32_t step_seed, int64_t start_idx, int tokens, int do_update, int32_t *losses,
                           int32_t *fitness) {
    const gru_layout L = gru_layout_of(c);
    const int H = c->hidden_dim, pairs = c->population_size / 2;
    int32_t exp2_table[256];
    oracle_gru_exp2_table(c, exp2_table);
    const int64_t stride = data_len / pairs;
#pragma omp parallel for schedule(dynamic, 1)
    for (int m = 0; m < 2 * pairs; m++) {
        const int p = m >> 1;
        const int64_t pos = (start_idx + (int64_t)p * stride) % (data_len - c->seq_len);
        losses[m] = gru_forward(c, &L, model, exp2_table, data + pos, data + pos + 1, tokens, step_seed + (uint32_t)p,
                                (m & 1) ? -1 : 1, states + (int64_t)m * c->n_layers * H, NULL);
    }
    for (int p = 0; p < pairs; p++)
        fitness[p] = losses[2 * p] < losses[2 * p + 1] ? 1 : (losses[2 * p + 1] < losses[2 * p] ? -1 : 0);
    if (!do_update) return;
    for (int l = 0; l < c->n_layers; l++) {
        uint32_t ls = step_seed + (uint32_t)(l * 100);
        int8_t *gw = model + L.gru_w + (int64_t)l * 4 * H * H, *mw = model + L.mlp_w + (int64_t)l * 8 * H * H;
        for (int g = 0; g < 4; g++) gru_update_matrix(c, gw + (int64_t)g * H * H, H, H, ls + 1 + (uint32_t)g, fitness);
        gru_update_matrix(c, mw, 4 * H, H, ls + 5, fitness);
        gru_update_matrix(c, mw + 4 * (int64_t)H * H, H, 4 * H, ls + 6, fitness);
    }
    gru_update_matrix(c, model + L.head, c->vocab_size, H, step_seed + 999, fitness);
}
