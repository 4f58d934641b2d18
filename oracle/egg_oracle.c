/*
 * egg_oracle.c — CPU restatement of the reference's EGGROLL hot path.
 *
 * TEST INFRASTRUCTURE ONLY (see egg_oracle.h).  Member-major, token-serial,
 * scalar C: deliberately the reference's own loop structure, so that it
 * cross-checks the layer-major batched CUDA path structurally as well as
 * numerically.  "mgpu.cu" = full_cuda_train_transformer_adam_mgpu.cu.
 *
 * Parity status: pinned by RNG known answers from the reference's egg_math.h,
 * by the ternary codec cases of d-eggs/test_ternary.cpp, and by golden
 * outputs of the reference's own kernels (tests/golden/).  The Muon
 * Newton–Schulz step is "parity unpinned" bit-wise: the reference computes it
 * with cuBLAS SGEMM, whose summation order is not specified; it is compared at
 * 1e-5 relative.
 */
#include "egg_oracle.h"

#include <limits.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ RNG */

/* mgpu.cu:525-527 */
uint32_t oracle_hash_rng(uint32_t s, uint32_t idx) {
    uint32_t x = s + idx * 0x9e3779b9u;
    x ^= x >> 16; x *= 0x85ebca6bu;
    x ^= x >> 13; x *= 0xc2b2ae35u;
    x ^= x >> 16;
    return x;
}

static inline int noise_field(uint32_t r, int sign_bit, int shift, int mask) {
    int mag = (int)((r >> shift) & (uint32_t)mask);
    return (r & (1u << sign_bit)) ? mag : -mag;
}

/* mgpu.cu:528-538 (the int8 casts there never truncate for mask <= 31) */
int oracle_noise(const egg_config *cfg, uint32_t s, uint32_t idx) {
    uint32_t r = oracle_hash_rng(s, idx);
    if (cfg->device_gaussian) {
        int n = noise_field(r, 0, 1, cfg->device_mask) + noise_field(r, 5, 6, cfg->device_mask) +
                noise_field(r, 10, 11, cfg->device_mask);
        return (int)(int8_t)n;
    }
    return noise_field(r, 0, 1, cfg->device_mask);
}

/* mgpu.cu:428-441 (HOST_GAUSSIAN=false path) */
int oracle_gen_noise_host(const egg_config *cfg, uint32_t *state) {
    uint32_t x = *state;
    x ^= x << 13; x ^= x >> 17; x ^= x << 5;
    *state = x;
    return noise_field(x, 0, 1, cfg->host_mask);
}

static inline int clip8(int64_t a) { return a > 127 ? 127 : (a < -127 ? -127 : (int)a); }

/* --------------------------------------------------------------- layout */

typedef struct {
    int64_t embedding, emb_bias, ntt_emb /* three V*H tables in a row, present when ntt_mode != 0 */, ln_init, ln_init_bias,
        w_emb_mlp_up, mlp_emb_bias_up,
        w_emb_mlp_down, mlp_emb_bias_down, ln_1, ln_1_bias, w_q, w_k, w_v, w_o, ln_2,
        ln_2_bias, w_up, mlp_bias_up, w_down, mlp_bias_down, ln_f, ln_f_bias, total;
} model_layout;

/* Field order of TransformerModel (mgpu.cu:284-318). Offsets in elements. */
static void layout_of(const egg_config *c, model_layout *L) {
    int64_t H = c->hidden_dim, V = c->vocab_size, NL = c->n_layers, o = 0;
    L->embedding = o;        o += V * H;
    L->emb_bias = o;         o += H;
    L->ntt_emb = o;          o += c->ntt_mode ? 3 * V * H : 0;     /* ntt_emb1..3, mgpu.cu:288-293 */
    L->ln_init = o;          o += H;
    L->ln_init_bias = o;     o += H;
    L->w_emb_mlp_up = o;     o += H * 4 * H;
    L->mlp_emb_bias_up = o;  o += 4 * H;
    L->w_emb_mlp_down = o;   o += 4 * H * H;
    L->mlp_emb_bias_down = o; o += H;
    L->ln_1 = o;             o += NL * H;
    L->ln_1_bias = o;        o += NL * H;
    L->w_q = o;              o += NL * H * H;
    L->w_k = o;              o += NL * H * H;
    L->w_v = o;              o += NL * H * H;
    L->w_o = o;              o += NL * H * H;
    L->ln_2 = o;             o += NL * H;
    L->ln_2_bias = o;        o += NL * H;
    L->w_up = o;             o += NL * H * 4 * H;
    L->mlp_bias_up = o;      o += NL * 4 * H;
    L->w_down = o;           o += NL * 4 * H * H;
    L->mlp_bias_down = o;    o += NL * H;
    L->ln_f = o;             o += H;
    L->ln_f_bias = o;        o += H;
    L->total = o;
}

int64_t oracle_model_bytes(const egg_config *cfg) {
    model_layout L; layout_of(cfg, &L); return L.total;
}

/* AdamModel (mgpu.cu:337-370): AdamParam = 12 B; hidden matrices use the 8 B
 * MuonParam when USE_MUON. */
static int is_hidden_matrix(const model_layout *L, const egg_config *c, int64_t off, int64_t *len) {
    int64_t H = c->hidden_dim, NL = c->n_layers;
    struct { int64_t o, n; } hm[] = {
        {L->w_emb_mlp_up, 4 * H * H}, {L->w_emb_mlp_down, 4 * H * H},
        {L->w_q, NL * H * H}, {L->w_k, NL * H * H}, {L->w_v, NL * H * H}, {L->w_o, NL * H * H},
        {L->w_up, NL * 4 * H * H}, {L->w_down, NL * 4 * H * H}};
    for (unsigned i = 0; i < sizeof(hm) / sizeof(hm[0]); i++)
        if (off == hm[i].o) { *len = hm[i].n; return 1; }
    return 0;
}

/* byte offset inside AdamModel of the state of model element `elem_off`
 * (elem_off must be the start of a field) */
static int64_t opt_offset_of(const egg_config *c, const model_layout *L, int64_t field_off) {
    /* walk the fields in order */
    int64_t H = c->hidden_dim, V = c->vocab_size, NL = c->n_layers;
    struct { int64_t o, n; int hidden; } f[] = {
        {L->embedding, V * H, 0}, {L->emb_bias, H, 0}, {L->ntt_emb, c->ntt_mode ? 3 * V * H : 0, 0},
        {L->ln_init, H, 0}, {L->ln_init_bias, H, 0},
        {L->w_emb_mlp_up, 4 * H * H, 1}, {L->mlp_emb_bias_up, 4 * H, 0},
        {L->w_emb_mlp_down, 4 * H * H, 1}, {L->mlp_emb_bias_down, H, 0},
        {L->ln_1, NL * H, 0}, {L->ln_1_bias, NL * H, 0},
        {L->w_q, NL * H * H, 1}, {L->w_k, NL * H * H, 1}, {L->w_v, NL * H * H, 1}, {L->w_o, NL * H * H, 1},
        {L->ln_2, NL * H, 0}, {L->ln_2_bias, NL * H, 0},
        {L->w_up, NL * 4 * H * H, 1}, {L->mlp_bias_up, NL * 4 * H, 0},
        {L->w_down, NL * 4 * H * H, 1}, {L->mlp_bias_down, NL * H, 0},
        {L->ln_f, H, 0}, {L->ln_f_bias, H, 0}, {L->total, 0, 0}};
    int64_t bytes = 0;
    for (unsigned i = 0; i < sizeof(f) / sizeof(f[0]); i++) {
        if (f[i].o == field_off) return bytes;
        bytes += f[i].n * ((f[i].hidden && c->use_muon) ? 8 : 12);
    }
    return -1;
}

int64_t oracle_opt_bytes(const egg_config *cfg) {
    model_layout L; layout_of(cfg, &L);
    return opt_offset_of(cfg, &L, L.total);
}

/* AdaptiveScales (d-eggs/include/model/definitions.h:92-142), offsets in bytes */
typedef struct {
    int64_t embedding_row, embedding_col, emb_bias, ln_init, ln_init_bias, w_emb_mlp_up_row,
        w_emb_mlp_up_col, mlp_emb_bias_up, w_emb_mlp_down_row, w_emb_mlp_down_col,
        mlp_emb_bias_down, ln_1, ln_1_bias, w_q_row, w_q_col, w_k_row, w_k_col, w_v_row, w_v_col,
        w_o_row, w_o_col, ln_2, ln_2_bias, w_up_row, w_up_col, mlp_bias_up, w_down_row,
        w_down_col, mlp_bias_down, ln_f, ln_f_bias, total;
} scales_layout;

static void scales_layout_of(const egg_config *c, scales_layout *S) {
    int64_t H = c->hidden_dim, V = c->vocab_size, NL = c->n_layers, o = 0;
    S->embedding_row = o; o += V;       S->embedding_col = o; o += H;   S->emb_bias = o; o += H;
    S->ln_init = o; o += H;             S->ln_init_bias = o; o += H;
    S->w_emb_mlp_up_row = o; o += H;    S->w_emb_mlp_up_col = o; o += 4 * H;
    S->mlp_emb_bias_up = o; o += 4 * H;
    S->w_emb_mlp_down_row = o; o += 4 * H; S->w_emb_mlp_down_col = o; o += H;
    S->mlp_emb_bias_down = o; o += H;
    S->ln_1 = o; o += NL * H;           S->ln_1_bias = o; o += NL * H;
    S->w_q_row = o; o += NL * H;        S->w_q_col = o; o += NL * H;
    S->w_k_row = o; o += NL * H;        S->w_k_col = o; o += NL * H;
    S->w_v_row = o; o += NL * H;        S->w_v_col = o; o += NL * H;
    S->w_o_row = o; o += NL * H;        S->w_o_col = o; o += NL * H;
    S->ln_2 = o; o += NL * H;           S->ln_2_bias = o; o += NL * H;
    S->w_up_row = o; o += NL * H;       S->w_up_col = o; o += NL * 4 * H;
    S->mlp_bias_up = o; o += NL * 4 * H;
    S->w_down_row = o; o += NL * 4 * H; S->w_down_col = o; o += NL * H;
    S->mlp_bias_down = o; o += NL * H;
    S->ln_f = o; o += H;                S->ln_f_bias = o; o += H;
    S->total = o;
}

int64_t oracle_scales_bytes(const egg_config *cfg) {
    scales_layout S; scales_layout_of(cfg, &S); return S.total;
}

/* --------------------------------------------------------------- tables */

/* mgpu.cu:394-426 — same double expressions, same libm calls */
void oracle_init_tables(const egg_config *cfg, int32_t *exp_lut, int8_t *act_lut, int32_t *rope_lut) {
    double softmax_scale = (double)(1 << cfg->softmax_scale_bit);
    for (int i = 0; i < 256; i++) {
        double val = exp(-(double)i / cfg->softmax_exp_scale) * softmax_scale;
        exp_lut[i] = (val >= 1.0) ? (int32_t)round(val) : 0;
    }
    for (int i = 0; i < 256; i++) {
        int8_t input = (int8_t)i;
        double x = (double)input / (1 << cfg->fixed_point);
        double y = 0.5 * x * (1.0 + erf(x / 1.41421356));
        int val = (int)round(y * (1 << cfg->fixed_point));
        act_lut[i] = (int8_t)((val > 127) ? 127 : ((val < -127) ? -127 : val));
    }
    if (!rope_lut) return;
    double rope_scale = (double)(1 << cfg->rope_scale_bit);
    int HD = cfg->head_dim;
    for (int t = 0; t < cfg->seq_len; t++)
        for (int i = 0; i < HD / 2; i++) {
            double theta = pow(10000.0, -2.0 * i / HD);
            double alpha = t * theta;
            rope_lut[t * HD + 2 * i] = (int32_t)round(cos(alpha) * rope_scale);
            rope_lut[t * HD + 2 * i + 1] = (int32_t)round(sin(alpha) * rope_scale);
        }
}

/* ------------------------------------------------------------ init_model */

/* mgpu.cu:443-459: src is [rows=in][cols=out]; dst word (k/4)*cols+n holds
 * bytes k..k+3 of column n. */
void oracle_repack_matrix(int8_t *dst, const int8_t *src, int rows, int cols) {
    for (int k = 0; k < rows; k++)
        for (int n = 0; n < cols; n++)
            dst[((int64_t)(k >> 2) * cols + n) * 4 + (k & 3)] = src[(int64_t)k * cols + n];
}

/* mgpu.cu:461-519 — draw order of the host xorshift stream is the contract */
void oracle_init_model(const egg_config *cfg, int8_t *model, uint32_t seed) {
    model_layout L; layout_of(cfg, &L);
    int64_t H = cfg->hidden_dim, V = cfg->vocab_size;
    uint32_t rng = seed;
    int8_t *tmp = (int8_t *)malloc((size_t)(4 * H * H > V * H ? 4 * H * H : V * H));
    memset(model, 0, (size_t)L.total);
#define DRAW(n) for (int64_t i_ = 0; i_ < (n); i_++) tmp[i_] = (int8_t)oracle_gen_noise_host(cfg, &rng)
    DRAW(V * H); oracle_repack_matrix(model + L.embedding, tmp, (int)H, (int)V);
    if (cfg->ntt_mode)          /* mgpu.cu:472-482 */
        for (int k = 0; k < 3; k++) { DRAW(V * H); oracle_repack_matrix(model + L.ntt_emb + k * V * H, tmp, (int)H, (int)V); }
    for (int64_t i = 0; i < H; i++) { model[L.ln_init + i] = 16; }
    DRAW(4 * H * H); oracle_repack_matrix(model + L.w_emb_mlp_up, tmp, (int)H, (int)(4 * H));
    DRAW(4 * H * H); oracle_repack_matrix(model + L.w_emb_mlp_down, tmp, (int)(4 * H), (int)H);
    for (int l = 0; l < cfg->n_layers; l++) {
        for (int64_t i = 0; i < H; i++) { model[L.ln_1 + l * H + i] = 16; model[L.ln_2 + l * H + i] = 16; }
        DRAW(H * H); oracle_repack_matrix(model + L.w_q + l * H * H, tmp, (int)H, (int)H);
        DRAW(H * H); oracle_repack_matrix(model + L.w_k + l * H * H, tmp, (int)H, (int)H);
        DRAW(H * H); oracle_repack_matrix(model + L.w_v + l * H * H, tmp, (int)H, (int)H);
        DRAW(H * H); oracle_repack_matrix(model + L.w_o + l * H * H, tmp, (int)H, (int)H);
        DRAW(4 * H * H); oracle_repack_matrix(model + L.w_up + l * 4 * H * H, tmp, (int)H, (int)(4 * H));
        DRAW(4 * H * H); oracle_repack_matrix(model + L.w_down + l * 4 * H * H, tmp, (int)(4 * H), (int)H);
    }
    for (int64_t i = 0; i < H; i++) model[L.ln_f + i] = 16;
#undef DRAW
    free(tmp);
}

/* ------------------------------------------------------------ evaluation */

typedef struct {
    const egg_config *c;
    const int8_t *model;
    const int8_t *scales;      /* may be NULL */
    model_layout L;
    scales_layout S;
    int32_t exp_lut[256];
    int8_t act_lut[256];
    int32_t *rope_lut;
} eval_env;

/* get_adaptive_factor, ADAPTIVE_NOISE_MODE==1 (d-eggs/include/model/layers.cuh:12-19) */
static inline float adaptive_factor(const eval_env *E, int64_t off, int64_t idx) {
    if (!E->scales) return 1.0f;
    int ov = E->scales[off + idx];
    if (ov < 0) return 0.0f;
    if (ov < 64) return (float)ov / 64.0f;
    return 1.0f;
}

static inline int32_t softmax_exp_lookup(const eval_env *E, int32_t diff) {   /* mgpu.cu:543-547 */
    int index = -diff;
    index = (index < 0) ? 0 : ((index > 255) ? 255 : index);
    return E->exp_lut[index];
}

/* packed [K/4][N][4] weight read */
static inline int wq(const int8_t *w, int k, int n, int N) {
    return w[((int64_t)(k >> 2) * N + n) * 4 + (k & 3)];
}

/* mgpu.cu:553-572 (+ float output factor of d-eggs layers.cuh:77-97) */
static int32_t linear_projection(const eval_env *E, const int8_t *in, const int8_t *w, int K, int N,
                                 int n, int32_t sb, uint32_t noise_seed, int ns, float scale_out) {
    int32_t acc = 0;
    for (int k = 0; k < K; k++) acc += (int32_t)in[k] * wq(w, k, n, N);
    if (ns != 0) {
        int32_t a = (int32_t)((float)oracle_noise(E->c, noise_seed, (uint32_t)n) * scale_out);
        acc += ((sb * a) * ns) >> (E->c->fixed_point + E->c->sigma_shift);
    }
    return acc;
}

/* Σ_k in[k]·noise(seed,k)·factor_k, summed as the reference does: each term
 * is an int×float product truncated when it is converted to the int32
 * argument of block_reduce_sum_broadcast (layers.cuh:250). */
static int32_t noise_dot(const eval_env *E, const int8_t *in, int K, uint32_t seed, int64_t sc_off) {
    int32_t s = 0;
    for (int k = 0; k < K; k++) {
        int32_t prod = (int32_t)in[k] * oracle_noise(E->c, seed, (uint32_t)k);
        if (E->scales && sc_off >= 0) s += (int32_t)((float)prod * adaptive_factor(E, sc_off, k));
        else s += prod;
    }
    return s;
}

/* The down projection's dot (layers.cuh:272-280): thread tid adds its four terms tid, tid+H, tid+2H, tid+3H
 * into an int32 with `pb += int * int8 * float`, i.e. pb = (int32)((float)pb + product) after every term, so
 * the truncation applies to the running sum of the thread, not to the term; the threads' sums are then added. */
static int32_t noise_dot_down(const eval_env *E, const int8_t *in, int H, uint32_t seed, int64_t sc_off) {
    if (!E->scales || sc_off < 0) return noise_dot(E, in, 4 * H, seed, sc_off);
    int32_t s = 0;
    for (int tid = 0; tid < H; tid++) {
        int32_t pb = 0;
        for (int sub = 0; sub < 4; sub++) {
            int k = tid + sub * H;
            int32_t prod = (int32_t)in[k] * oracle_noise(E->c, seed, (uint32_t)k);
            pb = (int32_t)((float)pb + (float)prod * adaptive_factor(E, sc_off, k));
        }
        s += pb;
    }
    return s;
}

/* vector ("universal rank-1") noise: ((n1*n2*f)*ns) >> SSV  (mgpu.cu:668-674) */
static inline int32_t vec_noise(const eval_env *E, uint32_t seed_base, int off_a, int off_b, int idx,
                                int ns, int64_t sc_off) {
    int32_t n1 = oracle_noise(E->c, seed_base + (uint32_t)off_a, (uint32_t)idx);
    int32_t n2 = oracle_noise(E->c, seed_base + (uint32_t)off_b, (uint32_t)idx);
    int32_t p = n1 * n2;
    if (E->scales && sc_off >= 0) p = (int32_t)((float)p * adaptive_factor(E, sc_off, idx));
    return (p * ns) >> E->c->sigma_shift_vector;
}

/* mgpu.cu:646-678 */
static void standard_norm(const eval_env *E, const int8_t *x, int8_t *out, const int8_t *w, const int8_t *b,
                          uint32_t seed_base, int off_w_a, int off_w_b, int off_b_a, int off_b_b, int ns,
                          int64_t sc_w, int64_t sc_b) {
    int H = E->c->hidden_dim;
    int32_t tot = 0;
    for (int d = 0; d < H; d++) tot += abs((int)x[d]);
    int32_t mn = tot / H;
    if (!mn) mn = 1;
    for (int d = 0; d < H; d++) {
        int32_t w_mod = w[d], b_mod = b[d];
        if (ns != 0) {
            w_mod += vec_noise(E, seed_base, off_w_a, off_w_b, d, ns, sc_w);
            b_mod += vec_noise(E, seed_base, off_b_a, off_b_b, d, ns, sc_b);
        }
        out[d] = (int8_t)clip8(((int32_t)x[d] * w_mod) / mn + b_mod);
    }
}

/* egg_adaptive_normalize.h:10-103 — both variants are the same arithmetic;
 * the spec is the sequential meaning: max over the row being normalised. */
static void adaptive_normalize(const int32_t *v, int8_t *out, int n) {
    int32_t mx = 0;
    for (int i = 0; i < n; i++) { int32_t a = abs(v[i]); if (a > mx) mx = a; }
    float scale = 127.0f / (float)((float)mx + 1e-9f);
    for (int i = 0; i < n; i++) {
        float sf = (float)v[i] * scale;
        int32_t s = (int32_t)roundf(sf);
        if (s > 127) s = 127;
        if (s < -127) s = -127;
        out[i] = (int8_t)s;
    }
}

/* mgpu.cu:624-644 */
static void rope_integer(const eval_env *E, int32_t *v, int t) {
    int H = E->c->hidden_dim, HD = E->c->head_dim, bit = E->c->rope_scale_bit;
    for (int d = 0; d < H; d += 2) {
        int pair = (d % HD) / 2;
        int64_t c = E->rope_lut[t * HD + pair * 2], s = E->rope_lut[t * HD + pair * 2 + 1];
        int64_t ev = v[d], od = v[d + 1];
        int64_t half = (int64_t)1 << (bit - 1);
        int64_t re = (ev * c - od * s + half) >> bit;
        int64_t ro = (ev * s + od * c + half) >> bit;
        v[d] = (int32_t)re; v[d + 1] = (int32_t)ro;
    }
}

typedef struct {
    int off_ln_a, off_ln_b, off_ln_bias_a, off_ln_bias_b, off_up_a, off_up_b, off_bias_up_a,
        off_bias_up_b, off_dn_a, off_dn_b, off_bias_dn_a, off_bias_dn_b;
} mlp_cfg;
static const mlp_cfg CFG_MLP_INIT = {500, 501, 502, 503, 510, 511, 514, 515, 512, 513, 516, 517};   /* mgpu.cu:689-697 */
static const mlp_cfg CFG_MLP_LAYER = {300, 301, 310, 311, 400, 401, 410, 411, 402, 403, 412, 413};  /* mgpu.cu:698-706 */

/* mgpu.cu:708-759; l < 0 selects the initial MLP */
static void mlp_block(const eval_env *E, int l, int8_t *x, uint32_t seed_base, int ns) {
    const egg_config *c = E->c; int H = c->hidden_dim; const model_layout *L = &E->L; const scales_layout *S = &E->S;
    int init = (l < 0);
    const mlp_cfg *cfg = init ? &CFG_MLP_INIT : &CFG_MLP_LAYER;
    const int8_t *M = E->model;
    const int8_t *ln_w = M + (init ? L->ln_init : L->ln_2 + (int64_t)l * H);
    const int8_t *ln_b = M + (init ? L->ln_init_bias : L->ln_2_bias + (int64_t)l * H);
    const int8_t *up_w = M + (init ? L->w_emb_mlp_up : L->w_up + (int64_t)l * 4 * H * H);
    const int8_t *up_b = M + (init ? L->mlp_emb_bias_up : L->mlp_bias_up + (int64_t)l * 4 * H);
    const int8_t *dn_w = M + (init ? L->w_emb_mlp_down : L->w_down + (int64_t)l * 4 * H * H);
    const int8_t *dn_b = M + (init ? L->mlp_emb_bias_down : L->mlp_bias_down + (int64_t)l * H);
    int64_t sc_ln = init ? S->ln_init : S->ln_2 + (int64_t)l * H;
    int64_t sc_lnb = init ? S->ln_init_bias : S->ln_2_bias + (int64_t)l * H;
    int64_t sc_up_row = init ? S->w_emb_mlp_up_row : S->w_up_row + (int64_t)l * H;
    int64_t sc_up_col = init ? S->w_emb_mlp_up_col : S->w_up_col + (int64_t)l * 4 * H;
    int64_t sc_up_b = init ? S->mlp_emb_bias_up : S->mlp_bias_up + (int64_t)l * 4 * H;
    int64_t sc_dn_row = init ? S->w_emb_mlp_down_row : S->w_down_row + (int64_t)l * 4 * H;
    int64_t sc_dn_col = init ? S->w_emb_mlp_down_col : S->w_down_col + (int64_t)l * H;
    int64_t sc_dn_b = init ? S->mlp_emb_bias_down : S->mlp_bias_down + (int64_t)l * H;

    int8_t *h = (int8_t *)malloc((size_t)H), *u = (int8_t *)malloc((size_t)4 * H);
    int32_t *pre = (int32_t *)malloc(sizeof(int32_t) * (size_t)H);
    standard_norm(E, x, h, ln_w, ln_b, seed_base, cfg->off_ln_a, cfg->off_ln_b, cfg->off_ln_bias_a,
                  cfg->off_ln_bias_b, ns, sc_ln, sc_lnb);
    int32_t sb = noise_dot(E, h, H, seed_base + (uint32_t)cfg->off_up_b, sc_up_row);
    for (int o = 0; o < 4 * H; o++) {
        int32_t a = linear_projection(E, h, up_w, H, 4 * H, o, sb, seed_base + (uint32_t)cfg->off_up_a, ns,
                                      adaptive_factor(E, sc_up_col, o));
        int32_t nv = vec_noise(E, seed_base, cfg->off_bias_up_a, cfg->off_bias_up_b, o, ns, sc_up_b);
        u[o] = E->act_lut[(uint8_t)(int8_t)clip8((a >> c->shift_mlp_up) + up_b[o] + nv)];
    }
    int32_t sb2 = noise_dot_down(E, u, H, seed_base + (uint32_t)cfg->off_dn_b, sc_dn_row);
    for (int d = 0; d < H; d++) {
        int32_t a = linear_projection(E, u, dn_w, 4 * H, H, d, sb2, seed_base + (uint32_t)cfg->off_dn_a, ns,
                                      adaptive_factor(E, sc_dn_col, d));
        int32_t nv = vec_noise(E, seed_base, cfg->off_bias_dn_a, cfg->off_bias_dn_b, d, ns, sc_dn_b);
        pre[d] = (int32_t)x[d] + (a >> c->shift_mlp_down) + dn_b[d] + nv;
    }
    adaptive_normalize(pre, x, H);
    free(h); free(u); free(pre);
}

/* mgpu.cu:761-833.  kcache/vcache: [seq_len][H] of this member and layer. */
static void attention_block(const eval_env *E, int l, int t, int8_t *x, int8_t *kcache, int8_t *vcache,
                            uint32_t seed_base, int ns) {
    const egg_config *c = E->c; int H = c->hidden_dim, HD = c->head_dim; const model_layout *L = &E->L;
    const scales_layout *S = &E->S; const int8_t *M = E->model;
    int8_t *h = (int8_t *)malloc((size_t)H), *q8 = (int8_t *)malloc((size_t)H), *ao = (int8_t *)malloc((size_t)H);
    int32_t *aq = (int32_t *)malloc(sizeof(int32_t) * (size_t)H), *ak = (int32_t *)malloc(sizeof(int32_t) * (size_t)H),
            *av = (int32_t *)malloc(sizeof(int32_t) * (size_t)H);
    standard_norm(E, x, h, M + L->ln_1 + (int64_t)l * H, M + L->ln_1_bias + (int64_t)l * H, seed_base, 100, 101,
                  110, 111, ns, S->ln_1 + (int64_t)l * H, S->ln_1_bias + (int64_t)l * H);
    int32_t sbq = noise_dot(E, h, H, seed_base + 201, S->w_q_row + (int64_t)l * H);
    int32_t sbk = noise_dot(E, h, H, seed_base + 203, S->w_k_row + (int64_t)l * H);
    int32_t sbv = noise_dot(E, h, H, seed_base + 205, S->w_v_row + (int64_t)l * H);
    for (int n = 0; n < H; n++) {
        aq[n] = linear_projection(E, h, M + L->w_q + (int64_t)l * H * H, H, H, n, sbq, seed_base + 200, ns,
                                  adaptive_factor(E, S->w_q_col + (int64_t)l * H, n));
        ak[n] = linear_projection(E, h, M + L->w_k + (int64_t)l * H * H, H, H, n, sbk, seed_base + 202, ns,
                                  adaptive_factor(E, S->w_k_col + (int64_t)l * H, n));
        av[n] = linear_projection(E, h, M + L->w_v + (int64_t)l * H * H, H, H, n, sbv, seed_base + 204, ns,
                                  adaptive_factor(E, S->w_v_col + (int64_t)l * H, n));
    }
    rope_integer(E, aq, t);
    rope_integer(E, ak, t);
    adaptive_normalize(aq, q8, H);
    adaptive_normalize(ak, kcache + (int64_t)t * H, H);
    adaptive_normalize(av, vcache + (int64_t)t * H, H);

    for (int hd = 0; hd < H / HD; hd++) {
        int32_t mx = INT_MIN;
        for (int ctx = 0; ctx <= t; ctx++) {                     /* pass 1, mgpu.cu:795-802 */
            int32_t sc = 0;
            for (int d = 0; d < HD; d++) sc += (int32_t)q8[hd * HD + d] * kcache[(int64_t)ctx * H + hd * HD + d];
            if (sc > mx) mx = sc;
        }
        int64_t *wv = (int64_t *)calloc((size_t)HD, sizeof(int64_t));
        uint64_t tot = 0;
        for (int ctx = 0; ctx <= t; ctx++) {                     /* pass 2, mgpu.cu:810-822 */
            int32_t sc = 0;
            for (int d = 0; d < HD; d++) sc += (int32_t)q8[hd * HD + d] * kcache[(int64_t)ctx * H + hd * HD + d];
            int32_t wt = softmax_exp_lookup(E, (sc >> c->shift_attn) - (mx >> c->shift_attn));
            for (int d = 0; d < HD; d++) wv[d] += (int64_t)wt * vcache[(int64_t)ctx * H + hd * HD + d];
            tot += (uint64_t)wt;
        }
        for (int d = 0; d < HD; d++) {
            int64_t qn = wv[d] / (tot ? (int64_t)tot : 1);
            ao[hd * HD + d] = (int8_t)clip8((int32_t)qn);
        }
        free(wv);
    }
    int32_t sbo = noise_dot(E, ao, H, seed_base + 207, S->w_o_row + (int64_t)l * H);
    for (int n = 0; n < H; n++) {
        int32_t aco = linear_projection(E, ao, M + L->w_o + (int64_t)l * H * H, H, H, n, sbo, seed_base + 206, ns,
                                        adaptive_factor(E, S->w_o_col + (int64_t)l * H, n));
        aq[n] = (int32_t)x[n] + (aco >> c->shift_out);
    }
    adaptive_normalize(aq, x, H);
    free(h); free(q8); free(ao); free(aq); free(ak); free(av);
}

/* TokenType (mgpu.cu:58-66): bytes when vocab_size == 256, uint32_t otherwise.  `dataset` points at the token
 * array of either width; positions and data_len count tokens. */
static inline int token_at(const egg_config *c, const uint8_t *dataset, int64_t i) {
    return c->vocab_size == 256 ? (int)dataset[i] : (int)((const uint32_t *)dataset)[i];
}

/* ---- the optional transform of the input window (egg_ntt.cuh; NTT_MODE 1, 2, 3) ----
 * The reference runs it with one thread per hidden unit; with seq_len <= hidden_dim (required here) every element
 * is loaded and every butterfly of every stage is executed, which is what this serial form computes. */
static int64_t fermat_p(int mode) { return mode == 2 ? 257 : 65537; }

/* 3^k mod p by square-and-multiply with k taken mod p-1 (pow_omega257 / pow_omega65537, egg_ntt.cuh:187-201, 273-289) */
static int64_t fermat_pow3(int mode, int k) {
    int64_t p = fermat_p(mode), r = 1, b = 3;
    k &= (int)(p - 2);          /* p-1 is a power of two: k mod (p-1) */
    while (k > 0) { if (k & 1) r = r * b % p; b = b * b % p; k >>= 1; }
    return r;
}

static void window_transform(const egg_config *c, int32_t *d, int len) {
    int mode = c->ntt_mode;
    if (mode == 1) {            /* Walsh-Hadamard, natural order (wht_transform_inplace, egg_ntt.cuh:105-122) */
        for (int stride = 1; stride < len; stride <<= 1)
            for (int t = 0; t < len / 2; t++) {
                int base = (t / stride) * 2 * stride + t % stride;
                int32_t a = d[base], b = d[base + stride];
                d[base] = a + b; d[base + stride] = a - b;
            }
        return;
    }
    /* fermat_ntt_inplace + ntt_dit_inplace (egg_ntt.cuh:330-366, 420-428): reduce, bit-reverse, then log2(len)
     * stages whose twiddle is 3^(j * len / m) -- the root of the full-length transform whatever len is */
    int64_t p = fermat_p(mode);
    int lg = 0; while ((1 << lg) < len) lg++;
    for (int i = 0; i < len; i++) d[i] = (int32_t)(((int64_t)d[i] % p + p) % p);
    for (int i = 0; i < len; i++) {
        int rev = 0;
        for (int b = 0; b < lg; b++) rev |= ((i >> b) & 1) << (lg - 1 - b);
        if (i < rev) { int32_t t = d[i]; d[i] = d[rev]; d[rev] = t; }
    }
    for (int s = 1; s <= lg; s++) {
        int m = 1 << s, m2 = m >> 1, w_step = len >> s;
        for (int k = 0; k < len / 2; k++) {
            int j = k % m2, i1 = (k / m2) * m + j, i2 = i1 + m2;
            int64_t wb = fermat_pow3(mode, j * w_step) * d[i2] % p;
            int64_t a = d[i1];
            d[i1] = (int32_t)((a + wb) % p);
            d[i2] = (int32_t)((a - wb + p) % p);
        }
    }
}

void oracle_window_transform(const egg_config *cfg, int32_t *data, int len) { window_transform(cfg, data, len); }

/* One member, whole sequence (mgpu.cu:847-1029). */
static int32_t eval_member(const eval_env *E, const uint8_t *dataset, int64_t data_len, int64_t start_idx,
                           uint32_t step_seed, int p_idx, int8_t *trace_x, int32_t *trace_logits) {
    const egg_config *c = E->c; int H = c->hidden_dim, V = c->vocab_size, S = c->seq_len, NL = c->n_layers;
    const model_layout *L = &E->L; const scales_layout *SC = &E->S; const int8_t *M = E->model;
    int64_t pair_idx = p_idx / 2;
    int64_t stride = data_len / (c->population_size / 2);
    int64_t stream_pos = c->use_same_data ? (start_idx % (data_len - S))
                                          : ((start_idx + pair_idx * stride) % (data_len - S));
    int ns = (p_idx % 2 == 0) ? 1 : -1;
    uint32_t S0 = step_seed + (uint32_t)pair_idx;
    int8_t *x = (int8_t *)malloc((size_t)H), *nf = (int8_t *)malloc((size_t)H);
    int8_t *kv = (int8_t *)calloc((size_t)NL * 2 * S * H, 1);
    int32_t *lg = (int32_t *)malloc(sizeof(int32_t) * (size_t)V);
    int64_t my_loss = 0;
    int32_t *coef = NULL;
    if (c->ntt_mode) {          /* mgpu.cu:877-887: the window's first seq_len tokens, transformed once */
        coef = (int32_t *)malloc(sizeof(int32_t) * (size_t)S);
        for (int t = 0; t < S; t++) coef[t] = token_at(c, dataset, stream_pos + t);
        window_transform(c, coef, S);
    }

    for (int t = 0; t < S; t++) {
        int tok = token_at(c, dataset, stream_pos + t);
        /* embedding, mgpu.cu:902-931 (+ d-eggs kernels.cu:134-156 factors) */
        uint32_t seed_emb = S0 + 0;
        for (int d = 0; d < H; d++) {
            int32_t emb = M[L->embedding + ((int64_t)(d >> 2) * V + tok) * 4 + (d & 3)];
            int32_t ebias = M[L->emb_bias + d];
            int32_t chk = vec_noise(E, S0, 50, 51, d, ns, SC->emb_bias);
            int32_t a_tok = oracle_noise(c, seed_emb, (uint32_t)tok);
            int32_t b_dim = oracle_noise(c, seed_emb + (uint32_t)H, (uint32_t)d);
            int32_t prod = a_tok * b_dim;
            if (E->scales)
                prod = (int32_t)((float)prod * adaptive_factor(E, SC->embedding_row, tok) *
                                 adaptive_factor(E, SC->embedding_col, d));
            int32_t perturb = (prod * ns) >> (c->fixed_point + c->sigma_shift);
            int32_t extra = 0;
            if (coef) {         /* bytes 1, 2, 3 of the coefficient index three more tables, each added >> 2 (mgpu.cu:916-929) */
                for (int k = 0; k < 3; k++) {
                    int nb = (coef[t] >> (8 * (k + 1))) & 0xFF;
                    extra += M[L->ntt_emb + (int64_t)k * V * H + ((int64_t)(d >> 2) * V + nb) * 4 + (d & 3)] >> 2;
                }
            }
            x[d] = (int8_t)clip8(emb + ebias + chk + perturb + extra);
        }
        const int nst = 3 + 2 * NL;
#define STAGE(i, buf) do { if (trace_x) memcpy(trace_x + ((int64_t)t * nst + (i)) * H, (buf), (size_t)H); } while (0)
        STAGE(0, x);
        mlp_block(E, -1, x, S0, ns);
        STAGE(1, x);
        for (int l = 0; l < NL; l++) {
            uint32_t seed_base = S0 + (uint32_t)(l * 1000);
            int8_t *kc = kv + (int64_t)l * 2 * S * H, *vc = kc + (int64_t)S * H;
            attention_block(E, l, t, x, kc, vc, seed_base, ns);
            STAGE(2 + 2 * l, x);
            mlp_block(E, l, x, seed_base, ns);
            STAGE(3 + 2 * l, x);
        }
        /* head + loss, mgpu.cu:954-1024 */
        standard_norm(E, x, nf, M + L->ln_f, M + L->ln_f_bias, S0, 900, 901, 910, 911, ns, SC->ln_f, SC->ln_f_bias);
        STAGE(2 + 2 * NL, nf);
#undef STAGE
        int32_t sbh = noise_dot(E, nf, H, S0 + (uint32_t)H, SC->embedding_col);
        int32_t mx = INT_MIN;
        for (int v = 0; v < V; v++) {
            int32_t ah = linear_projection(E, nf, M + L->embedding, H, V, v, sbh, S0, ns,
                                           adaptive_factor(E, SC->embedding_row, v));
            lg[v] = ah >> c->shift_logit;
            if (lg[v] > mx) mx = lg[v];
        }
        if (trace_logits) memcpy(trace_logits + (int64_t)t * V, lg, sizeof(int32_t) * (size_t)V);
        int64_t sum_ex = 0;
        for (int v = 0; v < V; v++) sum_ex += softmax_exp_lookup(E, lg[v] - mx);
        int target = token_at(c, dataset, stream_pos + t + 1);
        int64_t log_sum = 0;
        if (sum_ex > 0) {
            uint64_t xx = (uint64_t)sum_ex; int pos = 0;
            while (xx >= 256) { xx >>= 8; pos += 8; }
            if (xx >= 16) { xx >>= 4; pos += 4; }
            if (xx >= 4) { xx >>= 2; pos += 2; }
            if (xx >= 2) { pos += 1; }
            log_sum = (pos << 4) - (c->softmax_scale_bit << 4);
        }
        /* a target outside the vocabulary matches no column: the reference's s_target_logit stays 0 (mgpu.cu:989-1002) */
        my_loss += (log_sum >> 1) + mx - ((target >= 0 && target < V) ? lg[target] : 0);
    }
    free(x); free(nf); free(kv); free(lg); free(coef);
    return (int32_t)my_loss;
}

static void env_init(eval_env *E, const egg_config *cfg, const int8_t *model, const int8_t *scales) {
    E->c = cfg; E->model = model; E->scales = scales;
    layout_of(cfg, &E->L); scales_layout_of(cfg, &E->S);
    E->rope_lut = (int32_t *)malloc(sizeof(int32_t) * (size_t)cfg->seq_len * cfg->head_dim);
    oracle_init_tables(cfg, E->exp_lut, E->act_lut, E->rope_lut);
}

void oracle_eval(const egg_config *cfg, const int8_t *model, const int8_t *scales, const uint8_t *dataset,
                 int64_t data_len, int64_t start_idx, uint32_t step_seed, int pop_offset, int count,
                 int32_t *losses_out) {
    eval_env E; env_init(&E, cfg, model, scales);
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < count; i++)
        losses_out[i] = eval_member(&E, dataset, data_len, start_idx, step_seed, pop_offset + i, NULL, NULL);
    free(E.rope_lut);
}

void oracle_eval_trace(const egg_config *cfg, const int8_t *model, const int8_t *scales, const uint8_t *dataset,
                       int64_t data_len, int64_t start_idx, uint32_t step_seed, int member,
                       int8_t *x_after_layers, int32_t *logits, int32_t *loss_out) {
    eval_env E; env_init(&E, cfg, model, scales);
    int32_t l = eval_member(&E, dataset, data_len, start_idx, step_seed, member, x_after_layers, logits);
    if (loss_out) *loss_out = l;
    free(E.rope_lut);
}

/* generate_sequence_kernel (d-eggs/src/kernels.cu:307-490; mgpu.cu:1154-1285 is the same with temp 1, no min-p
 * filter and no penalty): one un-perturbed stream decoded token by token with a KV cache; the first seed_len
 * tokens of `tokens` are given, the following gen_len are written.  The weighted draw walks the vocabulary in
 * the order the kernel's block scan sees it: thread-major, thread tid owning v = tid, tid + B, ... with
 * B = EGG_BLOCK_THREADS = min(hidden_dim rounded up to 32, 1024) (config.h:36-37). */
void oracle_generate(const egg_config *cfg, const int8_t *model, uint8_t *tokens, int seed_len, int gen_len,
                     uint32_t seed, float temp, float min_p, float penalty) {
    eval_env E; env_init(&E, cfg, model, NULL);
    const egg_config *c = cfg; const int H = c->hidden_dim, V = c->vocab_size, NL = c->n_layers;
    const model_layout *L = &E.L; const int8_t *M = model;
    const int total = seed_len + gen_len;
    int8_t *x = malloc((size_t)H), *nf = malloc((size_t)H);
    int8_t *kv = calloc((size_t)NL * 2 * total * H, 1);
    int32_t *lg = malloc(sizeof(int32_t) * (size_t)V), *ex = malloc(sizeof(int32_t) * (size_t)V);
    const int32_t penalty_int = (int32_t)(penalty * (float)(1 << c->shift_logit));
    const int filter = min_p > 0.0f;
    const int32_t min_p_limit = filter ? (int32_t)(logf(min_p) * c->softmax_exp_scale) : 0;
    int B = (H + 31) & ~31; if (B > 1024) B = 1024;
    for (int t = 0; t < total - 1; t++) {
        const int tok = tokens[t];
        for (int d = 0; d < H; d++)
            x[d] = (int8_t)clip8((int32_t)M[L->embedding + ((int64_t)(d >> 2) * V + tok) * 4 + (d & 3)] + M[L->emb_bias + d]);
        mlp_block(&E, -1, x, 0, 0);
        for (int l = 0; l < NL; l++) {
            /* the kernel's cache is [layer][k|v][total][H]; attention_block only needs one k and one v plane per layer */
            int8_t *kc = kv + (int64_t)l * 2 * total * H, *vc = kc + (int64_t)total * H;
            attention_block(&E, l, t, x, kc, vc, 0, 0);
            mlp_block(&E, l, x, 0, 0);
        }
        standard_norm(&E, x, nf, M + L->ln_f, M + L->ln_f_bias, 0, 0, 0, 0, 0, 0, -1, -1);
        int32_t mx = INT_MIN;
        for (int v = 0; v < V; v++) {
            int32_t ah = linear_projection(&E, nf, M + L->embedding, H, V, v, 0, 0, 0, 1.0f);
            int32_t l = ah >> c->shift_logit;
            for (int i = 0; i <= t && i < 256; i++) if (tokens[i] == (uint8_t)v) l -= penalty_int;   /* presence penalty, per occurrence */
            lg[v] = l;
            if (l > mx) mx = l;
        }
        int64_t sum = 0;
        for (int v = 0; v < V; v++) {
            int32_t scaled = (int32_t)((float)(lg[v] - mx) / temp);
            ex[v] = (!filter || scaled >= min_p_limit) ? softmax_exp_lookup(&E, scaled) : 0;
            sum += ex[v];
        }
        uint32_t r = oracle_hash_rng(seed + (uint32_t)t * 555u, 0);
        int64_t thresh = sum > 0 ? (int64_t)(r % (uint64_t)sum) : 0;
        int selected = 0; int64_t running = 0; int done = 0;
        for (int tid = 0; tid < B && !done; tid++)
            for (int v = tid; v < V; v += B) {
                running += ex[v];
                if (running > thresh) { selected = v; done = 1; break; }
            }
        if (t >= seed_len - 1) tokens[t + 1] = (uint8_t)selected;
    }
    free(x); free(nf); free(kv); free(lg); free(ex); free(E.rope_lut);
}

/* mgpu.cu:1031-1036 / 1305-1311 */
void oracle_fitness(const int32_t *losses, int32_t *fitness, int pairs) {
    for (int i = 0; i < pairs; i++) {
        int32_t p = losses[2 * i], n = losses[2 * i + 1];
        fitness[i] = (p < n) ? 1 : ((n < p) ? -1 : 0);
    }
}

/* ---------------------------------------------------------------- update */

/* mgpu.cu:1085-1098: packed index idx -> (k, n); the reference skips fit==0,
 * which does not change the sum. */
void oracle_vote_matrix(const egg_config *cfg, const int32_t *fitness, int pairs, int rows_k, int cols_n,
                        int off_a, int off_b, int seed_base, uint32_t step_seed, int32_t *vote) {
    /* regenerate the two noise matrices once: O((K+N)·P) hashes instead of O(K·N·P) */
    int8_t *A = (int8_t *)malloc((size_t)pairs * cols_n), *B = (int8_t *)malloc((size_t)pairs * rows_k);
    for (int p = 0; p < pairs; p++) {
        uint32_t s = step_seed + (uint32_t)p + (uint32_t)seed_base;
        for (int n = 0; n < cols_n; n++) A[(int64_t)p * cols_n + n] = (int8_t)oracle_noise(cfg, s + (uint32_t)off_a, (uint32_t)n);
        for (int k = 0; k < rows_k; k++) B[(int64_t)p * rows_k + k] = (int8_t)oracle_noise(cfg, s + (uint32_t)off_b, (uint32_t)k);
    }
    int64_t total = (int64_t)rows_k * cols_n;
#pragma omp parallel for schedule(static)
    for (int64_t idx = 0; idx < total; idx++) {
        int byte_off = (int)(idx & 3);
        int64_t word = idx >> 2;
        int n = (int)(word % cols_n);
        int k = (int)(word / cols_n) * 4 + byte_off;
        int32_t v = 0;
        for (int p = 0; p < pairs; p++) {
            int32_t f = fitness[p];
            if (f == 0) continue;
            v += f * A[(int64_t)p * cols_n + n] * B[(int64_t)p * rows_k + k];
        }
        vote[idx] = v;
    }
    free(A); free(B);
}

static void vote_vector(const egg_config *cfg, const int32_t *fitness, int pairs, int len, int off_a, int off_b,
                        int seed_base, uint32_t step_seed, int32_t *vote) {   /* mgpu.cu:1131-1139 */
    for (int i = 0; i < len; i++) vote[i] = 0;
    for (int p = 0; p < pairs; p++) {
        int32_t f = fitness[p];
        if (f == 0) continue;
        uint32_t s = step_seed + (uint32_t)p + (uint32_t)seed_base;
        for (int i = 0; i < len; i++)
            vote[i] += f * oracle_noise(cfg, s + (uint32_t)off_a, (uint32_t)i) * oracle_noise(cfg, s + (uint32_t)off_b, (uint32_t)i);
    }
}

/* apply_quantized_update (d-eggs/include/optimizer/sgd.cuh:10-18; mgpu.cu:1057-1063) */
static int quantized_update(int8_t *w, float *acc) {
    if (*acc >= 1.0f) {
        if (*w < 127) { (*w)++; *acc -= 1.0f; return 1; }
        *acc = 1.0f;
    } else if (*acc <= -1.0f) {
        if (*w > -127) { (*w)--; *acc += 1.0f; return 1; }
        *acc = -1.0f;
    }
    return 0;
}

/* mgpu.cu:1040-1064.  fma_mode selects which multiply-adds are contracted into a
 * single-rounding fma, as nvcc's default -fmad=true may do on the reference source:
 *   mode = m_sel + 3*v_sel + 9*inner_sel + 18*acc_sel
 *   m_sel:     0 separate | 1 fma(b1, m, (1-b1)*g)        | 2 fma(1-b1, g, b1*m)
 *   v_sel:     0 separate | 1 fma(b2, v, (1-b2)*(g*g))    | 2 fma(1-b2, g*g, b2*v)
 *   inner_sel: 0 separate | 1 fma(wd, w, m/(sqrt(v)+eps))
 *   acc_sel:   0 separate | 1 fma(-lr, inner, acc)
 * ORACLE_FMA_NVCC is the pattern calibrated against the reference kernels on a B200. */
static inline float mul_rn(float a, float b) { volatile float r = a * b; return r; }
static inline float add_rn(float a, float b) { volatile float r = a + b; return r; }
int oracle_adam_step(const egg_config *c, float *m, float *v, float *acc, int8_t *w, float g, float lr, int fma_mode) {
    const float b1 = c->adam_beta1, b2 = c->adam_beta2;
    const float omb1 = 1.0f - b1, omb2 = 1.0f - b2;
    const int m_sel = fma_mode % 3, v_sel = (fma_mode / 3) % 3, inner_sel = (fma_mode / 9) % 2, acc_sel = (fma_mode / 18) % 2;
    if (m_sel == 1) *m = fmaf(b1, *m, mul_rn(omb1, g));
    else if (m_sel == 2) *m = fmaf(omb1, g, mul_rn(b1, *m));
    else *m = add_rn(mul_rn(b1, *m), mul_rn(omb1, g));
    const float gg = mul_rn(g, g);
    if (v_sel == 1) *v = fmaf(b2, *v, mul_rn(omb2, gg));
    else if (v_sel == 2) *v = fmaf(omb2, gg, mul_rn(b2, *v));
    else *v = add_rn(mul_rn(b2, *v), mul_rn(omb2, gg));
    volatile float den = sqrtf(*v) + c->adam_eps;
    volatile float dv = *m / den;
    const float inner = inner_sel ? fmaf(c->adam_weight_decay, (float)*w, dv) : add_rn(dv, mul_rn(c->adam_weight_decay, (float)*w));
    *acc = acc_sel ? fmaf(-lr, inner, *acc) : add_rn(*acc, mul_rn(-lr, inner));
    return quantized_update(w, acc);
}

/* muon_internal.cuh:182-342: Frobenius normalise, 5 cubic Newton–Schulz
 * iterations on the short side.  x is row-major rows×cols. */
void oracle_newton_schulz(float *x, int rows, int cols) {
    int use_rows = rows < cols;
    int K = use_rows ? rows : cols;
    int64_t n = (int64_t)rows * cols;
    double ss = 0;
    for (int64_t i = 0; i < n; i++) ss += (double)x[i] * x[i];
    float norm = (float)sqrt(ss);
    if (norm > 1e-6f) for (int64_t i = 0; i < n; i++) x[i] /= norm;
    float *G = (float *)malloc(sizeof(float) * (size_t)K * K), *Y = (float *)malloc(sizeof(float) * (size_t)n);
    for (int it = 0; it < 5; it++) {
#pragma omp parallel for schedule(static)
        for (int i = 0; i < K; i++)
            for (int j = 0; j < K; j++) {
                double s = 0;
                if (use_rows) for (int t = 0; t < cols; t++) s += (double)x[(int64_t)i * cols + t] * x[(int64_t)j * cols + t];
                else for (int t = 0; t < rows; t++) s += (double)x[(int64_t)t * cols + i] * x[(int64_t)t * cols + j];
                float g = (float)s;
                G[(int64_t)i * K + j] = (i == j) ? 3.0f - g : -g;
            }
#pragma omp parallel for schedule(static)
        for (int r = 0; r < rows; r++)
            for (int cc = 0; cc < cols; cc++) {
                double s = 0;
                if (use_rows) for (int t = 0; t < K; t++) s += (double)G[(int64_t)r * K + t] * x[(int64_t)t * cols + cc];
                else for (int t = 0; t < K; t++) s += (double)x[(int64_t)r * cols + t] * G[(int64_t)t * K + cc];
                Y[(int64_t)r * cols + cc] = (float)(0.5 * s);
            }
        memcpy(x, Y, sizeof(float) * (size_t)n);
    }
    free(G); free(Y);
}

typedef struct { int64_t off; int rows, cols, off_a, off_b, seed_base; float lr_scale; int hidden; int64_t ov_in, ov_out; } param_desc;

/* the launch sequence of mgpu.cu:1603-1643 as a table (matrices: rows=K in, cols=N out; vectors: rows=0) */
/* ov_in / ov_out: AdaptiveScales offsets of the overlay over the input index k ("*_row") and the output index n
 * ("*_col"), as worker.cu:465-517 passes them; for the embedding these are embedding_col / embedding_row. */
static int build_params(const egg_config *c, const model_layout *L, const scales_layout *S, param_desc *P) {
    int H = c->hidden_dim, V = c->vocab_size, n = 0;
#define MAT(o, r, cl, a, b, base, hid, oi, oo) P[n++] = (param_desc){(o), (r), (cl), (a), (b), (base), 1.0f, (hid), (oi), (oo)}
#define VEC(o, len, a, b, base, sc, oi) P[n++] = (param_desc){(o), 0, (len), (a), (b), (base), (sc), 0, (oi), -1}
    for (int l = 0; l < c->n_layers; l++) {
        int sb = l * 1000; int64_t hh = (int64_t)H * H, lH = (int64_t)l * H;
        MAT(L->w_q + l * hh, H, H, 200, 201, sb, 1, S->w_q_row + lH, S->w_q_col + lH);  MAT(L->w_k + l * hh, H, H, 202, 203, sb, 1, S->w_k_row + lH, S->w_k_col + lH);
        MAT(L->w_v + l * hh, H, H, 204, 205, sb, 1, S->w_v_row + lH, S->w_v_col + lH);  MAT(L->w_o + l * hh, H, H, 206, 207, sb, 1, S->w_o_row + lH, S->w_o_col + lH);
        MAT(L->w_up + l * 4 * hh, H, 4 * H, 400, 401, sb, 1, S->w_up_row + lH, S->w_up_col + 4 * lH);
        MAT(L->w_down + l * 4 * hh, 4 * H, H, 402, 403, sb, 1, S->w_down_row + 4 * lH, S->w_down_col + lH);
        VEC(L->ln_1 + (int64_t)l * H, H, 100, 101, sb, 1.0f, S->ln_1 + lH);   VEC(L->ln_1_bias + (int64_t)l * H, H, 110, 111, sb, 1.0f, S->ln_1_bias + lH);
        VEC(L->ln_2 + (int64_t)l * H, H, 300, 301, sb, 1.0f, S->ln_2 + lH);   VEC(L->ln_2_bias + (int64_t)l * H, H, 310, 311, sb, 1.0f, S->ln_2_bias + lH);
        VEC(L->mlp_bias_up + (int64_t)l * 4 * H, 4 * H, 410, 411, sb, 1.0f, S->mlp_bias_up + 4 * lH);
        VEC(L->mlp_bias_down + (int64_t)l * H, H, 412, 413, sb, 1.0f, S->mlp_bias_down + lH);
    }
    VEC(L->ln_f, H, 900, 901, 0, 1.0f, S->ln_f);        VEC(L->ln_f_bias, H, 910, 911, 0, 1.0f, S->ln_f_bias);
    VEC(L->ln_init, H, 500, 501, 0, 1.0f, S->ln_init);     VEC(L->ln_init_bias, H, 502, 503, 0, 1.0f, S->ln_init_bias);
    MAT(L->w_emb_mlp_up, H, 4 * H, 510, 511, 0, 1, S->w_emb_mlp_up_row, S->w_emb_mlp_up_col);    VEC(L->mlp_emb_bias_up, 4 * H, 514, 515, 0, 1.0f, S->mlp_emb_bias_up);
    MAT(L->w_emb_mlp_down, 4 * H, H, 512, 513, 0, 1, S->w_emb_mlp_down_row, S->w_emb_mlp_down_col);  VEC(L->mlp_emb_bias_down, H, 516, 517, 0, 1.0f, S->mlp_emb_bias_down);
    VEC(L->emb_bias, H, 50, 51, 0, 0.1f, S->emb_bias);
    MAT(L->embedding, H, V, 0, 0 + H, 0, 0, S->embedding_col, S->embedding_row);    /* always AdamW, mgpu.cu:1636-1643 */
    if (c->ntt_mode) {          /* mgpu.cu:1645-1668: AdamW at half the learning rate, seeds 600 / 610 / 620 */
        for (int k = 0; k < 3; k++) {
            MAT(L->ntt_emb + (int64_t)k * V * H, H, V, 600 + 10 * k, 600 + 10 * k + H, 0, 0, -1, -1);
            P[n - 1].lr_scale = 0.5f;
        }
    }
#undef MAT
#undef VEC
    return n;
}

/* update_overlay_kernel (d-eggs/src/kernels.cu:61-77): +5 where something changed, -1 elsewhere, clamped */
static void overlay_step(int8_t *ov, const uint8_t *changed, int n) {
    for (int i = 0; i < n; i++) {
        int v = ov[i];
        if (changed[i]) { v += 5; if (v > 127) v = 127; } else { v -= 1; if (v < -127) v = -127; }
        ov[i] = (int8_t)v;
    }
}

uint64_t oracle_update(const egg_config *c, int8_t *model, void *opt_state, const int32_t *fitness,
                       uint32_t step_seed, float lr, int fma_mode) {
    return oracle_update_scaled(c, model, opt_state, fitness, step_seed, lr, fma_mode, NULL);
}

uint64_t oracle_update_scaled(const egg_config *c, int8_t *model, void *opt_state, const int32_t *fitness,
                              uint32_t step_seed, float lr, int fma_mode, int8_t *scales) {
    model_layout L; layout_of(c, &L);
    scales_layout SL; scales_layout_of(c, &SL);
    param_desc *P = (param_desc *)malloc(sizeof(param_desc) * (size_t)(c->n_layers * 12 + 20));
    int np = build_params(c, &L, &SL, P);
    int maxdim = 4 * c->hidden_dim > c->vocab_size ? 4 * c->hidden_dim : c->vocab_size;
    uint8_t *ch_in = (uint8_t *)malloc((size_t)maxdim), *ch_out = (uint8_t *)malloc((size_t)maxdim);
    int pairs = c->population_size / 2;
    uint64_t total_updates = 0;
    for (int i = 0; i < np; i++) {
        param_desc *d = &P[i];
        /* the field this parameter starts in, to locate its optimiser state */
        int64_t field_off, within;
        {
            int64_t H = c->hidden_dim;
            int64_t starts[] = {L.embedding, L.emb_bias, L.ntt_emb, L.ln_init, L.ln_init_bias, L.w_emb_mlp_up,
                                L.mlp_emb_bias_up, L.w_emb_mlp_down, L.mlp_emb_bias_down, L.ln_1, L.ln_1_bias,
                                L.w_q, L.w_k, L.w_v, L.w_o, L.ln_2, L.ln_2_bias, L.w_up, L.mlp_bias_up,
                                L.w_down, L.mlp_bias_down, L.ln_f, L.ln_f_bias};
            field_off = 0; (void)H;
            for (unsigned s = 0; s < sizeof(starts) / sizeof(starts[0]); s++)
                if (starts[s] <= d->off) field_off = starts[s];
            within = d->off - field_off;
        }
        int muon = d->hidden && c->use_muon;
        int esz = muon ? 8 : 12;
        char *st = (char *)opt_state + opt_offset_of(c, &L, field_off) + within * esz;
        int64_t count = d->rows ? (int64_t)d->rows * d->cols : d->cols;
        int32_t *vote = (int32_t *)malloc(sizeof(int32_t) * (size_t)count);
        float plr = lr * d->lr_scale;
        if (d->rows) oracle_vote_matrix(c, fitness, pairs, d->rows, d->cols, d->off_a, d->off_b, d->seed_base, step_seed, vote);
        else vote_vector(c, fitness, pairs, d->cols, d->off_a, d->off_b, d->seed_base, step_seed, vote);
        int8_t *w = model + d->off;
        if (!muon) {
            memset(ch_in, 0, (size_t)maxdim); memset(ch_out, 0, (size_t)maxdim);
            for (int64_t j = 0; j < count; j++) {
                float *s = (float *)(st + j * 12);
                int ch = oracle_adam_step(c, &s[0], &s[1], &s[2], &w[j], -(float)vote[j], plr, fma_mode);
                total_updates += (uint64_t)ch;
                if (ch) {
                    if (d->rows) { ch_out[(j >> 2) % d->cols] = 1; ch_in[((j >> 2) / d->cols) * 4 + (j & 3)] = 1; }
                    else ch_in[j] = 1;
                }
            }
            if (scales && d->ov_in >= 0) {   /* worker.cu:445-463: overlay of the input index, then of the output index */
                overlay_step(scales + d->ov_in, ch_in, d->rows ? d->rows : d->cols);
                if (d->rows) overlay_step(scales + d->ov_out, ch_out, d->cols);
            }
        } else {
            /* muon_internal.cuh:15-50 momentum, :53-74 gather, NS, :112-166 apply */
            int R = d->rows, C = d->cols;
            float *buf = (float *)malloc(sizeof(float) * (size_t)count);
            for (int64_t j = 0; j < count; j++) {
                float *s = (float *)(st + j * 8);
                s[0] = fma_mode ? fmaf(c->muon_momentum, s[0], (float)vote[j]) : (c->muon_momentum * s[0] + (float)vote[j]);
                int n = (int)((j >> 2) % C), k = (int)((j >> 2) / C) * 4 + (int)(j & 3);
                buf[(int64_t)k * C + n] = s[0];
            }
            oracle_newton_schulz(buf, R, C);
            float mlr = lr * c->muon_lr_scale;
            for (int64_t j = 0; j < count; j++) {
                float *s = (float *)(st + j * 8);
                int n = (int)((j >> 2) % C), k = (int)((j >> 2) / C) * 4 + (int)(j & 3);
                float u = buf[(int64_t)k * C + n];
                float inner = fma_mode ? fmaf(c->adam_weight_decay, (float)w[j], u) : (u + c->adam_weight_decay * (float)w[j]);
                s[1] = fma_mode ? fmaf(-mlr, inner, s[1]) : (s[1] + (-mlr * inner));
                total_updates += (uint64_t)quantized_update(&w[j], &s[1]);
            }
            free(buf);
        }
        free(vote);
    }
    free(P); free(ch_in); free(ch_out);
    return total_updates;
}

/* ----------------------------------------------------- isolated projection */

void oracle_projection(const egg_config *cfg, const int8_t *x, const int8_t *w_packed, int8_t *y, int64_t rows,
                       int K, int N, int rows_per_member, uint32_t seed, int off_a, int off_b, int rank1_shift,
                       int out_shift) {
    /* the packed [K/4][N][4] weights once as [N][K] so that the inner sums run over contiguous bytes; the noise
     * vectors of a pair once per row (they are functions of the pair only) */
    int8_t *wt = (int8_t *)malloc((size_t)K * N);
    for (int n = 0; n < N; n++)
        for (int k = 0; k < K; k++) wt[(int64_t)n * K + k] = (int8_t)wq(w_packed, k, n, N);
#pragma omp parallel
    {
        int8_t *nb = (int8_t *)malloc((size_t)K), *na = (int8_t *)malloc((size_t)N);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; r++) {
            int64_t member = r / rows_per_member;
            uint32_t s = seed + (uint32_t)(member / 2);
            int ns = (member % 2 == 0) ? 1 : -1;
            const int8_t *xr = x + r * K;
            for (int k = 0; k < K; k++) nb[k] = (int8_t)oracle_noise(cfg, s + (uint32_t)off_b, (uint32_t)k);
            for (int n = 0; n < N; n++) na[n] = (int8_t)oracle_noise(cfg, s + (uint32_t)off_a, (uint32_t)n);
            int32_t xb = 0;
            for (int k = 0; k < K; k++) xb += (int32_t)xr[k] * nb[k];
            for (int n = 0; n < N; n++) {
                const int8_t *wn = wt + (int64_t)n * K;
                int32_t acc = 0;
                for (int k = 0; k < K; k++) acc += (int32_t)xr[k] * wn[k];
                acc += ((xb * (int32_t)na[n]) * ns) >> rank1_shift;
                y[r * N + n] = (int8_t)clip8(acc >> out_shift);
            }
        }
        free(nb); free(na);
    }
    free(wt);
}

/* Votes of selected output columns n of one matrix (mgpu.cu:1085-1098): out[i][k] = Σ_p f_p · A_p[n_i] · B_p[k].
 * The whole vote matrix of a 4096 x 4096 weight with 32 768 pairs is 5.5e11 terms; a sample of columns is what a
 * CPU can check. */
void oracle_vote_columns(const egg_config *cfg, const int32_t *fitness, int pairs, int rows_k, int off_a, int off_b,
                         int seed_base, uint32_t step_seed, const int32_t *n_list, int n_count, int32_t *out) {
    int8_t *B = (int8_t *)malloc((size_t)pairs * rows_k);
    int32_t *FA = (int32_t *)malloc(sizeof(int32_t) * (size_t)pairs * n_count);
#pragma omp parallel for schedule(static)
    for (int p = 0; p < pairs; p++) {
        uint32_t s = step_seed + (uint32_t)p + (uint32_t)seed_base;
        for (int k = 0; k < rows_k; k++) B[(int64_t)p * rows_k + k] = (int8_t)oracle_noise(cfg, s + (uint32_t)off_b, (uint32_t)k);
        for (int i = 0; i < n_count; i++) FA[(int64_t)p * n_count + i] = fitness[p] * oracle_noise(cfg, s + (uint32_t)off_a, (uint32_t)n_list[i]);
    }
#pragma omp parallel for schedule(static)
    for (int i = 0; i < n_count; i++) {
        int32_t *o = out + (int64_t)i * rows_k;
        for (int k = 0; k < rows_k; k++) o[k] = 0;
        for (int p = 0; p < pairs; p++) {
            int32_t fa = FA[(int64_t)p * n_count + i];
            if (!fa) continue;
            const int8_t *b = B + (int64_t)p * rows_k;
            for (int k = 0; k < rows_k; k++) o[k] += fa * b[k];
        }
    }
    free(B); free(FA);
}

/* ES-AdamW on an array of elements from their votes (update_matrix_adam_kernel's tail, mgpu.cu:1100-1110):
 * state = AdamParam{m, v, acc} per element; returns the number of weights that changed. */
uint64_t oracle_adam_from_votes(const egg_config *cfg, int8_t *w, float *state, const int32_t *vote, int64_t count, float lr,
                                int fma_mode) {
    uint64_t changed = 0;
    for (int64_t j = 0; j < count; j++)
        changed += (uint64_t)oracle_adam_step(cfg, &state[3 * j], &state[3 * j + 1], &state[3 * j + 2], &w[j], -(float)vote[j], lr, fma_mode);
    return changed;
}

/* ------------------------------------------------- d-eggs per-chunk fitness */

/* d-eggs/src/worker.cu:635-687 with CHUNK_MEAN_FILTER and USE_ADAPTIVE_THRESHOLD as flags */
void oracle_deggs_chunk_fitness(const int32_t *losses, int count, int mean_filter, double exponent, int adaptive,
                                double alpha, int32_t *fit, int64_t *sum_loss) {
    int num = count / 2;
    int32_t *diffs = (int32_t *)malloc(sizeof(int32_t) * (size_t)num);
    int64_t sl = 0; double sum_diff_val = 0.0;
    for (int i = 0; i < num; i++) {
        int32_t p = losses[2 * i], n = losses[2 * i + 1];
        sl += p + n;
        diffs[i] = n - p;
        sum_diff_val += diffs[i];
    }
    if (mean_filter) {
        double mean_diff = sum_diff_val / num;
        if (mean_diff != 0.0) {
            double sign = (mean_diff > 0) ? 1.0 : -1.0;
            mean_diff = sign * pow(fabs(mean_diff), exponent);
        }
        for (int i = 0; i < num; i++) diffs[i] += (int32_t)mean_diff;
    }
    if (adaptive) {
        double sum_abs_diff = 0.0;
        for (int i = 0; i < num; i++) sum_abs_diff += fabs((double)diffs[i]);
        double threshold = (sum_abs_diff / num) * alpha;
        for (int i = 0; i < num; i++) fit[i] = (fabs((double)diffs[i]) < threshold) ? 0 : ((diffs[i] > 0) ? 1 : -1);
    } else {
        for (int i = 0; i < num; i++) fit[i] = (diffs[i] > 0) ? 1 : ((diffs[i] < 0) ? -1 : 0);
    }
    if (sum_loss) *sum_loss = sl;
    free(diffs);
}

/* --------------------------------------------------------- ternary codec */

/* d-eggs/include/utils/ternary_pack.h:12-14 */
int64_t oracle_ternary_packed_size(int64_t count) { return (count + 4) / 5; }

/* ternary_pack.h:16-52: digit = (v+3)%3, little-endian base 3, 5 per byte */
void oracle_ternary_pack(const int32_t *values, int64_t count, uint8_t *out) {
    int64_t o = 0;
    for (int64_t i = 0; i < count; i += 5) {
        int val = 0, mult = 1;
        for (int64_t j = i; j < i + 5 && j < count; j++) { val += ((values[j] + 3) % 3) * mult; mult *= 3; }
        out[o++] = (uint8_t)val;
    }
}

/* ternary_pack.h:54-87 */
void oracle_ternary_unpack(const uint8_t *in, int64_t count, int32_t *values) {
    int64_t o = 0;
    for (int64_t i = 0; i < count; i += 5) {
        int val = in[o++];
        for (int64_t j = i; j < i + 5 && j < count; j++) { int v = val % 3; val /= 3; values[j] = (v == 2) ? -1 : v; }
    }
}
