// Drives the d-eggs worker's own kernels (train_sequence_kernel with AdaptiveScales,
// update_*_adam_kernel with change counters, update_overlay_kernel) over several
// generations with fixed seeds, so that losses, weights, optimiser state and noise
// overlays can be compared bit for bit.  TEST INFRASTRUCTURE ONLY.  The reference
// sources are #include'd from where they lie (never copied).  One binary per
// compile-time configuration, built by oracle/Makefile into oracle/_ref/.
//
//   ref_deggs_<tag> <in.bin> <out.bin>
//   ref_deggs_<tag> --generate <in.bin> <out.bin>      (generate_sequence_kernel, see below)
//
// in.bin : struct deggs_case_header, TransformerModel, AdamModel, AdaptiveScales, dataset bytes
// out.bin: per generation: int32 losses[POPULATION_SIZE], uint64 updates, AdaptiveScales;
//          then TransformerModel, AdamModel
//
// Per generation (d-eggs/src/worker.cu:430-545, 617-622): every chunk of the population is
// evaluated with the current seed at start index step*SEQ_LEN, fitness is the sign of the pair's
// loss difference (compute_fitness_kernel), every parameter is updated followed by its overlay
// update(s), then seed = hash_rng(seed, step + 1) and step += 1.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string>

#include "protocol.h"
#include "config.h"
#include "model/definitions.h"
#include "utils/egg_math.h"
#include "optimizer/adam.cuh"
#include REF_KERNELS_INCLUDE

struct deggs_case_header {
    uint32_t magic;        // 0x53474745 "EGGS"
    uint32_t seed;
    int64_t step;
    int64_t data_len;
    int32_t generations;
    float lr;
    int32_t cfg_check[6];  // hidden_dim, n_layers, seq_len, population_size, device_mask, chunk_size
};

static void die(const char *m) { fprintf(stderr, "d-eggs harness: %s\n", m); exit(2); }
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "CUDA %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(1); } } while (0)

int main(int argc, char **argv) {
    if (argc == 2 && std::string(argv[1]) == "--sizes") {
        printf("{\"model_bytes\": %zu, \"opt_bytes\": %zu, \"scales_bytes\": %zu, \"hidden_dim\": %d, \"head_dim\": %d, \"n_layers\": %d, "
               "\"seq_len\": %d, \"vocab_size\": %d, \"population_size\": %d, \"device_mask\": %d, \"chunk_size\": %d, "
               "\"fixed_point\": %d, \"sigma_shift\": %d, \"sigma_shift_vector\": %d, \"softmax_scale_bit\": %d, "
               "\"softmax_exp_scale\": %.17g, \"rope_scale_bit\": %d, \"shift_attn\": %d, \"shift_qkv\": %d, \"shift_out\": %d, "
               "\"shift_logit\": %d, \"shift_mlp_up\": %d, \"shift_mlp_down\": %d, \"use_same_data\": %d, \"device_gaussian\": %d, "
               "\"adam_beta1\": %.9g, \"adam_beta2\": %.9g, \"adam_eps\": %.9g, \"adam_weight_decay\": %.9g, "
               "\"adaptive_noise_mode\": %d, \"adaptive_noise_inc\": %d, \"adaptive_noise_dec\": %d, \"adaptive_noise_init\": %d}\n",
               sizeof(TransformerModel), sizeof(AdamModel), sizeof(AdaptiveScales), HIDDEN_DIM, HEAD_DIM, N_LAYERS, SEQ_LEN,
               VOCAB_SIZE, POPULATION_SIZE, DEVICE_MASK, CHUNK_SIZE, FIXED_POINT, SIGMA_SHIFT, SIGMA_SHIFT_VECTOR,
               SOFTMAX_SCALE_BIT, (double)SOFTMAX_EXP_SCALE, ROPE_SCALE_BIT, SHIFT_ATTN, SHIFT_QKV, SHIFT_OUT, SHIFT_LOGIT,
               SHIFT_MLP_UP, SHIFT_MLP_DOWN, USE_SAME_DATA, (int)DEVICE_GAUSSIAN, (double)ADAM_BETA1, (double)ADAM_BETA2,
               (double)ADAM_EPS, (double)ADAM_WEIGHT_DECAY, ADAPTIVE_NOISE_MODE, ADAPTIVE_NOISE_INC, ADAPTIVE_NOISE_DEC,
               ADAPTIVE_NOISE_INIT);
        return 0;
    }
    if (argc == 4 && std::string(argv[1]) == "--generate") {
        // in : struct {u32 magic "EGGG", u32 seed, i32 seed_len, i32 gen_len, f32 temp, f32 min_p, f32 penalty, i32 cfg_check[3]},
        //      TransformerModel, seed_len token bytes;   out: seed_len + gen_len token bytes
        // ≙ worker.cu:563-573: generate_sequence_kernel<<<1, EGG_BLOCK_THREADS, sm_size>>>(buf, seed_len, gen_len, model, kv, seed, temp, min_p, penalty)
        struct { uint32_t magic, seed; int32_t seed_len, gen_len; float temp, min_p, penalty; int32_t cfg_check[3]; } g;
        FILE *f = fopen(argv[2], "rb");
        if (!f || fread(&g, sizeof(g), 1, f) != 1 || g.magic != 0x47474745u) die("bad generate header");
        const int want[3] = {HIDDEN_DIM, N_LAYERS, SEQ_LEN};
        for (int i = 0; i < 3; i++) if (g.cfg_check[i] != want[i]) { fprintf(stderr, "d-eggs harness: case was made for another configuration\n"); return 3; }
        const int total = g.seed_len + g.gen_len;
        if (g.seed_len < 1 || g.gen_len < 0 || total > SEQ_LEN || total > 256) die("bad lengths");
        TransformerModel *h_model = (TransformerModel *)calloc(1, sizeof(TransformerModel));
        if (fread(h_model, sizeof(TransformerModel), 1, f) != 1) die("short model");
        uint8_t raw[256] = {0};
        if (fread(raw, 1, g.seed_len, f) != (size_t)g.seed_len) die("short tokens");
        fclose(f);
        TokenType h_buf[256] = {0};
        for (int i = 0; i < g.seed_len; i++) h_buf[i] = raw[i];
        CK(cudaSetDevice(0));
        init_tables();
        copy_tables_to_device();
        TransformerModel *d_model; TokenType *d_buf; ActType *d_kv;
        CK(cudaMalloc(&d_model, sizeof(TransformerModel)));
        CK(cudaMalloc(&d_buf, 256 * sizeof(TokenType)));
        CK(cudaMalloc(&d_kv, (size_t)N_LAYERS * 2 * total * HIDDEN_DIM));
        CK(cudaMemset(d_kv, 0, (size_t)N_LAYERS * 2 * total * HIDDEN_DIM));
        CK(cudaMemcpy(d_model, h_model, sizeof(TransformerModel), cudaMemcpyHostToDevice));
        CK(cudaMemcpy(d_buf, h_buf, sizeof(h_buf), cudaMemcpyHostToDevice));
        const size_t sm = 2 * HIDDEN_DIM + 512 + (4 * HIDDEN_DIM);
        generate_sequence_kernel<<<1, EGG_BLOCK_THREADS, sm>>>(d_buf, g.seed_len, g.gen_len, d_model, d_kv, g.seed, g.temp, g.min_p, g.penalty);
        CK(cudaDeviceSynchronize());
        CK(cudaMemcpy(h_buf, d_buf, sizeof(h_buf), cudaMemcpyDeviceToHost));
        FILE *o = fopen(argv[3], "wb");
        if (!o) die("cannot open output");
        for (int i = 0; i < total; i++) { uint8_t b = (uint8_t)h_buf[i]; fwrite(&b, 1, 1, o); }
        fclose(o);
        printf("{\"ref\": \"d-eggs generate\", \"total\": %d}\n", total);
        return 0;
    }
    if (argc < 3) die("usage: ref_deggs_<tag> in.bin out.bin | --generate in.bin out.bin | --sizes");
    FILE *f = fopen(argv[1], "rb");
    if (!f) die("cannot open input");
    deggs_case_header h;
    if (fread(&h, sizeof(h), 1, f) != 1 || h.magic != 0x53474745u) die("bad header");
    {
        const int want[6] = {HIDDEN_DIM, N_LAYERS, SEQ_LEN, POPULATION_SIZE, DEVICE_MASK, CHUNK_SIZE};
        for (int i = 0; i < 6; i++)
            if (h.cfg_check[i] != want[i]) { fprintf(stderr, "d-eggs harness: case was made for another configuration (field %d: %d vs compiled %d)\n", i, h.cfg_check[i], want[i]); return 3; }
    }
    TransformerModel *h_model = (TransformerModel *)calloc(1, sizeof(TransformerModel));
    AdamModel *h_opt = (AdamModel *)calloc(1, sizeof(AdamModel));
    AdaptiveScales *h_scales = (AdaptiveScales *)calloc(1, sizeof(AdaptiveScales));
    if (fread(h_model, sizeof(TransformerModel), 1, f) != 1) die("short model");
    if (fread(h_opt, sizeof(AdamModel), 1, f) != 1) die("short opt state");
    if (fread(h_scales, sizeof(AdaptiveScales), 1, f) != 1) die("short scales");
    TokenType *h_data = (TokenType *)malloc(h.data_len * sizeof(TokenType));
    {
        uint8_t *raw = (uint8_t *)malloc(h.data_len);
        if (fread(raw, 1, h.data_len, f) != (size_t)h.data_len) die("short dataset");
        for (int64_t i = 0; i < h.data_len; i++) h_data[i] = raw[i];
        free(raw);
    }
    fclose(f);
    if (POPULATION_SIZE % CHUNK_SIZE) die("population must be whole chunks");

    CK(cudaSetDevice(0));
    init_tables();
    copy_tables_to_device();

    cudaStream_t stream; CK(cudaStreamCreate(&stream));
    TransformerModel *d_model; AdamModel *d_opt; AdaptiveScales *d_scales; TokenType *d_dataset;
    int32_t *d_loss, *d_fit; ActType *d_kv; int *d_row_accum, *d_col_accum;
    uint32_t *d_seed; float *d_lr, *d_lr_bias;
    CK(cudaMalloc(&d_model, sizeof(TransformerModel)));
    CK(cudaMalloc(&d_opt, sizeof(AdamModel)));
    CK(cudaMalloc(&d_scales, sizeof(AdaptiveScales)));
    CK(cudaMalloc(&d_dataset, h.data_len * sizeof(TokenType)));
    CK(cudaMalloc(&d_loss, POPULATION_SIZE * sizeof(int32_t)));
    CK(cudaMalloc(&d_fit, (POPULATION_SIZE / 2) * sizeof(int32_t)));
    CK(cudaMalloc(&d_kv, (size_t)CHUNK_SIZE * N_LAYERS * 2 * SEQ_LEN * HIDDEN_DIM));
    const int accum_n = (4 * HIDDEN_DIM > VOCAB_SIZE) ? 4 * HIDDEN_DIM : VOCAB_SIZE;
    CK(cudaMalloc(&d_row_accum, accum_n * sizeof(int)));
    CK(cudaMalloc(&d_col_accum, accum_n * sizeof(int)));
    CK(cudaMalloc(&d_seed, 4)); CK(cudaMalloc(&d_lr, 4)); CK(cudaMalloc(&d_lr_bias, 4));
    CK(cudaMemcpy(d_model, h_model, sizeof(TransformerModel), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_opt, h_opt, sizeof(AdamModel), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_scales, h_scales, sizeof(AdaptiveScales), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_dataset, h_data, h.data_len * sizeof(TokenType), cudaMemcpyHostToDevice));
    unsigned long long *d_updates_ptr;
    CK(cudaGetSymbolAddress((void **)&d_updates_ptr, d_total_updates));

    FILE *o = fopen(argv[2], "wb");
    if (!o) die("cannot open output");
    int32_t *h_loss = (int32_t *)malloc(POPULATION_SIZE * sizeof(int32_t));
    uint32_t seed = h.seed;
    uint64_t step = (uint64_t)h.step;
    const int H = HIDDEN_DIM;
    const size_t sm_size = 2 * HIDDEN_DIM + 512 + (4 * HIDDEN_DIM);

    for (int g = 0; g < h.generations; g++) {
        for (int off = 0; off < POPULATION_SIZE; off += CHUNK_SIZE)
            train_sequence_kernel<<<CHUNK_SIZE, EGG_BLOCK_THREADS, sm_size, stream>>>(
                d_dataset, (long)h.data_len, (int)(step * SEQ_LEN), d_model, d_kv, d_loss + off, seed, off, (long)step, d_scales);
        compute_fitness_kernel<<<(POPULATION_SIZE / 2 + 255) / 256, 256, 0, stream>>>(d_loss, d_fit, POPULATION_SIZE / 2);
        CK(cudaStreamSynchronize(stream));
        CK(cudaGetLastError());
        CK(cudaMemcpy(h_loss, d_loss, POPULATION_SIZE * sizeof(int32_t), cudaMemcpyDeviceToHost));

        float lr = h.lr, lr_bias = h.lr * 0.1f;
        CK(cudaMemcpyAsync(d_seed, &seed, 4, cudaMemcpyHostToDevice, stream));
        CK(cudaMemcpyAsync(d_lr, &lr, 4, cudaMemcpyHostToDevice, stream));
        CK(cudaMemcpyAsync(d_lr_bias, &lr_bias, 4, cudaMemcpyHostToDevice, stream));
        CK(cudaMemsetAsync(d_updates_ptr, 0, sizeof(unsigned long long), stream));
        // This harness's own statement of the worker's launch list: (rows, cols, off_A, off_B,
        // seed base, learning-rate source, overlay over the input index, overlay over the output index).
        auto overlay = [&](int *accum, WeightType *ov, int count) {
            if (ADAPTIVE_NOISE_MODE > 0) update_overlay_kernel<<<(count + 255) / 256, 256, 0, stream>>>(accum, ov, count);
        };
        auto mat = [&](WeightType *w, AdamParam *st, int rows, int cols, int a, int b, int base, WeightType *ov_in, WeightType *ov_out) {
            cudaMemsetAsync(d_row_accum, 0, rows * sizeof(int), stream);
            cudaMemsetAsync(d_col_accum, 0, cols * sizeof(int), stream);
            update_matrix_adam_kernel<<<(rows * cols + 511) / 512, 512, 0, stream>>>(w, st, rows, cols, a, b, base, d_fit, d_seed, d_lr, d_row_accum, d_col_accum);
            overlay(d_row_accum, ov_in, rows);
            overlay(d_col_accum, ov_out, cols);
        };
        auto vec = [&](WeightType *v, AdamParam *st, int len, int a, int b, int base, const float *lrp, WeightType *ov) {
            cudaMemsetAsync(d_row_accum, 0, len * sizeof(int), stream);
            update_vector_adam_kernel<<<(len + 255) / 256, 256, 0, stream>>>(v, st, len, a, b, base, d_fit, d_seed, lrp, d_row_accum);
            overlay(d_row_accum, ov, len);
        };
        for (int l = 0; l < N_LAYERS; l++) {
            int sb = l * 1000;
            mat(d_model->w_q[l], (AdamParam *)d_opt->w_q[l], H, H, SEED_OFF_Q_A, SEED_OFF_Q_B, sb, d_scales->w_q_row[l], d_scales->w_q_col[l]);
            mat(d_model->w_k[l], (AdamParam *)d_opt->w_k[l], H, H, SEED_OFF_K_A, SEED_OFF_K_B, sb, d_scales->w_k_row[l], d_scales->w_k_col[l]);
            mat(d_model->w_v[l], (AdamParam *)d_opt->w_v[l], H, H, SEED_OFF_V_A, SEED_OFF_V_B, sb, d_scales->w_v_row[l], d_scales->w_v_col[l]);
            mat(d_model->w_o[l], (AdamParam *)d_opt->w_o[l], H, H, SEED_OFF_O_A, SEED_OFF_O_B, sb, d_scales->w_o_row[l], d_scales->w_o_col[l]);
            mat(d_model->w_up[l], (AdamParam *)d_opt->w_up[l], H, 4 * H, SEED_OFF_MLP_UP_A, SEED_OFF_MLP_UP_B, sb, d_scales->w_up_row[l], d_scales->w_up_col[l]);
            mat(d_model->w_down[l], (AdamParam *)d_opt->w_down[l], 4 * H, H, SEED_OFF_MLP_DOWN_A, SEED_OFF_MLP_DOWN_B, sb, d_scales->w_down_row[l], d_scales->w_down_col[l]);
            vec(d_model->ln_1[l], d_opt->ln_1[l], H, SEED_OFF_LN_1_A, SEED_OFF_LN_1_B, sb, d_lr, d_scales->ln_1[l]);
            vec(d_model->ln_1_bias[l], d_opt->ln_1_bias[l], H, SEED_OFF_LN_1_BIAS_A, SEED_OFF_LN_1_BIAS_B, sb, d_lr, d_scales->ln_1_bias[l]);
            vec(d_model->ln_2[l], d_opt->ln_2[l], H, SEED_OFF_LN_2_A, SEED_OFF_LN_2_B, sb, d_lr, d_scales->ln_2[l]);
            vec(d_model->ln_2_bias[l], d_opt->ln_2_bias[l], H, SEED_OFF_LN_2_BIAS_A, SEED_OFF_LN_2_BIAS_B, sb, d_lr, d_scales->ln_2_bias[l]);
            vec(d_model->mlp_bias_up[l], d_opt->mlp_bias_up[l], 4 * H, SEED_OFF_MLP_BIAS_UP_A, SEED_OFF_MLP_BIAS_UP_B, sb, d_lr, d_scales->mlp_bias_up[l]);
            vec(d_model->mlp_bias_down[l], d_opt->mlp_bias_down[l], H, SEED_OFF_MLP_BIAS_DOWN_A, SEED_OFF_MLP_BIAS_DOWN_B, sb, d_lr, d_scales->mlp_bias_down[l]);
        }
        vec(d_model->ln_f, d_opt->ln_f, H, SEED_OFF_LN_F_A, SEED_OFF_LN_F_B, 0, d_lr, d_scales->ln_f);
        vec(d_model->ln_f_bias, d_opt->ln_f_bias, H, SEED_OFF_LN_F_BIAS_A, SEED_OFF_LN_F_BIAS_B, 0, d_lr, d_scales->ln_f_bias);
        vec(d_model->ln_init, d_opt->ln_init, H, SEED_OFF_LN_INIT_A, SEED_OFF_LN_INIT_B, 0, d_lr, d_scales->ln_init);
        vec(d_model->ln_init_bias, d_opt->ln_init_bias, H, SEED_OFF_LN_INIT_BIAS_A, SEED_OFF_LN_INIT_BIAS_B, 0, d_lr, d_scales->ln_init_bias);
        mat(d_model->w_emb_mlp_up, (AdamParam *)d_opt->w_emb_mlp_up, H, 4 * H, SEED_OFF_EMB_MLP_UP_A, SEED_OFF_EMB_MLP_UP_B, 0, d_scales->w_emb_mlp_up_row, d_scales->w_emb_mlp_up_col);
        vec(d_model->mlp_emb_bias_up, d_opt->mlp_emb_bias_up, 4 * H, SEED_OFF_EMB_MLP_BIAS_UP_A, SEED_OFF_EMB_MLP_BIAS_UP_B, 0, d_lr, d_scales->mlp_emb_bias_up);
        mat(d_model->w_emb_mlp_down, (AdamParam *)d_opt->w_emb_mlp_down, 4 * H, H, SEED_OFF_EMB_MLP_DOWN_A, SEED_OFF_EMB_MLP_DOWN_B, 0, d_scales->w_emb_mlp_down_row, d_scales->w_emb_mlp_down_col);
        vec(d_model->mlp_emb_bias_down, d_opt->mlp_emb_bias_down, H, SEED_OFF_EMB_MLP_BIAS_DOWN_A, SEED_OFF_EMB_MLP_BIAS_DOWN_B, 0, d_lr, d_scales->mlp_emb_bias_down);
        vec(d_model->emb_bias, d_opt->emb_bias, H, SEED_OFF_EMB_BIAS_A, SEED_OFF_EMB_BIAS_B, 0, d_lr_bias, d_scales->emb_bias);
        mat(d_model->embedding, d_opt->embedding, H, VOCAB_SIZE, SEED_OFF_EMB, SEED_OFF_EMB + H, 0, d_scales->embedding_col, d_scales->embedding_row);
        CK(cudaStreamSynchronize(stream));
        CK(cudaGetLastError());
        unsigned long long h_updates = 0;
        CK(cudaMemcpy(&h_updates, d_updates_ptr, sizeof(h_updates), cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(h_scales, d_scales, sizeof(AdaptiveScales), cudaMemcpyDeviceToHost));
        fwrite(h_loss, sizeof(int32_t), POPULATION_SIZE, o);
        uint64_t u = h_updates; fwrite(&u, sizeof(u), 1, o);
        fwrite(h_scales, sizeof(AdaptiveScales), 1, o);
        step += 1;
        seed = hash_rng(seed, (uint32_t)step);
    }
    CK(cudaMemcpy(h_model, d_model, sizeof(TransformerModel), cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(h_opt, d_opt, sizeof(AdamModel), cudaMemcpyDeviceToHost));
    fwrite(h_model, sizeof(TransformerModel), 1, o);
    fwrite(h_opt, sizeof(AdamModel), 1, o);
    fclose(o);
    printf("{\"ref\": \"d-eggs\", \"hidden_dim\": %d, \"n_layers\": %d, \"seq_len\": %d, \"population_size\": %d, \"generations\": %d}\n",
           HIDDEN_DIM, N_LAYERS, SEQ_LEN, POPULATION_SIZE, h.generations);
    return 0;
}
