// Drives the REFERENCE's own kernels (train_sequence_kernel, update_*_adam_kernel,
// Muon) with fixed seeds so that their outputs can be compared bit for bit.
// TEST INFRASTRUCTURE ONLY.  The reference translation unit is #include'd from
// where it lies (never copied); its main() is renamed away.  One binary per
// compile-time configuration, built by oracle/Makefile into oracle/_ref/.
//
//   ref_mgpu_<tag> <in.bin> <out.bin>
//
// in.bin : struct ref_case_header, TransformerModel bytes, [AdamModel bytes], data_len tokens of the reference's
//          TokenType (bytes at VOCAB_SIZE 256, uint32_t otherwise)
// out.bin: int32 losses[count]; if do_update: int32 fitness[POP/2], uint64 total_updates,
//          TransformerModel bytes, AdamModel bytes
// stdout : one JSON line with the configuration and kernel timings.
#define main ref_main_unused
#include REF_DIR_INCLUDE
#undef main

#include <string>

struct ref_case_header {
    uint32_t magic;        // 0x46524745 "EGRF"
    uint32_t step_seed;
    int64_t start_idx;
    int64_t data_len;      // tokens
    int32_t pop_offset;
    int32_t count;
    float lr;
    int32_t do_update;     // needs pop_offset == 0 && count == POPULATION_SIZE
    int32_t has_opt;
    int32_t vocab_size;    // 0: not checked (cases written before the field had a meaning)
    int32_t cfg_check[6];  // hidden_dim, n_layers, seq_len, population_size, device_mask, use_muon
};

static void die(const char *m) { fprintf(stderr, "ref harness: %s\n", m); exit(2); }

int main(int argc, char **argv) {
    if (argc == 2 && std::string(argv[1]) == "--sizes") {
        printf("{\"model_bytes\": %zu, \"opt_bytes\": %zu, \"hidden_dim\": %d, \"head_dim\": %d, \"n_layers\": %d, "
               "\"seq_len\": %d, \"vocab_size\": %d, \"population_size\": %d, \"device_mask\": %d, \"use_muon\": %d, \"ntt_mode\": %d}\n",
               sizeof(TransformerModel), sizeof(AdamModel), HIDDEN_DIM, HEAD_DIM, N_LAYERS, SEQ_LEN, VOCAB_SIZE,
               POPULATION_SIZE, DEVICE_MASK, USE_MUON, NTT_MODE);
        return 0;
    }
    if (argc < 3) die("usage: ref_mgpu_<tag> in.bin out.bin | --sizes");
    FILE *f = fopen(argv[1], "rb");
    if (!f) die("cannot open input");
    ref_case_header h;
    if (fread(&h, sizeof(h), 1, f) != 1 || h.magic != 0x46524745u) die("bad header");
    {
        const int want[6] = {HIDDEN_DIM, N_LAYERS, SEQ_LEN, POPULATION_SIZE, DEVICE_MASK, USE_MUON};
        for (int i = 0; i < 6; i++)
            if (h.cfg_check[i] != want[i]) { fprintf(stderr, "ref harness: case was made for another configuration (field %d: %d vs compiled %d)\n", i, h.cfg_check[i], want[i]); return 3; }
    }
    if (h.vocab_size != 0 && h.vocab_size != VOCAB_SIZE) { fprintf(stderr, "ref harness: case was made for vocab_size %d, compiled %d\n", h.vocab_size, VOCAB_SIZE); return 3; }
    const size_t data_bytes = (size_t)h.data_len * sizeof(TokenType);
    TransformerModel *h_model = (TransformerModel *)calloc(1, sizeof(TransformerModel));
    AdamModel *h_opt = (AdamModel *)calloc(1, sizeof(AdamModel));
    if (fread(h_model, sizeof(TransformerModel), 1, f) != 1) die("short model");
    if (h.has_opt && fread(h_opt, sizeof(AdamModel), 1, f) != 1) die("short opt state");
    uint8_t *h_data = (uint8_t *)malloc(data_bytes);
    if (fread(h_data, 1, data_bytes, f) != data_bytes) die("short dataset");
    fclose(f);
    if (h.count <= 0 || h.pop_offset < 0 || h.pop_offset + h.count > POPULATION_SIZE) die("bad population range");
    if (h.do_update && (h.pop_offset != 0 || h.count != POPULATION_SIZE)) die("update needs the whole population");

    CHECK_CUDA(cudaSetDevice(0));
    init_tables();
    cudaMemcpyToSymbol(d_EXP_LUT, h_EXP_LUT, SOFTMAX_LUT_SIZE * sizeof(int32_t));
    cudaMemcpyToSymbol(d_ACT_LUT, h_ACT_LUT, 256 * sizeof(int8_t));
    cudaMemcpyToSymbol(d_ROPE_LUT, h_ROPE_LUT, ROPE_LUT_SIZE * sizeof(int32_t));

    cudaStream_t stream; CHECK_CUDA(cudaStreamCreate(&stream));
    TransformerModel *d_model; AdamModel *d_opt; TokenType *d_dataset; int32_t *d_loss, *d_fit; ActType *d_kv;
    CHECK_CUDA(cudaMalloc(&d_model, sizeof(TransformerModel)));
    CHECK_CUDA(cudaMalloc(&d_opt, sizeof(AdamModel)));
    CHECK_CUDA(cudaMalloc(&d_dataset, data_bytes));
    CHECK_CUDA(cudaMalloc(&d_loss, POPULATION_SIZE * sizeof(int32_t)));
    CHECK_CUDA(cudaMalloc(&d_fit, (POPULATION_SIZE / 2) * sizeof(int32_t)));
    int batch_cap = h.count < POPULATION_BATCH_SIZE ? h.count : POPULATION_BATCH_SIZE;
    size_t kv_size = (size_t)batch_cap * N_LAYERS * 2 * SEQ_LEN * HIDDEN_DIM;
    CHECK_CUDA(cudaMalloc(&d_kv, kv_size));
    CHECK_CUDA(cudaMemcpy(d_model, h_model, sizeof(TransformerModel), cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(d_opt, h_opt, sizeof(AdamModel), cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(d_dataset, h_data, data_bytes, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemset(d_loss, 0, POPULATION_SIZE * sizeof(int32_t)));

    cudaEvent_t e0, e1, e2; cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventCreate(&e2);
    size_t sm_size = 2 * HIDDEN_DIM + 512 + (4 * HIDDEN_DIM);
#if NTT_MODE != 0
    sm_size += SEQ_LEN * sizeof(int32_t);      // the transformed window (mgpu.cu:1512-1517)
#endif
    const long step = 1;   // only gates the reference's debug printf
    cudaEventRecord(e0, stream);
    for (int off = h.pop_offset; off < h.pop_offset + h.count; off += batch_cap) {
        int batch = batch_cap;
        if (off + batch > h.pop_offset + h.count) batch = h.pop_offset + h.count - off;
        train_sequence_kernel<<<batch, BLOCK_THREADS, sm_size, stream>>>(
            d_dataset, (long)h.data_len, (int)h.start_idx, d_model, d_kv, d_loss, h.step_seed, off, step);
    }
    cudaEventRecord(e1, stream);
    CHECK_CUDA(cudaStreamSynchronize(stream));
    CHECK_CUDA(cudaGetLastError());
    int32_t *h_loss = (int32_t *)malloc(POPULATION_SIZE * sizeof(int32_t));
    CHECK_CUDA(cudaMemcpy(h_loss, d_loss, POPULATION_SIZE * sizeof(int32_t), cudaMemcpyDeviceToHost));

    FILE *o = fopen(argv[2], "wb");
    if (!o) die("cannot open output");
    fwrite(h_loss + h.pop_offset, sizeof(int32_t), h.count, o);

    float ms_eval = 0, ms_update = 0;
    cudaEventElapsedTime(&ms_eval, e0, e1);
    unsigned long long h_updates = 0;
    if (h.do_update) {
        int32_t *h_fit = (int32_t *)malloc((POPULATION_SIZE / 2) * sizeof(int32_t));
        compute_fitness_host(h_loss, h_fit, POPULATION_SIZE / 2);
        CHECK_CUDA(cudaMemcpy(d_fit, h_fit, (POPULATION_SIZE / 2) * sizeof(int32_t), cudaMemcpyHostToDevice));
        unsigned long long *d_updates_ptr;
        CHECK_CUDA(cudaGetSymbolAddress((void **)&d_updates_ptr, d_total_updates));
        CHECK_CUDA(cudaMemsetAsync(d_updates_ptr, 0, sizeof(unsigned long long), stream));
        uint32_t seed = h.step_seed; float current_lr = h.lr;
#if USE_MUON == 1
        cublasHandle_t cublas_handle; MuonWorkspace muon_ws;
        CHECK_CUBLAS(cublasCreate(&cublas_handle));
        CHECK_CUBLAS(cublasSetStream(cublas_handle, stream));
        size_t max_mx_elems = HIDDEN_DIM * (HIDDEN_DIM * 4), gram_elems = HIDDEN_DIM * HIDDEN_DIM;
        CHECK_CUDA(cudaMalloc(&muon_ws.d_buf1, max_mx_elems * sizeof(float)));
        CHECK_CUDA(cudaMalloc(&muon_ws.d_buf2, gram_elems * sizeof(float)));
        CHECK_CUDA(cudaMalloc(&muon_ws.d_buf3, gram_elems * sizeof(float)));
        CHECK_CUDA(cudaMalloc(&muon_ws.d_buf_swap, max_mx_elems * sizeof(float)));
        CHECK_CUDA(cudaMalloc(&muon_ws.d_scalar, sizeof(float)));
#endif
        // One call per parameter with the reference's kernels; the table of
        // (rows, cols, off_A, off_B, seed_base, lr scale) is this harness's own
        // statement of the reference's launch list.
        auto vec = [&](WeightType *v, AdamParam *st, int len, int a, int b, int base, float sc) {
            update_vector_adam_kernel<<<(len + 255) / 256, 256, 0, stream>>>(v, st, len, a, b, base, d_fit, seed, current_lr * sc);
        };
        auto mat_adam = [&](WeightType *w, AdamParam *st, int rows, int cols, int a, int b, int base, float sc = 1.0f) {
            update_matrix_adam_kernel<<<(rows * cols + 511) / 512, 512, 0, stream>>>(w, st, rows, cols, a, b, base, d_fit, seed, current_lr * sc);
        };
        auto mat = [&](WeightType *w, HIDDEN_OPT_TYPE *st, int rows, int cols, int a, int b, int base) {
#if USE_MUON == 1
            muon_momentum_update_kernel<<<(rows * cols + 511) / 512, 512, 0, stream>>>(st, rows, cols, a, b, base, d_fit, seed, MUON_MOMENTUM);
            muon_gather_m_kernel<<<(rows * cols + 511) / 512, 512, 0, stream>>>(st, muon_ws.d_buf1, rows, cols);
            perform_newton_schulz(cublas_handle, muon_ws, muon_ws.d_buf1, rows, cols, stream);
            muon_apply_update_kernel<<<(rows * cols + 511) / 512, 512, 0, stream>>>(w, st, muon_ws.d_buf1, rows, cols, current_lr * MUON_LR_SCALE, ADAM_WEIGHT_DECAY);
#else
            mat_adam(w, st, rows, cols, a, b, base);
#endif
        };
        const int H = HIDDEN_DIM;
        cudaEventRecord(e1, stream);
        for (int l = 0; l < N_LAYERS; l++) {
            int sb = l * 1000;
            mat(d_model->w_q[l], d_opt->w_q[l], H, H, SEED_OFF_Q_A, SEED_OFF_Q_B, sb);
            mat(d_model->w_k[l], d_opt->w_k[l], H, H, SEED_OFF_K_A, SEED_OFF_K_B, sb);
            mat(d_model->w_v[l], d_opt->w_v[l], H, H, SEED_OFF_V_A, SEED_OFF_V_B, sb);
            mat(d_model->w_o[l], d_opt->w_o[l], H, H, SEED_OFF_O_A, SEED_OFF_O_B, sb);
            mat(d_model->w_up[l], d_opt->w_up[l], H, 4 * H, SEED_OFF_MLP_UP_A, SEED_OFF_MLP_UP_B, sb);
            mat(d_model->w_down[l], d_opt->w_down[l], 4 * H, H, SEED_OFF_MLP_DOWN_A, SEED_OFF_MLP_DOWN_B, sb);
            vec(d_model->ln_1[l], d_opt->ln_1[l], H, SEED_OFF_LN_1_A, SEED_OFF_LN_1_B, sb, 1.0f);
            vec(d_model->ln_1_bias[l], d_opt->ln_1_bias[l], H, SEED_OFF_LN_1_BIAS_A, SEED_OFF_LN_1_BIAS_B, sb, 1.0f);
            vec(d_model->ln_2[l], d_opt->ln_2[l], H, SEED_OFF_LN_2_A, SEED_OFF_LN_2_B, sb, 1.0f);
            vec(d_model->ln_2_bias[l], d_opt->ln_2_bias[l], H, SEED_OFF_LN_2_BIAS_A, SEED_OFF_LN_2_BIAS_B, sb, 1.0f);
            vec(d_model->mlp_bias_up[l], d_opt->mlp_bias_up[l], 4 * H, SEED_OFF_MLP_BIAS_UP_A, SEED_OFF_MLP_BIAS_UP_B, sb, 1.0f);
            vec(d_model->mlp_bias_down[l], d_opt->mlp_bias_down[l], H, SEED_OFF_MLP_BIAS_DOWN_A, SEED_OFF_MLP_BIAS_DOWN_B, sb, 1.0f);
        }
        vec(d_model->ln_f, d_opt->ln_f, H, SEED_OFF_LN_F_A, SEED_OFF_LN_F_B, 0, 1.0f);
        vec(d_model->ln_f_bias, d_opt->ln_f_bias, H, SEED_OFF_LN_F_BIAS_A, SEED_OFF_LN_F_BIAS_B, 0, 1.0f);
        vec(d_model->ln_init, d_opt->ln_init, H, SEED_OFF_LN_INIT_A, SEED_OFF_LN_INIT_B, 0, 1.0f);
        vec(d_model->ln_init_bias, d_opt->ln_init_bias, H, SEED_OFF_LN_INIT_BIAS_A, SEED_OFF_LN_INIT_BIAS_B, 0, 1.0f);
        mat(d_model->w_emb_mlp_up, d_opt->w_emb_mlp_up, H, 4 * H, SEED_OFF_EMB_MLP_UP_A, SEED_OFF_EMB_MLP_UP_B, 0);
        vec(d_model->mlp_emb_bias_up, d_opt->mlp_emb_bias_up, 4 * H, SEED_OFF_EMB_MLP_BIAS_UP_A, SEED_OFF_EMB_MLP_BIAS_UP_B, 0, 1.0f);
        mat(d_model->w_emb_mlp_down, d_opt->w_emb_mlp_down, 4 * H, H, SEED_OFF_EMB_MLP_DOWN_A, SEED_OFF_EMB_MLP_DOWN_B, 0);
        vec(d_model->mlp_emb_bias_down, d_opt->mlp_emb_bias_down, H, SEED_OFF_EMB_MLP_BIAS_DOWN_A, SEED_OFF_EMB_MLP_BIAS_DOWN_B, 0, 1.0f);
        vec(d_model->emb_bias, d_opt->emb_bias, H, SEED_OFF_EMB_BIAS_A, SEED_OFF_EMB_BIAS_B, 0, 0.1f);
        mat_adam(d_model->embedding, d_opt->embedding, H, VOCAB_SIZE, SEED_OFF_EMB, SEED_OFF_EMB + H, 0);
#if NTT_MODE != 0
        mat_adam(d_model->ntt_emb1, d_opt->ntt_emb1, H, VOCAB_SIZE, SEED_OFF_NTT_EMB1, SEED_OFF_NTT_EMB1 + H, 0, 0.5f);
        mat_adam(d_model->ntt_emb2, d_opt->ntt_emb2, H, VOCAB_SIZE, SEED_OFF_NTT_EMB2, SEED_OFF_NTT_EMB2 + H, 0, 0.5f);
        mat_adam(d_model->ntt_emb3, d_opt->ntt_emb3, H, VOCAB_SIZE, SEED_OFF_NTT_EMB3, SEED_OFF_NTT_EMB3 + H, 0, 0.5f);
#endif
        cudaEventRecord(e2, stream);
        CHECK_CUDA(cudaStreamSynchronize(stream));
        CHECK_CUDA(cudaGetLastError());
        cudaEventElapsedTime(&ms_update, e1, e2);
        CHECK_CUDA(cudaMemcpy(&h_updates, d_updates_ptr, sizeof(h_updates), cudaMemcpyDeviceToHost));
        CHECK_CUDA(cudaMemcpy(h_model, d_model, sizeof(TransformerModel), cudaMemcpyDeviceToHost));
        CHECK_CUDA(cudaMemcpy(h_opt, d_opt, sizeof(AdamModel), cudaMemcpyDeviceToHost));
        fwrite(h_fit, sizeof(int32_t), POPULATION_SIZE / 2, o);
        uint64_t u = h_updates; fwrite(&u, sizeof(u), 1, o);
        fwrite(h_model, sizeof(TransformerModel), 1, o);
        fwrite(h_opt, sizeof(AdamModel), 1, o);
    }
    fclose(o);
    printf("{\"ref\": \"mgpu\", \"hidden_dim\": %d, \"n_layers\": %d, \"seq_len\": %d, \"population_size\": %d, "
           "\"count\": %d, \"use_muon\": %d, \"eval_ms\": %.3f, \"update_ms\": %.3f, \"updates\": %llu}\n",
           HIDDEN_DIM, N_LAYERS, SEQ_LEN, POPULATION_SIZE, h.count, USE_MUON, ms_eval, ms_update, h_updates);
    return 0;
}
