// Debug aid (TEST INFRASTRUCTURE ONLY): runs the REFERENCE's own __device__ layer
// functions for one population member, in the order train_sequence_kernel calls
// them (mgpu.cu:889-963), and dumps the residual stream after every stage so that
// the oracle's stage trace can be compared position by position.
//   ref_trace_<tag> <in.bin> <out.bin>    (same input file as ref_mgpu_<tag>; member = pop_offset)
// out.bin: int8 stages[SEQ_LEN][3 + 2*N_LAYERS][HIDDEN_DIM]
#define main ref_main_unused
#include REF_DIR_INCLUDE
#undef main

struct ref_case_header { uint32_t magic, step_seed; int64_t start_idx, data_len; int32_t pop_offset, count; float lr; int32_t do_update, has_opt, reserved; int32_t cfg_check[6]; };

__global__ void __launch_bounds__(MAX_BLOCK_THREADS) trace_kernel(const TokenType *dataset, long data_len, int start_idx,
                                                                  const TransformerModel *model, ActType *kv, uint32_t step_seed,
                                                                  int p_idx, int8_t *out) {
    int tid = threadIdx.x;
    if (tid >= HIDDEN_DIM) return;
    extern __shared__ ActType s_mem[];
    ActType *s_x = s_mem;
    __shared__ typename BlockReduce::TempStorage temp_storage;
    __shared__ AccumType shared_scalar;
    long pair_idx = p_idx / 2;
    long stride = data_len / (POPULATION_SIZE / 2);
    long stream_pos = (start_idx + (pair_idx * stride)) % (data_len - SEQ_LEN);
    int ns = (p_idx % 2 == 0) ? 1 : -1;
    size_t kv_layer_stride = 2ULL * SEQ_LEN * HIDDEN_DIM;
    const int nst = 3 + 2 * N_LAYERS;
    for (int t = 0; t < SEQ_LEN; t++) {
        TokenType input_token = dataset[stream_pos + t];
        uint32_t seed_emb = (step_seed + pair_idx) + SEED_OFF_EMB;
        WeightType emb = get_embedding_byte(model->embedding, tid, input_token);
        WeightType ebias = model->emb_bias[tid];
        int8_t n1 = noise_from_hash((step_seed + pair_idx) + SEED_OFF_EMB_BIAS_A, tid);
        int8_t n2 = noise_from_hash((step_seed + pair_idx) + SEED_OFF_EMB_BIAS_B, tid);
        AccumType chk = ((AccumType)n1 * n2 * ns) >> SIGMA_SHIFT_VECTOR;
        int8_t a_tok = noise_from_hash(seed_emb, input_token);
        int8_t b_dim = noise_from_hash(seed_emb + HIDDEN_DIM, tid);
        AccumType perturb = ((AccumType)a_tok * b_dim * ns) >> (FIXED_POINT + SIGMA_SHIFT);
        s_x[tid] = clip((AccumType)emb + ebias + chk + perturb);
        __syncthreads();
        out[((size_t)t * nst + 0) * HIDDEN_DIM + tid] = s_x[tid];
        compute_mlp(0, t, tid, s_x, s_mem, temp_storage, shared_scalar, model->ln_init, model->ln_init_bias, model->w_emb_mlp_up,
                    model->mlp_emb_bias_up, model->w_emb_mlp_down, model->mlp_emb_bias_down, step_seed + pair_idx, ns, 1, 0, CFG_MLP_INIT);
        out[((size_t)t * nst + 1) * HIDDEN_DIM + tid] = s_x[tid];
        for (int l = 0; l < N_LAYERS; l++) {
            uint32_t seed_base = (step_seed + pair_idx) + (l * 1000);
            ActType *lkv_k = kv + l * kv_layer_stride, *lkv_v = lkv_k + SEQ_LEN * HIDDEN_DIM;
            compute_attention(l, t, tid, model, lkv_k, lkv_v, s_x, s_mem, temp_storage, shared_scalar, seed_base, ns, 1, 0);
            out[((size_t)t * nst + 2 + 2 * l) * HIDDEN_DIM + tid] = s_x[tid];
            compute_mlp(l, t, tid, s_x, s_mem, temp_storage, shared_scalar, model->ln_2[l], model->ln_2_bias[l], model->w_up[l],
                        model->mlp_bias_up[l], model->w_down[l], model->mlp_bias_down[l], seed_base, ns, 1, 0, CFG_MLP_LAYER);
            out[((size_t)t * nst + 3 + 2 * l) * HIDDEN_DIM + tid] = s_x[tid];
        }
        ActType nf = apply_standard_norm(s_x[tid], tid, temp_storage, shared_scalar, model->ln_f[tid], model->ln_f_bias[tid],
                                         step_seed + pair_idx, SEED_OFF_LN_F_A, SEED_OFF_LN_F_B, SEED_OFF_LN_F_BIAS_A, SEED_OFF_LN_F_BIAS_B, ns);
        out[((size_t)t * nst + 2 + 2 * N_LAYERS) * HIDDEN_DIM + tid] = nf;
        __syncthreads();
    }
}

int main(int argc, char **argv) {
    if (argc < 3) return 2;
    FILE *f = fopen(argv[1], "rb");
    ref_case_header h;
    if (!f || fread(&h, sizeof(h), 1, f) != 1) return 2;
    {
        const int want[6] = {HIDDEN_DIM, N_LAYERS, SEQ_LEN, POPULATION_SIZE, DEVICE_MASK, USE_MUON};
        for (int i = 0; i < 6; i++)
            if (h.cfg_check[i] != want[i]) { fprintf(stderr, "ref harness: case was made for another configuration (field %d: %d vs compiled %d)\n", i, h.cfg_check[i], want[i]); return 3; }
    }
    TransformerModel *h_model = (TransformerModel *)calloc(1, sizeof(TransformerModel));
    if (fread(h_model, sizeof(TransformerModel), 1, f) != 1) return 2;
    if (h.has_opt) fseek(f, sizeof(AdamModel), SEEK_CUR);
    uint8_t *h_data = (uint8_t *)malloc(h.data_len);
    if (fread(h_data, 1, h.data_len, f) != (size_t)h.data_len) return 2;
    fclose(f);
    init_tables();
    cudaMemcpyToSymbol(d_EXP_LUT, h_EXP_LUT, SOFTMAX_LUT_SIZE * sizeof(int32_t));
    cudaMemcpyToSymbol(d_ACT_LUT, h_ACT_LUT, 256 * sizeof(int8_t));
    cudaMemcpyToSymbol(d_ROPE_LUT, h_ROPE_LUT, ROPE_LUT_SIZE * sizeof(int32_t));
    TransformerModel *d_model; TokenType *d_dataset; ActType *d_kv; int8_t *d_out;
    const size_t out_bytes = (size_t)SEQ_LEN * (3 + 2 * N_LAYERS) * HIDDEN_DIM;
    CHECK_CUDA(cudaMalloc(&d_model, sizeof(TransformerModel)));
    CHECK_CUDA(cudaMalloc(&d_dataset, h.data_len));
    CHECK_CUDA(cudaMalloc(&d_kv, (size_t)N_LAYERS * 2 * SEQ_LEN * HIDDEN_DIM));
    CHECK_CUDA(cudaMalloc(&d_out, out_bytes));
    CHECK_CUDA(cudaMemcpy(d_model, h_model, sizeof(TransformerModel), cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(d_dataset, h_data, h.data_len, cudaMemcpyHostToDevice));
    size_t sm_size = 2 * HIDDEN_DIM + 512 + (4 * HIDDEN_DIM);
    trace_kernel<<<1, BLOCK_THREADS, sm_size>>>(d_dataset, (long)h.data_len, (int)h.start_idx, d_model, d_kv, h.step_seed, h.pop_offset, d_out);
    CHECK_CUDA(cudaDeviceSynchronize());
    int8_t *h_out = (int8_t *)malloc(out_bytes);
    CHECK_CUDA(cudaMemcpy(h_out, d_out, out_bytes, cudaMemcpyDeviceToHost));
    FILE *o = fopen(argv[2], "wb");
    fwrite(h_out, 1, out_bytes, o);
    fclose(o);
    return 0;
}
