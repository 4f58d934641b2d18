/*
 * Deterministic driver around the REFERENCE's CPU trainer functions
 * (full_trained_egg.c lines 1-476: everything except main), which oracle/Makefile
 * extracts into oracle/_ref/ at build time and compiles unmodified against the
 * scalar arm_neon.h stand-in.  TEST / BASELINE INFRASTRUCTURE ONLY.
 *
 * Replaces the reference's main() (full_trained_egg.c:477-583): fixed step seed,
 * synthetic weights and input supplied by the caller, one task per population
 * pair across the host cores (the decomposition of its dispatch_apply, :547-562).
 *
 *   ref_cpu_gru <in.bin> <out.bin> [pairs_to_run] [tokens] [steps]
 *
 * in.bin : uint32 step_seed, int64 data_len, EggModel bytes, dataset bytes
 * out.bin: per step: int32 losses[2*pairs_run], int32 fitness[pairs_run];
 *          then EggModel bytes and RecurrentState[POPULATION_SIZE] bytes after the last step.
 * The update runs when every pair was evaluated (any token count).  Step s uses the seed
 * step_seed ^ (s * 0x9e3779b9) (the reference's mix with its time(NULL) replaced by the fixed
 * seed, :530) and start index s * SEQ_LEN (:531); recurrent states carry over (:515-517).
 * stdout : JSON line with seconds and member-tokens/s.
 */
#include "full_trained_egg_body.inc"
#include <omp.h>

int main(int argc, char **argv) {
    if (argc >= 2 && strcmp(argv[1], "--sizes") == 0) {
        printf("{\"model_bytes\": %zu, \"hidden_dim\": %d, \"n_layers\": %d, \"seq_len\": %d, \"population_size\": %d}\n",
               sizeof(EggModel), HIDDEN_DIM, N_LAYERS, SEQ_LEN, POPULATION_SIZE);
        return 0;
    }
    if (argc < 3) { fprintf(stderr, "usage: ref_cpu_gru in.bin out.bin [pairs] [tokens] [steps]\n"); return 2; }
    int pairs = POPULATION_SIZE / 2, tokens = SEQ_LEN;
    if (argc > 3) pairs = atoi(argv[3]);
    if (argc > 4) tokens = atoi(argv[4]);
    if (pairs < 1 || pairs > POPULATION_SIZE / 2 || tokens < 1 || tokens > SEQ_LEN) return 2;
    FILE *f = fopen(argv[1], "rb");
    if (!f) return 2;
    uint32_t step_seed; int64_t data_len;
    EggModel *model = (EggModel *)malloc(sizeof(EggModel));
    if (fread(&step_seed, 4, 1, f) != 1 || fread(&data_len, 8, 1, f) != 1 || fread(model, sizeof(EggModel), 1, f) != 1) return 2;
    uint8_t *data = (uint8_t *)malloc(data_len);
    if (fread(data, 1, data_len, f) != (size_t)data_len) return 2;
    fclose(f);
    init_tables();
    int32_t *losses = (int32_t *)calloc(POPULATION_SIZE, sizeof(int32_t));
    int *fit = (int *)calloc(POPULATION_SIZE / 2, sizeof(int));
    RecurrentState *states = (RecurrentState *)calloc(POPULATION_SIZE, sizeof(RecurrentState));
    int steps = argc > 5 ? atoi(argv[5]) : 1;
    if (steps < 1) return 2;
    FILE *o = fopen(argv[2], "wb");
    if (!o) return 2;
    long stride = data_len / (POPULATION_SIZE / 2);       /* :545 */
    const uint32_t seed0 = step_seed;
    double eval_s = 0, update_s = 0;
    for (long step = 0; step < steps; step++) {
        step_seed = seed0 ^ (uint32_t)(step * 0x9e3779b9);
        int start_idx = step * SEQ_LEN;                   /* :531 */
        double t0 = omp_get_wtime();
#pragma omp parallel for schedule(dynamic, 1)
        for (int p = 0; p < pairs; p++) {                 /* body of the dispatch_apply block, :547-562 */
            uint32_t p_seed = step_seed + p;
            long stream_pos = (start_idx + (p * stride)) % (data_len - SEQ_LEN);
            int8_t logits[VOCAB_SIZE];
            forward_pass(model, &data[stream_pos], &data[stream_pos + 1], tokens, logits, &losses[2 * p], p_seed, 1, &states[2 * p]);
            forward_pass(model, &data[stream_pos], &data[stream_pos + 1], tokens, logits, &losses[2 * p + 1], p_seed, -1, &states[2 * p + 1]);
            if (losses[2 * p] < losses[2 * p + 1]) fit[p] = 1;
            else if (losses[2 * p + 1] < losses[2 * p]) fit[p] = -1;
            else fit[p] = 0;
        }
        double t1 = omp_get_wtime();
        if (pairs == POPULATION_SIZE / 2) {               /* :564-574 */
            for (int l = 0; l < N_LAYERS; l++) {
                uint32_t l_seed = step_seed + (l * 100);
                update_matrix(model->gru_weights[l][0], HIDDEN_DIM, HIDDEN_DIM, l_seed + 1, fit, POPULATION_SIZE);
                update_matrix(model->gru_weights[l][1], HIDDEN_DIM, HIDDEN_DIM, l_seed + 2, fit, POPULATION_SIZE);
                update_matrix(model->gru_weights[l][2], HIDDEN_DIM, HIDDEN_DIM, l_seed + 3, fit, POPULATION_SIZE);
                update_matrix(model->gru_weights[l][3], HIDDEN_DIM, HIDDEN_DIM, l_seed + 4, fit, POPULATION_SIZE);
                update_matrix(model->mlp_weights[l][0], HIDDEN_DIM * 4, HIDDEN_DIM, l_seed + 5, fit, POPULATION_SIZE);
                update_matrix(model->mlp_weights[l][1], HIDDEN_DIM, HIDDEN_DIM * 4, l_seed + 6, fit, POPULATION_SIZE);
            }
            update_matrix(model->head, VOCAB_SIZE, HIDDEN_DIM, step_seed + 999, fit, POPULATION_SIZE);
        }
        double t2 = omp_get_wtime();
        eval_s += t1 - t0; update_s += t2 - t1;
        fwrite(losses, 4, 2 * pairs, o);
        for (int p = 0; p < pairs; p++) { int32_t v = fit[p]; fwrite(&v, 4, 1, o); }
    }
    fwrite(model, sizeof(EggModel), 1, o);
    fwrite(states, sizeof(RecurrentState), POPULATION_SIZE, o);
    fclose(o);
    double t0 = 0, t1 = eval_s, t2 = eval_s + update_s;
    tokens *= steps;
    double mt = 2.0 * pairs * tokens;
    printf("{\"ref\": \"cpu_gru\", \"threads\": %d, \"pairs\": %d, \"tokens\": %d, \"eval_s\": %.4f, \"update_s\": %.4f, "
           "\"member_tokens_per_s\": %.2f}\n", omp_get_max_threads(), pairs, tokens, t1 - t0, t2 - t1, mt / (t2 - t0));
    return 0;
}
