/*
 * egg_oracle.h — CPU restatement of the reference's EGGROLL hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is the checker the CUDA library is compared
 * against; the product never links, imports or calls it.  Every function
 * cites the reference lines it restates ("mgpu.cu" =
 * full_cuda_train_transformer_adam_mgpu.cu).
 *
 * Parity pinning: the reference holds no golden vectors for this path (its
 * only test is d-eggs/test_ternary.cpp).  The oracle is pinned by (1) the
 * hash/noise known answers produced by compiling the reference's own
 * d-eggs/include/utils/egg_math.h with g++ (tests/golden/rng_kat.json),
 * (2) the ternary codec cases of d-eggs/test_ternary.cpp, and (3) losses /
 * fitness / post-update weights produced by the reference's own kernels
 * (built from the reference sources by oracle/Makefile into oracle/_ref/ and
 * run on a B200), committed under tests/golden/.
 */
#ifndef EGG_ORACLE_H
#define EGG_ORACLE_H

#include <stdint.h>
#include "../include/egg_b200.h"   /* egg_config only */

#ifdef __cplusplus
extern "C" {
#endif

/* --- RNG (mgpu.cu:525-538; d-eggs/include/utils/egg_math.h:17-34) --- */
uint32_t oracle_hash_rng(uint32_t s, uint32_t idx);
int      oracle_noise(const egg_config *cfg, uint32_t s, uint32_t idx);
/* host xorshift stream used by init_model (mgpu.cu:428-441) */
int      oracle_gen_noise_host(const egg_config *cfg, uint32_t *state);

/* --- sizes / layout --- */
int64_t oracle_model_bytes(const egg_config *cfg);
int64_t oracle_opt_bytes(const egg_config *cfg);
int64_t oracle_scales_bytes(const egg_config *cfg);

/* --- tables (mgpu.cu:394-426) --- */
void oracle_init_tables(const egg_config *cfg, int32_t *exp_lut256, int8_t *act_lut256,
                        int32_t *rope_lut /* seq_len*head_dim */);

/* --- model initialisation (mgpu.cu:443-519) --- */
void oracle_repack_matrix(int8_t *dst, const int8_t *src, int rows, int cols);
void oracle_init_model(const egg_config *cfg, int8_t *model, uint32_t seed);

/* --- evaluation (mgpu.cu:847-1029; d-eggs/src/kernels.cu:90-298) ---
 * losses_out[i] is the loss of member pop_offset+i (always chunk-relative).
 * scales: AdaptiveScales bytes (d-eggs/include/model/definitions.h:92-142) or NULL.
 * dataset: data_len tokens of the reference's TokenType (mgpu.cu:58-66): one byte each when vocab_size == 256,
 * uint32_t each otherwise (the pointer is then a uint32_t array passed as bytes). */
void oracle_eval(const egg_config *cfg, const int8_t *model, const int8_t *scales,
                 const uint8_t *dataset, int64_t data_len, int64_t start_idx,
                 uint32_t step_seed, int pop_offset, int count, int32_t *losses_out);

/* the transform cfg->ntt_mode (1 Walsh-Hadamard, 2 Fermat-257, 3 Fermat-65537) applies to a member's input window
 * before the embedding (ntt_transform_sequence, egg_ntt.cuh:446-455), in place on `len` values (a power of two) */
void oracle_window_transform(const egg_config *cfg, int32_t *data, int len);

/* per-token trace of one member for debugging/cross-checks: fills
 * stages[seq_len][3 + 2*n_layers][H] with the residual stream after the
 * embedding, after the initial MLP, after each layer's attention and MLP block,
 * and the final normalised vector; logits[seq_len][V] (int32, after
 * >>shift_logit).  Either may be NULL. */
void oracle_eval_trace(const egg_config *cfg, const int8_t *model, const int8_t *scales,
                       const uint8_t *dataset, int64_t data_len, int64_t start_idx,
                       uint32_t step_seed, int member, int8_t *x_after_layers,
                       int32_t *logits, int32_t *loss_out);

/* --- sampling (generate_sequence_kernel, d-eggs/src/kernels.cu:307-490; mgpu.cu:1154-1285) ---
 * tokens[0..seed_len) given, tokens[seed_len..seed_len+gen_len) written; min_p <= 0 disables the filter. */
void oracle_generate(const egg_config *cfg, const int8_t *model, uint8_t *tokens, int seed_len, int gen_len,
                     uint32_t seed, float temp, float min_p, float penalty);

/* --- fitness (mgpu.cu:1031-1036, 1305-1311) --- */
void oracle_fitness(const int32_t *losses, int32_t *fitness, int pairs);

/* --- update (mgpu.cu:1040-1152, 1573-1668; muon_internal.cuh) ---
 * fma_mode: 0 = every float op rounded separately; 34 = the contraction
 * pattern nvcc's default -fmad=true produces for the reference source
 * (calibrated on a B200; encoding in oracle_adam_step). */
uint64_t oracle_update(const egg_config *cfg, int8_t *model, void *opt_state,
                       const int32_t *fitness, uint32_t step_seed, float lr, int fma_mode);

/* d-eggs variant: after each parameter's AdamW step the adaptive-noise overlays of the rows / columns that
 * changed go up by 5, the others down by 1 (worker.cu:445-517, kernels.cu:61-77). scales may be NULL. */
uint64_t oracle_update_scaled(const egg_config *cfg, int8_t *model, void *opt_state,
                              const int32_t *fitness, uint32_t step_seed, float lr, int fma_mode, int8_t *scales);

/* vote of one matrix in packed index order (mgpu.cu:1085-1098) */
void oracle_vote_matrix(const egg_config *cfg, const int32_t *fitness, int pairs,
                        int rows_k, int cols_n, int off_a, int off_b, int seed_base,
                        uint32_t step_seed, int32_t *vote);

/* one AdamW element step (mgpu.cu:1040-1064); returns 1 if w changed */
int oracle_adam_step(const egg_config *cfg, float *m, float *v, float *acc, int8_t *w,
                     float g, float lr, int fma_mode);

/* Newton–Schulz orthogonalisation of a row-major rows×cols fp32 matrix
 * (muon_internal.cuh:182-342), double accumulation, fp32 storage. */
void oracle_newton_schulz(float *x, int rows, int cols);

/* --- isolated perturbed projection (mgpu.cu:553-572 + ">>8, clip" of
 * full_cuda_train_egg_transformer.cu:249) --- */
void oracle_projection(const egg_config *cfg, const int8_t *x, const int8_t *w_packed,
                       int8_t *y, int64_t rows, int k_dim, int n_dim, int rows_per_member,
                       uint32_t seed, int off_a, int off_b, int rank1_shift, int out_shift);

/* votes of selected output columns: out[n_count][rows_k], out[i][k] = Σ_p f_p A_p[n_list[i]] B_p[k] (mgpu.cu:1085-1098) */
void oracle_vote_columns(const egg_config *cfg, const int32_t *fitness, int pairs, int rows_k, int off_a, int off_b,
                         int seed_base, uint32_t step_seed, const int32_t *n_list, int n_count, int32_t *out);

/* ES-AdamW over `count` elements from their votes; state = {m, v, acc} per element (mgpu.cu:1040-1064, 1100-1110) */
uint64_t oracle_adam_from_votes(const egg_config *cfg, int8_t *w, float *state, const int32_t *vote, int64_t count, float lr,
                                int fma_mode);

/* --- d-eggs worker host fitness (d-eggs/src/worker.cu:635-687). Parity unpinned: the reference
 * has this code inline in main(), it cannot be called; restated by reading. --- */
void oracle_deggs_chunk_fitness(const int32_t *losses, int count, int mean_filter, double exponent, int adaptive,
                                double alpha, int32_t *fit, int64_t *sum_loss);

/* --- ternary codec (d-eggs/include/utils/ternary_pack.h:12-87) --- */
int64_t oracle_ternary_packed_size(int64_t count);
void oracle_ternary_pack(const int32_t *values, int64_t count, uint8_t *out);
void oracle_ternary_unpack(const uint8_t *in, int64_t count, int32_t *values);

/* --- the recurrent model of full_trained_egg.c (egg_gru_oracle.c) --- */
int64_t oracle_gru_model_bytes(const egg_gru_config *cfg);
void oracle_gru_init_model(const egg_gru_config *cfg, int8_t *model, uint32_t seed);          /* main(), :491-515 */
void oracle_gru_exp2_table(const egg_gru_config *cfg, int32_t *table256);                      /* init_tables, :58-61 */
/* one iteration of the training loop (:529-575); states [population][n_layers][H] are carried */
void oracle_gru_generation(const egg_gru_config *cfg, int8_t *model, int8_t *states, const uint8_t *data,
                           int64_t data_len, uint32_t step_seed, int64_t start_idx, int tokens, int do_update,
                           int32_t *losses, int32_t *fitness);

#ifdef __cplusplus
}
#endif
#endif
