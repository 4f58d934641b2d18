/*
 * egg_b200.h — C ABI of the B200-native EGGROLL population-evaluation path.
 *
 * The reference project (d0rc/egg.c) has no library interface: its hot path is
 * a handful of kernel launches inside main() of
 * full_cuda_train_transformer_adam_mgpu.cu and d-eggs/src/worker.cu.  Every
 * entry point below stands where one of those launches (or the host code
 * between them) stands, takes plain pointers and sizes, and returns 0 or a
 * negative EGG_E_* code.  No exceptions cross the boundary, nothing here
 * falls back to the CPU: if the CUDA side is unavailable the call fails.
 *
 * Threading: one host thread per egg_ctx; all work is enqueued on the
 * context's stream; egg_sync() and the *_host / read_* calls block.
 */
#ifndef EGG_B200_H
#define EGG_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes ------------------------------------------------------- */
#define EGG_OK            0
#define EGG_E_INVALID    -1   /* bad argument / unsupported configuration      */
#define EGG_E_CUDA       -2   /* a CUDA runtime / driver call failed            */
#define EGG_E_NOMEM      -3   /* device or host allocation failed               */
#define EGG_E_TIMEOUT    -4   /* a bounded device-side wait gave up             */
#define EGG_E_NCCL       -5   /* an NCCL call failed                            */
#define EGG_E_STATE      -6   /* call made in the wrong state (no model, ...)   */

/*
 * Run-time mirror of the reference's compile-time configuration macros
 * (full_cuda_train_transformer_adam_mgpu.cu:35-270, d-eggs/include/config.h:5-242).
 * Field names are the lower-cased macro names.  egg_config_defaults() fills in
 * the reference's own defaults.
 */
typedef struct egg_config {
    int32_t hidden_dim;          /* HIDDEN_DIM  (multiple of 128, <= 1024)         */
    int32_t head_dim;            /* HEAD_DIM    (64)                                */
    int32_t n_layers;            /* N_LAYERS                                        */
    int32_t seq_len;             /* SEQ_LEN     (multiple of 16, <= 1024)           */
    int32_t vocab_size;          /* VOCAB_SIZE  (256: byte tokens; else uint32_t)   */
    int32_t population_size;     /* POPULATION_SIZE (even)                          */
    int32_t fixed_point;         /* FIXED_POINT                                     */
    int32_t sigma_shift;         /* SIGMA_SHIFT                                     */
    int32_t sigma_shift_vector;  /* SIGMA_SHIFT_VECTOR                              */
    int32_t shift_attn;          /* SHIFT_ATTN                                      */
    int32_t shift_out;           /* SHIFT_OUT                                       */
    int32_t shift_logit;         /* SHIFT_LOGIT                                     */
    int32_t shift_mlp_up;        /* SHIFT_MLP_UP                                    */
    int32_t shift_mlp_down;      /* SHIFT_MLP_DOWN                                  */
    int32_t softmax_scale_bit;   /* SOFTMAX_SCALE_BIT                               */
    int32_t rope_scale_bit;      /* ROPE_SCALE_BIT                                  */
    int32_t device_mask;         /* DEVICE_MASK                                     */
    int32_t device_gaussian;     /* DEVICE_GAUSSIAN (0/1)                           */
    int32_t host_mask;           /* HOST_MASK (weight initialisation only)          */
    int32_t use_same_data;       /* USE_SAME_DATA                                   */
    int32_t use_muon;            /* USE_MUON: hidden matrices use Muon, rest AdamW  */
    int32_t chunk_relative_loss; /* 0: accum_loss[global member] (mgpu :1028);
                                    1: accum_loss[member - pop_offset] (d-eggs
                                       kernels.cu:297)                              */
    double  softmax_exp_scale;   /* SOFTMAX_EXP_SCALE                               */
    float   adam_beta1;          /* ADAM_BETA1                                      */
    float   adam_beta2;          /* ADAM_BETA2                                      */
    float   adam_eps;            /* ADAM_EPS                                        */
    float   adam_weight_decay;   /* ADAM_WEIGHT_DECAY                               */
    float   muon_momentum;       /* MUON_MOMENTUM                                   */
    float   muon_lr_scale;       /* MUON_LR_SCALE                                   */
    int32_t ntt_mode;            /* NTT_MODE (mgpu.cu:50-53, egg_ntt.cuh): 0 off; 1 Walsh-Hadamard, 2 Fermat-257,
                                    3 Fermat-65537 transform of each member's input window, whose coefficient bytes
                                    1..3 index three more embedding tables (ntt_emb1..3 in TransformerModel and
                                    AdamModel).  Needs a power-of-two seq_len <= hidden_dim (mode 2: <= 256). */
} egg_config;

/* Defaults of full_cuda_train_transformer_adam_mgpu.cu:35-270. */
void egg_config_defaults(egg_config *cfg);

/* Returns EGG_OK or EGG_E_INVALID; *why (optional) gets a static message. */
int egg_config_validate(const egg_config *cfg, const char **why);

/* sizeof(TransformerModel) / sizeof(AdamModel) for this configuration
 * (mgpu.cu:284-370, d-eggs/include/model/definitions.h:21-89). */
int64_t egg_model_bytes(const egg_config *cfg);
int64_t egg_opt_state_bytes(const egg_config *cfg);

/* ---- context ----------------------------------------------------------- */
typedef struct egg_ctx egg_ctx;

/*
 * One context per process per GPU (≙ struct GPUContext, mgpu.cu:1287-1302).
 * wave_members: how many population members are evaluated per internal wave
 * (activation scratch scales with it: about 23 * hidden_dim + 40 bytes per member-token plus the pair's noise table;
 * 0 picks a default: up to 8192 members, at most a third of the free memory and 48 GB).
 */
int  egg_ctx_create(const egg_config *cfg, int device, int wave_members, egg_ctx **out);
void egg_ctx_destroy(egg_ctx *ctx);
/* Message of the last failing call made on this thread ("" if none). */
const char *egg_last_error(void);
/* cudaStreamSynchronize of the context stream; also surfaces device-side
 * timeout flags as EGG_E_TIMEOUT. */
int  egg_sync(egg_ctx *ctx);

/* ---- model / optimiser bytes (reference layout, host pointers) ---------- */
/* ≙ cudaMemcpy(d_model, h_model, sizeof(TransformerModel)) (mgpu.cu:1461).
 * Matrices are in the reference's packed [K/4][N][4] layout (repack_matrix,
 * mgpu.cu:443-459); the library derives its own K-major shadow copies. */
int egg_upload_model(egg_ctx *ctx, const void *host_model, int64_t nbytes);
int egg_download_model(egg_ctx *ctx, void *host_model, int64_t nbytes);
/* ≙ cudaMemcpy of AdamModel (mgpu.cu:1464). */
int egg_upload_opt_state(egg_ctx *ctx, const void *host_state, int64_t nbytes);
int egg_download_opt_state(egg_ctx *ctx, void *host_state, int64_t nbytes);

/* ---- checkpoint files ---------------------------------------------------- */
/*
 * ≙ save_checkpoint (egg_disk_utils.h:46-68; d-eggs/include/utils/io.h:55-79): writes the raw
 * TransformerModel bytes to <dir>/egg_step-%08ld.model.bin and the raw AdamModel bytes to
 * <dir>/egg_step-%08ld.adam.bin (the reference hard-codes dir = "models" and creates it), then points the
 * symlinks <dir>/egg_transformer_last.{model,adam}.bin at them.  Files written by either code base load
 * into the other.
 */
int egg_save_checkpoint(egg_ctx *ctx, const char *dir, int64_t step);
/* ≙ load_model (egg_disk_utils.h:70-81) and the matching read of the optimiser state (mgpu.cu:1431-1441);
 * adam_path may be NULL (state stays as it is).  A file whose size differs from the struct is rejected. */
int egg_load_checkpoint(egg_ctx *ctx, const char *model_path, const char *adam_path);

/* ---- adaptive-noise overlays (d-eggs only) ------------------------------ */
/* sizeof(AdaptiveScales) (d-eggs/include/model/definitions.h:92-142). */
int64_t egg_scales_bytes(const egg_config *cfg);
/*
 * ≙ the worker's d_scales (worker.cu: cudaMallocManaged + init to ADAPTIVE_NOISE_INIT) and the
 * `scales` argument of train_sequence_kernel (d-eggs/src/kernels.cu:96).  Uploading the bytes
 * switches the context to ADAPTIVE_NOISE_MODE 1: every noise term of the evaluation is multiplied by
 * get_adaptive_factor(overlay) (layers.cuh:12-19) and every egg_apply_update is followed by
 * update_overlay_kernel (kernels.cu:61-77) per parameter.  host_scales == NULL switches back to
 * unscaled noise (ADAPTIVE_NOISE_MODE 0, the mgpu program).  Mode 2 (stochastic gate) is not provided.
 * Muon-optimised matrices keep their overlays unchanged (the worker never combines the two).
 */
int egg_upload_scales(egg_ctx *ctx, const void *host_scales, int64_t nbytes);
int egg_download_scales(egg_ctx *ctx, void *host_scales, int64_t nbytes);
/* ADAPTIVE_NOISE_INC / ADAPTIVE_NOISE_DEC (d-eggs/include/config.h:231-236); defaults 5 and 1. */
int egg_set_overlay_steps(egg_ctx *ctx, int inc, int dec);

/* ≙ cudaMemcpy(d_dataset, ds.data, ds.length) (mgpu.cu:1466-1467). Byte tokens: vocab_size == 256 only. */
int egg_set_dataset(egg_ctx *ctx, const uint8_t *host_tokens, int64_t n_tokens);
/*
 * The same for the reference's tokenizer build (VOCAB_SIZE != 256 makes TokenType uint32_t, mgpu.cu:58-66; the
 * stream is its input.bin, mgpu.cu:1329-1339): vocab_size a multiple of 256 up to 65536, every token below
 * vocab_size (checked here; EGG_E_INVALID otherwise).  Evaluation then embeds 32-bit tokens and takes the head in
 * two passes over the vocabulary (row maximum, then the exp-table sum in 64 bits and the target logit,
 * mgpu.cu:969-1023); update, fitness and the multi-GPU exchange are unchanged.  egg_generate and the d-eggs
 * worker engine stay byte-token only.
 */
int egg_set_dataset_tokens(egg_ctx *ctx, const uint32_t *host_tokens, int64_t n_tokens);

/* ---- evaluation -------------------------------------------------------- */
/*
 * ≙ train_sequence_kernel<<<count, ...>>>(dataset, len, start_idx, model, kv,
 *     accum_loss, step_seed, pop_offset, step)  (mgpu.cu:847-1029, launch :1531;
 *     d-eggs/src/kernels.cu:90-298, launch worker.cu:626).
 * Evaluates members [pop_offset, pop_offset+count) (both even) and leaves
 * int32 losses in the context's device loss buffer.
 */
int egg_eval_chunk(egg_ctx *ctx, uint32_t step_seed, int64_t start_idx,
                   int pop_offset, int count);
/* ≙ cudaMemcpyAsync(h_loss+off, d_loss+off, n*4, D2H) + sync (mgpu.cu:1537-1552). */
int egg_read_losses(egg_ctx *ctx, int32_t *host_losses, int offset, int count);

/* ≙ compute_fitness_kernel / compute_fitness_host (mgpu.cu:1031-1036, 1305-1311):
 * fitness[p] = sign(loss[2p+1] - loss[2p]) for pairs [pair_offset, +pair_count). */
int egg_compute_fitness_pairs(egg_ctx *ctx, int pair_offset, int pair_count);
/* ≙ cudaMemcpyAsync(d_fit, h_fit, POP/2*4, H2D) (mgpu.cu:1571). */
int egg_write_fitness(egg_ctx *ctx, const int32_t *host_fitness, int pair_offset, int pair_count);
int egg_read_fitness(egg_ctx *ctx, int32_t *host_fitness, int pair_offset, int pair_count);

/* ---- sampling ---------------------------------------------------------- */
/*
 * ≙ generate_sequence_kernel<<<1, ...>>>(buffer, seed_len, gen_len, model, kv, seed, temp, min_p, penalty)
 * (d-eggs/src/kernels.cu:307-490, launch worker.cu:568; mgpu.cu:1154-1285, launch :1703 is the case
 * temp = 1, min_p = 0, penalty = 0): decodes one un-perturbed stream with a KV cache.  host_tokens holds
 * seed_len given bytes followed by room for gen_len sampled ones; seed_len >= 1 and
 * seed_len + gen_len <= min(seq_len, 256) (the reference's RoPE table and token window).  The draw at
 * position t uses hash_rng(seed + 555 t, 0); min_p <= 0 switches the min-p filter off.
 */
int egg_generate(egg_ctx *ctx, uint8_t *host_tokens, int seed_len, int gen_len, uint32_t seed,
                 float temp, float min_p, float penalty);

/* ---- multi-GPU --------------------------------------------------------- */
/* NCCL communicator over the ranks that share one population.  The caller
 * obtains the 128-byte unique id on rank 0 and distributes it out of band. */
int egg_nccl_unique_id(void *id128);
int egg_comm_init(egg_ctx *ctx, const void *id128, int rank, int world);
/*
 * Replaces the reference's host bounce (D2H losses → compute_fitness_host →
 * H2D to every GPU, mgpu.cu:1537-1571): each rank contributes the fitness of
 * its contiguous slice of POP/2/world pairs; one ncclAllGather fills the whole
 * device fitness vector on every rank.
 */
int egg_allgather_fitness(egg_ctx *ctx);

/*
 * Shards the update over the ranks of the communicator (no counterpart in the reference, which repeats the whole
 * update on every GPU, mgpu.cu:1573-1668): every parameter is reconstructed and stepped by ONE rank -- parameters
 * are dealt in order of decreasing cost to the least loaded rank -- and its new int8 weights reach the others by one
 * grouped ncclBroadcast per generation; the change counts are summed with ncclAllReduce.  The weights are identical
 * on every rank afterwards, as without sharding.  The optimiser state of a parameter is current on its owner only:
 * egg_download_opt_state (and egg_save_checkpoint through it) first collects it, which makes them collective calls
 * while sharding is on.  Not combined with adaptive-noise overlays (either call refuses while the other is on).
 * Call after egg_comm_init; enable = 0 switches back and, being the moment every rank needs every state again, is
 * a collective call too.
 */
int egg_set_update_sharding(egg_ctx *ctx, int enable);
/* The owner (rank), the cost weight, the byte offset inside TransformerModel and the number of int8 weights of every
 * parameter, in the library's update order, as the sharded update deals them for `world` ranks; needs no GPU.  Writes
 * at most `cap` entries to each non-NULL array, returns the number of parameters (or a negative error). */
int egg_update_owner_plan(const egg_config *cfg, int world, int32_t *owner_out, int64_t *cost_out, int64_t *model_off_out,
                          int64_t *weights_out, int cap);

/* ---- update ------------------------------------------------------------ */
/*
 * ≙ the LAUNCH_ADAM_MATRIX / LAUNCH_ADAM_VECTOR sequence (mgpu.cu:1573-1668):
 * rebuilds vote = Σ_p fit_p·a_p·b_pᵀ for every parameter from the device
 * fitness vector and applies ES-AdamW (or Muon for hidden matrices when
 * use_muon), emb_bias at 0.1·lr.  *total_updates ≙ d_total_updates.
 */
int egg_apply_update(egg_ctx *ctx, uint32_t step_seed, float learning_rate,
                     uint64_t *total_updates);

/*
 * One whole generation through host buffers (≙ one iteration of the training
 * loop, mgpu.cu:1506-1688): uploads the dataset if host_tokens != NULL (n_tokens
 * tokens: bytes at vocab_size 256, uint32_t otherwise),
 * evaluates this rank's slice of the population, computes fitness, exchanges
 * it when a communicator is attached, applies the update, copies this rank's
 * losses back.  host_losses may be NULL.
 */
int egg_generation_host(egg_ctx *ctx, const void *host_tokens, int64_t n_tokens,
                        int64_t step, uint32_t step_seed, float learning_rate,
                        int32_t *host_losses, uint64_t *total_updates);

/* ---- isolated primitives ---------------------------------------------- */
/*
 * Perturbed int8 projection, host or device buffers chosen by `on_device`
 * (≙ compute_linear_projection + ">>8 and clip", mgpu.cu:553-572 and
 * full_cuda_train_egg_transformer.cu:249):
 *   y[r][n] = clip((Σ_k x[r][k]·W[k][n] + ((xb_r·a_j[n]·ns_r) >> rank1_shift)) >> out_shift)
 * with member = r / rows_per_member, j = member/2, ns = +1/-1 for even/odd
 * member, a_j[n] = noise(seed + j + off_a, n), b_j[k] = noise(seed + j + off_b, k),
 * xb_r = Σ_k x[r][k]·b_j[k].  W is in the packed [K/4][N][4] layout.
 */
int egg_perturbed_projection(egg_ctx *ctx, const int8_t *x, const int8_t *w_packed,
                             int8_t *y, int64_t rows, int k_dim, int n_dim,
                             int rows_per_member, uint32_t seed, int off_a, int off_b,
                             int rank1_shift, int out_shift, int on_device);

/*
 * Update reconstruction for one matrix (≙ the vote loop of
 * update_matrix_adam_kernel, mgpu.cu:1092-1098), accepting any int fitness in
 * [-127,127]: vote[idx] (packed index order) = Σ_p f_p·noise(s_p+off_a, n)·
 * noise(s_p+off_b, k), s_p = step_seed + p + seed_base.
 */
int egg_update_reconstruct(egg_ctx *ctx, const int32_t *fitness, int pairs,
                           int rows_k, int cols_n, int off_a, int off_b, int seed_base,
                           uint32_t step_seed, int32_t *vote_out, int on_device);

/*
 * One whole update of one weight matrix outside any model (≙ one launch of update_matrix_adam_kernel,
 * mgpu.cu:1067-1111, with its argument list: W, optimiser state, rows, cols, off_A, off_B, seed_base,
 * fitnesses, step_seed, lr — or, with optimizer = 1, the Muon sequence of mgpu.cu:1587-1595:
 * muon_momentum_update_kernel, gather, perform_newton_schulz, muon_apply_update_kernel,
 * muon_internal.cuh:15-342).  d_w_packed is the matrix in the reference's [rows_k/4][cols_n][4] layout,
 * d_opt_state its AdamParam{m,v,acc} (optimizer 0, 12 bytes per weight) or MuonParam{m,acc}
 * (optimizer 1, 8 bytes per weight) array in the same index order; both are updated in place.
 * d_fitness holds `pairs` int32 values; split = 1 takes the two-digit operand form for fitness
 * beyond ternary (|f| <= 127; needs 16 * noise magnitude <= 127).  All pointers are DEVICE pointers.
 * Hyper-parameters (betas, eps, weight decay, Muon momentum and lr scale, noise mask) come from the
 * context's configuration.  *total_updates = number of weights that changed.  Its scratch (operands,
 * partial votes, Newton-Schulz workspace) is allocated on first use, kept in the context for later calls
 * of the same or a smaller size, and freed with the context.  Blocks until done.
 */
int egg_update_matrix(egg_ctx *ctx, int8_t *d_w_packed, void *d_opt_state, int rows_k, int cols_n,
                      int off_a, int off_b, int seed_base, const int32_t *d_fitness, int pairs,
                      uint32_t step_seed, float learning_rate, int optimizer, int split,
                      uint64_t *total_updates);

/*
 * Allocation-free variant of egg_update_reconstruct.  It has no counterpart in the
 * reference.  It exists for callers that must not allocate device memory while they
 * run: a d-eggs style worker that was handed a fixed memory budget at start-up, code
 * running inside a memory pool that forbids cudaMalloc, or a loop where the implicit
 * device synchronisation of cudaMalloc/cudaFree would stall other streams.
 *
 * The two noise operand matrices that the vote GEMM needs are kept in one fixed
 * 8 MiB buffer that lives inside the library image on every GPU that loads it
 * (EGG_NOALLOC_SCRATCH_BYTES, held until the process exits).  The call is refused
 * with EGG_E_INVALID when (rows_k + cols_n) * K exceeds it, where K is `pairs`
 * rounded up to 128, doubled when `split` is set.
 *
 * fitness and vote_out are DEVICE pointers owned by the caller.  split = 0 promises
 * |fitness| * (largest noise magnitude) <= 127 (ternary fitness always qualifies);
 * split = 1 selects the two-digit operand form for int8 fitness (needs
 * 16 * noise magnitude <= 127).  Nothing is read back to check the promise.
 *
 * The buffer's device address is looked up once per device, in egg_ctx_create (with
 * that device current); create the context outside any stream capture.  All calls share the buffer and it keeps the last
 * call's operands; every call rewrites the whole region it uses (zero padding
 * included), so nothing has to be cleared, but two calls that overlap on the GPU
 * (different contexts or streams on one device) race on it.
 * Calls no cudaMalloc / cudaFree; blocks until the votes are written.
 */
#define EGG_NOALLOC_SCRATCH_BYTES (8u << 20)
int egg_update_reconstruct_noalloc(egg_ctx *ctx, const int32_t *d_fitness, int pairs,
                                   int rows_k, int cols_n, int off_a, int off_b, int seed_base,
                                   uint32_t step_seed, int split, int32_t *d_vote_out);

/* ---- the recurrent (GRU + MLP) model of full_trained_egg.c ------------------ */
/*
 * The reference's CPU trainer is a different model from the transformer above: a 4-layer
 * minGRU-style recurrent network with one persistent RecurrentState per population member and
 * noise drawn from a sequential xorshift32 stream (full_trained_egg.c:70-105), updated by a plain
 * vote threshold instead of AdamW.  Its compile-time #defines (full_trained_egg.c:10-21) become
 * this struct; bytes of EggModel (:42-50) and RecurrentState (:37-39) are the reference's.
 */
typedef struct egg_gru_config {
    int32_t hidden_dim;        /* HIDDEN_DIM, multiple of 128, <= 1024            */
    int32_t n_layers;          /* N_LAYERS                                        */
    int32_t vocab_size;        /* VOCAB_SIZE, must be 256                         */
    int32_t seq_len;           /* SEQ_LEN: tokens per generation and the modulus of the stream position (:546) */
    int32_t population_size;   /* POPULATION_SIZE (even, multiple of 32, <= 1024) */
    int32_t fixed_point;       /* FIXED_POINT                                     */
    int32_t sigma_shift;       /* SIGMA_SHIFT                                     */
    int32_t update_threshold;  /* UPDATE_THRESHOLD                                */
} egg_gru_config;
/* Defaults of full_trained_egg.c:10-21 (H 512, 4 layers, seq 4096, population 128, threshold 160). */
void egg_gru_config_defaults(egg_gru_config *cfg);
/* sizeof(EggModel) and sizeof(RecurrentState) * POPULATION_SIZE. */
int64_t egg_gru_model_bytes(const egg_gru_config *cfg);
int64_t egg_gru_state_bytes(const egg_gru_config *cfg);

typedef struct egg_gru_ctx egg_gru_ctx;
int  egg_gru_create(const egg_gru_config *cfg, int device, egg_gru_ctx **out);
void egg_gru_destroy(egg_gru_ctx *ctx);
/* EggModel bytes: matrices are row-major [out][in] as matmul_perturbed reads them (:108-177). */
int egg_gru_upload_model(egg_gru_ctx *ctx, const void *host_model, int64_t nbytes);
int egg_gru_download_model(egg_gru_ctx *ctx, void *host_model, int64_t nbytes);
/* pop_states (:515-517): RecurrentState[POPULATION_SIZE], zero after create. */
int egg_gru_upload_states(egg_gru_ctx *ctx, const void *host_states, int64_t nbytes);
int egg_gru_download_states(egg_gru_ctx *ctx, void *host_states, int64_t nbytes);
int egg_gru_set_dataset(egg_gru_ctx *ctx, const uint8_t *host_tokens, int64_t n_tokens);
/*
 * ≙ one iteration of the training loop (full_trained_egg.c:529-575): every pair p runs
 * forward_pass twice (noise sign +1 / -1, seed step_seed + p) over `tokens` tokens (<= seq_len; the
 * reference always runs seq_len) starting at (start_idx + p * (len / pairs)) % (len - seq_len),
 * carrying its RecurrentState; fitness = sign of the loss difference; if do_update, every matrix goes
 * through update_matrix (:332-409, :564-574).  host_losses[POPULATION_SIZE] and
 * host_fitness[POPULATION_SIZE/2] may be NULL.
 */
int egg_gru_generation(egg_gru_ctx *ctx, uint32_t step_seed, int64_t start_idx, int tokens, int do_update,
                       int32_t *host_losses, int32_t *host_fitness);
/* Kernel launches issued by this context so far. */
int64_t egg_gru_launch_count(egg_gru_ctx *ctx);

/* ---- d-eggs worker boundary (host side, no GPU involved) ------------------ */
/* Opcodes and the 10-byte "JOBS" header of d-eggs/include/protocol.h:8-56. */
#define EGG_OP_JOB_REQUEST  0
#define EGG_OP_RESULT       1
#define EGG_OP_JOB_RESPONSE 2
#define EGG_OP_LOG_MESSAGE  3
#define EGG_WIRE_HEADER_BYTES 10
/* Union of the fields of EggJobRequest / EggJobResponseHeader / EggResultHeader
 * (protocol.h:61-160); payload_size is model_size resp. result_size. */
typedef struct egg_wire_msg {
    int32_t  opcode;
    uint32_t payload_size;
    uint64_t seed, last_step, data_position;   /* data_position == (uint64_t)-1: "wait" (coordinator.cpp:277-286) */
    uint64_t updates_count;
    int64_t  sum_loss;
} egg_wire_msg;
int egg_wire_fixed_bytes(int opcode);
/* ≙ egg_write_header + egg_serialize_* ; returns bytes written (header + fixed body). */
int egg_wire_encode(const egg_wire_msg *msg, uint8_t *out, int cap);
/* ≙ egg_parse_header: 0, or -1 bad magic, -2 bad version. total_len = fixed body + payload. */
int egg_wire_decode_header(const uint8_t *buf10, int *opcode, uint32_t *total_len);
/* ≙ egg_deserialize_* */
int egg_wire_decode_body(int opcode, const uint8_t *body, int len, egg_wire_msg *msg);
/* ≙ ternary_pack_estimate_size / ternary_pack / ternary_unpack (d-eggs/include/utils/ternary_pack.h:12-87). */
int64_t egg_ternary_packed_size(int64_t count);
void egg_ternary_pack(const int32_t *values, int64_t count, uint8_t *out);
void egg_ternary_unpack(const uint8_t *in, int64_t count, int32_t *values);
/* ≙ the worker's per-chunk host fitness (worker.cu:635-687): CHUNK_MEAN_FILTER with
 * CHUNK_MEAN_EXPONENT, USE_ADAPTIVE_THRESHOLD with ADAPTIVE_THRESHOLD_ALPHA.
 * losses[count] chunk-relative; fitness[count/2] in {-1,0,1}; *sum_loss = Σ losses. */
int egg_deggs_chunk_fitness(const int32_t *losses, int count, int mean_filter, double exponent,
                            int adaptive_threshold, double alpha, int32_t *fitness, int64_t *sum_loss);
/* ≙ seed = hash_rng(seed, step) after every update (worker.cu:542, coordinator.cpp:406). */
uint32_t egg_next_seed(uint32_t seed, uint64_t step);

/* ≙ get_learning_rate (d-eggs/include/utils/training.h:5-9): 0.5 below step 100, 0.25 below 200, then 0.125. */
float egg_learning_rate(int64_t step);

/*
 * The worker loop of d-eggs/src/worker.cu:390-717 against an unmodified coordinator
 * (d-eggs/src/coordinator.cpp) over d-eggs/include/protocol.h.  Per iteration: JOB_REQUEST(seed,
 * last_step); the answer is either the packed fitness of the whole population for the worker's step
 * (-> apply_update with the learning rate of that step, step = answer's step, seed = hash_rng(seed, step);
 * worker.cu:416-547), a wait (data_position == -1 -> sleep, worker.cu:550-554), or a chunk
 * (data_position = first member -> eval_chunk of chunk_size members at start index step * SEQ_LEN, the
 * per-chunk fitness filter, ternary pack, RESULT with the update count of the last update and the loss
 * sum; worker.cu:557-713).  Every `generate_every` steps the worker that gets chunk 0 sends a sampled
 * continuation as LOG_MESSAGE when the engine can generate.
 *
 * The GPU work is behind three callbacks so that the same loop runs on an egg_ctx
 * (egg_worker_engine_from_ctx) and, in tests, on host-side fakes.  Callbacks return 0 or a negative
 * EGG_E_* code, which ends the loop and is returned.  The loop also ends when the coordinator closes the
 * connection or stays silent for recv_timeout_ms (EGG_E_STATE), when *stop_flag becomes non-zero, at
 * stop_at_step, or after max_requests requests (both -1: never).
 */
typedef struct egg_worker_engine {
    void *self;
    /* losses[count] of members [pop_offset, pop_offset + count) for (seed, step); chunk-relative order */
    int (*eval_chunk)(void *self, uint32_t seed, int64_t step, int pop_offset, int count, int32_t *losses);
    /* one optimiser step from the fitness of all pairs; lr_bias is what the reference passes for emb_bias */
    int (*apply_update)(void *self, const int32_t *fitness, int pairs, uint32_t seed, float lr, float lr_bias, uint64_t *updates);
    /* optional: writes up to cap bytes of text for the coordinator's console, returns their number */
    int (*generate)(void *self, int64_t step, uint32_t seed, char *text, int cap);
} egg_worker_engine;

typedef struct egg_worker_options {
    char host[64];               /* dotted IPv4 address of the coordinator (default 127.0.0.1) */
    int port;                    /* coordinator.cpp:26 listens on 12345 */
    int population_size, chunk_size;     /* POPULATION_SIZE, CHUNK_SIZE of d-eggs/include/config.h:14-46 */
    uint64_t initial_seed;       /* 42, worker.cu:386 */
    int wait_sleep_ms;           /* 100, worker.cu:552 */
    int recv_timeout_ms;         /* give up on a silent coordinator after this long */
    int generate_every;          /* 5, worker.cu:564; 0: never */
    int mean_filter; double mean_exponent; int adaptive_threshold; double threshold_alpha;   /* config.h:212-224 */
    int64_t stop_at_step, max_requests;
    const volatile int *stop_flag;       /* polled once per iteration (the reference's SIGINT flag, worker.cu:244) or NULL */
    /* test hook, called before a RESULT is sent: a non-zero return drops that result (a worker that went silent) */
    int (*before_result)(void *hook_self, int64_t step, int chunk_index);
    void *hook_self;
} egg_worker_options;

typedef struct egg_worker_stats {
    uint64_t requests, chunks_done, updates_applied, waits, results_dropped;
    uint64_t bytes_sent, bytes_received;
    uint64_t final_step, final_seed;
} egg_worker_stats;

void egg_worker_options_defaults(egg_worker_options *opts);
int egg_worker_run(const egg_worker_options *opts, const egg_worker_engine *engine, egg_worker_stats *stats);
/* Binds the callbacks to a context of this library (evaluation through egg_eval_chunk + egg_read_losses,
 * updates through egg_write_fitness + egg_apply_update). */
int egg_worker_engine_from_ctx(egg_ctx *ctx, egg_worker_engine *out);
/* The configuration a context was created with. */
int egg_get_config(egg_ctx *ctx, egg_config *out);

/* ---- run log (≙ egg_disk_log.h / d-eggs/include/utils/log.h) ------------------ */
/*
 * The reference's plain-text run log: a header block with the configuration (egg_disk_log.h:111-138),
 * the column line "Step,RelTime,Loss,Updates,LR" (:139) and one row per step (:222), appended to `path`.
 * The reference also posts every run and step to a third-party tracking service through curl
 * (:177-198, 238-261); that part is left out on purpose: this library opens no network connection here.
 */
typedef struct egg_log egg_log;
int egg_log_open(const char *path, const egg_config *cfg, int num_gpus, uint64_t vram_bytes_per_gpu, egg_log **out);
int egg_log_record(egg_log *log, int64_t step, double loss, uint64_t updates, float learning_rate);
void egg_log_close(egg_log *log);

/* ---- measurement ------------------------------------------------------ */
/*
 * The reference times a generation with clock_gettime around its launches
 * (mgpu.cu:1510, 1680) and has no per-kernel timing.  These helpers time on the
 * device instead: CUDA events recorded on the context's own stream.
 */
int egg_timer_start(egg_ctx *ctx);
/* Records the stop event, synchronises the stream, returns elapsed milliseconds. */
int egg_timer_stop(egg_ctx *ctx, float *ms);

/* Kernel classes of the per-class profile. */
enum {
    EGG_PROF_NOISE = 0,     /* per-pair noise tables                                  */
    EGG_PROF_ROWWISE,       /* embedding / adaptive-normalise / mean-abs norm rows    */
    EGG_PROF_GEMM_GELU,     /* MLP up projection  (tcgen05 int8)                      */
    EGG_PROF_GEMM_PRE32,    /* O and MLP down projections                             */
    EGG_PROF_GEMM_QKV,      /* fused Q|K|V projection + RoPE                          */
    EGG_PROF_GEMM_HEAD,     /* tied-embedding head + cross-entropy                    */
    EGG_PROF_AQN,           /* Q/K/V requantisation                                   */
    EGG_PROF_ATTENTION,     /* causal integer-softmax attention                       */
    EGG_PROF_FITNESS,
    EGG_PROF_UPD_OPERANDS,  /* noise operands of the update GEMM                      */
    EGG_PROF_UPD_GEMM,      /* update reconstruction GEMM + AdamW / Muon momentum     */
    EGG_PROF_UPD_VECTOR,    /* vector parameters                                      */
    EGG_PROF_MUON,          /* Newton–Schulz + apply                                  */
    EGG_PROF_TRANSPOSE,     /* packed -> K-major weight shadows                       */
    EGG_PROF_OVERLAY,       /* adaptive-noise: scaled row dots, overlay steps          */
    EGG_PROF_UPD_APPLY,     /* optimiser step of a matrix from its vote matrices      */
    EGG_PROF_N
};
/* enable != 0: every launch is bracketed by events (a few microseconds each). */
int egg_profile_enable(egg_ctx *ctx, int enable);
/* Synchronises, then adds up what was recorded since the last read:
 * ms[EGG_PROF_N] device time and launches[EGG_PROF_N] launch counts per class. */
int egg_profile_read(egg_ctx *ctx, float *ms, int64_t *launches);
const char *egg_profile_name(int cls);
/* Kernels launched by this context since it was created. */
int64_t egg_launch_count(egg_ctx *ctx);
/* Members evaluated per internal wave (chosen at creation). */
int egg_wave_members(egg_ctx *ctx);
/*
 * The projections that feed an adaptive normalisation (Q/K/V -> adaptive_qkv_normalize, O and MLP-down ->
 * adaptive_layer_normalize; egg_adaptive_normalize.h:10-103, called at mgpu.cu:782-784, 756, 830) run as
 * row-owning kernels that keep a whole output row in tensor memory and write the requantised int8 row
 * directly, whenever seq_len % 128 == 0 and hidden_dim is a multiple of 128 up to 512 (one thread block per
 * 128-row tile) or a multiple of 256 up to 1024 (a cluster of two thread blocks per tile, each owning half of
 * the columns and exchanging the row maxima through the other's shared memory); other shapes take the
 * two-kernel form (int32 pre-activations + row maxima, then a requantisation kernel).  Both forms give
 * identical bytes.
 * At level 2 (the default) the MLP-down projection's epilogue also runs the mean-abs norm that follows the
 * block (apply_standard_norm, mgpu.cu:646-678: LN1 of the next layer or the final norm) and the row dots of the
 * projections after it, so that row-wise kernel launch disappears.  Level 3 does the same for LN2 inside the
 * output projection; it is selectable and tested but not the default: that projection's epilogue is not hidden
 * behind its short contraction (K = hidden_dim), and the norm costs more there than as a kernel of its own
 * (measured on B200: +15 ms in the projections against -12 ms of row-wise kernels per 40960-member generation).
 * enable = 1 keeps the row-owning projections without either, enable = 0 forces the two-kernel form (for A/B timing and for tests that compare the forms); no
 * counterpart in the reference.  egg_fused_epilogues_active returns the level this context's evaluations take
 * (0 when the configuration only allows the two-kernel form).
 */
int egg_set_fused_epilogues(egg_ctx *ctx, int enable);
int egg_fused_epilogues_active(egg_ctx *ctx);
/*
 * Selects the attention kernel (compute_attention's context loop, mgpu.cu:787-825); all forms give identical
 * bytes.  mode 0 (default): warp-level mma.sync kernel, accumulators in registers.  mode 1: scores and the three
 * weight-limb products as tensor-memory MMAs (tcgen05), one thread block per member and head.  mode 2: scores,
 * maxima and weights per warp on mma.sync, the weight-limb products on tcgen05 with the accumulators in tensor
 * memory (two blocks per SM, the tensor core works on one 32-key block while the warps prepare the next).
 * Modes 1 and 2 need seq_len % 128 == 0, seq_len <= 512, head_dim 64.  Off by default: as measured on B200 the
 * per-pair weight arithmetic on the CUDA cores bounds all three, and the default kernel is the fastest
 * (per 262 144 rows at seq_len 256: 0.57 ms, 1.02 ms, about 0.64 ms); kept selectable for comparison.
 */
int egg_set_attention_tensor_core(egg_ctx *ctx, int mode);
/*
 * Measures what the tensor-core loop of the projection GEMM sustains by itself on this GPU: the same
 * kernel (TMA loads, tcgen05.mma kind::i8, two TMEM accumulator stages) with an epilogue that drops the
 * accumulators, on zero-filled operands A[m][k], B[n][k] small enough to stay in L2 (m, n multiples of
 * 256, k a multiple of 128).  *tops = 2*m*n*k*iters / device time, in 1e12 int8 ops per second.  No
 * counterpart in the reference; it is the denominator the projection GEMMs are reported against.
 */
int egg_measure_int8_peak(egg_ctx *ctx, int m, int n, int k, int iters, double *tops);

/*
 * Host-side self test of the index arithmetic the kernels share with the host (no GPU needed): the
 * multiply-shift division that replaces `/ SEQ_LEN`, `/ tiles`, `% HEAD_DIM` in the per-tile code is
 * compared with C division for every divisor up to 4096 (and powers of two and their neighbours up to
 * 2^30) on boundary and pseudo-random dividends below 2^31.  Returns EGG_OK or EGG_E_STATE with the
 * first mismatch in egg_last_error().  No counterpart in the reference (it divides at run time).
 */
int egg_selftest_index_math(void);

#ifdef __cplusplus
}
#endif
#endif /* EGG_B200_H */
