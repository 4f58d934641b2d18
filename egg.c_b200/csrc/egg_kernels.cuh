// Declarations shared between the kernel translation units and the C-ABI layer.
#pragma once

#include <cuda.h>
#include "egg_common.cuh"
#include "egg_gemm.cuh"

namespace egg {

// ---- per-pair noise table -------------------------------------------------
// Every noise vector a wave needs is generated once per (pair, generation) by
// the counter hash and kept in HBM/L2; the 2*seq_len rows of a pair share it.
struct NoiseSeg {
    int off;        // byte offset inside the pair's table
    int len;        // elements (a delta segment occupies 2*len bytes: [+sign][len], [-sign][len])
    int kind;       // 0: noise(S0+seed_a, i)   1: ((n(S0+seed_a,i)*n(S0+seed_b,i)*sign) >> shift) per sign, int8 [2][len]
                    // 2: model[model_off+i] + that delta, int16 [2][len] (occupies 4*len bytes)
    int seed_a, seed_b;
    int shift;
    int64_t model_off;
    int64_t scale_off;   // AdaptiveScales offset of the overlay scaling this segment (-1: raw noise)
    int first;           // index of the segment's first 1024-element slice in the table-wide slice order (set by noise_index_slices)
};

// Fills NoiseSeg::first for a finished segment list and returns the total number of slices.
int noise_index_slices(NoiseSeg *segs, int nsegs);

struct NormOff { int w_m, b_m; };                       // perturbed gain / bias, int16 [2][H] each
struct MlpOff { int up_b, up_a, bup_d, dn_b, dn_a, bdn_d; };
struct LayerOff { NormOff ln1; int qkv_b; int qkv_a; int o_b, o_a; NormOff ln2; MlpOff mlp; };

struct NoiseMap {
    int64_t stride;          // bytes per pair (multiple of 16)
    int emb_a, emb_b, emb_bias_d;
    int head_a;              // emb_a scaled by the embedding_row overlay (equal to emb_a without overlays)
    NormOff ln_init, ln_f;
    MlpOff mlp_init;
    int layer0, layer_stride;   // byte offset of layer 0 block, bytes per layer block
    LayerOff layer_rel;         // offsets relative to the layer block
};

// Builds the map and the segment list for a configuration (host).
void build_noise_map(const egg_config &c, NoiseMap *map, NoiseSeg *segs, int *nsegs, int max_segs);

int launch_noise_fill(cudaStream_t st, int8_t *nt, int64_t stride, const NoiseSeg *d_segs, int nsegs, int n_pairs,
                      uint32_t step_seed, int pair_base, int mask, int gaussian, const int8_t *model, const int8_t *scales);

// ---- row-wise kernels -------------------------------------------------------
struct RowParams {
    int M, H, seq_len;
    FastDiv fd_seq;              // seq_len as a multiply-shift divisor (filled by launch_rowwise)
    const int8_t *nt; int64_t nt_stride;
    // source: embedding (mode 0), adaptive layer normalise of pre32 (mode 1), or the finished int8 stream (mode 2)
    const uint8_t *dataset; int64_t data_len, start_idx, data_stride; int pop_base, use_same_data;
    int tok_wide;                // 0: byte tokens; 1: dataset is a uint32_t array (vocab_size != 256), positions count tokens
    const int8_t *emb_rows;      // token-major copy of the embedding, [vocab][H] (the K-major shadow of the tied head)
    const int8_t *emb_bias; int vocab;
    int nt_emb_a, nt_emb_b, nt_emb_bias_d, emb_shift;
    const int8_t *ov_emb_row, *ov_emb_col;   // adaptive-noise overlays of the embedding ([vocab], [H]) or null
    const int32_t *ntt_coef;     // transformed-window coefficients [wave pairs][seq_len] (ntt_mode != 0) or null
    const int8_t *ntt_rows;      // token-major copies of ntt_emb1..3, [3][vocab][H]
    const int32_t *pre32; int32_t *rowmax;
    // residual stream out (modes 0, 1); in mode 2 the residual stream is final already and is only read, from x_out
    int8_t *x_out;
    // mean-abs norm (apply_standard_norm, mgpu.cu:646-678)
    int nt_w_m, nt_b_m;          // perturbed gain / bias tables (int16 [2][H])
    int8_t *h_out;
    // Σ_d h_d * noise_B[d] for up to three following projections
    int ndots; int nt_dot[3]; int32_t *xb_out; int xb_stride;
    // accumulators to clear for the kernels that follow
    int32_t *zero1;      // [M]
    int32_t *zero2;      // [M]
    int32_t *zero3;      // [M][3]
    int one;             // 1 (filled by launch_rowwise): the multiplier of additions issued as multiply-adds
};
int launch_rowwise(cudaStream_t st, const RowParams &p, int mode);

// Σ x·noise·factor per row under adaptive-noise overlays; overwrites out[r*out_stride + q].
struct ScaledDotParams {
    int M, H, seq_len;
    int terms;                   // 1: x is [M][H];  4: x is [M][4H], four terms per thread summed with a running truncation
    const int8_t *x;
    const int8_t *nt; int64_t nt_stride;
    int ndots; int nt_dot[3];    // offsets of the raw noise vectors (length H*terms) in the pair table
    const int8_t *ov[3];         // overlays over the input index (length H*terms)
    int32_t *out; int out_stride;
};
int launch_scaled_dot(cudaStream_t st, const ScaledDotParams &p);
int launch_overlay_step(cudaStream_t st, int8_t *ov, uint8_t *changed, int n, int inc, int dec);

struct AqnParams {
    int M, H;
    const int32_t *pre3;      // [M][3H]
    const int32_t *rowmax3;   // [M][3]
    int8_t *q, *k, *v;        // [M][H] each
};
int launch_aqn(cudaStream_t st, const AqnParams &p);

struct AttnParams {
    int members, H, head_dim, seq_len, shift_attn;
    const int8_t *q, *k, *v;  // [members*seq_len][H]
    int8_t *ao;               // [members*seq_len][H]
    const int32_t *exp_lut;
    const int8_t *nt; int64_t nt_stride; int nt_o_b;
    int32_t *xbo;             // [members*seq_len] += Σ_d ao_d * noise_B_o[d]
};
int launch_attention(cudaStream_t st, const AttnParams &p);
// the same attention on tcgen05 (egg_attention_tc.cu): whole 128-query blocks of one member, head_dim 64, seq_len <= 512
bool attention_tc_supported(int seq_len, int head_dim);
int launch_attention_tc(cudaStream_t st, const AttnParams &p, int *err);
// scores on mma.sync per warp, Σ wt·v on tcgen05 with the accumulators in tensor memory (egg_attention_tc.cu)
int launch_attention_hy(cudaStream_t st, const AttnParams &p, int *err);

// ---- sampling -----------------------------------------------------------------
struct GenParams {
    int H, V, head_dim, n_layers;
    int shift_attn, shift_out, shift_logit, shift_mlp_up, shift_mlp_down, rope_bit;
    const int8_t *model; ModelLayout L;
    const int8_t *act_lut; const int32_t *exp_lut; const int32_t *rope_lut;
    int8_t *kv;                  // [n_layers][2][seed_len + gen_len][H]
    uint8_t *tokens;             // [seed_len + gen_len]: first seed_len given, rest written
    int seed_len, gen_len;
    uint32_t seed;
    float temp; int filter, min_p_limit, penalty_int;
    int scan_block;              // block size of the reference kernel: fixes the order of its weighted draw
};
int launch_generate(cudaStream_t st, const GenParams &p);

// ---- weights ----------------------------------------------------------------
// packed [K/4][N][4] -> K-major shadow [N][K]
int launch_unpack_transpose(cudaStream_t st, const int8_t *packed, int8_t *shadow, int rows_k, int cols_n);

// ---- row-owning GEMM with the adaptive normalisation fused (egg_gemm_fused.cuh) -----
struct FusedParams;
// mode: FUSED_QKV (out = [3][part_rows][H] int8: q, k, v) or FUSED_RES (out = x [M][H] int8, resid = x, may alias out)
int launch_gemm_fused(cudaStream_t st, int mode, const int8_t *A, const int8_t *B, int8_t *out, const int8_t *resid,
                      const FusedParams &p, int num_sms);
// whether the row-owning kernels can run a configuration (whole tiles inside one member, a row fits tensor memory)
int fused_cluster_size(int hidden);       // blocks per unit of the row-owning GEMM, 0 when the width is unsupported
inline bool fused_supported(int hidden, int seq_len) { return seq_len % 128 == 0 && fused_cluster_size(hidden) > 0; }

// ---- GEMM -------------------------------------------------------------------
// A: [M][K] int8 row-major, B: [N][K] int8 row-major (both device pointers).
int launch_gemm(cudaStream_t st, int epi, const int8_t *A, const int8_t *B, const GemmParams &p, int num_sms);
int gemm_init();   // resolves the driver entry point for tensor-map encoding, sets smem attributes

// ---- fitness / update -------------------------------------------------------
// Transform of every pair's input window (ntt_mode 1..3): see window_transform_kernel.
struct WindowParams {
    int mode, seq_len, pairs;
    const uint8_t *dataset; int tok_wide; int64_t data_len, start_idx, data_stride; int pair_base, use_same_data;
    int32_t *coef;               // [pairs][seq_len]
};
int launch_window_transform(cudaStream_t st, const WindowParams &p);
// Second pass of the head over int32 logits kept in memory (vocab_size != 256): see head_loss_kernel.
struct HeadLossParams {
    int M, V, seq_len;
    FastDiv fd_seq;              // filled by launch_head_loss
    const int32_t *logits;       // [M][V], after >> SHIFT_LOGIT
    const int32_t *rowmax;       // [M] signed row maxima
    const int32_t *exp_lut;      // 256
    const uint32_t *dataset; int64_t data_len, start_idx, data_stride; int pop_base, use_same_data;
    int softmax_scale_bit;
    int32_t *loss;               // [wave members] +=
};
int launch_head_loss(cudaStream_t st, const HeadLossParams &p);
int launch_fitness(cudaStream_t st, const int32_t *loss, int32_t *fit, int pairs);

// operand generation for the update GEMM: NA[n][Kp] = f_p * noise(s_p+off_a, n), NB[k][Kp] = noise(s_p+off_b, k)
// split = 1 doubles the contraction: [f0*a | f1*a] x [b ; 16 b] with f = 16 f1 + f0.
int launch_update_operands(cudaStream_t st, int8_t *na, int8_t *nb, const int32_t *fit, int pairs, int kp, int rows_k,
                           int cols_n, int off_a, int off_b, int seed_base, uint32_t step_seed, int mask, int gaussian,
                           int split);

// Splits of the pair index for the vote GEMM of a rows_k x cols_n matrix over kp (padded) pairs: enough work items to
// fill the GPU twice over, never an empty split.
int vote_gemm_splits(int rows_k, int cols_n, int kp, int num_sms);

// Optimiser step of one matrix from its (partial) vote matrices, element order = the packed weight layout.
struct VoteApplyParams {
    int8_t *w_packed;            // [rows_k/4][cols_n][4]
    float *opt;                  // AdamParam{m,v,acc} (AdamW) or MuonParam{m,acc} (Muon momentum) per packed index
    const int32_t *votes;        // [nsplits][rows_k * cols_n]
    int nsplits; int64_t split_stride;
    int rows_k, cols_n;
    float lr, beta1, beta2, eps, wd, mu;
    unsigned long long *total_updates;
    uint8_t *ch_in, *ch_out;     // AdamW: set to 1 for every input index k / output index n with a changed weight (or null)
    float *m_rowmajor;           // Muon: [rows_k][cols_n] copy of the new momentum
};
int launch_adam_from_votes(cudaStream_t st, const VoteApplyParams &p);        // ES-AdamW (mgpu.cu:1040-1064, 1100-1110)
int launch_muon_m_from_votes(cudaStream_t st, const VoteApplyParams &p);      // m = mu*m + vote, gather (muon_internal.cuh:15-74)

struct VecUpdParams {
    int8_t *v; float *opt; int len; int off_a, off_b, seed_base; const int32_t *fit; int pairs;
    uint32_t step_seed; float lr, beta1, beta2, eps, wd; int mask, gaussian; unsigned long long *total_updates;
    uint8_t *changed;    // [len] set to 1 where the element changed (adaptive-noise overlays) or null
};
int launch_update_vector(cudaStream_t st, const VecUpdParams &p);

// Muon (muon_internal.cuh:77-342): Frobenius normalise, 5 Newton–Schulz steps, quantised apply.
struct MuonWs { float *x, *g, *y; double *norm2; };   // x: rows*cols, g: K*K, y: rows*cols, norm2: 1
int launch_newton_schulz(cudaStream_t st, const MuonWs &ws, int rows, int cols);
int launch_muon_apply(cudaStream_t st, int8_t *w_packed, float *opt, const float *upd_rowmajor, int rows_k, int cols_n,
                      float lr, float wd, unsigned long long *total_updates);

}  // namespace egg
