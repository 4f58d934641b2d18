/* Stand-in for the reference's d-eggs/include/utils/log.h, used ONLY to build its unmodified coordinator.cpp as a test
 * peer (oracle/Makefile, target _ref/ref_coordinator_*).  The reference's header posts every run and every step to a
 * third-party web service by shelling out to curl; a test peer must not do that, so this header keeps the three entry
 * points and the configuration record the coordinator fills in, writes the plain CSV rows to the file it is given, and
 * opens no network connection.  TEST INFRASTRUCTURE ONLY: nothing in the library includes it. */
#ifndef EGG_SHIM_UTILS_LOG_H
#define EGG_SHIM_UTILS_LOG_H

#include <stddef.h>
#include <stdio.h>
#include <string.h>
#include <time.h>

typedef struct {
    char filename[256];
    struct timespec start_ts;
    long rows;
} EggLogState;

/* every field coordinator.cpp assigns before egg_log_init */
typedef struct {
    int num_gpus;
    size_t vram_per_gpu;
    int hidden_dim, head_dim, n_layers, seq_len, vocab_size, n_heads, pop_size, softmax_scale_bit;
    int host_gaussian, device_gaussian, host_mask, device_mask;
    int fixed_point, sigma_shift, sigma_shift_vector;
    int shift_attn, shift_qkv, shift_out, shift_logit, shift_mlp_up, shift_mlp_down;
    float softmax_exp_scale;
    float adam_beta1, adam_beta2, adam_eps, adam_weight_decay;
    int use_muon;
    float muon_momentum, muon_lr_scale;
} EggLogConfig;

static inline EggLogState egg_log_init(const char *filename, EggLogConfig config) {
    EggLogState s;
    memset(&s, 0, sizeof(s));
    strncpy(s.filename, filename, sizeof(s.filename) - 1);
    clock_gettime(CLOCK_MONOTONIC, &s.start_ts);
    FILE *f = fopen(s.filename, "a");
    if (f) {
        fprintf(f, "=== Training Run (test peer) === Hidden=%d Layers=%d SeqLen=%d PopSize=%d\n", config.hidden_dim, config.n_layers,
                config.seq_len, config.pop_size);
        fprintf(f, "Step,RelTime,Loss,Updates,LR\n");
        fclose(f);
    }
    return s;
}

static inline void egg_log_record(EggLogState *state, long step, double loss, unsigned long long updates, float lr) {
    struct timespec now;
    clock_gettime(CLOCK_MONOTONIC, &now);
    const double rel = (double)(now.tv_sec - state->start_ts.tv_sec) + (double)(now.tv_nsec - state->start_ts.tv_nsec) / 1e9;
    FILE *f = fopen(state->filename, "a");
    if (f) {
        fprintf(f, "%ld,%.4f,%.4f,%llu,%.6f\n", step, rel, loss, updates, lr);
        fclose(f);
    }
    state->rows++;
}

static inline void egg_log_close(EggLogState *state) { (void)state; }

#endif
