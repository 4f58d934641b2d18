// C ABI of the library (include/egg_b200.h): context, uploads, the layer-major
// evaluation pipeline, fitness, NCCL exchange, update reconstruction + optimiser.
// "mgpu.cu" = full_cuda_train_transformer_adam_mgpu.cu of the reference.
#include "egg_kernels.cuh"
#include "egg_gemm_fused.cuh"

#include <string>
#include <sys/stat.h>
#include <unistd.h>

#include <dlfcn.h>
#include <math.h>
#include <stdarg.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include <nccl.h>

namespace egg {

static thread_local char g_err[512] = "";
void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

// ---- NCCL, resolved at run time so that single-GPU users need no NCCL at all ----
struct NcclApi {
    void *h = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    // sharded update only
    ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
};
static NcclApi g_nccl;
static int nccl_load() {
    if (g_nccl.h) return EGG_OK;
    const char *names[] = {getenv("EGG_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n) continue;
        g_nccl.h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.h) break;
    }
    if (!g_nccl.h) { set_error("cannot load NCCL (set EGG_NCCL_LIB): %s", dlerror()); return EGG_E_NCCL; }
    *(void **)&g_nccl.GetUniqueId = dlsym(g_nccl.h, "ncclGetUniqueId");
    *(void **)&g_nccl.CommInitRank = dlsym(g_nccl.h, "ncclCommInitRank");
    *(void **)&g_nccl.AllGather = dlsym(g_nccl.h, "ncclAllGather");
    *(void **)&g_nccl.CommDestroy = dlsym(g_nccl.h, "ncclCommDestroy");
    *(void **)&g_nccl.GetErrorString = dlsym(g_nccl.h, "ncclGetErrorString");
    *(void **)&g_nccl.Broadcast = dlsym(g_nccl.h, "ncclBroadcast");
    *(void **)&g_nccl.AllReduce = dlsym(g_nccl.h, "ncclAllReduce");
    *(void **)&g_nccl.GroupStart = dlsym(g_nccl.h, "ncclGroupStart");
    *(void **)&g_nccl.GroupEnd = dlsym(g_nccl.h, "ncclGroupEnd");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllGather || !g_nccl.CommDestroy) {
        set_error("NCCL library lacks required symbols");
        return EGG_E_NCCL;
    }
    return EGG_OK;
}

}  // namespace egg

using namespace egg;

struct ShadowOff { int64_t init_up, init_dn, emb, ntt, layer0, layer_stride, qkv, o, up, dn; };

struct egg_ctx {
    egg_config cfg;
    int device = 0, num_sms = 0;
    cudaStream_t stream = nullptr;
    ModelLayout L;
    int64_t model_bytes = 0, opt_bytes = 0;
    int8_t *d_model = nullptr;
    uint8_t *d_opt = nullptr;
    int8_t *d_shadow = nullptr;
    ShadowOff so;
    std::vector<ParamDesc> params;
    bool have_model = false;
    // adaptive-noise overlays (d-eggs): null until uploaded
    ScalesLayout SL;
    int8_t *d_scales = nullptr;
    bool scales_on = false;
    uint8_t *d_ch_in = nullptr, *d_ch_out = nullptr;
    int ov_inc = 5, ov_dec = 1;
    // tables
    int32_t *d_exp_lut = nullptr, *d_rope_lut = nullptr;
    int2 *d_rope_t = nullptr;           // the same (cos, sin) pairs, [head_dim/2][seq_len]: consecutive tokens are consecutive in memory
    int8_t *d_act_lut = nullptr;
    // dataset
    uint8_t *d_data = nullptr;          // data_len tokens of tok_bytes bytes each
    int64_t data_len = 0, data_cap = 0;  // data_cap in bytes
    int tok_bytes = 1;                  // sizeof(TokenType), mgpu.cu:62-66: 1 at vocab_size 256, 4 otherwise
    int32_t *d_logits = nullptr;        // [wave rows][vocab] int32 logits of the two-pass head (vocab_size != 256 only)
    int32_t *d_coef = nullptr;          // [wave pairs][seq_len] transformed-window coefficients (ntt_mode != 0 only)
    // population buffers
    int32_t *d_loss = nullptr, *d_fit = nullptr;
    // wave scratch
    int wave_members = 0;
    int64_t R = 0;
    int8_t *d_x = nullptr, *d_h = nullptr, *d_u = nullptr, *d_q = nullptr, *d_k = nullptr, *d_v = nullptr, *d_ao = nullptr;
    int32_t *d_pre = nullptr, *d_xb = nullptr, *d_xb2 = nullptr, *d_rowmax = nullptr, *d_rowmax3 = nullptr, *d_xbo = nullptr,
            *d_wave_loss = nullptr;
    // noise
    NoiseMap nmap;
    NoiseSeg *d_segs = nullptr;
    int nsegs = 0;
    int8_t *d_nt = nullptr;
    // update scratch
    int8_t *d_na = nullptr, *d_nb = nullptr;
    int32_t *d_votes = nullptr;         // partial vote matrices of the matrix being updated: [splits][rows*cols]
    int kp = 0;
    MuonWs muon = {nullptr, nullptr, nullptr, nullptr};
    // Newton-Schulz of one matrix runs on a side stream while the main stream builds the next matrix's votes: two
    // workspaces / streams take turns (a 1024-wide product is 64 tiles on 148 SMs, two at a time fill the GPU better)
    MuonWs muon_alt = {nullptr, nullptr, nullptr, nullptr};
    cudaStream_t side[2] = {nullptr, nullptr};
    cudaEvent_t ev_m[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr};
    bool side_used[2] = {false, false};
    int muon_turn = 0;
    unsigned long long *d_updates = nullptr;
    int *d_err = nullptr;
    // grow-only scratch of the isolated entry points (projection, reconstruct, matrix update): allocated on first use,
    // kept for the next call, freed with the context
    void *scratch[16] = {};
    size_t scratch_bytes[16] = {};
    // row-owning projections with the adaptive normalisations fused (default wherever the shapes allow)
    int fused_level = 2;      // 0: two-kernel adaptive norms; 1: row-owning projections; 2: + the next mean-abs norm inside MLP-down;
                              // 3: + LN2 inside the output projection (selectable, slower: that epilogue is not hidden behind its MMAs)
    // attention on tcgen05 (egg_attention_tc.cu) instead of the mma.sync kernel: correct but slower as measured, off by default
    int attention_mode = 0;       // 0: mma.sync kernel; 1: tcgen05 scores and sums; 2: mma.sync scores, tcgen05 sums
    // measurement
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    bool prof_on = false;
    std::vector<cudaEvent_t> prof_ev;      // pairs
    std::vector<int> prof_cls;             // class of pair i
    size_t prof_used = 0;
    int64_t launches = 0;
    int64_t prof_launches[EGG_PROF_N] = {};
    // multi-GPU
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    // sharded update: every parameter is reconstructed and stepped by one rank (owner[i] for params[i]) and its new int8
    // weights are broadcast.  The optimiser state of a parameter is current on its owner only.
    bool shard_update = false;
    std::vector<int> owner;
};

// Brackets one launch (or launch group) with events when profiling is on.
struct ProfScope {
    egg_ctx *c; int idx; cudaStream_t st;
    ProfScope(egg_ctx *ctx, int cls, int nlaunch = 1, cudaStream_t stream = nullptr) : c(ctx), idx(-1), st(stream ? stream : ctx->stream) {
        c->launches += nlaunch;
        if (!c->prof_on) return;
        c->prof_launches[cls] += nlaunch;
        if (c->prof_used + 2 > c->prof_ev.size()) {
            size_t old = c->prof_ev.size();
            c->prof_ev.resize(old + 512);
            for (size_t i = old; i < c->prof_ev.size(); i++) cudaEventCreate(&c->prof_ev[i]);
        }
        idx = (int)c->prof_used;
        c->prof_used += 2;
        c->prof_cls.resize(c->prof_used / 2);
        c->prof_cls[idx / 2] = cls;
        cudaEventRecord(c->prof_ev[idx], st);
    }
    ~ProfScope() { if (idx >= 0) cudaEventRecord(c->prof_ev[idx + 1], st); }
};
#define PROF(cls, call) [&]() { ProfScope ps_(c, cls); return (call); }()
#define PROFN(cls, n, call) [&]() { ProfScope ps_(c, cls, n); return (call); }()

// ---------------------------------------------------------------- config

extern "C" void egg_config_defaults(egg_config *c) {
    memset(c, 0, sizeof(*c));
    c->hidden_dim = 256; c->head_dim = 64; c->n_layers = 4; c->seq_len = 32; c->vocab_size = 256;
    c->population_size = 8192 * 2 * 4;
    c->fixed_point = 4; c->sigma_shift = 3; c->sigma_shift_vector = 4;
    c->shift_attn = 8; c->shift_out = 9; c->shift_logit = 8; c->shift_mlp_up = 8; c->shift_mlp_down = 10;
    c->softmax_scale_bit = 18; c->rope_scale_bit = 20;
    c->device_mask = 15; c->device_gaussian = 0; c->host_mask = 15;
    c->use_same_data = 0; c->use_muon = 0; c->chunk_relative_loss = 0;
    c->softmax_exp_scale = 6.0;
    c->adam_beta1 = 0.9f; c->adam_beta2 = 0.95f; c->adam_eps = 1e-8f; c->adam_weight_decay = 0.01f;
    c->muon_momentum = 0.85f; c->muon_lr_scale = 1.0f;
}

extern "C" int egg_config_validate(const egg_config *c, const char **why) {
    const char *w = nullptr;
    if (c->hidden_dim < 128 || c->hidden_dim > 1024 || c->hidden_dim % 128) w = "hidden_dim must be a multiple of 128 in [128,1024]";
    else if (c->head_dim != 64) w = "head_dim must be 64";
    else if (c->n_layers < 1 || c->n_layers > 64) w = "n_layers out of range";
    else if (c->seq_len < 16 || c->seq_len % 16 || c->seq_len > 1024) w = "seq_len must be a multiple of 16 in [16,1024] (a head's K and V stay in shared memory for the whole attention block)";
    else if (c->vocab_size < 256 || c->vocab_size > 65536 || c->vocab_size % 256) w = "vocab_size must be a multiple of 256 in [256,65536]";
    else if (c->population_size < 2 || c->population_size % 2) w = "population_size must be even";
    else if (c->device_mask < 0 || c->device_mask > 15) w = "device_mask must be in [0,15]";
    else if (c->softmax_scale_bit < 1 || c->softmax_scale_bit > 20) w = "softmax_scale_bit must be in [1,20] (three 7-bit weight limbs)";
    else if (c->rope_scale_bit < 1 || c->rope_scale_bit > 30) w = "rope_scale_bit out of range";
    else if (c->fixed_point < 0 || c->fixed_point > 7) w = "fixed_point out of range";
    else if (c->ntt_mode < 0 || c->ntt_mode > 3) w = "ntt_mode must be 0, 1, 2 or 3";
    else if (c->ntt_mode && ((c->seq_len & (c->seq_len - 1)) || c->seq_len > c->hidden_dim))
        w = "ntt_mode needs a power-of-two seq_len no larger than hidden_dim (the reference transforms the window with one thread per hidden unit)";
    else if (c->ntt_mode == 2 && c->seq_len > 256) w = "ntt_mode 2 (Fermat-257) needs seq_len <= 256";
    else if (c->sigma_shift_vector < 0 || c->sigma_shift_vector > 16 || c->sigma_shift < 0 || c->sigma_shift > 16) w = "sigma shifts out of range";
    if (!w) {
        // the mean-abs norm divides x * (gain + noise delta) exactly only below 2^16 in magnitude
        const int nmax = (c->device_gaussian ? 3 : 1) * c->device_mask;
        const int gain_max = 127 + ((nmax * nmax) >> c->sigma_shift_vector);
        if (127 * gain_max >= (1 << 16)) w = "sigma_shift_vector too small for this noise amplitude (perturbed norm gains exceed the exact range)";
    }
    if (why) *why = w ? w : "";
    if (w) { set_error("invalid configuration: %s", w); return EGG_E_INVALID; }
    return EGG_OK;
}

extern "C" int64_t egg_model_bytes(const egg_config *c) { return model_layout(*c).total; }

static void build_params(const egg_config &c, const ModelLayout &L, const ShadowOff &so, std::vector<ParamDesc> &out, int64_t *opt_total) {
    // optimiser-state offsets follow the field order of AdamModel (mgpu.cu:337-370)
    const int64_t H = c.hidden_dim, V = c.vocab_size, NL = c.n_layers;
    struct F { int64_t off, n; int hidden; };
    F fields[] = {{L.embedding, V * H, 0}, {L.emb_bias, H, 0}, {L.ntt_emb, c.ntt_mode ? 3 * V * H : 0, 0}, {L.ln_init, H, 0}, {L.ln_init_bias, H, 0},
                  {L.w_emb_mlp_up, 4 * H * H, 1}, {L.mlp_emb_bias_up, 4 * H, 0}, {L.w_emb_mlp_down, 4 * H * H, 1},
                  {L.mlp_emb_bias_down, H, 0}, {L.ln_1, NL * H, 0}, {L.ln_1_bias, NL * H, 0}, {L.w_q, NL * H * H, 1},
                  {L.w_k, NL * H * H, 1}, {L.w_v, NL * H * H, 1}, {L.w_o, NL * H * H, 1}, {L.ln_2, NL * H, 0},
                  {L.ln_2_bias, NL * H, 0}, {L.w_up, NL * 4 * H * H, 1}, {L.mlp_bias_up, NL * 4 * H, 0},
                  {L.w_down, NL * 4 * H * H, 1}, {L.mlp_bias_down, NL * H, 0}, {L.ln_f, H, 0}, {L.ln_f_bias, H, 0}};
    const int nf = sizeof(fields) / sizeof(fields[0]);
    std::vector<int64_t> fopt(nf);
    int64_t bytes = 0;
    for (int i = 0; i < nf; i++) { fopt[i] = bytes; bytes += fields[i].n * ((fields[i].hidden && c.use_muon) ? 8 : 12); }
    if (opt_total) *opt_total = bytes;
    auto opt_of = [&](int64_t model_off, int *esz) {
        for (int i = nf - 1; i >= 0; i--)
            if (fields[i].off <= model_off) {
                int e = (fields[i].hidden && c.use_muon) ? 8 : 12;
                if (esz) *esz = e;
                return fopt[i] + (model_off - fields[i].off) * e;
            }
        return (int64_t)-1;
    };
    const ScalesLayout S = scales_layout(c);
    // ov_in / ov_out: overlays over the input index k ("_row") and the output index n ("_col") as the worker passes
    // them (worker.cu:465-517); for the embedding these are embedding_col / embedding_row (worker.cu:499-519)
    auto mat = [&](int64_t off, int rows, int cols, int a, int b, int base, int hidden, int64_t shadow, int64_t ov_in, int64_t ov_out, float sc = 1.0f) {
        ParamDesc d; d.model_off = off; d.opt_off = opt_of(off, nullptr); d.rows_k = rows; d.cols_n = cols; d.off_a = a; d.off_b = b;
        d.seed_base = base; d.lr_scale = sc; d.muon = hidden && c.use_muon; d.shadow_off = shadow; d.ov_in = ov_in; d.ov_out = ov_out;
        out.push_back(d);
    };
    auto vec = [&](int64_t off, int len, int a, int b, int base, float sc, int64_t ov) {
        ParamDesc d; d.model_off = off; d.opt_off = opt_of(off, nullptr); d.rows_k = 0; d.cols_n = len; d.off_a = a; d.off_b = b;
        d.seed_base = base; d.lr_scale = sc; d.muon = 0; d.shadow_off = -1; d.ov_in = ov; d.ov_out = -1; out.push_back(d);
    };
    const int h = (int)H;
    for (int l = 0; l < c.n_layers; l++) {     // mgpu.cu:1603-1621
        int sb = l * 1000;
        int64_t hh = H * H, sl = so.layer0 + l * so.layer_stride, lH = l * H;
        mat(L.w_q + l * hh, h, h, 200, 201, sb, 1, sl + so.qkv, S.w_q_row + lH, S.w_q_col + lH);
        mat(L.w_k + l * hh, h, h, 202, 203, sb, 1, sl + so.qkv + hh, S.w_k_row + lH, S.w_k_col + lH);
        mat(L.w_v + l * hh, h, h, 204, 205, sb, 1, sl + so.qkv + 2 * hh, S.w_v_row + lH, S.w_v_col + lH);
        mat(L.w_o + l * hh, h, h, 206, 207, sb, 1, sl + so.o, S.w_o_row + lH, S.w_o_col + lH);
        mat(L.w_up + l * 4 * hh, h, 4 * h, 400, 401, sb, 1, sl + so.up, S.w_up_row + lH, S.w_up_col + 4 * lH);
        mat(L.w_down + l * 4 * hh, 4 * h, h, 402, 403, sb, 1, sl + so.dn, S.w_down_row + 4 * lH, S.w_down_col + lH);
        vec(L.ln_1 + l * H, h, 100, 101, sb, 1.0f, S.ln_1 + lH);
        vec(L.ln_1_bias + l * H, h, 110, 111, sb, 1.0f, S.ln_1_bias + lH);
        vec(L.ln_2 + l * H, h, 300, 301, sb, 1.0f, S.ln_2 + lH);
        vec(L.ln_2_bias + l * H, h, 310, 311, sb, 1.0f, S.ln_2_bias + lH);
        vec(L.mlp_bias_up + l * 4 * H, 4 * h, 410, 411, sb, 1.0f, S.mlp_bias_up + 4 * lH);
        vec(L.mlp_bias_down + l * H, h, 412, 413, sb, 1.0f, S.mlp_bias_down + lH);
    }
    vec(L.ln_f, h, 900, 901, 0, 1.0f, S.ln_f);             // mgpu.cu:1623-1643
    vec(L.ln_f_bias, h, 910, 911, 0, 1.0f, S.ln_f_bias);
    vec(L.ln_init, h, 500, 501, 0, 1.0f, S.ln_init);
    vec(L.ln_init_bias, h, 502, 503, 0, 1.0f, S.ln_init_bias);
    mat(L.w_emb_mlp_up, h, 4 * h, 510, 511, 0, 1, so.init_up, S.w_emb_mlp_up_row, S.w_emb_mlp_up_col);
    vec(L.mlp_emb_bias_up, 4 * h, 514, 515, 0, 1.0f, S.mlp_emb_bias_up);
    mat(L.w_emb_mlp_down, 4 * h, h, 512, 513, 0, 1, so.init_dn, S.w_emb_mlp_down_row, S.w_emb_mlp_down_col);
    vec(L.mlp_emb_bias_down, h, 516, 517, 0, 1.0f, S.mlp_emb_bias_down);
    vec(L.emb_bias, h, 50, 51, 0, 0.1f, S.emb_bias);
    mat(L.embedding, h, (int)V, 0, 0 + h, 0, 0, so.emb, S.embedding_col, S.embedding_row);
    // the three coefficient-byte tables of the transformed-window variant: AdamW at half the rate, seeds 600 / 610 / 620
    // (mgpu.cu:168-170, 1645-1668); the adaptive-noise overlays have no entry for them
    if (c.ntt_mode)
        for (int k = 0; k < 3; k++)
            mat(L.ntt_emb + k * V * H, h, (int)V, 600 + 10 * k, 600 + 10 * k + h, 0, 0, so.ntt + k * V * H, -1, -1, 0.5f);
}

static ShadowOff shadow_offsets(const egg_config &c, int64_t *total) {
    const int64_t H = c.hidden_dim, V = c.vocab_size;
    ShadowOff s; int64_t o = 0;
    s.init_up = o; o += 4 * H * H;
    s.init_dn = o; o += 4 * H * H;
    s.emb = o; o += V * H;
    s.ntt = o; o += c.ntt_mode ? 3 * V * H : 0;
    s.layer0 = o;
    s.qkv = 0; s.o = 3 * H * H; s.up = 4 * H * H; s.dn = 8 * H * H; s.layer_stride = 12 * H * H;
    o += c.n_layers * s.layer_stride;
    if (total) *total = o;
    return s;
}

extern "C" int64_t egg_opt_state_bytes(const egg_config *c) {
    ModelLayout L = model_layout(*c);
    ShadowOff so = shadow_offsets(*c, nullptr);
    std::vector<ParamDesc> p; int64_t total = 0;
    build_params(*c, L, so, p, &total);
    return total;
}

extern "C" const char *egg_last_error(void) { return g_err; }

// ---------------------------------------------------------------- tables (init_tables, mgpu.cu:394-426)
static void host_tables(const egg_config &c, std::vector<int32_t> &exp_lut, std::vector<int8_t> &act_lut, std::vector<int32_t> &rope) {
    exp_lut.resize(256); act_lut.resize(256); rope.resize((size_t)c.seq_len * c.head_dim);
    const double softmax_scale = (double)(1 << c.softmax_scale_bit);
    for (int i = 0; i < 256; i++) {
        double val = exp(-(double)i / c.softmax_exp_scale) * softmax_scale;
        exp_lut[i] = (val >= 1.0) ? (int32_t)round(val) : 0;
    }
    for (int i = 0; i < 256; i++) {
        int8_t input = (int8_t)i;
        double x = (double)input / (1 << c.fixed_point);
        double y = 0.5 * x * (1.0 + erf(x / 1.41421356));
        int val = (int)round(y * (1 << c.fixed_point));
        act_lut[i] = (int8_t)((val > 127) ? 127 : ((val < -127) ? -127 : val));
    }
    const double rope_scale = (double)(1 << c.rope_scale_bit);
    for (int t = 0; t < c.seq_len; t++)
        for (int i = 0; i < c.head_dim / 2; i++) {
            double theta = pow(10000.0, -2.0 * i / c.head_dim);
            double alpha = t * theta;
            rope[(size_t)t * c.head_dim + 2 * i] = (int32_t)round(cos(alpha) * rope_scale);
            rope[(size_t)t * c.head_dim + 2 * i + 1] = (int32_t)round(sin(alpha) * rope_scale);
        }
}

// ---------------------------------------------------------------- context

template <typename T>
static int dev_alloc(T **p, int64_t count) {
    cudaError_t e = cudaMalloc((void **)p, (size_t)(count > 0 ? count : 1) * sizeof(T));
    if (e != cudaSuccess) { set_error("cudaMalloc of %lld bytes failed: %s", (long long)(count * (int64_t)sizeof(T)), cudaGetErrorString(e)); *p = nullptr; return EGG_E_NOMEM; }
    return EGG_OK;
}

extern "C" void egg_ctx_destroy(egg_ctx *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(c->comm);
    void *ptrs[] = {c->d_model, c->d_opt, c->d_shadow, c->d_exp_lut, c->d_rope_lut, c->d_rope_t, c->d_act_lut, c->d_data, c->d_loss, c->d_fit,
                    c->d_x, c->d_h, c->d_u, c->d_q, c->d_ao, c->d_pre, c->d_xb, c->d_xb2, c->d_rowmax,
                    c->d_rowmax3, c->d_xbo, c->d_wave_loss, c->d_logits, c->d_coef, c->d_segs, c->d_nt, c->d_na, c->d_nb, c->d_votes, c->muon.x, c->muon.g,
                    c->muon.y, c->muon.norm2, c->d_updates, c->d_err, c->d_scales, c->d_ch_in, c->d_ch_out};
    for (void *p : ptrs) if (p) cudaFree(p);
    void *alt[] = {c->muon_alt.x, c->muon_alt.g, c->muon_alt.y, c->muon_alt.norm2};
    for (void *p : alt) if (p) cudaFree(p);
    for (int b = 0; b < 2; b++) {
        if (c->side[b]) { cudaStreamSynchronize(c->side[b]); cudaStreamDestroy(c->side[b]); }
        if (c->ev_m[b]) cudaEventDestroy(c->ev_m[b]);
        if (c->ev_done[b]) cudaEventDestroy(c->ev_done[b]);
    }
    for (void *p : c->scratch) if (p) cudaFree(p);
    for (cudaEvent_t e : c->prof_ev) cudaEventDestroy(e);
    if (c->t0) cudaEventDestroy(c->t0);
    if (c->t1) cudaEventDestroy(c->t1);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

static int noalloc_scratch_address(int device, int8_t **out);

extern "C" int egg_ctx_create(const egg_config *cfg, int device, int wave_members, egg_ctx **out) {
    if (!cfg || !out) { set_error("null argument"); return EGG_E_INVALID; }
    *out = nullptr;
    int rc = egg_config_validate(cfg, nullptr);
    if (rc) return rc;
    int ndev = 0;
    EGG_CUDA(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev) { set_error("device %d not present (%d devices)", device, ndev); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    EGG_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) { set_error("this library is built for sm_100a only (device is sm_%d%d)", prop.major, prop.minor); return EGG_E_INVALID; }
    if ((rc = gemm_init())) return rc;
    {   // resolve the built-in scratch buffer of egg_update_reconstruct_noalloc now (this device is current), so that
        // the module that holds it is loaded here and that call itself stays a table lookup
        int8_t *unused = nullptr;
        if ((rc = noalloc_scratch_address(device, &unused))) return rc;
    }

    egg_ctx *c = new egg_ctx();
    c->cfg = *cfg; c->device = device; c->num_sms = prop.multiProcessorCount;
    c->L = model_layout(*cfg);
    c->model_bytes = c->L.total;
    int64_t shadow_total = 0;
    c->so = shadow_offsets(*cfg, &shadow_total);
    build_params(*cfg, c->L, c->so, c->params, &c->opt_bytes);
#define TRY(x) do { rc = (x); if (rc) { egg_ctx_destroy(c); return rc; } } while (0)
#define TRYC(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { set_error("%s: %s", #x, cudaGetErrorString(e_)); egg_ctx_destroy(c); return EGG_E_CUDA; } } while (0)
    TRYC(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    TRYC(cudaEventCreate(&c->t0)); TRYC(cudaEventCreate(&c->t1));
    const int64_t H = cfg->hidden_dim, S = cfg->seq_len, POP = cfg->population_size;
    TRY(dev_alloc(&c->d_model, c->model_bytes));
    TRY(dev_alloc(&c->d_opt, c->opt_bytes));
    TRY(dev_alloc(&c->d_shadow, shadow_total));
    TRYC(cudaMemset(c->d_opt, 0, (size_t)c->opt_bytes));
    TRY(dev_alloc(&c->d_exp_lut, 256)); TRY(dev_alloc(&c->d_act_lut, 256)); TRY(dev_alloc(&c->d_rope_lut, S * cfg->head_dim));
    {
        std::vector<int32_t> e, r; std::vector<int8_t> a;
        host_tables(*cfg, e, a, r);
        TRYC(cudaMemcpy(c->d_exp_lut, e.data(), 256 * 4, cudaMemcpyHostToDevice));
        TRYC(cudaMemcpy(c->d_act_lut, a.data(), 256, cudaMemcpyHostToDevice));
        TRYC(cudaMemcpy(c->d_rope_lut, r.data(), r.size() * 4, cudaMemcpyHostToDevice));
        const int hp = cfg->head_dim / 2;
        std::vector<int2> rt((size_t)hp * S);
        for (int t = 0; t < S; t++)
            for (int i = 0; i < hp; i++) rt[(size_t)i * S + t] = make_int2(r[(size_t)t * cfg->head_dim + 2 * i], r[(size_t)t * cfg->head_dim + 2 * i + 1]);
        TRY(dev_alloc(&c->d_rope_t, (int64_t)hp * S));
        TRYC(cudaMemcpy(c->d_rope_t, rt.data(), rt.size() * sizeof(int2), cudaMemcpyHostToDevice));
    }
    TRY(dev_alloc(&c->d_loss, POP)); TRY(dev_alloc(&c->d_fit, POP / 2));
    TRYC(cudaMemset(c->d_loss, 0, (size_t)POP * 4)); TRYC(cudaMemset(c->d_fit, 0, (size_t)(POP / 2) * 4));
    TRY(dev_alloc(&c->d_updates, 1)); TRY(dev_alloc(&c->d_err, 2));
    TRYC(cudaMemset(c->d_err, 0, 8));

    // adaptive-noise overlays and the per-index change flags of one parameter update
    c->SL = scales_layout(*cfg);
    TRY(dev_alloc(&c->d_scales, c->SL.total));
    {
        const int64_t nflag = 4 * H > cfg->vocab_size ? 4 * H : cfg->vocab_size;
        TRY(dev_alloc(&c->d_ch_in, nflag)); TRY(dev_alloc(&c->d_ch_out, nflag));
        TRYC(cudaMemset(c->d_ch_in, 0, (size_t)nflag)); TRYC(cudaMemset(c->d_ch_out, 0, (size_t)nflag));
    }

    // noise map
    std::vector<NoiseSeg> segs(32 + 32 * cfg->n_layers);
    build_noise_map(*cfg, &c->nmap, segs.data(), &c->nsegs, (int)segs.size());
    TRY(dev_alloc(&c->d_segs, c->nsegs));
    TRYC(cudaMemcpy(c->d_segs, segs.data(), c->nsegs * sizeof(NoiseSeg), cudaMemcpyHostToDevice));

    // wave scratch: 23 H bytes + 36 bytes per row, noise table per pair
    // (+ a row of int32 logits per token when the head takes two passes over a vocabulary wider than one tile)
    c->tok_bytes = cfg->vocab_size == 256 ? 1 : 4;
    const int64_t logit_bytes = cfg->vocab_size == 256 ? 0 : (int64_t)cfg->vocab_size * 4;
    const int64_t per_member = S * (23 * H + 40 + logit_bytes) + c->nmap.stride / 2 + 8;
    if (wave_members <= 0) {
        size_t free_b = 0, total_b = 0;
        TRYC(cudaMemGetInfo(&free_b, &total_b));
        int64_t budget = (int64_t)(free_b / 3);
        if (budget > (48ll << 30)) budget = 48ll << 30;
        int64_t wm = budget / per_member;
        wave_members = (int)(wm > 8192 ? 8192 : wm);          // larger waves: fewer launch tails (about 1 % per doubling at H 512)
    }
    if (wave_members > POP) wave_members = (int)POP;
    wave_members &= ~1;
    // keep rows a multiple of the GEMM tile where possible
    while (wave_members > 2 && (wave_members * S) % 128) wave_members -= 2;
    if (wave_members < 2) wave_members = 2;
    c->wave_members = wave_members;
    const int64_t R = (int64_t)wave_members * S;
    c->R = R;
    TRY(dev_alloc(&c->d_x, R * H)); TRY(dev_alloc(&c->d_h, R * H)); TRY(dev_alloc(&c->d_u, R * 4 * H));
    TRY(dev_alloc(&c->d_q, 3 * R * H)); c->d_k = c->d_q + R * H; c->d_v = c->d_q + 2 * R * H;   // one [3][R][H] block: q, k, v
    TRY(dev_alloc(&c->d_ao, R * H));
    TRY(dev_alloc(&c->d_pre, R * 3 * H));
    TRY(dev_alloc(&c->d_xb, R * 3)); TRY(dev_alloc(&c->d_xb2, R)); TRY(dev_alloc(&c->d_rowmax, R)); TRY(dev_alloc(&c->d_rowmax3, R * 3));
    TRY(dev_alloc(&c->d_xbo, R)); TRY(dev_alloc(&c->d_wave_loss, wave_members));
    if (logit_bytes) TRY(dev_alloc(&c->d_logits, R * cfg->vocab_size));
    if (cfg->ntt_mode) TRY(dev_alloc(&c->d_coef, (int64_t)(wave_members / 2) * S));
    TRY(dev_alloc(&c->d_nt, (int64_t)(wave_members / 2) * c->nmap.stride));

    // update scratch
    c->kp = (int)(((POP / 2) + 127) / 128 * 128);
    {
        // the widest output / input dimension of any matrix: 4 H, or the vocabulary of the embedding when that is wider
        const int64_t wide_n = 4 * H > cfg->vocab_size ? 4 * H : cfg->vocab_size;
        TRY(dev_alloc(&c->d_na, wide_n * (int64_t)c->kp)); TRY(dev_alloc(&c->d_nb, 4 * H * (int64_t)c->kp));
    }
    {
        int64_t vmax = 0;
        for (const ParamDesc &d : c->params) {
            if (!d.rows_k) continue;
            const int64_t n = (int64_t)d.rows_k * d.cols_n * vote_gemm_splits(d.rows_k, d.cols_n, c->kp, c->num_sms);
            if (n > vmax) vmax = n;
        }
        TRY(dev_alloc(&c->d_votes, vmax));
    }
    if (cfg->use_muon) {
        TRY(dev_alloc(&c->muon.x, 4 * H * H)); TRY(dev_alloc(&c->muon.y, 4 * H * H)); TRY(dev_alloc(&c->muon.g, H * H));
        TRY(dev_alloc(&c->muon.norm2, 1));
        TRY(dev_alloc(&c->muon_alt.x, 4 * H * H)); TRY(dev_alloc(&c->muon_alt.y, 4 * H * H)); TRY(dev_alloc(&c->muon_alt.g, H * H));
        TRY(dev_alloc(&c->muon_alt.norm2, 1));
        for (int b = 0; b < 2; b++) {
            TRYC(cudaStreamCreateWithFlags(&c->side[b], cudaStreamNonBlocking));
            TRYC(cudaEventCreateWithFlags(&c->ev_m[b], cudaEventDisableTiming));
            TRYC(cudaEventCreateWithFlags(&c->ev_done[b], cudaEventDisableTiming));
        }
    }
#undef TRY
#undef TRYC
    *out = c;
    return EGG_OK;
}

// Scratch slot `slot` with room for `count` elements of T: reuses the slot's buffer when it is large enough.
template <typename T>
static int ctx_scratch(egg_ctx *c, int slot, int64_t count, T **out) {
    const size_t need = (size_t)(count > 0 ? count : 1) * sizeof(T);
    if (c->scratch_bytes[slot] < need) {
        if (c->scratch[slot]) { cudaStreamSynchronize(c->stream); cudaFree(c->scratch[slot]); c->scratch[slot] = nullptr; c->scratch_bytes[slot] = 0; }
        cudaError_t e = cudaMalloc(&c->scratch[slot], need);
        if (e != cudaSuccess) { set_error("cudaMalloc of %zu scratch bytes failed: %s", need, cudaGetErrorString(e)); c->scratch[slot] = nullptr; return EGG_E_NOMEM; }
        c->scratch_bytes[slot] = need;
    }
    *out = static_cast<T *>(c->scratch[slot]);
    return EGG_OK;
}

static int check_dev_err(egg_ctx *c) {
    int h[2] = {0, 0};
    EGG_CUDA(cudaMemcpy(h, c->d_err, 8, cudaMemcpyDeviceToHost));
    if (h[0]) {
        set_error("a device-side wait timed out (code %d)", h[0]);
        cudaMemset(c->d_err, 0, 8);
        return EGG_E_TIMEOUT;
    }
    return EGG_OK;
}

extern "C" int egg_sync(egg_ctx *c) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return check_dev_err(c);
}

// ---------------------------------------------------------------- uploads

static int refresh_shadows(egg_ctx *c) {
    for (const ParamDesc &d : c->params) {
        if (d.rows_k == 0) continue;
        int rc = PROF(EGG_PROF_TRANSPOSE, launch_unpack_transpose(c->stream, c->d_model + d.model_off, c->d_shadow + d.shadow_off, d.rows_k, d.cols_n));
        if (rc) return rc;
    }
    return EGG_OK;
}

extern "C" int egg_upload_model(egg_ctx *c, const void *host_model, int64_t nbytes) {
    if (!c || !host_model) { set_error("null argument"); return EGG_E_INVALID; }
    if (nbytes != c->model_bytes) { set_error("model is %lld bytes, this configuration needs %lld", (long long)nbytes, (long long)c->model_bytes); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaMemcpyAsync(c->d_model, host_model, (size_t)nbytes, cudaMemcpyHostToDevice, c->stream));
    int rc = refresh_shadows(c);
    if (rc) return rc;
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    c->have_model = true;
    return EGG_OK;
}

extern "C" int egg_download_model(egg_ctx *c, void *host_model, int64_t nbytes) {
    if (!c || !host_model) { set_error("null argument"); return EGG_E_INVALID; }
    if (nbytes != c->model_bytes) { set_error("model is %lld bytes", (long long)c->model_bytes); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaMemcpyAsync(host_model, c->d_model, (size_t)nbytes, cudaMemcpyDeviceToHost, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return EGG_OK;
}

extern "C" int egg_upload_opt_state(egg_ctx *c, const void *host_state, int64_t nbytes) {
    if (!c || !host_state) { set_error("null argument"); return EGG_E_INVALID; }
    if (nbytes != c->opt_bytes) { set_error("optimiser state is %lld bytes, expected %lld", (long long)nbytes, (long long)c->opt_bytes); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaMemcpyAsync(c->d_opt, host_state, (size_t)nbytes, cudaMemcpyHostToDevice, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return EGG_OK;
}

static bool update_is_sharded(const egg_ctx *c);
static int broadcast_params(egg_ctx *c, bool opt_state);

extern "C" int egg_download_opt_state(egg_ctx *c, void *host_state, int64_t nbytes) {
    if (!c || !host_state) { set_error("null argument"); return EGG_E_INVALID; }
    if (nbytes != c->opt_bytes) { set_error("optimiser state is %lld bytes", (long long)c->opt_bytes); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    if (update_is_sharded(c)) {
        // every parameter's state is current on its owner only: collect it first (a collective: every rank calls this)
        int rc = broadcast_params(c, true);
        if (rc) return rc;
    }
    EGG_CUDA(cudaMemcpyAsync(host_state, c->d_opt, (size_t)nbytes, cudaMemcpyDeviceToHost, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return EGG_OK;
}

// ---------------------------------------------------------------- checkpoint files (egg_disk_utils.h:1-81)

static int write_file(const std::string &path, const void *data, size_t n) {
    FILE *f = fopen(path.c_str(), "wb");
    if (!f) { set_error("cannot open %s for writing", path.c_str()); return EGG_E_INVALID; }
    size_t w = fwrite(data, 1, n, f);
    if (fclose(f) != 0 || w != n) { set_error("short write to %s", path.c_str()); return EGG_E_INVALID; }
    return EGG_OK;
}

static int read_file(const char *path, std::vector<uint8_t> &out, int64_t want) {
    FILE *f = fopen(path, "rb");
    if (!f) { set_error("cannot open %s", path); return EGG_E_INVALID; }
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    if (n != want) { fclose(f); set_error("%s is %ld bytes, this configuration needs %lld", path, n, (long long)want); return EGG_E_INVALID; }
    out.resize((size_t)n);
    size_t r = fread(out.data(), 1, (size_t)n, f);
    fclose(f);
    if (r != (size_t)n) { set_error("short read from %s", path); return EGG_E_INVALID; }
    return EGG_OK;
}

extern "C" int egg_save_checkpoint(egg_ctx *c, const char *dir, int64_t step) {
    if (!c || !dir || step < 0) { set_error("bad checkpoint arguments"); return EGG_E_INVALID; }
    if (!c->have_model) { set_error("upload a model first"); return EGG_E_STATE; }
    struct stat sb;
    if (stat(dir, &sb) == -1 && mkdir(dir, 0700) != 0) { set_error("cannot create directory %s", dir); return EGG_E_INVALID; }
    std::vector<uint8_t> model((size_t)c->model_bytes), opt((size_t)c->opt_bytes);
    int rc;
    if ((rc = egg_download_model(c, model.data(), c->model_bytes))) return rc;
    if ((rc = egg_download_opt_state(c, opt.data(), c->opt_bytes))) return rc;
    char name_model[128], name_adam[128];
    snprintf(name_model, sizeof(name_model), "egg_step-%08ld.model.bin", (long)step);
    snprintf(name_adam, sizeof(name_adam), "egg_step-%08ld.adam.bin", (long)step);
    const std::string d(dir);
    auto relink = [&](const char *target, const char *link) {
        const std::string lp = d + "/" + link;
        unlink(lp.c_str());
        (void)!symlink(target, lp.c_str());
    };
    if ((rc = write_file(d + "/" + name_model, model.data(), model.size()))) return rc;
    relink(name_model, "egg_transformer_last.model.bin");
    if ((rc = write_file(d + "/" + name_adam, opt.data(), opt.size()))) return rc;
    relink(name_adam, "egg_transformer_last.adam.bin");
    return EGG_OK;
}

extern "C" int egg_load_checkpoint(egg_ctx *c, const char *model_path, const char *adam_path) {
    if (!c || !model_path) { set_error("bad checkpoint arguments"); return EGG_E_INVALID; }
    std::vector<uint8_t> buf;
    int rc;
    if ((rc = read_file(model_path, buf, c->model_bytes))) return rc;
    if ((rc = egg_upload_model(c, buf.data(), c->model_bytes))) return rc;
    if (adam_path) {
        if ((rc = read_file(adam_path, buf, c->opt_bytes))) return rc;
        if ((rc = egg_upload_opt_state(c, buf.data(), c->opt_bytes))) return rc;
    }
    return EGG_OK;
}

extern "C" int64_t egg_scales_bytes(const egg_config *c) { return c ? scales_layout(*c).total : 0; }

extern "C" int egg_upload_scales(egg_ctx *c, const void *host_scales, int64_t nbytes) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    if (!host_scales) { EGG_CUDA(cudaStreamSynchronize(c->stream)); c->scales_on = false; return EGG_OK; }
    if (c->shard_update) { set_error("adaptive-noise overlays are not combined with the sharded update: switch it off first (egg_set_update_sharding(ctx, 0))"); return EGG_E_STATE; }
    if (c->cfg.ntt_mode) { set_error("adaptive-noise overlays are not built for ntt_mode != 0 (AdaptiveScales has no entry for the coefficient tables)"); return EGG_E_INVALID; }
    if (nbytes != c->SL.total) { set_error("overlays are %lld bytes, this configuration needs %lld", (long long)nbytes, (long long)c->SL.total); return EGG_E_INVALID; }
    EGG_CUDA(cudaMemcpyAsync(c->d_scales, host_scales, (size_t)nbytes, cudaMemcpyHostToDevice, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    c->scales_on = true;
    return EGG_OK;
}

extern "C" int egg_download_scales(egg_ctx *c, void *host_scales, int64_t nbytes) {
    if (!c || !host_scales) { set_error("null argument"); return EGG_E_INVALID; }
    if (!c->scales_on) { set_error("no overlays uploaded"); return EGG_E_STATE; }
    if (c->shard_update) { set_error("adaptive-noise overlays are not combined with the sharded update: switch it off first (egg_set_update_sharding(ctx, 0))"); return EGG_E_STATE; }
    if (c->cfg.ntt_mode) { set_error("adaptive-noise overlays are not built for ntt_mode != 0 (AdaptiveScales has no entry for the coefficient tables)"); return EGG_E_INVALID; }
    if (nbytes != c->SL.total) { set_error("overlays are %lld bytes, buffer is %lld", (long long)c->SL.total, (long long)nbytes); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaMemcpyAsync(host_scales, c->d_scales, (size_t)nbytes, cudaMemcpyDeviceToHost, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return EGG_OK;
}

extern "C" int egg_set_overlay_steps(egg_ctx *c, int inc, int dec) {
    if (!c || inc < 0 || dec < 0 || inc > 127 || dec > 127) { set_error("overlay steps must be in [0, 127]"); return EGG_E_INVALID; }
    c->ov_inc = inc; c->ov_dec = dec;
    return EGG_OK;
}

// host_tokens: n tokens of the configuration's TokenType (bytes, or uint32_t when vocab_size != 256)
static int set_dataset_async(egg_ctx *c, const void *host_tokens, int64_t n) {
    if (n <= c->cfg.seq_len + 1) { set_error("dataset must be longer than seq_len+1"); return EGG_E_INVALID; }
    if (c->tok_bytes == 4) {
        // a token outside the vocabulary would index past the embedding table (the reference reads whatever lies there)
        const uint32_t *t = static_cast<const uint32_t *>(host_tokens);
        const uint32_t V = (uint32_t)c->cfg.vocab_size;
        uint32_t top = 0;
        for (int64_t i = 0; i < n; i++) top = t[i] > top ? t[i] : top;      // one vectorisable pass; the position only if it fails
        if (top >= V) {
            int64_t i = 0;
            while (t[i] < V) i++;
            set_error("token %u at position %lld is outside the vocabulary of %u", t[i], (long long)i, V);
            return EGG_E_INVALID;
        }
    }
    const int64_t bytes = n * c->tok_bytes;
    if (bytes > c->data_cap) {
        if (c->d_data) { EGG_CUDA(cudaStreamSynchronize(c->stream)); cudaFree(c->d_data); c->d_data = nullptr; }
        int rc = dev_alloc(&c->d_data, bytes);
        if (rc) return rc;
        c->data_cap = bytes;
    }
    EGG_CUDA(cudaMemcpyAsync(c->d_data, host_tokens, (size_t)bytes, cudaMemcpyHostToDevice, c->stream));
    c->data_len = n;
    return EGG_OK;
}

static int set_dataset_checked(egg_ctx *c, const void *host_tokens, int64_t n_tokens, int width) {
    if (!c || !host_tokens) { set_error("null argument"); return EGG_E_INVALID; }
    if (c->tok_bytes != width) {
        set_error("vocab_size %d takes %s tokens: use %s", c->cfg.vocab_size, c->tok_bytes == 1 ? "byte" : "uint32_t",
                  c->tok_bytes == 1 ? "egg_set_dataset" : "egg_set_dataset_tokens");
        return EGG_E_INVALID;
    }
    EGG_CUDA(cudaSetDevice(c->device));
    int rc = set_dataset_async(c, host_tokens, n_tokens);
    if (rc) return rc;
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return EGG_OK;
}

extern "C" int egg_set_dataset(egg_ctx *c, const uint8_t *host_tokens, int64_t n_tokens) {
    return set_dataset_checked(c, host_tokens, n_tokens, 1);
}

extern "C" int egg_set_dataset_tokens(egg_ctx *c, const uint32_t *host_tokens, int64_t n_tokens) {
    return set_dataset_checked(c, host_tokens, n_tokens, 4);
}

// ---------------------------------------------------------------- evaluation

static bool use_fused(const egg_ctx *c) {
    return c->fused_level > 0 && fused_supported(c->cfg.hidden_dim, c->cfg.seq_len);
}

static FusedParams base_fused(egg_ctx *c, int M, int K, int parts) {
    FusedParams f;
    memset(&f, 0, sizeof(f));
    f.M = M; f.H = c->cfg.hidden_dim; f.K = K; f.parts = parts; f.seq_len = c->cfg.seq_len;
    f.nt = c->d_nt; f.nt_stride = c->nmap.stride; f.nt_c_off = -1;
    f.rank1_shift = c->cfg.fixed_point + c->cfg.sigma_shift;
    f.rope_t = c->d_rope_t; f.head_dim = c->cfg.head_dim; f.rope_bit = c->cfg.rope_scale_bit;
    f.part_rows = c->R;
    f.err = c->d_err;
    return f;
}

static GemmParams base_gemm(egg_ctx *c, int M, int N, int K) {
    GemmParams g;
    memset(&g, 0, sizeof(g));
    g.M = M; g.N = N; g.K = K;
    g.seq_len = c->cfg.seq_len;
    g.nt = c->d_nt; g.nt_stride = c->nmap.stride;
    g.nt_c_off = -1;
    g.rank1_shift = c->cfg.fixed_point + c->cfg.sigma_shift;
    g.act_lut = c->d_act_lut; g.exp_lut = c->d_exp_lut; g.rope_lut = c->d_rope_lut; g.rope_t = c->d_rope_t;
    g.head_dim = c->cfg.head_dim; g.rope_bit = c->cfg.rope_scale_bit;
    g.err = c->d_err;
    return g;
}

// norm + up + down of one MLP block (compute_mlp, mgpu.cu:708-759); X, Hn, xb[.,0] are ready on entry
// Row dots under adaptive-noise overlays: overwrite what the unscaled producers left in `out`.
static int scaled_dots(egg_ctx *c, int M, const int8_t *x, int terms, int ndots, const int *nt_dot, const int64_t *ov_off,
                       int32_t *out, int out_stride) {
    ScaledDotParams sp;
    memset(&sp, 0, sizeof(sp));
    sp.M = M; sp.H = c->cfg.hidden_dim; sp.seq_len = c->cfg.seq_len; sp.terms = terms; sp.x = x;
    sp.nt = c->d_nt; sp.nt_stride = c->nmap.stride; sp.ndots = ndots;
    for (int q = 0; q < ndots; q++) { sp.nt_dot[q] = nt_dot[q]; sp.ov[q] = c->d_scales + ov_off[q]; }
    sp.out = out; sp.out_stride = out_stride;
    return PROF(EGG_PROF_OVERLAY, launch_scaled_dot(c->stream, sp));
}
static int scaled_dot1(egg_ctx *c, int M, const int8_t *x, int terms, int nt_dot, int64_t ov_off, int32_t *out, int out_stride) {
    return scaled_dots(c, M, x, terms, 1, &nt_dot, &ov_off, out, out_stride);
}

// The mean-abs norm that follows an MLP block (LN1 of the next layer or the final norm) and the row dots after it.
struct NextNorm { int w_m, b_m, ndots, dot[3]; };

// nn != null and *norm_done == true on return: the down projection's epilogue also wrote h = norm(x) and the dots.
static int run_mlp(egg_ctx *c, int M, const MlpOff &mo, int nt_base, const int8_t *up_t, const int8_t *up_bias, const int8_t *dn_t,
                   const int8_t *dn_bias, int64_t ov_dn_row, const NextNorm *nn = nullptr, bool *norm_done = nullptr) {
    if (norm_done) *norm_done = false;
    const int H = c->cfg.hidden_dim;
    GemmParams g = base_gemm(c, M, 4 * H, H);
    g.nt_a_off = nt_base + mo.up_a; g.nt_c_off = nt_base + mo.bup_d; g.nt_d_off = nt_base + mo.dn_b;
    g.xb = c->d_xb; g.xb_stride = 3; g.out_shift = c->cfg.shift_mlp_up; g.bias = up_bias; g.out8 = c->d_u; g.rowstat = c->d_xb2;
    int rc = PROF(EGG_PROF_GEMM_GELU, launch_gemm(c->stream, EPI_GELU, c->d_h, up_t, g, c->num_sms));
    if (rc) return rc;
    if (c->scales_on && (rc = scaled_dot1(c, M, c->d_u, 4, nt_base + mo.dn_b, ov_dn_row, c->d_xb2, 1))) return rc;
    if (use_fused(c)) {
        // down projection + residual + bias, adaptive layer normalise in the epilogue: x is rewritten in place
        FusedParams f = base_fused(c, M, 4 * H, 1);
        f.nt_a_off = nt_base + mo.dn_a; f.nt_c_off = nt_base + mo.bdn_d;
        f.xb = c->d_xb2; f.xb_stride = 1; f.out_shift = c->cfg.shift_mlp_down; f.bias = dn_bias;
        if (nn && c->fused_level > 1) {
            // ... and the next mean-abs norm with its row dots (added to a cleared xb) while the row is still on chip
            f.nt_w_m = nn->w_m; f.nt_b_m = nn->b_m; f.ndots = nn->ndots;
            for (int q = 0; q < nn->ndots; q++) f.nt_dot[q] = nn->dot[q];
            f.h_out = c->d_h; f.xb_out = c->d_xb; f.xb_out_stride = 3;
            EGG_CUDA(cudaMemsetAsync(c->d_xb, 0, (size_t)M * 3 * sizeof(int32_t), c->stream));
            if (norm_done) *norm_done = true;
            return PROF(EGG_PROF_GEMM_PRE32, launch_gemm_fused(c->stream, FUSED_RES_LN, c->d_u, dn_t, c->d_x, c->d_x, f, c->num_sms));
        }
        return PROF(EGG_PROF_GEMM_PRE32, launch_gemm_fused(c->stream, FUSED_RES, c->d_u, dn_t, c->d_x, c->d_x, f, c->num_sms));
    }
    GemmParams d = base_gemm(c, M, H, 4 * H);
    d.nt_a_off = nt_base + mo.dn_a; d.nt_c_off = nt_base + mo.bdn_d;
    d.xb = c->d_xb2; d.xb_stride = 1; d.out_shift = c->cfg.shift_mlp_down; d.bias = dn_bias; d.resid = c->d_x; d.out32 = c->d_pre;
    d.rowstat = c->d_rowmax;
    return PROF(EGG_PROF_GEMM_PRE32, launch_gemm(c->stream, EPI_PRE32, c->d_u, dn_t, d, c->num_sms));
}

static RowParams base_row(egg_ctx *c, int M) {
    RowParams r;
    memset(&r, 0, sizeof(r));
    r.M = M; r.H = c->cfg.hidden_dim; r.seq_len = c->cfg.seq_len;
    r.nt = c->d_nt; r.nt_stride = c->nmap.stride;
    r.pre32 = c->d_pre; r.rowmax = c->d_rowmax;
    r.x_out = c->d_x; r.h_out = c->d_h;
    r.xb_out = c->d_xb; r.xb_stride = 3;
    r.zero1 = c->d_xb2; r.zero2 = c->d_xbo; r.zero3 = c->d_rowmax3;
    return r;
}

static int eval_wave(egg_ctx *c, uint32_t step_seed, int64_t start_idx, int pop_base, int members, int32_t *loss_dst) {
    const egg_config &cf = c->cfg;
    const int H = cf.hidden_dim, S = cf.seq_len, V = cf.vocab_size;
    const int M = members * S;
    const ModelLayout &L = c->L;
    const NoiseMap &nm = c->nmap;
    const int8_t *mdl = c->d_model, *sh = c->d_shadow;
    cudaStream_t st = c->stream;
    const ScalesLayout &SL = c->SL;
    const bool sc = c->scales_on;
    int rc;
    if ((rc = PROF(EGG_PROF_NOISE, launch_noise_fill(st, c->d_nt, nm.stride, c->d_segs, c->nsegs, members / 2, step_seed, pop_base / 2, cf.device_mask, cf.device_gaussian, mdl, c->scales_on ? c->d_scales : nullptr)))) return rc;
    EGG_CUDA(cudaMemsetAsync(c->d_wave_loss, 0, (size_t)members * 4, st));
    EGG_CUDA(cudaMemsetAsync(c->d_rowmax, 0, (size_t)M * 4, st));
    const int64_t data_stride = c->data_len / (cf.population_size / 2);

    // embedding + initial norm (mgpu.cu:902-934)
    RowParams r0 = base_row(c, M);
    r0.dataset = c->d_data; r0.data_len = c->data_len; r0.start_idx = start_idx; r0.data_stride = data_stride;
    r0.pop_base = pop_base; r0.use_same_data = cf.use_same_data; r0.tok_wide = c->tok_bytes == 4;
    r0.emb_rows = sh + c->so.emb; r0.emb_bias = mdl + L.emb_bias; r0.vocab = V;
    r0.nt_emb_a = nm.emb_a; r0.nt_emb_b = nm.emb_b; r0.nt_emb_bias_d = nm.emb_bias_d; r0.emb_shift = cf.fixed_point + cf.sigma_shift;
    r0.nt_w_m = nm.ln_init.w_m; r0.nt_b_m = nm.ln_init.b_m;
    r0.ndots = 1; r0.nt_dot[0] = nm.mlp_init.up_b;
    if (sc) { r0.ov_emb_row = c->d_scales + SL.embedding_row; r0.ov_emb_col = c->d_scales + SL.embedding_col; }
    if (cf.ntt_mode) {
        // the pair's window, transformed once (mgpu.cu:877-887); its coefficients pick rows of three more tables
        WindowParams wp;
        memset(&wp, 0, sizeof(wp));
        wp.mode = cf.ntt_mode; wp.seq_len = S; wp.pairs = members / 2; wp.dataset = c->d_data; wp.tok_wide = c->tok_bytes == 4;
        wp.data_len = c->data_len; wp.start_idx = start_idx; wp.data_stride = data_stride; wp.pair_base = pop_base / 2;
        wp.use_same_data = cf.use_same_data; wp.coef = c->d_coef;
        if ((rc = PROF(EGG_PROF_ROWWISE, launch_window_transform(st, wp)))) return rc;
        r0.ntt_coef = c->d_coef; r0.ntt_rows = sh + c->so.ntt;
    }
    if ((rc = PROF(EGG_PROF_ROWWISE, launch_rowwise(st, r0, 0)))) return rc;
    if (sc && (rc = scaled_dot1(c, M, c->d_h, 1, nm.mlp_init.up_b, SL.w_emb_mlp_up_row, c->d_xb, 3))) return rc;
    // the norm after every MLP block: LN1 of the next layer (three dots for q, k, v) or the final norm (one dot for the head)
    auto next_norm = [&](int layer) {
        NextNorm n;
        memset(&n, 0, sizeof(n));
        if (layer < cf.n_layers) {
            const int nbl = nm.layer0 + layer * nm.layer_stride;
            n.w_m = nbl + nm.layer_rel.ln1.w_m; n.b_m = nbl + nm.layer_rel.ln1.b_m; n.ndots = 3;
            n.dot[0] = nbl + nm.layer_rel.qkv_b; n.dot[1] = n.dot[0] + H; n.dot[2] = n.dot[0] + 2 * H;
        } else {
            n.w_m = nm.ln_f.w_m; n.b_m = nm.ln_f.b_m; n.ndots = 1; n.dot[0] = nm.emb_b;
        }
        return n;
    };
    bool norm_done = false;
    NextNorm nn = next_norm(0);
    if ((rc = run_mlp(c, M, nm.mlp_init, 0, sh + c->so.init_up, mdl + L.mlp_emb_bias_up, sh + c->so.init_dn, mdl + L.mlp_emb_bias_down,
                      SL.w_emb_mlp_down_row, &nn, &norm_done))) return rc;

    for (int l = 0; l < cf.n_layers; l++) {
        const int nb = nm.layer0 + l * nm.layer_stride;
        const LayerOff &lo = nm.layer_rel;
        const int8_t *shl = sh + c->so.layer0 + (int64_t)l * c->so.layer_stride;
        // ALN of the previous block -> x (already done by the producing projection on the row-owning path) ; LN1 -> h ;
        // Σ h·b for q,k,v (mgpu.cu:770-776)
        const bool fused = use_fused(c);
        const int row_mode = fused ? 2 : 1;
        RowParams ra = base_row(c, M);
        ra.nt_w_m = nb + lo.ln1.w_m; ra.nt_b_m = nb + lo.ln1.b_m;
        ra.ndots = 3; ra.nt_dot[0] = nb + lo.qkv_b; ra.nt_dot[1] = nb + lo.qkv_b + H; ra.nt_dot[2] = nb + lo.qkv_b + 2 * H;
        if (!norm_done && (rc = PROF(EGG_PROF_ROWWISE, launch_rowwise(st, ra, row_mode)))) return rc;
        const int64_t lH = (int64_t)l * H;
        if (sc) {
            const int64_t ovq[3] = {SL.w_q_row + lH, SL.w_k_row + lH, SL.w_v_row + lH};
            if ((rc = scaled_dots(c, M, c->d_h, 1, 3, ra.nt_dot, ovq, c->d_xb, 3))) return rc;
        }
        if (fused) {
            // Q|K|V projection + RoPE + adaptive_qkv_normalize in one kernel (mgpu.cu:779-784): int8 q, k, v
            FusedParams fq = base_fused(c, M, H, 3);
            fq.nt_a_off = nb + lo.qkv_a; fq.xb = c->d_xb; fq.xb_stride = 3;
            if ((rc = PROF(EGG_PROF_GEMM_QKV, launch_gemm_fused(st, FUSED_QKV, c->d_h, shl + c->so.qkv, c->d_q, nullptr, fq, c->num_sms)))) return rc;
        } else {
            // fused Q|K|V projection + RoPE (mgpu.cu:779-784)
            GemmParams gq = base_gemm(c, M, 3 * H, H);
            gq.nt_a_off = nb + lo.qkv_a; gq.xb = c->d_xb; gq.xb_stride = 3; gq.out32 = c->d_pre; gq.rowstat = c->d_rowmax3; gq.third = H;
            if ((rc = PROF(EGG_PROF_GEMM_QKV, launch_gemm(st, EPI_QKV, c->d_h, shl + c->so.qkv, gq, c->num_sms)))) return rc;
            AqnParams aq; aq.M = M; aq.H = H; aq.pre3 = c->d_pre; aq.rowmax3 = c->d_rowmax3; aq.q = c->d_q; aq.k = c->d_k; aq.v = c->d_v;
            if ((rc = PROF(EGG_PROF_AQN, launch_aqn(st, aq)))) return rc;
        }
        AttnParams ap; ap.members = members; ap.H = H; ap.head_dim = cf.head_dim; ap.seq_len = S; ap.shift_attn = cf.shift_attn;
        ap.q = c->d_q; ap.k = c->d_k; ap.v = c->d_v; ap.ao = c->d_ao; ap.exp_lut = c->d_exp_lut; ap.nt = c->d_nt;
        ap.nt_stride = nm.stride; ap.nt_o_b = nb + lo.o_b; ap.xbo = c->d_xbo;
        if (c->attention_mode == 1 && attention_tc_supported(S, cf.head_dim)) rc = PROF(EGG_PROF_ATTENTION, launch_attention_tc(st, ap, c->d_err));
        else if (c->attention_mode == 2 && attention_tc_supported(S, cf.head_dim)) rc = PROF(EGG_PROF_ATTENTION, launch_attention_hy(st, ap, c->d_err));
        else rc = PROF(EGG_PROF_ATTENTION, launch_attention(st, ap));
        if (rc) return rc;
        if (sc && (rc = scaled_dot1(c, M, c->d_ao, 1, nb + lo.o_b, SL.w_o_row + lH, c->d_xbo, 1))) return rc;
        // output projection + residual (mgpu.cu:828-830)
        bool ln2_done = false;
        if (fused) {
            FusedParams fo = base_fused(c, M, H, 1);
            fo.nt_a_off = nb + lo.o_a; fo.xb = c->d_xbo; fo.xb_stride = 1; fo.out_shift = cf.shift_out;
            if (c->fused_level > 2) {
                // ... and LN2 with the row dot of the MLP's up projection while the row is still on chip; the accumulators the
                // row-wise launch used to clear for the kernels that follow are cleared here instead
                fo.nt_w_m = nb + lo.ln2.w_m; fo.nt_b_m = nb + lo.ln2.b_m; fo.ndots = 1; fo.nt_dot[0] = nb + lo.mlp.up_b;
                fo.h_out = c->d_h; fo.xb_out = c->d_xb; fo.xb_out_stride = 3;
                EGG_CUDA(cudaMemsetAsync(c->d_xb, 0, (size_t)M * 3 * sizeof(int32_t), st));
                if ((rc = PROF(EGG_PROF_GEMM_PRE32, launch_gemm_fused(st, FUSED_RES_LN, c->d_ao, shl + c->so.o, c->d_x, c->d_x, fo, c->num_sms)))) return rc;
                EGG_CUDA(cudaMemsetAsync(c->d_xb2, 0, (size_t)M * sizeof(int32_t), st));
                EGG_CUDA(cudaMemsetAsync(c->d_xbo, 0, (size_t)M * sizeof(int32_t), st));
                ln2_done = true;
            } else if ((rc = PROF(EGG_PROF_GEMM_PRE32, launch_gemm_fused(st, FUSED_RES, c->d_ao, shl + c->so.o, c->d_x, c->d_x, fo, c->num_sms)))) return rc;
        } else {
            GemmParams go = base_gemm(c, M, H, H);
            go.nt_a_off = nb + lo.o_a; go.xb = c->d_xbo; go.xb_stride = 1; go.out_shift = cf.shift_out; go.resid = c->d_x;
            go.out32 = c->d_pre; go.rowstat = c->d_rowmax;
            if ((rc = PROF(EGG_PROF_GEMM_PRE32, launch_gemm(st, EPI_PRE32, c->d_ao, shl + c->so.o, go, c->num_sms)))) return rc;
        }
        // ALN -> x ; LN2 -> h ; Σ h·b_up
        RowParams rb = base_row(c, M);
        rb.nt_w_m = nb + lo.ln2.w_m; rb.nt_b_m = nb + lo.ln2.b_m;
        rb.ndots = 1; rb.nt_dot[0] = nb + lo.mlp.up_b;
        if (!ln2_done && (rc = PROF(EGG_PROF_ROWWISE, launch_rowwise(st, rb, row_mode)))) return rc;
        if (sc && (rc = scaled_dot1(c, M, c->d_h, 1, nb + lo.mlp.up_b, SL.w_up_row + lH, c->d_xb, 3))) return rc;
        nn = next_norm(l + 1);
        if ((rc = run_mlp(c, M, lo.mlp, nb, shl + c->so.up, mdl + L.mlp_bias_up + (int64_t)l * 4 * H, shl + c->so.dn,
                          mdl + L.mlp_bias_down + (int64_t)l * H, SL.w_down_row + 4 * lH, &nn, &norm_done))) return rc;
    }
    // final norm + tied-embedding head + cross-entropy (mgpu.cu:954-1024)
    RowParams rf = base_row(c, M);
    rf.nt_w_m = nm.ln_f.w_m; rf.nt_b_m = nm.ln_f.b_m;
    rf.ndots = 1; rf.nt_dot[0] = nm.emb_b;
    if (!norm_done && (rc = PROF(EGG_PROF_ROWWISE, launch_rowwise(st, rf, use_fused(c) ? 2 : 1)))) return rc;
    if (sc && (rc = scaled_dot1(c, M, c->d_h, 1, nm.emb_b, SL.embedding_col, c->d_xb, 3))) return rc;
    GemmParams gh = base_gemm(c, M, V, H);
    gh.nt_a_off = nm.head_a; gh.xb = c->d_xb; gh.xb_stride = 3; gh.out_shift = cf.shift_logit;
    gh.dataset = c->d_data; gh.data_len = c->data_len; gh.start_idx = start_idx; gh.data_stride = data_stride; gh.pop_base = pop_base;
    gh.use_same_data = cf.use_same_data; gh.softmax_scale_bit = cf.softmax_scale_bit; gh.loss = c->d_wave_loss;
    if (V == 256) {
        if ((rc = PROF(EGG_PROF_GEMM_HEAD, launch_gemm(st, EPI_HEAD, c->d_h, sh + c->so.emb, gh, c->num_sms)))) return rc;
    } else {
        // vocabulary wider than one tile (the reference's strided two-pass loop, mgpu.cu:969-1023): the projection runs once,
        // leaving int32 logits and the row maxima; a row-wise pass then sums the exp table and picks the target logit
        EGG_CUDA(cudaMemsetAsync(c->d_rowmax, 0x80, (size_t)M * 4, st));       // 0x80808080: below every logit
        gh.out32 = c->d_logits; gh.rowstat = c->d_rowmax;
        if ((rc = PROF(EGG_PROF_GEMM_HEAD, launch_gemm(st, EPI_LOGITS, c->d_h, sh + c->so.emb, gh, c->num_sms)))) return rc;
        HeadLossParams hl;
        memset(&hl, 0, sizeof(hl));
        hl.M = M; hl.V = V; hl.seq_len = S; hl.logits = c->d_logits; hl.rowmax = c->d_rowmax; hl.exp_lut = c->d_exp_lut;
        hl.dataset = reinterpret_cast<const uint32_t *>(c->d_data); hl.data_len = c->data_len; hl.start_idx = start_idx;
        hl.data_stride = data_stride; hl.pop_base = pop_base; hl.use_same_data = cf.use_same_data;
        hl.softmax_scale_bit = cf.softmax_scale_bit; hl.loss = c->d_wave_loss;
        if ((rc = PROF(EGG_PROF_GEMM_HEAD, launch_head_loss(st, hl)))) return rc;
    }
    EGG_CUDA(cudaMemcpyAsync(loss_dst, c->d_wave_loss, (size_t)members * 4, cudaMemcpyDeviceToDevice, st));
    return EGG_OK;
}

extern "C" int egg_eval_chunk(egg_ctx *c, uint32_t step_seed, int64_t start_idx, int pop_offset, int count) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    if (!c->have_model || !c->d_data) { set_error("upload a model and a dataset first"); return EGG_E_STATE; }
    if (pop_offset < 0 || count <= 0 || (pop_offset & 1) || (count & 1) || pop_offset + count > c->cfg.population_size) {
        set_error("population range [%d,%d) must be pair-aligned and inside the population", pop_offset, pop_offset + count);
        return EGG_E_INVALID;
    }
    EGG_CUDA(cudaSetDevice(c->device));
    for (int off = 0; off < count; off += c->wave_members) {
        int members = count - off < c->wave_members ? count - off : c->wave_members;
        int32_t *dst = c->d_loss + (c->cfg.chunk_relative_loss ? off : pop_offset + off);
        int rc = eval_wave(c, step_seed, start_idx, pop_offset + off, members, dst);
        if (rc) return rc;
    }
    return EGG_OK;
}

extern "C" int egg_read_losses(egg_ctx *c, int32_t *host_losses, int offset, int count) {
    if (!c || !host_losses || offset < 0 || count < 0 || offset + count > c->cfg.population_size) { set_error("bad loss range"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaMemcpyAsync(host_losses, c->d_loss + offset, (size_t)count * 4, cudaMemcpyDeviceToHost, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return check_dev_err(c);
}

extern "C" int egg_compute_fitness_pairs(egg_ctx *c, int pair_offset, int pair_count) {
    if (!c || pair_offset < 0 || pair_count <= 0 || pair_offset + pair_count > c->cfg.population_size / 2) { set_error("bad pair range"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    return PROF(EGG_PROF_FITNESS, launch_fitness(c->stream, c->d_loss + 2 * (int64_t)pair_offset, c->d_fit + pair_offset, pair_count));
}

extern "C" int egg_write_fitness(egg_ctx *c, const int32_t *host_fitness, int pair_offset, int pair_count) {
    if (!c || !host_fitness || pair_offset < 0 || pair_count < 0 || pair_offset + pair_count > c->cfg.population_size / 2) { set_error("bad pair range"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaMemcpyAsync(c->d_fit + pair_offset, host_fitness, (size_t)pair_count * 4, cudaMemcpyHostToDevice, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return EGG_OK;
}

extern "C" int egg_read_fitness(egg_ctx *c, int32_t *host_fitness, int pair_offset, int pair_count) {
    if (!c || !host_fitness || pair_offset < 0 || pair_count < 0 || pair_offset + pair_count > c->cfg.population_size / 2) { set_error("bad pair range"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaMemcpyAsync(host_fitness, c->d_fit + pair_offset, (size_t)pair_count * 4, cudaMemcpyDeviceToHost, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return EGG_OK;
}

// ---------------------------------------------------------------- sampling

extern "C" int egg_generate(egg_ctx *c, uint8_t *host_tokens, int seed_len, int gen_len, uint32_t seed, float temp, float min_p,
                            float penalty) {
    if (!c || !host_tokens) { set_error("null argument"); return EGG_E_INVALID; }
    if (!c->have_model) { set_error("upload a model first"); return EGG_E_STATE; }
    const egg_config &cf = c->cfg;
    if (cf.vocab_size != 256) { set_error("sampling is built for byte tokens only (vocab_size 256)"); return EGG_E_INVALID; }
    if (cf.ntt_mode) { set_error("sampling is not built for ntt_mode != 0"); return EGG_E_INVALID; }
    const int total = seed_len + gen_len;
    if (seed_len < 1 || gen_len < 0 || total > cf.seq_len || total > 256) { set_error("need 1 <= seed_len and seed_len + gen_len <= min(seq_len, 256)"); return EGG_E_INVALID; }
    if (!(temp > 0.0f)) { set_error("temperature must be positive"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    int8_t *kv = nullptr; uint8_t *tok = nullptr;
    auto cleanup = [&]() { cudaStreamSynchronize(c->stream); if (kv) cudaFree(kv); if (tok) cudaFree(tok); };
#define GTRYC(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { set_error("%s: %s", #x, cudaGetErrorString(e_)); cleanup(); return EGG_E_CUDA; } } while (0)
    const size_t kvb = (size_t)cf.n_layers * 2 * total * cf.hidden_dim;
    GTRYC(cudaMalloc(&kv, kvb)); GTRYC(cudaMalloc(&tok, 256));
    GTRYC(cudaMemsetAsync(kv, 0, kvb, c->stream));
    GTRYC(cudaMemsetAsync(tok, 0, 256, c->stream));
    GTRYC(cudaMemcpyAsync(tok, host_tokens, (size_t)seed_len, cudaMemcpyHostToDevice, c->stream));
    GenParams g;
    memset(&g, 0, sizeof(g));
    g.H = cf.hidden_dim; g.V = cf.vocab_size; g.head_dim = cf.head_dim; g.n_layers = cf.n_layers;
    g.shift_attn = cf.shift_attn; g.shift_out = cf.shift_out; g.shift_logit = cf.shift_logit; g.shift_mlp_up = cf.shift_mlp_up;
    g.shift_mlp_down = cf.shift_mlp_down; g.rope_bit = cf.rope_scale_bit;
    g.model = c->d_model; g.L = c->L; g.act_lut = c->d_act_lut; g.exp_lut = c->d_exp_lut; g.rope_lut = c->d_rope_lut;
    g.kv = kv; g.tokens = tok; g.seed_len = seed_len; g.gen_len = gen_len; g.seed = seed; g.temp = temp;
    g.filter = min_p > 0.0f;
    g.min_p_limit = g.filter ? (int32_t)(logf(min_p) * cf.softmax_exp_scale) : 0;     // kernels.cu:375
    g.penalty_int = (int32_t)(penalty * (float)(1 << cf.shift_logit));                // kernels.cu:374
    g.scan_block = ((cf.hidden_dim + 31) & ~31) > 1024 ? 1024 : ((cf.hidden_dim + 31) & ~31);   // EGG_BLOCK_THREADS, config.h:36-37
    int rc = launch_generate(c->stream, g);
    if (rc) { cleanup(); return rc; }
    c->launches++;
    GTRYC(cudaMemcpyAsync(host_tokens, tok, (size_t)total, cudaMemcpyDeviceToHost, c->stream));
    GTRYC(cudaStreamSynchronize(c->stream));
#undef GTRYC
    cleanup();
    return check_dev_err(c);
}

// ---------------------------------------------------------------- multi-GPU

extern "C" int egg_nccl_unique_id(void *id128) {
    int rc = nccl_load();
    if (rc) return rc;
    ncclUniqueId id;
    ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) { set_error("ncclGetUniqueId failed (%d)", (int)r); return EGG_E_NCCL; }
    memcpy(id128, &id, sizeof(id));
    return EGG_OK;
}

extern "C" int egg_comm_init(egg_ctx *c, const void *id128, int rank, int world) {
    if (!c || !id128 || world < 1 || rank < 0 || rank >= world) { set_error("bad communicator arguments"); return EGG_E_INVALID; }
    if ((c->cfg.population_size / 2) % world) { set_error("POP/2 = %d pairs do not divide over %d ranks", c->cfg.population_size / 2, world); return EGG_E_INVALID; }
    int rc = nccl_load();
    if (rc) return rc;
    EGG_CUDA(cudaSetDevice(c->device));
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclResult_t r = g_nccl.CommInitRank(&c->comm, world, id, rank);
    if (r != ncclSuccess) { set_error("ncclCommInitRank failed (%d)", (int)r); return EGG_E_NCCL; }
    c->rank = rank; c->world = world;
    return EGG_OK;
}

// owners: parameters in order of decreasing cost, each to the rank with the least work so far; the same
// deterministic walk on every rank.  Cost ~ weights for a matrix (tensor-core vote GEMM); a vector element costs
// about 300 matrix elements (its votes are hashed and summed pair by pair on the ordinary cores).
static int64_t update_cost(const ParamDesc &d) { return d.rows_k ? (int64_t)d.rows_k * d.cols_n : (int64_t)d.cols_n * 300; }
static void plan_owners(const std::vector<ParamDesc> &params, int world, std::vector<int> &owner) {
    std::vector<size_t> order(params.size());
    for (size_t i = 0; i < order.size(); i++) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return update_cost(params[a]) > update_cost(params[b]); });
    std::vector<int64_t> load(world, 0);
    owner.assign(params.size(), 0);
    for (size_t i : order) {
        int best = 0;
        for (int r = 1; r < world; r++) if (load[r] < load[best]) best = r;
        owner[i] = best;
        load[best] += update_cost(params[i]);
    }
}

extern "C" int egg_update_owner_plan(const egg_config *cfg, int world, int32_t *owner_out, int64_t *cost_out, int64_t *model_off_out,
                                     int64_t *weights_out, int cap) {
    if (!cfg || world < 1) { set_error("bad arguments"); return EGG_E_INVALID; }
    int rc = egg_config_validate(cfg, nullptr);
    if (rc) return rc;
    const ModelLayout L = model_layout(*cfg);
    const ShadowOff so = shadow_offsets(*cfg, nullptr);
    std::vector<ParamDesc> params;
    build_params(*cfg, L, so, params, nullptr);
    std::vector<int> owner;
    plan_owners(params, world, owner);
    for (size_t i = 0; i < params.size() && (int)i < cap; i++) {
        if (owner_out) owner_out[i] = owner[i];
        if (cost_out) cost_out[i] = update_cost(params[i]);
        if (model_off_out) model_off_out[i] = params[i].model_off;
        if (weights_out) weights_out[i] = params[i].rows_k ? (int64_t)params[i].rows_k * params[i].cols_n : (int64_t)params[i].cols_n;
    }
    return (int)params.size();
}

extern "C" int egg_set_update_sharding(egg_ctx *c, int enable) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    if (!enable) {
        // back to the replicated update: every rank needs every parameter's current state first (a collective)
        if (update_is_sharded(c)) {
            EGG_CUDA(cudaSetDevice(c->device));
            int rc = broadcast_params(c, true);
            if (rc) return rc;
            EGG_CUDA(cudaStreamSynchronize(c->stream));
        }
        c->shard_update = false;
        return EGG_OK;
    }
    if (!c->comm || c->world < 2) { set_error("update sharding needs a communicator over at least two ranks"); return EGG_E_STATE; }
    if (c->scales_on) { set_error("update sharding is not combined with adaptive-noise overlays"); return EGG_E_STATE; }
    plan_owners(c->params, c->world, c->owner);
    c->shard_update = true;
    return EGG_OK;
}

extern "C" int egg_allgather_fitness(egg_ctx *c) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    if (c->world == 1) return EGG_OK;
    if (!c->comm) { set_error("no communicator attached"); return EGG_E_STATE; }
    EGG_CUDA(cudaSetDevice(c->device));
    const size_t per = (size_t)(c->cfg.population_size / 2 / c->world);
    // in place: rank r's slice already sits at d_fit + r*per
    ncclResult_t r = g_nccl.AllGather(c->d_fit + (size_t)c->rank * per, c->d_fit, per, ncclInt32, c->comm, c->stream);
    if (r != ncclSuccess) { set_error("ncclAllGather failed (%d)", (int)r); return EGG_E_NCCL; }
    return EGG_OK;
}

// ---------------------------------------------------------------- update

// One matrix: operands -> vote GEMM (pair index split over the GPU) -> optimiser step from the votes.
// Shared by the model update and by the isolated entry point; all pointers are device pointers.
struct MatrixUpdate {
    int8_t *w_packed; float *opt;
    int rows_k, cols_n, off_a, off_b, seed_base;
    const int32_t *fit; int pairs, kp, operand_split;
    int8_t *na, *nb; int32_t *votes;
    float lr; int muon;
    uint8_t *ch_in, *ch_out;
};

static int run_matrix_update(egg_ctx *c, const MatrixUpdate &u, uint32_t step_seed, bool overlap_muon = false) {
    const egg_config &cf = c->cfg;
    int rc = PROF(EGG_PROF_UPD_OPERANDS, launch_update_operands(c->stream, u.na, u.nb, u.fit, u.pairs, u.kp, u.rows_k, u.cols_n, u.off_a, u.off_b,
                                    u.seed_base, step_seed, cf.device_mask, cf.device_gaussian, u.operand_split));
    if (rc) return rc;
    const int ktot = u.operand_split ? 2 * u.kp : u.kp;
    const int splits = vote_gemm_splits(u.rows_k, u.cols_n, ktot, c->num_sms);
    GemmParams g;
    memset(&g, 0, sizeof(g));
    g.M = u.cols_n; g.N = u.rows_k; g.K = ktot; g.seq_len = 1 << 20;
    g.vote_out = u.votes; g.k_splits = splits; g.split_stride = (int64_t)u.rows_k * u.cols_n; g.err = c->d_err;
    if ((rc = PROF(EGG_PROF_UPD_GEMM, launch_gemm(c->stream, EPI_VOTE, u.na, u.nb, g, c->num_sms)))) return rc;
    VoteApplyParams a;
    memset(&a, 0, sizeof(a));
    a.w_packed = u.w_packed; a.opt = u.opt; a.votes = u.votes; a.nsplits = splits; a.split_stride = g.split_stride;
    a.rows_k = u.rows_k; a.cols_n = u.cols_n;
    a.lr = u.lr; a.beta1 = cf.adam_beta1; a.beta2 = cf.adam_beta2; a.eps = cf.adam_eps; a.wd = cf.adam_weight_decay; a.mu = cf.muon_momentum;
    a.total_updates = c->d_updates; a.ch_in = u.ch_in; a.ch_out = u.ch_out;
    if (!u.muon) return PROF(EGG_PROF_UPD_APPLY, launch_adam_from_votes(c->stream, a));
    if (overlap_muon && c->side[0] && c->muon_alt.x) {
        // momentum on the main stream into workspace b (free once its previous matrix has been applied), then
        // Newton-Schulz and the quantised apply of this matrix on side stream b
        const int b = c->muon_turn++ & 1;
        const MuonWs &ws = b ? c->muon_alt : c->muon;
        if (c->side_used[b]) EGG_CUDA(cudaStreamWaitEvent(c->stream, c->ev_done[b], 0));
        a.m_rowmajor = ws.x;
        if ((rc = PROF(EGG_PROF_UPD_APPLY, launch_muon_m_from_votes(c->stream, a)))) return rc;
        EGG_CUDA(cudaEventRecord(c->ev_m[b], c->stream));
        EGG_CUDA(cudaStreamWaitEvent(c->side[b], c->ev_m[b], 0));
        {
            ProfScope ps_ns(c, EGG_PROF_MUON, 13, c->side[b]);
            if ((rc = launch_newton_schulz(c->side[b], ws, u.rows_k, u.cols_n))) return rc;
            if ((rc = launch_muon_apply(c->side[b], u.w_packed, u.opt, ws.x, u.rows_k, u.cols_n, u.lr * cf.muon_lr_scale, cf.adam_weight_decay, c->d_updates))) return rc;
        }
        EGG_CUDA(cudaEventRecord(c->ev_done[b], c->side[b]));
        c->side_used[b] = true;
        return EGG_OK;
    }
    a.m_rowmajor = c->muon.x;
    if ((rc = PROF(EGG_PROF_UPD_APPLY, launch_muon_m_from_votes(c->stream, a)))) return rc;
    if ((rc = PROFN(EGG_PROF_MUON, 12, launch_newton_schulz(c->stream, c->muon, u.rows_k, u.cols_n)))) return rc;
    ProfScope ps_apply(c, EGG_PROF_MUON);
    return launch_muon_apply(c->stream, u.w_packed, u.opt, c->muon.x, u.rows_k, u.cols_n, u.lr * cf.muon_lr_scale, cf.adam_weight_decay, c->d_updates);
}

static int update_matrix(egg_ctx *c, const ParamDesc &d, uint32_t step_seed, float lr) {
    MatrixUpdate u;
    memset(&u, 0, sizeof(u));
    u.w_packed = c->d_model + d.model_off; u.opt = reinterpret_cast<float *>(c->d_opt + d.opt_off);
    u.rows_k = d.rows_k; u.cols_n = d.cols_n; u.off_a = d.off_a; u.off_b = d.off_b; u.seed_base = d.seed_base;
    u.fit = c->d_fit; u.pairs = c->cfg.population_size / 2; u.kp = c->kp; u.operand_split = 0;
    u.na = c->d_na; u.nb = c->d_nb; u.votes = c->d_votes;
    u.lr = lr * d.lr_scale; u.muon = d.muon;
    if (!d.muon && c->scales_on) { u.ch_in = c->d_ch_in; u.ch_out = c->d_ch_out; }
    int rc = run_matrix_update(c, u, step_seed, true);
    if (rc || d.muon || !c->scales_on) return rc;
    // UPDATE_OVERLAY of the input-index and the output-index overlay (worker.cu:445-455)
    if ((rc = PROF(EGG_PROF_OVERLAY, launch_overlay_step(c->stream, c->d_scales + d.ov_in, c->d_ch_in, d.rows_k, c->ov_inc, c->ov_dec)))) return rc;
    return PROF(EGG_PROF_OVERLAY, launch_overlay_step(c->stream, c->d_scales + d.ov_out, c->d_ch_out, d.cols_n, c->ov_inc, c->ov_dec));
}

static bool update_is_sharded(const egg_ctx *c) { return c->shard_update && c->comm && c->world > 1 && !c->scales_on; }

// One grouped broadcast per parameter from its owner: of the int8 weights, or of the optimiser state.
static int broadcast_params(egg_ctx *c, bool opt_state) {
    if (!g_nccl.Broadcast || !g_nccl.GroupStart || !g_nccl.GroupEnd) { set_error("this NCCL build lacks ncclBroadcast / group calls"); return EGG_E_NCCL; }
    ncclResult_t r = g_nccl.GroupStart();
    for (size_t i = 0; r == ncclSuccess && i < c->params.size(); i++) {
        const ParamDesc &d = c->params[i];
        const size_t n = d.rows_k ? (size_t)d.rows_k * d.cols_n : (size_t)d.cols_n;
        if (opt_state) {
            void *p = c->d_opt + d.opt_off;
            r = g_nccl.Broadcast(p, p, n * (d.muon ? 8 : 12), ncclInt8, c->owner[i], c->comm, c->stream);
        } else {
            void *p = c->d_model + d.model_off;
            r = g_nccl.Broadcast(p, p, n, ncclInt8, c->owner[i], c->comm, c->stream);
        }
    }
    ncclResult_t e = g_nccl.GroupEnd();
    if (r != ncclSuccess || e != ncclSuccess) { set_error("ncclBroadcast of the sharded update failed (%d / %d)", (int)r, (int)e); return EGG_E_NCCL; }
    return EGG_OK;
}

static int apply_update_async(egg_ctx *c, uint32_t step_seed, float lr) {
    const egg_config &cf = c->cfg;
    EGG_CUDA(cudaMemsetAsync(c->d_updates, 0, sizeof(unsigned long long), c->stream));
    const bool sharded = update_is_sharded(c);
    for (size_t i = 0; i < c->params.size(); i++) {
        const ParamDesc &d = c->params[i];
        if (sharded && c->owner[i] != c->rank) continue;       // another rank steps this parameter and sends the result
        int rc;
        if (d.rows_k) {
            rc = update_matrix(c, d, step_seed, lr);
        } else {
            VecUpdParams v;
            v.v = c->d_model + d.model_off; v.opt = reinterpret_cast<float *>(c->d_opt + d.opt_off); v.len = d.cols_n;
            v.off_a = d.off_a; v.off_b = d.off_b; v.seed_base = d.seed_base; v.fit = c->d_fit; v.pairs = cf.population_size / 2;
            v.step_seed = step_seed; v.lr = lr * d.lr_scale; v.beta1 = cf.adam_beta1; v.beta2 = cf.adam_beta2; v.eps = cf.adam_eps;
            v.wd = cf.adam_weight_decay; v.mask = cf.device_mask; v.gaussian = cf.device_gaussian; v.total_updates = c->d_updates;
            v.changed = c->scales_on ? c->d_ch_in : nullptr;
            rc = PROF(EGG_PROF_UPD_VECTOR, launch_update_vector(c->stream, v));
            if (!rc && c->scales_on)
                rc = PROF(EGG_PROF_OVERLAY, launch_overlay_step(c->stream, c->d_scales + d.ov_in, c->d_ch_in, d.cols_n, c->ov_inc, c->ov_dec));
        }
        if (rc) return rc;
    }
    // every matrix still on a side stream must be applied before its K-major shadow is rebuilt
    for (int b = 0; b < 2; b++)
        if (c->side_used[b]) { EGG_CUDA(cudaStreamWaitEvent(c->stream, c->ev_done[b], 0)); c->side_used[b] = false; }
    if (sharded) {
        // the new weights travel from their owners; the owners' change counts add up to the generation's
        int rc = broadcast_params(c, false);
        if (rc) return rc;
        if (!g_nccl.AllReduce) { set_error("this NCCL build lacks ncclAllReduce"); return EGG_E_NCCL; }
        ncclResult_t r = g_nccl.AllReduce(c->d_updates, c->d_updates, 1, ncclUint64, ncclSum, c->comm, c->stream);
        if (r != ncclSuccess) { set_error("ncclAllReduce of the update count failed (%d)", (int)r); return EGG_E_NCCL; }
    }
    return refresh_shadows(c);
}

extern "C" int egg_apply_update(egg_ctx *c, uint32_t step_seed, float learning_rate, uint64_t *total_updates) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    if (!c->have_model) { set_error("upload a model first"); return EGG_E_STATE; }
    EGG_CUDA(cudaSetDevice(c->device));
    int rc = apply_update_async(c, step_seed, learning_rate);
    if (rc) return rc;
    unsigned long long u = 0;
    EGG_CUDA(cudaMemcpyAsync(&u, c->d_updates, sizeof(u), cudaMemcpyDeviceToHost, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    if (total_updates) *total_updates = u;
    return check_dev_err(c);
}

extern "C" int egg_generation_host(egg_ctx *c, const void *host_tokens, int64_t n_tokens, int64_t step, uint32_t step_seed,
                                   float learning_rate, int32_t *host_losses, uint64_t *total_updates) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    if (!c->have_model) { set_error("upload a model first"); return EGG_E_STATE; }
    EGG_CUDA(cudaSetDevice(c->device));
    int rc;
    if (host_tokens && (rc = set_dataset_async(c, host_tokens, n_tokens))) return rc;
    if (!c->d_data) { set_error("no dataset"); return EGG_E_STATE; }
    const int POP = c->cfg.population_size;
    const int per = POP / c->world, off = c->rank * per;
    if (per & 1) { set_error("population slice per rank must be even"); return EGG_E_INVALID; }
    const int saved = c->cfg.chunk_relative_loss;
    c->cfg.chunk_relative_loss = 0;                       // the fitness vector is indexed globally
    rc = egg_eval_chunk(c, step_seed, step * c->cfg.seq_len, off, per);   // start_idx = step*SEQ_LEN, mgpu.cu:1532
    c->cfg.chunk_relative_loss = saved;
    if (rc) return rc;
    if ((rc = PROF(EGG_PROF_FITNESS, launch_fitness(c->stream, c->d_loss + off, c->d_fit + off / 2, per / 2)))) return rc;
    if ((rc = egg_allgather_fitness(c))) return rc;
    if ((rc = apply_update_async(c, step_seed, learning_rate))) return rc;
    unsigned long long u = 0;
    if (host_losses) EGG_CUDA(cudaMemcpyAsync(host_losses, c->d_loss + off, (size_t)per * 4, cudaMemcpyDeviceToHost, c->stream));
    EGG_CUDA(cudaMemcpyAsync(&u, c->d_updates, sizeof(u), cudaMemcpyDeviceToHost, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    if (total_updates) *total_updates = u;
    return check_dev_err(c);
}

// ---------------------------------------------------------------- isolated primitives

__global__ void rowdot_kernel(const int8_t *x, const int8_t *nt, int64_t nt_stride, int nt_b_off, int rows_per_member, int64_t rows,
                              int K, int32_t *xb) {
    const int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= rows) return;
    const int8_t *b = nt + ((r / rows_per_member) >> 1) * nt_stride + nt_b_off;
    int s = 0;
    for (int k = lane * 4; k < K; k += 128) {
        int32_t xv = *reinterpret_cast<const int32_t *>(x + r * K + k);
        int32_t bv = *reinterpret_cast<const int32_t *>(b + k);
        s = __dp4a(xv, bv, s);
    }
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
    if (lane == 0) xb[r] = s;
}

extern "C" int egg_perturbed_projection(egg_ctx *c, const int8_t *x, const int8_t *w_packed, int8_t *y, int64_t rows, int K, int N,
                                        int rows_per_member, uint32_t seed, int off_a, int off_b, int rank1_shift, int out_shift,
                                        int on_device) {
    if (!c || !x || !w_packed || !y) { set_error("null argument"); return EGG_E_INVALID; }
    if (rows <= 0 || rows > 0x7FFFFF00ll || K % 128 || N % 128 || K <= 0 || N <= 0 || rows_per_member < 16 || rows % (2 * (int64_t)rows_per_member)) {
        set_error("projection shape unsupported (rows %lld, K %d, N %d, rows/member %d)", (long long)rows, K, N, rows_per_member);
        return EGG_E_INVALID;
    }
    EGG_CUDA(cudaSetDevice(c->device));
    cudaStream_t st = c->stream;
    const int64_t pairs = rows / rows_per_member / 2;
    const int64_t stride = (int64_t)N + K;
    int8_t *d_x = nullptr, *d_w = nullptr, *d_y = nullptr, *d_wt = nullptr, *d_nt = nullptr;
    int32_t *d_xb = nullptr;
    NoiseSeg *d_segs = nullptr;
    int rc = EGG_OK;
    auto cleanup = [&]() { cudaStreamSynchronize(st); };      // buffers live in the context's scratch slots
#define PTRY(e) do { rc = (e); if (rc) { cleanup(); return rc; } } while (0)
#define PTRYC(e) do { cudaError_t e_ = (e); if (e_ != cudaSuccess) { set_error("%s: %s", #e, cudaGetErrorString(e_)); cleanup(); return EGG_E_CUDA; } } while (0)
    if (on_device) { d_x = const_cast<int8_t *>(x); d_w = const_cast<int8_t *>(w_packed); d_y = y; }
    else {
        PTRY(ctx_scratch(c, 4, rows * K, &d_x)); PTRY(ctx_scratch(c, 5, (int64_t)K * N, &d_w)); PTRY(ctx_scratch(c, 6, rows * N, &d_y));
        PTRYC(cudaMemcpyAsync(d_x, x, (size_t)(rows * K), cudaMemcpyHostToDevice, st));
        PTRYC(cudaMemcpyAsync(d_w, w_packed, (size_t)K * N, cudaMemcpyHostToDevice, st));
    }
    PTRY(ctx_scratch(c, 0, (int64_t)K * N, &d_wt)); PTRY(ctx_scratch(c, 1, pairs * stride, &d_nt)); PTRY(ctx_scratch(c, 2, rows, &d_xb));
    PTRY(ctx_scratch(c, 3, 2, &d_segs));
    NoiseSeg segs[2] = {{0, N, 0, off_a, 0, 0, -1, -1, 0}, {N, K, 0, off_b, 0, 0, -1, -1, 0}};
    noise_index_slices(segs, 2);
    PTRYC(cudaMemcpyAsync(d_segs, segs, sizeof(segs), cudaMemcpyHostToDevice, st));
    PTRY(launch_unpack_transpose(st, d_w, d_wt, K, N));
    PTRY(launch_noise_fill(st, d_nt, stride, d_segs, 2, (int)pairs, seed, 0, c->cfg.device_mask, c->cfg.device_gaussian, nullptr, nullptr));
    rowdot_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(d_x, d_nt, stride, N, rows_per_member, rows, K, d_xb);
    PTRYC(cudaGetLastError());
    GemmParams g;
    memset(&g, 0, sizeof(g));
    g.M = (int)rows; g.N = N; g.K = K; g.seq_len = rows_per_member; g.nt = d_nt; g.nt_stride = stride; g.nt_a_off = 0; g.nt_c_off = -1;
    g.xb = d_xb; g.xb_stride = 1; g.rank1_shift = rank1_shift; g.out_shift = out_shift; g.out8 = d_y; g.err = c->d_err;
    PTRY(launch_gemm(st, EPI_CLIP8, d_x, d_wt, g, c->num_sms));
    if (!on_device) PTRYC(cudaMemcpyAsync(y, d_y, (size_t)(rows * N), cudaMemcpyDeviceToHost, st));
    PTRYC(cudaStreamSynchronize(st));
    cleanup();
#undef PTRY
#undef PTRYC
    return check_dev_err(c);
}

extern "C" int egg_update_reconstruct(egg_ctx *c, const int32_t *fitness, int pairs, int rows_k, int cols_n, int off_a, int off_b,
                                      int seed_base, uint32_t step_seed, int32_t *vote_out, int on_device) {
    if (!c || !fitness || !vote_out) { set_error("null argument"); return EGG_E_INVALID; }
    if (pairs <= 0 || rows_k % 128 || cols_n % 128 || rows_k <= 0 || cols_n <= 0) { set_error("reconstruct shape unsupported"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    cudaStream_t st = c->stream;
    const int kp = (pairs + 127) / 128 * 128;
    int32_t *d_fit = nullptr, *d_vote = nullptr;
    int8_t *d_na = nullptr, *d_nb = nullptr;
    int rc = EGG_OK;
    auto cleanup = [&]() { cudaStreamSynchronize(st); };      // buffers live in the context's scratch slots
#define PTRY(e) do { rc = (e); if (rc) { cleanup(); return rc; } } while (0)
#define PTRYC(e) do { cudaError_t e_ = (e); if (e_ != cudaSuccess) { set_error("%s: %s", #e, cudaGetErrorString(e_)); cleanup(); return EGG_E_CUDA; } } while (0)
    // fitness range decides whether f*a fits int8 directly or needs the base-16 split
    int fmax = 0;
    if (on_device) {
        d_fit = const_cast<int32_t *>(fitness); d_vote = vote_out;
        std::vector<int32_t> hf((size_t)pairs);
        PTRYC(cudaMemcpyAsync(hf.data(), fitness, (size_t)pairs * 4, cudaMemcpyDeviceToHost, st));
        PTRYC(cudaStreamSynchronize(st));
        for (int i = 0; i < pairs; i++) { int a = hf[i] < 0 ? -hf[i] : hf[i]; if (a > fmax) fmax = a; }
    } else {
        for (int i = 0; i < pairs; i++) { int a = fitness[i] < 0 ? -fitness[i] : fitness[i]; if (a > fmax) fmax = a; }
        PTRY(ctx_scratch(c, 10, pairs, &d_fit)); PTRY(ctx_scratch(c, 11, (int64_t)rows_k * cols_n, &d_vote));
        PTRYC(cudaMemcpyAsync(d_fit, fitness, (size_t)pairs * 4, cudaMemcpyHostToDevice, st));
    }
    const int amax = c->cfg.device_gaussian ? 3 * c->cfg.device_mask : c->cfg.device_mask;
    if (fmax > 127) { set_error("fitness magnitude %d exceeds 127", fmax); cleanup(); return EGG_E_INVALID; }
    int split = fmax * amax > 127;
    if (split && (15 * amax > 127 || 16 * amax > 127)) {
        set_error("int8 fitness with noise magnitude %d does not fit the two-digit operand split", amax); cleanup(); return EGG_E_INVALID;
    }
    const int ktot = split ? 2 * kp : kp;
    PTRY(ctx_scratch(c, 7, (int64_t)cols_n * ktot, &d_na)); PTRY(ctx_scratch(c, 8, (int64_t)rows_k * ktot, &d_nb));
    PTRY(launch_update_operands(st, d_na, d_nb, d_fit, pairs, kp, rows_k, cols_n, off_a, off_b, seed_base, step_seed,
                                c->cfg.device_mask, c->cfg.device_gaussian, split));
    GemmParams g;
    memset(&g, 0, sizeof(g));
    g.M = cols_n; g.N = rows_k; g.K = ktot; g.seq_len = 1 << 20; g.vote_out = d_vote; g.err = c->d_err;
    PTRY(launch_gemm(st, EPI_VOTE, d_na, d_nb, g, c->num_sms));
    if (!on_device) PTRYC(cudaMemcpyAsync(vote_out, d_vote, (size_t)rows_k * cols_n * 4, cudaMemcpyDeviceToHost, st));
    PTRYC(cudaStreamSynchronize(st));
    cleanup();
#undef PTRY
#undef PTRYC
    return check_dev_err(c);
}

// ---------------------------------------------------------------- isolated matrix update

extern "C" int egg_update_matrix(egg_ctx *c, int8_t *d_w_packed, void *d_opt_state, int rows_k, int cols_n, int off_a, int off_b,
                                 int seed_base, const int32_t *d_fitness, int pairs, uint32_t step_seed, float lr, int optimizer,
                                 int split, uint64_t *total_updates) {
    if (!c || !d_w_packed || !d_opt_state || !d_fitness) { set_error("null argument"); return EGG_E_INVALID; }
    if (pairs <= 0 || rows_k % 128 || cols_n % 128 || rows_k <= 0 || cols_n <= 0 || (optimizer != 0 && optimizer != 1)) {
        set_error("matrix update shape or optimiser unsupported"); return EGG_E_INVALID;
    }
    const int amax = c->cfg.device_gaussian ? 3 * c->cfg.device_mask : c->cfg.device_mask;
    if (split && 16 * amax > 127) { set_error("noise magnitude %d does not fit the two-digit operand split", amax); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    cudaStream_t st = c->stream;
    const int kp = (pairs + 127) / 128 * 128;
    const int ktot = split ? 2 * kp : kp;
    const int splits = vote_gemm_splits(rows_k, cols_n, ktot, c->num_sms);
    MatrixUpdate u;
    memset(&u, 0, sizeof(u));
    MuonWs saved = c->muon, ws = {nullptr, nullptr, nullptr, nullptr};
    int rc = EGG_OK;
    auto cleanup = [&]() { cudaStreamSynchronize(st); c->muon = saved; };      // buffers live in the context's scratch slots
#define UTRY(e) do { rc = (e); if (rc) { cleanup(); return rc; } } while (0)
    UTRY(ctx_scratch(c, 7, (int64_t)cols_n * ktot, &u.na)); UTRY(ctx_scratch(c, 8, (int64_t)rows_k * ktot, &u.nb));
    UTRY(ctx_scratch(c, 9, (int64_t)rows_k * cols_n * splits, &u.votes));
    if (optimizer == 1) {
        const int kmin = rows_k < cols_n ? rows_k : cols_n;
        UTRY(ctx_scratch(c, 12, (int64_t)rows_k * cols_n, &ws.x)); UTRY(ctx_scratch(c, 13, (int64_t)rows_k * cols_n, &ws.y));
        UTRY(ctx_scratch(c, 14, (int64_t)kmin * kmin, &ws.g)); UTRY(ctx_scratch(c, 15, 1, &ws.norm2));
        c->muon = ws;
    }
    u.w_packed = d_w_packed; u.opt = static_cast<float *>(d_opt_state);
    u.rows_k = rows_k; u.cols_n = cols_n; u.off_a = off_a; u.off_b = off_b; u.seed_base = seed_base;
    u.fit = d_fitness; u.pairs = pairs; u.kp = kp; u.operand_split = split ? 1 : 0;
    u.lr = lr; u.muon = optimizer;
    cudaError_t e = cudaMemsetAsync(c->d_updates, 0, sizeof(unsigned long long), st);
    if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); cleanup(); return EGG_E_CUDA; }
    UTRY(run_matrix_update(c, u, step_seed));
    unsigned long long n = 0;
    e = cudaMemcpyAsync(&n, c->d_updates, sizeof(n), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) { set_error("cudaMemcpyAsync: %s", cudaGetErrorString(e)); cleanup(); return EGG_E_CUDA; }
#undef UTRY
    cleanup();
    if (total_updates) *total_updates = n;
    return check_dev_err(c);
}

// ---------------------------------------------------------------- allocation-free reconstruct

// Operand scratch of egg_update_reconstruct_noalloc: part of the library image, one copy per GPU.
// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to hand to a kernel.
static __device__ __align__(256) int8_t g_noalloc_scratch[EGG_NOALLOC_SCRATCH_BYTES];
static int8_t *g_noalloc_ptr[64] = {};     // device address of the array, per device ordinal

// Device address of the array on `device`, which must be the current device: looked up once per device and cached.
static int noalloc_scratch_address(int device, int8_t **out) {
    if (device < 0 || device >= 64) { set_error("device ordinal out of range"); return EGG_E_INVALID; }
    if (!g_noalloc_ptr[device]) {
        void *ptr = nullptr;
        EGG_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        g_noalloc_ptr[device] = static_cast<int8_t *>(ptr);
    }
    *out = g_noalloc_ptr[device];
    return EGG_OK;
}

extern "C" int egg_update_reconstruct_noalloc(egg_ctx *c, const int32_t *d_fitness, int pairs, int rows_k, int cols_n, int off_a,
                                              int off_b, int seed_base, uint32_t step_seed, int split, int32_t *d_vote_out) {
    if (!c || !d_fitness || !d_vote_out) { set_error("null argument"); return EGG_E_INVALID; }
    if (pairs <= 0 || rows_k % 128 || cols_n % 128 || rows_k <= 0 || cols_n <= 0) { set_error("reconstruct shape unsupported"); return EGG_E_INVALID; }
    const int kp = (pairs + 127) / 128 * 128;
    const int64_t ktot = split ? 2 * (int64_t)kp : kp;
    const int64_t need = ((int64_t)rows_k + cols_n) * ktot;
    if (need > (int64_t)EGG_NOALLOC_SCRATCH_BYTES) {
        set_error("needs %lld bytes of operand scratch, the built-in buffer holds %u: use egg_update_reconstruct", (long long)need,
                  EGG_NOALLOC_SCRATCH_BYTES);
        return EGG_E_INVALID;
    }
    const int amax = c->cfg.device_gaussian ? 3 * c->cfg.device_mask : c->cfg.device_mask;
    if (split && 16 * amax > 127) { set_error("noise magnitude %d does not fit the two-digit operand split", amax); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    int8_t *na = nullptr;                  // set-up happened in egg_ctx_create on this device; this is the cached address
    int rc0 = noalloc_scratch_address(c->device, &na);
    if (rc0) return rc0;
    int8_t *nb = na + (int64_t)cols_n * ktot;           // cols_n*ktot is a multiple of 128*128: stays 256-byte aligned
    int rc = launch_update_operands(c->stream, na, nb, d_fitness, pairs, kp, rows_k, cols_n, off_a, off_b, seed_base, step_seed,
                                    c->cfg.device_mask, c->cfg.device_gaussian, split ? 1 : 0);
    if (rc) return rc;
    c->launches += 2;
    GemmParams g;
    memset(&g, 0, sizeof(g));
    g.M = cols_n; g.N = rows_k; g.K = (int)ktot; g.seq_len = 1 << 20; g.vote_out = d_vote_out; g.err = c->d_err;
    if ((rc = launch_gemm(c->stream, EPI_VOTE, na, nb, g, c->num_sms))) return rc;
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return check_dev_err(c);
}

// ---------------------------------------------------------------- measurement

extern "C" int egg_timer_start(egg_ctx *c) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaEventRecord(c->t0, c->stream));
    return EGG_OK;
}

extern "C" int egg_timer_stop(egg_ctx *c, float *ms) {
    if (!c || !ms) { set_error("null argument"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaEventRecord(c->t1, c->stream));
    EGG_CUDA(cudaEventSynchronize(c->t1));
    EGG_CUDA(cudaEventElapsedTime(ms, c->t0, c->t1));
    return check_dev_err(c);
}

extern "C" int egg_profile_enable(egg_ctx *c, int enable) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    c->prof_on = enable != 0;
    return EGG_OK;
}

extern "C" int egg_profile_read(egg_ctx *c, float *ms, int64_t *launches) {
    if (!c || !ms || !launches) { set_error("null argument"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    for (int i = 0; i < EGG_PROF_N; i++) { ms[i] = 0.0f; launches[i] = c->prof_launches[i]; c->prof_launches[i] = 0; }
    for (size_t i = 0; i + 1 < c->prof_used; i += 2) {
        float t = 0.0f;
        EGG_CUDA(cudaEventElapsedTime(&t, c->prof_ev[i], c->prof_ev[i + 1]));
        ms[c->prof_cls[i / 2]] += t;
    }
    c->prof_used = 0;
    return EGG_OK;
}

extern "C" const char *egg_profile_name(int cls) {
    static const char *names[EGG_PROF_N] = {"noise_fill", "rowwise", "gemm_gelu", "gemm_pre32", "gemm_qkv", "gemm_head", "aqn",
                                            "attention", "fitness", "update_operands", "update_gemm", "update_vector", "muon",
                                            "transpose", "overlay", "update_apply"};
    return (cls >= 0 && cls < EGG_PROF_N) ? names[cls] : "";
}

extern "C" int egg_selftest_index_math(void) {
    uint64_t rng = 0x9E3779B97F4A7C15ull;
    auto next = [&]() { rng ^= rng << 13; rng ^= rng >> 7; rng ^= rng << 17; return (int)(rng & 0x7FFFFFFFull); };
    auto check = [&](int d) -> bool {
        const FastDiv f = make_fastdiv(d);
        const int top = 0x7FFFFFFF;
        const long long fixed[] = {0, 1, d - 1, d, (long long)d + 1, 2ll * d - 1, top, top - 1, top - d, (long long)(top / d) * d, (long long)(top / d) * d - 1};
        for (long long nn : fixed) {
            if (nn < 0 || nn > top) continue;
            const int n = (int)nn;
            if (fast_div(n, f) != n / d || fast_mod(n, f) != n % d) { set_error("fast_div(%d, %d) = %d, expected %d", n, d, fast_div(n, f), n / d); return false; }
        }
        for (int i = 0; i < 64; i++) {
            const int n = next();
            if (fast_div(n, f) != n / d || fast_mod(n, f) != n % d) { set_error("fast_div(%d, %d) = %d, expected %d", n, d, fast_div(n, f), n / d); return false; }
        }
        return true;
    };
    for (int d = 1; d <= 4096; d++) if (!check(d)) return EGG_E_STATE;
    for (int k = 12; k <= 30; k++) {
        if (!check(1 << k) || !check((1 << k) - 1) || !check((1 << k) + 1)) return EGG_E_STATE;
    }
    return EGG_OK;
}

extern "C" int egg_measure_int8_peak(egg_ctx *c, int m, int n, int k, int iters, double *tops) {
    if (!c || !tops || m <= 0 || n <= 0 || k <= 0 || iters <= 0 || m % 256 || n % 256 || k % 128) { set_error("m, n must be multiples of 256, k of 128, iters positive"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    int8_t *a = nullptr, *b = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = EGG_OK;
    auto cleanup = [&]() { cudaStreamSynchronize(c->stream); if (a) cudaFree(a); if (b) cudaFree(b); if (e0) cudaEventDestroy(e0); if (e1) cudaEventDestroy(e1); };
#define MTRY(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { set_error("%s: %s", #x, cudaGetErrorString(e_)); cleanup(); return EGG_E_CUDA; } } while (0)
    MTRY(cudaMalloc(&a, (size_t)m * k)); MTRY(cudaMalloc(&b, (size_t)n * k));
    MTRY(cudaMemsetAsync(a, 0, (size_t)m * k, c->stream)); MTRY(cudaMemsetAsync(b, 0, (size_t)n * k, c->stream));
    MTRY(cudaEventCreate(&e0)); MTRY(cudaEventCreate(&e1));
    GemmParams g;
    memset(&g, 0, sizeof(g));
    g.M = m; g.N = n; g.K = k; g.seq_len = 1 << 20; g.err = c->d_err;
    for (int i = 0; i < 3 && !rc; i++) rc = launch_gemm(c->stream, EPI_NULL, a, b, g, c->num_sms);
    if (rc) { cleanup(); return rc; }
    MTRY(cudaEventRecord(e0, c->stream));
    for (int i = 0; i < iters && !rc; i++) rc = launch_gemm(c->stream, EPI_NULL, a, b, g, c->num_sms);
    if (rc) { cleanup(); return rc; }
    MTRY(cudaEventRecord(e1, c->stream));
    MTRY(cudaEventSynchronize(e1));
    float ms = 0;
    MTRY(cudaEventElapsedTime(&ms, e0, e1));
#undef MTRY
    c->launches += iters + 3;
    *tops = 2.0 * m * n * (double)k * iters / (ms * 1e-3) / 1e12;
    cleanup();
    return check_dev_err(c);
}

extern "C" int egg_set_fused_epilogues(egg_ctx *c, int enable) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    c->fused_level = enable <= 0 ? 0 : (enable >= 3 ? 3 : enable);
    return EGG_OK;
}

extern "C" int egg_fused_epilogues_active(egg_ctx *c) { return (c && use_fused(c)) ? c->fused_level : 0; }

extern "C" int egg_set_attention_tensor_core(egg_ctx *c, int enable) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    if (enable && !attention_tc_supported(c->cfg.seq_len, c->cfg.head_dim)) {
        set_error("tensor-core attention needs seq_len %% 128 == 0, seq_len <= 512 and head_dim 64");
        return EGG_E_INVALID;
    }
    c->attention_mode = enable < 0 ? 0 : (enable > 2 ? 2 : enable);
    return EGG_OK;
}

extern "C" int egg_get_config(egg_ctx *c, egg_config *out) {
    if (!c || !out) { set_error("null argument"); return EGG_E_INVALID; }
    *out = c->cfg;
    return EGG_OK;
}

extern "C" int64_t egg_launch_count(egg_ctx *c) { return c ? c->launches : 0; }
extern "C" int egg_wave_members(egg_ctx *c) { return c ? c->wave_members : 0; }
