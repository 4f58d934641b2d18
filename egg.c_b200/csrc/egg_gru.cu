// The reference's recurrent model (full_trained_egg.c: GRU + MLP blocks, sequential xorshift noise,
// vote-threshold update) on the GPU.  The reference runs one population member at a time through the
// whole sequence on one CPU core; here every token step is batched over the population: the six
// perturbed matrix products of a layer become [population x K] x [K x N] int8 contractions on the
// tensor cores (mma.sync m16n8k32, exact int32 accumulation; the contraction split over the warps of a block
// because the population is only a few hundred rows), with the member's rank-1 term, the
// shift/clip and the GRU gate arithmetic fused behind them.  The recurrence over tokens is inherently
// serial: a generation is seq_len dependent steps of 6*layers+3 small kernels, replayed from a CUDA graph.
#include <math.h>
#include <string.h>

#include <vector>

#include "egg_common.cuh"

namespace egg {

// ------------------------------------------------------------------ layout (EggModel, full_trained_egg.c:42-50)
struct GruLayout { int64_t embedding, gru_w, gru_b, mlp_w, head, ln_w, ln_out, total; };
static GruLayout gru_layout(const egg_gru_config &c) {
    GruLayout L; int64_t H = c.hidden_dim, V = c.vocab_size, NL = c.n_layers, o = 0;
    L.embedding = o; o += V * H;
    L.gru_w = o;     o += NL * 4 * H * H;
    L.gru_b = o;     o += NL * 2 * H;
    L.mlp_w = o;     o += NL * 8 * H * H;
    L.head = o;      o += H * V;
    L.ln_w = o;      o += NL * 2 * H;
    L.ln_out = o;    o += H;
    L.total = o;
    return L;
}

// One noise stream = one perturbed matrix: A (rows = outputs) then B (cols = inputs) from xorshift32 seeded
// with step_seed + pair + seed_off (full_trained_egg.c:118-120, 242, 548).
struct GruStream { int rows, cols, seed_off; int64_t a_off, b_off; };   // offsets into the noise buffer: [pair][rows], [pair][cols]

__device__ __forceinline__ uint32_t xorshift32(uint32_t &x) { x ^= x << 13; x ^= x >> 17; x ^= x << 5; return x; }
__device__ __forceinline__ int gru_clip(int v) { return v > 127 ? 127 : (v < -127 ? -127 : v); }

// gen_noise_vector_neon (full_trained_egg.c:88-104): four draws are discarded before every 16 values.
__device__ void gru_noise_vector(uint32_t &rng, int8_t *out, int count) {
    for (int i = 0; i < count; i += 16) {
        xorshift32(rng); xorshift32(rng); xorshift32(rng); xorshift32(rng);
        for (int j = i; j < i + 16 && j < count; j++) {
            const uint32_t r = xorshift32(rng);
            const int mag = (int)((r >> 1) & 31u);
            out[j] = (int8_t)((r & 1u) ? mag : -mag);
        }
    }
}

// one thread per (stream, pair): the streams are sequential by construction
__global__ void gru_noise_kernel(const GruStream *streams, int nstreams, int pairs, uint32_t step_seed, int8_t *noise) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nstreams * pairs) return;
    const GruStream s = streams[i / pairs];
    const int p = i % pairs;
    uint32_t rng = step_seed + (uint32_t)p + (uint32_t)s.seed_off;
    gru_noise_vector(rng, noise + s.a_off + (int64_t)p * s.rows, s.rows);
    gru_noise_vector(rng, noise + s.b_off + (int64_t)p * s.cols, s.cols);
}

// stream position of pair p (full_trained_egg.c:545-546)
__device__ __forceinline__ int64_t gru_pos(int64_t start_idx, int p, int64_t data_len, int pairs, int seq_len) {
    return (start_idx + (int64_t)p * (data_len / pairs)) % (data_len - seq_len);
}

// ------------------------------------------------------------------ egg_ln (+ embedding gather), one warp per member
struct GruLnParams {
    int pop, H;
    const int8_t *x_in;          // [pop][H] or null: gather from the embedding
    const int8_t *embedding;     // [V][H]
    const uint8_t *data; int64_t data_len; const long long *start_idx; int seq_len; const int *t;
    int8_t *x_out;               // gather only: the residual stream starts as the embedding row
    const int8_t *w;             // [H]
    int8_t *xn;                  // [pop][H]
};

__global__ void __launch_bounds__(128) gru_ln_kernel(const GruLnParams p) {
    const int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (m >= p.pop) return;
    const int8_t *src;
    if (p.x_in) src = p.x_in + (int64_t)m * p.H;
    else {
        const int tok = p.data[gru_pos(*p.start_idx, m >> 1, p.data_len, p.pop / 2, p.seq_len) + *p.t];
        src = p.embedding + (int64_t)tok * p.H;
    }
    int sum = 0;
    for (int d = lane * 4; d < p.H; d += 128) {
        const int32_t v = *reinterpret_cast<const int32_t *>(src + d);
        sum = __dp4a((int)__vabsss4((unsigned)v), 0x01010101, sum);
        if (!p.x_in) *reinterpret_cast<int32_t *>(p.x_out + (int64_t)m * p.H + d) = v;
    }
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    if (sum == 0) sum = 1;                               // full_trained_egg.c:199-201
    int mean = sum / p.H;
    if (mean == 0) mean = 1;
    // (x * w) / mean truncates toward zero; |x * w| < 2^15 and mean <= 127, so |a| / mean == (|a| * M) >> 22 with
    // M = floor(2^22 / mean) + 1 exactly (the error term |a| * (M * mean - 2^22) stays below 2^22)
    const int M = (1 << 22) / mean + 1;
    for (int d = lane * 4; d < p.H; d += 128) {
        const int32_t v = *reinterpret_cast<const int32_t *>(src + d);
        const int32_t w = *reinterpret_cast<const int32_t *>(p.w + d);
        uint32_t o = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int a = (int)(int8_t)(v >> (8 * i)) * (int)(int8_t)(w >> (8 * i));
            const int qa = (abs(a) * M) >> 22;
            const int val = a < 0 ? -qa : qa;
            o |= (uint32_t)(gru_clip(val) & 0xFF) << (8 * i);
        }
        *reinterpret_cast<uint32_t *>(p.xn + (int64_t)m * p.H + d) = o;
    }
}

// ------------------------------------------------------------------ perturbed matrix products (matmul_perturbed, :108-177)
enum { GRU_FT = 0, GRU_HT = 1, GRU_EXP = 2, GRU_PROJ = 3, GRU_HEAD = 4 };

struct GruOperand {
    const int8_t *x; int64_t x_stride;     // input rows: x[m * x_stride + k]
    const int8_t *w;                       // [N][K] row-major (the reference's w[r * cols + c])
    const int8_t *na, *nb;                 // noise: A [pairs][N], B [pairs][K]
};

struct GruMmParams {
    int pop, N, K, shift, rank1_shift;
    GruOperand op[2];
    const int8_t *bias;                    // [N] (FT, HT)
    int8_t *state; int64_t state_stride;   // h of this layer: state[m * state_stride + n] (FT reads, HT updates)
    int8_t *ft, *gp;                       // [pop][N]
    int8_t *x;                             // [pop][N] residual stream (HT, PROJ: read-modify-write)
    int8_t *out;                           // [pop][N] (EXP, HEAD)
};

__device__ __forceinline__ void gru_mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int GRU_BN = 32;      // outputs per block
constexpr int GRU_BM = 32;      // members per block
// Block = KS warps, all on the same 32 members x 32 outputs, each over its own K / KS slice of the contraction
// (the population is small, so parallelism has to come from the contraction: 4 warps for K = H, 8 for K = 4H).
// A warp's fragment loop also carries xB = x·B_pair: the B vectors of the block's 16 pairs are two more
// 8-column operand tiles, and member row r needs only column r/2 of them, which lies in tile mt for both
// 16-row tiles — one extra MMA per 16 rows and k-step, no reduction loop.
// The partial accumulators meet in shared memory; warp w < 4 then owns the 8-output tile nt = w and returns
//   r[mt][e] = clip((x·w[n] + ((xB * A[n] * sign) >> rank1_shift)) >> shift)
// for member = m0 + 16*mt + g + 8*(e>>1), output = n0 + 8*w + 2*q + (e&1).
template <int KS>
__device__ __forceinline__ void gru_product(const GruMmParams &p, const GruOperand &op, int m0, int n0, int warp, int lane,
                                            int (*red)[40][32], int (&r)[2][4]) {
    const int g = lane >> 2, q = lane & 3;
    const int K = p.K, ksl = K / KS, kb = warp * ksl;
    int acc[2][4][4], xacc[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; mt++) {
        xacc[mt][0] = xacc[mt][1] = xacc[mt][2] = xacc[mt][3] = 0;
#pragma unroll
        for (int nt = 0; nt < 4; nt++) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0;
    }
    const int8_t *xa = op.x + (int64_t)(m0 + g) * op.x_stride + 4 * q + kb;
    const int8_t *wb = op.w + (int64_t)(n0 + g) * K + 4 * q + kb;
    const int8_t *nbp = op.nb + (int64_t)((m0 >> 1) + g) * K + 4 * q + kb;     // B of pair (m0/2 + 8*mt + g)
#pragma unroll 4
    for (int k0 = 0; k0 < ksl; k0 += 32) {
        uint32_t a[2][4], b[4][2], bn[2][2];
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            const int8_t *xp = xa + (int64_t)(16 * mt) * op.x_stride + k0;
            a[mt][0] = *reinterpret_cast<const uint32_t *>(xp);
            a[mt][1] = *reinterpret_cast<const uint32_t *>(xp + 8 * op.x_stride);
            a[mt][2] = *reinterpret_cast<const uint32_t *>(xp + 16);
            a[mt][3] = *reinterpret_cast<const uint32_t *>(xp + 8 * op.x_stride + 16);
            const int8_t *np = nbp + (int64_t)(8 * mt) * K + k0;
            bn[mt][0] = __ldg(reinterpret_cast<const uint32_t *>(np));
            bn[mt][1] = __ldg(reinterpret_cast<const uint32_t *>(np + 16));
        }
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            const int8_t *wp = wb + (int64_t)(8 * nt) * K + k0;
            b[nt][0] = __ldg(reinterpret_cast<const uint32_t *>(wp));
            b[nt][1] = __ldg(reinterpret_cast<const uint32_t *>(wp + 16));
        }
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
#pragma unroll
            for (int nt = 0; nt < 4; nt++) gru_mma(acc[mt][nt], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b[nt][0], b[nt][1]);
            gru_mma(xacc[mt], a[mt][0], a[mt][1], a[mt][2], a[mt][3], bn[mt][0], bn[mt][1]);
        }
    }
    // partial sums -> shared memory, value index major / lane minor (conflict-free)
#pragma unroll
    for (int mt = 0; mt < 2; mt++) {
#pragma unroll
        for (int nt = 0; nt < 4; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) red[warp][(mt * 4 + nt) * 4 + e][lane] = acc[mt][nt][e];
#pragma unroll
        for (int e = 0; e < 4; e++) red[warp][32 + mt * 4 + e][lane] = xacc[mt][e];
    }
    __syncthreads();
    if (warp < 4) {
        int a8[2][4], x8[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int sa = 0, sx = 0;
#pragma unroll
                for (int w = 0; w < KS; w++) { sa += red[w][(mt * 4 + warp) * 4 + e][lane]; sx += red[w][32 + mt * 4 + e][lane]; }
                a8[mt][e] = sa; x8[mt][e] = sx;
            }
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int e2 = 0; e2 < 2; e2++) {
                const int ml = 16 * mt + g + 8 * e2, m = m0 + ml;
                // column (ml/2 - 8*mt) of the xB tile: held by lane 4*g + (col >> 1), element 2*e2 + (col & 1)
                const int col = (g + 8 * e2) >> 1;
                const int mine = (col & 1) ? x8[mt][2 * e2 + 1] : x8[mt][2 * e2];
                const int xb = __shfl_sync(0xFFFFFFFFu, mine, 4 * g + (col >> 1));
                const int sign = (m & 1) ? -1 : 1;
                const int16_t a2 = *reinterpret_cast<const int16_t *>(op.na + (int64_t)(m >> 1) * p.N + n0 + 8 * warp + 2 * q);
#pragma unroll
                for (int e1 = 0; e1 < 2; e1++) {
                    const int an = (int)(int8_t)(a2 >> (8 * e1));
                    const int v = a8[mt][2 * e2 + e1] + (((xb * an) * sign) >> p.rank1_shift);
                    r[mt][2 * e2 + e1] = gru_clip(v >> p.shift);
                }
            }
    }
    __syncthreads();          // the partial-sum buffer is reused by the next product
}

template <int MODE, int KS>
__global__ void __launch_bounds__(KS * 32) gru_mm_kernel(const GruMmParams p) {
    __shared__ int red[KS][40][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * GRU_BN, m0 = blockIdx.y * GRU_BM;      // population is a multiple of 32
    const int g = lane >> 2, q = lane & 3;
    int r1[2][4], r2[2][4];
    gru_product<KS>(p, p.op[0], m0, n0, warp, lane, red, r1);
    if (MODE == GRU_FT || MODE == GRU_HT) gru_product<KS>(p, p.op[1], m0, n0, warp, lane, red, r2);
    if (warp >= 4) return;
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int e2 = 0; e2 < 2; e2++) {
            const int m = m0 + 16 * mt + g + 8 * e2;
            const int n = n0 + 8 * warp + 2 * q;
            int o0[2], o1[2];
#pragma unroll
            for (int e1 = 0; e1 < 2; e1++) {
                const int v1 = r1[mt][2 * e2 + e1];
                o1[e1] = 0;
                if (MODE == GRU_FT) {
                    // ft = clip(clip(b1 + b2) + bf); gated_past = ((ft + 127) * h) >> 8   (:248-252)
                    const int ft = gru_clip(gru_clip(v1 + r2[mt][2 * e2 + e1]) + (int)p.bias[n + e1]);
                    const int h = p.state[(int64_t)m * p.state_stride + n + e1];
                    o0[e1] = ft; o1[e1] = ((ft + 127) * h) >> 8;
                } else if (MODE == GRU_HT) {
                    // ht = clip(clip(b1 + b2) + bh); h += ((ft + 127) * (ht - h)) >> 8; x = clip(h + residual)   (:257-268)
                    const int ht = gru_clip(gru_clip(v1 + r2[mt][2 * e2 + e1]) + (int)p.bias[n + e1]);
                    const int h = p.state[(int64_t)m * p.state_stride + n + e1];
                    const int ft = p.ft[(int64_t)m * p.N + n + e1];
                    const int hn = gru_clip(h + (((ft + 127) * (ht - h)) >> 8));
                    o0[e1] = hn; o1[e1] = gru_clip(hn + (int)p.x[(int64_t)m * p.N + n + e1]);
                } else if (MODE == GRU_PROJ) {
                    o0[e1] = gru_clip(v1 + (int)p.x[(int64_t)m * p.N + n + e1]);          // :283-285
                } else {
                    o0[e1] = v1;
                }
            }
            const uint16_t w0 = (uint16_t)((o0[0] & 0xFF) | ((o0[1] & 0xFF) << 8));
            const uint16_t w1 = (uint16_t)((o1[0] & 0xFF) | ((o1[1] & 0xFF) << 8));
            if (MODE == GRU_FT) {
                *reinterpret_cast<uint16_t *>(p.ft + (int64_t)m * p.N + n) = w0;
                *reinterpret_cast<uint16_t *>(p.gp + (int64_t)m * p.N + n) = w1;
            } else if (MODE == GRU_HT) {
                *reinterpret_cast<uint16_t *>(p.state + (int64_t)m * p.state_stride + n) = w0;
                *reinterpret_cast<uint16_t *>(p.x + (int64_t)m * p.N + n) = w1;
            } else if (MODE == GRU_PROJ) {
                *reinterpret_cast<uint16_t *>(p.x + (int64_t)m * p.N + n) = w0;
            } else {
                *reinterpret_cast<uint16_t *>(p.out + (int64_t)m * p.N + n) = w0;
            }
        }
}

// ------------------------------------------------------------------ compute_loss (:298-330), one warp per member; last block advances t
struct GruLossParams {
    int pop, V;
    const int8_t *logits; const int32_t *exp2_table;
    const uint8_t *data; int64_t data_len; const long long *start_idx; int seq_len; int *t;
    int32_t *loss;
};

__global__ void __launch_bounds__(256) gru_loss_kernel(const GruLossParams p) {
    const int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (m >= p.pop) return;
    const int8_t *lg = p.logits + (int64_t)m * p.V;
    int sum = 0;
    for (int i = lane; i < p.V; i += 32) sum += p.exp2_table[(int)lg[i] + 128];
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    if (lane == 0) {
        int log_sum = 0;
        if (sum > 0) {                                          // log2_fixed, :311-321
            const int k = 31 - __clz(sum);
            const int frac = k >= 4 ? (sum - (1 << k)) >> (k - 4) : (sum - (1 << k)) << (4 - k);
            log_sum = (k << 4) + frac - 64;
        }
        const int target = p.data[gru_pos(*p.start_idx, m >> 1, p.data_len, p.pop / 2, p.seq_len) + *p.t + 1];
        p.loss[m] += log_sum - ((int)lg[target] + 128);
    }
}
__global__ void gru_advance_kernel(int *t) { *t += 1; }

__global__ void gru_fitness_kernel(const int32_t *loss, int32_t *fit, int pairs) {   // :558-560
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pairs) return;
    const int a = loss[2 * i], b = loss[2 * i + 1];
    fit[i] = a < b ? 1 : (b < a ? -1 : 0);
}

// ------------------------------------------------------------------ update_matrix (:332-409)
// vote[r][c] = Σ_p (int8)(A_p[r] * f_p) * B_p[c]; w += 1 above the threshold, -= 1 below minus the threshold.
// Block: 32 outputs x 32 inputs; A*f and B of every pair for the tile are staged in shared memory.
__global__ void __launch_bounds__(256) gru_update_kernel(int8_t *W, int rows, int cols, const int8_t *na, const int8_t *nb,
                                                         const int32_t *fit, int pairs, int threshold) {
    extern __shared__ int8_t s_upd[];
    int8_t *sa = s_upd, *sb = s_upd + pairs * 32;
    const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
    for (int i = threadIdx.x; i < pairs * 32; i += 256) {
        const int pp = i >> 5, j = i & 31;
        const int f = fit[pp];
        sa[i] = (int8_t)((int)na[(int64_t)pp * rows + r0 + j] * f);
        sb[i] = nb[(int64_t)pp * cols + c0 + j];
    }
    __syncthreads();
    const int c = threadIdx.x & 31;
    for (int rr = threadIdx.x >> 5; rr < 32; rr += 8) {
        int vote = 0;
        for (int pp = 0; pp < pairs; pp++) vote += (int)sa[pp * 32 + rr] * (int)sb[pp * 32 + c];
        int8_t *w = W + (int64_t)(r0 + rr) * cols + c0 + c;
        const int wv = *w;
        if (vote > threshold && wv < 127) *w = (int8_t)(wv + 1);
        else if (vote < -threshold && wv > -127) *w = (int8_t)(wv - 1);
    }
}

}  // namespace egg

// =========================================================================== C ABI
using namespace egg;

struct egg_gru_ctx {
    egg_gru_config cfg;
    int device = 0;
    cudaStream_t stream = nullptr;
    GruLayout L;
    int8_t *d_model = nullptr, *d_states = nullptr, *d_noise = nullptr;
    uint8_t *d_data = nullptr; int64_t data_len = 0;
    std::vector<GruStream> streams;
    GruStream *d_streams = nullptr;
    int8_t *d_x = nullptr, *d_xn = nullptr, *d_ft = nullptr, *d_gp = nullptr, *d_buf = nullptr, *d_logits = nullptr;
    int32_t *d_loss = nullptr, *d_fit = nullptr, *d_exp2 = nullptr;
    int *d_t = nullptr;                 // [0]: token index inside the generation; bytes 8..15: start index (int64)
    // token-step graphs: everything that changes between generations is read from device memory
    cudaGraphExec_t graph1 = nullptr, graph16 = nullptr;
    int64_t launches = 0;
    bool have_model = false;
};

extern "C" void egg_gru_config_defaults(egg_gru_config *c) {
    if (!c) return;
    c->hidden_dim = 512; c->n_layers = 4; c->vocab_size = 256; c->seq_len = 4096; c->population_size = 128;
    c->fixed_point = 4; c->sigma_shift = 4; c->update_threshold = 160;
}

static int gru_validate(const egg_gru_config *c) {
    if (!c) { set_error("null configuration"); return EGG_E_INVALID; }
    if (c->hidden_dim < 128 || c->hidden_dim > 1024 || c->hidden_dim % 128) { set_error("hidden_dim must be a multiple of 128 up to 1024"); return EGG_E_INVALID; }
    if (c->vocab_size != 256) { set_error("vocab_size must be 256"); return EGG_E_INVALID; }
    if (c->n_layers < 1 || c->n_layers > 64) { set_error("n_layers out of range"); return EGG_E_INVALID; }
    if (c->population_size < 32 || c->population_size > 1024 || c->population_size % 32) { set_error("population_size must be a multiple of 32 up to 1024"); return EGG_E_INVALID; }
    if (c->seq_len < 1) { set_error("seq_len must be positive"); return EGG_E_INVALID; }
    if (c->fixed_point < 0 || c->sigma_shift < 0 || c->fixed_point + c->sigma_shift > 24) { set_error("shift out of range"); return EGG_E_INVALID; }
    return EGG_OK;
}

extern "C" int64_t egg_gru_model_bytes(const egg_gru_config *c) { return c ? gru_layout(*c).total : 0; }
extern "C" int64_t egg_gru_state_bytes(const egg_gru_config *c) { return c ? (int64_t)c->population_size * c->n_layers * c->hidden_dim : 0; }

static void gru_drop_graphs(egg_gru_ctx *c) {
    if (c->graph1) { cudaGraphExecDestroy(c->graph1); c->graph1 = nullptr; }
    if (c->graph16) { cudaGraphExecDestroy(c->graph16); c->graph16 = nullptr; }
}

extern "C" void egg_gru_destroy(egg_gru_ctx *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    gru_drop_graphs(c);
    void *ptrs[] = {c->d_model, c->d_states, c->d_noise, c->d_data, c->d_streams, c->d_x, c->d_xn, c->d_ft, c->d_gp, c->d_buf,
                    c->d_logits, c->d_loss, c->d_fit, c->d_exp2, c->d_t};
    for (void *p : ptrs) if (p) cudaFree(p);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

extern "C" int egg_gru_create(const egg_gru_config *cfg, int device, egg_gru_ctx **out) {
    if (!out) { set_error("null argument"); return EGG_E_INVALID; }
    *out = nullptr;
    int rc = gru_validate(cfg);
    if (rc) return rc;
    int ndev = 0;
    EGG_CUDA(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev) { set_error("device %d not present (%d devices)", device, ndev); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    EGG_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) { set_error("this library is built for sm_100a only (device is sm_%d%d)", prop.major, prop.minor); return EGG_E_INVALID; }
    egg_gru_ctx *c = new egg_gru_ctx();
    c->cfg = *cfg; c->device = device; c->L = gru_layout(*cfg);
    const int64_t H = cfg->hidden_dim, V = cfg->vocab_size, POP = cfg->population_size, pairs = POP / 2;
    // noise streams in the order of the forward pass: per layer seeds l*100 + 1..6, head 999 (:242, 292)
    int64_t noff = 0;
    auto add = [&](int rows, int cols, int seed_off) {
        GruStream s; s.rows = rows; s.cols = cols; s.seed_off = seed_off;
        s.a_off = noff; noff += pairs * rows; s.b_off = noff; noff += pairs * cols;
        noff = (noff + 15) & ~(int64_t)15;
        c->streams.push_back(s);
    };
    for (int l = 0; l < cfg->n_layers; l++) {
        for (int k = 1; k <= 4; k++) add((int)H, (int)H, l * 100 + k);
        add((int)(4 * H), (int)H, l * 100 + 5);
        add((int)H, (int)(4 * H), l * 100 + 6);
    }
    add((int)V, (int)H, 999);
#define GTRY(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { set_error("%s: %s", #x, cudaGetErrorString(e_)); egg_gru_destroy(c); return EGG_E_CUDA; } } while (0)
    GTRY(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    GTRY(cudaMalloc(&c->d_model, (size_t)c->L.total));
    GTRY(cudaMalloc(&c->d_states, (size_t)(POP * cfg->n_layers * H)));
    GTRY(cudaMemset(c->d_states, 0, (size_t)(POP * cfg->n_layers * H)));
    GTRY(cudaMalloc(&c->d_noise, (size_t)noff));
    GTRY(cudaMalloc(&c->d_streams, c->streams.size() * sizeof(GruStream)));
    GTRY(cudaMemcpy(c->d_streams, c->streams.data(), c->streams.size() * sizeof(GruStream), cudaMemcpyHostToDevice));
    GTRY(cudaMalloc(&c->d_x, (size_t)(POP * H))); GTRY(cudaMalloc(&c->d_xn, (size_t)(POP * H)));
    GTRY(cudaMalloc(&c->d_ft, (size_t)(POP * H))); GTRY(cudaMalloc(&c->d_gp, (size_t)(POP * H)));
    GTRY(cudaMalloc(&c->d_buf, (size_t)(POP * 4 * H))); GTRY(cudaMalloc(&c->d_logits, (size_t)(POP * V)));
    GTRY(cudaMalloc(&c->d_loss, (size_t)POP * 4)); GTRY(cudaMalloc(&c->d_fit, (size_t)pairs * 4));
    GTRY(cudaMalloc(&c->d_exp2, 256 * 4)); GTRY(cudaMalloc(&c->d_t, 16));
    {
        int32_t tab[256];                                                      // init_tables, :58-61
        for (int i = 0; i < 256; i++) tab[i] = (int32_t)(pow(2.0, (double)i / (1 << cfg->fixed_point)) * (1 << cfg->fixed_point));
        GTRY(cudaMemcpy(c->d_exp2, tab, sizeof(tab), cudaMemcpyHostToDevice));
    }
#undef GTRY
    *out = c;
    return EGG_OK;
}

static int gru_copy(egg_gru_ctx *c, void *dst, const void *src, int64_t nbytes, int64_t want, cudaMemcpyKind kind, const char *what) {
    if (!c || !dst || !src) { set_error("null argument"); return EGG_E_INVALID; }
    if (nbytes != want) { set_error("%s is %lld bytes, this configuration needs %lld", what, (long long)nbytes, (long long)want); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaMemcpyAsync(dst, src, (size_t)nbytes, kind, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    return EGG_OK;
}
extern "C" int egg_gru_upload_model(egg_gru_ctx *c, const void *h, int64_t n) {
    int rc = gru_copy(c, c ? c->d_model : nullptr, h, n, c ? c->L.total : 0, cudaMemcpyHostToDevice, "model");
    if (!rc) c->have_model = true;
    return rc;
}
extern "C" int egg_gru_download_model(egg_gru_ctx *c, void *h, int64_t n) {
    return gru_copy(c, h, c ? c->d_model : nullptr, n, c ? c->L.total : 0, cudaMemcpyDeviceToHost, "model");
}
extern "C" int egg_gru_upload_states(egg_gru_ctx *c, const void *h, int64_t n) {
    return gru_copy(c, c ? c->d_states : nullptr, h, n, c ? egg_gru_state_bytes(&c->cfg) : 0, cudaMemcpyHostToDevice, "recurrent state");
}
extern "C" int egg_gru_download_states(egg_gru_ctx *c, void *h, int64_t n) {
    return gru_copy(c, h, c ? c->d_states : nullptr, n, c ? egg_gru_state_bytes(&c->cfg) : 0, cudaMemcpyDeviceToHost, "recurrent state");
}

extern "C" int egg_gru_set_dataset(egg_gru_ctx *c, const uint8_t *host_tokens, int64_t n) {
    if (!c || !host_tokens) { set_error("null argument"); return EGG_E_INVALID; }
    if (n <= (int64_t)c->cfg.seq_len + 1) { set_error("dataset of %lld bytes is shorter than seq_len + 2", (long long)n); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    gru_drop_graphs(c);
    if (c->d_data) { cudaFree(c->d_data); c->d_data = nullptr; }
    EGG_CUDA(cudaMalloc(&c->d_data, (size_t)n));
    EGG_CUDA(cudaMemcpyAsync(c->d_data, host_tokens, (size_t)n, cudaMemcpyHostToDevice, c->stream));
    EGG_CUDA(cudaStreamSynchronize(c->stream));
    c->data_len = n;
    return EGG_OK;
}

// the kernels of one token step (forward_pass body, :233-295), enqueued on the context stream; returns launches
static int gru_token_step(egg_gru_ctx *c, int *nlaunch) {
    const long long *start_idx = reinterpret_cast<const long long *>(c->d_t + 2);
    const egg_gru_config &cf = c->cfg;
    const int H = cf.hidden_dim, V = cf.vocab_size, POP = cf.population_size;
    const GruLayout &L = c->L;
    cudaStream_t st = c->stream;
    const int ln_blocks = (POP + 3) / 4;          // one warp per member, 4 per block: the rows spread over more SMs
    const unsigned mby = (unsigned)(POP / GRU_BM);
    int n = 0;
    auto operand = [&](const int8_t *x, int64_t xs, const int8_t *w, const GruStream &s) {
        GruOperand o; o.x = x; o.x_stride = xs; o.w = w; o.na = c->d_noise + s.a_off; o.nb = c->d_noise + s.b_off; return o;
    };
    auto base = [&](int N, int K, int shift) {
        GruMmParams p; memset(&p, 0, sizeof(p));
        p.pop = POP; p.N = N; p.K = K; p.shift = shift; p.rank1_shift = cf.fixed_point + cf.sigma_shift;
        return p;
    };
    for (int l = 0; l < cf.n_layers; l++) {
        const int8_t *gw = c->d_model + L.gru_w + (int64_t)l * 4 * H * H, *gb = c->d_model + L.gru_b + (int64_t)l * 2 * H;
        const int8_t *mw = c->d_model + L.mlp_w + (int64_t)l * 8 * H * H, *lw = c->d_model + L.ln_w + (int64_t)l * 2 * H;
        const GruStream *S = &c->streams[l * 6];
        int8_t *hl = c->d_states + (int64_t)l * H;
        const int64_t hs = (int64_t)cf.n_layers * H;
        GruLnParams ln; memset(&ln, 0, sizeof(ln));
        ln.pop = POP; ln.H = H; ln.w = lw; ln.xn = c->d_xn;
        if (l == 0) {
            ln.embedding = c->d_model + L.embedding; ln.data = c->d_data; ln.data_len = c->data_len; ln.start_idx = start_idx;
            ln.seq_len = cf.seq_len; ln.t = c->d_t; ln.x_out = c->d_x;
        } else ln.x_in = c->d_x;
        gru_ln_kernel<<<ln_blocks, 128, 0, st>>>(ln); n++;
        GruMmParams ft = base(H, H, 8);
        ft.op[0] = operand(c->d_xn, H, gw, S[0]); ft.op[1] = operand(hl, hs, gw + (int64_t)H * H, S[1]);
        ft.bias = gb; ft.state = hl; ft.state_stride = hs; ft.ft = c->d_ft; ft.gp = c->d_gp;
        gru_mm_kernel<GRU_FT, 4><<<dim3(H / GRU_BN, mby), 128, 0, st>>>(ft); n++;
        GruMmParams ht = base(H, H, 8);
        ht.op[0] = operand(c->d_xn, H, gw + 2 * (int64_t)H * H, S[2]); ht.op[1] = operand(c->d_gp, H, gw + 3 * (int64_t)H * H, S[3]);
        ht.bias = gb + H; ht.state = hl; ht.state_stride = hs; ht.ft = c->d_ft; ht.x = c->d_x;
        gru_mm_kernel<GRU_HT, 4><<<dim3(H / GRU_BN, mby), 128, 0, st>>>(ht); n++;
        GruLnParams ln2; memset(&ln2, 0, sizeof(ln2));
        ln2.pop = POP; ln2.H = H; ln2.w = lw + H; ln2.xn = c->d_xn; ln2.x_in = c->d_x;
        gru_ln_kernel<<<ln_blocks, 128, 0, st>>>(ln2); n++;
        GruMmParams ex = base(4 * H, H, 8);
        ex.op[0] = operand(c->d_xn, H, mw, S[4]); ex.out = c->d_buf;
        gru_mm_kernel<GRU_EXP, 4><<<dim3(4 * H / GRU_BN, mby), 128, 0, st>>>(ex); n++;
        GruMmParams pr = base(H, 4 * H, 9);
        pr.op[0] = operand(c->d_buf, 4 * H, mw + 4 * (int64_t)H * H, S[5]); pr.x = c->d_x;
        gru_mm_kernel<GRU_PROJ, 8><<<dim3(H / GRU_BN, mby), 256, 0, st>>>(pr); n++;
    }
    GruLnParams lf; memset(&lf, 0, sizeof(lf));
    lf.pop = POP; lf.H = H; lf.w = c->d_model + L.ln_out; lf.xn = c->d_xn; lf.x_in = c->d_x;
    gru_ln_kernel<<<ln_blocks, 128, 0, st>>>(lf); n++;
    GruMmParams hd = base(V, H, 8);
    hd.op[0] = operand(c->d_xn, H, c->d_model + L.head, c->streams[cf.n_layers * 6]); hd.out = c->d_logits;
    gru_mm_kernel<GRU_HEAD, 4><<<dim3(V / GRU_BN, mby), 128, 0, st>>>(hd); n++;
    GruLossParams lp; lp.pop = POP; lp.V = V; lp.logits = c->d_logits; lp.exp2_table = c->d_exp2; lp.data = c->d_data;
    lp.data_len = c->data_len; lp.start_idx = start_idx; lp.seq_len = cf.seq_len; lp.t = c->d_t; lp.loss = c->d_loss;
    gru_loss_kernel<<<(POP + 7) / 8, 256, 0, st>>>(lp); n++;
    gru_advance_kernel<<<1, 1, 0, st>>>(c->d_t); n++;
    EGG_CUDA(cudaGetLastError());
    *nlaunch = n;
    return EGG_OK;
}

static int gru_capture(egg_gru_ctx *c, int steps, cudaGraphExec_t *exec, int *per_step) {
    cudaGraph_t graph = nullptr;
    EGG_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    int rc = EGG_OK;
    for (int i = 0; i < steps && !rc; i++) rc = gru_token_step(c, per_step);
    cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (e != cudaSuccess) { set_error("stream capture failed: %s", cudaGetErrorString(e)); return EGG_E_CUDA; }
    e = cudaGraphInstantiate(exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { set_error("graph instantiation failed: %s", cudaGetErrorString(e)); return EGG_E_CUDA; }
    return EGG_OK;
}

extern "C" int egg_gru_generation(egg_gru_ctx *c, uint32_t step_seed, int64_t start_idx, int tokens, int do_update,
                                  int32_t *host_losses, int32_t *host_fitness) {
    if (!c) { set_error("null context"); return EGG_E_INVALID; }
    if (!c->have_model || !c->d_data) { set_error("upload a model and a dataset first"); return EGG_E_STATE; }
    const egg_gru_config &cf = c->cfg;
    if (tokens < 1 || tokens > cf.seq_len || start_idx < 0) { set_error("tokens must be in [1, seq_len] and start_idx >= 0"); return EGG_E_INVALID; }
    EGG_CUDA(cudaSetDevice(c->device));
    const int H = cf.hidden_dim, V = cf.vocab_size, POP = cf.population_size, pairs = POP / 2;
    cudaStream_t st = c->stream;
    const int ns = (int)c->streams.size();
    gru_noise_kernel<<<(ns * pairs + 127) / 128, 128, 0, st>>>(c->d_streams, ns, pairs, step_seed, c->d_noise);
    EGG_CUDA(cudaGetLastError());
    c->launches++;
    EGG_CUDA(cudaMemsetAsync(c->d_loss, 0, (size_t)POP * 4, st));
    const long long hdr[2] = {0, (long long)start_idx};
    EGG_CUDA(cudaMemcpyAsync(c->d_t, hdr, 16, cudaMemcpyHostToDevice, st));
    EGG_CUDA(cudaStreamSynchronize(st));       // hdr lives on this stack frame
    int per_step = 6 * cf.n_layers + 4, rc;
    if (!c->graph1) {
        // both or neither: a lone single-step graph would make the next call skip the capture of the 16-step one
        if ((rc = gru_capture(c, 1, &c->graph1, &per_step)) || (rc = gru_capture(c, 16, &c->graph16, &per_step))) {
            gru_drop_graphs(c);
            return rc;
        }
    }
    int t = 0;
    for (; t + 16 <= tokens; t += 16) EGG_CUDA(cudaGraphLaunch(c->graph16, st));
    for (; t < tokens; t++) EGG_CUDA(cudaGraphLaunch(c->graph1, st));
    c->launches += (int64_t)per_step * tokens;
    gru_fitness_kernel<<<(pairs + 127) / 128, 128, 0, st>>>(c->d_loss, c->d_fit, pairs);
    c->launches++;
    if (do_update) {
        const GruLayout &L = c->L;
        auto upd = [&](int8_t *W, int rows, int cols, const GruStream &s) {
            gru_update_kernel<<<dim3(cols / 32, rows / 32), 256, (size_t)pairs * 64, st>>>(W, rows, cols, c->d_noise + s.a_off,
                                                                                       c->d_noise + s.b_off, c->d_fit, pairs, cf.update_threshold);
            c->launches++;
        };
        for (int l = 0; l < cf.n_layers; l++) {
            int8_t *gw = c->d_model + L.gru_w + (int64_t)l * 4 * H * H, *mw = c->d_model + L.mlp_w + (int64_t)l * 8 * H * H;
            for (int g = 0; g < 4; g++) upd(gw + (int64_t)g * H * H, H, H, c->streams[l * 6 + g]);
            upd(mw, 4 * H, H, c->streams[l * 6 + 4]);
            upd(mw + 4 * (int64_t)H * H, H, 4 * H, c->streams[l * 6 + 5]);
        }
        upd(c->d_model + L.head, V, H, c->streams[cf.n_layers * 6]);
    }
    EGG_CUDA(cudaGetLastError());
    if (host_losses) EGG_CUDA(cudaMemcpyAsync(host_losses, c->d_loss, (size_t)POP * 4, cudaMemcpyDeviceToHost, st));
    if (host_fitness) EGG_CUDA(cudaMemcpyAsync(host_fitness, c->d_fit, (size_t)pairs * 4, cudaMemcpyDeviceToHost, st));
    EGG_CUDA(cudaStreamSynchronize(st));
    return EGG_OK;
}

extern "C" int64_t egg_gru_launch_count(egg_gru_ctx *c) { return c ? c->launches : 0; }
