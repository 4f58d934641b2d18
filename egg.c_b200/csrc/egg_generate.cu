// Sampling: one un-perturbed stream decoded token by token with a KV cache
// (generate_sequence_kernel, d-eggs/src/kernels.cu:307-490; mgpu.cu:1154-1285 is the case temp = 1,
// no min-p filter, no presence penalty).  Inherently serial over tokens and a single row wide, so it is one
// thread block walking the layers with block-wide reductions; matrix-vector products read the reference's
// packed [K/4][N][4] weights (one coalesced 32-bit word per thread and k-quad, dp4a), with the contraction
// split over thread groups where a product has fewer outputs than the block has threads.
#include "egg_kernels.cuh"

#include <limits.h>

namespace egg {

constexpr int GEN_THREADS = 1024;

struct GenSmem {
    int8_t x[1024], h[1024], u[4096], q8[1024], ao[1024];
    int32_t pre[3 * 1024];                 // pre-activations (q | k | v for the attention block)
    int32_t part[GEN_THREADS];             // split-k partial sums
    int32_t sc[16 * 256];                  // scores, then softmax weights: [head][ctx]
    int32_t red[64];
    long long red64[32];
    int32_t lg[256], ex[256];
    int8_t act_lut[256];
    int32_t exp_lut[256];
};

__device__ __forceinline__ int gen_block_sum(GenSmem &s, int v) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s.red[threadIdx.x >> 5] = v;
    __syncthreads();
    int t = 0;
    for (int i = 0; i < GEN_THREADS / 32; i++) t += s.red[i];
    return t;
}
__device__ __forceinline__ int gen_block_max(GenSmem &s, int v) {
    for (int off = 16; off > 0; off >>= 1) v = max(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s.red[threadIdx.x >> 5] = v;
    __syncthreads();
    int t = INT_MIN;
    for (int i = 0; i < GEN_THREADS / 32; i++) t = max(t, s.red[i]);
    return t;
}

// out[n] = Σ_k in[k] * W[k][n] for n < N, W packed [K/4][N][4]; result left in s.pre[out_off + n].
// Threads are split into GEN_THREADS / N' groups over k when N is small (N' = N rounded to the block).
__device__ void gen_matvec(GenSmem &s, const int8_t *in, const int8_t *w_packed, int K, int N, int out_off) {
    const int32_t *w32 = reinterpret_cast<const int32_t *>(w_packed);
    const int32_t *in32 = reinterpret_cast<const int32_t *>(in);
    const int kq = K >> 2;
    if (N >= GEN_THREADS) {
        for (int n = threadIdx.x; n < N; n += GEN_THREADS) {
            int acc = 0;
            for (int k = 0; k < kq; k++) acc = __dp4a(in32[k], __ldg(w32 + (int64_t)k * N + n), acc);
            s.pre[out_off + n] = acc;
        }
        __syncthreads();
        return;
    }
    const int groups = GEN_THREADS / N;            // N is a multiple of 128 (or 256): divides 1024
    const int n = threadIdx.x % N, gidx = threadIdx.x / N;
    const int per = (kq + groups - 1) / groups;
    int acc = 0;
    for (int k = gidx * per; k < min(kq, (gidx + 1) * per); k++) acc = __dp4a(in32[k], __ldg(w32 + (int64_t)k * N + n), acc);
    s.part[threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.x < N) {
        int t = 0;
        for (int g2 = 0; g2 < groups; g2++) t += s.part[g2 * N + threadIdx.x];
        s.pre[out_off + threadIdx.x] = t;
    }
    __syncthreads();
}

// apply_standard_norm without noise (mgpu.cu:646-678, ns = 0): out = clip((x * w) / mean|x| + b)
__device__ void gen_norm(GenSmem &s, const int8_t *x, int8_t *out, const int8_t *w, const int8_t *b, int H) {
    int a = 0;
    for (int d = threadIdx.x; d < H; d += GEN_THREADS) a += abs((int)x[d]);
    int mn = gen_block_sum(s, a) / H;
    if (!mn) mn = 1;
    for (int d = threadIdx.x; d < H; d += GEN_THREADS) out[d] = (int8_t)clip8(((int)x[d] * (int)w[d]) / mn + (int)b[d]);
    __syncthreads();
}

// adaptive_layer_normalize / adaptive_qkv_normalize (egg_adaptive_normalize.h:10-103) of n values in s.pre[off..]
__device__ void gen_adaptive(GenSmem &s, int off, int8_t *out, int n) {
    int m = 0;
    for (int d = threadIdx.x; d < n; d += GEN_THREADS) m = max(m, abs(s.pre[off + d]));
    m = gen_block_max(s, m);
    const float scale = 127.0f / (float)((float)m + 1e-9f);
    for (int d = threadIdx.x; d < n; d += GEN_THREADS) {
        int q = (int)roundf(__fmul_rn((float)s.pre[off + d], scale));
        out[d] = (int8_t)max(-127, min(127, q));
    }
    __syncthreads();
}

// compute_mlp without noise (mgpu.cu:708-759)
__device__ void gen_mlp(GenSmem &s, const GenParams &p, const int8_t *ln_w, const int8_t *ln_b, const int8_t *up_w, const int8_t *up_b,
                        const int8_t *dn_w, const int8_t *dn_b) {
    const int H = p.H;
    gen_norm(s, s.x, s.h, ln_w, ln_b, H);
    {
        const int32_t *w32 = reinterpret_cast<const int32_t *>(up_w);
        const int32_t *in32 = reinterpret_cast<const int32_t *>(s.h);
        for (int n = threadIdx.x; n < 4 * H; n += GEN_THREADS) {
            int acc = 0;
            for (int k = 0; k < (H >> 2); k++) acc = __dp4a(in32[k], __ldg(w32 + (int64_t)k * 4 * H + n), acc);
            s.u[n] = s.act_lut[(uint8_t)(int8_t)clip8((acc >> p.shift_mlp_up) + (int)up_b[n])];
        }
    }
    __syncthreads();
    gen_matvec(s, s.u, dn_w, 4 * H, H, 0);
    for (int d = threadIdx.x; d < H; d += GEN_THREADS) s.pre[d] = (int)s.x[d] + (s.pre[d] >> p.shift_mlp_down) + (int)dn_b[d];
    __syncthreads();
    gen_adaptive(s, 0, s.x, H);
}

__global__ void __launch_bounds__(GEN_THREADS, 1) generate_kernel(const GenParams p) {
    extern __shared__ __align__(16) uint8_t gen_raw[];
    GenSmem &s = *reinterpret_cast<GenSmem *>(gen_raw);
    const int H = p.H, V = p.V, HD = p.head_dim, NH = H / HD;
    const int total = p.seed_len + p.gen_len;
    const int8_t *M = p.model;
    const ModelLayout &L = p.L;
    for (int i = threadIdx.x; i < 256; i += GEN_THREADS) { s.act_lut[i] = p.act_lut[i]; s.exp_lut[i] = p.exp_lut[i]; }
    __syncthreads();

    for (int t = 0; t < total - 1; t++) {
        const int tok = p.tokens[t];
        for (int d = threadIdx.x; d < H; d += GEN_THREADS)
            s.x[d] = (int8_t)clip8((int)M[L.embedding + ((int64_t)(d >> 2) * V + tok) * 4 + (d & 3)] + (int)M[L.emb_bias + d]);
        __syncthreads();
        gen_mlp(s, p, M + L.ln_init, M + L.ln_init_bias, M + L.w_emb_mlp_up, M + L.mlp_emb_bias_up, M + L.w_emb_mlp_down, M + L.mlp_emb_bias_down);

        for (int l = 0; l < p.n_layers; l++) {
            const int64_t lH = (int64_t)l * H, lHH = (int64_t)l * H * H;
            int8_t *kc = p.kv + (int64_t)l * 2 * total * H, *vc = kc + (int64_t)total * H;
            gen_norm(s, s.x, s.h, M + L.ln_1 + lH, M + L.ln_1_bias + lH, H);
            gen_matvec(s, s.h, M + L.w_q + lHH, H, H, 0);
            gen_matvec(s, s.h, M + L.w_k + lHH, H, H, H);
            gen_matvec(s, s.h, M + L.w_v + lHH, H, H, 2 * H);
            // integer RoPE on q and k (apply_rope_integer, mgpu.cu:624-644)
            for (int i = threadIdx.x; i < H; i += GEN_THREADS) {      // i = pair index over q (H/2 pairs) then k
                const int which = i / (H / 2), pr = i % (H / 2), d = 2 * pr;
                const int32_t c = p.rope_lut[t * HD + (d % HD)], sn = p.rope_lut[t * HD + (d % HD) + 1];
                const long long ev = s.pre[which * H + d], od = s.pre[which * H + d + 1];
                const long long half_ulp = 1ll << (p.rope_bit - 1);
                s.pre[which * H + d] = (int)((ev * c - od * sn + half_ulp) >> p.rope_bit);
                s.pre[which * H + d + 1] = (int)((ev * sn + od * c + half_ulp) >> p.rope_bit);
            }
            __syncthreads();
            gen_adaptive(s, 0, s.q8, H);
            gen_adaptive(s, H, kc + (int64_t)t * H, H);
            gen_adaptive(s, 2 * H, vc + (int64_t)t * H, H);
            __threadfence_block();
            __syncthreads();
            // pass 1: scores and the per-head maximum over ctx <= t (mgpu.cu:795-802)
            for (int i = threadIdx.x; i < NH * (t + 1); i += GEN_THREADS) {
                const int hd = i / (t + 1), ctx = i % (t + 1);
                const int32_t *q32 = reinterpret_cast<const int32_t *>(s.q8 + hd * HD);
                const int32_t *k32 = reinterpret_cast<const int32_t *>(kc + (int64_t)ctx * H + hd * HD);
                int acc = 0;
                for (int j = 0; j < HD / 4; j++) acc = __dp4a(q32[j], k32[j], acc);
                s.sc[hd * 256 + ctx] = acc;
            }
            __syncthreads();
            if (threadIdx.x < NH) {                                   // head maxima, then weights (mgpu.cu:810-815)
                int mx = INT_MIN;
                for (int ctx = 0; ctx <= t; ctx++) mx = max(mx, s.sc[threadIdx.x * 256 + ctx]);
                s.red[32 + threadIdx.x] = mx;
            }
            __syncthreads();
            for (int i = threadIdx.x; i < NH * (t + 1); i += GEN_THREADS) {
                const int hd = i / (t + 1), ctx = i % (t + 1);
                int idx = (s.red[32 + hd] >> p.shift_attn) - (s.sc[hd * 256 + ctx] >> p.shift_attn);
                idx = idx < 0 ? 0 : (idx > 255 ? 255 : idx);
                s.sc[hd * 256 + ctx] = s.exp_lut[idx];
            }
            __syncthreads();
            // pass 2: Σ w·v in 64 bits and the truncating division (mgpu.cu:816-824)
            for (int d = threadIdx.x; d < H; d += GEN_THREADS) {
                const int hd = d / HD;
                long long wv = 0; unsigned long long tot = 0;
                for (int ctx = 0; ctx <= t; ctx++) {
                    const int w = s.sc[hd * 256 + ctx];
                    wv += (long long)w * (long long)vc[(int64_t)ctx * H + d];
                    tot += (unsigned long long)w;
                }
                s.ao[d] = (int8_t)clip8((int)(wv / (tot ? (long long)tot : 1)));
            }
            __syncthreads();
            gen_matvec(s, s.ao, M + L.w_o + lHH, H, H, 0);
            for (int d = threadIdx.x; d < H; d += GEN_THREADS) s.pre[d] = (int)s.x[d] + (s.pre[d] >> p.shift_out);
            __syncthreads();
            gen_adaptive(s, 0, s.x, H);
            gen_mlp(s, p, M + L.ln_2 + lH, M + L.ln_2_bias + lH, M + L.w_up + 4 * lHH, M + L.mlp_bias_up + 4 * lH, M + L.w_down + 4 * lHH,
                    M + L.mlp_bias_down + lH);
        }

        // head on the tied embedding, presence penalty, temperature, min-p filter, weighted draw
        gen_norm(s, s.x, s.h, M + L.ln_f, M + L.ln_f_bias, H);
        gen_matvec(s, s.h, M + L.embedding, H, V, 0);
        int lgt = INT_MIN;
        if (threadIdx.x < V) {
            lgt = s.pre[threadIdx.x] >> p.shift_logit;
            for (int i = 0; i <= t && i < 256; i++) if (p.tokens[i] == (uint8_t)threadIdx.x) lgt -= p.penalty_int;
            s.lg[threadIdx.x] = lgt;
        }
        const int mx = gen_block_max(s, lgt);
        if (threadIdx.x < V) {
            const int scaled = (int)__fdiv_rn((float)(s.lg[threadIdx.x] - mx), p.temp);      // (int32_t)(shifted / temp)
            int e = 0;
            if (!p.filter || scaled >= p.min_p_limit) { int idx = -scaled; idx = idx < 0 ? 0 : (idx > 255 ? 255 : idx); e = s.exp_lut[idx]; }
            s.ex[threadIdx.x] = e;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            long long sum = 0;
            for (int v = 0; v < V; v++) sum += s.ex[v];
            const uint32_t r = hash_rng(p.seed + (uint32_t)t * 555u, 0);
            const long long thresh = sum > 0 ? (long long)((unsigned long long)r % (unsigned long long)sum) : 0;
            // the reference's block scan runs thread-major: thread i owns v = i, i + B, ... (B = its block size)
            int selected = 0; long long running = 0; bool done = false;
            for (int i = 0; i < p.scan_block && !done; i++)
                for (int v = i; v < V; v += p.scan_block) {
                    running += s.ex[v];
                    if (running > thresh) { selected = v; done = true; break; }
                }
            if (t >= p.seed_len - 1) p.tokens[t + 1] = (uint8_t)selected;
        }
        __threadfence_block();
        __syncthreads();
    }
}

int launch_generate(cudaStream_t st, const GenParams &p) {
    static bool attr_set[EGG_MAX_DEVICES] = {};
    const int dev = current_device_slot();
    if (!attr_set[dev]) {
        EGG_CUDA(cudaFuncSetAttribute(generate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(GenSmem)));
        attr_set[dev] = true;
    }
    generate_kernel<<<1, GEN_THREADS, sizeof(GenSmem), st>>>(p);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

}  // namespace egg
