// Non-GEMM kernels of the evaluation and update paths: per-pair noise tables,
// row-wise embedding / adaptive-normalise / mean-abs-norm, Q/K/V requantisation,
// causal integer-softmax attention, fitness, update operand generation, vector
// AdamW, Muon Newton–Schulz.  "mgpu.cu" = full_cuda_train_transformer_adam_mgpu.cu.
#include "egg_kernels.cuh"

#include <limits.h>

namespace egg {

// =========================================================================
// noise table
// =========================================================================

void build_noise_map(const egg_config &c, NoiseMap *map, NoiseSeg *segs, int *nsegs, int max_segs) {
    const int H = c.hidden_dim, V = c.vocab_size;
    const int ssv = c.sigma_shift_vector;
    const ScalesLayout SL = scales_layout(c);
    int n = 0, off = 0;
    // sc = AdaptiveScales offset of the overlay that scales the segment (-1: the segment holds raw noise)
    auto put = [&](int kind, int len, int sa, int sb, int shift, int64_t moff, int64_t sc, int bytes) {
        int o = off;
        if (n < max_segs) { segs[n] = NoiseSeg{off, len, kind, sa, sb, shift, moff, sc}; }
        n++; off += bytes; return o;
    };
    auto plain = [&](int len, int seed, int64_t sc) { return put(0, len, seed, 0, 0, -1, sc, len); };
    auto delta = [&](int len, int sa, int sb, int64_t sc) { return put(1, len, sa, sb, ssv, -1, sc, 2 * len); };
    // kind 2: model byte + delta, both signs, as int16 [2][len] (4*len bytes); moff = element offset in TransformerModel
    auto comb = [&](int len, int sa, int sb, int64_t moff, int64_t sc) { return put(2, len, sa, sb, ssv, moff, sc, 4 * len); };
    auto norm = [&](int base, int wa, int wb, int ba, int bb, int64_t mw, int64_t mb, int64_t sw, int64_t sbias) {
        NormOff r; r.w_m = comb(H, base + wa, base + wb, mw, sw); r.b_m = comb(H, base + ba, base + bb, mb, sbias); return r;
    };
    auto mlp = [&](int base, int up_a, int up_b, int bu_a, int bu_b, int dn_a, int dn_b, int bd_a, int bd_b, int64_t s_up_col,
                   int64_t s_bup, int64_t s_dn_col, int64_t s_bdn) {
        MlpOff r;
        r.up_b = plain(H, base + up_b, -1);
        r.up_a = plain(4 * H, base + up_a, s_up_col);
        r.bup_d = delta(4 * H, base + bu_a, base + bu_b, s_bup);
        r.dn_b = plain(4 * H, base + dn_b, -1);
        r.dn_a = plain(H, base + dn_a, s_dn_col);
        r.bdn_d = delta(H, base + bd_a, base + bd_b, s_bdn);
        return r;
    };
    // seed offsets: mgpu.cu:114-165.  Vectors that feed a row dot (the "B" side) stay raw: their overlay is
    // applied per term of the dot.  emb_a is read raw by the embedding and scaled (head_a) by the head.
    map->emb_a = plain(V, 0, -1);
    map->head_a = plain(V, 0, SL.embedding_row);
    map->emb_b = plain(H, 0 + H, -1);
    map->emb_bias_d = delta(H, 50, 51, SL.emb_bias);
    const ModelLayout ML = model_layout(c);
    map->ln_init = norm(0, 500, 501, 502, 503, ML.ln_init, ML.ln_init_bias, SL.ln_init, SL.ln_init_bias);
    map->ln_f = norm(0, 900, 901, 910, 911, ML.ln_f, ML.ln_f_bias, SL.ln_f, SL.ln_f_bias);
    map->mlp_init = mlp(0, 510, 511, 514, 515, 512, 513, 516, 517, SL.w_emb_mlp_up_col, SL.mlp_emb_bias_up, SL.w_emb_mlp_down_col,
                        SL.mlp_emb_bias_down);
    map->layer0 = off;
    for (int l = 0; l < c.n_layers; l++) {
        int base = l * 1000, start = off;
        const int64_t lH = (int64_t)l * H;
        LayerOff lo;
        lo.ln1 = norm(base, 100, 101, 110, 111, ML.ln_1 + lH, ML.ln_1_bias + lH, SL.ln_1 + lH, SL.ln_1_bias + lH);
        lo.qkv_b = plain(H, base + 201, -1); plain(H, base + 203, -1); plain(H, base + 205, -1);
        lo.qkv_a = plain(H, base + 200, SL.w_q_col + lH); plain(H, base + 202, SL.w_k_col + lH); plain(H, base + 204, SL.w_v_col + lH);
        lo.o_b = plain(H, base + 207, -1);
        lo.o_a = plain(H, base + 206, SL.w_o_col + lH);
        lo.ln2 = norm(base, 300, 301, 310, 311, ML.ln_2 + lH, ML.ln_2_bias + lH, SL.ln_2 + lH, SL.ln_2_bias + lH);
        lo.mlp = mlp(base, 400, 401, 410, 411, 402, 403, 412, 413, SL.w_up_col + 4 * lH, SL.mlp_bias_up + 4 * lH, SL.w_down_col + lH,
                     SL.mlp_bias_down + lH);
        if (l == 0) {
            map->layer_stride = off - start;
            LayerOff rel = lo;
            int *pi = reinterpret_cast<int *>(&rel);
            for (size_t i = 0; i < sizeof(LayerOff) / sizeof(int); i++) pi[i] -= start;
            map->layer_rel = rel;
        }
    }
    map->stride = (off + 15) & ~15;
    *nsegs = n;
    noise_index_slices(segs, n < max_segs ? n : max_segs);
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d);

// scales: AdaptiveScales bytes or null.  With scales, every segment that has an overlay holds
// (int)(noise * factor) (A vectors, layers.cuh:90) or the delta built from (int)(n1 * n2 * factor)
// (vectors, layers.cuh:176-180), so that the consumers of the table need not know about overlays.
int noise_index_slices(NoiseSeg *segs, int nsegs) {
    int acc = 0;
    for (int i = 0; i < nsegs; i++) { segs[i].first = acc; acc += (segs[i].len + 1023) >> 10; }
    return acc;
}

__global__ void __launch_bounds__(256) noise_fill_kernel(int8_t *nt, int64_t stride, const NoiseSeg *segs, int nsegs, uint32_t step_seed,
                                                         int pair_base, int mask, int gaussian, const int8_t *model, const int8_t *scales) {
    extern __shared__ NoiseSeg s_segs[];
    for (int i = threadIdx.x; i < nsegs; i += blockDim.x) s_segs[i] = segs[i];
    __syncthreads();
    const int total_slices = s_segs[nsegs - 1].first + ((s_segs[nsegs - 1].len + 1023) >> 10);
    const int pair = blockIdx.y;
    const uint32_t S0 = step_seed + (uint32_t)(pair_base + pair);
    int8_t *dst = nt + (int64_t)pair * stride;
    // one block iteration = 1024 consecutive elements of one segment, four per thread (segment lengths are multiples
    // of four); an element of a delta segment is hashed once and written for both signs
    int g = 0;
    for (int sl = blockIdx.x; sl < total_slices; sl += gridDim.x) {
        while (g + 1 < nsegs && s_segs[g + 1].first <= sl) g++;    // slices are visited in increasing order
        const NoiseSeg sg = s_segs[g];
        const int i0 = ((sl - sg.first) << 10) + (threadIdx.x << 2);
        if (i0 >= sg.len) continue;
        const bool scaled = scales != nullptr && sg.scale_off >= 0;
        int vp[4], vn[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int i = i0 + e;
            int val = noise_from_hash(S0 + (uint32_t)sg.seed_a, (uint32_t)i, mask, gaussian);
            if (sg.kind != 0) val *= noise_from_hash(S0 + (uint32_t)sg.seed_b, (uint32_t)i, mask, gaussian);
            if (scaled) val = scale_trunc(val, overlay_num(scales[sg.scale_off + i]));
            if (sg.kind == 0) { vp[e] = val; vn[e] = 0; }
            else {
                vp[e] = val >> sg.shift; vn[e] = (-val) >> sg.shift;
                if (sg.kind == 2) { const int m = model[sg.model_off + i]; vp[e] += m; vn[e] += m; }
            }
        }
        if (sg.kind == 2) {
            int16_t *d16 = reinterpret_cast<int16_t *>(dst + sg.off);
            *reinterpret_cast<int2 *>(d16 + i0) = make_int2((vp[0] & 0xFFFF) | (vp[1] << 16), (vp[2] & 0xFFFF) | (vp[3] << 16));
            *reinterpret_cast<int2 *>(d16 + sg.len + i0) = make_int2((vn[0] & 0xFFFF) | (vn[1] << 16), (vn[2] & 0xFFFF) | (vn[3] << 16));
        } else {
            *reinterpret_cast<uint32_t *>(dst + sg.off + i0) = pack4(vp[0], vp[1], vp[2], vp[3]);
            if (sg.kind == 1) *reinterpret_cast<uint32_t *>(dst + sg.off + sg.len + i0) = pack4(vn[0], vn[1], vn[2], vn[3]);
        }
    }
}

int launch_noise_fill(cudaStream_t st, int8_t *nt, int64_t stride, const NoiseSeg *d_segs, int nsegs, int n_pairs,
                      uint32_t step_seed, int pair_base, int mask, int gaussian, const int8_t *model, const int8_t *scales) {
    int gx = (int)((stride + 255) / 256); if (gx > 16) gx = 16;      // a few slices per block amortise the segment-table load
    dim3 grid((unsigned)gx, (unsigned)n_pairs);
    const size_t smem = nsegs * sizeof(NoiseSeg);
    noise_fill_kernel<<<grid, 256, smem, st>>>(nt, stride, d_segs, nsegs, step_seed, pair_base, mask, gaussian, model, scales);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// =========================================================================
// row-wise: embedding | adaptive layer normalise -> x ; mean-abs norm -> h ; noise dots
// =========================================================================

__device__ __forceinline__ int warp_sum(int v) {
    return __reduce_add_sync(0xFFFFFFFFu, v);       // one warp-wide integer reduction instruction; every lane gets the sum
}

__device__ __forceinline__ int8_t byte_of(int32_t w, int i) { return (int8_t)(w >> (8 * i)); }
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xFF) | ((uint32_t)(b & 0xFF) << 8) | ((uint32_t)(c & 0xFF) << 16) | ((uint32_t)(d & 0xFF) << 24);
}

// One warp per run of ROW_RUN consecutive rows of ONE population member (seq_len is a multiple of 16, so a run never
// crosses members); NJ = H/128 chunks of 4 elements per lane.  Everything that depends on the member only -- the
// perturbed gain / bias tables and the noise vectors of the following projections, 3.5 H bytes -- is loaded once per
// run and kept in registers; per row only the row itself is read, and the next row's bytes are requested before the
// current row is worked on (mode 2), so that the warp always has a load in flight.
constexpr int ROW_RUN = 8;
#ifndef ROW_EMB_BLOCKS
#define ROW_EMB_BLOCKS 2          // resident blocks asked for in embedding mode (its per-member tables are the widest)
#endif

// WIDE (embedding mode only): the dataset holds uint32_t tokens below 65536 (vocab_size != 256, mgpu.cu:58-66)
// NTT (embedding mode only): bytes 1..3 of the row's transformed-window coefficient index three more tables whose
// rows are added >> 2 each (NTT_MODE != 0, mgpu.cu:916-929)
template <int MODE, int NJ, int NDOTS, bool WIDE = false, bool NTT = false>
__global__ void __launch_bounds__(256, MODE == 0 ? ROW_EMB_BLOCKS : 1) rowwise_kernel(const RowParams p) {
    const int run = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int r0 = run * ROW_RUN;
    if (r0 >= p.M) return;
    const int r_end = min(r0 + ROW_RUN, p.M);
    const int H = NJ * 128;
    const int mem = fast_div(r0, p.fd_seq);
    const int sgn = mem & 1, ns = sgn ? -1 : 1;
    const int8_t *ntp = p.nt + (int64_t)(mem >> 1) * p.nt_stride;
    const int16_t *wm = reinterpret_cast<const int16_t *>(ntp + p.nt_w_m) + sgn * H;   // w + ((n1*n2*sign)>>SSV)
    const int16_t *bm = reinterpret_cast<const int16_t *>(ntp + p.nt_b_m) + sgn * H;

    // ---- per-member tables: gains and biases widened once per run, not once per row ----
    int wv[NJ][4], bv[NJ][4];
    int32_t n4[NDOTS][NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int d = (j << 7) + (lane << 2);
        const int2 w4 = *reinterpret_cast<const int2 *>(wm + d);
        const int2 b4 = *reinterpret_cast<const int2 *>(bm + d);
        // low halves sign-extended by one byte permute (selector msb = replicate the byte's sign), high halves by a shift
        wv[j][0] = ptx::sx_half0(w4.x); wv[j][1] = w4.x >> 16; wv[j][2] = ptx::sx_half0(w4.y); wv[j][3] = w4.y >> 16;
        bv[j][0] = ptx::sx_half0(b4.x); bv[j][1] = b4.x >> 16; bv[j][2] = ptx::sx_half0(b4.y); bv[j][3] = b4.y >> 16;
#pragma unroll
        for (int q = 0; q < NDOTS; q++) n4[q][j] = *reinterpret_cast<const int32_t *>(ntp + p.nt_dot[q] + d);
    }
    // embedding mode: bias + bias-noise delta, the B-noise of the embedding's rank-1 term and the column overlays of the run's member
    int emb_add[MODE == 0 ? NJ : 1][4];
    int32_t emb_nb[MODE == 0 ? NJ : 1], emb_oc[MODE == 0 ? NJ : 1];
    if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const int d = (j << 7) + (lane << 2);
            const int32_t eb4 = *reinterpret_cast<const int32_t *>(p.emb_bias + d);
            const int32_t dl4 = *reinterpret_cast<const int32_t *>(ntp + p.nt_emb_bias_d + sgn * H + d);
#pragma unroll
            for (int i = 0; i < 4; i++) emb_add[j][i] = (int)byte_of(eb4, i) + (int)byte_of(dl4, i);
            emb_nb[j] = *reinterpret_cast<const int32_t *>(ntp + p.nt_emb_b + d);
            emb_oc[j] = p.ov_emb_col ? *reinterpret_cast<const int32_t *>(p.ov_emb_col + d) : 0;
        }
    }
    uint32_t xw_next[NJ];
    if (MODE == 2) {
#pragma unroll
        for (int j = 0; j < NJ; j++) xw_next[j] = *reinterpret_cast<const uint32_t *>(p.x_out + (int64_t)r0 * H + (j << 7) + (lane << 2));
    }

    // embedding mode: the run's tokens and their A-noise bytes are fetched up front (two dependent loads that would
    // otherwise sit at the head of every row), and the embedding row of the next token is requested a row ahead
    unsigned long long toks = 0, atoks = 0;          // one byte per row of the run (ROW_RUN = 8)
    unsigned long long toks_hi = 0;                  // WIDE: bits 8..15 of the run's tokens, packed the same way
    auto tok_of = [&](int i) { return (int)((toks >> (8 * i)) & 0xFF) | (WIDE ? (int)((toks_hi >> (8 * i)) & 0xFF) << 8 : 0); };
    int32_t e4_next[MODE == 0 ? NJ : 1];
    if (MODE == 0) {
        static_assert(ROW_RUN == 8, "the run's tokens are packed into one 64-bit register");
        const int64_t pair = (p.pop_base + mem) >> 1;
        const int64_t pos = p.use_same_data ? (p.start_idx % (p.data_len - p.seq_len))
                                            : ((p.start_idx + pair * p.data_stride) % (p.data_len - p.seq_len));
        const int64_t tpos = pos + (r0 - mem * p.seq_len);
#pragma unroll
        for (int i = 0; i < ROW_RUN; i++) {
            unsigned tok = 0u;
            if (r0 + i < r_end) tok = WIDE ? reinterpret_cast<const uint32_t *>(p.dataset)[tpos + i] : (unsigned)p.dataset[tpos + i];
            toks |= (unsigned long long)(tok & 0xFF) << (8 * i);
            if (WIDE) toks_hi |= (unsigned long long)((tok >> 8) & 0xFF) << (8 * i);
        }
#pragma unroll
        for (int i = 0; i < ROW_RUN; i++) atoks |= (unsigned long long)(uint8_t)ntp[p.nt_emb_a + tok_of(i)] << (8 * i);
#pragma unroll
        for (int j = 0; j < NJ; j++) e4_next[j] = *reinterpret_cast<const int32_t *>(p.emb_rows + (int64_t)tok_of(0) * H + (j << 7) + (lane << 2));
    }

    for (int ri = 0; ri < ROW_RUN; ri++) {
        const int r = r0 + ri;
        if (r >= r_end) break;
        int x[NJ][4];
        uint32_t xw_cur[MODE == 2 ? NJ : 1];
        if (MODE == 0) {
            // embedding (mgpu.cu:902-931): the token's row comes from the token-major copy of the table ([V][H], the same
            // K-major shadow the head projection multiplies with), 4 contiguous bytes per lane and chunk
            const int tok = tok_of(ri);
            const int a_tok = (int)(int8_t)((atoks >> (8 * ri)) & 0xFF);
            const float f_row = p.ov_emb_row ? __fdiv_rn((float)overlay_num(p.ov_emb_row[tok]), 64.0f) : 1.0f;
            int32_t e4c[NJ];
#pragma unroll
            for (int j = 0; j < NJ; j++) e4c[j] = e4_next[j];
            if (ri + 1 < ROW_RUN && r + 1 < r_end) {
#pragma unroll
                for (int j = 0; j < NJ; j++) e4_next[j] = *reinterpret_cast<const int32_t *>(p.emb_rows + (int64_t)tok_of(ri + 1) * H + (j << 7) + (lane << 2));
            }
            int ex[NTT ? NJ : 1][4];
            if (NTT) {
                const int cw = p.ntt_coef[(int64_t)(mem >> 1) * p.seq_len + (r - mem * p.seq_len)];
#pragma unroll
                for (int j = 0; j < NJ; j++) { ex[j][0] = 0; ex[j][1] = 0; ex[j][2] = 0; ex[j][3] = 0; }
#pragma unroll
                for (int k = 0; k < 3; k++) {
                    const int8_t *nrow = p.ntt_rows + ((int64_t)k * p.vocab + ((cw >> (8 * (k + 1))) & 0xFF)) * H;
#pragma unroll
                    for (int j = 0; j < NJ; j++) {
                        const int32_t w4 = *reinterpret_cast<const int32_t *>(nrow + (j << 7) + (lane << 2));
#pragma unroll
                        for (int i = 0; i < 4; i++) ex[j][i] += (int)byte_of(w4, i) >> 2;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const int32_t e4 = e4c[j];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    int prod = a_tok * (int)byte_of(emb_nb[j], i);
                    if (p.ov_emb_col) {
                        // (AccumType)(a_tok * b_dim * s_emb_row * s_emb_col), d-eggs kernels.cu:150-158: two float
                        // multiplications, each rounded, then the truncating conversion
                        const float fc = __fdiv_rn((float)overlay_num(byte_of(emb_oc[j], i)), 64.0f);
                        prod = __float2int_rz(__fmul_rn(__fmul_rn((float)prod, f_row), fc));
                    }
                    int perturb = (prod * ns) >> p.emb_shift;
                    x[j][i] = clip8((int)byte_of(e4, i) + emb_add[j][i] + perturb + (NTT ? ex[j][i] : 0));
                }
            }
        } else if (MODE == 2) {
            // the residual stream was requantised by the projection that produced it: only read it
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const uint32_t w = xw_next[j];
                xw_cur[j] = w;
                x[j][0] = ptx::sx_byte0(w); x[j][1] = ptx::sx_byte1(w); x[j][2] = ptx::sx_byte2(w); x[j][3] = (int)w >> 24;
            }
            if (r + 1 < r_end) {
#pragma unroll
                for (int j = 0; j < NJ; j++) xw_next[j] = *reinterpret_cast<const uint32_t *>(p.x_out + (int64_t)(r + 1) * H + (j << 7) + (lane << 2));
            }
        } else {
            int4 v[NJ];
#pragma unroll
            for (int j = 0; j < NJ; j++) v[j] = *reinterpret_cast<const int4 *>(p.pre32 + (int64_t)r * H + (j << 7) + (lane << 2));
            const int mx = p.rowmax[r];
            const float scale = aln_scale24(mx);
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                x[j][0] = aln_quant(v[j].x, scale); x[j][1] = aln_quant(v[j].y, scale);
                x[j][2] = aln_quant(v[j].z, scale); x[j][3] = aln_quant(v[j].w, scale);
            }
        }
        int tot = 0;
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const int d = (j << 7) + (lane << 2);
            uint32_t w;
            if (MODE == 2) {
                w = xw_cur[j];                                                       // the bytes as they were read
            } else {
                w = ptx::pack_sat_s8(x[j][0], x[j][1], x[j][2], x[j][3]);            // |x| <= 127: the saturating pack is exact, two instructions
                *reinterpret_cast<uint32_t *>(p.x_out + (int64_t)r * H + d) = w;
            }
            tot = __dp4a((int)__vabsss4(w), 0x01010101, tot);    // sum of |x|, four at a time
        }
        // mean-abs norm with perturbed gain / bias (mgpu.cu:646-678): y = clip((x*w')/mn + b')
        tot = warp_sum(tot);
        int mn = tot / H;
        if (!mn) mn = 1;
        const float rinv = c_rinv_up.v[mn];                     // mn <= 127: a mean of absolute values of int8
        int dot[NDOTS];
#pragma unroll
        for (int q = 0; q < NDOTS; q++) dot[q] = 0;
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const int d = (j << 7) + (lane << 2);
            int y[4];
#pragma unroll
            for (int i = 0; i < 4; i++) y[i] = div_small(x[j][i] * wv[j][i], rinv) * p.one + bv[j][i];   // the add as a multiply-add by a run-time 1: off the busier integer pipe
            const uint32_t yw = pack_clip8(y[0], y[1], y[2], y[3]);
            *reinterpret_cast<uint32_t *>(p.h_out + (int64_t)r * H + d) = yw;
#pragma unroll
            for (int q = 0; q < NDOTS; q++) dot[q] = __dp4a((int)yw, n4[q][j], dot[q]);
        }
#pragma unroll
        for (int q = 0; q < NDOTS; q++) {
            const int s = warp_sum(dot[q]);
            if (lane == 0) p.xb_out[(int64_t)r * p.xb_stride + q] = s;
        }
        if (lane == 0) {
            if (MODE == 1) p.rowmax[r] = 0;
            if (p.zero1) p.zero1[r] = 0;
            if (p.zero2) p.zero2[r] = 0;
            if (p.zero3) { p.zero3[(int64_t)r * 3] = 0; p.zero3[(int64_t)r * 3 + 1] = 0; p.zero3[(int64_t)r * 3 + 2] = 0; }
        }
    }
}

template <int MODE, int NDOTS, bool WIDE = false, bool NTT = false>
static int launch_rowwise_nj(cudaStream_t st, const RowParams &p) {
    const int blocks = ((p.M + ROW_RUN - 1) / ROW_RUN + 7) / 8;       // 8 warps per block, one run of rows per warp
    switch (p.H >> 7) {
        case 1: rowwise_kernel<MODE, 1, NDOTS, WIDE, NTT><<<blocks, 256, 0, st>>>(p); break;
        case 2: rowwise_kernel<MODE, 2, NDOTS, WIDE, NTT><<<blocks, 256, 0, st>>>(p); break;
        case 3: rowwise_kernel<MODE, 3, NDOTS, WIDE, NTT><<<blocks, 256, 0, st>>>(p); break;
        case 4: rowwise_kernel<MODE, 4, NDOTS, WIDE, NTT><<<blocks, 256, 0, st>>>(p); break;
        case 5: rowwise_kernel<MODE, 5, NDOTS, WIDE, NTT><<<blocks, 256, 0, st>>>(p); break;
        case 6: rowwise_kernel<MODE, 6, NDOTS, WIDE, NTT><<<blocks, 256, 0, st>>>(p); break;
        case 7: rowwise_kernel<MODE, 7, NDOTS, WIDE, NTT><<<blocks, 256, 0, st>>>(p); break;
        case 8: rowwise_kernel<MODE, 8, NDOTS, WIDE, NTT><<<blocks, 256, 0, st>>>(p); break;
        default: set_error("hidden_dim %d unsupported by the row-wise kernel", p.H); return EGG_E_INVALID;
    }
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

int launch_rowwise(cudaStream_t st, const RowParams &p_in, int mode) {
    RowParams p = p_in;
    p.fd_seq = make_fastdiv(p.seq_len);
    p.one = 1;
    if (p.ndots != 1 && p.ndots != 3) { set_error("row-wise kernel computes one or three row dots, not %d", p.ndots); return EGG_E_INVALID; }
    if (mode == 0 && (p.tok_wide || p.ntt_coef)) {
        if (p.ndots != 1 || p.vocab > 65536) { set_error("wide-token / transformed-window embedding takes one row dot and a vocabulary of at most 65536"); return EGG_E_INVALID; }
        if (p.ntt_coef) return p.tok_wide ? launch_rowwise_nj<0, 1, true, true>(st, p) : launch_rowwise_nj<0, 1, false, true>(st, p);
        return launch_rowwise_nj<0, 1, true>(st, p);
    }
    if (p.ndots == 1) return mode == 0 ? launch_rowwise_nj<0, 1>(st, p) : (mode == 1 ? launch_rowwise_nj<1, 1>(st, p) : launch_rowwise_nj<2, 1>(st, p));
    return mode == 0 ? launch_rowwise_nj<0, 3>(st, p) : (mode == 1 ? launch_rowwise_nj<1, 3>(st, p) : launch_rowwise_nj<2, 3>(st, p));
}

// Row dots under adaptive-noise overlays (d-eggs/include/model/layers.cuh:250, 272-280, 339-341, 396):
//   out[r][q] = Σ_tid pb(tid),  pb = 0;  for sub < terms:  pb = (int)((float)pb + x[k] * noise_q[k] * factor_q[k]),
//   k = tid + sub*H
// — with one term per thread this truncates every product, with four (the down projection) it truncates
// the thread's running sum.  All values are multiples of 1/64 below 2^17, so the float arithmetic of the
// reference is exact and is done here in integers: pb = trunc((64*pb + x*n*num) / 64).
__global__ void __launch_bounds__(256) scaled_dot_kernel(const ScaledDotParams p) {
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= p.M) return;
    const int H = p.H, K = H * p.terms;
    const int mem = r / p.seq_len;
    const int8_t *ntp = p.nt + (int64_t)(mem >> 1) * p.nt_stride;
    const int8_t *xr = p.x + (int64_t)r * K;
    for (int q = 0; q < p.ndots; q++) {
        const int8_t *nz = ntp + p.nt_dot[q];
        const int8_t *ov = p.ov[q];
        int acc = 0;
        for (int d = lane << 2; d < H; d += 128) {
            int pb[4] = {0, 0, 0, 0};
            for (int sub = 0; sub < p.terms; sub++) {
                const int k = d + sub * H;
                const int32_t x4 = *reinterpret_cast<const int32_t *>(xr + k);
                const int32_t n4 = *reinterpret_cast<const int32_t *>(nz + k);
                const int32_t o4 = *reinterpret_cast<const int32_t *>(ov + k);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int t = (pb[i] << 6) + (int)byte_of(x4, i) * (int)byte_of(n4, i) * overlay_num(byte_of(o4, i));
                    pb[i] = (t + ((t >> 31) & 63)) >> 6;
                }
            }
            acc += pb[0] + pb[1] + pb[2] + pb[3];
        }
        acc = warp_sum(acc);
        if (lane == 0) p.out[(int64_t)r * p.out_stride + q] = acc;
    }
}

int launch_scaled_dot(cudaStream_t st, const ScaledDotParams &p) {
    scaled_dot_kernel<<<(p.M + 7) / 8, 256, 0, st>>>(p);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// update_overlay_kernel (d-eggs/src/kernels.cu:61-77): +inc where a weight of the row / column / element
// changed in this update, -dec elsewhere, clamped to [-127, 127]; the change flags are cleared for the next use.
__global__ void overlay_step_kernel(int8_t *ov, uint8_t *changed, int n, int inc, int dec) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int v = ov[i];
    if (changed[i]) { v += inc; if (v > 127) v = 127; } else { v -= dec; if (v < -127) v = -127; }
    ov[i] = (int8_t)v;
    changed[i] = 0;
}

int launch_overlay_step(cudaStream_t st, int8_t *ov, uint8_t *changed, int n, int inc, int dec) {
    overlay_step_kernel<<<(n + 255) / 256, 256, 0, st>>>(ov, changed, n, inc, dec);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// Q/K/V requantisation (adaptive_qkv_normalize, mgpu.cu:782-784).  One warp per row; all of the row's loads
// (three parts x NJ 16-byte pieces per lane) are issued before any arithmetic.
template <int NJ>
__global__ void __launch_bounds__(256) aqn_kernel(const AqnParams p) {
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= p.M) return;
    constexpr int H = NJ * 128;
    const int32_t *src = p.pre3 + (int64_t)r * 3 * H + (lane << 2);
    int4 v[3][NJ];
#pragma unroll
    for (int which = 0; which < 3; which++)
#pragma unroll
        for (int j = 0; j < NJ; j++) v[which][j] = *reinterpret_cast<const int4 *>(src + which * H + (j << 7));
    const int mx0 = p.rowmax3[(int64_t)r * 3], mx1 = p.rowmax3[(int64_t)r * 3 + 1], mx2 = p.rowmax3[(int64_t)r * 3 + 2];
#pragma unroll
    for (int which = 0; which < 3; which++) {
        const int mx = which == 0 ? mx0 : (which == 1 ? mx1 : mx2);
        const float scale = aln_scale24(mx);
        int8_t *out = (which == 0 ? p.q : (which == 1 ? p.k : p.v)) + (int64_t)r * H + (lane << 2);
#pragma unroll
        for (int j = 0; j < NJ; j++)
            *reinterpret_cast<uint32_t *>(out + (j << 7)) = pack_clip8(aln_quant(v[which][j].x, scale), aln_quant(v[which][j].y, scale),
                                                                       aln_quant(v[which][j].z, scale), aln_quant(v[which][j].w, scale));
    }
}

int launch_aqn(cudaStream_t st, const AqnParams &p) {
    const int blocks = (p.M + 7) / 8;
    switch (p.H >> 7) {
        case 1: aqn_kernel<1><<<blocks, 256, 0, st>>>(p); break;
        case 2: aqn_kernel<2><<<blocks, 256, 0, st>>>(p); break;
        case 3: aqn_kernel<3><<<blocks, 256, 0, st>>>(p); break;
        case 4: aqn_kernel<4><<<blocks, 256, 0, st>>>(p); break;
        case 5: aqn_kernel<5><<<blocks, 256, 0, st>>>(p); break;
        case 6: aqn_kernel<6><<<blocks, 256, 0, st>>>(p); break;
        case 7: aqn_kernel<7><<<blocks, 256, 0, st>>>(p); break;
        case 8: aqn_kernel<8><<<blocks, 256, 0, st>>>(p); break;
        default: set_error("hidden_dim %d unsupported by the requantisation kernel", p.H); return EGG_E_INVALID;
    }
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// =========================================================================
// causal integer-softmax attention (mgpu.cu:787-825), one block per (member, head)
// =========================================================================
// Scores and weighted sums run on the int8 tensor-core path (mma.sync m16n8k32):
// exact, because every partial sum is proven to fit int32 — scores <= 64*127^2,
// and the 19-bit softmax weights are split into three 7-bit limbs so that each
// limb's Σ w·v <= 127*127*seq_len; the limbs are recombined in int64 before the
// reference's truncating division.

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// the same product started from a zero accumulator: the outputs are written, not read, so no register has to be
// cleared first
__device__ __forceinline__ void mma_s8_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

constexpr int ATT_KP = 80;   // K row pitch in shared memory (bytes): conflict-free fragment loads

// scores of one 16-query x 32-key block: c[nt][0..3] for the four 8-key n-tiles
__device__ __forceinline__ void att_scores(int (&c)[4][4], const uint32_t (&qa)[2][4], const int8_t *Ks, int kb, int g, int q) {
#pragma unroll
    for (int nt = 0; nt < 4; nt++) {
        const int8_t *kp = Ks + (kb * 32 + nt * 8 + g) * ATT_KP + 4 * q;
        mma_s8_first(c[nt], qa[0][0], qa[0][1], qa[0][2], qa[0][3], *reinterpret_cast<const uint32_t *>(kp), *reinterpret_cast<const uint32_t *>(kp + 16));
        mma_s8(c[nt], qa[1][0], qa[1][1], qa[1][2], qa[1][3], *reinterpret_cast<const uint32_t *>(kp + 32), *reinterpret_cast<const uint32_t *>(kp + 48));
    }
}

// exact float of an int with |v| < 2^23 (no conversion instruction)
__device__ __forceinline__ float i2f_23(int v) {
    float f = __int_as_float(0x4B000000 | abs(v)) - 8388608.0f;
    return v < 0 ? -f : f;
}

// trunc(num / den) as C does, for |num/den| <= 127: the quotient is estimated in float from the three
// limb sums and fixed up with one exact int64 remainder test.
__device__ __forceinline__ int att_div(int p0, int p1, int p2, long long den, float rden, bool small) {
    const long long num = (long long)p0 + ((long long)p1 << 7) + ((long long)p2 << 14);
    float fn = small ? fmaf(i2f_23(p2), 16384.0f, fmaf(i2f_23(p1), 128.0f, i2f_23(p0))) : (float)num;
    int k = f2i_exact(fn * rden);                     // nearest integer to the real quotient (|error| < 1e-3)
    long long r = num - (long long)k * den;
    if (num >= 0) { if (r < 0) k--; } else { if (r > 0) k++; }
    return k;
}

// The same quotient when every limb sum is below 2^23 (seq_len <= 512): the estimate needs two conversions, and the
// remainder num - k*den is assembled limb by limb in 32-bit arithmetic — it is at most den/2 (+ rounding) < 2^27 in
// magnitude, so the wrapping partial terms add up to its exact value.  d0..d2 are the limb sums of the denominator.
__device__ __forceinline__ int att_div_small(int p0, int p1, int p2, int d0, int d1, int d2, float rden) {
    const float fn = fmaf(__int2float_rn(p2 * 128 + p1), 128.0f, __int2float_rn(p0));
    int k = __float2int_rn(fn * rden);
    const int r = (p0 - k * d0) + (p1 - k * d1) * 128 + (p2 - k * d2) * 16384;
    if (k > 0 && r < 0) k--;
    else if (k < 0 && r > 0) k++;
    return k;
}

__global__ void __launch_bounds__(128) attention_kernel(const AttnParams p) {
    extern __shared__ __align__(16) uint8_t att_smem[];
    const int S = p.seq_len, SP = (S + 31) & ~31, VP = SP + 16, H = p.H;
    int8_t *Ks = reinterpret_cast<int8_t *>(att_smem);          // [SP][80]
    int8_t *Vt = Ks + SP * ATT_KP;                               // [64][VP]  (V transposed: dim-major)
    uint32_t *lut3 = reinterpret_cast<uint32_t *>(Vt + 64 * VP); // [256] softmax weight as three 7-bit limbs, one per byte
    const int n_heads = H / 64;
    const int mem = blockIdx.x / n_heads, hd = blockIdx.x % n_heads;
    const int64_t base = (int64_t)mem * S;
    const int col0 = hd * 64;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (int i = tid; i < SP * 4; i += 128) {
        int row = i >> 2, ch = i & 3;
        int4 v = make_int4(0, 0, 0, 0);
        if (row < S) v = *reinterpret_cast<const int4 *>(p.k + (base + row) * H + col0 + ch * 16);
        *reinterpret_cast<int4 *>(Ks + row * ATT_KP + ch * 16) = v;
    }
    // V: each item = 4 consecutive keys x 16 dims, transposed in registers (4x4 byte blocks) and written as
    // 32-bit words Vt[dim][key..key+3]; consecutive lanes take consecutive key groups -> conflict-free stores.
    for (int i = tid; i < (SP / 4) * 4; i += 128) {
        const int kg = i % (SP / 4), ch = i / (SP / 4);
        int4 r[4];
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            const int row = kg * 4 + kk;
            r[kk] = make_int4(0, 0, 0, 0);
            if (row < S) r[kk] = *reinterpret_cast<const int4 *>(p.v + (base + row) * H + col0 + ch * 16);
        }
        const uint32_t *w0 = reinterpret_cast<const uint32_t *>(&r[0]), *w1 = reinterpret_cast<const uint32_t *>(&r[1]);
        const uint32_t *w2 = reinterpret_cast<const uint32_t *>(&r[2]), *w3 = reinterpret_cast<const uint32_t *>(&r[3]);
#pragma unroll
        for (int dq = 0; dq < 4; dq++) {       // dims 4dq..4dq+3 of this chunk
            uint32_t t0 = __byte_perm(w0[dq], w1[dq], 0x5140), t1 = __byte_perm(w2[dq], w3[dq], 0x5140);   // [a0 b0 a1 b1]
            uint32_t t2 = __byte_perm(w0[dq], w1[dq], 0x7362), t3 = __byte_perm(w2[dq], w3[dq], 0x7362);   // [a2 b2 a3 b3]
            const int dim = ch * 16 + dq * 4;
            // keys are stored permuted inside every group of 16 so that the four keys an MMA B-fragment register needs
            // ({2q, 2q+1, 8+2q, 9+2q}) are one aligned word: keys 4m, 4m+1 go to slot (m&1)*8 + (m>>1)*2, keys 4m+2, 4m+3 four further
            const int m = kg & 3;
            const int so = (kg >> 2) * 16 + (m & 1) * 8 + (m >> 1) * 2;
            const uint32_t w0 = __byte_perm(t0, t1, 0x5410), w1 = __byte_perm(t0, t1, 0x7632);
            const uint32_t w2 = __byte_perm(t2, t3, 0x5410), w3 = __byte_perm(t2, t3, 0x7632);
            *reinterpret_cast<uint16_t *>(Vt + (dim + 0) * VP + so) = (uint16_t)w0; *reinterpret_cast<uint16_t *>(Vt + (dim + 0) * VP + so + 4) = (uint16_t)(w0 >> 16);
            *reinterpret_cast<uint16_t *>(Vt + (dim + 1) * VP + so) = (uint16_t)w1; *reinterpret_cast<uint16_t *>(Vt + (dim + 1) * VP + so + 4) = (uint16_t)(w1 >> 16);
            *reinterpret_cast<uint16_t *>(Vt + (dim + 2) * VP + so) = (uint16_t)w2; *reinterpret_cast<uint16_t *>(Vt + (dim + 2) * VP + so + 4) = (uint16_t)(w2 >> 16);
            *reinterpret_cast<uint16_t *>(Vt + (dim + 3) * VP + so) = (uint16_t)w3; *reinterpret_cast<uint16_t *>(Vt + (dim + 3) * VP + so + 4) = (uint16_t)(w3 >> 16);
        }
    }
    for (int i = tid; i < 256; i += 128) {
        uint32_t w = (uint32_t)p.exp_lut[i];
        lut3[i] = (w & 127u) | (((w >> 7) & 127u) << 8) | ((w >> 14) << 16);
    }
    __syncthreads();

    const int g = lane >> 2, q = lane & 3;
    const int8_t *nbo = p.nt + (int64_t)(mem >> 1) * p.nt_stride + p.nt_o_b + col0;
    const int sh = p.shift_attn;
    const bool small_limbs = S <= 512;     // every limb sum < 127*127*512 < 2^23

    // Query blocks are dealt to the four warps in boustrophedon order (w, 7-w, 8+w, 15-w, ...): block qb costs
    // qb/2 + 1 key blocks under the causal mask, and this order gives every warp the same total (18 of 72 at
    // seq_len 256) where the plain stride-4 order leaves warp 3 with 20 and warp 0 with 16.
    for (int rnd = 0; rnd * 4 < S / 16; rnd++) {
        const int qb = rnd * 4 + ((rnd & 1) ? 3 - warp : warp);
        if (qb >= S / 16) continue;
        const int q0 = qb * 16;
        const int row0 = q0 + g, row1 = q0 + g + 8;
        uint32_t qa[2][4];
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
            const int8_t *qp0 = p.q + (base + row0) * H + col0 + 32 * ks + 4 * q;
            const int8_t *qp1 = p.q + (base + row1) * H + col0 + 32 * ks + 4 * q;
            qa[ks][0] = *reinterpret_cast<const uint32_t *>(qp0);
            qa[ks][1] = *reinterpret_cast<const uint32_t *>(qp1);
            qa[ks][2] = *reinterpret_cast<const uint32_t *>(qp0 + 16);
            qa[ks][3] = *reinterpret_cast<const uint32_t *>(qp1 + 16);
        }
        const int last = (q0 + 15) / 32;          // the only key block that needs the causal mask

        // ---- pass 1: row maxima over ctx <= t (mgpu.cu:795-802) ----
        int mx0 = INT_MIN, mx1 = INT_MIN;
        int c[4][4];
        for (int kb = 0; kb < last; kb++) {
            att_scores(c, qa, Ks, kb, g, q);
#pragma unroll
            for (int nt = 0; nt < 4; nt++) { mx0 = max(mx0, max(c[nt][0], c[nt][1])); mx1 = max(mx1, max(c[nt][2], c[nt][3])); }
        }
        att_scores(c, qa, Ks, last, g, q);
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            const int key = last * 32 + nt * 8 + 2 * q;
            if (key <= row0) mx0 = max(mx0, c[nt][0]);
            if (key + 1 <= row0) mx0 = max(mx0, c[nt][1]);
            if (key <= row1) mx1 = max(mx1, c[nt][2]);
            if (key + 1 <= row1) mx1 = max(mx1, c[nt][3]);
        }
        mx0 = max(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1)); mx0 = max(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
        mx1 = max(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1)); mx1 = max(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
        const int mxs0 = mx0 >> sh, mxs1 = mx1 >> sh;

        // ---- pass 2: weights, Σ w·v in three 7-bit limbs (mgpu.cu:810-824) ----
        int acc[8][3][4];
#pragma unroll
        for (int a = 0; a < 8; a++)
#pragma unroll
            for (int l = 0; l < 3; l++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[a][l][i] = 0;
        int tl0[3] = {0, 0, 0}, tl1[3] = {0, 0, 0};      // per-limb Σ w for rows g and g+8
        for (int kb = 0; kb <= last; kb++) {
            att_scores(c, qa, Ks, kb, g, q);
            uint32_t w[4][4];                             // limb-packed weights
            if (kb < last) {
#pragma unroll
                for (int nt = 0; nt < 4; nt++) {
                    w[nt][0] = lut3[min(255, mxs0 - (c[nt][0] >> sh))];
                    w[nt][1] = lut3[min(255, mxs0 - (c[nt][1] >> sh))];
                    w[nt][2] = lut3[min(255, mxs1 - (c[nt][2] >> sh))];
                    w[nt][3] = lut3[min(255, mxs1 - (c[nt][3] >> sh))];
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < 4; nt++) {
                    const int key = kb * 32 + nt * 8 + 2 * q;
                    w[nt][0] = (key <= row0) ? lut3[min(255, mxs0 - (c[nt][0] >> sh))] : 0u;
                    w[nt][1] = (key + 1 <= row0) ? lut3[min(255, mxs0 - (c[nt][1] >> sh))] : 0u;
                    w[nt][2] = (key <= row1) ? lut3[min(255, mxs1 - (c[nt][2] >> sh))] : 0u;
                    w[nt][3] = (key + 1 <= row1) ? lut3[min(255, mxs1 - (c[nt][3] >> sh))] : 0u;
                }
            }
            // A fragments of the three limbs; k-slot 4q+{0,1,2,3} <-> keys {2q, 2q+1, 8+2q, 9+2q} (+16 for a2/a3)
            uint32_t al[3][4];
#pragma unroll
            for (int f = 0; f < 4; f++) {
                // 4 x 3 byte transpose of the four weights of fragment register f (7 byte permutes)
                const int n0 = (f >> 1) * 2, i0 = (f & 1) * 2;
                const uint32_t wa = w[n0][i0], wb = w[n0][i0 + 1], wc = w[n0 + 1][i0], wd = w[n0 + 1][i0 + 1];
                const uint32_t t0 = __byte_perm(wa, wb, 0x5140), t1 = __byte_perm(wc, wd, 0x5140);     // [a0 b0 a1 b1], [c0 d0 c1 d1]
                const uint32_t t2 = __byte_perm(wa, wb, 0x7362), t3 = __byte_perm(wc, wd, 0x7362);     // [a2 b2 . .], [c2 d2 . .]
                al[0][f] = __byte_perm(t0, t1, 0x5410);
                al[1][f] = __byte_perm(t0, t1, 0x7632);
                al[2][f] = __byte_perm(t2, t3, 0x5410);
            }
#pragma unroll
            for (int l = 0; l < 3; l++) {
                tl0[l] = __dp4a((int)al[l][0], 0x01010101, __dp4a((int)al[l][2], 0x01010101, tl0[l]));
                tl1[l] = __dp4a((int)al[l][1], 0x01010101, __dp4a((int)al[l][3], 0x01010101, tl1[l]));
            }
#pragma unroll
            for (int dn = 0; dn < 8; dn++) {
                const int8_t *vp = Vt + (dn * 8 + g) * VP + kb * 32 + 4 * q;
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(vp), b1 = *reinterpret_cast<const uint32_t *>(vp + 16);
#pragma unroll
                for (int l = 0; l < 3; l++) mma_s8(acc[dn][l], al[l][0], al[l][1], al[l][2], al[l][3], b0, b1);
            }
        }
#pragma unroll
        for (int l = 0; l < 3; l++) {                 // limb sums of Σw over the four lanes that share a row
            tl0[l] += __shfl_xor_sync(0xFFFFFFFFu, tl0[l], 1); tl0[l] += __shfl_xor_sync(0xFFFFFFFFu, tl0[l], 2);
            tl1[l] += __shfl_xor_sync(0xFFFFFFFFu, tl1[l], 1); tl1[l] += __shfl_xor_sync(0xFFFFFFFFu, tl1[l], 2);
        }
        const uint32_t tot0 = (uint32_t)tl0[0] + ((uint32_t)tl0[1] << 7) + ((uint32_t)tl0[2] << 14);
        const uint32_t tot1 = (uint32_t)tl1[0] + ((uint32_t)tl1[1] << 7) + ((uint32_t)tl1[2] << 14);
        const long long den0 = tot0 ? (long long)tot0 : 1, den1 = tot1 ? (long long)tot1 : 1;
        const float rden0 = 1.0f / (float)den0, rden1 = 1.0f / (float)den1;
        int dot0 = 0, dot1 = 0;
#pragma unroll
        for (int dn = 0; dn < 8; dn++) {
            int o[4];
            if (small_limbs) {
                // |Σw·v / Σw| <= 127 (a weighted mean of int8 values): the reference's clip cannot trigger
#pragma unroll
                for (int i = 0; i < 4; i++)
                    o[i] = i < 2 ? att_div_small(acc[dn][0][i], acc[dn][1][i], acc[dn][2][i], tl0[0], tl0[1], tl0[2], rden0)
                                 : att_div_small(acc[dn][0][i], acc[dn][1][i], acc[dn][2][i], tl1[0], tl1[1], tl1[2], rden1);
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++)
                    o[i] = clip8(att_div(acc[dn][0][i], acc[dn][1][i], acc[dn][2][i], i < 2 ? den0 : den1, i < 2 ? rden0 : rden1, false));
            }
            const int dim = dn * 8 + 2 * q;
            *reinterpret_cast<uint16_t *>(p.ao + (base + row0) * H + col0 + dim) = (uint16_t)((o[0] & 0xFF) | ((o[1] & 0xFF) << 8));
            *reinterpret_cast<uint16_t *>(p.ao + (base + row1) * H + col0 + dim) = (uint16_t)((o[2] & 0xFF) | ((o[3] & 0xFF) << 8));
            const int nb0 = nbo[dim], nb1 = nbo[dim + 1];
            dot0 += o[0] * nb0 + o[1] * nb1;
            dot1 += o[2] * nb0 + o[3] * nb1;
        }
        dot0 += __shfl_xor_sync(0xFFFFFFFFu, dot0, 1); dot0 += __shfl_xor_sync(0xFFFFFFFFu, dot0, 2);
        dot1 += __shfl_xor_sync(0xFFFFFFFFu, dot1, 1); dot1 += __shfl_xor_sync(0xFFFFFFFFu, dot1, 2);
        if (q == 0) {
            atomicAdd(&p.xbo[base + row0], dot0);
            atomicAdd(&p.xbo[base + row1], dot1);
        }
    }
}

static size_t attention_smem_bytes(int S) {
    int SP = (S + 31) & ~31;
    return (size_t)SP * ATT_KP + 64 * (size_t)(SP + 16) + 256 * 4;
}

int launch_attention(cudaStream_t st, const AttnParams &p) {
    size_t smem = attention_smem_bytes(p.seq_len);
    static size_t configured[EGG_MAX_DEVICES] = {};
    const int dev = current_device_slot();
    if (smem > configured[dev]) {
        EGG_CUDA(cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev] = smem;
    }
    int blocks = p.members * (p.H / 64);
    attention_kernel<<<blocks, 128, smem, st>>>(p);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// =========================================================================
// weights: packed [K/4][N][4] -> K-major shadow [N][K]
// =========================================================================
__global__ void unpack_transpose_kernel(const int32_t *packed, int8_t *shadow, int rows_k, int cols_n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t words = (int64_t)(rows_k >> 2) * cols_n;
    if (i >= words) return;
    // consecutive threads take consecutive k4 of one output column: 128-byte coalesced writes
    int k4 = (int)(i % (rows_k >> 2));
    int n = (int)(i / (rows_k >> 2));
    int32_t w = packed[(int64_t)k4 * cols_n + n];
    *reinterpret_cast<int32_t *>(shadow + (int64_t)n * rows_k + 4 * k4) = w;
}

int launch_unpack_transpose(cudaStream_t st, const int8_t *packed, int8_t *shadow, int rows_k, int cols_n) {
    int64_t words = (int64_t)(rows_k >> 2) * cols_n;
    unpack_transpose_kernel<<<(unsigned)((words + 255) / 256), 256, 0, st>>>(reinterpret_cast<const int32_t *>(packed), shadow, rows_k, cols_n);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// =========================================================================
// transform of each pair's input window (NTT_MODE 1..3; egg_ntt.cuh, called mgpu.cu:877-887): one block per pair,
// the window in shared memory.  Mode 1: Walsh-Hadamard butterflies (a, b) -> (a + b, a - b) over strides 1, 2, 4, ...
// Modes 2 / 3: values reduced mod p = 257 / 65537, bit-reversal, then log2(len) decimation-in-time stages whose
// twiddle is 3^(j * len / m) mod p -- the reference takes the root of the full-length transform whatever len is.
// Both members of a pair read the same window, so the coefficients are kept per pair.
// =========================================================================
__device__ __forceinline__ uint32_t fermat_pow3(uint32_t prime, int k) {
    k &= (int)(prime - 2);                 // prime - 1 is a power of two
    unsigned long long r = 1, b = 3;
    while (k > 0) {
        if (k & 1) r = r * b % prime;
        b = b * b % prime;
        k >>= 1;
    }
    return (uint32_t)r;
}

__global__ void __launch_bounds__(512) window_transform_kernel(const WindowParams p) {
    extern __shared__ int32_t s_win[];
    const int S = p.seq_len, tid = threadIdx.x;
    const int64_t pair = p.pair_base + blockIdx.x;
    const int64_t pos = p.use_same_data ? (p.start_idx % (p.data_len - S)) : ((p.start_idx + pair * p.data_stride) % (p.data_len - S));
    const uint32_t prime = p.mode == 2 ? 257u : 65537u;
    for (int i = tid; i < S; i += blockDim.x) {
        const uint32_t tok = p.tok_wide ? reinterpret_cast<const uint32_t *>(p.dataset)[pos + i] : (uint32_t)p.dataset[pos + i];
        s_win[i] = p.mode == 1 ? (int32_t)tok : (int32_t)(tok % prime);
    }
    __syncthreads();
    if (p.mode == 1) {
        for (int stride = 1; stride < S; stride <<= 1) {
            for (int t = tid; t < (S >> 1); t += blockDim.x) {
                const int base = (t / stride) * 2 * stride + (t % stride);
                const int32_t a = s_win[base], b = s_win[base + stride];
                s_win[base] = a + b; s_win[base + stride] = a - b;
            }
            __syncthreads();
        }
    } else {
        const int lg = 31 - __clz(S);
        for (int i = tid; i < S; i += blockDim.x) {
            const int rev = (int)(__brev((unsigned)i) >> (32 - lg));
            if (i < rev) { const int32_t t = s_win[i]; s_win[i] = s_win[rev]; s_win[rev] = t; }
        }
        __syncthreads();
        for (int s = 1; s <= lg; s++) {
            const int m2 = 1 << (s - 1), w_step = S >> s;
            for (int k = tid; k < (S >> 1); k += blockDim.x) {
                const int j = k & (m2 - 1), i1 = ((k >> (s - 1)) << s) + j, i2 = i1 + m2;
                const uint32_t wb = (uint32_t)((unsigned long long)fermat_pow3(prime, j * w_step) * (uint32_t)s_win[i2] % prime);
                const uint32_t a = (uint32_t)s_win[i1];
                s_win[i1] = (int32_t)((a + wb) % prime);
                s_win[i2] = (int32_t)((a + prime - wb) % prime);
            }
            __syncthreads();
        }
    }
    for (int i = tid; i < S; i += blockDim.x) p.coef[(int64_t)blockIdx.x * S + i] = s_win[i];
}
int launch_window_transform(cudaStream_t st, const WindowParams &p) {
    if (p.mode < 1 || p.mode > 3 || p.seq_len < 2 || (p.seq_len & (p.seq_len - 1)) || p.seq_len > 8192 || p.pairs <= 0) {
        set_error("window transform: mode %d, seq_len %d, %d pairs unsupported", p.mode, p.seq_len, p.pairs); return EGG_E_INVALID;
    }
    int threads = p.seq_len / 2 < 32 ? 32 : (p.seq_len / 2 > 512 ? 512 : p.seq_len / 2);
    window_transform_kernel<<<p.pairs, threads, (size_t)p.seq_len * sizeof(int32_t), st>>>(p);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// =========================================================================
// cross-entropy over stored logits: second pass of the head when the vocabulary is wider than one GEMM tile
// (mgpu.cu:985-1023).  One warp per row: Σ exp-table[max - logit] in 64 bits, the target's logit, then
// loss[member] += (log_sum >> 1) + max - target with log_sum = 16 * (floor(log2 Σ) - SOFTMAX_SCALE_BIT).
// =========================================================================
__global__ void __launch_bounds__(256) head_loss_kernel(const HeadLossParams p) {
    __shared__ int32_t s_exp[256];
    s_exp[threadIdx.x] = p.exp_lut[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= p.M) return;
    const int mem = fast_div(r, p.fd_seq), t = r - mem * p.seq_len;
    const int64_t pair = (p.pop_base + mem) >> 1;
    const int64_t pos = p.use_same_data ? (p.start_idx % (p.data_len - p.seq_len))
                                        : ((p.start_idx + pair * p.data_stride) % (p.data_len - p.seq_len));
    const uint32_t target = p.dataset[pos + t + 1];
    const int mx = p.rowmax[r];
    const int4 *row = reinterpret_cast<const int4 *>(p.logits + (int64_t)r * p.V);
    long long sum = 0;
    for (int c = lane; c < (p.V >> 2); c += 32) {
        const int4 l = __ldcs(row + c);            // read once
        sum += (long long)s_exp[min(255, mx - l.x)] + s_exp[min(255, mx - l.y)] + s_exp[min(255, mx - l.z)] + s_exp[min(255, mx - l.w)];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if (lane == 0) {
        const int tgt = target < (uint32_t)p.V ? p.logits[(int64_t)r * p.V + target] : 0;   // no column matches: s_target_logit stays 0
        long long log_sum = 0;
        if (sum > 0) log_sum = ((long long)(63 - __clzll(sum)) << 4) - ((long long)p.softmax_scale_bit << 4);   // shift ladder of mgpu.cu:1012-1019
        atomicAdd(&p.loss[mem], (int)((log_sum >> 1) + mx - tgt));
    }
}
int launch_head_loss(cudaStream_t st, const HeadLossParams &p_in) {
    HeadLossParams p = p_in;
    if (p.M <= 0 || p.V % 128 || p.V <= 0) { set_error("head loss: unsupported shape M=%d V=%d", p.M, p.V); return EGG_E_INVALID; }
    p.fd_seq = make_fastdiv(p.seq_len);
    head_loss_kernel<<<(p.M + 7) / 8, 256, 0, st>>>(p);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// =========================================================================
// fitness (mgpu.cu:1031-1036)
// =========================================================================
__global__ void fitness_kernel(const int32_t *loss, int32_t *fit, int pairs) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pairs) return;
    int32_t pz = loss[2 * i], n = loss[2 * i + 1];
    fit[i] = (pz < n) ? 1 : ((n < pz) ? -1 : 0);
}
int launch_fitness(cudaStream_t st, const int32_t *loss, int32_t *fit, int pairs) {
    fitness_kernel<<<(pairs + 255) / 256, 256, 0, st>>>(loss, fit, pairs);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// =========================================================================
// update operands: the two noise matrices of vote = Σ_p f_p a_p b_p^T, pair index contiguous
// =========================================================================
// The update kernels are bound by the integer pipe (half the rate of the multiply-add pipe): the single-field noise
// value's sign select and the seed additions are written as multiply-adds with run-time multipliers (constants would
// be folded back into integer-pipe instructions).  hash_mix(seed + idx * 0x9e3779b9) == hash_rng(seed, idx).
struct UpdMul { int one, two; };
static inline UpdMul make_upd_mul() { UpdMul m; m.one = 1; m.two = 2; return m; }
__device__ __forceinline__ uint32_t hash_mix(uint32_t x) {
    x ^= x >> 16; x *= 0x85ebca6bu;
    x ^= x >> 13; x *= 0xc2b2ae35u;
    x ^= x >> 16;
    return x;
}

constexpr int UPD_ROWS_PER_BLOCK = 8;     // operand rows one block writes: the pair seeds and fitness words are loaded once for all of them

template <bool GAUSS>
__global__ void __launch_bounds__(256) update_operands_kernel(int8_t *na, int8_t *nb, const int32_t *fit, int pairs, int kp, int rows_k, int cols_n,
                                       int off_a, int off_b, int seed_base, uint32_t step_seed, int mask, int split, const UpdMul um) {
    const int row0 = blockIdx.y * UPD_ROWS_PER_BLOCK;      // 0..cols_n-1 -> NA, cols_n.. -> NB (cols_n is a multiple of the group size)
    const int ktot = split ? 2 * kp : kp;
    const bool is_a = row0 < cols_n;
    // four consecutive pair slots per thread (kp is a multiple of 128): one word store per row
    for (int pp = (blockIdx.x * blockDim.x + threadIdx.x) * 4; pp < ktot; pp += gridDim.x * blockDim.x * 4) {
        const int hi = pp >= kp;
        const int pidx0 = hi ? pp - kp : pp;
        uint32_t seed[4];
        int f[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int pidx = pidx0 + j;
            seed[j] = step_seed + (uint32_t)pidx + (uint32_t)seed_base + (uint32_t)(is_a ? off_a : off_b);    // mgpu.cu:1095
            int fv = 0;
            if (pidx < pairs) {
                fv = is_a ? fit[pidx] : (hi ? 16 : 1);
                if (is_a && split) { const int f1 = fv >> 4, f0 = fv - (f1 << 4); fv = hi ? f1 : f0; }
            }
            f[j] = fv;                                    // 0 for the padding beyond the last pair
        }
#pragma unroll
        for (int rr = 0; rr < UPD_ROWS_PER_BLOCK; rr++) {
            const int row = row0 + rr;
            const uint32_t idx = (uint32_t)(is_a ? row : row - cols_n);
            int val[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (GAUSS) {
                    val[j] = f[j] * noise_from_hash(seed[j], idx, mask, 1);
                } else {
                    // f * noise_field(r, 0, 1, mask): magnitude (r >> 1) & mask, positive when bit 0 is set
                    const uint32_t r = hash_mix(seed[j] * (uint32_t)um.one + idx * 0x9e3779b9u);
                    val[j] = (f[j] * (int)((r >> 1) & (uint32_t)mask)) * ((int)(r & 1u) * um.two - 1);
                }
            }
            const uint32_t w = pack4(val[0], val[1], val[2], val[3]);
            if (is_a) *reinterpret_cast<uint32_t *>(na + (int64_t)row * ktot + pp) = w;
            else *reinterpret_cast<uint32_t *>(nb + (int64_t)(row - cols_n) * ktot + pp) = w;
        }
    }
}

int launch_update_operands(cudaStream_t st, int8_t *na, int8_t *nb, const int32_t *fit, int pairs, int kp, int rows_k,
                           int cols_n, int off_a, int off_b, int seed_base, uint32_t step_seed, int mask, int gaussian,
                           int split) {
    if (rows_k % UPD_ROWS_PER_BLOCK || cols_n % UPD_ROWS_PER_BLOCK) { set_error("update operand rows must come in groups of %d", UPD_ROWS_PER_BLOCK); return EGG_E_INVALID; }
    int ktot = split ? 2 * kp : kp;
    int gx = (ktot / 4 + 255) / 256; if (gx > 32) gx = 32;
    dim3 grid((unsigned)gx, (unsigned)((rows_k + cols_n) / UPD_ROWS_PER_BLOCK));
    if (gaussian) update_operands_kernel<true><<<grid, 256, 0, st>>>(na, nb, fit, pairs, kp, rows_k, cols_n, off_a, off_b, seed_base, step_seed, mask, split, make_upd_mul());
    else update_operands_kernel<false><<<grid, 256, 0, st>>>(na, nb, fit, pairs, kp, rows_k, cols_n, off_a, off_b, seed_base, step_seed, mask, split, make_upd_mul());
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

int vote_gemm_splits(int rows_k, int cols_n, int kp, int num_sms) {
    const int bn = (rows_k % 256 == 0) ? 256 : 128;
    const int tiles = ((cols_n + GEMM_BM - 1) / GEMM_BM) * (rows_k / bn);
    const int num_kb = (kp + GEMM_BK - 1) / GEMM_BK;
    int want = (2 * num_sms + tiles - 1) / tiles;
    if (want > num_kb) want = num_kb;
    if (want > 64) want = 64;
    if (want < 1) want = 1;
    const int kb_per = (num_kb + want - 1) / want;
    return (num_kb + kb_per - 1) / kb_per;
}

// =========================================================================
// optimiser step from the vote matrices: one thread per packed word (4 weights of one output column)
// =========================================================================
__device__ __forceinline__ int4 sum_votes(const VoteApplyParams &p, int64_t word) {
    int4 v = *reinterpret_cast<const int4 *>(p.votes + word * 4);
    for (int s = 1; s < p.nsplits; s++) {
        const int4 u = *reinterpret_cast<const int4 *>(p.votes + (int64_t)s * p.split_stride + word * 4);
        v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
    }
    return v;
}

__global__ void __launch_bounds__(256) adam_from_votes_kernel(const VoteApplyParams p) {
    const int64_t word = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t words = (int64_t)(p.rows_k >> 2) * p.cols_n;
    int changes = 0;
    if (word < words) {
        const int4 vt = sum_votes(p, word);
        const int vote[4] = {vt.x, vt.y, vt.z, vt.w};
        const int64_t idx = word * 4;
        const uint32_t wword = *reinterpret_cast<const uint32_t *>(p.w_packed + idx);
        float4 *st = reinterpret_cast<float4 *>(p.opt + idx * 3);
        const float4 s0 = st[0], s1 = st[1], s2 = st[2];
        float f[12] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w, s2.x, s2.y, s2.z, s2.w};
        uint32_t neww = 0;
        const int n = (int)(word % p.cols_n), k0 = (int)(word / p.cols_n) * 4;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int w = (int)(int8_t)(wword >> (8 * j));
            const float g = -(float)vote[j];
            const int ch = adam_apply(f[3 * j], f[3 * j + 1], f[3 * j + 2], w, g, p.lr, p.beta1, p.beta2, p.eps, p.wd);
            changes += ch;
            if (ch && p.ch_in) { p.ch_in[k0 + j] = 1; p.ch_out[n] = 1; }      // adam.cuh:77-83
            neww |= (uint32_t)(w & 0xFF) << (8 * j);
        }
        *reinterpret_cast<uint32_t *>(p.w_packed + idx) = neww;
        st[0] = make_float4(f[0], f[1], f[2], f[3]);
        st[1] = make_float4(f[4], f[5], f[6], f[7]);
        st[2] = make_float4(f[8], f[9], f[10], f[11]);
    }
    changes = warp_sum(changes);
    if ((threadIdx.x & 31) == 0 && changes > 0) atomicAdd(p.total_updates, (unsigned long long)changes);
}

__global__ void __launch_bounds__(256) muon_m_from_votes_kernel(const VoteApplyParams p) {
    const int64_t word = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t words = (int64_t)(p.rows_k >> 2) * p.cols_n;
    if (word >= words) return;
    const int4 vt = sum_votes(p, word);
    const int64_t idx = word * 4;
    float4 *st = reinterpret_cast<float4 *>(p.opt + idx * 2);
    float4 s0 = st[0], s1 = st[1];     // m0 acc0 m1 acc1 | m2 acc2 m3 acc3
    s0.x = __fmaf_rn(p.mu, s0.x, (float)vt.x);   // m = mu*m + vote, muon_internal.cuh:45-47
    s0.z = __fmaf_rn(p.mu, s0.z, (float)vt.y);
    s1.x = __fmaf_rn(p.mu, s1.x, (float)vt.z);
    s1.z = __fmaf_rn(p.mu, s1.z, (float)vt.w);
    st[0] = s0; st[1] = s1;
    const int n = (int)(word % p.cols_n);
    const int64_t k = (word / p.cols_n) * 4;
    p.m_rowmajor[k * p.cols_n + n] = s0.x;        // gather, muon_internal.cuh:53-74
    p.m_rowmajor[(k + 1) * p.cols_n + n] = s0.z;
    p.m_rowmajor[(k + 2) * p.cols_n + n] = s1.x;
    p.m_rowmajor[(k + 3) * p.cols_n + n] = s1.z;
}

int launch_adam_from_votes(cudaStream_t st, const VoteApplyParams &p) {
    const int64_t words = (int64_t)(p.rows_k >> 2) * p.cols_n;
    adam_from_votes_kernel<<<(unsigned)((words + 255) / 256), 256, 0, st>>>(p);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}
int launch_muon_m_from_votes(cudaStream_t st, const VoteApplyParams &p) {
    const int64_t words = (int64_t)(p.rows_k >> 2) * p.cols_n;
    muon_m_from_votes_kernel<<<(unsigned)((words + 255) / 256), 256, 0, st>>>(p);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// =========================================================================
// vector parameters (update_vector_adam_kernel, mgpu.cu:1114-1152): one block per element
// =========================================================================
template <bool FAST>
__global__ void __launch_bounds__(256) update_vector_kernel(const VecUpdParams p, const UpdMul um) {
    const int idx = blockIdx.x;
    int vote = 0;
    if (!FAST) {
#pragma unroll 4
        for (int pr = threadIdx.x; pr < p.pairs; pr += blockDim.x) {
            const int f = p.fit[pr];
            const uint32_t s = p.step_seed + (uint32_t)pr + (uint32_t)p.seed_base;
            vote += f * noise_from_hash(s + (uint32_t)p.off_a, (uint32_t)idx, p.mask, p.gaussian) *
                    noise_from_hash(s + (uint32_t)p.off_b, (uint32_t)idx, p.mask, p.gaussian);
        }
    } else {
        // f * na * nb with na, nb = ±((r >> 1) & mask), positive when bit 0 is set: the magnitudes are taken doubled
        // (r & (mask << 1), no shift; every term is then 4x and the thread's sum is divided exactly afterwards, with
        // |sum| < pairs/256 * 4 * 31^2 * |f| far inside int32), the sign of the product is + when the two bits agree.
        // No early-out on zero fitness: four pairs per trip keep eight independent hash chains in flight.
        const uint32_t base = p.step_seed + (uint32_t)p.seed_base + (uint32_t)idx * 0x9e3779b9u;
        const uint32_t ca = base + (uint32_t)p.off_a, cb = base + (uint32_t)p.off_b;
        const uint32_t m2 = (uint32_t)p.mask << 1;
        int vote4 = 0;
#pragma unroll 4
        for (int pr = threadIdx.x; pr < p.pairs; pr += blockDim.x) {
            const int f = p.fit[pr];
            const uint32_t ra = hash_mix((uint32_t)pr * (uint32_t)um.one + ca), rb = hash_mix((uint32_t)pr * (uint32_t)um.one + cb);
            const int mm = (int)(ra & m2) * (int)(rb & m2);
            const int sg = 1 - (int)((ra ^ rb) & 1u) * um.two;
            vote4 += (f * sg) * mm;
        }
        vote = vote4 >> 2;
    }
    __shared__ int s_part[8];
    vote = warp_sum(vote);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = vote;
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int i = 0; i < 8; i++) total += s_part[i];
        float m = p.opt[idx * 3], v = p.opt[idx * 3 + 1], acc = p.opt[idx * 3 + 2];
        int w = p.v[idx];
        int ch = adam_apply(m, v, acc, w, -(float)total, p.lr, p.beta1, p.beta2, p.eps, p.wd);
        p.opt[idx * 3] = m; p.opt[idx * 3 + 1] = v; p.opt[idx * 3 + 2] = acc;
        p.v[idx] = (int8_t)w;
        if (ch) { atomicAdd(p.total_updates, 1ull); if (p.changed) p.changed[idx] = 1; }
    }
}
int launch_update_vector(cudaStream_t st, const VecUpdParams &p) {
    // the single-field form sums 4x terms per thread: (pairs/256) * 4 * mask^2 * 127 must stay inside int32
    const bool fast = !p.gaussian && (int64_t)((p.pairs + 255) / 256) * 4 * p.mask * p.mask * 127 < (1ll << 31);
    if (fast) update_vector_kernel<true><<<p.len, 256, 0, st>>>(p, make_upd_mul());
    else update_vector_kernel<false><<<p.len, 256, 0, st>>>(p, make_upd_mul());
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// =========================================================================
// Muon: Frobenius normalise + 5 cubic Newton–Schulz steps in fp32 (muon_internal.cuh:182-342)
// =========================================================================
__global__ void sumsq_kernel(const float *x, int64_t n, double *out) {
    // double accumulation: the result feeds one fp32 division per element
    double s = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) s += (double)x[i] * x[i];
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
    __shared__ double part[8];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += part[i];
        atomicAdd(out, t);
    }
}
__global__ void scale_by_norm_kernel(float *x, int64_t n, const double *sumsq) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float norm = (float)sqrt(*sumsq);
    if (norm > 1e-6f) x[i] /= norm;          // muon_scale_by_norm_kernel, muon_internal.cuh:77-85
}

// C[i][j] = alpha * Σ_t A(i,t) B(t,j), strided operands, optional "3I - C" epilogue.
// 64x64 tile, 16-deep steps, 256 threads x (4x4) outputs, plain FFMA.
__global__ void __launch_bounds__(256) sgemm_strided_kernel(const float *A, int64_t as0, int64_t as1, const float *B, int64_t bs0,
                                                            int64_t bs1, float *C, int Mm, int Nn, int Kk, float alpha, int three_i_minus) {
    __shared__ float sa[16][64 + 4], sb[16][64 + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int i0 = blockIdx.y * 64, j0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int t0 = 0; t0 < Kk; t0 += 16) {
        for (int e = threadIdx.x; e < 64 * 16; e += 256) {
            int a_i, a_t, b_t, b_j;
            if (as1 == 1) { a_t = e & 15; a_i = e >> 4; } else { a_i = e & 63; a_t = e >> 6; }
            if (bs1 == 1) { b_j = e & 63; b_t = e >> 6; } else { b_t = e & 15; b_j = e >> 4; }
            int gi = i0 + a_i, gt = t0 + a_t;
            sa[a_t][a_i] = (gi < Mm && gt < Kk) ? A[gi * as0 + gt * as1] : 0.0f;
            int gj = j0 + b_j, gt2 = t0 + b_t;
            sb[b_t][b_j] = (gj < Nn && gt2 < Kk) ? B[gt2 * bs0 + gj * bs1] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int t = 0; t < 16; t++) {
            float a[4], b[4];
#pragma unroll
            for (int u = 0; u < 4; u++) { a[u] = sa[t][ty * 4 + u]; b[u] = sb[t][tx * 4 + u]; }
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int w = 0; w < 4; w++) acc[u][w] = fmaf(a[u], b[w], acc[u][w]);
        }
        __syncthreads();
    }
    for (int u = 0; u < 4; u++)
        for (int w = 0; w < 4; w++) {
            int i = i0 + ty * 4 + u, j = j0 + tx * 4 + w;
            if (i < Mm && j < Nn) {
                float val = alpha * acc[u][w];
                if (three_i_minus) val = (i == j) ? 3.0f - val : -val;     // muon_newton_schulz_term_kernel, :91-109
                C[(int64_t)i * Nn + j] = val;
            }
        }
}

// The same product for shapes that are multiples of 128 (every Muon matrix is): 128 x 128 tile, 16-deep steps, 256 threads
// x (8 x 8) outputs, operands staged k-major in shared memory so that both micro-tile reads are 128-bit, the next step's
// global loads in flight while the current one is multiplied.  Each output keeps ONE accumulator fed in ascending t by
// fused multiply-adds, exactly as sgemm_strided_kernel does: the two kernels give identical bits.
// a_kc / b_kc: the operand's contraction index is the contiguous one in memory (else its row / column index is).
template <bool A_KC, bool B_KC>
__global__ void __launch_bounds__(256, 2) sgemm128_kernel(const float *__restrict__ A, int64_t lda, const float *__restrict__ B, int64_t ldb,
                                                       float *__restrict__ C, int Nn, int Kk, float alpha, int three_i_minus) {
    __shared__ __align__(16) float sa[2][16][128 + 4], sb[2][16][128 + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int i0 = blockIdx.y * 128, j0 = blockIdx.x * 128;
    float acc[8][8];
#pragma unroll
    for (int u = 0; u < 8; u++)
#pragma unroll
        for (int w = 0; w < 8; w++) acc[u][w] = 0.0f;
    // each thread moves two float4 per operand and step
    float4 ra[2], rb[2];
    auto gload = [&](int t0) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int e = tid + h * 256;                    // 0..511
            if (A_KC) { const int i = e >> 2, t4 = (e & 3) * 4; ra[h] = *reinterpret_cast<const float4 *>(A + (int64_t)(i0 + i) * lda + t0 + t4); }
            else { const int t = e >> 5, i4 = (e & 31) * 4; ra[h] = *reinterpret_cast<const float4 *>(A + (int64_t)(t0 + t) * lda + i0 + i4); }
            if (B_KC) { const int j = e >> 2, t4 = (e & 3) * 4; rb[h] = *reinterpret_cast<const float4 *>(B + (int64_t)(j0 + j) * ldb + t0 + t4); }
            else { const int t = e >> 5, j4 = (e & 31) * 4; rb[h] = *reinterpret_cast<const float4 *>(B + (int64_t)(t0 + t) * ldb + j0 + j4); }
        }
    };
    auto sstore = [&](int buf) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int e = tid + h * 256;
            if (A_KC) { const int i = e >> 2, t4 = (e & 3) * 4; sa[buf][t4][i] = ra[h].x; sa[buf][t4 + 1][i] = ra[h].y; sa[buf][t4 + 2][i] = ra[h].z; sa[buf][t4 + 3][i] = ra[h].w; }
            else { const int t = e >> 5, i4 = (e & 31) * 4; *reinterpret_cast<float4 *>(&sa[buf][t][i4]) = ra[h]; }
            if (B_KC) { const int j = e >> 2, t4 = (e & 3) * 4; sb[buf][t4][j] = rb[h].x; sb[buf][t4 + 1][j] = rb[h].y; sb[buf][t4 + 2][j] = rb[h].z; sb[buf][t4 + 3][j] = rb[h].w; }
            else { const int t = e >> 5, j4 = (e & 31) * 4; *reinterpret_cast<float4 *>(&sb[buf][t][j4]) = rb[h]; }
        }
    };
    gload(0);
    sstore(0);
    __syncthreads();
    int buf = 0;
    for (int t0 = 0; t0 < Kk; t0 += 16) {
        if (t0 + 16 < Kk) gload(t0 + 16);
#pragma unroll
        for (int t = 0; t < 16; t++) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&sa[buf][t][ty * 8]), a1 = *reinterpret_cast<const float4 *>(&sa[buf][t][ty * 8 + 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&sb[buf][t][tx * 8]), b1 = *reinterpret_cast<const float4 *>(&sb[buf][t][tx * 8 + 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int u = 0; u < 8; u++)
#pragma unroll
                for (int w = 0; w < 8; w++) acc[u][w] = fmaf(a[u], b[w], acc[u][w]);
        }
        if (t0 + 16 < Kk) {
            sstore(buf ^ 1);
            __syncthreads();
            buf ^= 1;
        }
    }
#pragma unroll
    for (int u = 0; u < 8; u++) {
        const int i = i0 + ty * 8 + u;
        float o[8];
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const int j = j0 + tx * 8 + w;
            float val = alpha * acc[u][w];
            if (three_i_minus) val = (i == j) ? 3.0f - val : -val;     // muon_newton_schulz_term_kernel, muon_internal.cuh:91-109
            o[w] = val;
        }
        *reinterpret_cast<float4 *>(C + (int64_t)i * Nn + j0 + tx * 8) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4 *>(C + (int64_t)i * Nn + j0 + tx * 8 + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
}

int launch_newton_schulz(cudaStream_t st, const MuonWs &ws, int rows, int cols) {
    const int64_t n = (int64_t)rows * cols;
    const bool use_rows = rows < cols;
    const int K = use_rows ? rows : cols;
    EGG_CUDA(cudaMemsetAsync(ws.norm2, 0, sizeof(double), st));
    sumsq_kernel<<<256, 256, 0, st>>>(ws.x, n, ws.norm2);
    scale_by_norm_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ws.x, n, ws.norm2);
    float *x = ws.x, *y = ws.y;
    // 128 x 128 tiles for every Muon matrix of a valid configuration; the 64 x 64 kernel is the fallback for other shapes.
    // (Measured: switching the 1024-wide products of the d-eggs shapes, 64 big tiles on 148 SMs, to 256 small tiles made
    // the update 7 % slower.)  Both kernels feed every output's single accumulator in ascending contraction order.
    const bool mult128 = rows % 128 == 0 && cols % 128 == 0;
    const bool big_g = mult128, big_y = mult128;
    for (int it = 0; it < 5; it++) {
        if (big_g) {
            dim3 gg(K / 128, K / 128);
            if (use_rows) sgemm128_kernel<true, true><<<gg, 256, 0, st>>>(x, cols, x, cols, ws.g, K, cols, 1.0f, 1);     // G = X X^T : A(i,t)=X[i][t], B(t,j)=X[j][t]
            else sgemm128_kernel<false, false><<<gg, 256, 0, st>>>(x, cols, x, cols, ws.g, K, rows, 1.0f, 1);          // G = X^T X : A(i,t)=X[t][i], B(t,j)=X[t][j]
        } else {
            dim3 gg((K + 63) / 64, (K + 63) / 64);
            if (use_rows) sgemm_strided_kernel<<<gg, 256, 0, st>>>(x, cols, 1, x, 1, cols, ws.g, K, K, cols, 1.0f, 1);
            else sgemm_strided_kernel<<<gg, 256, 0, st>>>(x, 1, cols, x, cols, 1, ws.g, K, K, rows, 1.0f, 1);
        }
        if (big_y) {
            dim3 gy(cols / 128, rows / 128);
            if (use_rows) sgemm128_kernel<true, false><<<gy, 256, 0, st>>>(ws.g, K, x, cols, y, cols, K, 0.5f, 0);       // Y = 0.5 * G' X
            else sgemm128_kernel<true, false><<<gy, 256, 0, st>>>(x, cols, ws.g, K, y, cols, K, 0.5f, 0);              // Y = 0.5 * X G'
        } else {
            dim3 gy((cols + 63) / 64, (rows + 63) / 64);
            if (use_rows) sgemm_strided_kernel<<<gy, 256, 0, st>>>(ws.g, K, 1, x, cols, 1, y, rows, cols, K, 0.5f, 0);
            else sgemm_strided_kernel<<<gy, 256, 0, st>>>(x, cols, 1, ws.g, K, 1, y, rows, cols, K, 0.5f, 0);
        }
        float *tmp = x; x = y; y = tmp;
    }
    // five swaps: the result lives in ws.y; copy back so callers always read ws.x
    EGG_CUDA(cudaMemcpyAsync(ws.x, x, n * sizeof(float), cudaMemcpyDeviceToDevice, st));
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

// muon_apply_update_kernel (muon_internal.cuh:112-166)
__global__ void muon_apply_kernel(int8_t *w_packed, float *opt, const float *upd, int rows_k, int cols_n, float lr, float wd,
                                  unsigned long long *total_updates) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int change = 0;
    if (idx < (int64_t)rows_k * cols_n) {
        int byte_off = (int)(idx & 3);
        int64_t word = idx >> 2;
        int n = (int)(word % cols_n), k = (int)(word / cols_n) * 4 + byte_off;
        int8_t w = w_packed[idx];
        float acc = opt[idx * 2 + 1];
        float u = upd[(int64_t)k * cols_n + n];
        int wi = w;
        acc = __fmaf_rn(-lr, __fmaf_rn(wd, (float)wi, u), acc);     // acc += -lr*(u + wd*w), contracted as nvcc does
        change = quantized_step(acc, wi);
        w = (int8_t)wi;
        w_packed[idx] = w;
        opt[idx * 2 + 1] = acc;
    }
    unsigned ballot = __ballot_sync(0xFFFFFFFFu, change);
    if ((threadIdx.x & 31) == 0 && ballot) atomicAdd(total_updates, (unsigned long long)__popc(ballot));
}
int launch_muon_apply(cudaStream_t st, int8_t *w_packed, float *opt, const float *upd_rowmajor, int rows_k, int cols_n,
                      float lr, float wd, unsigned long long *total_updates) {
    int64_t n = (int64_t)rows_k * cols_n;
    muon_apply_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(w_packed, opt, upd_rowmajor, rows_k, cols_n, lr, wd, total_updates);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

}  // namespace egg
