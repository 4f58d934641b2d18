// Persistent, warp-specialised int8 GEMM for sm_100a:
//   D[M,N] (int32, TMEM) = A[M,K] (int8, K-major) x B[N,K]^T (int8, K-major)
// TMA (128-byte swizzle) -> 4-stage shared-memory ring -> tcgen05.mma kind::i8 ->
// two TMEM accumulator stages -> 8 epilogue warps.  The epilogue is where the
// EGGROLL arithmetic lives: the per-member rank-1 term
//   acc += ((x·b_p) * a_p[n] * sign) >> (FIXED_POINT + SIGMA_SHIFT)
// (compute_linear_projection, mgpu.cu:553-572) and the call-site specific
// requantisation (mgpu.cu:729-756, 779-784, 829-830, 975-1023) or, for the
// update GEMM, the ES-AdamW / Muon-momentum step (mgpu.cu:1040-1111,
// muon_internal.cuh:15-50).
#pragma once

#include "egg_common.cuh"
#include "egg_ptx.cuh"

// Additions of the evaluation epilogues issued as multiply-adds (define EGG_PLAIN_ADDS to compare against plain adds).
#ifdef EGG_PLAIN_ADDS
#define GEMM_FMA_ADDS 0
#else
#define GEMM_FMA_ADDS 1
#endif

namespace egg {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 128;            // bytes (= int8 elements) per k-block: one swizzle row
constexpr int GEMM_STAGES = 3;
constexpr int GEMM_THREADS = 576;       // warp0 TMA, warp1 MMA, warps 2..17 epilogue
constexpr int GEMM_EPI_THREADS = 512;
constexpr int GEMM_EPI_WARPS = 16;
constexpr int GEMM_MAX_SLOTS = 5;       // distinct population pairs a 128-row tile can touch (seq_len >= 16)
constexpr int GEMM_RPL_SLOTS = 3;       // the same bound for the row-per-lane epilogues (seq_len a multiple of 32)

enum GemmEpi {
    EPI_CLIP8 = 0,   // y = clip((acc + r1) >> out_shift)                       -> int8
    EPI_GELU = 1,    // u = GELU[(u8)clip(((acc+r1)>>s) + b + vn)]              -> int8, Σ u·noise -> xb2
    EPI_PRE32 = 2,   // pre = resid + ((acc+r1)>>s) + b + vn                    -> int32 + row abs-max
    EPI_QKV = 3,     // rope(acc + r1) for q,k ; acc + r1 for v                 -> int32 + row abs-max per q/k/v
    EPI_HEAD = 4,    // logits = (acc+r1)>>s ; integer cross-entropy            -> loss[member] +=
    EPI_LOGITS = 5,  // logits = (acc+r1)>>s                                    -> int32 + row max (vocabularies wider than one tile)
    EPI_VOTE = 7,    // vote tile -> int32 votes in packed index order; with k_splits > 1 every split of the contraction
                     // writes its own partial vote matrix (integer sums: any split adds up exactly)
    EPI_NULL = 8,    // accumulators are dropped: the loop of TMA loads and tcgen05 MMAs alone (peak measurement)
};

struct GemmParams {
    int M, N, K;
    // ---- row -> member mapping (evaluation epilogues) ----
    int seq_len;                 // rows per member
    const int8_t *nt;            // per-pair noise table of this wave
    int64_t nt_stride;           // bytes per pair
    int nt_a_off;                // A-noise vector (length N) of this projection
    int nt_c_off;                // bias-noise deltas [2][N] (-1: none)
    int nt_d_off;                // B-noise vector of the NEXT projection (EPI_GELU), length N
    const int32_t *xb;           // Σ_k x_k b_k per row: xb[r*xb_stride + xb_col(+n0/third)]
    int xb_stride;
    int rank1_shift;
    int out_shift;
    const int8_t *bias;          // [N] or null
    // outputs
    int8_t *out8;                // [M,N]
    int32_t *out32;              // [M,N]
    int32_t *rowstat;            // EPI_GELU: xb2[M] (+=); EPI_PRE32: rowmax[M]; EPI_QKV: rowmax[M][3]; EPI_LOGITS: signed row max[M] (max=)
    const int8_t *resid;         // [M,N] int8 (EPI_PRE32)
    const int8_t *act_lut;       // 256
    const int32_t *exp_lut;      // 256
    const int32_t *rope_lut;     // [seq_len][head_dim]
    const int2 *rope_t;          // [head_dim/2][seq_len] (cos, sin): the same values, token index fastest
    int third;                   // EPI_QKV: N/3 (= hidden)
    int head_dim;
    int rope_bit;                // ROPE_SCALE_BIT
    // EPI_HEAD
    const uint8_t *dataset;
    int64_t data_len, start_idx, data_stride;   // data_stride = data_len / (POP/2)
    int pop_base;                // global index of member 0 of this wave
    int use_same_data;
    int softmax_scale_bit;
    int32_t *loss;               // [wave members] +=
    // ---- vote epilogue: GEMM M = cols_n (output dim), GEMM N = rows_k (input dim), K = pairs ----
    int32_t *vote_out;           // [k_splits][rows_k * cols_n] in packed index order
    int k_splits;                // parts the contraction is cut into (0 or 1: none)
    int64_t split_stride;        // elements between the partial vote matrices
    // ---- device error record ----
    int *err;
    int rpl;                     // -1 forces the transposed evaluation epilogue (tests); otherwise chosen from seq_len
    // divisors of the per-tile index arithmetic (filled by launch_gemm)
    FastDiv fd_seq, fd_tiles_n, fd_third, fd_head;
    int lut_stride;              // bytes between entries of the replicated GELU table (filled by launch_gemm)
    int one;                     // 1 (filled by launch_gemm): the multiplier of additions issued as multiply-adds
    int pow_t;                   // EPI_GELU: 2^rank1_shift when both shifts may be merged into one (0: keep two shifts)
};

template <int BN>
struct GemmSmem {
    alignas(1024) uint8_t a[GEMM_STAGES][GEMM_BM * GEMM_BK];
    alignas(1024) uint8_t b[GEMM_STAGES][BN * GEMM_BK];
    union {
        alignas(1024) int32_t stage[GEMM_EPI_WARPS][32][20];   // transposed epilogues, per warp: 32 rows x 16 columns (+4 pad) transpose buffer
        struct {
            // row-per-lane outputs: dense 32 x 16-word box per warp (64-byte swizzle), the source of a TMA store.  The
            // int32 epilogues alternate between two boxes so that one store can drain while the next chunk is written;
            // the GELU epilogue needs one box per tile and keeps its lookup table where the second boxes would be.
            alignas(1024) int32_t ostage0[GEMM_EPI_WARPS][32 * 16];
            union {
                alignas(1024) int32_t ostage1[GEMM_EPI_WARPS][32 * 16];
                // GELU table for the row-per-lane epilogue: every lane looks up its own row's value, so a single 256-byte
                // table would serialise on bank conflicts; 32 word-wide copies (exactly the space of the second boxes) give
                // lane l its own bank whatever the indices are
                alignas(16) uint32_t lut32[256][32];
            };
        };
    };
    union {
        struct {                                            // transposed epilogues: compact tables
            alignas(16) int8_t a_tab[GEMM_MAX_SLOTS][BN];       // A-noise of this projection per pair slot
            alignas(16) int16_t bc_tab[GEMM_MAX_SLOTS][2][BN];  // bias + bias-noise delta per pair slot and sign
        };
        struct {                                            // row-per-lane epilogues: tables widened to int32, read as uniform LDS.128
            alignas(16) int32_t a32[GEMM_RPL_SLOTS][BN];        // A-noise of this projection per pair slot
            alignas(16) int32_t bcs32[GEMM_RPL_SLOTS][2][BN];   // (bias + bias-noise delta) << out_shift per pair slot and sign
        } rpl;
    };
    alignas(16) int8_t d_tab[GEMM_MAX_SLOTS][BN];       // B-noise of the next projection (EPI_GELU)
    alignas(16) int32_t rowpart[4][GEMM_BM];            // row-per-lane epilogues: per-row partial of each column quarter
    alignas(16) int8_t act_lut[256];
    alignas(16) int32_t exp_lut[256];
    alignas(8) uint64_t full[GEMM_STAGES];
    uint64_t empty[GEMM_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t rbar[GEMM_EPI_WARPS];      // per epilogue warp: arrival of its residual box (EPI_PRE32, row-per-lane, BN = 256)
    uint32_t tmem_base;
    volatile int abort_flag;
    volatile int epi_ok;
};

__device__ __forceinline__ void gemm_fail(const GemmParams &p, volatile int *abort_flag, int code) {
    *abort_flag = 1;
    if (p.err) { atomicCAS(p.err, 0, code); }
}

// AdamW element step (apply_adam_update, mgpu.cu:1040-1064).  The reference is built
// with nvcc's default -fmad=true; which multiply-adds it contracts was measured by
// running its kernels on a B200 and is written out here with explicit single-rounding
// intrinsics so that the result does not depend on this compiler's own choices:
//   m   = fma(b1, m, (1-b1)*g)          v     = fma(1-b2, g*g, b2*v)
//   in  = fma(wd, w, m/(sqrt(v)+eps))   acc   = fma(-lr, in, acc)
__device__ __forceinline__ int quantized_step(float &acc, int &w) {
    if (acc >= 1.0f) {
        if (w < 127) { w++; acc = __fadd_rn(acc, -1.0f); return 1; }
        acc = 1.0f;
    } else if (acc <= -1.0f) {
        if (w > -127) { w--; acc = __fadd_rn(acc, 1.0f); return 1; }
        acc = -1.0f;
    }
    return 0;
}
__device__ __forceinline__ int adam_apply(float &m, float &v, float &acc, int &w, float g, float lr, float b1, float b2,
                                          float eps, float wd) {
    const float omb1 = __fadd_rn(1.0f, -b1), omb2 = __fadd_rn(1.0f, -b2);
    m = __fmaf_rn(b1, m, __fmul_rn(omb1, g));
    v = __fmaf_rn(omb2, __fmul_rn(g, g), __fmul_rn(b2, v));
    const float inner = __fmaf_rn(wd, (float)w, __fdiv_rn(m, __fadd_rn(__fsqrt_rn(v), eps)));
    acc = __fmaf_rn(-lr, inner, acc);
    return quantized_step(acc, w);
}

// ---- per-tile epilogue tables ----
// One work item = 4 consecutive columns of one pair slot; GEMM_MAX_SLOTS * BN / 4 <= GEMM_EPI_THREADS, so a thread has at
// most one.  Split into the global loads and the shared-memory stores so that the loads of the NEXT tile can be in
// flight while the current one is computed.
struct TabWords { int32_t a, b, cp, cn, d; };

template <int BN, int EPI>
__device__ __forceinline__ bool tab_load(const GemmParams &p, int e, int m0, int n0, TabWords &w) {
    const int last_row = min(m0 + GEMM_BM, p.M) - 1;
    const int first_pl = fast_div(m0, p.fd_seq) >> 1;
    const int nslots = (fast_div(last_row, p.fd_seq) >> 1) - first_pl + 1;
    if (e >= nslots * (BN / 4)) return false;
    const int sl = e / (BN / 4), j = (e % (BN / 4)) * 4;
    const int8_t *base = p.nt + (int64_t)(first_pl + sl) * p.nt_stride;
    w.a = *reinterpret_cast<const int32_t *>(base + p.nt_a_off + n0 + j);
    w.b = 0; w.cp = 0; w.cn = 0; w.d = 0;
    if (EPI == EPI_GELU || EPI == EPI_PRE32) {
        if (p.bias) w.b = *reinterpret_cast<const int32_t *>(p.bias + n0 + j);
        if (p.nt_c_off >= 0) {
            w.cp = *reinterpret_cast<const int32_t *>(base + p.nt_c_off + n0 + j);
            w.cn = *reinterpret_cast<const int32_t *>(base + p.nt_c_off + p.N + n0 + j);
        }
    }
    if (EPI == EPI_GELU) w.d = *reinterpret_cast<const int32_t *>(base + p.nt_d_off + n0 + j);
    return true;
}

template <int BN, int EPI, int RPL>
__device__ __forceinline__ void tab_store(const GemmParams &p, GemmSmem<BN> &sm, int e, const TabWords &w) {
    const int sl = e / (BN / 4), j = (e % (BN / 4)) * 4;
    if (RPL) *reinterpret_cast<int4 *>(&sm.rpl.a32[sl][j]) = make_int4((int)(int8_t)w.a, (int)(int8_t)(w.a >> 8), (int)(int8_t)(w.a >> 16), w.a >> 24);
    else *reinterpret_cast<int32_t *>(&sm.a_tab[sl][j]) = w.a;
    if ((EPI == EPI_GELU || EPI == EPI_PRE32) && RPL) {
        int vp[4], vn[4];
        // GELU: shifted once more so that the sum joins the rank-1 product before its shift (see epilogue_rpl)
        const int tsh = p.out_shift + ((EPI == EPI_GELU && GEMM_FMA_ADDS) ? p.rank1_shift : 0);
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int bb = (int)(int8_t)(w.b >> (8 * b));
            vp[b] = (bb + (int)(int8_t)(w.cp >> (8 * b))) << tsh;
            vn[b] = (bb + (int)(int8_t)(w.cn >> (8 * b))) << tsh;
        }
        *reinterpret_cast<int4 *>(&sm.rpl.bcs32[sl][0][j]) = make_int4(vp[0], vp[1], vp[2], vp[3]);
        *reinterpret_cast<int4 *>(&sm.rpl.bcs32[sl][1][j]) = make_int4(vn[0], vn[1], vn[2], vn[3]);
    } else if (EPI == EPI_GELU || EPI == EPI_PRE32) {
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int bb = (int)(int8_t)(w.b >> (8 * b));
            {
                sm.bc_tab[sl][0][j + b] = (int16_t)(bb + (int)(int8_t)(w.cp >> (8 * b)));
                sm.bc_tab[sl][1][j + b] = (int16_t)(bb + (int)(int8_t)(w.cn >> (8 * b)));
            }
        }
    }
    if (EPI == EPI_GELU) *reinterpret_cast<int32_t *>(&sm.d_tab[sl][j]) = w.d;
}

// ---- row-per-lane evaluation epilogues ----
// Used when every warp's 32 accumulator rows belong to one population member (seq_len % 32 == 0): the rank-1 factor,
// pair slot and sign are then per-lane scalars and the per-column tables are read at warp-uniform addresses, so the
// accumulators are consumed straight from the TMEM layout (lane = row, registers = columns) with no transpose, no
// shuffles and about half the instructions of the transposed form.  TMEM loads are double-buffered.
template <int BN, int EPI, bool ROPE, bool RES_TMA>
__device__ __forceinline__ void epilogue_rpl(const GemmParams &p, GemmSmem<BN> &sm, uint32_t taddr, int r, bool row_ok, int n0,
                                             int cbase, int slot, int sgn, int32_t (*st)[20], int lane, int m0q, int xbs,
                                             const int4 (&rs_pre)[BN / 4 / 16], const CUtensorMap *tmap_o, int32_t *ost, int32_t *ost1) {
    constexpr int NCH = BN / 4 / 16;                       // 16-column chunks of this warp's quarter of the tile
    const int rc = row_ok ? r : (p.M - 1);
    const int mem = fast_div(rc, p.fd_seq);
    const uint32_t lut_base = ptx::smem_u32(&sm.lut32[0][lane]);
    const uint32_t lut_stride = (uint32_t)p.lut_stride;       // 128 bytes per table entry, read from the parameters
    const uint32_t a32 = ptx::smem_u32(sm.rpl.a32[slot] + cbase);           // 32-bit shared addresses of this lane's tables
    const uint32_t bcs = ptx::smem_u32(sm.rpl.bcs32[slot][sgn] + cbase);
    const uint32_t ost_s = ptx::smem_u32(ost) + lane * 64;
    const uint32_t ost1_s = ptx::smem_u32(ost1) + lane * 64;
    const int8_t *dt = sm.d_tab[slot] + cbase;
    const int2 *rope = p.rope_t + (rc - mem * p.seq_len);                                // column of this token position
    constexpr bool do_rope = (EPI == EPI_QKV) && ROPE;      // Q and K column tiles; V passes through
    const long long half_ulp = 1ll << (p.rope_bit - 1);
    int racc = 0, rmx = (EPI == EPI_LOGITS) ? INT_MIN : 0, rmn = 0;      // EPI_LOGITS: the signed row maximum
    uint32_t v[2][16];
    ptx::tmem_ld16(taddr, v[0]);
#pragma unroll
    for (int c = 0; c < NCH; c++) {
        int4 cs[4];
        if (EPI == EPI_QKV && do_rope) {
            // the lanes of a warp are consecutive tokens of one member: every load below is one contiguous run
            const int pair0 = fast_mod(n0 + cbase + 16 * c, p.fd_head) >> 1;
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
                const int2 c0 = __ldg(rope + (int64_t)(pair0 + 2 * q4) * p.seq_len), c1 = __ldg(rope + (int64_t)(pair0 + 2 * q4 + 1) * p.seq_len);
                cs[q4] = make_int4(c0.x, c0.y, c1.x, c1.y);
            }
        }
        uint32_t *vc = v[c & 1];
        ptx::tmem_ld_wait16(vc);
        if (c + 1 < NCH) ptx::tmem_ld16(taddr + 16 * (c + 1), v[(c + 1) & 1]);
        uint32_t outw[4];
        int4 o4[4];
        // residual bytes of this chunk: from the warp's box that the copy engine filled (same 64-byte swizzle as the
        // output boxes), or from the registers loaded with plain loads
        int4 rs4 = make_int4(0, 0, 0, 0);
        if (EPI == EPI_PRE32) rs4 = RES_TMA ? ptx::lds_v4(ost1_s + ((c ^ ((lane >> 1) & 3)) << 4)) : rs_pre[c];
#pragma unroll
        for (int q4 = 0; q4 < 4; q4++) {
            const int col = 16 * c + 4 * q4;
            const int4 an = ptx::lds_v4(a32 + 4 * col);
            int x0, x1, x2, x3;
            if (EPI == EPI_GELU && GEMM_FMA_ADDS) {
                // (((acc + r1) >> s) + b) with r1 = (xb*a) >> t  ==  (acc + ((xb*a + (b << (s+t))) >> t)) >> s.  The adds are issued
                // as multiply-adds (the bias joins the rank-1 product, the accumulator is added with a run-time multiplier
                // of 1): the integer pipe runs at half the rate of the multiply-add pipe and is the busy one here.
                const int4 b4 = ptx::lds_v4(bcs + 4 * col);
                uint32_t z;
                if (p.pow_t) {
                    // floor((acc + floor(y / 2^t)) / 2^s) == floor((acc * 2^t + y) / 2^(s+t)): one multiply-add and one shift per
                    // element; the launcher allows it only while acc * 2^t + y provably stays inside int32 (K <= 512 at t = 7)
                    const int sh2 = p.rank1_shift + p.out_shift;
                    x0 = (int)vc[4 * q4] * p.pow_t + (xbs * an.x + b4.x);
                    x1 = (int)vc[4 * q4 + 1] * p.pow_t + (xbs * an.y + b4.y);
                    x2 = (int)vc[4 * q4 + 2] * p.pow_t + (xbs * an.z + b4.z);
                    x3 = (int)vc[4 * q4 + 3] * p.pow_t + (xbs * an.w + b4.w);
                    z = ptx::pack_sat_s8(x0 >> sh2, x1 >> sh2, x2 >> sh2, x3 >> sh2);
                } else {
                    x0 = ((xbs * an.x + b4.x) >> p.rank1_shift) * p.one + (int)vc[4 * q4];
                    x1 = ((xbs * an.y + b4.y) >> p.rank1_shift) * p.one + (int)vc[4 * q4 + 1];
                    x2 = ((xbs * an.z + b4.z) >> p.rank1_shift) * p.one + (int)vc[4 * q4 + 2];
                    x3 = ((xbs * an.w + b4.w) >> p.rank1_shift) * p.one + (int)vc[4 * q4 + 3];
                    // saturate to [-128, 127] while packing; the table entry of -128 holds the value of -127 (the reference's clip)
                    z = ptx::pack_sat_s8(x0 >> p.out_shift, x1 >> p.out_shift, x2 >> p.out_shift, x3 >> p.out_shift);
                }
                // word (idx, lane) of the replicated table: 32-bit shared address = base + idx * 128, one dot-product
                // instruction per byte (the other three bytes meet a zero)
                const uint32_t u0 = ptx::lds_u32(__dp4a(z, lut_stride, lut_base)), u1 = ptx::lds_u32(__dp4a(z, lut_stride << 8, lut_base));
                const uint32_t u2 = ptx::lds_u32(__dp4a(z, lut_stride << 16, lut_base)), u3 = ptx::lds_u32(__dp4a(z, lut_stride << 24, lut_base));
                const uint32_t w = __byte_perm(__byte_perm(u0, u1, 0x0040), __byte_perm(u2, u3, 0x0040), 0x5410);
                racc = __dp4a((int)w, *reinterpret_cast<const int32_t *>(dt + col), racc);
                outw[q4] = w;
                continue;
            }
            x0 = (int)vc[4 * q4] + ((xbs * an.x) >> p.rank1_shift);
            x1 = (int)vc[4 * q4 + 1] + ((xbs * an.y) >> p.rank1_shift);
            x2 = (int)vc[4 * q4 + 2] + ((xbs * an.z) >> p.rank1_shift);
            x3 = (int)vc[4 * q4 + 3] + ((xbs * an.w) >> p.rank1_shift);
            if (EPI == EPI_GELU) {
                // ((acc + r1) >> s) + b  ==  (acc + r1 + (b << s)) >> s
                const int4 b4 = ptx::lds_v4(bcs + 4 * col);
                // saturate to [-128, 127] while packing; the table entry of -128 holds the value of -127 (the reference's clip)
                const uint32_t z = ptx::pack_sat_s8((x0 + b4.x) >> p.out_shift, (x1 + b4.y) >> p.out_shift, (x2 + b4.z) >> p.out_shift,
                                                    (x3 + b4.w) >> p.out_shift);
                // word (idx, lane) of the replicated table: 32-bit shared address = base + idx * 128
                const uint32_t u0 = ptx::lds_u32((z & 0xFFu) * lut_stride + lut_base), u1 = ptx::lds_u32(__byte_perm(z, 0, 0x4441) * lut_stride + lut_base);
                const uint32_t u2 = ptx::lds_u32(__byte_perm(z, 0, 0x4442) * lut_stride + lut_base), u3 = ptx::lds_u32((z >> 24) * lut_stride + lut_base);
                const uint32_t w = __byte_perm(__byte_perm(u0, u1, 0x0040), __byte_perm(u2, u3, 0x0040), 0x5410);
                racc = __dp4a((int)w, *reinterpret_cast<const int32_t *>(dt + col), racc);
                outw[q4] = w;
            } else if (EPI == EPI_PRE32) {
                const int4 b4 = ptx::lds_v4(bcs + 4 * col);
                const int32_t rs = q4 == 0 ? rs4.x : (q4 == 1 ? rs4.y : (q4 == 2 ? rs4.z : rs4.w));
                // residual bytes sign-extended by one byte permute each (selector msb = replicate the byte's sign)
                x0 = ptx::sx_byte0(rs) + ((x0 + b4.x) >> p.out_shift);
                x1 = ptx::sx_byte1(rs) + ((x1 + b4.y) >> p.out_shift);
                x2 = ptx::sx_byte2(rs) + ((x2 + b4.z) >> p.out_shift);
                x3 = (rs >> 24) + ((x3 + b4.w) >> p.out_shift);
                rmx = __vimax3_s32(__vimax3_s32(rmx, x0, x1), x2, x3);      // abs-max as max(max, -min): three-input min/max, no abs
                rmn = __vimin3_s32(__vimin3_s32(rmn, x0, x1), x2, x3);
                o4[q4] = make_int4(x0, x1, x2, x3);
            } else if (EPI == EPI_QKV) {
                if (do_rope) {
                    // integer RoPE on adjacent (even, odd) columns (apply_rope_integer, mgpu.cu:624-644)
                    // (e*c - o*s + half) >> bit and (e*s + o*c + half) >> bit: two wide multiply-adds and one funnel shift
                    // each (bits [bit, bit+32) of the 64-bit sum are what the cast of the shifted value keeps)
                    const int e0 = x0, o0 = x1, e1 = x2, o1 = x3;
                    x0 = ptx::shr64_lo(ptx::mad_wide(-o0, cs[q4].y, ptx::mad_wide(e0, cs[q4].x, half_ulp)), p.rope_bit);
                    x1 = ptx::shr64_lo(ptx::mad_wide(o0, cs[q4].x, ptx::mad_wide(e0, cs[q4].y, half_ulp)), p.rope_bit);
                    x2 = ptx::shr64_lo(ptx::mad_wide(-o1, cs[q4].w, ptx::mad_wide(e1, cs[q4].z, half_ulp)), p.rope_bit);
                    x3 = ptx::shr64_lo(ptx::mad_wide(o1, cs[q4].z, ptx::mad_wide(e1, cs[q4].w, half_ulp)), p.rope_bit);
                }
                rmx = __vimax3_s32(__vimax3_s32(rmx, x0, x1), x2, x3);
                rmn = __vimin3_s32(__vimin3_s32(rmn, x0, x1), x2, x3);
                o4[q4] = make_int4(x0, x1, x2, x3);
            } else if (EPI == EPI_LOGITS) {
                x0 >>= p.out_shift; x1 >>= p.out_shift; x2 >>= p.out_shift; x3 >>= p.out_shift;
                rmx = __vimax3_s32(__vimax3_s32(rmx, x0, x1), x2, x3);
                o4[q4] = make_int4(x0, x1, x2, x3);
            }
        }
        if (EPI == EPI_GELU) {
            if (NCH == 4) {
                // 64 output bytes per lane and tile: same dense swizzled box as below, one TMA store per warp and tile
                if (c == 0) {
                    if (lane == 0) ptx::tma_store_wait_read<0>();
                    __syncwarp();
                }
                ptx::sts_v4(ost_s + ((c ^ ((lane >> 1) & 3)) << 4), make_int4(outw[0], outw[1], outw[2], outw[3]));
            } else {
                *reinterpret_cast<int4 *>(&ost[lane * 16 + 4 * c]) = make_int4(outw[0], outw[1], outw[2], outw[3]);
            }
        }
        if (EPI == EPI_PRE32 || EPI == EPI_QKV || EPI == EPI_LOGITS) {
            // int32 results leave as one TMA store per warp and chunk: each lane writes its row's 64 bytes into a dense
            // 32 x 16 box (16-byte pieces XOR-swizzled with the row, the 64-byte pattern the tensor map expects, which
            // also makes the stores conflict-free); the copy engine does the coalescing and clips rows beyond M
            // QKV: chunks alternate between the warp's two boxes; before box c & 1 is rewritten only the store issued two
            // chunks ago (the same box) must have been read out, the previous one may still be draining (-3 % on that
            // projection).  The residual projections keep one box: with K = 2048 the copy engine and the shared-memory
            // port are the busy units, and a second store in flight made them 2.5 % slower on the same GPU.
            constexpr bool TWO_BOXES = (EPI == EPI_QKV || EPI == EPI_LOGITS);
            if (lane == 0) { if (TWO_BOXES) ptx::tma_store_wait_read<1>(); else ptx::tma_store_wait_read<0>(); }
            __syncwarp();
            const bool second = TWO_BOXES && (c & 1);
            const uint32_t ob_s = second ? ost1_s : ost_s;
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) ptx::sts_v4(ob_s + ((q4 ^ ((lane >> 1) & 3)) << 4), o4[q4]);
            ptx::fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                ptx::tma_store_2d(tmap_o, second ? ost1 : ost, n0 + cbase + 16 * c, m0q);
                ptx::tma_store_commit();
            }
        }
    }
    if (EPI == EPI_GELU && NCH == 4) {
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            ptx::tma_store_2d(tmap_o, ost, n0 + cbase, m0q);
            ptx::tma_store_commit();
        }
    } else if (EPI == EPI_GELU) {
        // the lane's 4*NCH packed words (its row's quarter of the tile) leave through the same transpose: one store
        // instruction then covers 8 rows x (BN/4) contiguous bytes
        __syncwarp();
        const int lrow = lane >> 2, pc = lane & 3;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int rr = m0q + i * 8 + lrow;
            int8_t *dst = p.out8 + (int64_t)rr * p.N + n0 + cbase + NCH * 4 * pc;
            if (NCH == 4) {
                const int4 o = *reinterpret_cast<const int4 *>(&ost[(i * 8 + lrow) * 16 + 4 * pc]);
                if (rr < p.M) *reinterpret_cast<int4 *>(dst) = o;
            } else {
                const int2 o = *reinterpret_cast<const int2 *>(&ost[(i * 8 + lrow) * 16 + 2 * pc]);
                if (rr < p.M) *reinterpret_cast<int2 *>(dst) = o;
            }
        }
        __syncwarp();
    }
    if (EPI == EPI_PRE32 || EPI == EPI_QKV) racc = max(rmx, -rmn);
    if (EPI == EPI_LOGITS) racc = rmx;
    // per-row partial of this column quarter; the quarters are combined after the end-of-tile barrier
    sm.rowpart[cbase / (BN / 4)][m0q + lane - (m0q & ~(GEMM_BM - 1))] = racc;
}

// Head + integer cross-entropy in the row-per-lane form (mgpu.cu:969-1023).  The four warps that share a TMEM lane
// quarter each take a quarter of the vocabulary columns of the same 32 rows: pass 0 finds the row maximum (partials
// exchanged through shared memory under a 128-thread named barrier), pass 1 re-reads the accumulators for
// Σ exp-LUT and the target logit, and the warp of the first column quarter adds one loss term per row, reduced over
// the warp (all its rows belong to one member) into a single atomic.
template <int BN>
__device__ __forceinline__ void epilogue_head_rpl(const GemmParams &p, GemmSmem<BN> &sm, uint32_t taddr, int r, bool row_ok, int cbase,
                                                  int slot, int lane, int quarter, int row_in_tile, int xbs) {
    constexpr int NCH = BN / 4 / 16;
    int32_t(*hp)[4][GEMM_BM] = reinterpret_cast<int32_t(*)[4][GEMM_BM]>(&sm.stage[0][0][0]);    // [max | sum | target][quarter][row]
    const int cq = cbase / (BN / 4);
    const int rc = row_ok ? r : (p.M - 1);
    const int mem = fast_div(rc, p.fd_seq);
    const int t = rc - mem * p.seq_len;
    const int64_t pair = (p.pop_base + mem) >> 1;
    const int64_t pos = p.use_same_data ? (p.start_idx % (p.data_len - p.seq_len)) : ((p.start_idx + pair * p.data_stride) % (p.data_len - p.seq_len));
    const int tgt_col = (int)p.dataset[pos + t + 1] - cbase;                    // target column relative to this warp's quarter
    const uint32_t a32 = ptx::smem_u32(sm.rpl.a32[slot] + cbase);
    uint32_t v[2][16];
    int mx = INT_MIN, sum = 0, tg = 0;
#pragma unroll 1
    for (int pass = 0; pass < 2; pass++) {
        ptx::tmem_ld16(taddr, v[0]);
#pragma unroll
        for (int c = 0; c < NCH; c++) {
            uint32_t *vc = v[c & 1];
            ptx::tmem_ld_wait16(vc);
            if (c + 1 < NCH) ptx::tmem_ld16(taddr + 16 * (c + 1), v[(c + 1) & 1]);
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
                const int col = 16 * c + 4 * q4;
                const int4 an = ptx::lds_v4(a32 + 4 * col);
                const int l0 = ((int)vc[4 * q4] + ((xbs * an.x) >> p.rank1_shift)) >> p.out_shift;
                const int l1 = ((int)vc[4 * q4 + 1] + ((xbs * an.y) >> p.rank1_shift)) >> p.out_shift;
                const int l2 = ((int)vc[4 * q4 + 2] + ((xbs * an.z) >> p.rank1_shift)) >> p.out_shift;
                const int l3 = ((int)vc[4 * q4 + 3] + ((xbs * an.w) >> p.rank1_shift)) >> p.out_shift;
                if (pass == 0) {
                    mx = __vimax3_s32(__vimax3_s32(mx, l0, l1), l2, l3);
                } else {
                    sum += sm.exp_lut[min(255, mx - l0)] + sm.exp_lut[min(255, mx - l1)] + sm.exp_lut[min(255, mx - l2)] +
                           sm.exp_lut[min(255, mx - l3)];
                    const int tc = tgt_col - col;
                    if (tc == 0) tg = l0; else if (tc == 1) tg = l1; else if (tc == 2) tg = l2; else if (tc == 3) tg = l3;
                }
            }
        }
        if (pass == 0) {
            hp[0][cq][row_in_tile] = mx;
            ptx::named_bar_sync(2 + quarter, 128);
            mx = max(max(hp[0][0][row_in_tile], hp[0][1][row_in_tile]), max(hp[0][2][row_in_tile], hp[0][3][row_in_tile]));
        }
    }
    hp[1][cq][row_in_tile] = sum;
    hp[2][cq][row_in_tile] = tg;                    // the target column lives in exactly one quarter: the others hold 0
    ptx::named_bar_sync(2 + quarter, 128);
    if (cq == 0) {
        const int sm_ = hp[1][0][row_in_tile] + hp[1][1][row_in_tile] + hp[1][2][row_in_tile] + hp[1][3][row_in_tile];
        const int tgl = hp[2][0][row_in_tile] + hp[2][1][row_in_tile] + hp[2][2][row_in_tile] + hp[2][3][row_in_tile];
        int log_sum = 0;
        if (sm_ > 0) log_sum = ((31 - __clz(sm_)) << 4) - (p.softmax_scale_bit << 4);   // floor(log2), shift ladder of mgpu.cu:1015-1019
        int term = row_ok ? ((log_sum >> 1) + mx - tgl) : 0;
        term = __reduce_add_sync(0xFFFFFFFFu, term);        // the warp's 32 rows are consecutive tokens of one member
        if (lane == 0) atomicAdd(&p.loss[mem], term);
    }
}

template <int BN, int EPI, int RPL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_o, const __grid_constant__ CUtensorMap tmap_r, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    GemmSmem<BN> &sm = *reinterpret_cast<GemmSmem<BN> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = p.N / BN;
    const int tiles_m = (p.M + GEMM_BM - 1) / GEMM_BM;
    const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;
    // the vote GEMM may cut its contraction (the pair index) into k_splits parts: work item = (split, tile)
    const int k_splits = (EPI == EPI_VOTE && p.k_splits > 1) ? p.k_splits : 1;
    const int kb_per = (num_kb + k_splits - 1) / k_splits;
    const int mn_tiles = tiles_m * tiles_n;
    const int num_tiles = mn_tiles * k_splits;
    constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));
    constexpr uint32_t STAGE_BYTES = GEMM_BM * GEMM_BK + BN * GEMM_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_STAGES; s++) { ptx::mbar_init(&sm.full[s], 1); ptx::mbar_init(&sm.empty[s], 1); }
        for (int a = 0; a < 2; a++) { ptx::mbar_init(&sm.tmem_full[a], 1); ptx::mbar_init(&sm.tmem_empty[a], GEMM_EPI_WARPS); }
        for (int w = 0; w < GEMM_EPI_WARPS; w++) ptx::mbar_init(&sm.rbar[w], 1);
        sm.abort_flag = 0;
        sm.epi_ok = 1;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(&sm.tmem_base, TMEM_COLS);
        ptx::tmem_relinquish();
    }
    if (warp >= 2) {
        int e = threadIdx.x - 64;
        if (EPI == EPI_GELU && p.act_lut && e < 256) sm.act_lut[e] = p.act_lut[e == 0x80 ? 0x81 : e];   // saturating pack yields -128 where the reference clips to -127
        if (EPI == EPI_HEAD && p.exp_lut && e < 256) sm.exp_lut[e] = p.exp_lut[e];
        if (EPI == EPI_GELU && RPL && p.act_lut) {
            for (int i = e; i < 256 * 32; i += GEMM_EPI_THREADS) {
                const int idx = i >> 5;
                sm.lut32[idx][i & 31] = (uint32_t)(uint8_t)p.act_lut[idx == 0x80 ? 0x81 : idx];
            }
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == 0) {
        // ===================== TMA producer =====================
        if (ptx::elect_one()) {
            ptx::prefetch_tmap(&tmap_a);
            ptx::prefetch_tmap(&tmap_b);
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int split = (k_splits > 1) ? tile / mn_tiles : 0, mn = tile - split * mn_tiles;
                int tm_ = fast_div(mn, p.fd_tiles_n), m0 = tm_ * GEMM_BM, n0 = (mn - tm_ * tiles_n) * BN;
                const int kb0 = split * kb_per, kb1 = min(num_kb, kb0 + kb_per);
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    int s = it % GEMM_STAGES;
                    uint32_t ph = (it / GEMM_STAGES) & 1;
                    if (!ptx::mbar_wait(&sm.empty[s], ph ^ 1) || sm.abort_flag) { gemm_fail(p, &sm.abort_flag, DEV_TIMEOUT_EMPTY); ok = false; break; }
                    ptx::mbar_arrive_expect_tx(&sm.full[s], STAGE_BYTES);
                    ptx::tma_load_2d(sm.a[s], &tmap_a, &sm.full[s], kb * GEMM_BK, m0);
                    ptx::tma_load_2d(sm.b[s], &tmap_b, &sm.full[s], kb * GEMM_BK, n0);
                }
            }
            if (!ok) {   // let copies already in flight land before the CTA tears down
                uint64_t t0 = ptx::globaltimer();
                while (ptx::globaltimer() - t0 < 200000ull) { __nanosleep(1000); }
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::make_idesc_i8(GEMM_BM, BN);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tcount++) {
                int as = tcount & 1;
                uint32_t aph = (tcount >> 1) & 1;
                if (!ptx::mbar_wait(&sm.tmem_empty[as], aph ^ 1) || sm.abort_flag) { gemm_fail(p, &sm.abort_flag, DEV_TIMEOUT_TMEM_EMPTY); ok = false; break; }
                ptx::tc_fence_after();
                uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
                const int split = (k_splits > 1) ? tile / mn_tiles : 0;
                const int kb0 = split * kb_per, kb1 = min(num_kb, kb0 + kb_per);
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    int s = it % GEMM_STAGES;
                    uint32_t ph = (it / GEMM_STAGES) & 1;
                    if (!ptx::mbar_wait(&sm.full[s], ph) || sm.abort_flag) { gemm_fail(p, &sm.abort_flag, DEV_TIMEOUT_FULL); ok = false; break; }
                    ptx::tc_fence_after();
                    uint64_t da = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.a[s]));
                    uint64_t db = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.b[s]));
#pragma unroll
                    for (int k = 0; k < GEMM_BK / 32; k++) {
                        // +32 bytes along K inside the swizzle row = +2 in the 16-byte address field
                        ptx::mma_i8(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    ptx::mma_commit(&sm.empty[s]);
                }
                if (ok) ptx::mma_commit(&sm.tmem_full[as]);
            }
        }
    } else {
        // ===================== epilogue (16 warps) =====================
        const int e = threadIdx.x - 64;            // 0..511
        const int ew = warp - 2;                   // 0..15
        const int quarter = warp & 3;              // TMEM lane quarter this warp may read
        constexpr int NHALF = (EPI == EPI_HEAD && !RPL) ? 1 : 4;   // column parts per lane quarter; the transposed head keeps whole rows in one warp
        constexpr int COLS_PER = BN / NHALF;
        const int half = (NHALF == 4) ? (ew >> 2) : 0;     // which part of the tile's columns
        const bool active = (NHALF == 4) || ew < 4;
        const int row_in_tile = quarter * 32 + lane;
        uint32_t tcount = 0;
        int pf_xb = 0;                              // row-per-lane form: values of the next tile, loaded a tile ahead
        int4 pf_rs0 = make_int4(0, 0, 0, 0);
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, tcount++) {
            const int as = tcount & 1;
            const uint32_t aph = (tcount >> 1) & 1;
            const int split = (k_splits > 1) ? tile / mn_tiles : 0, mn = tile - split * mn_tiles;
            const int tm_ = fast_div(mn, p.fd_tiles_n), m0 = tm_ * GEMM_BM, n0 = (mn - tm_ * tiles_n) * BN;
            const int r = m0 + row_in_tile;
            const bool row_ok = r < p.M;

            // ---- per-tile tables (evaluation epilogues): built here for a block's first tile, otherwise already
            // written at the end of the previous tile from words prefetched during its epilogue ----
            int first_pl = 0, slot = 0, sgn = 0;
            if (EPI <= EPI_LOGITS) {
                int last_row = min(m0 + GEMM_BM, p.M) - 1;
                first_pl = fast_div(m0, p.fd_seq) >> 1;
                int mem = fast_div(row_ok ? r : last_row, p.fd_seq);
                slot = (mem >> 1) - first_pl;
                sgn = mem & 1;
                if (tcount == 0) {
                    TabWords w;
                    if (tab_load<BN, EPI>(p, e, m0, n0, w)) tab_store<BN, EPI, RPL>(p, sm, e, w);
                }
            }
            // ---- per-row state of the 4 rows this lane owns after the transpose, and the loads that do not
            // depend on the accumulator: all issued before waiting for the MMAs of this tile ----
            const int cbase = half * COLS_PER;       // column offset inside the tile
            int32_t(*st)[20] = sm.stage[ew];
            const int lrow = lane >> 2, pc = lane & 3;          // row group / 4-column piece of this lane
            int rrow[4], xbs[4], slot_sgn[4], aux[4];           // per-row state of the 4 rows this lane touches
            bool rok[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (EPI > EPI_LOGITS || RPL) { rrow[i] = 0; xbs[i] = 0; slot_sgn[i] = 0; aux[i] = 0; rok[i] = false; continue; }
                const int rr = m0 + quarter * 32 + i * 8 + lrow;
                rok[i] = rr < p.M;
                const int rc = rok[i] ? rr : (p.M - 1);
                rrow[i] = rc;
                const int mem = fast_div(rc, p.fd_seq);
                const int sg = mem & 1;
                slot_sgn[i] = (((mem >> 1) - first_pl) << 1) | sg;
                const int xcol = (EPI == EPI_QKV) ? fast_div(n0, p.fd_third) : 0;
                const int xbv = p.xb[(int64_t)rc * p.xb_stride + xcol];
                xbs[i] = sg ? -xbv : xbv;
                aux[i] = 0;
                if (EPI == EPI_QKV) aux[i] = rc - mem * p.seq_len;                 // token position t
                if (EPI == EPI_HEAD) {                                             // target byte of this row
                    const int t = rc - mem * p.seq_len;
                    const int64_t pair = (p.pop_base + mem) >> 1;
                    const int64_t pos = p.use_same_data ? (p.start_idx % (p.data_len - p.seq_len))
                                                        : ((p.start_idx + pair * p.data_stride) % (p.data_len - p.seq_len));
                    aux[i] = p.dataset[pos + t + 1];
                }
            }
            // row-per-lane form: the lane's rank-1 factor (raw Σ x·b of its row) and the first chunk of residual bytes
            // were loaded during the previous tile (pf_*); only a block's first tile loads them here
            int xbs_l = 0;
            int4 rs_l[BN / 4 / 16];
            // The residual bytes of the residual projections: with BN = 256 every warp's 32 rows x 64 columns arrive as one
            // box through the copy engine (requested a tile ahead, at the end of the previous tile's epilogue) -- a lane
            // loading its own row 16 bytes at a time costs 32 half-used sectors per instruction (12 ms per generation).
            constexpr bool RES_TMA = (EPI == EPI_PRE32) && RPL && BN == 256;
            if (RES_TMA && tcount == 0 && lane == 0) {
                ptx::mbar_arrive_expect_tx(&sm.rbar[ew], 32 * 64);
                ptx::tma_load_2d(sm.ostage1[ew], &tmap_r, &sm.rbar[ew], n0 + cbase, m0 + quarter * 32);
            }
            if (RPL && active) {
                const int rc = row_ok ? r : (p.M - 1);
                if (tcount == 0) {
                    pf_xb = p.xb[(int64_t)rc * p.xb_stride + ((EPI == EPI_QKV) ? fast_div(n0, p.fd_third) : 0)];
                    if (EPI == EPI_PRE32 && !RES_TMA) pf_rs0 = *reinterpret_cast<const int4 *>(p.resid + (int64_t)rc * p.N + n0 + cbase);
                }
                xbs_l = sgn ? -pf_xb : pf_xb;
                if (EPI == EPI_PRE32 && !RES_TMA) {
                    rs_l[0] = pf_rs0;
#pragma unroll
                    for (int cc = 1; cc < BN / 4 / 16; cc++)      // used one chunk of arithmetic later each
                        rs_l[cc] = *reinterpret_cast<const int4 *>(p.resid + (int64_t)rc * p.N + n0 + cbase + 16 * cc);
                }
            }
            int32_t rs_pre[COLS_PER / 16][4];        // residual bytes of every chunk (EPI_PRE32)
            if (EPI == EPI_PRE32 && active && !RPL) {
#pragma unroll
                for (int cc = 0; cc < COLS_PER / 16; cc++)
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        rs_pre[cc][i] = *reinterpret_cast<const int32_t *>(p.resid + (int64_t)rrow[i] * p.N + n0 + cbase + cc * 16 + 4 * pc);
            }
            // one thread waits for the accumulator, everybody learns the outcome at the barrier
            if (e == 0) {
                bool ok = ptx::mbar_wait(&sm.tmem_full[as], aph) && !sm.abort_flag;
                if (!ok) { gemm_fail(p, &sm.abort_flag, DEV_TIMEOUT_TMEM_FULL); sm.epi_ok = 0; }
            }
            __syncwarp();
            ptx::named_bar_sync(1, GEMM_EPI_THREADS);
            if (!sm.epi_ok) break;
            ptx::tc_fence_after();
            // words of the next tile's tables: in flight while this tile is computed
            TabWords nxt;
            bool have_nxt = false;
            if (EPI <= EPI_LOGITS) {
                const int ntile = tile + gridDim.x;
                if (ntile < num_tiles) {
                    const int ntm = fast_div(ntile, p.fd_tiles_n), nm0 = ntm * GEMM_BM, nn0 = (ntile - ntm * tiles_n) * BN;
                    have_nxt = tab_load<BN, EPI>(p, e, nm0, nn0, nxt);
                    if (RPL && active) {
                        const int nr = nm0 + row_in_tile, nrc = nr < p.M ? nr : (p.M - 1);
                        pf_xb = p.xb[(int64_t)nrc * p.xb_stride + ((EPI == EPI_QKV) ? fast_div(nn0, p.fd_third) : 0)];
                        if (EPI == EPI_PRE32 && !RES_TMA) pf_rs0 = *reinterpret_cast<const int4 *>(p.resid + (int64_t)nrc * p.N + nn0 + half * COLS_PER);
                    }
                }
            }

            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * BN + half * COLS_PER);

            if (!active) {
                // nothing to compute; still takes part in the barrier protocol below
            } else if (RPL && EPI == EPI_HEAD) {
                epilogue_head_rpl<BN>(p, sm, taddr, r, row_ok, cbase, slot, lane, quarter, row_in_tile, xbs_l);
            } else if (RPL) {
                if (RES_TMA) {
                    if (lane == 0 && !ptx::mbar_wait(&sm.rbar[ew], tcount & 1)) gemm_fail(p, &sm.abort_flag, DEV_TIMEOUT_FULL);
                    __syncwarp();
                }
                if (EPI == EPI_QKV && n0 < 2 * p.third)
                    epilogue_rpl<BN, EPI, true, false>(p, sm, taddr, r, row_ok, n0, cbase, slot, sgn, sm.stage[ew], lane, m0 + quarter * 32, xbs_l, rs_l,
                                                       &tmap_o, sm.ostage0[ew], sm.ostage1[ew]);
                else
                    epilogue_rpl<BN, EPI, false, RES_TMA>(p, sm, taddr, r, row_ok, n0, cbase, slot, sgn, sm.stage[ew], lane, m0 + quarter * 32, xbs_l,
                                                          rs_l, &tmap_o, sm.ostage0[ew], sm.ostage1[ew]);
                if (RES_TMA) {
                    // every lane has read its residual bytes: the box may be refilled for the block's next tile
                    __syncwarp();
                    const int ntile = tile + gridDim.x;
                    if (lane == 0 && ntile < num_tiles) {
                        const int ntm = fast_div(ntile, p.fd_tiles_n);
                        ptx::mbar_arrive_expect_tx(&sm.rbar[ew], 32 * 64);
                        ptx::tma_load_2d(sm.ostage1[ew], &tmap_r, &sm.rbar[ew], (ntile - ntm * tiles_n) * BN + cbase, ntm * GEMM_BM + quarter * 32);
                    }
                }
            } else if (EPI <= EPI_LOGITS) {
                // ---------------- evaluation epilogues ----------------
                // Accumulators leave TMEM one row per lane; they are transposed through shared memory so
                // that 4 consecutive lanes own 16 consecutive columns of one row: every global access below
                // is then a run of full 32-byte sectors, and the per-column tables are read as words.
                int racc[4];                                        // running abs-max / dot / row max per row
#pragma unroll
                for (int i = 0; i < 4; i++) racc[i] = (EPI == EPI_HEAD || EPI == EPI_LOGITS) ? INT_MIN : 0;
                int rsum[4], rtgt[4];
#pragma unroll
                for (int i = 0; i < 4; i++) { rsum[i] = 0; rtgt[i] = 0; }

                constexpr int NPASS = (EPI == EPI_HEAD) ? 2 : 1;
#pragma unroll 1
                for (int pass = 0; pass < NPASS; pass++) {
                    if (EPI == EPI_HEAD && pass == 1) {
#pragma unroll
                        for (int i = 0; i < 4; i++) {               // finish the row maxima of pass 0
                            int m = racc[i];
                            m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
                            m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
                            racc[i] = m;
                        }
                    }
                    constexpr int CHUNK_UNROLL = (EPI == EPI_HEAD) ? 1 : COLS_PER / 16;
#pragma unroll CHUNK_UNROLL
                    for (int c = 0; c < COLS_PER; c += 16) {
                        {
                            uint32_t v[16];
                            ptx::tmem_ld16(taddr + c, v);
                            ptx::tmem_ld_wait();
#pragma unroll
                            for (int qd = 0; qd < 4; qd++)
                                *reinterpret_cast<int4 *>(&st[lane][4 * qd]) = make_int4(v[4 * qd], v[4 * qd + 1], v[4 * qd + 2], v[4 * qd + 3]);
                        }
                        __syncwarp();
                        const int col = cbase + c + 4 * pc;          // column inside the tile of this lane's 4 values
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int4 a4 = *reinterpret_cast<const int4 *>(&st[i * 8 + lrow][4 * pc]);
                            const int sl = slot_sgn[i] >> 1, sg = slot_sgn[i] & 1;
                            const int32_t aw = *reinterpret_cast<const int32_t *>(&sm.a_tab[sl][col]);
                            const int4 an = make_int4((int)(int8_t)aw, (int)(int8_t)(aw >> 8), (int)(int8_t)(aw >> 16), aw >> 24);
                            int v0 = a4.x + ((xbs[i] * an.x) >> p.rank1_shift);
                            int v1 = a4.y + ((xbs[i] * an.y) >> p.rank1_shift);
                            int v2 = a4.z + ((xbs[i] * an.z) >> p.rank1_shift);
                            int v3 = a4.w + ((xbs[i] * an.w) >> p.rank1_shift);
                            const int64_t gofs = (int64_t)rrow[i] * p.N + n0 + col;
                            if (EPI == EPI_CLIP8) {
                                // saturate to int8 and pack (two instructions), then lift -128 to the reference's -127
                                uint32_t w = ptx::pack_sat_s8(v0 >> p.out_shift, v1 >> p.out_shift, v2 >> p.out_shift, v3 >> p.out_shift);
                                w = __vmaxs4(w, 0x81818181u);
                                if (rok[i]) *reinterpret_cast<uint32_t *>(p.out8 + gofs) = w;
                            } else if (EPI == EPI_GELU) {
                                const int2 bcw = *reinterpret_cast<const int2 *>(&sm.bc_tab[sl][sg][col]);
                                const int4 bc = make_int4((int)(int16_t)(bcw.x & 0xFFFF), bcw.x >> 16, (int)(int16_t)(bcw.y & 0xFFFF), bcw.y >> 16);
                                const uint32_t z = ptx::pack_sat_s8((v0 >> p.out_shift) + bc.x, (v1 >> p.out_shift) + bc.y,
                                                                    (v2 >> p.out_shift) + bc.z, (v3 >> p.out_shift) + bc.w);
                                const uint32_t u0 = (uint8_t)sm.act_lut[z & 0xFF], u1 = (uint8_t)sm.act_lut[(z >> 8) & 0xFF];
                                const uint32_t u2 = (uint8_t)sm.act_lut[(z >> 16) & 0xFF], u3 = (uint8_t)sm.act_lut[z >> 24];
                                const uint32_t w = __byte_perm(__byte_perm(u0, u1, 0x0040), __byte_perm(u2, u3, 0x0040), 0x5410);
                                racc[i] = __dp4a((int)w, *reinterpret_cast<const int32_t *>(&sm.d_tab[sl][col]), racc[i]);
                                if (rok[i]) *reinterpret_cast<uint32_t *>(p.out8 + gofs) = w;
                            } else if (EPI == EPI_PRE32) {
                                const int2 bcw = *reinterpret_cast<const int2 *>(&sm.bc_tab[sl][sg][col]);
                                const int4 bc = make_int4((int)(int16_t)(bcw.x & 0xFFFF), bcw.x >> 16, (int)(int16_t)(bcw.y & 0xFFFF), bcw.y >> 16);
                                const int32_t rs = rs_pre[c / 16][i];
                                v0 = (int)(int8_t)(rs) + (v0 >> p.out_shift) + bc.x;
                                v1 = (int)(int8_t)(rs >> 8) + (v1 >> p.out_shift) + bc.y;
                                v2 = (int)(int8_t)(rs >> 16) + (v2 >> p.out_shift) + bc.z;
                                v3 = (int)(rs >> 24) + (v3 >> p.out_shift) + bc.w;
                                racc[i] = max(racc[i], max(max(abs(v0), abs(v1)), max(abs(v2), abs(v3))));
                                if (rok[i]) *reinterpret_cast<int4 *>(p.out32 + gofs) = make_int4(v0, v1, v2, v3);
                            } else if (EPI == EPI_QKV) {
                                if (n0 < 2 * p.third) {
                                    // integer RoPE on adjacent (even, odd) columns (apply_rope_integer, mgpu.cu:624-644)
                                    const int hd0 = fast_mod(n0 + col, p.fd_head);
                                    const int4 cs = __ldg(reinterpret_cast<const int4 *>(p.rope_lut + (int64_t)aux[i] * p.head_dim + hd0));
                                    const long long half_ulp = 1ll << (p.rope_bit - 1);
                                    const long long e0 = v0, o0 = v1, e1 = v2, o1 = v3;
                                    v0 = (int)((e0 * cs.x - o0 * cs.y + half_ulp) >> p.rope_bit);
                                    v1 = (int)((e0 * cs.y + o0 * cs.x + half_ulp) >> p.rope_bit);
                                    v2 = (int)((e1 * cs.z - o1 * cs.w + half_ulp) >> p.rope_bit);
                                    v3 = (int)((e1 * cs.w + o1 * cs.z + half_ulp) >> p.rope_bit);
                                }
                                racc[i] = max(racc[i], max(max(abs(v0), abs(v1)), max(abs(v2), abs(v3))));
                                if (rok[i]) *reinterpret_cast<int4 *>(p.out32 + gofs) = make_int4(v0, v1, v2, v3);
                            } else if (EPI == EPI_LOGITS) {
                                // the head of a vocabulary wider than one tile (mgpu.cu:969-983): logits to memory, row max so far
                                v0 >>= p.out_shift; v1 >>= p.out_shift; v2 >>= p.out_shift; v3 >>= p.out_shift;
                                racc[i] = max(racc[i], max(max(v0, v1), max(v2, v3)));
                                if (rok[i]) *reinterpret_cast<int4 *>(p.out32 + gofs) = make_int4(v0, v1, v2, v3);
                            } else if (EPI == EPI_HEAD) {
                                // pass 0: row max of the logits; pass 1: Σ exp-LUT and the target logit (mgpu.cu:969-1023)
                                const int l0 = v0 >> p.out_shift, l1 = v1 >> p.out_shift, l2 = v2 >> p.out_shift, l3 = v3 >> p.out_shift;
                                if (pass == 0) {
                                    racc[i] = max(racc[i], max(max(l0, l1), max(l2, l3)));
                                } else {
                                    const int mx = racc[i];
                                    rsum[i] += sm.exp_lut[min(255, mx - l0)] + sm.exp_lut[min(255, mx - l1)] +
                                               sm.exp_lut[min(255, mx - l2)] + sm.exp_lut[min(255, mx - l3)];
                                    const int tc = aux[i] - (n0 + col);
                                    if (tc == 0) rtgt[i] = l0; else if (tc == 1) rtgt[i] = l1; else if (tc == 2) rtgt[i] = l2; else if (tc == 3) rtgt[i] = l3;
                                }
                            }
                        }
                        __syncwarp();
                    }
                }
                // ---- per-row results: combine the 8 lanes that share a row ----
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (EPI == EPI_GELU) {
                        int d = racc[i];
                        d += __shfl_xor_sync(0xFFFFFFFFu, d, 1); d += __shfl_xor_sync(0xFFFFFFFFu, d, 2);
                        if (pc == 0 && rok[i]) atomicAdd(&p.rowstat[rrow[i]], d);
                    } else if (EPI == EPI_PRE32 || EPI == EPI_QKV) {
                        int m = racc[i];
                        m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1)); m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
                        if (pc == 0 && rok[i]) {
                            if (EPI == EPI_PRE32) atomicMax(&p.rowstat[rrow[i]], m);
                            else atomicMax(&p.rowstat[(int64_t)rrow[i] * 3 + fast_div(n0, p.fd_third)], m);
                        }
                    } else if (EPI == EPI_LOGITS) {
                        int m = racc[i];
                        m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1)); m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
                        if (pc == 0 && rok[i]) atomicMax(&p.rowstat[rrow[i]], m);
                    } else if (EPI == EPI_HEAD) {
                        int sm_ = rsum[i], tg = rtgt[i];          // the target column lives in exactly one lane: others hold 0
                        sm_ += __shfl_xor_sync(0xFFFFFFFFu, sm_, 1); sm_ += __shfl_xor_sync(0xFFFFFFFFu, sm_, 2);
                        tg += __shfl_xor_sync(0xFFFFFFFFu, tg, 1); tg += __shfl_xor_sync(0xFFFFFFFFu, tg, 2);
                        if (pc == 0 && rok[i]) {
                            int log_sum = 0;
                            if (sm_ > 0) log_sum = ((31 - __clz(sm_)) << 4) - (p.softmax_scale_bit << 4);   // floor(log2), shift ladder of mgpu.cu:1015-1019
                            atomicAdd(&p.loss[fast_div(rrow[i], p.fd_seq)], (log_sum >> 1) + racc[i] - tg);
                        }
                    }
                }
            } else if (EPI == EPI_NULL) {
                // nothing: the accumulator stage is released right away
            } else {
                // ---------------- vote epilogue: row r = output column n, tile columns = input index k ----------------
                const int n = r;
                const int cols_n = p.M;
                int32_t *vout = p.vote_out + (int64_t)split * p.split_stride;
                for (int c = 0; c < COLS_PER; c += 32) {
                    uint32_t v[32];
                    ptx::tmem_ld32(taddr + c, v);
                    ptx::tmem_ld_wait();
                    if (!row_ok) continue;
                    const int k0 = n0 + cbase + c;           // multiple of 32
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const int64_t word = (int64_t)((k0 >> 2) + q) * cols_n + n;
                        *reinterpret_cast<int4 *>(vout + word * 4) = make_int4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    }
                }
            }
            // release the accumulator stage
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&sm.tmem_empty[as]);
            // tables are rewritten at the top of the next tile: everybody must be done reading them
            ptx::named_bar_sync(1, GEMM_EPI_THREADS);
            if (RPL && EPI != EPI_HEAD && half == 0 && row_ok) {
                // one atomic per row and tile instead of one per column quarter
                const int a0 = sm.rowpart[0][row_in_tile], a1 = sm.rowpart[1][row_in_tile], a2 = sm.rowpart[2][row_in_tile],
                          a3 = sm.rowpart[3][row_in_tile];
                if (EPI == EPI_GELU) atomicAdd(&p.rowstat[r], a0 + a1 + a2 + a3);
                else if (EPI == EPI_PRE32 || EPI == EPI_LOGITS) atomicMax(&p.rowstat[r], max(max(a0, a1), max(a2, a3)));
                else if (EPI == EPI_QKV) atomicMax(&p.rowstat[(int64_t)r * 3 + fast_div(n0, p.fd_third)], max(max(a0, a1), max(a2, a3)));
            }
            if (EPI <= EPI_LOGITS && have_nxt) tab_store<BN, EPI, RPL>(p, sm, e, nxt);   // published by the next tile's barrier
        }
    }

    // output boxes still being copied out of shared memory must land before the block retires
    if (RPL && (EPI == EPI_PRE32 || EPI == EPI_QKV || EPI == EPI_GELU || EPI == EPI_LOGITS) && warp >= 2 && lane == 0) ptx::tma_store_wait_all<0>();
    __syncwarp();
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int BN>
constexpr size_t gemm_smem_bytes() { return sizeof(GemmSmem<BN>) + 1024; }
static_assert(gemm_smem_bytes<256>() <= 227 * 1024, "GEMM shared memory exceeds the 227 KB a block may use");

}  // namespace egg
