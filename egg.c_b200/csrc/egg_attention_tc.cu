// Causal integer-softmax attention (compute_attention, mgpu.cu:787-825) on the sm_100a tensor cores.
//
// One thread block per (population member, head).  For every block of 128 queries:
//   scores  S = Q K^T        tcgen05.mma kind::i8, M = 128 queries, N = 128 or 256 keys, K = 64 -> int32 in tensor memory
//   pass A  every worker lane owns one query row: max over the keys c <= t straight from tensor memory
//   pass B  wt_c = EXP_LUT[clamp((max >> shift) - (S_c >> shift), 0, 255)]; the 19-bit weights are cut into three 7-bit
//           limbs and written to shared memory as three int8 A operands P_l[query][key]
//   sums    O_l = P_l V      three tcgen05.mma chains, M = 128, N = 64 dims, K = keys -> three int32 accumulators
//   output  o_d = trunc((O_0 + 2^7 O_1 + 2^14 O_2)_d / max(1, Σ wt)): exact, because every limb sum is below
//           127 * 127 * seq_len < 2^31 and the recombination / division is done as in att_div below.
// Keys are processed in chunks of 256 (two 128-key operand tiles).  With more than one chunk per query block
// (seq_len > 256) the scores of a chunk are recomputed in pass B instead of being kept: tensor memory then holds one
// score chunk (256 columns) and the three accumulators (192 columns) whatever the sequence length.
// Q, K and the transposed V are staged by the worker warps in the K-major 128-byte-swizzled operand layout (rows of Q
// and K are 64 bytes: they occupy the first half of 128-byte operand rows).  Warp 0 issues the MMAs, warps 1..16 work
// (4 tensor-memory lane quarters x 4 column parts).  Every wait is bounded; a timeout makes all later waits fall through.
// Needs seq_len % 128 == 0 (whole query blocks of one member); other lengths take attention_kernel.
#include "egg_kernels.cuh"
#include "egg_gemm_fused.cuh"

#include <limits.h>

namespace egg {

constexpr int ATC_WORKERS = 16;
constexpr int ATC_THREADS = 32 * (1 + ATC_WORKERS);
constexpr int ATC_O_COL = 256;          // first tensor-memory column of the three accumulators (64 columns each)

struct AtcBars {
    uint64_t q_ready, s_full, s_free, p_ready, pv_done;
    uint32_t tmem_base;
    volatile int abort_flag;
};

// shared-memory carve-up (bytes), all operand tiles 1024-byte aligned
struct AtcLayout {
    int q, k, vt, p, lut, part, bars, total;
    int lut_copies;
};
static AtcLayout atc_layout(int S) {
    AtcLayout L;
    int o = 0;
    L.q = o; o += ((S <= 256) ? S / 128 : 1) * 128 * 128;      // every query block resident when there are at most two
    L.k = o; o += S * 128;
    L.vt = o; o += (S / 128) * 64 * 128;
    L.p = o; o += 2 * 3 * 128 * 128;
    L.lut_copies = (S <= 256) ? 32 : 4;              // lane-private copies of the weight table where shared memory allows
    L.lut = o; o += L.lut_copies * 256 * 4;
    L.part = o; o += (4 + 12 + 4) * 128 * 4;       // row maxima [4][128], limb sums [3][4][128], output dots [4][128]
    L.bars = o; o += 128;
    L.total = o + 1024;                            // slack for the 1024-byte alignment of the dynamic buffer
    return L;
}

// Bounded wait for the waits of this kernel, which all sit on its critical path (MMA warp and workers hand work back and
// forth once per phase): plain try_wait polling, which returns as soon as the phase completes, instead of the suspended
// form the GEMM pipelines use for waits that are normally satisfied in advance.
__device__ __forceinline__ void atc_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *err, int code) {
#ifdef EGG_ATC_SUSPENDED_WAITS
    fused_wait(bar, parity, abort_flag, err, code);
#else
    if (*abort_flag) return;
    if (ptx::mbar_try_wait(bar, parity)) return;
    const uint64_t t0 = ptx::globaltimer();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; i++)
            if (ptx::mbar_try_wait(bar, parity)) return;
        if (ptx::globaltimer() - t0 > 1000000000ull) {              // one second: give up, start the drain
            *abort_flag = 1;
            if (err) atomicCAS(err, 0, code);
            return;
        }
    }
#endif
}

__device__ __forceinline__ uint32_t sw128_addr(uint32_t base, int row, int piece) {
    // byte address of 16-byte piece `piece` of 128-byte operand row `row` (8-row groups of 1024 bytes)
    return base + (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((piece ^ (row & 7)) << 4));
}

// trunc(num / den) for num = p0 + 2^7 p1 + 2^14 p2 with every limb sum below 2^23 (seq_len <= 512), den = d0 + 2^7 d1 +
// 2^14 d2 >= 1 and |num / den| <= 127: a float estimate, then the exact remainder assembled limb by limb in 32-bit
// arithmetic (it is at most half the denominator in magnitude, so the wrapping partial terms add up to its true value).
__device__ __forceinline__ int atc_div(int p0, int p1, int p2, int d0, int d1, int d2, float rden) {
    const float fn = fmaf(__int2float_rn(p2 * 128 + p1), 128.0f, __int2float_rn(p0));
    int k = __float2int_rn(fn * rden);
    const int r = (p0 - k * d0) + (p1 - k * d1) * 128 + (p2 - k * d2) * 16384;
    if (k > 0 && r < 0) k--;
    else if (k < 0 && r > 0) k++;
    return k;
}

__global__ void __launch_bounds__(ATC_THREADS, 1) attention_tc_kernel(const AttnParams p, const AtcLayout L, int *err) {
    extern __shared__ uint8_t atc_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(atc_raw) + 1023) & ~uintptr_t(1023));
    AtcBars &bars = *reinterpret_cast<AtcBars *>(sm + L.bars);
    uint32_t *lut = reinterpret_cast<uint32_t *>(sm + L.lut);
    int32_t *part_max = reinterpret_cast<int32_t *>(sm + L.part);             // [4][128]
    int32_t *part_sum = part_max + 4 * 128;                                   // [3][4][128]
    int32_t *part_dot = part_sum + 12 * 128;                                  // [4][128]
    const uint32_t q_s = ptx::smem_u32(sm + L.q), k_s = ptx::smem_u32(sm + L.k), vt_s = ptx::smem_u32(sm + L.vt), p_s = ptx::smem_u32(sm + L.p);

    const int S = p.seq_len, H = p.H;
    const int n_heads = H / 64;
    const int mem = blockIdx.x / n_heads, hd = blockIdx.x % n_heads;
    const int64_t base = (int64_t)mem * S;
    const int col0 = hd * 64;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NQ = S / 128;                       // query blocks = 128-key tiles
    const int sh = p.shift_attn;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars.q_ready, ATC_WORKERS);
        ptx::mbar_init(&bars.s_full, 1);
        ptx::mbar_init(&bars.s_free, ATC_WORKERS);
        ptx::mbar_init(&bars.p_ready, ATC_WORKERS);
        ptx::mbar_init(&bars.pv_done, 1);
        bars.abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 0) {
        ptx::tmem_alloc(&bars.tmem_base, 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = bars.tmem_base;

    if (warp == 0) {
        // ===================== MMA issuer =====================
        if (ptx::elect_one()) {
            uint32_t n_q = 0, n_sfree = 0, n_p = 0;
            const bool q_all = NQ <= 2;                           // all query blocks were staged up front
            bool scores_issued = false;                           // the first score chunk of this block went out at the end of the previous block
            auto issue_scores = [&](int qb, int ch) {
                const int tiles = min(2, qb + 1 - 2 * ch);
                const uint32_t idesc = tiles == 2 ? ptx::make_idesc_i8(128, 256) : ptx::make_idesc_i8(128, 128);
                const uint64_t da = ptx::make_smem_desc_sw128(q_s + (q_all ? (uint32_t)qb * 16384u : 0u));
                const uint64_t db = ptx::make_smem_desc_sw128(k_s + (uint32_t)(2 * ch) * 16384u);
                ptx::mma_i8(tmem_base, da, db, idesc, 0u);
                ptx::mma_i8(tmem_base, da + 2, db + 2, idesc, 1u);          // head_dim 64 = two 32-byte k-steps
                ptx::mma_commit(&bars.s_full);
            };
            for (int qb = 0; qb < NQ && !bars.abort_flag; qb++) {
                const int ntile = qb + 1;                         // 128-key tiles this query block looks at
                const int nch = (ntile + 1) >> 1;                 // chunks of two tiles
                if (!q_all || qb == 0) {
                    atc_wait(&bars.q_ready, n_q++ & 1, &bars.abort_flag, err, DEV_TIMEOUT_FULL);
                    ptx::tc_fence_after();
                }
                // pass A: scores of every chunk for the row maxima
                for (int ch = 0; ch < nch && !bars.abort_flag; ch++) {
                    if (!(ch == 0 && scores_issued)) issue_scores(qb, ch);
                    atc_wait(&bars.s_free, n_sfree++ & 1, &bars.abort_flag, err, DEV_TIMEOUT_TMEM_EMPTY);     // the workers have read them
                    ptx::tc_fence_after();
                }
                scores_issued = false;
                // pass B: weights -> accumulators
                for (int ch = 0; ch < nch && !bars.abort_flag; ch++) {
                    if (nch > 1) issue_scores(qb, ch);            // a single chunk is still in tensor memory from pass A
                    atc_wait(&bars.p_ready, n_p++ & 1, &bars.abort_flag, err, DEV_TIMEOUT_FULL);
                    if (bars.abort_flag) break;
                    ptx::tc_fence_after();
                    const int tiles = min(2, ntile - 2 * ch);
                    constexpr uint32_t idesc_pv = ptx::make_idesc_i8(128, 64);
                    for (int t2 = 0; t2 < tiles; t2++) {
                        const uint64_t dv = ptx::make_smem_desc_sw128(vt_s + (uint32_t)(2 * ch + t2) * 8192u);
#pragma unroll
                        for (int l = 0; l < 3; l++) {
                            const uint64_t dp = ptx::make_smem_desc_sw128(p_s + (uint32_t)(t2 * 3 + l) * 16384u);
#pragma unroll
                            for (int ks = 0; ks < 4; ks++)
                                ptx::mma_i8(tmem_base + (uint32_t)(ATC_O_COL + 64 * l), dp + (uint64_t)(2 * ks), dv + (uint64_t)(2 * ks), idesc_pv,
                                            (ch > 0 || t2 > 0 || ks > 0) ? 1u : 0u);
                        }
                    }
                    ptx::mma_commit(&bars.pv_done);
                }
                // the score columns are free (the last weights have been taken from them) and the next block's queries are
                // resident: its first score chunk can run while the workers divide and store this block's outputs
                if (q_all && qb + 1 < NQ && !bars.abort_flag) { issue_scores(qb + 1, 0); scores_issued = true; }
            }
        }
    } else {
        // ===================== workers (16 warps) =====================
        const int ew = warp - 1;
        const int quarter = warp & 3;               // tensor-memory lane quarter this warp may touch
        const int cp = ew >> 2;                     // column part
        const int row = quarter * 32 + lane;        // query row inside the block
        const int tid = threadIdx.x - 32;           // 0..511
        const int copies = L.lut_copies;

        // ---- stage K, V^T and the weight table: every global load is issued before the first shared-memory store, so
        // that the block pays one memory latency here, not one per loop ----
        constexpr int NT = 32 * ATC_WORKERS;
        int4 kreg[4];                                             // S * 4 pieces / 512 threads <= 4 (seq_len <= 512)
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = tid + u * NT;
            kreg[u] = make_int4(0, 0, 0, 0);
            if (i < S * 4) kreg[u] = *reinterpret_cast<const int4 *>(p.k + (base + (i >> 2)) * H + col0 + (i & 3) * 16);
        }
        // V: one item = four consecutive keys x 16 dims; S items for 512 threads
        int4 vreg[4];
        const bool v_item = tid < S;
        const int kg = tid % (S / 4), dch = tid / (S / 4);
        if (v_item) {
#pragma unroll
            for (int kk = 0; kk < 4; kk++) vreg[kk] = *reinterpret_cast<const int4 *>(p.v + (base + kg * 4 + kk) * H + col0 + dch * 16);
        }
        const uint32_t lut_w = (uint32_t)p.exp_lut[tid & 255];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = tid + u * NT;
            if (i < S * 4) ptx::sts_v4(sw128_addr(k_s, i >> 2, i & 3), kreg[u]);
        }
        if (v_item) {
            // transposed in registers: for every dim a word of four consecutive keys
            const uint32_t *w0 = reinterpret_cast<const uint32_t *>(&vreg[0]), *w1 = reinterpret_cast<const uint32_t *>(&vreg[1]);
            const uint32_t *w2 = reinterpret_cast<const uint32_t *>(&vreg[2]), *w3 = reinterpret_cast<const uint32_t *>(&vreg[3]);
            const int key0 = kg * 4, tile = key0 >> 7, kin = key0 & 127;
#pragma unroll
            for (int dq = 0; dq < 4; dq++) {
                const uint32_t t0 = __byte_perm(w0[dq], w1[dq], 0x5140), t1 = __byte_perm(w2[dq], w3[dq], 0x5140);   // [a0 b0 a1 b1], [c0 d0 c1 d1]
                const uint32_t t2 = __byte_perm(w0[dq], w1[dq], 0x7362), t3 = __byte_perm(w2[dq], w3[dq], 0x7362);   // [a2 b2 a3 b3], [c2 d2 c3 d3]
                const uint32_t o[4] = {__byte_perm(t0, t1, 0x5410), __byte_perm(t0, t1, 0x7632), __byte_perm(t2, t3, 0x5410), __byte_perm(t2, t3, 0x7632)};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int dim = dch * 16 + dq * 4 + j;
                    const uint32_t a = sw128_addr(vt_s + (uint32_t)tile * 8192u, dim, kin >> 4) + (uint32_t)(kin & 15);
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(o[j]) : "memory");
                }
            }
        }
        {
            // entry e = tid & 255 as three 7-bit limbs, one per byte; the two halves of the threads fill half of the copies each
            const uint32_t packed = (lut_w & 127u) | (((lut_w >> 7) & 127u) << 8) | ((lut_w >> 14) << 16);
            const int e = tid & 255, half = copies >> 1;
            for (int cpy = (tid >> 8) * half; cpy < ((tid >> 8) + 1) * half; cpy++) lut[e * copies + cpy] = packed;   // entry e, copy c at [e * copies + c]
        }
        ptx::named_bar_sync(1, 32 * ATC_WORKERS);             // the weight table is read across warps
        const uint32_t lut_s = ptx::smem_u32(lut) + (uint32_t)(lane % copies) * 4u;
        const uint32_t lut_stride = (uint32_t)copies * 4u;
        const int8_t *nbo = p.nt + (int64_t)(mem >> 1) * p.nt_stride + p.nt_o_b + col0 + cp * 16;
        int4 nb4 = *reinterpret_cast<const int4 *>(nbo);        // the 16 noise values of this warp's output dims
        uint32_t n_sfull = 0, n_pv = 0;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const bool q_all = NQ <= 2;

        for (int qb = 0; qb < NQ; qb++) {
            const int ntile = qb + 1, nch = (ntile + 1) >> 1;
            const int t = qb * 128 + row;                        // this lane's query position
            // ---- Q block(s): all of them before the first block when they are resident, else this block's ----
            if (!q_all || qb == 0) {
                const int nblk = q_all ? NQ : 1;
                for (int b = 0; b < nblk; b++) {
                    const int r = tid >> 2, piece = tid & 3;        // 128 rows x 4 pieces = 512 threads
                    const int4 v = *reinterpret_cast<const int4 *>(p.q + (base + (qb + b) * 128 + r) * H + col0 + piece * 16);
                    ptx::sts_v4(sw128_addr(q_s + (uint32_t)b * 16384u, r, piece), v);
                }
                ptx::fence_proxy_async();                         // generic-proxy writes -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bars.q_ready);
            }

            // ---- pass A: row maximum over the keys c <= t ----
            int mx = INT_MIN;
            for (int ch = 0; ch < nch; ch++) {
                const int tiles = min(2, ntile - 2 * ch);
                const int ncol = tiles * 32;                      // columns per warp: a quarter of the chunk's keys
                atc_wait(&bars.s_full, n_sfull++ & 1, &bars.abort_flag, err, DEV_TIMEOUT_TMEM_FULL);
                __syncwarp();
                ptx::tc_fence_after();
                for (int c = 0; c < ncol; c += 16) {
                    const int colk = cp * ncol + c;               // first key of this piece inside the chunk
                    uint32_t v[16];
                    ptx::tmem_ld16(t_lane + (uint32_t)colk, v);
                    ptx::tmem_ld_wait16(v);
                    const int key0 = ch * 256 + colk;
                    if (key0 + 15 <= t) {
#pragma unroll
                        for (int j = 0; j < 16; j += 2) mx = __vimax3_s32(mx, (int)v[j], (int)v[j + 1]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++) if (key0 + j <= t) mx = max(mx, (int)v[j]);
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bars.s_free);
            }
            part_max[cp * 128 + row] = mx;
            ptx::named_bar_sync(2 + quarter, 128);
            mx = max(max(part_max[row], part_max[128 + row]), max(part_max[256 + row], part_max[384 + row]));
            const int mxs = mx >> sh;

            // ---- pass B: weights in three limbs -> shared-memory operands; limb sums of Σ wt ----
            int tl0 = 0, tl1 = 0, tl2 = 0;
            for (int ch = 0; ch < nch; ch++) {
                const int tiles = min(2, ntile - 2 * ch);
                const int ncol = tiles * 32;
                if (nch > 1) {
                    atc_wait(&bars.s_full, n_sfull++ & 1, &bars.abort_flag, err, DEV_TIMEOUT_TMEM_FULL);
                    __syncwarp();
                    ptx::tc_fence_after();
                }
                if (ch > 0) {                                     // the operand tiles are still being read by the previous chunk's MMAs
                    atc_wait(&bars.pv_done, n_pv++ & 1, &bars.abort_flag, err, DEV_TIMEOUT_TMEM_FULL);
                    __syncwarp();
                }
                for (int c = 0; c < ncol; c += 16) {
                    const int colk = cp * ncol + c;
                    uint32_t v[16];
                    ptx::tmem_ld16(t_lane + (uint32_t)colk, v);
                    ptx::tmem_ld_wait16(v);
                    const int key0 = ch * 256 + colk;
                    const bool full = key0 + 15 <= t;
                    uint32_t l0[4], l1[4], l2[4];
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint32_t d = min((uint32_t)(mxs - ((int)v[4 * g + j] >> sh)), 255u);      // a masked key may exceed the maximum: clamped, then dropped
                            const uint32_t wv = ptx::lds_u32(lut_s + d * lut_stride);
                            w[j] = (full || key0 + 4 * g + j <= t) ? wv : 0u;
                        }
                        // 4 x 3 byte transpose: the weights of four consecutive keys -> one word per limb
                        const uint32_t t0 = __byte_perm(w[0], w[1], 0x5140), t1 = __byte_perm(w[2], w[3], 0x5140);
                        const uint32_t t2 = __byte_perm(w[0], w[1], 0x7362), t3 = __byte_perm(w[2], w[3], 0x7362);
                        l0[g] = __byte_perm(t0, t1, 0x5410);
                        l1[g] = __byte_perm(t0, t1, 0x7632);
                        l2[g] = __byte_perm(t2, t3, 0x5410);
                        tl0 = __dp4a((int)l0[g], 0x01010101, tl0);
                        tl1 = __dp4a((int)l1[g], 0x01010101, tl1);
                        tl2 = __dp4a((int)l2[g], 0x01010101, tl2);
                    }
                    const int t2i = colk >> 7, piece = (colk & 127) >> 4;
                    const uint32_t pt = p_s + (uint32_t)(t2i * 3) * 16384u;
                    ptx::sts_v4(sw128_addr(pt, row, piece), make_int4((int)l0[0], (int)l0[1], (int)l0[2], (int)l0[3]));
                    ptx::sts_v4(sw128_addr(pt + 16384u, row, piece), make_int4((int)l1[0], (int)l1[1], (int)l1[2], (int)l1[3]));
                    ptx::sts_v4(sw128_addr(pt + 32768u, row, piece), make_int4((int)l2[0], (int)l2[1], (int)l2[2], (int)l2[3]));
                }
                ptx::tc_fence_before();
                ptx::fence_proxy_async();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bars.p_ready);
            }
            part_sum[(0 * 4 + cp) * 128 + row] = tl0;
            part_sum[(1 * 4 + cp) * 128 + row] = tl1;
            part_sum[(2 * 4 + cp) * 128 + row] = tl2;
            ptx::named_bar_sync(2 + quarter, 128);
            const int d0 = part_sum[0 * 128 + row] + part_sum[1 * 128 + row] + part_sum[2 * 128 + row] + part_sum[3 * 128 + row];
            const int d1 = part_sum[4 * 128 + row] + part_sum[5 * 128 + row] + part_sum[6 * 128 + row] + part_sum[7 * 128 + row];
            const int d2 = part_sum[8 * 128 + row] + part_sum[9 * 128 + row] + part_sum[10 * 128 + row] + part_sum[11 * 128 + row];
            const uint32_t tot = (uint32_t)d0 + ((uint32_t)d1 << 7) + ((uint32_t)d2 << 14);
            const float rden = 1.0f / (float)(tot ? tot : 1u);
            const int e0 = tot ? d0 : 1, e1 = tot ? d1 : 0, e2 = tot ? d2 : 0;          // total_weight == 0 -> divide by 1 (mgpu.cu:818)

            // ---- output: 16 dims of this lane's row ----
            atc_wait(&bars.pv_done, n_pv++ & 1, &bars.abort_flag, err, DEV_TIMEOUT_TMEM_FULL);
            __syncwarp();
            ptx::tc_fence_after();
            uint32_t a0[16], a1[16], a2[16];
            ptx::tmem_ld16(t_lane + (uint32_t)(ATC_O_COL + cp * 16), a0);
            ptx::tmem_ld16(t_lane + (uint32_t)(ATC_O_COL + 64 + cp * 16), a1);
            ptx::tmem_ld16(t_lane + (uint32_t)(ATC_O_COL + 128 + cp * 16), a2);
            ptx::tmem_ld_wait16(a0); ptx::tmem_ld_wait16(a1); ptx::tmem_ld_wait16(a2);
            uint32_t ow[4];
            int dot = 0;
#pragma unroll
            for (int g = 0; g < 4; g++) {
                int o[4];
#pragma unroll
                for (int j = 0; j < 4; j++) o[j] = atc_div((int)a0[4 * g + j], (int)a1[4 * g + j], (int)a2[4 * g + j], e0, e1, e2, rden);
                ow[g] = ptx::pack_sat_s8(o[0], o[1], o[2], o[3]);           // |o| <= 127: a weighted mean of int8 values
                const int nbw = g == 0 ? nb4.x : (g == 1 ? nb4.y : (g == 2 ? nb4.z : nb4.w));
                dot = __dp4a((int)ow[g], nbw, dot);
            }
            *reinterpret_cast<int4 *>(p.ao + (base + t) * H + col0 + cp * 16) = make_int4((int)ow[0], (int)ow[1], (int)ow[2], (int)ow[3]);
            part_dot[cp * 128 + row] = dot;
            ptx::tc_fence_before();
            ptx::named_bar_sync(2 + quarter, 128);               // also: every part of this quarter has read the accumulators and part_sum
            if (cp == 0) atomicAdd(&p.xbo[base + t], part_dot[row] + part_dot[128 + row] + part_dot[256 + row] + part_dot[384 + row]);
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, 512);
    }
}


bool attention_tc_supported(int seq_len, int head_dim) { return seq_len % 128 == 0 && seq_len <= 512 && head_dim == 64; }

// =====================================================================================================================
// Hybrid form: scores and weights per warp on mma.sync (as attention_kernel does), Σ wt·v on tcgen05.
//
// What bounds attention_kernel is not its tensor work but the 96 int32 accumulators every lane carries for Σ wt·v
// (168 registers, 12 warps per SM, dependent MMA chains).  Here a worker warp still owns 16 queries and computes their
// scores, maxima and three-limb weights with m16n8k32 MMAs exactly as before, but instead of multiplying the limbs with
// V itself it writes them as int8 rows of three K-major operand tiles P_l[128 queries][128 keys] in shared memory
// (8 bytes per row, limb and 32-key block: the key order inside a 32-key block is permuted so that the lane's eight
// keys are adjacent; V^T is staged with the same permutation).  Warp 0 issues O_l += P_l V as tcgen05.mma kind::i8
// (M = 128, N = 64, K = 32 per 32-key block) as soon as the eight workers have delivered a block; the accumulators live
// in tensor memory (192 columns), so the workers run ahead with the next block while the tensor core works, need about
// 100 registers, and two blocks of 288 threads fit on an SM.  The exact recombination and division are those of
// attention_kernel.  One thread block per (member, head); needs seq_len % 128 == 0, head_dim 64.
// Every wait is bounded; a timeout makes all later waits fall through.
// =====================================================================================================================
constexpr int AHY_WORKERS = 8;
constexpr int AHY_THREADS = 32 * (1 + AHY_WORKERS);
constexpr int AHY_KP = 80;              // K row pitch for the mma.sync B fragments (conflict-free)

struct AhyBars {
    uint64_t p_ready[4];                // the workers have written 32-key block sb of the current chunk (8 arrivals)
    uint64_t p_free;                    // the MMAs that read the current chunk's operand tiles are done
    uint64_t o_full;                    // all MMAs of a query block are done
    uint64_t o_free;                    // the workers have read the accumulators (8 arrivals)
    uint32_t tmem_base;
    volatile int abort_flag;
};
struct AhyLayout { int vt, p, ks, lut, rsum, bars, total; };
static AhyLayout ahy_layout(int S) {
    AhyLayout L;
    int o = 0;
    L.vt = o; o += (S / 128) * 64 * 128;            // V^T operand tiles, one per 128 keys
    L.p = o; o += 3 * 128 * 128;                    // three limb operand tiles of the current 128-key chunk
    L.ks = o; o += S * AHY_KP;
    L.lut = o; o += 256 * 4;
    L.rsum = o; o += 2 * 3 * 128 * 4;               // limb sums of Σ wt per row, double-buffered over query blocks
    L.bars = o; o += 128;
    L.total = o + 1024;
    return L;
}

__device__ __forceinline__ void mma_s8_sync(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8_sync_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// scores of one 16-query x 32-key block: c[nt][0..3] for the four 8-key n-tiles (rows g and g+8, keys nt*8 + 2q, +1)
__device__ __forceinline__ void ahy_scores(int (&c)[4][4], const uint32_t (&qa)[2][4], const int8_t *Ks, int kb, int g, int q) {
#pragma unroll
    for (int nt = 0; nt < 4; nt++) {
        const int8_t *kp = Ks + (kb * 32 + nt * 8 + g) * AHY_KP + 4 * q;
        mma_s8_sync_first(c[nt], qa[0][0], qa[0][1], qa[0][2], qa[0][3], *reinterpret_cast<const uint32_t *>(kp), *reinterpret_cast<const uint32_t *>(kp + 16));
        mma_s8_sync(c[nt], qa[1][0], qa[1][1], qa[1][2], qa[1][3], *reinterpret_cast<const uint32_t *>(kp + 32), *reinterpret_cast<const uint32_t *>(kp + 48));
    }
}

__global__ void __launch_bounds__(AHY_THREADS, 2) attention_hy_kernel(const AttnParams p, const AhyLayout L, int *err) {
    extern __shared__ uint8_t ahy_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(ahy_raw) + 1023) & ~uintptr_t(1023));
    AhyBars &bars = *reinterpret_cast<AhyBars *>(sm + L.bars);
    const int8_t *Ks = reinterpret_cast<const int8_t *>(sm + L.ks);
    uint32_t *lut3 = reinterpret_cast<uint32_t *>(sm + L.lut);
    int32_t *rsum = reinterpret_cast<int32_t *>(sm + L.rsum);                 // [2][3][128]
    const uint32_t vt_s = ptx::smem_u32(sm + L.vt), p_s = ptx::smem_u32(sm + L.p);

    const int S = p.seq_len, H = p.H;
    const int n_heads = H / 64;
    const int mem = blockIdx.x / n_heads, hd = blockIdx.x % n_heads;
    const int64_t base = (int64_t)mem * S;
    const int col0 = hd * 64;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NQ = S / 128;
    const int sh = p.shift_attn;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; i++) ptx::mbar_init(&bars.p_ready[i], AHY_WORKERS);
        ptx::mbar_init(&bars.p_free, 1);
        ptx::mbar_init(&bars.o_full, 1);
        ptx::mbar_init(&bars.o_free, AHY_WORKERS);
        bars.abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 0) {
        ptx::tmem_alloc(&bars.tmem_base, 256);
        ptx::tmem_relinquish();
    } else {
        // ---- stage K (padded rows for the mma.sync fragments), V^T (tensor-core operand tiles, permuted keys), the table ----
        const int tid = threadIdx.x - 32;                                     // 0..255
        for (int i = tid; i < S * 4; i += 32 * AHY_WORKERS) {
            const int row = i >> 2, ch = i & 3;
            const int4 v = *reinterpret_cast<const int4 *>(p.k + (base + row) * H + col0 + ch * 16);
            *reinterpret_cast<int4 *>(sm + L.ks + row * AHY_KP + ch * 16) = v;
        }
        // V: one item = two consecutive keys x 16 dims -> for every dim the two bytes, at the keys' permuted position
        // (key 8nt + 2q + b of a 32-key block sits at byte 8q + 2nt + b of the block)
        for (int i = tid; i < (S / 2) * 4; i += 32 * AHY_WORKERS) {
            const int kp2 = i % (S / 2), dch = i / (S / 2);
            const int key = 2 * kp2;
            const int4 v0 = *reinterpret_cast<const int4 *>(p.v + (base + key) * H + col0 + dch * 16);
            const int4 v1 = *reinterpret_cast<const int4 *>(p.v + (base + key + 1) * H + col0 + dch * 16);
            const int k32 = key & 31;
            const int pos = (key & ~31) + 8 * ((k32 & 7) >> 1) + 2 * (k32 >> 3);
            const uint32_t tile = vt_s + (uint32_t)(pos >> 7) * 8192u;
            const int pin = pos & 127;
            const uint32_t *w0 = reinterpret_cast<const uint32_t *>(&v0), *w1 = reinterpret_cast<const uint32_t *>(&v1);
#pragma unroll
            for (int dq = 0; dq < 4; dq++) {
                const uint32_t t0 = __byte_perm(w0[dq], w1[dq], 0x5140), t1 = __byte_perm(w0[dq], w1[dq], 0x7362);   // [a0 b0 a1 b1], [a2 b2 a3 b3]
                const uint32_t pr[4] = {t0 & 0xFFFFu, t0 >> 16, t1 & 0xFFFFu, t1 >> 16};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int dim = dch * 16 + dq * 4 + j;
                    const uint32_t a = sw128_addr(tile, dim, pin >> 4) + (uint32_t)(pin & 15);
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"((unsigned short)pr[j]) : "memory");
                }
            }
        }
        {
            const uint32_t w = (uint32_t)p.exp_lut[tid & 255];
            lut3[tid & 255] = (w & 127u) | (((w >> 7) & 127u) << 8) | ((w >> 14) << 16);
        }
        ptx::fence_proxy_async();             // the V^T tiles are read by the tensor core
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = bars.tmem_base;

    if (warp == 0) {
        // ===================== MMA issuer =====================
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::make_idesc_i8(128, 64);
            uint32_t n_chunk = 0;
            for (int qt = 0; qt < NQ && !bars.abort_flag; qt++) {
                if (qt > 0) {        // the workers have read the previous block's accumulators
                    atc_wait(&bars.o_free, (uint32_t)(qt - 1) & 1u, &bars.abort_flag, err, DEV_TIMEOUT_TMEM_EMPTY);
                    ptx::tc_fence_after();
                }
                for (int ch = 0; ch <= qt && !bars.abort_flag; ch++, n_chunk++) {
                    const uint64_t dv = ptx::make_smem_desc_sw128(vt_s + (uint32_t)ch * 8192u);
                    for (int sb = 0; sb < 4 && !bars.abort_flag; sb++) {
                        atc_wait(&bars.p_ready[sb], n_chunk & 1u, &bars.abort_flag, err, DEV_TIMEOUT_FULL);
                        if (bars.abort_flag) break;
                        ptx::tc_fence_after();
#pragma unroll
                        for (int l = 0; l < 3; l++) {
                            const uint64_t dp = ptx::make_smem_desc_sw128(p_s + (uint32_t)l * 16384u);
                            ptx::mma_i8(tmem_base + (uint32_t)(64 * l), dp + (uint64_t)(2 * sb), dv + (uint64_t)(2 * sb), idesc, (ch > 0 || sb > 0) ? 1u : 0u);
                        }
                    }
                    if (!bars.abort_flag) ptx::mma_commit(&bars.p_free);
                }
                if (!bars.abort_flag) ptx::mma_commit(&bars.o_full);
            }
        }
    } else {
        // ===================== workers (8 warps) =====================
        const int w = warp - 1;                     // 16 queries of every block: rows 16w .. 16w+15
        const int quarter = warp & 3;               // tensor-memory lane quarter this warp may read
        const int half = w >> 2;                    // which 32 of the 64 output dims it divides and stores
        const int g = lane >> 2, q = lane & 3;
        const int8_t *nbo = p.nt + (int64_t)(mem >> 1) * p.nt_stride + p.nt_o_b + col0 + half * 32;
        const int4 nb4a = *reinterpret_cast<const int4 *>(nbo), nb4b = *reinterpret_cast<const int4 *>(nbo + 16);
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        uint32_t n_chunk = 0;

        for (int qt = 0; qt < NQ; qt++) {
            const int q0 = qt * 128 + 16 * w;
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
            const int last = (q0 + 15) / 32;          // the only key block of this warp that needs the causal mask

            // ---- pass 1: row maxima over ctx <= t (mgpu.cu:795-802) ----
            int mx0 = INT_MIN, mx1 = INT_MIN;
            int c[4][4];
            for (int kb = 0; kb < last; kb++) {
                ahy_scores(c, qa, Ks, kb, g, q);
#pragma unroll
                for (int nt = 0; nt < 4; nt++) { mx0 = __vimax3_s32(mx0, c[nt][0], c[nt][1]); mx1 = __vimax3_s32(mx1, c[nt][2], c[nt][3]); }
            }
            ahy_scores(c, qa, Ks, last, g, q);
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

            // ---- pass 2: weights as three limbs -> operand tiles; limb sums of Σ wt (mgpu.cu:810-824) ----
            int tl0[3] = {0, 0, 0}, tl1[3] = {0, 0, 0};
            const int tr0 = 16 * w + g, tr1 = tr0 + 8;                        // rows inside the 128-query operand tiles
            for (int ch = 0; ch <= qt; ch++, n_chunk++) {
                if (n_chunk > 0) {          // the previous chunk's MMAs still read the tiles
                    atc_wait(&bars.p_free, (n_chunk - 1) & 1u, &bars.abort_flag, err, DEV_TIMEOUT_TMEM_FULL);
                    __syncwarp();
                }
#pragma unroll 1
                for (int sb = 0; sb < 4; sb++) {
                    const int kb = ch * 4 + sb;
                    uint32_t al[3][4];          // limb l: [0] row g keys of n-tiles 0,1; [1] row g+8; [2] row g n-tiles 2,3; [3] row g+8
                    if (kb <= last) {
                        ahy_scores(c, qa, Ks, kb, g, q);
                        uint32_t wt[4][4];
                        if (kb < last) {
#pragma unroll
                            for (int nt = 0; nt < 4; nt++) {
                                wt[nt][0] = lut3[min(255, mxs0 - (c[nt][0] >> sh))];
                                wt[nt][1] = lut3[min(255, mxs0 - (c[nt][1] >> sh))];
                                wt[nt][2] = lut3[min(255, mxs1 - (c[nt][2] >> sh))];
                                wt[nt][3] = lut3[min(255, mxs1 - (c[nt][3] >> sh))];
                            }
                        } else {
#pragma unroll
                            for (int nt = 0; nt < 4; nt++) {
                                const int key = kb * 32 + nt * 8 + 2 * q;
                                wt[nt][0] = (key <= row0) ? lut3[min(255u, (uint32_t)(mxs0 - (c[nt][0] >> sh)))] : 0u;
                                wt[nt][1] = (key + 1 <= row0) ? lut3[min(255u, (uint32_t)(mxs0 - (c[nt][1] >> sh)))] : 0u;
                                wt[nt][2] = (key <= row1) ? lut3[min(255u, (uint32_t)(mxs1 - (c[nt][2] >> sh)))] : 0u;
                                wt[nt][3] = (key + 1 <= row1) ? lut3[min(255u, (uint32_t)(mxs1 - (c[nt][3] >> sh)))] : 0u;
                            }
                        }
#pragma unroll
                        for (int f = 0; f < 4; f++) {
                            // 4 x 3 byte transpose of the four weights of word f (7 byte permutes)
                            const int n0 = (f >> 1) * 2, i0 = (f & 1) * 2;
                            const uint32_t wa = wt[n0][i0], wb = wt[n0][i0 + 1], wc = wt[n0 + 1][i0], wd = wt[n0 + 1][i0 + 1];
                            const uint32_t t0 = __byte_perm(wa, wb, 0x5140), t1 = __byte_perm(wc, wd, 0x5140);
                            const uint32_t t2 = __byte_perm(wa, wb, 0x7362), t3 = __byte_perm(wc, wd, 0x7362);
                            al[0][f] = __byte_perm(t0, t1, 0x5410);
                            al[1][f] = __byte_perm(t0, t1, 0x7632);
                            al[2][f] = __byte_perm(t2, t3, 0x5410);
                        }
#pragma unroll
                        for (int l = 0; l < 3; l++) {
                            tl0[l] = __dp4a((int)al[l][0], 0x01010101, __dp4a((int)al[l][2], 0x01010101, tl0[l]));
                            tl1[l] = __dp4a((int)al[l][1], 0x01010101, __dp4a((int)al[l][3], 0x01010101, tl1[l]));
                        }
                    } else {
#pragma unroll
                        for (int l = 0; l < 3; l++)
#pragma unroll
                            for (int f = 0; f < 4; f++) al[l][f] = 0u;       // keys beyond this warp's queries: zero rows
                    }
                    // bytes 8q .. 8q+7 of the block (keys nt*8 + 2q + b at 8q + 2nt + b) of rows tr0 and tr1, one 8-byte store each
                    const int piece = 2 * sb + (q >> 1);
                    const uint32_t bo = (uint32_t)(q & 1) * 8u;
#pragma unroll
                    for (int l = 0; l < 3; l++) {
                        const uint32_t tile = p_s + (uint32_t)l * 16384u;
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(sw128_addr(tile, tr0, piece) + bo), "r"(al[l][0]), "r"(al[l][2]) : "memory");
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(sw128_addr(tile, tr1, piece) + bo), "r"(al[l][1]), "r"(al[l][3]) : "memory");
                    }
                    ptx::fence_proxy_async();             // generic-proxy writes -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&bars.p_ready[sb]);
                }
            }
#pragma unroll
            for (int l = 0; l < 3; l++) {                 // limb sums of Σ wt over the four lanes that share a row
                tl0[l] += __shfl_xor_sync(0xFFFFFFFFu, tl0[l], 1); tl0[l] += __shfl_xor_sync(0xFFFFFFFFu, tl0[l], 2);
                tl1[l] += __shfl_xor_sync(0xFFFFFFFFu, tl1[l], 1); tl1[l] += __shfl_xor_sync(0xFFFFFFFFu, tl1[l], 2);
            }
            int32_t *rs = rsum + (qt & 1) * 3 * 128;
            if (q == 0) {
#pragma unroll
                for (int l = 0; l < 3; l++) { rs[l * 128 + tr0] = tl0[l]; rs[l * 128 + tr1] = tl1[l]; }
            }
            ptx::named_bar_sync(1, 32 * AHY_WORKERS);     // the sums of all 128 rows are in place

            // ---- output: this lane's row of the block, 32 of its 64 dims ----
            const int rowt = quarter * 32 + lane;
            const int t = qt * 128 + rowt;
            const int d0 = rs[rowt], d1 = rs[128 + rowt], d2 = rs[256 + rowt];
            const uint32_t tot = (uint32_t)d0 + ((uint32_t)d1 << 7) + ((uint32_t)d2 << 14);
            const float rden = 1.0f / (float)(tot ? tot : 1u);
            const int e0 = tot ? d0 : 1, e1 = tot ? d1 : 0, e2 = tot ? d2 : 0;          // total_weight == 0 -> divide by 1 (mgpu.cu:818)
            atc_wait(&bars.o_full, (uint32_t)qt & 1u, &bars.abort_flag, err, DEV_TIMEOUT_TMEM_FULL);
            __syncwarp();
            ptx::tc_fence_after();
            int dot = 0;
#pragma unroll
            for (int rd = 0; rd < 2; rd++) {
                uint32_t a0[16], a1[16], a2[16];
                const uint32_t colb = (uint32_t)(half * 32 + rd * 16);
                ptx::tmem_ld16(t_lane + colb, a0);
                ptx::tmem_ld16(t_lane + 64u + colb, a1);
                ptx::tmem_ld16(t_lane + 128u + colb, a2);
                ptx::tmem_ld_wait16(a0); ptx::tmem_ld_wait16(a1); ptx::tmem_ld_wait16(a2);
                uint32_t ow[4];
                const int4 nb4 = rd == 0 ? nb4a : nb4b;
#pragma unroll
                for (int gg = 0; gg < 4; gg++) {
                    int o[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) o[j] = atc_div((int)a0[4 * gg + j], (int)a1[4 * gg + j], (int)a2[4 * gg + j], e0, e1, e2, rden);
                    ow[gg] = ptx::pack_sat_s8(o[0], o[1], o[2], o[3]);          // |o| <= 127: a weighted mean of int8 values
                    const int nbw = gg == 0 ? nb4.x : (gg == 1 ? nb4.y : (gg == 2 ? nb4.z : nb4.w));
                    dot = __dp4a((int)ow[gg], nbw, dot);
                }
                *reinterpret_cast<int4 *>(p.ao + (base + t) * H + col0 + half * 32 + rd * 16) = make_int4((int)ow[0], (int)ow[1], (int)ow[2], (int)ow[3]);
            }
            atomicAdd(&p.xbo[base + t], dot);              // the two warps of a row add their halves
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&bars.o_free);
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, 256);
    }
}

int launch_attention_hy(cudaStream_t st, const AttnParams &p, int *err) {
    if (!attention_tc_supported(p.seq_len, p.head_dim)) { set_error("tensor-core attention needs seq_len %% 128 == 0, seq_len <= 512, head_dim 64"); return EGG_E_INVALID; }
    const AhyLayout L = ahy_layout(p.seq_len);
    static int configured[EGG_MAX_DEVICES] = {};
    const int dev = current_device_slot();
    if (L.total > configured[dev]) {
        EGG_CUDA(cudaFuncSetAttribute(attention_hy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total));
        configured[dev] = L.total;
    }
    const int blocks = p.members * (p.H / 64);
    attention_hy_kernel<<<blocks, AHY_THREADS, L.total, st>>>(p, L, err);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

int launch_attention_tc(cudaStream_t st, const AttnParams &p, int *err) {
    if (!attention_tc_supported(p.seq_len, p.head_dim)) { set_error("tensor-core attention needs seq_len %% 128 == 0, seq_len <= 512, head_dim 64"); return EGG_E_INVALID; }
    const AtcLayout L = atc_layout(p.seq_len);
    static int configured[EGG_MAX_DEVICES] = {};
    const int dev = current_device_slot();
    if (L.total > configured[dev]) {
        EGG_CUDA(cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total));
        configured[dev] = L.total;
    }
    const int blocks = p.members * (p.H / 64);
    attention_tc_kernel<<<blocks, ATC_THREADS, L.total, st>>>(p, L, err);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

}  // namespace egg
