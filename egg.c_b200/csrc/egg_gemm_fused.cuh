// Row-owning int8 GEMM for sm_100a: the projections whose results pass through one of the reference's adaptive
// normalisations (adaptive_qkv_normalize / adaptive_layer_normalize, egg_adaptive_normalize.h:10-103) before anything
// else reads them.  Those normalisations need the abs-max of a WHOLE output row of H values, so one thread block
// keeps all H int32 accumulators of its 128 rows in tensor memory (H <= 512 = the 512 TMEM columns), finds the row
// maximum there and writes the requantised int8 row directly:
//
//   FUSED_QKV   q, k, v = AQN(rope(h.Wq + r1)), AQN(rope(h.Wk + r1)), AQN(h.Wv + r1)       (mgpu.cu:779-784)
//   FUSED_RES   x       = ALN(x + ((a.W + r1) >> shift) + bias + bias noise)                (mgpu.cu:746-756, 829-830)
//
// with r1 = ((Σ_k a_k b_k) * a_n * sign) >> (FIXED_POINT + SIGMA_SHIFT) (compute_linear_projection, mgpu.cu:553-572).
// A work unit is one 128-row tile of one part (q, k or v; the single part of FUSED_RES), made of H/BN sub-tiles of BN
// columns that occupy consecutive slots of a ring of 512/BN TMEM slots.  Roles: warp 0 feeds a shared-memory ring by
// TMA, warp 1 issues tcgen05.mma kind::i8, warps 2..17 are the epilogue (4 TMEM lane quarters x 4 column quarters;
// lane = row).  Per unit the epilogue makes two passes over tensor memory:
//   pass 1 (per sub-tile, as soon as its MMAs are done): rank-1 term, RoPE / residual + bias, running abs-max per
//          lane; the int32 values go back to the same TMEM columns (tcgen05.st);
//   the four warps that share a lane quarter exchange their maxima through shared memory (128-thread named barrier);
//   pass 2 (per sub-tile): requantise (aln_quant_f), pack, write the warp's 32 x BN/4 int8 box to shared memory, release
//          the TMEM slot to the MMA warp, store the box with one TMA store.
// So the MMAs of the next unit's first sub-tile overlap pass 2 of this unit's last, and no int32 intermediate ever
// reaches HBM.  Rows of a tile must belong to one population member: seq_len % 128 == 0 (then M % 128 == 0 too).
// No multicast anywhere; every wait is bounded and a timeout makes all later waits fall through so that the block
// drains, frees its tensor memory and reports.
#pragma once

#include "egg_gemm.cuh"

namespace egg {

enum FusedMode { FUSED_QKV = 0, FUSED_RES = 1, FUSED_RES_LN = 2 };

struct FusedParams {
    int M, H, K;                 // rows (multiple of 128), width of one part, contraction
    int cl;                      // thread blocks that share a unit (1 or 2, = the cluster size of the launch): each owns
                                 // H/cl <= 512 columns of the unit's rows and the row maxima are exchanged through the
                                 // peer's shared memory
    int parts;                   // 3 (q, k, v: B is [3H][K]) or 1
    int seq_len;                 // multiple of 128
    const int8_t *nt;            // per-pair noise table of this wave
    int64_t nt_stride;
    int nt_a_off;                // A-noise of part 0 (length H); part p at + p*H
    int nt_c_off;                // FUSED_RES: bias-noise deltas [2][H] (-1: none)
    const int32_t *xb;           // Σ_k a_k b_k per row and part: xb[r * xb_stride + part]
    int xb_stride;
    int rank1_shift, out_shift;
    int one;                     // 1 (filled by launch_gemm_fused): the multiplier of additions issued as multiply-adds
    const int8_t *bias;          // FUSED_RES: [H] or null
    const int2 *rope_t;          // [head_dim/2][seq_len] (cos, sin)
    int head_dim, rope_bit;
    int64_t part_rows;           // row distance between the parts in the output tensor map
    int *err;
    FastDiv fd_head, fd_h;       // head_dim and H as multiply-shift divisors (filled by launch_gemm_fused)
    // FUSED_RES_LN: the mean-abs norm that follows the block (apply_standard_norm, mgpu.cu:646-678) and the row dots of
    // the projections after it, computed from the requantised row while it is still in shared memory
    int nt_w_m, nt_b_m;          // perturbed gain / bias tables (int16 [2][H]) in the noise table
    int ndots, nt_dot[3];        // B-noise vectors of the following projections
    int8_t *h_out;               // [M][H] normalised rows
    int32_t *xb_out;             // [M][xb_out_stride] row dots, ADDED to (cleared by the caller)
    int xb_out_stride;
};

constexpr int FUSED_MAX_H = 512;

template <int BN>
struct FusedSmem {
    static constexpr int NS = 512 / BN;                 // TMEM slots = most sub-tiles a unit can have
    static constexpr int BOX = 32 * (BN / 4);           // bytes of one warp's int8 box: 32 rows x BN/4 columns
    alignas(1024) uint8_t a[GEMM_STAGES][GEMM_BM * GEMM_BK];
    alignas(1024) uint8_t b[GEMM_STAGES][BN * GEMM_BK];
    // per epilogue warp and sub-tile: residual bytes in (FUSED_RES), requantised bytes out
    alignas(1024) uint8_t box[GEMM_EPI_WARPS][NS][BOX];
    alignas(16) int32_t a32[2][FUSED_MAX_H];            // A-noise of the unit (double-buffered across units)
    alignas(16) int32_t bcs32[2][FUSED_MAX_H];          // (bias + bias-noise delta of the member's sign) << out_shift
    alignas(16) int32_t rowpart[4][GEMM_BM];            // per-row abs-max of each column quarter
    alignas(16) int32_t peer_max[2][GEMM_BM];           // per-row abs-max of the peer block's columns (written by the peer)
    alignas(16) uint16_t rowsum[4][GEMM_BM];            // FUSED_RES_LN: per-row Σ|x| of each column quarter (<= 127 * 128 columns)
    alignas(16) int32_t peer_sum[2][GEMM_BM];           // ... and of the peer block's columns
    // FUSED_RES_LN, per group of 4 columns: the member's perturbed gains and biases {w0 w1 | w2 w3 | b0 b1 | b2 b3} (int16
    // pairs), and the B-noise of the following projections {dot 0 | dot 1 | dot 2 | -} (four int8 each): one 16-byte read each
    alignas(16) int4 ln_wb[FUSED_MAX_H / 4];
    alignas(16) int4 ln_d4[FUSED_MAX_H / 4];
    alignas(8) uint64_t xbar[2];                        // arrival of the peer's maxima, one barrier per unit parity
    uint64_t xbar2[2];                                  // arrival of the peer's sums
    alignas(8) uint64_t full[GEMM_STAGES];
    uint64_t empty[GEMM_STAGES];
    uint64_t tmem_full[NS];
    uint64_t tmem_empty[NS];
    uint64_t rbar[GEMM_EPI_WARPS][NS];                  // arrival of a residual box
    uint32_t tmem_base;
    volatile int abort_flag;
};

namespace ptx {
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
}  // namespace ptx

// Waits for an mbarrier phase unless the block is already draining after a timeout; a timeout here starts the drain.
__device__ __forceinline__ void fused_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *err, int code) {
    if (*abort_flag) return;
    if (!ptx::mbar_wait(bar, parity, 1000000000ull)) {
        *abort_flag = 1;
        if (err) atomicCAS(err, 0, code);
    }
}

// Words of the next unit's tables, loaded a unit ahead.
struct FusedTabWords { int32_t a, b, d; };
// One thread's share (4 columns) of the norm tables of a unit's member (FUSED_RES_LN).
struct FusedLnWords { int2 w, b; int32_t d[3]; };

template <int BN, int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_fused_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_o, const __grid_constant__ CUtensorMap tmap_r, const FusedParams p) {
    extern __shared__ uint8_t smem_raw[];
    FusedSmem<BN> &sm = *reinterpret_cast<FusedSmem<BN> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int NS = FusedSmem<BN>::NS;
    constexpr int CW = BN / 4;                  // columns of a sub-tile that one epilogue warp owns
    constexpr int NCH = CW / 16;                // 16-column chunks per warp and sub-tile
    constexpr uint32_t STAGE_BYTES = GEMM_BM * GEMM_BK + BN * GEMM_BK;
    constexpr bool RES = (MODE != FUSED_QKV);   // residual + bias projections (O, MLP down)
    constexpr bool LN = (MODE == FUSED_RES_LN); // ... followed in the same epilogue by the next mean-abs norm

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int HL = p.H / p.cl;                                      // columns of a part this block owns
    const int crank = (int)blockIdx.x % p.cl;                       // rank in the cluster (clusters are consecutive blocks)
    const int cofs = crank * HL;                                    // first of them
    const int first_unit = (int)blockIdx.x / p.cl, unit_step = (int)gridDim.x / p.cl;      // both blocks of a pair walk the same units
    const int NT = HL / BN;                                         // sub-tiles per unit, 1..NS
    const int num_units = (p.M / GEMM_BM) * p.parts;
    const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_STAGES; s++) { ptx::mbar_init(&sm.full[s], 1); ptx::mbar_init(&sm.empty[s], 1); }
        for (int a = 0; a < NS; a++) { ptx::mbar_init(&sm.tmem_full[a], 1); ptx::mbar_init(&sm.tmem_empty[a], GEMM_EPI_WARPS); }
        for (int w = 0; w < GEMM_EPI_WARPS; w++)
            for (int a = 0; a < NS; a++) ptx::mbar_init(&sm.rbar[w][a], 1);
        ptx::mbar_init(&sm.xbar[0], GEMM_EPI_THREADS / 4);       // the peer's first column quarter: one arrival per row
        ptx::mbar_init(&sm.xbar[1], GEMM_EPI_THREADS / 4);
        ptx::mbar_init(&sm.xbar2[0], GEMM_EPI_THREADS / 4);
        ptx::mbar_init(&sm.xbar2[1], GEMM_EPI_THREADS / 4);
        sm.abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(&sm.tmem_base, 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    if (p.cl > 1) ptx::cluster_sync_all();          // the peer's barriers exist before anything arrives on them
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == 0) {
        // ===================== TMA producer =====================
        if (ptx::elect_one()) {
            ptx::prefetch_tmap(&tmap_a);
            ptx::prefetch_tmap(&tmap_b);
            uint32_t it = 0;
            for (int unit = first_unit; unit < num_units && !sm.abort_flag; unit += unit_step) {
                const int mt = unit / p.parts, part = unit - mt * p.parts;
                const int m0 = mt * GEMM_BM;
                for (int j = 0; j < NT; j++) {
                    const int n0 = part * p.H + cofs + j * BN;
                    for (int kb = 0; kb < num_kb; kb++, it++) {
                        const int s = it % GEMM_STAGES;
                        const uint32_t ph = (it / GEMM_STAGES) & 1;
                        fused_wait(&sm.empty[s], ph ^ 1, &sm.abort_flag, p.err, DEV_TIMEOUT_EMPTY);
                        if (sm.abort_flag) break;
                        ptx::mbar_arrive_expect_tx(&sm.full[s], STAGE_BYTES);
                        ptx::tma_load_2d(sm.a[s], &tmap_a, &sm.full[s], kb * GEMM_BK, m0);
                        ptx::tma_load_2d(sm.b[s], &tmap_b, &sm.full[s], kb * GEMM_BK, n0);
                    }
                    if (sm.abort_flag) break;
                }
            }
            if (sm.abort_flag) {   // let copies already in flight land before the block tears down
                const uint64_t t0 = ptx::globaltimer();
                while (ptx::globaltimer() - t0 < 200000ull) { __nanosleep(1000); }
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::make_idesc_i8(GEMM_BM, BN);
            uint32_t it = 0, stc = 0;
            for (int unit = first_unit; unit < num_units && !sm.abort_flag; unit += unit_step) {
                for (int j = 0; j < NT && !sm.abort_flag; j++, stc++) {
                    const int slot = stc % NS;
                    const uint32_t sph = (stc / NS) & 1;
                    fused_wait(&sm.tmem_empty[slot], sph ^ 1, &sm.abort_flag, p.err, DEV_TIMEOUT_TMEM_EMPTY);
                    if (sm.abort_flag) break;
                    ptx::tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)(slot * BN);
                    for (int kb = 0; kb < num_kb; kb++, it++) {
                        const int s = it % GEMM_STAGES;
                        const uint32_t ph = (it / GEMM_STAGES) & 1;
                        fused_wait(&sm.full[s], ph, &sm.abort_flag, p.err, DEV_TIMEOUT_FULL);
                        if (sm.abort_flag) break;
                        ptx::tc_fence_after();
                        const uint64_t da = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.a[s]));
                        const uint64_t db = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.b[s]));
#pragma unroll
                        for (int k = 0; k < GEMM_BK / 32; k++)
                            ptx::mma_i8(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        ptx::mma_commit(&sm.empty[s]);
                    }
                    if (!sm.abort_flag) ptx::mma_commit(&sm.tmem_full[slot]);
                }
            }
        }
    } else {
        // ===================== epilogue (16 warps) =====================
        const int e = threadIdx.x - 64;            // 0..511
        const int ew = warp - 2;                   // 0..15
        const int quarter = warp & 3;              // TMEM lane quarter this warp may read
        const int cq = ew >> 2;                    // column quarter of every sub-tile
        const int row_in_tile = quarter * 32 + lane;
        const int tab_items = HL >> 2;             // one item = 4 consecutive columns of this block's share
        const long long half_ulp = 1ll << (p.rope_bit - 1);
        // shared address of this lane's row inside a box, and the XOR that swizzles its 16-byte pieces (64-byte swizzle
        // for 64-byte rows; 32-byte rows are stored densely)
        const uint32_t row_ofs = (uint32_t)lane * (uint32_t)CW;
        const uint32_t swz = (BN == 256) ? (uint32_t)((lane >> 1) & 3) : 0u;
        uint32_t stc = 0;
        int ucount = 0;
        int pf_xb = 0;
        FusedTabWords nxt = {0, 0, 0};
        bool have_nxt = false;

        auto tab_load = [&](int unit, FusedTabWords &w) -> bool {
            if (e >= tab_items) return false;
            const int mt = unit / p.parts, part = unit - mt * p.parts;
            const int mem = (mt * GEMM_BM) / p.seq_len;
            const int8_t *base = p.nt + (int64_t)(mem >> 1) * p.nt_stride;
            const int n = cofs + (e << 2);
            w.a = *reinterpret_cast<const int32_t *>(base + p.nt_a_off + part * p.H + n);
            w.b = 0; w.d = 0;
            if (RES) {
                if (p.bias) w.b = *reinterpret_cast<const int32_t *>(p.bias + n);
                if (p.nt_c_off >= 0) w.d = *reinterpret_cast<const int32_t *>(base + p.nt_c_off + (mem & 1) * p.H + n);
            }
            return true;
        };
        auto tab_store = [&](int buf, const FusedTabWords &w) {
            const int n = e << 2;
            *reinterpret_cast<int4 *>(&sm.a32[buf][n]) = make_int4((int)(int8_t)w.a, (int)(int8_t)(w.a >> 8), (int)(int8_t)(w.a >> 16), w.a >> 24);
            if (RES) {
                int v[4];
#pragma unroll
                for (int b = 0; b < 4; b++)      // pre-shifted so that the sum joins the rank-1 product before its shift
                    v[b] = ((int)(int8_t)(w.b >> (8 * b)) + (int)(int8_t)(w.d >> (8 * b))) << (p.out_shift + (GEMM_FMA_ADDS ? p.rank1_shift : 0));
                *reinterpret_cast<int4 *>(&sm.bcs32[buf][n]) = make_int4(v[0], v[1], v[2], v[3]);
            }
        };
        auto resid_request = [&](int unit) {      // lane 0: residual boxes of a unit, one per sub-tile
            const int m0 = (unit / p.parts) * GEMM_BM;
            for (int j = 0; j < NT; j++) {
                ptx::mbar_arrive_expect_tx(&sm.rbar[ew][j], 32 * CW);
                ptx::tma_load_2d(sm.box[ew][j], &tmap_r, &sm.rbar[ew][j], cofs + j * BN + cq * CW, m0 + quarter * 32);
            }
        };

        auto ln_load = [&](int mem, FusedLnWords &w) {      // threads e < tab_items: gains, biases and dot vectors of 4 columns
            const int8_t *base = p.nt + (int64_t)(mem >> 1) * p.nt_stride;
            const int n = cofs + (e << 2);
            w.w = *reinterpret_cast<const int2 *>(reinterpret_cast<const int16_t *>(base + p.nt_w_m) + (mem & 1) * p.H + n);
            w.b = *reinterpret_cast<const int2 *>(reinterpret_cast<const int16_t *>(base + p.nt_b_m) + (mem & 1) * p.H + n);
#pragma unroll
            for (int q = 0; q < 3; q++) w.d[q] = q < p.ndots ? *reinterpret_cast<const int32_t *>(base + p.nt_dot[q] + n) : 0;
        };
        auto ln_store = [&](const FusedLnWords &w) {
            sm.ln_wb[e] = make_int4(w.w.x, w.w.y, w.b.x, w.b.y);
            sm.ln_d4[e] = make_int4(w.d[0], w.d[1], w.d[2], 0);
        };

        const uint32_t peer_max_s = p.cl > 1 ? ptx::mapa_u32(ptx::smem_u32(&sm.peer_max[0][0]), (uint32_t)(crank ^ 1)) : 0u;
        const uint32_t peer_bar_s = p.cl > 1 ? ptx::mapa_u32(ptx::smem_u32(&sm.xbar[0]), (uint32_t)(crank ^ 1)) : 0u;
        const uint32_t peer_sum_s = (LN && p.cl > 1) ? ptx::mapa_u32(ptx::smem_u32(&sm.peer_sum[0][0]), (uint32_t)(crank ^ 1)) : 0u;
        const uint32_t peer_bar2_s = (LN && p.cl > 1) ? ptx::mapa_u32(ptx::smem_u32(&sm.xbar2[0]), (uint32_t)(crank ^ 1)) : 0u;
        for (int unit = first_unit; unit < num_units; unit += unit_step, ucount++) {
            const int mt = unit / p.parts, part = unit - mt * p.parts;
            const int m0 = mt * GEMM_BM;
            const int r = m0 + row_in_tile;
            const int mem = m0 / p.seq_len;
            const int sgn = mem & 1;
            const int tb = ucount & 1;
            if (ucount == 0) {
                FusedTabWords w;
                if (tab_load(unit, w)) tab_store(0, w);
                pf_xb = p.xb[(int64_t)r * p.xb_stride + part];
                if (RES && lane == 0) resid_request(unit);
            }
            // tables of this unit are published; everybody has left the previous unit
            ptx::named_bar_sync(1, GEMM_EPI_THREADS);
            const int xbs = sgn ? -pf_xb : pf_xb;
            const int nunit = unit + unit_step;
            have_nxt = false;
            if (nunit < num_units) {
                have_nxt = tab_load(nunit, nxt);
                const int nmt = nunit / p.parts;
                pf_xb = p.xb[(int64_t)(nmt * GEMM_BM + row_in_tile) * p.xb_stride + (nunit - nmt * p.parts)];
            }
            // the norm tables of this unit's member: requested now, stored after pass 1 (nobody reads the previous unit's
            // any more, and this unit's readers come after a 512-thread barrier)
            FusedLnWords lnw;
            if (LN && e < tab_items) ln_load(mem, lnw);
            const uint32_t a32_s = ptx::smem_u32(&sm.a32[tb][0]);
            const uint32_t bcs_s = ptx::smem_u32(&sm.bcs32[tb][0]);
            const bool do_rope = (MODE == FUSED_QKV) && part < 2;
            const int2 *rope = p.rope_t + (r - mem * p.seq_len);           // column of this token position

            // ---------------- pass 1: values and row abs-max, written back to tensor memory ----------------
            int rmx = 0, rmn = 0;
            for (int j = 0; j < NT; j++) {
                const uint32_t st = stc + (uint32_t)j;
                const int slot = st % NS;
                fused_wait(&sm.tmem_full[slot], (st / NS) & 1, &sm.abort_flag, p.err, DEV_TIMEOUT_TMEM_FULL);
                const uint32_t box_s = ptx::smem_u32(sm.box[ew][j]) + row_ofs;
                if (RES) fused_wait(&sm.rbar[ew][j], ucount & 1, &sm.abort_flag, p.err, DEV_TIMEOUT_FULL);
                __syncwarp();                           // lanes leave the waits at different times; the TMEM accesses are warp-wide
                ptx::tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(slot * BN + cq * CW);
                const int col0 = j * BN + cq * CW;                     // column inside this block's share of this warp's first element
                uint32_t v[2][16];
                ptx::tmem_ld16(taddr, v[0]);
#pragma unroll
                for (int c = 0; c < NCH; c++) {
                    int4 cs[4];
                    if (MODE == FUSED_QKV && do_rope) {
                        // the lanes of a warp are consecutive tokens of one member: every load below is one contiguous run
                        const int pair0 = fast_mod(cofs + col0 + 16 * c, p.fd_head) >> 1;
#pragma unroll
                        for (int q4 = 0; q4 < 4; q4++) {
                            const int2 c0 = __ldg(rope + (int64_t)(pair0 + 2 * q4) * p.seq_len), c1 = __ldg(rope + (int64_t)(pair0 + 2 * q4 + 1) * p.seq_len);
                            cs[q4] = make_int4(c0.x, c0.y, c1.x, c1.y);
                        }
                    }
                    int4 rs4 = make_int4(0, 0, 0, 0);
                    if (RES) rs4 = ptx::lds_v4(box_s + (((uint32_t)c ^ swz) << 4));
                    uint32_t *vc = v[c & 1];
                    ptx::tmem_ld_wait16(vc);
                    if (c + 1 < NCH) {
                        ptx::tmem_st_wait();            // the store of chunk c-1 read the registers the next load overwrites
                        ptx::tmem_ld16(taddr + 16 * (c + 1), v[(c + 1) & 1]);
                    }
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++) {
                        const int col = col0 + 16 * c + 4 * q4;
                        const int4 an = ptx::lds_v4(a32_s + 4 * col);
                        int x0, x1, x2, x3;
                        if (RES && GEMM_FMA_ADDS) {
                            // ((acc + r1 + (b << s)) >> s) + residual with r1 = (xb*a) >> t: the bias joins the rank-1 product
                            // ((b << (s+t)) is a multiple of 2^t), the other adds are multiply-adds by a run-time 1 — the
                            // integer pipe runs at half the rate of the multiply-add pipe and is the busy one here
                            const int4 b4 = ptx::lds_v4(bcs_s + 4 * col);
                            const int32_t rs = q4 == 0 ? rs4.x : (q4 == 1 ? rs4.y : (q4 == 2 ? rs4.z : rs4.w));
                            x0 = ((((xbs * an.x + b4.x) >> p.rank1_shift) * p.one + (int)vc[4 * q4]) >> p.out_shift) * p.one + ptx::sx_byte0(rs);
                            x1 = ((((xbs * an.y + b4.y) >> p.rank1_shift) * p.one + (int)vc[4 * q4 + 1]) >> p.out_shift) * p.one + ptx::sx_byte1(rs);
                            x2 = ((((xbs * an.z + b4.z) >> p.rank1_shift) * p.one + (int)vc[4 * q4 + 2]) >> p.out_shift) * p.one + ptx::sx_byte2(rs);
                            x3 = ((((xbs * an.w + b4.w) >> p.rank1_shift) * p.one + (int)vc[4 * q4 + 3]) >> p.out_shift) * p.one + (rs >> 24);
                        } else if (GEMM_FMA_ADDS) {
                            x0 = ((xbs * an.x) >> p.rank1_shift) * p.one + (int)vc[4 * q4];
                            x1 = ((xbs * an.y) >> p.rank1_shift) * p.one + (int)vc[4 * q4 + 1];
                            x2 = ((xbs * an.z) >> p.rank1_shift) * p.one + (int)vc[4 * q4 + 2];
                            x3 = ((xbs * an.w) >> p.rank1_shift) * p.one + (int)vc[4 * q4 + 3];
                        } else {
                            x0 = (int)vc[4 * q4] + ((xbs * an.x) >> p.rank1_shift);
                            x1 = (int)vc[4 * q4 + 1] + ((xbs * an.y) >> p.rank1_shift);
                            x2 = (int)vc[4 * q4 + 2] + ((xbs * an.z) >> p.rank1_shift);
                            x3 = (int)vc[4 * q4 + 3] + ((xbs * an.w) >> p.rank1_shift);
                        }
                        if (RES && !GEMM_FMA_ADDS) {
                            const int4 b4 = ptx::lds_v4(bcs_s + 4 * col);
                            const int32_t rs = q4 == 0 ? rs4.x : (q4 == 1 ? rs4.y : (q4 == 2 ? rs4.z : rs4.w));
                            x0 = ptx::sx_byte0(rs) + ((x0 + b4.x) >> p.out_shift);
                            x1 = ptx::sx_byte1(rs) + ((x1 + b4.y) >> p.out_shift);
                            x2 = ptx::sx_byte2(rs) + ((x2 + b4.z) >> p.out_shift);
                            x3 = (rs >> 24) + ((x3 + b4.w) >> p.out_shift);
                        } else if (do_rope) {
                            // integer RoPE on adjacent (even, odd) columns (apply_rope_integer, mgpu.cu:624-644)
                            const int e0 = x0, o0 = x1, e1 = x2, o1 = x3;
                            x0 = ptx::shr64_lo(ptx::mad_wide(-o0, cs[q4].y, ptx::mad_wide(e0, cs[q4].x, half_ulp)), p.rope_bit);
                            x1 = ptx::shr64_lo(ptx::mad_wide(o0, cs[q4].x, ptx::mad_wide(e0, cs[q4].y, half_ulp)), p.rope_bit);
                            x2 = ptx::shr64_lo(ptx::mad_wide(-o1, cs[q4].w, ptx::mad_wide(e1, cs[q4].z, half_ulp)), p.rope_bit);
                            x3 = ptx::shr64_lo(ptx::mad_wide(o1, cs[q4].z, ptx::mad_wide(e1, cs[q4].w, half_ulp)), p.rope_bit);
                        }
                        rmx = __vimax3_s32(__vimax3_s32(rmx, x0, x1), x2, x3);      // abs-max as max(max, -min)
                        rmn = __vimin3_s32(__vimin3_s32(rmn, x0, x1), x2, x3);
                        vc[4 * q4] = (uint32_t)x0; vc[4 * q4 + 1] = (uint32_t)x1; vc[4 * q4 + 2] = (uint32_t)x2; vc[4 * q4 + 3] = (uint32_t)x3;
                    }
                    ptx::tmem_st16(taddr + 16 * c, vc);
                }
                ptx::tmem_st_wait();
            }
            sm.rowpart[cq][row_in_tile] = max(rmx, -rmn);
            if (LN && e < tab_items) ln_store(lnw);
            ptx::named_bar_sync(2 + quarter, 128);            // the four column quarters of this lane quarter
            int row_max = max(max(sm.rowpart[0][row_in_tile], sm.rowpart[1][row_in_tile]),
                              max(sm.rowpart[2][row_in_tile], sm.rowpart[3][row_in_tile]));
            if (p.cl > 1) {
                // the other half of the row lives in the peer block: its first column quarter writes the maximum of its
                // columns into this block's peer_max and arrives (release, cluster scope) on this block's barrier, and
                // vice versa.  Buffers and barriers alternate with the unit parity: the peer cannot get past this
                // exchange of unit u+1 before this block has arrived for it, that is after it has read unit u's value.
                if (cq == 0) {
                    ptx::st_cluster_u32(peer_max_s + (uint32_t)(tb * GEMM_BM + row_in_tile) * 4u, (uint32_t)row_max);
                    ptx::mbar_arrive_cluster(peer_bar_s + (uint32_t)tb * 8u);
                }
                if (!sm.abort_flag && !ptx::mbar_wait_cluster(&sm.xbar[tb], (uint32_t)(ucount >> 1) & 1u, 1000000000ull)) {
                    sm.abort_flag = 1;
                    if (p.err) atomicCAS(p.err, 0, DEV_TIMEOUT_PEER);
                }
                row_max = max(row_max, sm.peer_max[tb][row_in_tile]);
            }
            const float scale = aln_scale(row_max);

            // ---------------- pass 2: requantise, pack, store ----------------
            int tot = 0;                                      // FUSED_RES_LN: Σ|x| over this warp's columns of the row
            for (int j = 0; j < NT; j++) {
                const uint32_t st = stc + (uint32_t)j;
                const int slot = st % NS;
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(slot * BN + cq * CW);
                const uint32_t box_s = ptx::smem_u32(sm.box[ew][j]) + row_ofs;
                if (MODE == FUSED_QKV) {
                    // the store that last read this box was issued NT stores ago
                    if (lane == 0) { if (BN == 256 && NT == 2) ptx::tma_store_wait_read<1>(); else ptx::tma_store_wait_read<0>(); }
                    __syncwarp();
                }
                uint32_t v[2][16];
                ptx::tmem_ld16(taddr, v[0]);
#pragma unroll
                for (int c = 0; c < NCH; c++) {
                    uint32_t *vc = v[c & 1];
                    ptx::tmem_ld_wait16(vc);
                    if (c + 1 < NCH) ptx::tmem_ld16(taddr + 16 * (c + 1), v[(c + 1) & 1]);
                    uint32_t w[4];
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++)
                        w[q4] = ptx::pack_sat_s8(aln_quant_f((int)vc[4 * q4], scale), aln_quant_f((int)vc[4 * q4 + 1], scale),
                                                 aln_quant_f((int)vc[4 * q4 + 2], scale), aln_quant_f((int)vc[4 * q4 + 3], scale));
                    if (LN) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; q4++) tot = __dp4a((int)__vabsss4(w[q4]), 0x01010101, tot);
                    }
                    ptx::sts_v4(box_s + (((uint32_t)c ^ swz) << 4), make_int4((int)w[0], (int)w[1], (int)w[2], (int)w[3]));
                }
                // this warp has read its part of the slot: hand it back to the MMA warp
                ptx::tc_fence_before();
                ptx::fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&sm.tmem_empty[slot]);
                    ptx::tma_store_2d(&tmap_o, sm.box[ew][j], cofs + j * BN + cq * CW, (int)(part * p.part_rows) + m0 + quarter * 32);
                    ptx::tma_store_commit();
                }
            }
            stc += (uint32_t)NT;
            if (LN) {
                // ---------------- the mean-abs norm of the finished row (apply_standard_norm, mgpu.cu:646-678) ----------------
                // y = clip((x * w') / mean|x| + b'), and the dots of y with the B-noise of the projections that read it.  The
                // row's bytes are still in this lane's boxes; TMEM has been handed back, so the next unit's MMAs run meanwhile.
                sm.rowsum[cq][row_in_tile] = (uint16_t)tot;
                ptx::named_bar_sync(1, GEMM_EPI_THREADS);        // sums and norm tables of this unit are published
                int total = (int)sm.rowsum[0][row_in_tile] + (int)sm.rowsum[1][row_in_tile] + (int)sm.rowsum[2][row_in_tile] + (int)sm.rowsum[3][row_in_tile];
                if (p.cl > 1) {      // the peer block's half of the row: same exchange as for the maxima
                    if (cq == 0) {
                        ptx::st_cluster_u32(peer_sum_s + (uint32_t)(tb * GEMM_BM + row_in_tile) * 4u, (uint32_t)total);
                        ptx::mbar_arrive_cluster(peer_bar2_s + (uint32_t)tb * 8u);
                    }
                    if (!sm.abort_flag && !ptx::mbar_wait_cluster(&sm.xbar2[tb], (uint32_t)(ucount >> 1) & 1u, 1000000000ull)) {
                        sm.abort_flag = 1;
                        if (p.err) atomicCAS(p.err, 0, DEV_TIMEOUT_PEER);
                    }
                    total += sm.peer_sum[tb][row_in_tile];
                }
                int mn = fast_div(total, p.fd_h);
                if (!mn) mn = 1;
                const float rinv = c_rinv_up.v[mn & 127];        // mn <= 127: a mean of absolute values of int8
                const uint32_t lwb_s = ptx::smem_u32(&sm.ln_wb[0]), ld4_s = ptx::smem_u32(&sm.ln_d4[0]);
                int8_t *hrow = p.h_out + (int64_t)r * p.H + cofs;
                int dot0 = 0, dot1 = 0, dot2 = 0;
                for (int j = 0; j < NT; j++) {
                    const uint32_t box_s = ptx::smem_u32(sm.box[ew][j]) + row_ofs;
#pragma unroll
                    for (int c = 0; c < NCH; c++) {
                        const int4 xw = ptx::lds_v4(box_s + (((uint32_t)c ^ swz) << 4));
                        const int col = j * BN + cq * CW + 16 * c;
                        uint32_t yw[4];
#pragma unroll
                        for (int q4 = 0; q4 < 4; q4++) {
                            const int xv = q4 == 0 ? xw.x : (q4 == 1 ? xw.y : (q4 == 2 ? xw.z : xw.w));
                            const uint32_t grp = (uint32_t)(col >> 2) + (uint32_t)q4;          // group of 4 columns
                            const int4 wb = ptx::lds_v4(lwb_s + 16u * grp), d4 = ptx::lds_v4(ld4_s + 16u * grp);
                            // x_i * w_i without widening either: a two-term dot product of the int16 pair with the word whose
                            // other byte is masked to zero, started from the bit pattern of 1.5 * 2^23 (i2f_small's addend);
                            // "+ b_i" the same way against a constant 1
                            const float f0 = __int_as_float(__dp2a_lo(wb.x, xv & 0x000000FF, kMagicBits)) - kMagic;
                            const float f1 = __int_as_float(__dp2a_lo(wb.x, xv & 0x0000FF00, kMagicBits)) - kMagic;
                            const float f2 = __int_as_float(__dp2a_hi(wb.y, xv & 0x00FF0000, kMagicBits)) - kMagic;
                            const float f3 = __int_as_float(__dp2a_hi(wb.y, xv & (int)0xFF000000, kMagicBits)) - kMagic;
                            const int y0 = __dp2a_lo(wb.z, 0x00000001, __float2int_rz(f0 * rinv));
                            const int y1 = __dp2a_lo(wb.z, 0x00000100, __float2int_rz(f1 * rinv));
                            const int y2 = __dp2a_lo(wb.w, 0x00000001, __float2int_rz(f2 * rinv));
                            const int y3 = __dp2a_lo(wb.w, 0x00000100, __float2int_rz(f3 * rinv));
                            yw[q4] = pack_clip8(y0, y1, y2, y3);
                            dot0 = __dp4a((int)yw[q4], d4.x, dot0);
                            if (p.ndots > 1) { dot1 = __dp4a((int)yw[q4], d4.y, dot1); dot2 = __dp4a((int)yw[q4], d4.z, dot2); }
                        }
                        *reinterpret_cast<int4 *>(hrow + col) = make_int4((int)yw[0], (int)yw[1], (int)yw[2], (int)yw[3]);
                    }
                }
                // every warp (and both blocks of a pair) adds its columns' share: integer sums, any order
                int32_t *xo = p.xb_out + (int64_t)r * p.xb_out_stride;
                atomicAdd(xo, dot0);
                if (p.ndots > 1) { atomicAdd(xo + 1, dot1); atomicAdd(xo + 2, dot2); }
                __syncwarp();          // all lanes have read their boxes before lane 0 lets the next residual bytes in
            }
            if (RES && lane == 0 && nunit < num_units) {
                // the boxes are free once their stores have read them: fetch the next unit's residual bytes
                ptx::tma_store_wait_read<0>();
                resid_request(nunit);
            }
            if (have_nxt) tab_store(tb ^ 1, nxt);      // published by the next unit's barrier
        }
        if (lane == 0) ptx::tma_store_wait_all<0>();     // boxes still being copied out must land before the block retires
        if (sm.abort_flag) {   // draining after a timeout: residual boxes may still be in flight towards this block
            const uint64_t t0 = ptx::globaltimer();
            while (ptx::globaltimer() - t0 < 200000ull) { __nanosleep(1000); }
        }
        __syncwarp();
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, 512);
    }
    // neither block of a pair retires while the other may still write its maxima into it
    if (p.cl > 1) ptx::cluster_sync_all();
}

template <int BN>
constexpr size_t fused_smem_bytes() { return sizeof(FusedSmem<BN>) + 1024; }
static_assert(fused_smem_bytes<256>() <= 227 * 1024, "fused GEMM shared memory exceeds the 227 KB a block may use");
static_assert(fused_smem_bytes<128>() <= 227 * 1024, "fused GEMM shared memory exceeds the 227 KB a block may use");

}  // namespace egg
