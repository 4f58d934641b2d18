// Instantiations and host launcher of the tcgen05 int8 GEMM.
#include "egg_kernels.cuh"
#include "egg_gemm_fused.cuh"

#include <cudaTypedefs.h>

namespace egg {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

template <int BN, int EPI, int RPL = 0>
static int set_attr() {
    EGG_CUDA(cudaFuncSetAttribute(gemm_i8_kernel<BN, EPI, RPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm_smem_bytes<BN>()));
    return EGG_OK;
}

template <int EPI, int RPL = 0>
static int set_attr_both() {
    int rc = set_attr<128, EPI, RPL>();
    if (rc) return rc;
    return set_attr<256, EPI, RPL>();
}

int gemm_init() {
    if (!g_encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        EGG_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return EGG_E_CUDA; }
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    int rc;
    if ((rc = set_attr_both<EPI_CLIP8>())) return rc;
    if ((rc = set_attr_both<EPI_GELU>())) return rc;
    if ((rc = set_attr_both<EPI_PRE32>())) return rc;
    if ((rc = set_attr_both<EPI_QKV>())) return rc;
    if ((rc = set_attr_both<EPI_GELU, 1>())) return rc;
    if ((rc = set_attr_both<EPI_PRE32, 1>())) return rc;
    if ((rc = set_attr_both<EPI_QKV, 1>())) return rc;
    if ((rc = set_attr<256, EPI_HEAD>())) return rc;
    if ((rc = set_attr<256, EPI_HEAD, 1>())) return rc;
    if ((rc = set_attr<256, EPI_LOGITS>())) return rc;
    if ((rc = set_attr<256, EPI_LOGITS, 1>())) return rc;
    if ((rc = set_attr_both<EPI_VOTE>())) return rc;
    if ((rc = set_attr<256, EPI_NULL>())) return rc;
    EGG_CUDA(cudaFuncSetAttribute(gemm_fused_kernel<256, FUSED_QKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fused_smem_bytes<256>()));
    EGG_CUDA(cudaFuncSetAttribute(gemm_fused_kernel<256, FUSED_RES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fused_smem_bytes<256>()));
    EGG_CUDA(cudaFuncSetAttribute(gemm_fused_kernel<128, FUSED_QKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fused_smem_bytes<128>()));
    EGG_CUDA(cudaFuncSetAttribute(gemm_fused_kernel<128, FUSED_RES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fused_smem_bytes<128>()));
    EGG_CUDA(cudaFuncSetAttribute(gemm_fused_kernel<256, FUSED_RES_LN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fused_smem_bytes<256>()));
    EGG_CUDA(cudaFuncSetAttribute(gemm_fused_kernel<128, FUSED_RES_LN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fused_smem_bytes<128>()));
    return EGG_OK;
}

// [rows][k] int8 row-major; box = 128 (k) x box_rows, 128-byte swizzle, out-of-range reads give zeros.
static int make_tmap(CUtensorMap *m, const void *ptr, uint64_t rows, uint64_t k, uint32_t box_rows) {
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (k & 15)) { set_error("GEMM operand is not 16-byte aligned (ptr %p, k %llu)", ptr, (unsigned long long)k); return EGG_E_INVALID; }
    cuuint64_t gdim[2] = {k, rows};
    cuuint64_t gstride[1] = {k};
    cuuint32_t box[2] = {(cuuint32_t)GEMM_BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d) rows=%llu k=%llu box_rows=%u", (int)r, (unsigned long long)rows, (unsigned long long)k, box_rows); return EGG_E_CUDA; }
    return EGG_OK;
}

// [rows][cols] int32 row-major output written by TMA stores of 16-column x 32-row boxes (64-byte swizzle in shared memory)
static int make_tmap_out(CUtensorMap *m, const void *ptr, uint64_t rows, uint64_t cols) {
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (cols & 3)) { set_error("GEMM output is not 16-byte aligned (ptr %p, cols %llu)", ptr, (unsigned long long)cols); return EGG_E_INVALID; }
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {cols * 4};
    cuuint32_t box[2] = {16, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<void *>(ptr), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (output) failed (%d) rows=%llu cols=%llu", (int)r, (unsigned long long)rows, (unsigned long long)cols); return EGG_E_CUDA; }
    return EGG_OK;
}

// [rows][cols] int8 row-major output written by TMA stores of 64-column x 32-row boxes (64-byte swizzle)
static int make_tmap_out8(CUtensorMap *m, const void *ptr, uint64_t rows, uint64_t cols) {
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (cols & 15)) { set_error("GEMM output is not 16-byte aligned (ptr %p, cols %llu)", ptr, (unsigned long long)cols); return EGG_E_INVALID; }
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {cols};
    cuuint32_t box[2] = {64, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (int8 output) failed (%d) rows=%llu cols=%llu", (int)r, (unsigned long long)rows, (unsigned long long)cols); return EGG_E_CUDA; }
    return EGG_OK;
}

// [rows][cols] int8 row-major moved as box_cols-column x 32-row boxes: 64-byte rows swizzled (64-byte pattern), 32-byte
// rows stored densely
static int make_tmap_box8(CUtensorMap *m, const void *ptr, uint64_t rows, uint64_t cols, uint32_t box_cols) {
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (cols & 15) || (box_cols != 64 && box_cols != 32)) {
        set_error("int8 box map unsupported (ptr %p, cols %llu, box %u)", ptr, (unsigned long long)cols, box_cols);
        return EGG_E_INVALID;
    }
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {cols};
    cuuint32_t box[2] = {box_cols, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (int8 boxes) failed (%d) rows=%llu cols=%llu", (int)r, (unsigned long long)rows, (unsigned long long)cols); return EGG_E_CUDA; }
    return EGG_OK;
}

// Blocks that share a unit of the row-owning GEMM: one up to 512 columns, a cluster of two above (0: unsupported width).
int fused_cluster_size(int hidden) {
    if (hidden <= 0 || hidden % 128) return 0;
    if (hidden <= FUSED_MAX_H) return 1;
    if (hidden <= 2 * FUSED_MAX_H && hidden % 256 == 0) return 2;
    return 0;
}

template <int BN, int MODE>
static int launch_fused_one(cudaStream_t st, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to, const CUtensorMap &tr,
                            const FusedParams &p, int units, int num_sms) {
    auto kern = gemm_fused_kernel<BN, MODE>;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = fused_smem_bytes<BN>();
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    int groups = num_sms / p.cl;                     // resident blocks (pairs of blocks)
    if (p.cl > 1) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)p.cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        // the pairs that can be resident at once (a GPC with an odd number of free SMs leaves one out): asked once
        static int max_pairs_dev[EGG_MAX_DEVICES] = {};
        int &max_pairs = max_pairs_dev[current_device_slot()];
        if (max_pairs == 0) {
            cfg.gridDim = dim3((unsigned)(num_sms / p.cl * p.cl));
            int n = 0;
            EGG_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
            if (n < 1) { set_error("no pair of blocks of the row-owning GEMM fits on the device"); return EGG_E_CUDA; }
            max_pairs = n;
        }
        if (groups > max_pairs) groups = max_pairs;
    }
    if (groups > units) groups = units;
    cfg.gridDim = dim3((unsigned)(groups * p.cl));
    EGG_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, to, tr, p));
    return EGG_OK;
}

int launch_gemm_fused(cudaStream_t st, int mode, const int8_t *A, const int8_t *B, int8_t *out, const int8_t *resid,
                      const FusedParams &p_in, int num_sms) {
    FusedParams p = p_in;
    if (!g_encode) { set_error("gemm_init() was not called"); return EGG_E_STATE; }
    p.cl = fused_cluster_size(p.H);
    if (p.M <= 0 || p.M % GEMM_BM || p.seq_len % GEMM_BM || p.cl == 0 || p.K % 16 || p.parts < 1 ||
        (mode != FUSED_QKV && (p.parts != 1 || !resid)) || (mode != FUSED_QKV && mode != FUSED_RES && mode != FUSED_RES_LN) ||
        (mode == FUSED_RES_LN && (!p.h_out || !p.xb_out || (p.ndots != 1 && p.ndots != 3)))) {
        set_error("unsupported row-owning GEMM shape M=%d H=%d K=%d parts=%d seq_len=%d", p.M, p.H, p.K, p.parts, p.seq_len);
        return EGG_E_INVALID;
    }
    if (mode != FUSED_QKV && p.out_shift + p.rank1_shift > 20) {     // (bias + noise) << (both shifts) joins a product below 2^30
        set_error("shifts %d + %d too large for the pre-shifted bias table", p.out_shift, p.rank1_shift);
        return EGG_E_INVALID;
    }
    const int hl = p.H / p.cl;                       // columns per block
    const int bn = (hl % 256 == 0) ? 256 : 128;      // (128-column sub-tiles at H = 512 were measured: +30 % on MLP-down)
    p.fd_head = make_fastdiv(p.head_dim > 0 ? p.head_dim : 64);
    p.fd_h = make_fastdiv(p.H);
    p.one = 1;
    CUtensorMap ta, tb, to, tr;
    int rc;
    if ((rc = make_tmap(&ta, A, (uint64_t)p.M, (uint64_t)p.K, GEMM_BM))) return rc;
    if ((rc = make_tmap(&tb, B, (uint64_t)p.parts * p.H, (uint64_t)p.K, (uint32_t)bn))) return rc;
    const uint64_t out_rows = p.parts > 1 ? (uint64_t)p.parts * (uint64_t)p.part_rows : (uint64_t)p.M;
    if ((rc = make_tmap_box8(&to, out, out_rows, (uint64_t)p.H, (uint32_t)bn / 4))) return rc;
    tr = to;
    if (mode != FUSED_QKV && (rc = make_tmap_box8(&tr, resid, (uint64_t)p.M, (uint64_t)p.H, (uint32_t)bn / 4))) return rc;
    const int units = (p.M / GEMM_BM) * p.parts;
    if (bn == 256) {
        if (mode == FUSED_QKV) return launch_fused_one<256, FUSED_QKV>(st, ta, tb, to, tr, p, units, num_sms);
        if (mode == FUSED_RES_LN) return launch_fused_one<256, FUSED_RES_LN>(st, ta, tb, to, tr, p, units, num_sms);
        return launch_fused_one<256, FUSED_RES>(st, ta, tb, to, tr, p, units, num_sms);
    }
    if (mode == FUSED_QKV) return launch_fused_one<128, FUSED_QKV>(st, ta, tb, to, tr, p, units, num_sms);
    if (mode == FUSED_RES_LN) return launch_fused_one<128, FUSED_RES_LN>(st, ta, tb, to, tr, p, units, num_sms);
    return launch_fused_one<128, FUSED_RES>(st, ta, tb, to, tr, p, units, num_sms);
}

template <int BN, int EPI, int RPL = 0>
static int launch_one(cudaStream_t st, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to, const GemmParams &p, int num_sms) {
    int tiles = ((p.M + GEMM_BM - 1) / GEMM_BM) * (p.N / BN) * ((EPI == EPI_VOTE && p.k_splits > 1) ? p.k_splits : 1);
    int grid = tiles < num_sms ? tiles : num_sms;
    CUtensorMap tr = ta;       // residual bytes as 64-column x 32-row boxes (row-per-lane residual projections with BN = 256 only)
    if (EPI == EPI_PRE32 && RPL && BN == 256) {
        int rc = make_tmap_out8(&tr, p.resid, (uint64_t)p.M, (uint64_t)p.N);
        if (rc) return rc;
    }
    gemm_i8_kernel<BN, EPI, RPL><<<grid, GEMM_THREADS, gemm_smem_bytes<BN>(), st>>>(ta, tb, to, tr, p);
    EGG_CUDA(cudaGetLastError());
    return EGG_OK;
}

template <int EPI, int RPL = 0>
static int launch_bn(cudaStream_t st, int bn, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to, const GemmParams &p, int num_sms) {
    if (bn == 256) return launch_one<256, EPI, RPL>(st, ta, tb, to, p, num_sms);
    return launch_one<128, EPI, RPL>(st, ta, tb, to, p, num_sms);
}

// evaluation epilogues whose rows come in whole 32-row groups per member take the row-per-lane form
template <int EPI>
static int launch_eval(cudaStream_t st, int bn, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to, const GemmParams &p, int num_sms) {
    if (p.seq_len % 32 == 0 && p.rpl >= 0) return launch_bn<EPI, 1>(st, bn, ta, tb, to, p, num_sms);
    return launch_bn<EPI, 0>(st, bn, ta, tb, to, p, num_sms);
}

int launch_gemm(cudaStream_t st, int epi, const int8_t *A, const int8_t *B, const GemmParams &p_in, int num_sms) {
    GemmParams p = p_in;
    if (!g_encode) { set_error("gemm_init() was not called"); return EGG_E_STATE; }
    if (p.M <= 0 || p.N % 128 || p.K % 16) { set_error("unsupported GEMM shape M=%d N=%d K=%d", p.M, p.N, p.K); return EGG_E_INVALID; }
    int bn = (p.N % 256 == 0) ? 256 : 128;
    if (epi == EPI_QKV && (p.third % bn)) bn = 128;
    if (epi == EPI_QKV && (p.third % 128)) { set_error("hidden_dim must be a multiple of 128"); return EGG_E_INVALID; }
    if (epi == EPI_HEAD && p.N != 256) { set_error("the one-tile head GEMM needs vocab_size == 256"); return EGG_E_INVALID; }
    if (epi == EPI_LOGITS && p.N % 256) { set_error("the logits GEMM needs a vocabulary that is a multiple of 256"); return EGG_E_INVALID; }
    if (epi <= EPI_LOGITS) {
        int max_slots = ((GEMM_BM - 1) / p.seq_len) / 2 + 2;
        const bool rpl = p.seq_len % 32 == 0 && p.rpl >= 0 && epi != EPI_CLIP8;
        if (max_slots > (rpl ? GEMM_RPL_SLOTS : GEMM_MAX_SLOTS)) { set_error("seq_len %d too small for the epilogue tables", p.seq_len); return EGG_E_INVALID; }
    }
    if (epi == EPI_VOTE && p.k_splits > 1) {
        // every split must own at least one k-block: the kernel cuts ceil(num_kb / k_splits) blocks per split
        const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;
        const int kb_per = (num_kb + p.k_splits - 1) / p.k_splits;
        if ((num_kb + kb_per - 1) / kb_per != p.k_splits) { set_error("k_splits %d leaves an empty split of %d k-blocks", p.k_splits, num_kb); return EGG_E_INVALID; }
    }
    p.fd_seq = make_fastdiv(p.seq_len);
    p.fd_tiles_n = make_fastdiv(p.N / bn);
    p.fd_third = make_fastdiv(p.third);
    p.fd_head = make_fastdiv(p.head_dim);
    p.lut_stride = 32 * 4;
    p.one = 1;
    if (epi == EPI_GELU && p.out_shift + p.rank1_shift > 20) {       // (bias + noise) << (both shifts) joins a product below 2^30
        set_error("shifts %d + %d too large for the pre-shifted bias table", p.out_shift, p.rank1_shift);
        return EGG_E_INVALID;
    }
    p.pow_t = 0;
    if (epi == EPI_GELU) {
        // both shifts as one when |acc| * 2^t + |xb * a| + |(bias + noise) << (s + t)| < 2^31 for every input:
        // |acc| <= K * 127^2, |xb| <= K * 127 * 31, |a| <= 31 (the largest noise mask), |bias + noise| <= 254
        const int64_t bound = (int64_t)p.K * 16129 * (1ll << p.rank1_shift) + (int64_t)p.K * 127 * 961 + (254ll << (p.out_shift + p.rank1_shift));
        if (bound < (1ll << 31)) p.pow_t = 1 << p.rank1_shift;
    }
    CUtensorMap ta, tb;
    int rc;
    if ((rc = make_tmap(&ta, A, (uint64_t)p.M, (uint64_t)p.K, GEMM_BM))) return rc;
    if ((rc = make_tmap(&tb, B, (uint64_t)p.N, (uint64_t)p.K, (uint32_t)bn))) return rc;
    CUtensorMap to = ta;       // only the row-per-lane int32 epilogues store through a tensor map
    if ((epi == EPI_PRE32 || epi == EPI_QKV || epi == EPI_LOGITS) && p.seq_len % 32 == 0 && p.rpl >= 0) {
        if ((rc = make_tmap_out(&to, p.out32, (uint64_t)p.M, (uint64_t)p.N))) return rc;
    }
    if (epi == EPI_GELU && bn == 256 && p.seq_len % 32 == 0 && p.rpl >= 0) {
        if ((rc = make_tmap_out8(&to, p.out8, (uint64_t)p.M, (uint64_t)p.N))) return rc;
    }
    switch (epi) {
        case EPI_CLIP8: return launch_bn<EPI_CLIP8>(st, bn, ta, tb, to, p, num_sms);
        case EPI_GELU: return launch_eval<EPI_GELU>(st, bn, ta, tb, to, p, num_sms);
        case EPI_PRE32: return launch_eval<EPI_PRE32>(st, bn, ta, tb, to, p, num_sms);
        case EPI_QKV: return launch_eval<EPI_QKV>(st, bn, ta, tb, to, p, num_sms);
        case EPI_HEAD:
            if (p.seq_len % 32 == 0 && p.rpl >= 0) return launch_one<256, EPI_HEAD, 1>(st, ta, tb, to, p, num_sms);
            return launch_one<256, EPI_HEAD>(st, ta, tb, to, p, num_sms);
        case EPI_LOGITS:
            if (p.seq_len % 32 == 0 && p.rpl >= 0) return launch_one<256, EPI_LOGITS, 1>(st, ta, tb, to, p, num_sms);
            return launch_one<256, EPI_LOGITS>(st, ta, tb, to, p, num_sms);
        case EPI_VOTE: return launch_bn<EPI_VOTE>(st, bn, ta, tb, to, p, num_sms);
        case EPI_NULL: return launch_one<256, EPI_NULL>(st, ta, tb, to, p, num_sms);
    }
    set_error("unknown epilogue %d", epi);
    return EGG_E_INVALID;
}

}  // namespace egg
