// Shared device/host definitions of the B200 EGGROLL library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/egg_b200.h"

namespace egg {

// ---------------------------------------------------------------- RNG
// Counter hash of the reference (full_cuda_train_transformer_adam_mgpu.cu:525-538;
// d-eggs/include/utils/egg_math.h:17-34).
__host__ __device__ __forceinline__ uint32_t hash_rng(uint32_t s, uint32_t idx) {
    uint32_t x = s + idx * 0x9e3779b9u;
    x ^= x >> 16; x *= 0x85ebca6bu;
    x ^= x >> 13; x *= 0xc2b2ae35u;
    x ^= x >> 16;
    return x;
}

__host__ __device__ __forceinline__ int noise_field(uint32_t r, int sign_bit, int shift, int mask) {
    int mag = (int)((r >> shift) & (uint32_t)mask);
    return (r & (1u << sign_bit)) ? mag : -mag;
}

// gaussian: sum of three fields (DEVICE_GAUSSIAN), else one field.
__host__ __device__ __forceinline__ int noise_from_hash(uint32_t s, uint32_t idx, int mask, int gaussian) {
    uint32_t r = hash_rng(s, idx);
    if (gaussian)
        return (int)(int8_t)(noise_field(r, 0, 1, mask) + noise_field(r, 5, 6, mask) + noise_field(r, 10, 11, mask));
    return noise_field(r, 0, 1, mask);
}

__host__ __device__ __forceinline__ int clip8(int a) { return a > 127 ? 127 : (a < -127 ? -127 : a); }

// ---------------------------------------------------------------- model layout
// Field order of TransformerModel (mgpu.cu:284-318); element offsets.
struct ModelLayout {
    int64_t embedding, emb_bias, ntt_emb /* ntt_emb1..3 in a row (mgpu.cu:288-293); empty when ntt_mode == 0 */, ln_init, ln_init_bias,
        w_emb_mlp_up, mlp_emb_bias_up, w_emb_mlp_down,
        mlp_emb_bias_down, ln_1, ln_1_bias, w_q, w_k, w_v, w_o, ln_2, ln_2_bias, w_up, mlp_bias_up, w_down,
        mlp_bias_down, ln_f, ln_f_bias, total;
};

inline ModelLayout model_layout(const egg_config &c) {
    ModelLayout L;
    int64_t H = c.hidden_dim, V = c.vocab_size, NL = c.n_layers, o = 0;
    L.embedding = o;         o += V * H;
    L.emb_bias = o;          o += H;
    L.ntt_emb = o;           o += c.ntt_mode ? 3 * V * H : 0;
    L.ln_init = o;           o += H;
    L.ln_init_bias = o;      o += H;
    L.w_emb_mlp_up = o;      o += H * 4 * H;
    L.mlp_emb_bias_up = o;   o += 4 * H;
    L.w_emb_mlp_down = o;    o += 4 * H * H;
    L.mlp_emb_bias_down = o; o += H;
    L.ln_1 = o;              o += NL * H;
    L.ln_1_bias = o;         o += NL * H;
    L.w_q = o;               o += NL * H * H;
    L.w_k = o;               o += NL * H * H;
    L.w_v = o;               o += NL * H * H;
    L.w_o = o;               o += NL * H * H;
    L.ln_2 = o;              o += NL * H;
    L.ln_2_bias = o;         o += NL * H;
    L.w_up = o;              o += NL * H * 4 * H;
    L.mlp_bias_up = o;       o += NL * 4 * H;
    L.w_down = o;            o += NL * 4 * H * H;
    L.mlp_bias_down = o;     o += NL * H;
    L.ln_f = o;              o += H;
    L.ln_f_bias = o;         o += H;
    L.total = o;
    return L;
}

// AdaptiveScales (d-eggs/include/model/definitions.h:92-142): one int8 overlay per input index ("_row")
// and per output index ("_col") of every matrix and per element of every vector; byte offsets.
struct ScalesLayout {
    int64_t embedding_row, embedding_col, emb_bias, ln_init, ln_init_bias, w_emb_mlp_up_row, w_emb_mlp_up_col,
        mlp_emb_bias_up, w_emb_mlp_down_row, w_emb_mlp_down_col, mlp_emb_bias_down, ln_1, ln_1_bias, w_q_row, w_q_col,
        w_k_row, w_k_col, w_v_row, w_v_col, w_o_row, w_o_col, ln_2, ln_2_bias, w_up_row, w_up_col, mlp_bias_up,
        w_down_row, w_down_col, mlp_bias_down, ln_f, ln_f_bias, total;
};

inline ScalesLayout scales_layout(const egg_config &c) {
    ScalesLayout S;
    int64_t H = c.hidden_dim, V = c.vocab_size, NL = c.n_layers, o = 0;
    S.embedding_row = o;      o += V;
    S.embedding_col = o;      o += H;
    S.emb_bias = o;           o += H;
    S.ln_init = o;            o += H;
    S.ln_init_bias = o;       o += H;
    S.w_emb_mlp_up_row = o;   o += H;
    S.w_emb_mlp_up_col = o;   o += 4 * H;
    S.mlp_emb_bias_up = o;    o += 4 * H;
    S.w_emb_mlp_down_row = o; o += 4 * H;
    S.w_emb_mlp_down_col = o; o += H;
    S.mlp_emb_bias_down = o;  o += H;
    S.ln_1 = o;               o += NL * H;
    S.ln_1_bias = o;          o += NL * H;
    S.w_q_row = o;            o += NL * H;
    S.w_q_col = o;            o += NL * H;
    S.w_k_row = o;            o += NL * H;
    S.w_k_col = o;            o += NL * H;
    S.w_v_row = o;            o += NL * H;
    S.w_v_col = o;            o += NL * H;
    S.w_o_row = o;            o += NL * H;
    S.w_o_col = o;            o += NL * H;
    S.ln_2 = o;               o += NL * H;
    S.ln_2_bias = o;          o += NL * H;
    S.w_up_row = o;           o += NL * H;
    S.w_up_col = o;           o += NL * 4 * H;
    S.mlp_bias_up = o;        o += NL * 4 * H;
    S.w_down_row = o;         o += NL * 4 * H;
    S.w_down_col = o;         o += NL * H;
    S.mlp_bias_down = o;      o += NL * H;
    S.ln_f = o;               o += H;
    S.ln_f_bias = o;          o += H;
    S.total = o;
    return S;
}

// get_adaptive_factor, ADAPTIVE_NOISE_MODE 1 (d-eggs/include/model/layers.cuh:12-19), as the numerator of
// a fraction over 64: negative overlays switch the noise off, 0..63 scale it by ov/64, larger ones leave it.
__host__ __device__ __forceinline__ int overlay_num(int ov) { return ov < 0 ? 0 : (ov < 64 ? ov : 64); }
// (int)(v * (num / 64.0f)) for an integer v with |v * num| < 2^24: the float product is exact, the
// conversion truncates toward zero.
__host__ __device__ __forceinline__ int scale_trunc(int v, int num) {
    const int q = v * num;
    return (q + ((q >> 31) & 63)) >> 6;
}

// Division of 0 <= n < 2^31 by a run-time constant d >= 1 as one wide multiply and a shift:
// with l = ceil(log2 d) and mul = floor(2^(31+l) / d) + 1,  mul*d - 2^(31+l) lies in [1, d] <= 2^l, which makes
// floor(n * mul / 2^(31+l)) == floor(n / d) for every n below 2^31.
struct FastDiv {
    uint32_t mul, shift;
    int d;
};
inline FastDiv make_fastdiv(int d) {
    FastDiv f;
    if (d < 1) d = 1;
    int l = 0;
    while ((1ll << l) < d) l++;
    f.mul = (uint32_t)(((1ull << (31 + l)) / (uint64_t)d) + 1ull);
    f.shift = (uint32_t)(31 + l);
    f.d = d;
    return f;
}
__host__ __device__ __forceinline__ int fast_div(int n, const FastDiv &f) { return (int)(((uint64_t)(uint32_t)n * f.mul) >> f.shift); }
__host__ __device__ __forceinline__ int fast_mod(int n, const FastDiv &f) { return n - fast_div(n, f) * f.d; }

// One trainable parameter of the update sequence (mgpu.cu:1603-1643).
struct ParamDesc {
    int64_t model_off;   // element offset in TransformerModel
    int64_t opt_off;     // byte offset in AdamModel
    int rows_k;          // input dim (0 for vectors)
    int cols_n;          // output dim (length for vectors)
    int off_a, off_b, seed_base;
    float lr_scale;
    int muon;            // state is MuonParam{m,acc} and the step is Muon
    int64_t shadow_off;  // element offset of the K-major shadow copy (-1: none)
    int64_t ov_in, ov_out;   // AdaptiveScales offsets of the overlays over the input index (or the vector) and the output index
};

// ---------------------------------------------------------------- adaptive requantisation
// adaptive_layer_normalize / adaptive_qkv_normalize (egg_adaptive_normalize.h:10-103):
//   scale = 127.0f / (float)(max + 1e-9f);  out = clamp((int)roundf((float)v * scale), -127, 127)
__device__ __forceinline__ float aln_scale(int layer_max) { return 127.0f / (float)(layer_max + 1e-9f); }
__device__ __forceinline__ float aln_scale24(int layer_max) { return aln_scale(layer_max) * 16777216.0f; }    // exact: a power of two
// clamp((int)roundf((float)v * scale), -127, 127) for |v| <= max, in fixed point: |v| * (scale * 2^24) is the same
// float product scaled by a power of two (|x| <= 127 * (1 + 2^-23), so x * 2^24 < 2^31), its truncation to an integer
// keeps every bit that decides the rounding (for |x| >= 1 the product has at most 23 fraction bits; below 1 only
// "is it >= 0.5" matters, which truncation preserves), and round-half-away-from-zero becomes (xi + 2^23) >> 24.
// The result cannot leave [-127, 127], so the reference's clamp needs no instruction.
// The float product and its truncation are symmetric in the sign of v, so the sign is carried through: for a negative
// truncated product xi = -a, -((a + 2^23) >> 24) == (xi + 2^23 - 1) >> 24 (the arithmetic shift floors), which is the
// positive formula plus the sign word xi >> 31.
__device__ __forceinline__ int aln_quant(int val, float scale24) {
    const int xi = __float2int_rz(__int2float_rn(val) * scale24);
    return (xi + (1 << 23) + (xi >> 31)) >> 24;
}
// The same value from the unscaled product p = (float)v * scale (|p| <= 127 * (1 + 2^-23)): round-half-away-from-zero is
// trunc(p + copysign(c, p)) with c = 0.5 - 2^-25, the largest float below one half.  Take p = k + f >= 0 with integer k
// and fraction f.  If f < 0.5, the largest such p is one ulp(p) >= 2^-25 below k + 0.5, so the exact sum p + c is at
// least ulp(p) + 2^-25 below k + 1; the floats just below k + 1 are spaced ulp(p) (or ulp(p)/2 at a power of two) apart,
// so the sum rounds to a float below k + 1 and truncates to k.  If f >= 0.5, the exact sum is k + 1 - 2^-25 or more;
// for p >= 0.5 no float lies strictly between k + 1 - 2^-25 and k + 1 except at k = 0, f = 0.5, where the tie rounds to
// the even mantissa 1.0: the sum rounds to k + 1 or above and truncates to k + 1 (f < 1 keeps it below k + 2).
// Checked on every neighbour of every half-integer up to 127.5 and on 2*10^7 random products.
// One logic operation and one float add in place of two shifts and a three-input add.
__device__ __forceinline__ int aln_quant_f(int val, float scale) {
    const float p = __int2float_rn(val) * scale;
    const float c = __int_as_float(0x3EFFFFFF | (__float_as_int(p) & 0x80000000));
    return __float2int_rz(p + c);
}

// ---- exact float arithmetic without the conversion unit ----
// The reference's requantisation is float math ((float)v * scale, roundf, int division);
// the same values are produced here with adds against 1.5*2^23 on the ALU/FMA pipes,
// because int<->float conversion instructions run at a small fraction of their rate.
constexpr float kMagic = 12582912.0f;          // 1.5 * 2^23
constexpr int kMagicBits = 0x4B400000;
// (float)v for |v| < 2^22, exact
__device__ __forceinline__ float i2f_small(int v) { return __int_as_float(kMagicBits + v) - kMagic; }
// the same value through the conversion unit: used for a share of the conversions so that the otherwise idle unit
// takes load off the integer/float pipes
__device__ __forceinline__ float i2f_cvt(int v) { return __int2float_rn(v); }
// roundf(x) (half away from zero) as a float, for |x| < 2^22: round-to-nearest-even by the
// magic add, then the two tie cases that differ are corrected (x - rint(x) is exact).
__device__ __forceinline__ float roundf_small(float x) {
    float rf = (x + kMagic) - kMagic;
    float d = x - rf;
    if (d == 0.5f && x > 0.0f) rf += 1.0f;
    if (d == -0.5f && x < 0.0f) rf -= 1.0f;
    return rf;
}
// integer value of a float that holds an integer, |f| < 2^22
__device__ __forceinline__ int f2i_exact(float f) { return __float_as_int(f + kMagic) - kMagicBits; }

// trunc(a / mn) as C integer division does, for |a| < 2^16 and 1 <= mn <= 127, with rinv_up = (1/mn) * (1 + 2^-17):
// the factor pushes every quotient away from zero by |q| * 7.6e-6 -- more than the float error of the product
// (three roundings, < |q| * 1.8e-7), so an exact quotient k lands beyond k and truncates to k, and less than the
// distance 1/mn from a non-integer quotient to the next integer (|q| * 7.8e-6 < 1/mn because |q| * mn = |a| < 2^16).
// The configuration check bounds |x * gain| by 2^16 from the noise amplitude.
__device__ __forceinline__ int div_small(int a, float rinv_up) {
    return __float2int_rz(i2f_small(a) * rinv_up);
}

// [sat8(a), sat8(b), sat8(c), sat8(d)] as bytes 0..3 with the reference's clip to [-127, 127]
__device__ __forceinline__ uint32_t pack_clip8(int a, int b, int c, int d) {
    uint32_t hi, r;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
    return __vmaxs4(r, 0x81818181u);
}

// (1/mn) * (1 + 2^-17) for mn = 1..127 (div_small's factor): the mean is the same for every lane of a row, so the
// reciprocal is one constant-bank read instead of a division per row.  Compile-time IEEE single arithmetic, the same two
// roundings as the expression it replaces.  One copy per translation unit.
struct RinvTable { float v[128]; };
constexpr RinvTable make_rinv_table() {
    RinvTable t = {};
    for (int mn = 1; mn < 128; mn++) t.v[mn] = (1.0f / (float)mn) * (1.0f + 0x1p-17f);
    return t;
}
static __constant__ RinvTable c_rinv_up = make_rinv_table();

// Function attributes (dynamic shared-memory limits, cluster occupancy) belong to a device: caches of "already set" are
// kept per device so that one process may hold contexts on several GPUs.
constexpr int EGG_MAX_DEVICES = 64;
inline int current_device_slot() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0) d = 0;
    return d % EGG_MAX_DEVICES;
}

// ---------------------------------------------------------------- errors
void set_error(const char *fmt, ...);

#define EGG_CUDA(call)                                                                        \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess) {                                                              \
            egg::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
            return EGG_E_CUDA;                                                                \
        }                                                                                     \
    } while (0)

// device-side error record: flag[0] = code (0 ok), flag[1] = where
enum DevErr { DEV_OK = 0, DEV_TIMEOUT_FULL = 1, DEV_TIMEOUT_EMPTY = 2, DEV_TIMEOUT_TMEM_FULL = 3, DEV_TIMEOUT_TMEM_EMPTY = 4, DEV_TIMEOUT_PEER = 5 };

}  // namespace egg
