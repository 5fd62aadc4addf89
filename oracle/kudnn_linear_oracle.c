/*
 * CPU oracle for the KuDNN Linear(+post-op) path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a scalar restatement, in plain C, of what the reference library
 * computes for Gemm / LinearActivationLayerFWD / LinearResFWD.  It exists to
 * check the CUDA kernels and to serve as the timed CPU baseline; the shipped
 * library never links, loads or calls it.
 *
 * PARITY UNPINNED at bit level: the reference delegates the GEMM arithmetic to
 * the closed KML BLAS (kblas.h, HPCKit 26.0.RC1; call sites
 * src/dnn/src/kudnn_gemm.cpp:168-257) whose summation order is not published,
 * the reference needs aarch64 SVE/SME and cannot be built on x86, and its test
 * suite holds no golden vectors (inputs are time-seeded, results are compared
 * to a naive loop within a tolerance).  What IS pinned here is every step the
 * reference performs in its own source around that GEMM: the order of scaling,
 * bias, rounding, activation and residual, and the rounding mode of each.
 *
 * Reference steps restated (file:line in the reference tree):
 *   gemm + bias, fp32      src/dnn/src/kudnn_gemm.cpp:157-180  (sgemm, then AddBias :106-149)
 *   gemm + bias, fp16      src/dnn/src/kudnn_gemm.cpp:182-193  (hgemm -> fp16, AddBias in fp16)
 *   gemm + bias, bf16      src/dnn/src/kudnn_gemm.cpp:208-227  (sbgemm -> fp32, AddBias fp32, RNE -> bf16;
 *                                                               no bias: bgemm -> bf16)
 *   fp32 -> bf16 / fp16    src/dnn/src/service.cpp:48-75       (round to nearest even)
 *   activation pass        src/dnn/src/kudnn_linear_activationlayer.cpp:40-56 (runs on the rounded dst)
 *   relu                   src/dnn/src/kernels/vml/relu/relu.c:31-49
 *   swish / sigmoid        src/dnn/src/kernels/vml/swish/vml_sve_la_swishf.c:20-50,
 *                          src/dnn/src/kernels/vml/vml_sve_la_sigmoid.h:15-48 (argument clamp at +-87)
 *   gelu_tanh / tanh       src/dnn/src/kernels/vml/gelu_tanh/vml_sve_la_gelu_tanh.h:18-39,
 *                          src/dnn/src/kernels/vml/vml_sve_la_tanh.h:116-142
 *   gelu_erf               src/dnn/src/kernels/vml/gelu_erf/vml_sve_la_gelu_erf.h:20-28
 *   bf16 out = truncation  src/dnn/src/kernels/vml/vml_sve_base.h:111-118 ; fp16 out = RNE
 *   residual add / ext     src/dnn/src/kudnn_linear_res.cpp:57-122
 *   stand-alone activation src/dnn/src/kudnn_eltwise.cpp:500-586
 *   RMS normalisation      src/dnn/src/kernels/rmsnorm/kudnn_rmsnorm_fwd_last_def.hpp:128-180
 * The element-wise product with a gate tensor (KO_RES_ELTWISE_MUL) has no
 * counterpart in the reference (its RES_MUL is a second matrix product,
 * kudnn_linear_res.cpp:188-190); it is defined as rne(f32(c) * f32(gate)).
 * exp/tanh/erf use libm; the reference's SVE polynomial versions agree with
 * libm to about 1-2 ulp of fp32.
 *
 * Accumulation modes:
 *   KO_ACC_F32  fp32 products summed in 16 interleaved fp32 lanes (k mod 16), lanes
 *               then summed in order 0..15.  Fast (vectorises); this is the
 *               "faithful" stand-in for a fp32-accumulating BLAS and the CPU baseline.
 *   KO_ACC_F64  products and sum in fp64, strictly sequential in k, one final
 *               rounding to fp32.  Machine independent; this is the "ideal" oracle.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define KO_F32 1
#define KO_F16 2
#define KO_BF16 3
#define KO_S32 4
#define KO_S8 5
#define KO_U8 6

#define KO_ACT_NONE 0
#define KO_ACT_RELU 5
#define KO_ACT_TANH 9
#define KO_ACT_SIGMOID 10
#define KO_ACT_GELU_TANH 20
#define KO_ACT_SWISH 25
#define KO_ACT_GELU_ERF 27

#define KO_RES_NONE 0
#define KO_RES_EXT 1
#define KO_RES_IDENTICAL 2
#define KO_RES_ELTWISE_MUL 3

#define KO_ACC_F32 0
#define KO_ACC_F64 1

/* Same field order as the shipped library's descriptor so one Python structure serves both. */
typedef struct {
    int64_t m, n, k;
    int64_t batch[3];
    int32_t a_dtype, b_dtype, c_dtype, bias_dtype, res_dtype, out_dtype;
    int32_t has_bias, act, res_op, reserved;
    float act_alpha, act_beta;
    int64_t a_sm, a_sk, a_sb[3];
    int64_t b_sk, b_sn, b_sb[3];
    int64_t c_sm, c_sn, c_sb[3];
    int64_t bias_sm, bias_sn, bias_sb[3];
    int64_t res_sm, res_sn, res_sb[3];
    int64_t out_sm, out_sn, out_sb[3];
} ko_desc;

/* ------------------------------------------------------------------ 16-bit formats */

static inline float ko_bits_to_f32(uint32_t u)
{
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint32_t ko_f32_to_bits(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

float ko_bf16_to_f32(uint16_t h)
{
    return ko_bits_to_f32((uint32_t)h << 16);
}

/* round to nearest even, as BFCVT / vcvth_bf16_f32 do (service.cpp:48-68) */
uint16_t ko_f32_to_bf16_rne(float f)
{
    uint32_t u = ko_f32_to_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
        return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    }
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/* plain truncation, as the uzp2-based store of the bf16 activation kernels does (vml_sve_base.h:111-118) */
uint16_t ko_f32_to_bf16_trunc(float f)
{
    return (uint16_t)(ko_f32_to_bits(f) >> 16);
}

float ko_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) {
            return ko_bits_to_f32(sign);
        }
        /* subnormal: man * 2^-24 */
        float v = (float)man * 5.9604644775390625e-8f;
        return (sign != 0) ? -v : v;
    }
    if (exp == 31) {
        return ko_bits_to_f32(sign | 0x7f800000u | (man << 13));
    }
    return ko_bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* round to nearest even fp32 -> fp16 (the __fp16 conversion of service.cpp:70-75) */
uint16_t ko_f32_to_f16_rne(float f)
{
    uint32_t u = ko_f32_to_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t au = u & 0x7fffffffu;
    if (au > 0x7f800000u) {
        return (uint16_t)(sign | 0x7e00u);
    }
    if (au >= 0x47800000u) { /* >= 65536 -> inf (65520 rounds to inf too, handled below) */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (au < 0x38800000u) { /* below the smallest normal half: subnormal or zero */
        if (au < 0x33000000u) { /* < 2^-25 rounds to zero */
            return (uint16_t)sign;
        }
        int e = (int)(au >> 23);              /* biased exponent, 102..112 */
        uint32_t man = (au & 0x7fffffu) | 0x800000u;
        int shift = 126 - e;                  /* bits to drop: 14..24 */
        uint32_t q = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) {
            q++;
        }
        return (uint16_t)(sign | q);
    }
    uint32_t e = (au >> 23) - 112u;
    uint32_t man = au & 0x7fffffu;
    uint32_t q = (e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) {
        q++; /* carries into the exponent correctly, up to inf */
    }
    return (uint16_t)(sign | q);
}

static inline size_t ko_elem_size(int dtype)
{
    return (dtype == KO_F32 || dtype == KO_S32) ? 4 : ((dtype == KO_S8 || dtype == KO_U8) ? 1 : 2);
}

static inline float ko_load(const void *p, int dtype, int64_t idx)
{
    switch (dtype) {
        case KO_F32:
            return ((const float *)p)[idx];
        case KO_S8: /* widened exactly, as MatrixConverter S8 -> F16 does (kudnn_gemm.cpp:337-344) */
            return (float)((const int8_t *)p)[idx];
        case KO_U8:
            return (float)((const uint8_t *)p)[idx];
        case KO_S32:
            return (float)((const int32_t *)p)[idx];
        case KO_F16:
            return ko_f16_to_f32(((const uint16_t *)p)[idx]);
        default:
            return ko_bf16_to_f32(((const uint16_t *)p)[idx]);
    }
}

/* round v to the storage type and return the value it then holds */
static inline float ko_round_rne(float v, int dtype)
{
    switch (dtype) {
        case KO_F32:
            return v;
        case KO_F16:
            return ko_f16_to_f32(ko_f32_to_f16_rne(v));
        default:
            return ko_bf16_to_f32(ko_f32_to_bf16_rne(v));
    }
}

static inline void ko_store_exact(void *p, int dtype, int64_t idx, float v)
{
    /* v is already representable in dtype */
    switch (dtype) {
        case KO_F32:
            ((float *)p)[idx] = v;
            break;
        case KO_F16:
            ((uint16_t *)p)[idx] = ko_f32_to_f16_rne(v);
            break;
        default:
            ((uint16_t *)p)[idx] = ko_f32_to_bf16_trunc(v);
            break;
    }
}

/* ------------------------------------------------------------------ activations (fp32 math) */

static inline float ko_sigmoid_neg(float t)
{
    /* 1 / (1 + exp(t)) with the reference's argument clamp (vml_sve_la_sigmoid.h:39-48) */
    if (t > 87.0f) {
        return 0.0f;
    }
    if (t < -87.0f) {
        return 1.0f;
    }
    return 1.0f / (1.0f + expf(t));
}

static inline float ko_tanh_ref(float y)
{
    /* vml_sve_la_tanh.h:116-142 */
    if (fabsf(y) < 0.05f) {
        return y * (1.0f - y * y * (1.0f / 3.0f));
    }
    float e = expf(y + y);
    return 1.0f - 2.0f / (1.0f + e);
}

float ko_activation(float x, int act, float alpha)
{
    switch (act) {
        case KO_ACT_NONE:
            return x;
        case KO_ACT_RELU:
            return (x <= 0.0f) ? x * alpha : x;
        case KO_ACT_SWISH:
            return x * ko_sigmoid_neg(-(x * alpha));
        case KO_ACT_SIGMOID:
            return ko_sigmoid_neg(-x);
        case KO_ACT_TANH:
            return tanhf(x);
        case KO_ACT_GELU_TANH: {
            float y = (1.0f + x * x * 0.044715f) * x * 0.7978845608f;
            return (1.0f + ko_tanh_ref(y)) * 0.5f * x;
        }
        case KO_ACT_GELU_ERF: {
            float s = x * 0.5f;
            return s * erff(x * 0.70710678118f) + s;
        }
        default:
            return NAN;
    }
}

/* rounding of an activation result into the storage type: f16 RNE, bf16 truncation.  The bf16 relu kernel first
 * turns a finite result whose magnitude pattern is 0x7f7f8000 or above (it would round to infinity) into infinity
 * (vml_sve_base.h:97-109, relu/relu.c:229-232). */
static inline float ko_round_act(float v, int dtype, int act)
{
    switch (dtype) {
        case KO_F32:
            return v;
        case KO_F16:
            return ko_f16_to_f32(ko_f32_to_f16_rne(v));
        default: {
            uint32_t u = ko_f32_to_bits(v);
            if (act == KO_ACT_RELU && (u & 0x7fffffffu) >= 0x7f7f8000u && (u & 0x7fffffffu) < 0x7f800000u) {
                u = (u & 0x80000000u) | 0x7f800000u;
            }
            return ko_bits_to_f32(u & 0xffff0000u);
        }
    }
}

/* ------------------------------------------------------------------ post-GEMM chain for one element */

typedef struct {
    float c;   /* value stored to c   */
    float out; /* value stored to out */
} ko_pair;

static inline ko_pair ko_finish(const ko_desc *d, float acc, float alpha, float beta, float gamma, float c_old,
                                int have_bias, float bias, int have_res, float res)
{
    const int ct = d->c_dtype;
    float t = alpha * acc;
    if (beta != 0.0f) {
        t += beta * c_old;
    }
    float c1;
    if (ct == KO_F16 && d->a_dtype == KO_F16 && d->b_dtype == KO_F16 && (!have_bias || d->bias_dtype == KO_F16)) {
        /* hgemm writes fp16, the bias is then added in __fp16 (kudnn_gemm.cpp:189-192, :111) */
        c1 = ko_round_rne(t, KO_F16);
        if (have_bias) {
            c1 = ko_round_rne(c1 + bias, KO_F16);
        }
    } else {
        /* fp32: plain add; bf16: add in fp32 then one RNE (kudnn_gemm.cpp:216-221); fp16 result with a wider
         * bias or with 8-bit weights (W8A16): the product and the bias add run in fp32 and the result is rounded
         * once (kudnn_gemm.cpp:679-692 and the <fp16, s8|u8, fp16, float> wrappers :336-372) */
        if (have_bias) {
            t += bias;
        }
        c1 = ko_round_rne(t, ct);
    }
    float c2 = c1;
    if (d->act != KO_ACT_NONE) {
        c2 = ko_round_act(ko_activation(c1, d->act, d->act_alpha), ct, d->act);
    }
    ko_pair r;
    r.c = c2;
    r.out = 0.0f;
    if (have_res) {
        float o;
        switch (d->res_op) {
            case KO_RES_IDENTICAL:
                o = c2 + res;
                break;
            case KO_RES_EXT:
                o = fmaf(res, gamma, c2);
                break;
            default: /* KO_RES_ELTWISE_MUL */
                o = c2 * res;
                break;
        }
        r.out = ko_round_rne(o, d->out_dtype);
    }
    return r;
}

/* ------------------------------------------------------------------ GEMM cores */

#define KO_LANES 16
typedef float ko_vf __attribute__((vector_size(KO_LANES * 4), aligned(4)));

static inline float ko_lane_sum(const ko_vf *v)
{
    float lanes[KO_LANES];
    memcpy(lanes, v, sizeof(lanes));
    float s = 0.0f;
    for (int i = 0; i < KO_LANES; ++i) {
        s += lanes[i];
    }
    return s;
}

/* dot of two contiguous fp32 rows of length kp (multiple of 16, zero padded): lane l sums k = l mod 16 */
static inline float ko_dot_f32(const float *a, const float *b, int64_t kp)
{
    ko_vf acc = {0};
    for (int64_t k = 0; k < kp; k += KO_LANES) {
        ko_vf va, vb;
        memcpy(&va, a + k, sizeof(va));
        memcpy(&vb, b + k, sizeof(vb));
        acc += va * vb;
    }
    return ko_lane_sum(&acc);
}

/* 4 x 4 register block of the same lane-wise sums; bit-identical to ko_dot_f32 per element */
static inline void ko_dot_4x4(const float *a, int64_t lda, const float *b, int64_t ldb, int64_t kp, float out[4][4])
{
    ko_vf acc[4][4];
    memset(acc, 0, sizeof(acc));
    for (int64_t k = 0; k < kp; k += KO_LANES) {
        ko_vf va[4], vb[4];
        for (int i = 0; i < 4; ++i) {
            memcpy(&va[i], a + i * lda + k, sizeof(ko_vf));
            memcpy(&vb[i], b + i * ldb + k, sizeof(ko_vf));
        }
        for (int i = 0; i < 4; ++i) {
            for (int j = 0; j < 4; ++j) {
                acc[i][j] += va[i] * vb[j];
            }
        }
    }
    for (int i = 0; i < 4; ++i) {
        for (int j = 0; j < 4; ++j) {
            out[i][j] = ko_lane_sum(&acc[i][j]);
        }
    }
}

static inline float ko_dot_f64(const float *a, const float *b, int64_t k)
{
    double s = 0.0;
    for (int64_t i = 0; i < k; ++i) {
        s += (double)a[i] * (double)b[i];
    }
    return (float)s;
}

/* gather one [rows, k] operand into contiguous, zero-padded fp32 rows */
static void ko_pack(const void *src, int dtype, int64_t rows, int64_t k, int64_t s_row, int64_t s_k, float *dst,
                    int64_t kp)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float *o = dst + r * kp;
        for (int64_t i = 0; i < k; ++i) {
            o[i] = ko_load(src, dtype, r * s_row + i * s_k);
        }
        for (int64_t i = k; i < kp; ++i) {
            o[i] = 0.0f;
        }
    }
}

int ko_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * One Linear(+post-op) evaluation.  Returns 0 on success, -1 on bad arguments, -2 on allocation failure.
 * c may be NULL when only `out` is wanted; out must be non-NULL iff res_op != KO_RES_NONE.
 */
int ko_linear(const ko_desc *d, const void *a, const void *b, void *c, const void *bias, const void *res, void *out,
              float alpha, float beta, float gamma, int acc_mode, int num_threads)
{
    if (d == NULL || a == NULL || b == NULL || d->m <= 0 || d->n <= 0 || d->k <= 0) {
        return -1;
    }
    if ((d->has_bias != 0) != (bias != NULL)) {
        return -1;
    }
    if ((d->res_op != KO_RES_NONE) != (res != NULL && out != NULL)) {
        return -1;
    }
    if (c == NULL && out == NULL) {
        return -1;
    }
#ifdef _OPENMP
    if (num_threads > 0) {
        omp_set_num_threads(num_threads);
    }
#else
    (void)num_threads;
#endif
    if (d->a_dtype == KO_BF16 && d->b_dtype == KO_BF16 && d->c_dtype == KO_BF16 && !d->has_bias) {
        /* the bias-free bf16 product is cblas_bgemm, which takes its two scalars as bf16 (kudnn_gemm.cpp:222-226) */
        alpha = ko_bf16_to_f32(ko_f32_to_bf16_rne(alpha));
        beta = ko_bf16_to_f32(ko_f32_to_bf16_rne(beta));
    }
    const int64_t m = d->m, n = d->n, k = d->k;
    const int64_t kp = (k + KO_LANES - 1) / KO_LANES * KO_LANES;
    float *pa = (float *)aligned_alloc(64, (size_t)(m * kp) * sizeof(float));
    float *pb = (float *)aligned_alloc(64, (size_t)(n * kp) * sizeof(float));
    if (pa == NULL || pb == NULL) {
        free(pa);
        free(pb);
        return -2;
    }
    const int64_t nb0 = d->batch[0] > 0 ? d->batch[0] : 1;
    const int64_t nb1 = d->batch[1] > 0 ? d->batch[1] : 1;
    const int64_t nb2 = d->batch[2] > 0 ? d->batch[2] : 1;
    for (int64_t i0 = 0; i0 < nb0; ++i0) {
        for (int64_t i1 = 0; i1 < nb1; ++i1) {
            for (int64_t i2 = 0; i2 < nb2; ++i2) {
                const int64_t oa = i0 * d->a_sb[0] + i1 * d->a_sb[1] + i2 * d->a_sb[2];
                const int64_t ob = i0 * d->b_sb[0] + i1 * d->b_sb[1] + i2 * d->b_sb[2];
                const int64_t oc = i0 * d->c_sb[0] + i1 * d->c_sb[1] + i2 * d->c_sb[2];
                const int64_t obias = i0 * d->bias_sb[0] + i1 * d->bias_sb[1] + i2 * d->bias_sb[2];
                const int64_t ores = i0 * d->res_sb[0] + i1 * d->res_sb[1] + i2 * d->res_sb[2];
                const int64_t oout = i0 * d->out_sb[0] + i1 * d->out_sb[1] + i2 * d->out_sb[2];
                const size_t esa = ko_elem_size(d->a_dtype);
                const size_t esb = ko_elem_size(d->b_dtype);
                ko_pack((const char *)a + oa * (int64_t)esa, d->a_dtype, m, k, d->a_sm, d->a_sk, pa, kp);
                ko_pack((const char *)b + ob * (int64_t)esb, d->b_dtype, n, k, d->b_sn, d->b_sk, pb, kp);
                const int64_t mb = (m + 3) / 4, nbk = (n + 3) / 4;
#pragma omp parallel for collapse(2) schedule(static)
                for (int64_t bi = 0; bi < mb; ++bi) {
                    for (int64_t bj = 0; bj < nbk; ++bj) {
                        const int64_t r0 = bi * 4, c0 = bj * 4;
                        float blk[4][4];
                        const int full = (r0 + 4 <= m) && (c0 + 4 <= n);
                        if (acc_mode == KO_ACC_F32 && full) {
                            ko_dot_4x4(pa + r0 * kp, kp, pb + c0 * kp, kp, kp, blk);
                        } else {
                            for (int i = 0; i < 4 && r0 + i < m; ++i) {
                                for (int j = 0; j < 4 && c0 + j < n; ++j) {
                                    blk[i][j] = (acc_mode == KO_ACC_F64)
                                                    ? ko_dot_f64(pa + (r0 + i) * kp, pb + (c0 + j) * kp, k)
                                                    : ko_dot_f32(pa + (r0 + i) * kp, pb + (c0 + j) * kp, kp);
                                }
                            }
                        }
                        for (int i = 0; i < 4 && r0 + i < m; ++i) {
                            for (int j = 0; j < 4 && c0 + j < n; ++j) {
                                const int64_t mi = r0 + i, ni = c0 + j;
                                const int64_t ic = oc + mi * d->c_sm + ni * d->c_sn;
                                float c_old = 0.0f, bv = 0.0f, rv = 0.0f;
                                if (beta != 0.0f && c != NULL) {
                                    c_old = ko_load(c, d->c_dtype, ic);
                                }
                                if (d->has_bias) {
                                    bv = ko_load(bias, d->bias_dtype, obias + mi * d->bias_sm + ni * d->bias_sn);
                                }
                                if (d->res_op != KO_RES_NONE) {
                                    rv = ko_load(res, d->res_dtype, ores + mi * d->res_sm + ni * d->res_sn);
                                }
                                ko_pair r = ko_finish(d, blk[i][j], alpha, beta, gamma, c_old, d->has_bias, bv,
                                                      d->res_op != KO_RES_NONE, rv);
                                if (c != NULL) {
                                    ko_store_exact(c, d->c_dtype, ic, r.c);
                                }
                                if (d->res_op != KO_RES_NONE) {
                                    ko_store_exact(out, d->out_dtype, oout + mi * d->out_sm + ni * d->out_sn, r.out);
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    free(pa);
    free(pb);
    return 0;
}

/*
 * 8-bit integer product <s8|u8, s8|u8, s32, s32> (GEMMWrapper, src/dnn/src/kudnn_gemm.cpp:259-334: cblas_gemm_*s32
 * with zero operand offsets, the bias passed as the row / column / fixed offset of c or added afterwards by AddBias).
 * The arithmetic of the closed BLAS is taken to be exact 32-bit sums; with alpha = 1 and beta = 0 or 1 everything
 * stays in integers, other scalars go through fp64 and round to nearest.  2-D or batched, any strides.
 */
int ko_linear_int(const ko_desc *d, const void *a, const void *b, void *c, const void *bias, float alpha, float beta)
{
    if (d == NULL || a == NULL || b == NULL || c == NULL || d->c_dtype != KO_S32 || (d->has_bias != 0) != (bias != NULL)) {
        return -1;
    }
    const int64_t nb0 = d->batch[0] > 0 ? d->batch[0] : 1, nb1 = d->batch[1] > 0 ? d->batch[1] : 1;
    const int64_t nb2 = d->batch[2] > 0 ? d->batch[2] : 1;
    int32_t *cc = (int32_t *)c;
    for (int64_t i0 = 0; i0 < nb0; ++i0) {
        for (int64_t i1 = 0; i1 < nb1; ++i1) {
            for (int64_t i2 = 0; i2 < nb2; ++i2) {
                const int64_t oa = i0 * d->a_sb[0] + i1 * d->a_sb[1] + i2 * d->a_sb[2];
                const int64_t ob = i0 * d->b_sb[0] + i1 * d->b_sb[1] + i2 * d->b_sb[2];
                const int64_t oc = i0 * d->c_sb[0] + i1 * d->c_sb[1] + i2 * d->c_sb[2];
                const int64_t obias = i0 * d->bias_sb[0] + i1 * d->bias_sb[1] + i2 * d->bias_sb[2];
#pragma omp parallel for collapse(2) schedule(static)
                for (int64_t mi = 0; mi < d->m; ++mi) {
                    for (int64_t ni = 0; ni < d->n; ++ni) {
                        int64_t acc = 0;
                        for (int64_t kk = 0; kk < d->k; ++kk) {
                            const int64_t ia = oa + mi * d->a_sm + kk * d->a_sk, ib = ob + kk * d->b_sk + ni * d->b_sn;
                            const int av = d->a_dtype == KO_S8 ? ((const int8_t *)a)[ia] : ((const uint8_t *)a)[ia];
                            const int bv = d->b_dtype == KO_S8 ? ((const int8_t *)b)[ib] : ((const uint8_t *)b)[ib];
                            acc += av * bv;
                        }
                        const int64_t ic = oc + mi * d->c_sm + ni * d->c_sn;
                        int64_t r = acc;
                        if (alpha != 1.0f || (beta != 0.0f && beta != 1.0f)) {
                            double t = (double)alpha * (double)acc;
                            if (beta != 0.0f) {
                                t += (double)beta * cc[ic];
                            }
                            r = llrint(t);
                        } else if (beta == 1.0f) {
                            r += cc[ic];
                        }
                        if (d->has_bias) {
                            r += ((const int32_t *)bias)[obias + mi * d->bias_sm + ni * d->bias_sn];
                        }
                        r = r > 2147483647ll ? 2147483647ll : (r < -2147483648ll ? -2147483648ll : r);
                        cc[ic] = (int32_t)r;
                    }
                }
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ the operators either side of Linear */

/*
 * Stand-alone activation pass over a dense tensor (ActivationLayerImplFWD::RunSequential,
 * src/dnn/src/kudnn_eltwise.cpp:500-586): equal types run the typed kernel (fp32 arithmetic, fp16 RNE, bf16
 * truncation, bf16 relu overflow rule); different types convert to fp32, run the fp32 kernel and convert back with
 * one rounding to nearest even (:512-523, :577-584).
 */
int ko_activation_run(const void *src, void *dst, int64_t count, int src_dtype, int dst_dtype, int act, float alpha)
{
    if (src == NULL || dst == NULL || count <= 0) {
        return -1;
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        const float y = ko_activation(ko_load(src, src_dtype, i), act, alpha);
        if (src_dtype == dst_dtype) {
            ko_store_exact(dst, dst_dtype, i, ko_round_act(y, dst_dtype, act));
        } else {
            ko_store_exact(dst, dst_dtype, i, ko_round_rne(y, dst_dtype));
        }
    }
    return 0;
}

/*
 * RMS normalisation over the last axis of a dense [rows, axis] tensor (RMSNorm::EvaluateLastAxis,
 * src/dnn/src/kernels/rmsnorm/kudnn_rmsnorm_fwd_last_def.hpp:128-180): the variance is the mean of the squares,
 * accumulated in fp32 vector lanes (here 16) and divided by the axis length, or the caller's value with
 * USE_GLOBAL_STATS (flag 1); the multiplier of an element is scale * (1 / sqrt(variance + eps)) (flag 2, :49-72) or
 * the inverse root alone; x times the multiplier is computed in fp32 and rounded once.
 */
int ko_rmsnorm(const void *src, void *dst, const void *scale, float *variance, int64_t rows, int64_t axis, int dtype,
               int flags, int save_stats, float eps)
{
    const int use_stats = (flags & 1) != 0, use_scale = (flags & 2) != 0;
    if (src == NULL || dst == NULL || rows <= 0 || axis <= 0 || ((use_stats || save_stats) && variance == NULL) ||
        (use_scale && scale == NULL)) {
        return -1;
    }
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < rows; ++n) {
        float var;
        if (use_stats) {
            var = variance[n];
        } else {
            float lanes[KO_LANES] = {0};
            for (int64_t i = 0; i < axis; ++i) {
                const float x = ko_load(src, dtype, n * axis + i);
                lanes[i % KO_LANES] += x * x;
            }
            float sum = 0.0f;
            for (int l = 0; l < KO_LANES; ++l) {
                sum += lanes[l];
            }
            var = sum / (float)axis;
            if (save_stats) {
                variance[n] = var;
            }
        }
        const float inv = 1.0f / sqrtf(var + eps);
        for (int64_t i = 0; i < axis; ++i) {
            const float c = use_scale ? ko_load(scale, dtype, i) * inv : inv;
            ko_store_exact(dst, dtype, n * axis + i, ko_round_rne(ko_load(src, dtype, n * axis + i) * c, dtype));
        }
    }
    return 0;
}

/* Bulk converters for the Python side (fixtures, input preparation). */
void ko_convert_f32_to_bf16(const float *src, uint16_t *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) {
        dst[i] = ko_f32_to_bf16_rne(src[i]);
    }
}
void ko_convert_f32_to_f16(const float *src, uint16_t *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) {
        dst[i] = ko_f32_to_f16_rne(src[i]);
    }
}
void ko_convert_bf16_to_f32(const uint16_t *src, float *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) {
        dst[i] = ko_bf16_to_f32(src[i]);
    }
}
void ko_convert_f16_to_f32(const uint16_t *src, float *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) {
        dst[i] = ko_f16_to_f32(src[i]);
    }
}
