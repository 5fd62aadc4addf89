// Shared device helpers: storage-type conversion, the post-GEMM chain (scale, bias, rounding,
// activation, second output) and the parameter blocks every kernel family consumes.
//
// The chain follows the order and rounding modes of the reference library:
//   bias / rounding   src/dnn/src/kudnn_gemm.cpp:157-227 (fp32: add; fp16: round, add in fp16; bf16: add in fp32, RNE;
//                     fp16 result with a wider bias: add in fp32, one RNE, :348-360 and :679-692)
//   activation        src/dnn/src/kudnn_linear_activationlayer.cpp:40-56 on the rounded value, fp32 math,
//                     fp16 result RNE, bf16 result truncated (src/dnn/src/kernels/vml/vml_sve_base.h:111-118)
//   second output     src/dnn/src/kudnn_linear_res.cpp:57-122 (RNE)
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kudnn_b200.h"

namespace kb {

constexpr int kErrNone = 0;
constexpr int kErrTimeout = 1;

// Device-visible status block of a handle.
struct DeviceStatus {
    int code;   // kErr*
    int where;  // which wait gave up (kernel-specific tag)
    int block;  // blockIdx.x of the reporter
    int pad;
};

constexpr int kMaxMirrors = 7;

struct EpiParams {
    void *c;
    const void *bias;
    const void *res;
    void *out;
    long long c_sm, c_sn, bias_sm, bias_sn, res_sm, res_sn, out_sm, out_sn;
    float alpha, beta, gamma, act_alpha;
    int c_dtype, bias_dtype, res_dtype, out_dtype;
    int has_bias, act, res_op;
    // fp16 result of the <fp16, fp16, fp16, fp16> instance: rounded to fp16 before the bias is added in fp16.  Every
    // other fp16 result (wider bias, 8-bit weights) adds the bias in fp32 and rounds once.
    int half_chain;
    int m, n;
    // Mirrors: further copies of the outputs (same strides), e.g. the same tensor in every peer GPU's memory, written
    // by the same stores.  Byte distance of each mirror from c / out.
    int n_mirrors;
    long long c_delta[kMaxMirrors], out_delta[kMaxMirrors];
    // Multicast: byte distance from c / out to the address at which the same tensor is mapped through an NVLink
    // multicast object that spans every rank's copy (this rank's included).  Where a kernel has a multicast store
    // path, one such store replaces the local store and all the mirror stores; elsewhere the mirrors are used.
    int use_multicast;
    long long c_mc_delta, out_mc_delta;
};

// Writes v (exactly representable in dtype) to base[idx] and to the same element of every mirror.
__device__ __forceinline__ void store_exact_mirrored(void *base, int dtype, long long idx, float v, int n_mirrors,
                                                     const long long *delta);

__device__ __forceinline__ float bf16_bits_to_f32(unsigned short h)
{
    return __uint_as_float(static_cast<unsigned>(h) << 16);
}
__device__ __forceinline__ unsigned short f32_to_bf16_rne_bits(float f)
{
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float f16_bits_to_f32(unsigned short h)
{
    return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ unsigned short f32_to_f16_rne_bits(float f)
{
    return __half_as_ushort(__float2half_rn(f));
}

__device__ __forceinline__ float load_as_f32(const void *p, int dtype, long long idx)
{
    if (dtype == KUDNN_B200_F32) {
        return static_cast<const float *>(p)[idx];
    }
    if (dtype == KUDNN_B200_S8) {
        return static_cast<float>(static_cast<const signed char *>(p)[idx]);
    }
    if (dtype == KUDNN_B200_U8) {
        return static_cast<float>(static_cast<const unsigned char *>(p)[idx]);
    }
    if (dtype == KUDNN_B200_S32) {
        return static_cast<float>(static_cast<const int *>(p)[idx]);
    }
    unsigned short h = static_cast<const unsigned short *>(p)[idx];
    return dtype == KUDNN_B200_F16 ? f16_bits_to_f32(h) : bf16_bits_to_f32(h);
}

// value held after a round-to-nearest-even store into `dtype`
__device__ __forceinline__ float round_rne(float v, int dtype)
{
    if (dtype == KUDNN_B200_F32) {
        return v;
    }
    if (dtype == KUDNN_B200_F16) {
        return __half2float(__float2half_rn(v));
    }
    return __bfloat162float(__float2bfloat16_rn(v));
}

// The reference's bf16 relu turns a finite result that would round to infinity (magnitude pattern 0x7f7f8000 or
// above) into infinity before it truncates (src/dnn/src/kernels/vml/vml_sve_base.h:97-109).  Only a negative slope
// can produce such a value from a bf16 input.
__device__ __forceinline__ float relu_bf16_overflow(float v)
{
    const unsigned u = __float_as_uint(v), mag = u & 0x7fffffffu;
    return (mag >= 0x7f7f8000u && mag < 0x7f800000u) ? __uint_as_float((u & 0x80000000u) | 0x7f800000u) : v;
}

// value held after storing an activation result: fp16 RNE, bf16 truncation
__device__ __forceinline__ float round_act(float v, int dtype, int act = KUDNN_B200_ACT_NONE, float act_alpha = 0.0f)
{
    if (dtype == KUDNN_B200_F32) {
        return v;
    }
    if (dtype == KUDNN_B200_F16) {
        return __half2float(__float2half_rn(v));
    }
    if (act == KUDNN_B200_ACT_RELU && act_alpha != 0.0f) {
        v = relu_bf16_overflow(v);
    }
    return __uint_as_float(__float_as_uint(v) & 0xffff0000u);
}

// v is exactly representable in dtype
__device__ __forceinline__ void store_exact(void *p, int dtype, long long idx, float v)
{
    if (dtype == KUDNN_B200_F32) {
        static_cast<float *>(p)[idx] = v;
    } else if (dtype == KUDNN_B200_F16) {
        static_cast<unsigned short *>(p)[idx] = f32_to_f16_rne_bits(v);
    } else {
        static_cast<unsigned short *>(p)[idx] = static_cast<unsigned short>(__float_as_uint(v) >> 16);
    }
}

__device__ __forceinline__ void store_exact_mirrored(void *base, int dtype, long long idx, float v, int n_mirrors,
                                                     const long long *delta)
{
    store_exact(base, dtype, idx, v);
    for (int i = 0; i < n_mirrors; ++i) {
        store_exact(static_cast<char *>(base) + delta[i], dtype, idx, v);
    }
}

// 1 / (1 + exp(t)); the reference clamps the exponent argument to [-87, 87]
// (src/dnn/src/kernels/vml/vml_sve_la_sigmoid.h:39-48).
template <bool kPrecise>
__device__ __forceinline__ float sigmoid_neg(float t)
{
    // No explicit clamp is needed: beyond +87 the exponential overflows to +inf and the quotient is 0, beyond -87 it
    // underflows and the quotient is 1, which are the reference's clamped values (a denormal instead of 0 in the
    // sliver 87 < t < 88.7).  Branch-free, so eight of these interleave in the epilogues.
    return kPrecise ? (1.0f / (1.0f + expf(t))) : __fdividef(1.0f, 1.0f + __expf(t));
}

// kPrecise selects libm-grade exp/erf (fp32 outputs); otherwise the fast hardware approximations, whose error
// (about 1e-6 relative) is far below one unit of a 16-bit result.
template <bool kPrecise>
__device__ __forceinline__ float activation(float x, int act, float alpha)
{
    switch (act) {
        case KUDNN_B200_ACT_RELU:
            return (x <= 0.0f) ? x * alpha : x;
        case KUDNN_B200_ACT_SWISH:
            return x * sigmoid_neg<kPrecise>(-(x * alpha));
        case KUDNN_B200_ACT_SIGMOID:
            return sigmoid_neg<kPrecise>(-x);
        case KUDNN_B200_ACT_TANH:
            return tanhf(x);
        case KUDNN_B200_ACT_GELU_TANH: {
            // src/dnn/src/kernels/vml/gelu_tanh/vml_sve_la_gelu_tanh.h:22-39, tanh as vml_sve_la_tanh.h:116-142:
            // y (1 - y^2 / 3) below 0.05, 1 - 2 / (1 + exp(2y)) otherwise; both evaluated, one selected
            const float y = (1.0f + x * x * 0.044715f) * x * 0.7978845608f;
            const float small = y * (1.0f - y * y * (1.0f / 3.0f));
            const float yc = fminf(y, 40.0f);  // exp(2 * 40) is finite; tanh is 1 to fp32 precision long before
            const float e = kPrecise ? expf(yc + yc) : __expf(yc + yc);
            const float big = kPrecise ? (1.0f - 2.0f / (1.0f + e)) : (1.0f - __fdividef(2.0f, 1.0f + e));
            const float th = (fabsf(y) < 0.05f) ? small : big;
            return (1.0f + th) * 0.5f * x;
        }
        case KUDNN_B200_ACT_GELU_ERF: {
            float s = x * 0.5f;
            return s * erff(x * 0.70710678118f) + s;
        }
        default:
            return x;
    }
}

struct EpiResult {
    float c;
    float out;
};

// Out-of-line evaluation of any supported activation, for callers that do not fix the activation at compile time.
static __device__ __noinline__ float activation_any(float x, int act, float alpha, int precise)
{
    return precise ? activation<true>(x, act, alpha) : activation<false>(x, act, alpha);
}

// The post-GEMM chain for one element, everything already widened to fp32.  kAct >= 0 fixes the activation at
// compile time and kPrecise its arithmetic (1 = libm grade, for fp32 results; 0 = fast approximations), so that only
// that code is emitted; kAct = -1 reads the activation from the parameters and evaluates it out of line.
template <int kAct = -1, int kPrecise = -1>
__device__ __forceinline__ EpiResult finish_element(const EpiParams &p, float acc, float c_old, float bias, float res)
{
    const int ct = p.c_dtype;
    float t = p.alpha * acc;
    if (p.beta != 0.0f) {
        t += p.beta * c_old;
    }
    float c1;
    if (p.half_chain != 0) {
        c1 = round_rne(t, KUDNN_B200_F16);
        if (p.has_bias) {
            c1 = round_rne(c1 + bias, KUDNN_B200_F16);
        }
    } else {
        // fp32 and bf16 results, and fp16 results with a wider bias: the bias is added in fp32, one rounding
        if (p.has_bias) {
            t += bias;
        }
        c1 = round_rne(t, ct);
    }
    float c2 = c1;
    if (kAct < 0) {
        if (p.act != KUDNN_B200_ACT_NONE) {
            c2 = round_act(activation_any(c1, p.act, p.act_alpha, ct == KUDNN_B200_F32 ? 1 : 0), ct, p.act, p.act_alpha);
        }
    } else if (kAct != KUDNN_B200_ACT_NONE) {
        float a;
        if (kPrecise == 1) {
            a = activation<true>(c1, kAct, p.act_alpha);
        } else if (kPrecise == 0) {
            a = activation<false>(c1, kAct, p.act_alpha);
        } else {
            a = (ct == KUDNN_B200_F32) ? activation<true>(c1, kAct, p.act_alpha) : activation<false>(c1, kAct, p.act_alpha);
        }
        c2 = round_act(a, ct, kAct, p.act_alpha);
    }
    EpiResult r;
    r.c = c2;
    r.out = 0.0f;
    if (p.res_op != KUDNN_B200_RES_NONE) {
        float o;
        if (p.res_op == KUDNN_B200_RES_IDENTICAL) {
            o = c2 + res;
        } else if (p.res_op == KUDNN_B200_RES_EXT) {
            o = fmaf(res, p.gamma, c2);
        } else {
            o = c2 * res;
        }
        r.out = round_rne(o, p.out_dtype);
    }
    return r;
}

// Scalar form used by the general and the streaming kernels: loads the side inputs for (mi, ni), finishes, stores.
// Pointers are already offset to the current batch.
__device__ __forceinline__ void epilogue_scalar(const EpiParams &p, float acc, long long mi, long long ni)
{
    float c_old = 0.0f, bias = 0.0f, res = 0.0f;
    const long long ic = mi * p.c_sm + ni * p.c_sn;
    if (p.beta != 0.0f && p.c != nullptr) {
        c_old = load_as_f32(p.c, p.c_dtype, ic);
    }
    if (p.has_bias) {
        bias = load_as_f32(p.bias, p.bias_dtype, mi * p.bias_sm + ni * p.bias_sn);
    }
    if (p.res_op != KUDNN_B200_RES_NONE) {
        res = load_as_f32(p.res, p.res_dtype, mi * p.res_sm + ni * p.res_sn);
    }
    EpiResult r = finish_element(p, acc, c_old, bias, res);
    if (p.c != nullptr) {
        store_exact_mirrored(p.c, p.c_dtype, ic, r.c, p.n_mirrors, p.c_delta);
    }
    if (p.res_op != KUDNN_B200_RES_NONE) {
        store_exact_mirrored(p.out, p.out_dtype, mi * p.out_sm + ni * p.out_sn, r.out, p.n_mirrors, p.out_delta);
    }
}

// Batch addressing shared by all kernels: up to three leading dimensions, element strides per tensor.
struct BatchParams {
    long long n1, n2;  // extents of the two inner batch dimensions (outer extent is implied by the grid)
    long long a_sb[3], b_sb[3], c_sb[3], bias_sb[3], res_sb[3], out_sb[3];
};

__device__ __forceinline__ void batch_decompose(const BatchParams &bp, long long flat, long long idx[3])
{
    idx[2] = flat % bp.n2;
    long long r = flat / bp.n2;
    idx[1] = r % bp.n1;
    idx[0] = r / bp.n1;
}

__device__ __forceinline__ long long batch_offset(const long long sb[3], const long long idx[3])
{
    return idx[0] * sb[0] + idx[1] * sb[1] + idx[2] * sb[2];
}

__host__ __device__ __forceinline__ int dtype_size(int dtype)
{
    return (dtype == KUDNN_B200_F32 || dtype == KUDNN_B200_S32) ? 4 : ((dtype == KUDNN_B200_S8 || dtype == KUDNN_B200_U8) ? 1 : 2);
}

__device__ __forceinline__ void *offset_ptr(void *p, int dtype, long long elems)
{
    return p == nullptr ? nullptr : static_cast<void *>(static_cast<char *>(p) + elems * dtype_size(dtype));
}
__device__ __forceinline__ const void *offset_ptr(const void *p, int dtype, long long elems)
{
    return p == nullptr ? nullptr
                        : static_cast<const void *>(static_cast<const char *>(p) + elems * dtype_size(dtype));
}

// Applies the batch offsets of flat batch index `flat` to the epilogue pointers.
__device__ __forceinline__ EpiParams epi_for_batch(const EpiParams &p, const BatchParams &bp, long long flat)
{
    long long idx[3];
    batch_decompose(bp, flat, idx);
    EpiParams q = p;
    q.c = offset_ptr(p.c, p.c_dtype, batch_offset(bp.c_sb, idx));
    q.bias = offset_ptr(p.bias, p.bias_dtype, batch_offset(bp.bias_sb, idx));
    q.res = offset_ptr(p.res, p.res_dtype, batch_offset(bp.res_sb, idx));
    q.out = offset_ptr(p.out, p.out_dtype, batch_offset(bp.out_sb, idx));
    return q;
}

}  // namespace kb
