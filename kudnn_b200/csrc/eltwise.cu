// The two operators that sit either side of Linear in a transformer block, as stand-alone HBM-bound kernels:
//   * the element-wise activation pass (reference: ActivationLayerImplFWD::RunSequential,
//     src/dnn/src/kudnn_eltwise.cpp:500-586: fp32 arithmetic, fp16 results rounded to nearest even, bf16 results
//     truncated, src/dnn/src/kernels/vml/vml_sve_base.h:111-118; different source and result types go through fp32
//     and one rounding);
//   * RMS normalisation over the last axis (reference: RMSNorm::EvaluateLastAxis,
//     src/dnn/src/kernels/rmsnorm/kudnn_rmsnorm_fwd_last_def.hpp:128-180: variance = mean of squares in fp32, or the
//     caller's statistics; y = x * (scale * 1 / sqrt(variance + eps)), fp32 arithmetic, one rounding).
// Both read every input once and write every output once with 16-byte accesses; a row of the normalisation stays in
// registers between the reduction and the scaling.
#include "kernels.cuh"

namespace kb {

namespace {

constexpr int kEltThreads = 256;

// 8 values of a 16-bit type, as loaded in one 16-byte piece
template <int kDtype>
__device__ __forceinline__ void unpack_chunk16(const uint4 &q, float (&v)[8])
{
    const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (kDtype == KUDNN_B200_BF16) {
            v[2 * j] = __uint_as_float(w[j] << 16);
            v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
        }
    }
}

template <int kDtype>
__device__ __forceinline__ void load_chunk(const void *src, long long idx, float (&v)[8])
{
    // 8 elements starting at element idx (idx a multiple of 8, 16-byte aligned for 16-bit types, 32 for fp32)
    if (kDtype == KUDNN_B200_F32) {
        const float4 a = reinterpret_cast<const float4 *>(static_cast<const float *>(src) + idx)[0];
        const float4 b = reinterpret_cast<const float4 *>(static_cast<const float *>(src) + idx)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 q = *reinterpret_cast<const uint4 *>(static_cast<const unsigned short *>(src) + idx);
        const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (kDtype == KUDNN_B200_BF16) {
                v[2 * j] = __uint_as_float(w[j] << 16);
                v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            } else {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
                v[2 * j] = f.x;
                v[2 * j + 1] = f.y;
            }
        }
    }
}

// kTrunc: bf16 results are truncated (the activation kernels' store) instead of rounded
template <int kDtype, bool kTrunc>
__device__ __forceinline__ void store_chunk(void *dst, long long idx, const float (&v)[8])
{
    if (kDtype == KUDNN_B200_F32) {
        reinterpret_cast<float4 *>(static_cast<float *>(dst) + idx)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4 *>(static_cast<float *>(dst) + idx)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        unsigned w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (kDtype == KUDNN_B200_BF16) {
                if (kTrunc) {
                    w[j] = (__float_as_uint(v[2 * j]) >> 16) | (__float_as_uint(v[2 * j + 1]) & 0xffff0000u);
                } else {
                    w[j] = static_cast<unsigned>(f32_to_bf16_rne_bits(v[2 * j])) |
                           (static_cast<unsigned>(f32_to_bf16_rne_bits(v[2 * j + 1])) << 16);
                }
            } else {
                const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                w[j] = *reinterpret_cast<const unsigned *>(&h);
            }
        }
        *reinterpret_cast<uint4 *>(static_cast<unsigned short *>(dst) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// kAct >= 0: the activation is fixed at compile time and evaluated in line; -1: read from the argument, out of line.
// A thread has four 16-byte loads in flight before it touches the first value.
template <int kSrc, int kDst, int kAct>
__global__ void __launch_bounds__(kEltThreads) activation_kernel(const void *src, void *dst, long long count, int act,
                                                                 float alpha)
{
    // same type in and out: the reference's typed kernels (bf16 store truncates, relu first saturates near-overflow
    // values to infinity); different types: fp32 in between and one rounding to nearest
    constexpr bool kSame = kSrc == kDst;
    constexpr bool kPrecise = kSrc == KUDNN_B200_F32 || !kSame;
    constexpr int kUnroll = 4;
    const long long chunks = count / 8;
    const long long stride = static_cast<long long>(gridDim.x) * kEltThreads;
    for (long long c0 = static_cast<long long>(blockIdx.x) * kEltThreads + threadIdx.x; c0 < chunks; c0 += stride * kUnroll) {
        float v[kUnroll][8];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long long c = c0 + u * stride;
            if (c < chunks) {
                load_chunk<kSrc>(src, c * 8, v[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long long c = c0 + u * stride;
            if (c < chunks) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[u][j] = kAct < 0 ? activation_any(v[u][j], act, alpha, kPrecise ? 1 : 0)
                                       : activation<kPrecise>(v[u][j], kAct, alpha);
                    if (kSame && kDst == KUDNN_B200_BF16 && (kAct < 0 ? act : kAct) == KUDNN_B200_ACT_RELU && alpha != 0.0f) {
                        v[u][j] = relu_bf16_overflow(v[u][j]);
                    }
                }
                store_chunk<kDst, kSame>(dst, c * 8, v[u]);
            }
        }
    }
    // the last count % 8 elements
    const long long tail0 = chunks * 8;
    const long long t = tail0 + static_cast<long long>(blockIdx.x) * kEltThreads + threadIdx.x;
    if (t < count) {
        float x = load_as_f32(src, kSrc, t);
        x = activation_any(x, act, alpha, kPrecise ? 1 : 0);
        if (kSame) {
            store_exact(dst, kDst, t, round_act(x, kDst, act, alpha));
        } else {
            store_exact(dst, kDst, t, round_rne(x, kDst));
        }
    }
}

__device__ __forceinline__ float block_sum(float v, float *scratch)
{
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, off);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        scratch[warp] = v;
    }
    __syncthreads();
    float total = 0.0f;
    const int warps = static_cast<int>(blockDim.x) >> 5;
    for (int w = 0; w < warps; ++w) {  // fixed order: the result does not depend on timing
        total += scratch[w];
    }
    __syncthreads();
    return total;
}

constexpr int kRmsMaxChunks = 8;  // chunks of 8 elements a thread keeps in registers: rows up to 16384 elements

// One CTA per row.  kChunks > 0: the row is held in registers between the two passes (one read of x from memory),
// kChunks chunks of 8 elements per thread; kChunks = 0: rows longer than that are read twice.  The launcher gives
// rows of up to 8192 elements to CTAs of 128 threads, so that a thread has several 16-byte loads in flight and an SM
// holds more bytes in flight than with one chunk per thread.
template <int kDtype, int kChunks>
__global__ void __launch_bounds__(kEltThreads) rmsnorm_kernel(const void *src, void *dst, const void *scale, float *variance,
                                                              long long rows, int axis, int use_stats, int use_scale,
                                                              int save_stats, float eps)
{
    __shared__ float scratch[kEltThreads / 32];
    const int chunks = axis / 8;  // axis is a multiple of 8 on this path
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const long long base = row * axis;
        constexpr bool kResident = kChunks > 0;
        float x[kResident ? kChunks : 1][8];
        float sum = 0.0f;
        if (kResident || use_stats == 0) {
#pragma unroll
            for (int i = 0; i < kChunks; ++i) {
                const int c = threadIdx.x + i * static_cast<int>(blockDim.x);
                if (kResident) {
                    if (c < chunks) {
                        load_chunk<kDtype>(src, base + c * 8ll, x[i]);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            sum = fmaf(x[i][j], x[i][j], sum);
                        }
                    }
                }
            }
            if (!kResident) {
                for (int c = threadIdx.x; c < chunks; c += static_cast<int>(blockDim.x)) {
                    float v[8];
                    load_chunk<kDtype>(src, base + c * 8ll, v);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        sum = fmaf(v[j], v[j], sum);
                    }
                }
            }
        }
        float var;
        if (use_stats != 0) {
            var = variance[row];
        } else {
            var = block_sum(sum, scratch) / static_cast<float>(axis);
            if (save_stats != 0 && threadIdx.x == 0) {
                variance[row] = var;
            }
        }
        const float inv = 1.0f / sqrtf(var + eps);
        auto finish = [&](int c, float(&v)[8]) {
            if (use_scale != 0) {
                float s[8];
                load_chunk<kDtype>(scale, c * 8ll, s);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[j] = v[j] * (s[j] * inv);  // scale * 1/sqrt first, as the reference does
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[j] = v[j] * inv;
                }
            }
            store_chunk<kDtype, false>(dst, base + c * 8ll, v);
        };
        if (kResident) {
#pragma unroll
            for (int i = 0; i < kChunks; ++i) {
                const int c = threadIdx.x + i * static_cast<int>(blockDim.x);
                if (c < chunks) {
                    finish(c, x[i]);
                }
            }
        } else {
            for (int c = threadIdx.x; c < chunks; c += static_cast<int>(blockDim.x)) {
                float v[8];
                load_chunk<kDtype>(src, base + c * 8ll, v);
                finish(c, v);
            }
        }
    }
}

// 16-bit rows that fit in registers: like rmsnorm_kernel<kDtype, kChunks>, same arithmetic in the same order, but the row
// is kept as loaded (4 registers per chunk) and the next row of this CTA is already on its way from memory while the
// current one is reduced, scaled and stored.
template <int kDtype, int kChunks>
__global__ void __launch_bounds__(kEltThreads) rmsnorm_rows16_kernel(const void *src, void *dst, const void *scale,
                                                                     float *variance, long long rows, int axis, int use_stats,
                                                                     int use_scale, int save_stats, float eps)
{
    __shared__ float scratch[kEltThreads / 32];
    const int chunks = axis / 8;
    const unsigned short *in = static_cast<const unsigned short *>(src);
    uint4 cur[kChunks], nxt[kChunks];
    auto load_row = [&](long long row, uint4(&r)[kChunks]) {
#pragma unroll
        for (int i = 0; i < kChunks; ++i) {
            const int c = threadIdx.x + i * static_cast<int>(blockDim.x);
            if (c < chunks) {
                r[i] = *reinterpret_cast<const uint4 *>(in + row * axis + c * 8ll);
            }
        }
    };
    long long row = blockIdx.x;
    if (row < rows) {
        load_row(row, nxt);
    }
    for (; row < rows; row += gridDim.x) {
#pragma unroll
        for (int i = 0; i < kChunks; ++i) {
            cur[i] = nxt[i];
        }
        if (row + gridDim.x < rows) {
            load_row(row + gridDim.x, nxt);
        }
        const long long base = row * axis;
        float var;
        if (use_stats != 0) {
            var = variance[row];
        } else {
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < kChunks; ++i) {
                if (threadIdx.x + i * static_cast<int>(blockDim.x) < chunks) {
                    float v[8];
                    unpack_chunk16<kDtype>(cur[i], v);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        sum = fmaf(v[j], v[j], sum);
                    }
                }
            }
            var = block_sum(sum, scratch) / static_cast<float>(axis);
            if (save_stats != 0 && threadIdx.x == 0) {
                variance[row] = var;
            }
        }
        const float inv = 1.0f / sqrtf(var + eps);
#pragma unroll
        for (int i = 0; i < kChunks; ++i) {
            const int c = threadIdx.x + i * static_cast<int>(blockDim.x);
            if (c < chunks) {
                float v[8];
                unpack_chunk16<kDtype>(cur[i], v);
                if (use_scale != 0) {
                    float sc[8];
                    load_chunk<kDtype>(scale, c * 8ll, sc);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        v[j] = v[j] * (sc[j] * inv);  // scale * 1/sqrt first, as the reference does
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        v[j] = v[j] * inv;
                    }
                }
                store_chunk<kDtype, false>(dst, base + c * 8ll, v);
            }
        }
    }
}

// any axis length and alignment: one element at a time (small or odd rows)
template <int kDtype>
__global__ void __launch_bounds__(kEltThreads) rmsnorm_scalar_kernel(const void *src, void *dst, const void *scale,
                                                                     float *variance, long long rows, int axis,
                                                                     int use_stats, int use_scale, int save_stats, float eps)
{
    __shared__ float scratch[kEltThreads / 32];
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const long long base = row * axis;
        float var;
        if (use_stats != 0) {
            var = variance[row];
        } else {
            float sum = 0.0f;
            for (int i = threadIdx.x; i < axis; i += kEltThreads) {
                const float v = load_as_f32(src, kDtype, base + i);
                sum = fmaf(v, v, sum);
            }
            var = block_sum(sum, scratch) / static_cast<float>(axis);
            if (save_stats != 0 && threadIdx.x == 0) {
                variance[row] = var;
            }
        }
        const float inv = 1.0f / sqrtf(var + eps);
        for (int i = threadIdx.x; i < axis; i += kEltThreads) {
            const float c = use_scale != 0 ? load_as_f32(scale, kDtype, i) * inv : inv;
            store_exact(dst, kDtype, base + i, round_rne(load_as_f32(src, kDtype, base + i) * c, kDtype));
        }
    }
}

template <int kSrc, int kDst>
cudaError_t launch_act_typed(const void *src, void *dst, long long count, int act, float alpha, int grid, cudaStream_t stream)
{
    // the activations of the Linear path get kernels of their own when source and result share a type (the usual
    // stand-alone use); everything else takes the generic form
#define KB_ACT_CASE(A)                                                                                    \
    case A:                                                                                               \
        activation_kernel<kSrc, kDst, A><<<grid, kEltThreads, 0, stream>>>(src, dst, count, act, alpha);  \
        break
    if (kSrc == kDst) {
        switch (act) {
            KB_ACT_CASE(KUDNN_B200_ACT_RELU);
            KB_ACT_CASE(KUDNN_B200_ACT_SWISH);
            KB_ACT_CASE(KUDNN_B200_ACT_GELU_TANH);
            KB_ACT_CASE(KUDNN_B200_ACT_GELU_ERF);
            KB_ACT_CASE(KUDNN_B200_ACT_SIGMOID);
            KB_ACT_CASE(KUDNN_B200_ACT_TANH);
            default:
                activation_kernel<kSrc, kDst, -1><<<grid, kEltThreads, 0, stream>>>(src, dst, count, act, alpha);
                break;
        }
    } else {
        activation_kernel<kSrc, kDst, -1><<<grid, kEltThreads, 0, stream>>>(src, dst, count, act, alpha);
    }
#undef KB_ACT_CASE
    return cudaGetLastError();
}

template <int kSrc>
cudaError_t launch_act_dst(const void *src, void *dst, long long count, int dst_dtype, int act, float alpha, int grid,
                           cudaStream_t stream)
{
    switch (dst_dtype) {
        case KUDNN_B200_F32:
            return launch_act_typed<kSrc, KUDNN_B200_F32>(src, dst, count, act, alpha, grid, stream);
        case KUDNN_B200_F16:
            return launch_act_typed<kSrc, KUDNN_B200_F16>(src, dst, count, act, alpha, grid, stream);
        default:
            return launch_act_typed<kSrc, KUDNN_B200_BF16>(src, dst, count, act, alpha, grid, stream);
    }
}

}  // namespace

cudaError_t launch_activation(const void *src, int src_dtype, void *dst, int dst_dtype, long long count, int act, float alpha,
                              int sm_count, cudaStream_t stream)
{
    // grid: a multiple of the SM count, at most 8 CTAs of 256 threads per SM, no more CTAs than chunks
    const long long chunks = (count + 7) / 8;
    long long want = (chunks + kEltThreads - 1) / kEltThreads;
    const long long cap = static_cast<long long>(sm_count) * 8;
    const int grid = static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
    switch (src_dtype) {
        case KUDNN_B200_F32:
            return launch_act_dst<KUDNN_B200_F32>(src, dst, count, dst_dtype, act, alpha, grid, stream);
        case KUDNN_B200_F16:
            return launch_act_dst<KUDNN_B200_F16>(src, dst, count, dst_dtype, act, alpha, grid, stream);
        default:
            return launch_act_dst<KUDNN_B200_BF16>(src, dst, count, dst_dtype, act, alpha, grid, stream);
    }
}

cudaError_t launch_rmsnorm(const void *src, void *dst, const void *scale, float *variance, long long rows, long long axis,
                           int dtype, int use_stats, int use_scale, int save_stats, float eps, int sm_count,
                           cudaStream_t stream)
{
    const int threads = axis <= kRmsMaxChunks * 8 * 128 ? 128 : kEltThreads;
    const long long cap = static_cast<long long>(sm_count) * 16;
    const int grid = static_cast<int>(rows < cap ? rows : cap);
    const int ax = static_cast<int>(axis);
    const uintptr_t align = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) |
                            reinterpret_cast<uintptr_t>(use_scale != 0 ? scale : nullptr);
    const bool vec = axis % 8 == 0 && (align & (dtype == KUDNN_B200_F32 ? 31u : 15u)) == 0;
// rows held in registers: fp32 by the generic kernel, 16-bit types by the one that keeps the next row in flight
#define KB_RMS_RES(DT, N) ((DT) == KUDNN_B200_F32 ? rmsnorm_kernel<DT, N> : rmsnorm_rows16_kernel<DT, N>)
#define KB_RMS_LAUNCH(DT)                                                                                              \
    do {                                                                                                               \
        void (*kernel)(const void *, void *, const void *, float *, long long, int, int, int, int, float) =           \
            rmsnorm_kernel<DT, 0>;                                                                                     \
        int block = threads;                                                                                           \
        if (!vec) {                                                                                                    \
            kernel = rmsnorm_scalar_kernel<DT>;                                                                        \
            block = kEltThreads;                                                                                       \
        } else if (axis <= 1 * 8 * threads) {                                                                          \
            kernel = KB_RMS_RES(DT, 1);                                                                                \
        } else if (axis <= 2 * 8 * threads) {                                                                          \
            kernel = KB_RMS_RES(DT, 2);                                                                                \
        } else if (axis <= 4 * 8 * threads) {                                                                          \
            kernel = KB_RMS_RES(DT, 4);                                                                                \
        } else if (axis <= kRmsMaxChunks * 8 * threads) {                                                              \
            kernel = KB_RMS_RES(DT, kRmsMaxChunks);                                                                    \
        }                                                                                                              \
        kernel<<<grid, block, 0, stream>>>(src, dst, scale, variance, rows, ax, use_stats, use_scale, save_stats, eps); \
    } while (0)
    switch (dtype) {
        case KUDNN_B200_F32:
            KB_RMS_LAUNCH(KUDNN_B200_F32);
            break;
        case KUDNN_B200_F16:
            KB_RMS_LAUNCH(KUDNN_B200_F16);
            break;
        default:
            KB_RMS_LAUNCH(KUDNN_B200_BF16);
            break;
    }
#undef KB_RMS_LAUNCH
#undef KB_RMS_RES
    return cudaGetLastError();
}

}  // namespace kb
