// Operand packing: brings an arbitrarily strided [rows, k] operand into the K-major, 16-byte aligned form the
// tensor-core and streaming kernels read, converting the element type on the way.  fp32 operands are split
// into TF32 planes here.  The reference does the corresponding work per call and per thread inside its JIT
// GEMM (pack routines, src/dnn/src/matmul_jit/MatrixComputation/kudnn_default_impl_fp16fp16f32f32.cpp:929-962)
// and through ReorderLayer for type conversion (src/dnn/src/kudnn_gemm.cpp:36-63).
#include "kernels.cuh"

namespace kb {

namespace {

__device__ __forceinline__ void store_converted(void *dst, int dtype, long long idx, float v)
{
    if (dtype == KUDNN_B200_F32) {
        static_cast<float *>(dst)[idx] = v;
    } else if (dtype == KUDNN_B200_F16) {
        static_cast<unsigned short *>(dst)[idx] = f32_to_f16_rne_bits(v);
    } else if (dtype == KUDNN_B200_S8) {
        static_cast<signed char *>(dst)[idx] = static_cast<signed char>(static_cast<int>(v));  // 8-bit values are exact in fp32
    } else if (dtype == KUDNN_B200_U8) {
        static_cast<unsigned char *>(dst)[idx] = static_cast<unsigned char>(static_cast<int>(v));
    } else {
        static_cast<unsigned short *>(dst)[idx] = f32_to_bf16_rne_bits(v);
    }
}

// 32 x 32 tile through shared memory so both the strided read and the K-major write are coalesced
// blockIdx.z = flat batch index: the source matrix of a batch entry starts at the element offset its three batch
// strides give, the packed one at flat * dst_batch elements
__device__ __forceinline__ long long src_batch_offset(const PackBatch &pb, long long flat)
{
    const long long i2 = flat % pb.n2, r = flat / pb.n2;
    return (r / pb.n1) * pb.sb[0] + (r % pb.n1) * pb.sb[1] + i2 * pb.sb[2];
}

__global__ void __launch_bounds__(256) pack_kmajor_kernel(const void *src_base, int src_dtype, long long rows, long long k,
                                                          long long s_row, long long s_k, void *dst_base, int dst_dtype,
                                                          long long ldd, long long k_pad, const PackBatch pb)
{
    __shared__ float tile[32][33];
    const void *src = static_cast<const char *>(src_base) + src_batch_offset(pb, blockIdx.z) * dtype_size(src_dtype);
    void *dst = static_cast<char *>(dst_base) + static_cast<long long>(blockIdx.z) * pb.dst_batch * dtype_size(dst_dtype);
    const long long r0 = static_cast<long long>(blockIdx.x) * 32;
    const long long k0 = static_cast<long long>(blockIdx.y) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const bool rows_fast = (s_row == 1 && s_k != 1);
    for (int i = ty; i < 32; i += 8) {
        // rows_fast: tx walks rows (unit stride in memory), i walks k; otherwise tx walks k
        const long long r = rows_fast ? r0 + tx : r0 + i;
        const long long kk = rows_fast ? k0 + i : k0 + tx;
        float v = 0.0f;
        if (r < rows && kk < k) {
            v = load_as_f32(src, src_dtype, r * s_row + kk * s_k);
        }
        if (rows_fast) {
            tile[tx][i] = v;
        } else {
            tile[i][tx] = v;
        }
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        const long long r = r0 + i, kk = k0 + tx;
        if (r < rows && kk < k_pad) {
            store_converted(dst, dst_dtype, r * ldd + kk, tile[i][tx]);
        }
    }
}

__device__ __forceinline__ float to_tf32(float x)
{
    unsigned u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}

// dst row (pitch ldd floats) starts with three planes of k_pad floats.  Activations: [lo | hi | hi]; weights: [hi | lo | hi].
__global__ void __launch_bounds__(256) split_tf32_kernel(const float *src_base, long long rows, long long k, long long s_row,
                                                         long long s_k, float *dst_base, long long ldd, long long k_pad,
                                                         int is_weight, const PackBatch pb)
{
    __shared__ float tile[32][33];
    const float *src = src_base + src_batch_offset(pb, blockIdx.z);
    float *dst = dst_base + static_cast<long long>(blockIdx.z) * pb.dst_batch;
    const long long r0 = static_cast<long long>(blockIdx.x) * 32;
    const long long k0 = static_cast<long long>(blockIdx.y) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const bool rows_fast = (s_row == 1 && s_k != 1);
    for (int i = ty; i < 32; i += 8) {
        const long long r = rows_fast ? r0 + tx : r0 + i;
        const long long kk = rows_fast ? k0 + i : k0 + tx;
        float v = 0.0f;
        if (r < rows && kk < k) {
            v = src[r * s_row + kk * s_k];
        }
        if (rows_fast) {
            tile[tx][i] = v;
        } else {
            tile[i][tx] = v;
        }
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        const long long r = r0 + i, kk = k0 + tx;
        if (r < rows && kk < k_pad) {
            const float v = tile[i][tx];
            const float hi = to_tf32(v);
            const float lo = to_tf32(v - hi);
            float *row = dst + r * ldd;
            if (is_weight) {
                row[kk] = hi;
                row[k_pad + kk] = lo;
            } else {
                row[kk] = lo;
                row[k_pad + kk] = hi;
            }
            row[2 * k_pad + kk] = hi;
        }
    }
}

// one thread per 16-byte chunk of the destination
__global__ void __launch_bounds__(256) pack_blocks_kernel(const unsigned short *src, long long rows, long long k, long long ld,
                                                          uint4 *dst, long long nkb, long long total_chunks)
{
    const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (idx >= total_chunks) {
        return;
    }
    // position in the block -> (row, 16-byte chunk): byte (c & 1) * 512 + (4 r + c / 2) * 16 holds chunk c of row r
    const int pos = static_cast<int>(idx & 63);
    const int r = (pos & 31) >> 2, c = (pos & 3) * 2 + (pos >> 5);
    const long long blk = idx >> 6;
    const long long kb = blk % nkb, g = blk / nkb;
    const long long row = g * 8 + r, kk = kb * 64 + c * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows && kk < k) {  // k is a multiple of 8: a chunk is inside the row or outside of it
        v = *reinterpret_cast<const uint4 *>(src + row * ld + kk);
    }
    dst[idx] = v;
}

}  // namespace

cudaError_t launch_pack_blocks(const void *src, long long rows, long long k, long long ld, void *dst, long long k_pad,
                               cudaStream_t stream)
{
    const long long nkb = k_pad / 64;
    const long long total = (rows + 7) / 8 * nkb * 64;
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffll) {
        return cudaErrorInvalidValue;
    }
    pack_blocks_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const unsigned short *>(src), rows, k, ld,
                                                                          static_cast<uint4 *>(dst), nkb, total);
    return cudaGetLastError();
}

cudaError_t launch_pack_kmajor(const void *src, int src_dtype, long long rows, long long k, long long s_row,
                               long long s_k, void *dst, int dst_dtype, long long ldd, long long k_pad,
                               cudaStream_t stream, const PackBatch *batch)
{
    const PackBatch one = {1, 1, 1, {0, 0, 0}, 0};
    const PackBatch &pb = batch != nullptr ? *batch : one;
    dim3 grid(static_cast<unsigned>((rows + 31) / 32), static_cast<unsigned>((k_pad + 31) / 32), static_cast<unsigned>(pb.count));
    if (grid.y > 65535 || pb.count > 65535) {
        return cudaErrorInvalidValue;
    }
    pack_kmajor_kernel<<<grid, 256, 0, stream>>>(src, src_dtype, rows, k, s_row, s_k, dst, dst_dtype, ldd, k_pad, pb);
    return cudaGetLastError();
}

cudaError_t launch_split_tf32(const void *src, long long rows, long long k, long long s_row, long long s_k, float *dst,
                              long long ldd, long long k_pad, int is_weight, cudaStream_t stream, const PackBatch *batch)
{
    const PackBatch one = {1, 1, 1, {0, 0, 0}, 0};
    const PackBatch &pb = batch != nullptr ? *batch : one;
    dim3 grid(static_cast<unsigned>((rows + 31) / 32), static_cast<unsigned>((k_pad + 31) / 32), static_cast<unsigned>(pb.count));
    if (grid.y > 65535 || pb.count > 65535) {
        return cudaErrorInvalidValue;
    }
    split_tf32_kernel<<<grid, 256, 0, stream>>>(static_cast<const float *>(src), rows, k, s_row, s_k, dst, ldd, k_pad,
                                                is_weight, pb);
    return cudaGetLastError();
}

}  // namespace kb
