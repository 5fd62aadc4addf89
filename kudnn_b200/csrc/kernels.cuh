// Launch interface between the C-ABI dispatcher and the kernel families.
#pragma once

#include "common.cuh"

namespace kb {

// One resolved problem: device pointers, element strides, epilogue, batch.
struct LinearProblem {
    const void *a;
    const void *b;
    long long m, n, k;
    long long a_sm, a_sk, b_sk, b_sn;
    int a_dtype, b_dtype;
    // the weights once more in the decode-packed layout (see GemvParams::w_blk in gemv.cu), or null
    const void *b_blocked = nullptr;
    long long b_blocked_kpad = 0;
    EpiParams epi;
    BatchParams batch;
    long long batch_count;
};

// Scratch for the streaming kernels' cross-warp reduction (device memory owned by the handle).
struct GemvWorkspace {
    float *partials;         // slots of partial sums
    unsigned int *counters;  // one arrival counter per row (FMA kernel) or per 8-row group (MMA kernel); zero at rest
    long long partial_floats;
    long long counter_count;
};

struct GemvPlan {
    int kernel;         // KUDNN_B200_KERNEL_GEMV_FMA / _MMA
    int grid, block;    // launch shape
    int shape;          // index of the compiled (threads, CTAs per SM) variant
    int ksplit;         // K chunks (MMA kernel)
    int wide;           // MMA kernel with fragment-shaped loads: 1 = blocks of 64 k, 32 bytes per lane
    int active_warps;   // warps that take a span of the flattened work
    long long span;     // work blocks per active warp
    int slots;          // partial slots per row / row group
    size_t smem_bytes;
    long long partial_floats, counter_count;
};

// Records the calling thread's last error text and returns `code`.
int set_last_error(int code, const char *message);

cudaError_t launch_simt(const LinearProblem &pr, cudaStream_t stream);
// 8-bit integer operands (S8 / U8), 32-bit integer result and bias: exact sums
cudaError_t launch_int_gemm(const LinearProblem &pr, cudaStream_t stream);

// Streaming kernels for m <= 16 (2-D problems, K-contiguous operands).
bool gemv_plan(const LinearProblem &pr, int sm_count, int forced_kernel, GemvPlan *plan);
cudaError_t launch_gemv(const LinearProblem &pr, const GemvPlan &plan, const GemvWorkspace &ws, cudaStream_t stream);

// Tensor-core kernel.  Operands must be K-major with 16-byte aligned rows; see tc_eligible().
struct TcOperands {
    const void *a;  // [m, k_total] K-major
    const void *b;  // [n, k_total] K-major
    long long lda, ldb;   // row pitch in elements
    long long k_total;    // contraction length as laid out (3*k for the split-fp32 form)
    int kind;             // KUDNN_B200_F16 / _BF16 / _F32 (tf32 planes) / _S8 (8-bit integers, signedness below)
    int a_signed = 1, b_signed = 1;  // kind _S8 only: whether each operand holds signed values
    // batched problems: `batch` matrices per operand, a_bstride / b_bstride elements apart (0: every entry shares one)
    long long batch = 1, a_bstride = 0, b_bstride = 0;
};
struct TcPlan {
    int block_n;   // 128 or 256
    int stages;
    int grid;
    size_t smem_bytes;
    // split-K (splits > 1) for problems with far fewer tiles than SMs: the kernel is launched as clusters of
    // `splits` CTAs, grid = tiles * splits
    int splits, kb_per_split;
    int pair;      // 1: clusters of two CTAs share 256 x block_n tiles (cta_group::2)
    int narrow_from;  // pair mode: tiles from this index on are processed as two pieces of half the width
    unsigned char tmap_a[128] __attribute__((aligned(64)));
    unsigned char tmap_b[128] __attribute__((aligned(64)));
};
bool tc_available();
const char *tc_unavailable_reason();
// Tensor map (written into 128 bytes at map128) of a K-major matrix [rows, k_total] with row pitch ld_elems, for TMA
// boxes of 128 bytes of K x box_rows rows with the 128-byte swizzle; rows and columns out of range read as zero.
cudaError_t tc_encode_kmajor(void *map128, const void *base, int kind, long long rows, long long k_total, long long ld_elems,
                             int box_rows);
// with_staging: the launch writes output mirrors and needs the epilogue's row staging in shared memory
cudaError_t tc_make_plan(const TcOperands &ops, long long m, long long n, int sm_count, bool with_staging, TcPlan *plan);
// wait_limit_cycles: SM cycles after which a device-side wait gives up (0 = the default of about two seconds);
// skip_kblock: test hook for the timeout path, -1 = off (see TcParams::skip_kb).
// bp: batch strides of the epilogue tensors (ignored unless ops.batch > 1)
cudaError_t launch_tc(const TcOperands &ops, const TcPlan &plan, const EpiParams &epi, long long m, long long n,
                      DeviceStatus *status, cudaStream_t stream, long long wait_limit_cycles = 0, int skip_kblock = -1,
                      const BatchParams *bp = nullptr);

// Batched packing: `count` matrices; entry `flat` of the source starts sb[0] * i0 + sb[1] * i1 + sb[2] * i2 elements
// into the tensor, (i0, i1, i2) the decomposition of flat over the extents (.., n1, n2); entry `flat` of the packed
// copy starts flat * dst_batch elements into dst.
struct PackBatch {
    long long count, n1, n2;
    long long sb[3];
    long long dst_batch;
};

// Packing / conversion kernels.
// dst[r, kk] (row pitch ldd, K-major) = src[r*s_row + kk*s_k] converted to dst_dtype; columns [k, k_pad) are zeroed.
cudaError_t launch_pack_kmajor(const void *src, int src_dtype, long long rows, long long k, long long s_row,
                               long long s_k, void *dst, int dst_dtype, long long ldd, long long k_pad,
                               cudaStream_t stream, const PackBatch *batch = nullptr);
// 16-bit K-major rows (pitch ld elements) -> the decode-packed layout: [ceil(rows / 8)][k_pad / 64] blocks of 1 KiB
// (8 rows x 64 k, chunk order as described at GemvParams::w_blk), zero padded.
cudaError_t launch_pack_blocks(const void *src, long long rows, long long k, long long ld, void *dst, long long k_pad,
                               cudaStream_t stream);
// fp32 -> three K-major TF32 planes side by side at the start of each dst row (row pitch ldd floats).  With
// hi = tf32(x) and lo = tf32(x - hi), activations are laid out [lo | hi | hi] and weights [hi | lo | hi], so that one
// contraction over the 3 * k_pad columns yields a_lo.b_hi + a_hi.b_lo + a_hi.b_hi.
cudaError_t launch_split_tf32(const void *src, long long rows, long long k, long long s_row, long long s_k, float *dst,
                              long long ldd, long long k_pad, int is_weight, cudaStream_t stream,
                              const PackBatch *batch = nullptr);

// Stand-alone element-wise activation and RMS normalisation (eltwise.cu); device pointers.
cudaError_t launch_activation(const void *src, int src_dtype, void *dst, int dst_dtype, long long count, int act, float alpha,
                              int sm_count, cudaStream_t stream);
cudaError_t launch_rmsnorm(const void *src, void *dst, const void *scale, float *variance, long long rows, long long axis,
                           int dtype, int use_stats, int use_scale, int save_stats, float eps, int sm_count,
                           cudaStream_t stream);

}  // namespace kb
