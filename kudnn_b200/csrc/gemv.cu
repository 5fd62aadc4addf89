// Streaming kernels for decode-shaped Linear (m <= 16): the weight matrix is read from HBM exactly once,
// everything else stays on chip.  The reference reaches this shape through cblas_sgemv / cblas_bgemm
// (src/dnn/src/kudnn_gemm.cpp:165-176, :222-226).
//
// Work decomposition (both kernels).  The weight matrix [n, k], K-contiguous, is cut into "blocks" of one
// 16-byte load per lane.  All blocks are numbered row-major (unit by unit, k ascending inside a unit; a unit is a
// weight row for the FMA kernel and a group of 8 weight rows for the MMA kernel) and the numbering is split into
// equal contiguous spans, one per active warp, so every warp streams the same number of bytes no matter how n
// relates to the SM count.  A warp whose span covers a unit completely finishes that unit on its own; a unit cut
// by a span boundary is a split-K case: each warp involved stores its partial sums into its slot of the scratch
// buffer, bumps the unit's arrival counter, and the warp that arrives last adds the slots in slot order (so the
// result does not depend on timing) and runs the fused epilogue.  Counters return to zero before the kernel ends.
//
//   FMA kernel  m <= 4, fp32 / fp16 / bf16.  Lane l of a warp owns k = 8l..8l+7 (16-bit) of every block of a row,
//               accumulates with fp32 FMA against the activations held in shared memory as fp32, and a
//               warp-shuffle tree folds the 32 lanes when the row (or the span) ends.
//   MMA kernel  m <= 16, fp16 / bf16.  A block is 8 rows x 32 k; the 16 bytes a lane loads feed two
//               mma.sync.m16n8k16 (activations as the 16-row operand, zero padded), fp32 accumulators.  The
//               contraction index inside a block is permuted identically for both operands so a lane's 16 bytes
//               are consecutive in memory.  K is additionally cut into `ksplit` chunks across CTAs so the
//               activation chunk fits shared memory.
#include "kernels.cuh"

#include <algorithm>
#include <cstdlib>

namespace kb {

namespace {

constexpr int kMmaRowPadBytes = 64;  // keeps the 8 quarter-warp rows of an A-fragment load on distinct banks

struct GemvParams {
    const void *x;   // [m, k], K-contiguous, row pitch x_ld elements
    const void *w;   // [n, k], K-contiguous, row pitch w_ld elements
    long long x_ld, w_ld;
    int m, n, k;
    int kb;            // blocks per unit (per chunk for the MMA kernel)
    int kc;            // chunk length in k (MMA kernel), multiple of 32
    int ksplit;
    int active_warps;  // per chunk
    long long span;
    long long total;   // blocks per chunk
    int slots;         // slots per unit per chunk
    float *partials;
    unsigned int *counters;
    // Decode-packed weights, when the handle holds them: groups of 8 rows, each cut into blocks of 64 k; a block is
    // 1 KiB of contiguous memory, zero padded to 8 rows and to blk_kb * 64 columns.  Inside a block the 16-byte chunk
    // c (k = 8c .. 8c+7) of row r sits at byte (c & 1) * 512 + (4 r + c / 2) * 16: lane 4 r + t of a warp finds the
    // two chunks 2t and 2t+1 it feeds to the tensor cores at the same place in the two halves, so every load
    // instruction of a warp reads 512 consecutive bytes instead of 8 pieces that lie a weight row apart, which HBM
    // serves a few percent faster.  The MMA kernels read this copy; the FMA kernel reads the plain K-major rows.
    const unsigned short *w_blk;
    int blk_kb;  // 64-k blocks per group
    int w8;      // MMA kernel: the weights are 8-bit integers (1 = signed, 2 = unsigned), the activations fp16
    EpiParams epi;
};

__device__ __forceinline__ uint4 ld_stream_16(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int kDtype>
__device__ __forceinline__ void unpack2(unsigned w, float &lo, float &hi)
{
    if (kDtype == KUDNN_B200_BF16) {
        lo = __uint_as_float(w << 16);
        hi = __uint_as_float(w & 0xffff0000u);
    } else {
        __half2 h = *reinterpret_cast<__half2 *>(&w);
        float2 f = __half22float2(h);
        lo = f.x;
        hi = f.y;
    }
}

// Four 8-bit integers of a word as floats: each byte is dropped into the mantissa of 2^23 (the sum is exact), signed
// bytes after a flip of their top bit, and the offset is subtracted again.
template <bool kSigned>
__device__ __forceinline__ void unpack4_i8(unsigned w, float *f)
{
    if (kSigned) {
        w ^= 0x80808080u;  // byte + 128 as an unsigned byte
    }
    const float offset = kSigned ? 8388608.0f + 128.0f : 8388608.0f;
    f[0] = __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7650)) - offset;
    f[1] = __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7651)) - offset;
    f[2] = __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7652)) - offset;
    f[3] = __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7653)) - offset;
}

// Two pairs of 8-bit integers of a word as two half2 words (k order kept): each byte is dropped into the mantissa of
// 1024 (exact), signed bytes after a flip of their top bit, and the offset is subtracted again in fp16 (exact).
template <bool kSigned>
__device__ __forceinline__ void unpack4_i8_h2(unsigned w, unsigned &lo, unsigned &hi)
{
    if (kSigned) {
        w ^= 0x80808080u;
    }
    const unsigned off = kSigned ? 0x64806480u : 0x64006400u;  // 1024 + 128, or 1024, twice
    const unsigned a = __byte_perm(w, 0x64646464u, 0x5140);     // bytes 0 and 1
    const unsigned b = __byte_perm(w, 0x64646464u, 0x5342);     // bytes 2 and 3
    const __half2 ha = __hsub2(*reinterpret_cast<const __half2 *>(&a), *reinterpret_cast<const __half2 *>(&off));
    const __half2 hb = __hsub2(*reinterpret_cast<const __half2 *>(&b), *reinterpret_cast<const __half2 *>(&off));
    lo = *reinterpret_cast<const unsigned *>(&ha);
    hi = *reinterpret_cast<const unsigned *>(&hb);
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, off);
    }
    return v;
}

// ------------------------------------------------------------------------------------------------ FMA kernel

// kDtype KUDNN_B200_S8 / _U8: 8-bit weights streamed as they are (16 per load, half the bytes of their fp16 form) and
// widened in registers, against fp16 activations.
template <int kDtype, int kM, int kUnroll, int kThreads, int kMinBlocks>
__global__ void __launch_bounds__(kThreads, kMinBlocks) gemv_fma_kernel(const GemvParams p)
{
    constexpr bool kInt8 = kDtype == KUDNN_B200_S8 || kDtype == KUDNN_B200_U8;
    constexpr int kXDtype = kInt8 ? KUDNN_B200_F16 : kDtype;  // type of the activations
    constexpr int kVec = (kDtype == KUDNN_B200_F32) ? 4 : (kInt8 ? 16 : 8);  // elements per 16-byte load
    constexpr int kBlockK = 32 * kVec;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *xs = reinterpret_cast<float *>(smem_raw);  // [kM][kpad]
    const int kpad = p.kb * kBlockK;

    for (int i = threadIdx.x; i < kM * kpad; i += kThreads) {
        const int mi = i / kpad, kk = i - mi * kpad;
        float v = 0.0f;
        if (kk < p.k) {
            v = load_as_f32(p.x, kXDtype, static_cast<long long>(mi) * p.x_ld + kk);
        }
        if (kInt8) {
            // a lane's 16 activations of a k-block are four float4 reads; the q-th reads of the 32 lanes lie side by
            // side (element lane * 16 + q * 4 + j of the block sits at (q * 32 + lane) * 4 + j): no bank conflicts
            const int blk = kk / kBlockK, r = kk - blk * kBlockK;
            const int ln = r / 16, q = (r % 16) / 4, j = r % 4;
            xs[mi * kpad + blk * kBlockK + (q * 32 + ln) * 4 + j] = v;
        } else {
            xs[i] = v;
        }
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int warp = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (warp >= p.active_warps) {
        return;
    }
    long long f = static_cast<long long>(warp) * p.span;
    const long long f_end = (f + p.span < p.total) ? f + p.span : p.total;
    const char *wbase = static_cast<const char *>(p.w);
    const int esize = (kDtype == KUDNN_B200_F32) ? 4 : (kInt8 ? 1 : 2);

    while (f < f_end) {
        const long long row = f / p.kb;
        const int kb0 = static_cast<int>(f - row * p.kb);
        const int nb = static_cast<int>(((p.kb - kb0) < (f_end - f)) ? (p.kb - kb0) : (f_end - f));
        const char *wrow = wbase + (row * p.w_ld + static_cast<long long>(lane) * kVec) * esize;

        float acc[kM];
#pragma unroll
        for (int mi = 0; mi < kM; ++mi) {
            acc[mi] = 0.0f;
        }
        for (int i = 0; i < nb; i += kUnroll) {
            uint4 wv[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int kk = (kb0 + i + u) * kBlockK + lane * kVec;
                wv[u] = make_uint4(0u, 0u, 0u, 0u);
                if (i + u < nb && kk < p.k) {
                    wv[u] = ld_stream_16(wrow + static_cast<long long>(kb0 + i + u) * kBlockK * esize);
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                if (i + u < nb) {
                    const int kk = (kb0 + i + u) * kBlockK + lane * kVec;
                    if (kInt8) {
                        // four weights at a time, so that only four widened values are alive
                        const unsigned words[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
                        const float4 *xb = reinterpret_cast<const float4 *>(xs + (kb0 + i + u) * kBlockK) + lane;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            float wq[4];
                            unpack4_i8<kDtype == KUDNN_B200_S8>(words[q], wq);
#pragma unroll
                            for (int mi = 0; mi < kM; ++mi) {
                                const float4 xv = xb[mi * (kpad / 4) + q * 32];
                                acc[mi] = fmaf(wq[0], xv.x, acc[mi]);
                                acc[mi] = fmaf(wq[1], xv.y, acc[mi]);
                                acc[mi] = fmaf(wq[2], xv.z, acc[mi]);
                                acc[mi] = fmaf(wq[3], xv.w, acc[mi]);
                            }
                        }
                        continue;
                    }
                    float wf[kVec];
                    if (kDtype == KUDNN_B200_F32) {
                        wf[0] = __uint_as_float(wv[u].x);
                        wf[1] = __uint_as_float(wv[u].y);
                        wf[2] = __uint_as_float(wv[u].z);
                        wf[3] = __uint_as_float(wv[u].w);
                    } else {
                        unpack2<kDtype>(wv[u].x, wf[0], wf[1]);
                        unpack2<kDtype>(wv[u].y, wf[2], wf[3]);
                        unpack2<kDtype>(wv[u].z, wf[4 % kVec], wf[5 % kVec]);
                        unpack2<kDtype>(wv[u].w, wf[6 % kVec], wf[7 % kVec]);
                    }
#pragma unroll
                    for (int mi = 0; mi < kM; ++mi) {
                        const float4 *xp = reinterpret_cast<const float4 *>(xs + mi * kpad + kk);
#pragma unroll
                        for (int q = 0; q < kVec / 4; ++q) {
                            const float4 xv = xp[q];
                            acc[mi] = fmaf(wf[q * 4 + 0], xv.x, acc[mi]);
                            acc[mi] = fmaf(wf[q * 4 + 1], xv.y, acc[mi]);
                            acc[mi] = fmaf(wf[q * 4 + 2], xv.z, acc[mi]);
                            acc[mi] = fmaf(wf[q * 4 + 3], xv.w, acc[mi]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int mi = 0; mi < kM; ++mi) {
            acc[mi] = warp_sum(acc[mi]);
        }

        const bool whole = (kb0 == 0) && (nb == p.kb);
        if (whole) {
            if (lane < kM) {
                float v = acc[0];
#pragma unroll
                for (int mi = 1; mi < kM; ++mi) {
                    v = (lane == mi) ? acc[mi] : v;
                }
                epilogue_scalar(p.epi, v, lane, row);
            }
        } else {
            // split row: slot = position of this warp among the warps that touch the row
            const long long first_blk = row * p.kb;
            const int w0 = static_cast<int>(first_blk / p.span);
            const int w1 = static_cast<int>((first_blk + p.kb - 1) / p.span);
            const int pieces = w1 - w0 + 1;
            const int slot = warp - w0;
            float *mine = p.partials + (row * p.slots + slot) * kM;
            if (lane == 0) {
#pragma unroll
                for (int mi = 0; mi < kM; ++mi) {
                    mine[mi] = acc[mi];
                }
                __threadfence();
                const unsigned old = atomicAdd(p.counters + row, 1u);
                if (old == static_cast<unsigned>(pieces - 1)) {
                    __threadfence();
                    const float *all = p.partials + row * p.slots * kM;
#pragma unroll
                    for (int mi = 0; mi < kM; ++mi) {
                        float s = 0.0f;
                        for (int j = 0; j < pieces; ++j) {
                            s += __ldcg(all + j * kM + mi);
                        }
                        epilogue_scalar(p.epi, s, mi, row);
                    }
                    p.counters[row] = 0u;
                }
            }
            __syncwarp();
        }
        f += nb;
    }
}

// ------------------------------------------------------------------------------------------------ MMA kernel

template <int kDtype>
__device__ __forceinline__ void mma_16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                          unsigned b0, unsigned b1)
{
    if (kDtype == KUDNN_B200_BF16) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// Ends a warp's work on one group of 8 weight rows.  The lane holds y[gid][n0 + 2*tig + {0,1}] in acc[0..1] and
// y[gid + 8][...] in acc[2..3].  A group that one warp covered alone goes straight to the epilogue; otherwise the
// partial tile goes to the warp's slot and the last arrival adds all slots in slot order.
__device__ __forceinline__ void mma_finish_group(const GemvParams &p, float (&acc)[4], long long group, int chunk, int warp,
                                                 int lane)
{
    const int gid = lane >> 2, tig = lane & 3;
    const long long n0 = group * 8 + tig * 2;
    const long long first_blk = group * p.kb;
    const int w0 = static_cast<int>(first_blk / p.span);
    const int w1 = static_cast<int>((first_blk + p.kb - 1) / p.span);
    const int pieces = w1 - w0 + 1;
    const bool whole = (p.ksplit == 1) && (pieces == 1);
    bool finish = whole;
    if (!whole) {
        const int slot = chunk * p.slots + (warp - w0);
        float *unit = p.partials + group * (static_cast<long long>(p.ksplit) * p.slots * 128);
        *reinterpret_cast<float4 *>(unit + slot * 128 + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        __threadfence();
        __syncwarp();
        unsigned old = 0u;
        if (lane == 0) {
            old = atomicAdd(p.counters + group, 1u);
        }
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == static_cast<unsigned>(p.ksplit * pieces - 1)) {
            __threadfence();
            float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int c = 0; c < p.ksplit; ++c) {
                for (int j = 0; j < pieces; ++j) {
                    const float4 v = __ldcg(reinterpret_cast<const float4 *>(unit + (c * p.slots + j) * 128 + lane * 4));
                    s[0] += v.x;
                    s[1] += v.y;
                    s[2] += v.z;
                    s[3] += v.w;
                }
            }
            acc[0] = s[0];
            acc[1] = s[1];
            acc[2] = s[2];
            acc[3] = s[3];
            finish = true;
            if (lane == 0) {
                p.counters[group] = 0u;
            }
        }
    }
    if (finish) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int mi = gid + ((e >= 2) ? 8 : 0);
            const long long ni = n0 + (e & 1);
            if (mi < p.m && ni < p.n) {
                epilogue_scalar(p.epi, acc[e], mi, ni);
            }
        }
    }
}

// kRows16: activations occupy both 8-row halves of the 16-row operand (m > 8).
// kWide: a block is 8 rows x 64 k and a lane loads 32 consecutive bytes of its row (two 16-byte loads), feeding four
// MMAs; a warp instruction then touches 8 rows x 128 bytes instead of 8 x 64, which HBM serves about 5 % faster.
// kW8 (1 signed, 2 unsigned; with kWide and fp16): the weights are 8-bit integers read as they are, 16 bytes = 16 values
// of a row per lane and block, and widened to fp16 in registers; the activations are laid out as for kWide.
template <int kDtype, bool kRows16, bool kWide, int kUnroll, int kThreads, int kMinBlocks, int kW8 = 0>
__global__ void __launch_bounds__(kThreads, kMinBlocks) gemv_mma_kernel(const GemvParams p)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kRows = kRows16 ? 16 : 8;
    constexpr int kBlockK = kWide ? 64 : 32;
    constexpr int kLaneBytes = kWide ? 32 : 16;
    // row pitch of the activations in shared memory: the skew keeps the 8 lanes of a 16-byte load phase on distinct banks
    const int row_bytes = p.kc * 2 + (kWide ? 16 : kMmaRowPadBytes);
    const int chunk = blockIdx.x % p.ksplit;
    const int cta_in_chunk = blockIdx.x / p.ksplit;
    const int kc0 = chunk * p.kc;

    // activations of this chunk -> shared memory (16-bit, zero padded in m and k)
    {
        const int vec_per_row = p.kc / 8;
        const unsigned short *xg = static_cast<const unsigned short *>(p.x);
        for (int i = threadIdx.x; i < kRows * vec_per_row; i += kThreads) {
            const int mi = i / vec_per_row, v = i - mi * vec_per_row;
            const int kk = kc0 + v * 8;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (mi < p.m && kk < p.k) {
                val = *reinterpret_cast<const uint4 *>(xg + static_cast<long long>(mi) * p.x_ld + kk);
            }
            *reinterpret_cast<uint4 *>(smem_raw + mi * row_bytes + v * 16) = val;
        }
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int warp = cta_in_chunk * (kThreads / 32) + (threadIdx.x >> 5);
    if (warp >= p.active_warps) {
        return;
    }
    long long f = static_cast<long long>(warp) * p.span;
    const long long f_end = (f + p.span < p.total) ? f + p.span : p.total;
    const unsigned short *wg = static_cast<const unsigned short *>(p.w);
    const unsigned char *xa_row = smem_raw + gid * row_bytes + tig * kLaneBytes;
    const unsigned char *xb_row = smem_raw + (gid + 8) * row_bytes + tig * kLaneBytes;

    while (f < f_end) {
        const long long group = f / p.kb;
        const int kb0 = static_cast<int>(f - group * p.kb);
        const int nb = static_cast<int>(((p.kb - kb0) < (f_end - f)) ? (p.kb - kb0) : (f_end - f));
        const long long wrow_idx = group * 8 + gid;
        const bool row_ok = wrow_idx < p.n;
        const unsigned short *wrow = wg + wrow_idx * p.w_ld + kc0 + tig * (kLaneBytes / 2);
        const unsigned char *wrow8 = static_cast<const unsigned char *>(p.w) + wrow_idx * p.w_ld + kc0 + tig * 16;

        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int i = 0; i < nb; i += kUnroll) {
            uint4 wv[kUnroll][kWide ? 2 : 1];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int kloc = (kb0 + i + u) * kBlockK;
#pragma unroll
                for (int h = 0; h < (kWide ? 2 : 1); ++h) {
                    wv[u][h] = make_uint4(0u, 0u, 0u, 0u);
                    if (kW8 != 0) {
                        if (h == 0 && i + u < nb && row_ok && (kc0 + kloc + tig * 16) < p.k) {
                            wv[u][0] = ld_stream_16(wrow8 + kloc);
                        }
                    } else if (p.w_blk != nullptr) {
                        const int k_abs = kc0 + kloc + tig * (kLaneBytes / 2) + h * 8;
                        if (i + u < nb && (k_abs >> 6) < p.blk_kb) {
                            const int c = (k_abs & 63) >> 3;
                            wv[u][h] = ld_stream_16(p.w_blk + (group * p.blk_kb + (k_abs >> 6)) * 512 + (c & 1) * 256 +
                                                    (gid * 4 + (c >> 1)) * 8);
                        }
                    } else if (i + u < nb && row_ok && (kc0 + kloc + tig * (kLaneBytes / 2) + h * 8) < p.k) {
                        wv[u][h] = ld_stream_16(wrow + kloc + h * 8);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                if (i + u < nb) {
                    const int kloc = (kb0 + i + u) * kBlockK;
#pragma unroll
                    for (int h = 0; h < (kWide ? 2 : 1); ++h) {
                        const uint4 xa = *reinterpret_cast<const uint4 *>(xa_row + kloc * 2 + h * 16);
                        uint4 xb = make_uint4(0u, 0u, 0u, 0u);
                        if (kRows16) {
                            xb = *reinterpret_cast<const uint4 *>(xb_row + kloc * 2 + h * 16);
                        }
                        if (kW8 != 0) {
                            // values 8h .. 8h + 7 of the lane's 16: two words of the one load
                            unsigned c0, c1, c2, c3;
                            unpack4_i8_h2<kW8 == 1>(h == 0 ? wv[u][0].x : wv[u][0].z, c0, c1);
                            unpack4_i8_h2<kW8 == 1>(h == 0 ? wv[u][0].y : wv[u][0].w, c2, c3);
                            mma_16816<kDtype>(acc, xa.x, xb.x, xa.y, xb.y, c0, c1);
                            mma_16816<kDtype>(acc, xa.z, xb.z, xa.w, xb.w, c2, c3);
                        } else {
                            mma_16816<kDtype>(acc, xa.x, xb.x, xa.y, xb.y, wv[u][h].x, wv[u][h].y);
                            mma_16816<kDtype>(acc, xa.z, xb.z, xa.w, xb.w, wv[u][h].z, wv[u][h].w);
                        }
                    }
                }
            }
        }

        mma_finish_group(p, acc, group, chunk, warp, lane);
        f += nb;
    }
}

// ------------------------------------------------------------------------------- MMA kernel, staged weight feed
//
// Same arithmetic and the same work decomposition as gemv_mma_kernel, with a block of 8 rows x 256 k.  What changes is
// how the weights reach the fragment layout.  HBM delivers about 12 % more for loads in which a warp reads 512
// consecutive bytes of one row than for the 8 rows x 64 bytes a fragment-shaped load touches, so here every load
// instruction reads one row segment; the 8 segments of a block go through 4 KiB of shared memory that belongs to
// the warp alone (no CTA-wide barrier anywhere in the loop) and come back in fragment layout through ldmatrix.  The
// loads of the next block are issued before the current one is staged, so a warp always has 4 KiB in flight.
// ldmatrix hands thread (gid, tig) of matrix j the elements k = 8j + 2*tig, +1 of row gid; the activations are
// stored in shared memory with the words of every 32-k block transposed 4 x 4 so that the four words a thread needs
// for the two MMAs of that block are one 16-byte load.
constexpr int kStagedThreads = 512;
constexpr int kStagedBlockK = 256;
constexpr int kStagedPitch = kStagedBlockK * 2 + 16;  // bytes per staged row; the skew spreads the 8 rows over the banks
constexpr int kStagedWarpBytes = 8 * kStagedPitch;

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

template <int kDtype, bool kRows16>
__global__ void __launch_bounds__(kStagedThreads, 1) gemv_mma_staged_kernel(const GemvParams p)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kRows = kRows16 ? 16 : 8;
    const int row_bytes = p.kc * 2 + kMmaRowPadBytes;
    const int chunk = blockIdx.x % p.ksplit;
    const int cta_in_chunk = blockIdx.x / p.ksplit;
    const int kc0 = chunk * p.kc;

    const int lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int warp_in_cta = threadIdx.x >> 5;
    const int warp = cta_in_chunk * (kStagedThreads / 32) + warp_in_cta;
    const bool active = warp < p.active_warps;
    long long f = static_cast<long long>(warp) * p.span;
    const long long f_end = (f + p.span < p.total) ? f + p.span : p.total;
    const unsigned short *wg = static_cast<const unsigned short *>(p.w);
    const int k_end = (kc0 + p.kc < p.k) ? kc0 + p.kc : p.k;

    // rows [row0, row0 + rows_ok) of the weights, block blk of this chunk: one 512-byte row segment per instruction
    auto load_block = [&](uint4 (&v)[8], long long row0, int rows_ok, int blk) {
        const int kloc = blk * kStagedBlockK;
        if (p.w_blk != nullptr) {
            // the block is 4 KiB of contiguous memory (four 64-k blocks of this group): instruction i reads bytes
            // [512 i, 512 i + 512), i.e. 64-k block i / 2, row lane / 4, 16-byte chunk 2 (lane % 4) + i % 2
            const int kb64 = (kc0 + kloc) >> 6;
            const unsigned short *src = p.w_blk + ((row0 >> 3) * p.blk_kb + kb64) * 512 + lane * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = make_uint4(0u, 0u, 0u, 0u);
                if (kb64 + (i >> 1) < p.blk_kb) {
                    v[i] = ld_stream_16(src + i * 256);
                }
            }
            return;
        }
        const bool k_ok = kc0 + kloc + lane * 8 < k_end;
        const unsigned short *src = wg + row0 * p.w_ld + kc0 + kloc + lane * 8;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            v[r] = make_uint4(0u, 0u, 0u, 0u);
            if (k_ok && r < rows_ok) {
                v[r] = ld_stream_16(src + r * p.w_ld);
            }
        }
    };
    auto rows_of = [&](long long group) {
        const long long left = p.n - group * 8;
        return left >= 8 ? 8 : static_cast<int>(left);
    };

    // the first weight block is requested before anything else, so HBM is already busy while the activations load
    uint4 va[8], vb[8];
    if (active && f < f_end) {
        const long long group = f / p.kb;
        load_block(va, group * 8, rows_of(group), static_cast<int>(f - group * p.kb));
    }

    // Activations of this chunk -> shared memory.  Every thread issues eight 16-byte loads before it stores anything
    // (one round trip to L2 per eight vectors).  The 16 words of a 32-k block are stored transposed 4 x 4: vector q
    // of a block supplies word q of each of the block's four 16-byte groups.  Which group a lane writes first is
    // rotated with the block index, which keeps the 32 lanes of a store on distinct banks.
    {
        const int vec_per_row = p.kc / 8;
        const int total_vec = kRows * vec_per_row;
        const unsigned short *xg = static_cast<const unsigned short *>(p.x);
        for (int base = threadIdx.x; base < total_vec; base += kStagedThreads * 8) {
            uint4 xv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * kStagedThreads;
                xv[u] = make_uint4(0u, 0u, 0u, 0u);
                if (i < total_vec) {
                    const int mi = i / vec_per_row, vi = i - mi * vec_per_row;
                    const int kk = kc0 + vi * 8;
                    if (mi < p.m && kk < p.k) {
                        xv[u] = *reinterpret_cast<const uint4 *>(xg + static_cast<long long>(mi) * p.x_ld + kk);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * kStagedThreads;
                if (i < total_vec) {
                    const int mi = i / vec_per_row, vi = i - mi * vec_per_row;
                    const int blk = vi >> 2, q = vi & 3;
                    const int rot = (blk >> 1) & 3;
                    // c[t] = component (t + rot) & 3 of the vector
                    unsigned c0 = xv[u].x, c1 = xv[u].y, c2 = xv[u].z, c3 = xv[u].w;
                    if (rot & 1) {
                        const unsigned tmp = c0;
                        c0 = c1;
                        c1 = c2;
                        c2 = c3;
                        c3 = tmp;
                    }
                    if (rot & 2) {
                        unsigned tmp = c0;
                        c0 = c2;
                        c2 = tmp;
                        tmp = c1;
                        c1 = c3;
                        c3 = tmp;
                    }
                    unsigned *dst = reinterpret_cast<unsigned *>(smem_raw + mi * row_bytes) + (blk << 4) + q;
                    dst[((0 + rot) & 3) << 2] = c0;
                    dst[((1 + rot) & 3) << 2] = c1;
                    dst[((2 + rot) & 3) << 2] = c2;
                    dst[((3 + rot) & 3) << 2] = c3;
                }
            }
        }
    }
    __syncthreads();
    if (!active) {
        return;
    }

    const unsigned char *xa_row = smem_raw + gid * row_bytes + tig * 16;
    const unsigned char *xb_row = smem_raw + (gid + 8) * row_bytes + tig * 16;
    unsigned char *stage = smem_raw + kRows * row_bytes + warp_in_cta * kStagedWarpBytes;
    const uint32_t stage_st = static_cast<uint32_t>(__cvta_generic_to_shared(stage)) + static_cast<uint32_t>(lane * 16);
    // decode-packed weights: where register i of load_block goes in the staged [8 rows][256 k] block
    const uint32_t stage_st_blk = static_cast<uint32_t>(__cvta_generic_to_shared(stage)) +
                                  static_cast<uint32_t>((lane >> 2) * kStagedPitch + (lane & 3) * 32);
    const uint32_t stage_ld = static_cast<uint32_t>(__cvta_generic_to_shared(stage)) +
                              static_cast<uint32_t>((lane & 7) * kStagedPitch + (lane >> 3) * 16);
    bool preloaded = true;

    while (f < f_end) {
        const long long group = f / p.kb;
        const int kb0 = static_cast<int>(f - group * p.kb);
        const int nb = static_cast<int>(((p.kb - kb0) < (f_end - f)) ? (p.kb - kb0) : (f_end - f));
        const long long row0 = group * 8;
        const int rows_ok = rows_of(group);

        float acc0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, acc1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        auto consume_block = [&](const uint4 (&v)[8], int blk) {
            __syncwarp();  // the ldmatrix reads of the previous block are done
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const uint32_t dst = (p.w_blk != nullptr) ? stage_st_blk + (r & 1) * 16 + (r >> 1) * 128
                                                          : stage_st + r * kStagedPitch;
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[r].x), "r"(v[r].y), "r"(v[r].z),
                             "r"(v[r].w)
                             : "memory");
            }
            __syncwarp();
            const int xoff = blk * kStagedBlockK * 2;
#pragma unroll
            for (int s = 0; s < kStagedBlockK / 32; ++s) {
                unsigned b0, b1, b2, b3;
                ldmatrix_x4(stage_ld + s * 64, b0, b1, b2, b3);
                const uint4 xa = *reinterpret_cast<const uint4 *>(xa_row + xoff + s * 64);
                uint4 xb = make_uint4(0u, 0u, 0u, 0u);
                if (kRows16) {
                    xb = *reinterpret_cast<const uint4 *>(xb_row + xoff + s * 64);
                }
                mma_16816<kDtype>(acc0, xa.x, xb.x, xa.y, xb.y, b0, b1);
                mma_16816<kDtype>(acc1, xa.z, xb.z, xa.w, xb.w, b2, b3);
            }
        };

        if (!preloaded) {
            load_block(va, row0, rows_ok, kb0);
        }
        preloaded = false;
        for (int i = 0; i < nb; i += 2) {
            if (i + 1 < nb) {
                load_block(vb, row0, rows_ok, kb0 + i + 1);
            }
            consume_block(va, kb0 + i);
            if (i + 1 < nb) {
                if (i + 2 < nb) {
                    load_block(va, row0, rows_ok, kb0 + i + 2);
                }
                consume_block(vb, kb0 + i + 1);
            }
        }
        float acc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            acc[e] = acc0[e] + acc1[e];
        }
        mma_finish_group(p, acc, group, chunk, warp, lane);
        f += nb;
    }
}

int env_int(const char *name, int fallback)
{
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') {
        return fallback;
    }
    return std::atoi(v);
}

template <typename K>
cudaError_t set_smem(K kernel, size_t bytes)
{
    if (bytes > 48 * 1024) {
        return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    }
    return cudaSuccess;
}

template <int kDtype, int kUnroll, int kThreads, int kMinBlocks>
cudaError_t launch_fma_m(const GemvParams &p, const GemvPlan &plan, cudaStream_t stream)
{
#define KB_FMA_CASE(M)                                                                                            \
    case M: {                                                                                                     \
        auto kernel = gemv_fma_kernel<kDtype, M, kUnroll, kThreads, kMinBlocks>;                                  \
        cudaError_t e = set_smem(kernel, plan.smem_bytes);                                                        \
        if (e != cudaSuccess) return e;                                                                           \
        kernel<<<plan.grid, plan.block, plan.smem_bytes, stream>>>(p);                                            \
        break;                                                                                                    \
    }
    if constexpr (kDtype == KUDNN_B200_S8 || kDtype == KUDNN_B200_U8) {
        // 8-bit weights take this kernel for a single activation row only
        switch (p.m) {
            KB_FMA_CASE(1)
            default:
                return cudaErrorInvalidValue;
        }
    } else {
        switch (p.m) {
            KB_FMA_CASE(1)
            KB_FMA_CASE(2)
            KB_FMA_CASE(3)
            KB_FMA_CASE(4)
            default:
                return cudaErrorInvalidValue;
        }
    }
#undef KB_FMA_CASE
    return cudaGetLastError();
}

template <int kDtype, int kUnroll, int kThreads, int kMinBlocks>
cudaError_t launch_mma_rows(const GemvParams &p, const GemvPlan &plan, cudaStream_t stream)
{
    if (p.w8 != 0) {
        if constexpr (kDtype == KUDNN_B200_F16) {
#define KB_W8_CASE(ROWS16, SIGN)                                                                                   \
    {                                                                                                              \
        auto kernel = gemv_mma_kernel<kDtype, ROWS16, true, kUnroll, kThreads, kMinBlocks, SIGN>;                    \
        cudaError_t e = set_smem(kernel, plan.smem_bytes);                                                         \
        if (e != cudaSuccess) return e;                                                                            \
        kernel<<<plan.grid, plan.block, plan.smem_bytes, stream>>>(p);                                             \
    }
            if (p.m > 8) {
                if (p.w8 == 1) KB_W8_CASE(true, 1) else KB_W8_CASE(true, 2)
            } else {
                if (p.w8 == 1) KB_W8_CASE(false, 1) else KB_W8_CASE(false, 2)
            }
#undef KB_W8_CASE
            return cudaGetLastError();
        } else {
            return cudaErrorInvalidValue;
        }
    }
    if (p.m > 8 && plan.wide != 0) {
        // three blocks (96 bytes per lane) in flight: 91.0 us against 91.7 us with two and 98.3 us with four (spills)
        auto kernel = gemv_mma_kernel<kDtype, true, true, (kUnroll > 2 ? kUnroll * 3 / 4 : 1), kThreads, kMinBlocks>;
        cudaError_t e = set_smem(kernel, plan.smem_bytes);
        if (e != cudaSuccess) return e;
        kernel<<<plan.grid, plan.block, plan.smem_bytes, stream>>>(p);
    } else if (p.m > 8) {
        auto kernel = gemv_mma_kernel<kDtype, true, false, kUnroll, kThreads, kMinBlocks>;
        cudaError_t e = set_smem(kernel, plan.smem_bytes);
        if (e != cudaSuccess) return e;
        kernel<<<plan.grid, plan.block, plan.smem_bytes, stream>>>(p);
    } else {
        auto kernel = gemv_mma_kernel<kDtype, false, false, kUnroll, kThreads, kMinBlocks>;
        cudaError_t e = set_smem(kernel, plan.smem_bytes);
        if (e != cudaSuccess) return e;
        kernel<<<plan.grid, plan.block, plan.smem_bytes, stream>>>(p);
    }
    return cudaGetLastError();
}

template <int kDtype>
cudaError_t launch_mma_staged(const GemvParams &p, const GemvPlan &plan, cudaStream_t stream)
{
    if (p.m > 8) {
        auto kernel = gemv_mma_staged_kernel<kDtype, true>;
        cudaError_t e = set_smem(kernel, plan.smem_bytes);
        if (e != cudaSuccess) return e;
        kernel<<<plan.grid, plan.block, plan.smem_bytes, stream>>>(p);
    } else {
        auto kernel = gemv_mma_staged_kernel<kDtype, false>;
        cudaError_t e = set_smem(kernel, plan.smem_bytes);
        if (e != cudaSuccess) return e;
        kernel<<<plan.grid, plan.block, plan.smem_bytes, stream>>>(p);
    }
    return cudaGetLastError();
}

// Launch shapes: threads per CTA / resident CTAs per SM the kernel is compiled for.
struct GemvShape {
    int threads, min_blocks;
};
constexpr GemvShape kShapes[3] = {{512, 2}, {1024, 1}, {1024, 2}};
constexpr int kStagedShape = 3;  // GemvPlan::shape of the staged-feed MMA kernel

template <int kDtype, bool kFma>
cudaError_t launch_shape(const GemvParams &p, const GemvPlan &plan, int shape, cudaStream_t stream)
{
#define KB_SHAPE_CASE(S, T, B)                                                                       \
    case S:                                                                                          \
        if constexpr (kFma) {                                                                        \
            return launch_fma_m<kDtype, 4, T, B>(p, plan, stream);                                   \
        } else if constexpr (kDtype == KUDNN_B200_F16 || kDtype == KUDNN_B200_BF16) {                \
            return launch_mma_rows<kDtype, 4, T, B>(p, plan, stream);                                \
        }                                                                                            \
        return cudaErrorInvalidValue;
    switch (shape) {
        KB_SHAPE_CASE(0, 512, 2)
        KB_SHAPE_CASE(1, 1024, 1)
        KB_SHAPE_CASE(2, 1024, 2)
        default:
            return cudaErrorInvalidValue;
    }
#undef KB_SHAPE_CASE
}

}  // namespace

// Decides whether a problem can take a streaming kernel and how it is cut.  Pure host arithmetic.
bool gemv_plan(const LinearProblem &pr, int sm_count, int forced_kernel, GemvPlan *plan)
{
    if (pr.batch_count != 1 || pr.m > 16 || pr.m < 1) {
        return false;
    }
    // fp16 activations against 8-bit weights: the FMA kernel streams the weights as they are (a single row)
    const bool w8 = pr.a_dtype == KUDNN_B200_F16 && (pr.b_dtype == KUDNN_B200_S8 || pr.b_dtype == KUDNN_B200_U8);
    if ((pr.a_dtype != pr.b_dtype && !w8) || pr.a_sk != 1 || pr.b_sk != 1) {
        return false;
    }
    // The 8-bit weights are streamed as they are.  One row: FMA kernel (64 us on a 28672 x 8192 matrix against 85 us for
    // the fp16 form of the weights; with 2 rows its shared-memory reads of the activations take over, 87 us, 142 us
    // with 4).  More rows: the MMA kernel, which widens the values to fp16 in registers.
    if (w8 && pr.m > 1 && forced_kernel == KUDNN_B200_KERNEL_GEMV_FMA) {
        return false;
    }
    const int dt = w8 ? pr.b_dtype : pr.a_dtype;
    const int vec = (dt == KUDNN_B200_F32) ? 4 : (w8 ? 16 : 8);
    if (pr.k % vec != 0 || (pr.m > 1 && pr.a_sm % vec != 0) || (pr.n > 1 && pr.b_sn % vec != 0) || pr.k > (1 << 24) ||
        pr.n > (1 << 28)) {
        return false;
    }
    if ((reinterpret_cast<uintptr_t>(pr.a) & 15u) != 0 || (reinterpret_cast<uintptr_t>(pr.b) & 15u) != 0) {
        return false;
    }
    const size_t max_smem = 200 * 1024;
    int kernel = forced_kernel;
    if (kernel != KUDNN_B200_KERNEL_GEMV_FMA && kernel != KUDNN_B200_KERNEL_GEMV_MMA) {
        kernel = (dt == KUDNN_B200_F32 || pr.m <= 1) ? KUDNN_B200_KERNEL_GEMV_FMA : KUDNN_B200_KERNEL_GEMV_MMA;
    }
    plan->kernel = kernel;
    int shape = -1;
    if (kernel == KUDNN_B200_KERNEL_GEMV_FMA) {
        if (pr.m > 4) {
            return false;
        }
        const int block_k = 32 * vec;
        const long long kb = (pr.k + block_k - 1) / block_k;
        const size_t smem = static_cast<size_t>(pr.m) * kb * block_k * sizeof(float);
        if (smem > max_smem) {
            return false;
        }
        if (shape < 0 || shape > 2) {
            shape = (smem <= 100 * 1024) ? 0 : 1;
        }
        if (smem > 100 * 1024) {
            shape = 1;  // only one CTA fits per SM
        }
        const int threads = kShapes[shape].threads, warps = threads / 32;
        const int grid = sm_count * kShapes[shape].min_blocks;
        const long long total = pr.n * kb;
        long long active = std::min<long long>(static_cast<long long>(grid) * warps, pr.n);  // keeps span >= kb
        active = std::max<long long>(active, 1);
        const long long span = (total + active - 1) / active;
        active = (total + span - 1) / span;
        plan->shape = shape;
        plan->wide = 0;
        plan->block = threads;
        plan->grid = static_cast<int>((active + warps - 1) / warps);
        plan->ksplit = 1;
        plan->active_warps = static_cast<int>(active);
        plan->span = span;
        plan->slots = 2;
        plan->smem_bytes = smem;
        plan->partial_floats = pr.n * 2 * pr.m;
        plan->counter_count = pr.n;
        return true;
    }
    // MMA kernel
    if (dt == KUDNN_B200_F32) {
        return false;
    }
    const int rows = pr.m > 8 ? 16 : 8;
    // Which feed (measured on config 4, microseconds per call).  Up to 8 activation rows: 88 for the staged feed on
    // decode-packed weights and for the fragment-shaped loads on plain rows, 92-94 for the other two pairings.  With
    // 16 rows the second half of the activation operand doubles the shared-memory reads per staged block (107
    // against 90 for the fragment-shaped loads of 32 bytes per lane).  The environment switches exist for the tests,
    // which run every feed on every shape: KUDNN_B200_GEMV_STAGED forces the staged feed for every m (1) or turns it
    // off (0), KUDNN_B200_GEMV_WIDE=0 makes the fragment-shaped loads 16 bytes per lane.
    const int staged_env = env_int("KUDNN_B200_GEMV_STAGED", -1);
    const bool staged = !w8 && (staged_env < 0 ? (rows == 8 && pr.b_blocked != nullptr) : staged_env != 0);
    if (staged && (shape < 0 || shape == kStagedShape)) {
        // staged feed: 512 threads, one CTA per SM, blocks of 8 rows x 256 k
        const int warps = kStagedThreads / 32;
        const size_t staging = static_cast<size_t>(warps) * kStagedWarpBytes;
        const size_t budget = 225 * 1024 - staging;
        int ksplit = 0;
        auto chunk_len = [&](int parts) {
            return ((pr.k + parts - 1) / parts + kStagedBlockK - 1) / kStagedBlockK * kStagedBlockK;
        };
        if (ksplit <= 0) {
            ksplit = 1;
            while (ksplit < 64 && static_cast<size_t>(rows) * (chunk_len(ksplit) * 2 + kMmaRowPadBytes) > budget) {
                ksplit *= 2;
            }
        }
        const long long kc = chunk_len(ksplit);
        const size_t xbytes = static_cast<size_t>(rows) * (kc * 2 + kMmaRowPadBytes);
        if (xbytes <= budget) {
            const int grid = std::max(sm_count / ksplit, 1) * ksplit;
            const long long groups = (pr.n + 7) / 8;
            const long long kbc = kc / kStagedBlockK;
            const long long total = groups * kbc;
            long long active = std::min<long long>(static_cast<long long>(grid / ksplit) * warps, 2 * groups);
            active = std::max<long long>(active, 1);
            const long long span = (total + active - 1) / active;
            active = (total + span - 1) / span;
            plan->shape = kStagedShape;
            plan->wide = 0;
            plan->block = kStagedThreads;
            plan->grid = static_cast<int>((active + warps - 1) / warps) * ksplit;
            plan->ksplit = ksplit;
            plan->active_warps = static_cast<int>(active);
            plan->span = span;
            plan->slots = static_cast<int>((kbc + span - 1) / span) + 1;
            plan->smem_bytes = xbytes + staging;
            plan->partial_floats = groups * ksplit * plan->slots * 128;
            plan->counter_count = groups;
            return true;
        }
    }
    if (shape < 0 || shape > 2) {
        // 16 activation rows: one 1024-thread CTA per SM leaves room for a longer K chunk (fewer partial sums)
        shape = (rows == 16) ? 1 : 0;
    }
    const size_t smem_budget = (kShapes[shape].min_blocks == 2) ? 100 * 1024 : max_smem;
    int ksplit = 0;
    // 16 activation rows: blocks of 64 k with 32 bytes per lane (see gemv_mma_kernel)
    const bool wide = w8 || (rows == 16 && env_int("KUDNN_B200_GEMV_WIDE", 1) != 0);
    const long long block_k = wide ? 64 : 32;
    if (ksplit <= 0) {
        ksplit = 1;
        while (ksplit < 64) {
            const long long kc = ((pr.k + ksplit - 1) / ksplit + block_k - 1) / block_k * block_k;
            if (static_cast<size_t>(rows) * (kc * 2 + kMmaRowPadBytes) <= smem_budget) {
                break;
            }
            ksplit *= 2;
        }
    }
    const long long kc = ((pr.k + ksplit - 1) / ksplit + block_k - 1) / block_k * block_k;
    const size_t smem = static_cast<size_t>(rows) * (kc * 2 + kMmaRowPadBytes);
    if (smem > max_smem) {
        return false;
    }
    if (smem > 100 * 1024 && kShapes[shape].min_blocks == 2) {
        shape = 1;
    }
    const int threads = kShapes[shape].threads, warps = threads / 32;
    int grid = sm_count * kShapes[shape].min_blocks;
    grid = std::max(grid / ksplit, 1) * ksplit;
    const long long groups = (pr.n + 7) / 8;
    const long long kbc = kc / block_k;
    const long long total = groups * kbc;
    long long active = std::min<long long>(static_cast<long long>(grid / ksplit) * warps, 2 * groups);
    active = std::max<long long>(active, 1);
    const long long span = (total + active - 1) / active;
    active = (total + span - 1) / span;
    plan->wide = wide ? 1 : 0;
    plan->shape = shape;
    plan->block = threads;
    plan->grid = static_cast<int>((active + warps - 1) / warps) * ksplit;
    plan->ksplit = ksplit;
    plan->active_warps = static_cast<int>(active);
    plan->span = span;
    plan->slots = static_cast<int>((kbc + span - 1) / span) + 1;
    plan->smem_bytes = smem;
    plan->partial_floats = groups * ksplit * plan->slots * 128;
    plan->counter_count = groups;
    return true;
}

cudaError_t launch_gemv(const LinearProblem &pr, const GemvPlan &plan, const GemvWorkspace &ws, cudaStream_t stream)
{
    if (ws.partial_floats < plan.partial_floats || ws.counter_count < plan.counter_count) {
        return cudaErrorInvalidValue;
    }
    GemvParams p;
    p.x = pr.a;
    p.w = pr.b;
    p.x_ld = pr.a_sm;
    p.w_ld = pr.b_sn;
    p.m = static_cast<int>(pr.m);
    p.n = static_cast<int>(pr.n);
    p.k = static_cast<int>(pr.k);
    p.ksplit = plan.ksplit;
    p.active_warps = plan.active_warps;
    p.span = plan.span;
    p.slots = plan.slots;
    p.partials = ws.partials;
    p.counters = ws.counters;
    p.epi = pr.epi;
    p.w_blk = plan.kernel == KUDNN_B200_KERNEL_GEMV_MMA ? static_cast<const unsigned short *>(pr.b_blocked) : nullptr;
    p.w8 = pr.b_dtype == KUDNN_B200_S8 ? 1 : (pr.b_dtype == KUDNN_B200_U8 ? 2 : 0);
    p.blk_kb = static_cast<int>(pr.b_blocked_kpad / 64);
    const bool w8 = pr.b_dtype == KUDNN_B200_S8 || pr.b_dtype == KUDNN_B200_U8;
    const int dt = w8 ? pr.b_dtype : pr.a_dtype;
    if (plan.kernel == KUDNN_B200_KERNEL_GEMV_FMA) {
        const int vec = (dt == KUDNN_B200_F32) ? 4 : (w8 ? 16 : 8);
        p.kb = static_cast<int>((pr.k + 32 * vec - 1) / (32 * vec));
        p.kc = 0;
        p.total = pr.n * p.kb;
        if (dt == KUDNN_B200_F32) {
            return launch_shape<KUDNN_B200_F32, true>(p, plan, plan.shape, stream);
        }
        if (dt == KUDNN_B200_S8) {
            return launch_shape<KUDNN_B200_S8, true>(p, plan, plan.shape, stream);
        }
        if (dt == KUDNN_B200_U8) {
            return launch_shape<KUDNN_B200_U8, true>(p, plan, plan.shape, stream);
        }
        if (dt == KUDNN_B200_F16) {
            return launch_shape<KUDNN_B200_F16, true>(p, plan, plan.shape, stream);
        }
        return launch_shape<KUDNN_B200_BF16, true>(p, plan, plan.shape, stream);
    }
    if (plan.shape == kStagedShape) {
        const long long kcs = ((pr.k + plan.ksplit - 1) / plan.ksplit + kStagedBlockK - 1) / kStagedBlockK * kStagedBlockK;
        p.kc = static_cast<int>(kcs);
        p.kb = static_cast<int>(kcs / kStagedBlockK);
        p.total = ((pr.n + 7) / 8) * p.kb;
        return dt == KUDNN_B200_F16 ? launch_mma_staged<KUDNN_B200_F16>(p, plan, stream)
                                    : launch_mma_staged<KUDNN_B200_BF16>(p, plan, stream);
    }
    const long long block_k = plan.wide != 0 ? 64 : 32;
    const long long kc = ((pr.k + plan.ksplit - 1) / plan.ksplit + block_k - 1) / block_k * block_k;
    p.kc = static_cast<int>(kc);
    p.kb = static_cast<int>(kc / block_k);
    p.total = ((pr.n + 7) / 8) * p.kb;
    if (pr.a_dtype == KUDNN_B200_F16) {
        return launch_shape<KUDNN_B200_F16, false>(p, plan, plan.shape, stream);
    }
    return launch_shape<KUDNN_B200_BF16, false>(p, plan, plan.shape, stream);
}

}  // namespace kb
