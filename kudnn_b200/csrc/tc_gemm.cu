// Tensor-core Linear kernel for sm_100a: tcgen05.mma with the accumulator in tensor memory, operands brought
// into a multi-stage shared-memory ring by TMA, bias / activation / second output fused into the
// TMEM -> register epilogue.  It replaces the blocked, packed GEMM of the reference's JIT backend
// (src/dnn/src/matmul_jit/MatrixComputation/kudnn_default_impl_fp16fp16f32f32.cpp:900-983) and the BLAS calls of
// src/dnn/src/kudnn_gemm.cpp:157-227.
//
// Shape of one CTA (320 threads, persistent over output tiles, one CTA per SM):
//   warp 0       producer: one lane issues the TMA loads of the A tile [128 x 128 B] and the B tile [rows x 128 B]
//                of every k-block into the ring (4 to 6 stages), 128-byte swizzle, completion on an mbarrier
//   warp 1       one lane issues tcgen05.mma (K = 32 bytes per instruction, four per k-block) into one of two TMEM
//                accumulators and commits to the stage's "empty" barrier / the tile's "full" barrier; the warp also
//                owns TMEM allocation
//   warps 2..9   epilogue: a warp reads its 32 TMEM lanes (= 32 output rows; two warps share a lane quarter and
//                split the columns) 8 columns at a time, applies the post-GEMM chain and stores 16 or 32 bytes per
//                tensor straight from registers (with output mirrors: 128-byte row pieces collected in shared memory); the
//                second accumulator lets this overlap the next tile's main loop
// Three launch shapes (tc_make_plan): clusters of two CTAs on 256 x 256 tiles with cta_group::2 MMAs (large
// problems), single CTAs on 128 x 256 / 128 x 128 tiles, and clusters of 2-8 CTAs that cut K of one 128 x 128 tile
// and add their partial tiles through distributed shared memory (few tiles, long K).
// Operands are K-major ([rows, k], k contiguous).  16-bit inputs run as kind::f16 with fp32 accumulation.  fp32
// inputs run as kind::tf32 on split planes: x = hi + lo with hi = tf32(x), and the packed operands
// A' = [a_lo | a_hi | a_hi], B' = [b_hi | b_lo | b_hi] make one pass over 3k compute a_lo.b_hi + a_hi.b_lo + a_hi.b_hi.
//
// Every wait on an mbarrier is bounded: after about two seconds (4e9 SM cycles) the waiting thread records a timeout in the
// handle's status block, raises a CTA-wide abort flag that all other waits poll, and the CTA drains and frees its
// tensor memory before returning.
#include "kernels.cuh"
#include "sm100_ptx.cuh"

#include <cuda.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace kb {

namespace {

constexpr int kBM = 128;
// Two epilogue warps per scheduler (8 in all, 320 threads per CTA).  With three (12 warps, 128 registers each and some
// spills) every shape measured 1.3-2.5 % slower on the same box: config 3's shape 208.8 against 203.7 us without
// post-operation and 251 against 246 us with GELU and residual, config 2 290 against 285 us, the 32768-row layer 12.6
// against 12.4 ms.
constexpr int kEpiWarps = 8;
constexpr int kTcThreads = 64 + 32 * kEpiWarps;  // warp 0: TMA, warp 1: MMA, the rest: epilogue
constexpr int kStageRowBytes = 128;  // one swizzle row: 64 16-bit or 32 32-bit elements
constexpr int kABytes = kBM * kStageRowBytes;
constexpr int kMaxGroupM = 16;  // most tile rows per raster group
constexpr int kWarpBiasFloats = 128;  // per epilogue warp: the bias values of its columns of the current tile, as fp32
constexpr int kWarpStageBytes = 32 * 128;  // per epilogue warp: 32 rows x 128 bytes of output on their way to memory
// after the stage ring: barriers and flags (256 bytes), the bias slices; then, if present, the output staging
constexpr int kTailBytes = 256 + kEpiWarps * kWarpBiasFloats * 4;
constexpr int kStagingBytes = kEpiWarps * kWarpStageBytes;  // only launches with output mirrors carry it (one stage less)
constexpr int kMaxStages = 6;

struct TcParams {
    EpiParams epi;
    int m, n;
    int num_kb;
    int tiles_m, tiles_n, num_tiles;
    unsigned idesc;
    DeviceStatus *status;
    // split-K for problems with fewer tiles than SMs: the `splits` CTAs of a thread-block cluster share one tile,
    // each contracts over kb_per_split k-blocks, and the partial tiles are added through distributed shared memory
    int splits, kb_per_split;
    int stages;  // depth of the shared-memory ring
    int group_m;  // tile rows per raster group: consecutive work items walk down group_m tile rows, then one tile right
    // CTA pairs: work items [0, narrow_from) are whole 256 x BN tiles; each later tile is two items of half the width,
    // so that a last wave that would keep fewer than half the pairs busy is spread over twice as many
    int num_items, narrow_from;
    unsigned idesc_narrow;
    // Batched problems: `batch` matrices share the launch, work items run over (batch entry, tile, split).  The tensor
    // maps are then three-dimensional; an operand every entry shares (a_bz / b_bz = 0) is always read at entry 0.  The
    // epilogue tensors are addressed through the batch strides in bp.
    int batch, a_bz, b_bz;
    BatchParams bp;
    long long wait_limit;  // SM cycles after which a wait on an mbarrier gives up
    // Test hook for the timeout path: the producer of CTA 0 leaves out the loads of this k-block of its first work
    // item (-1 = never), so the MMA thread's wait for that stage runs into wait_limit.  Nothing faults or hangs.
    int skip_kb;
    // Epilogue warps that work (4 or 8 of the kEpiWarps launched; the rest wait at the end of the kernel).  A light
    // epilogue (no activation, relu or SiLU, one output) is finished by one warp per scheduler long before the next
    // accumulator is ready, and every further warp only takes issue slots and power from the MMA and load threads;
    // GELU or a second output need two per scheduler.  Same-box runs, 8 against 4 working warps: config 2 281.5
    // against 276.5 us, a 4096-row shard of the large layer 1.432 against 1.405 ms, the whole layer 12.48 against
    // 12.34 ms; with GELU and a residual 242 against 291 us (config 3's shape).
    int epi_warps;
};


// ---- epilogue side-input / output access, 8 consecutive columns at a time ---------------------------------

// Reads 8 values at element index idx0 + j * sn.  `vec` promises sn == 1, all 8 in range and 16-byte alignment.
__device__ __forceinline__ void load8(const void *base, int dtype, long long idx0, long long sn, bool vec, int valid,
                                      float (&o)[8])
{
    if (sn == 0) {
        const float v = load_as_f32(base, dtype, idx0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            o[j] = v;
        }
        return;
    }
    if (vec) {
        if (dtype == KUDNN_B200_F32) {
            const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(base) + idx0);
            const float4 v0 = p[0], v1 = p[1];
            o[0] = v0.x; o[1] = v0.y; o[2] = v0.z; o[3] = v0.w;
            o[4] = v1.x; o[5] = v1.y; o[6] = v1.z; o[7] = v1.w;
        } else {
            const uint4 v = *reinterpret_cast<const uint4 *>(static_cast<const unsigned short *>(base) + idx0);
            const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (dtype == KUDNN_B200_BF16) {
                    o[2 * j] = __uint_as_float(w[j] << 16);
                    o[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
                } else {
                    o[2 * j] = f16_bits_to_f32(static_cast<unsigned short>(w[j] & 0xffffu));
                    o[2 * j + 1] = f16_bits_to_f32(static_cast<unsigned short>(w[j] >> 16));
                }
            }
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        o[j] = (j < valid) ? load_as_f32(base, dtype, idx0 + j * sn) : 0.0f;
    }
}

// Stores 8 values that are exactly representable in dtype.
__device__ __forceinline__ void store8(void *base, int dtype, long long idx0, long long sn, bool vec, int valid,
                                       const float (&v)[8])
{
    if (vec) {
        if (dtype == KUDNN_B200_F32) {
            float4 *p = reinterpret_cast<float4 *>(static_cast<float *>(base) + idx0);
            p[0] = make_float4(v[0], v[1], v[2], v[3]);
            p[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
            unsigned w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                unsigned lo, hi;
                if (dtype == KUDNN_B200_BF16) {
                    lo = __float_as_uint(v[2 * j]) >> 16;
                    hi = __float_as_uint(v[2 * j + 1]) & 0xffff0000u;
                } else {
                    lo = f32_to_f16_rne_bits(v[2 * j]);
                    hi = static_cast<unsigned>(f32_to_f16_rne_bits(v[2 * j + 1])) << 16;
                }
                w[j] = lo | hi;
            }
            *reinterpret_cast<uint4 *>(static_cast<unsigned short *>(base) + idx0) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (j < valid) {
            store_exact(base, dtype, idx0 + j * sn, v[j]);
        }
    }
}

__device__ __forceinline__ bool vec_ok(const void *base, int dtype, long long idx0, long long sn)
{
    if (sn != 1 || base == nullptr) {
        return false;
    }
    const uintptr_t addr = reinterpret_cast<uintptr_t>(base) + static_cast<uintptr_t>(idx0) * dtype_size(dtype);
    return (addr & 15u) == 0;
}

// Post-GEMM chain and stores for 8 consecutive columns of one output row, starting at column ni.  Same arithmetic
// as finish_element(), but organised as passes over the 8 values: every run-time switch (element type, bias,
// second output) is tested once per pass instead of once per element, which leaves straight-line code with eight
// independent dependency chains: with three epilogue warps per scheduler, instruction-level parallelism is what
// hides the arithmetic latency.
template <int kAct, int kPrecise>
__device__ __forceinline__ void epilogue_group8(const EpiParams &e, const uint32_t (&raw)[8], long long mi, long long ni)
{
    const int valid = (e.n - ni >= 8) ? 8 : static_cast<int>(e.n - ni);
    if (valid <= 0) {
        return;
    }
    const bool full8 = valid == 8;
    const int ct = e.c_dtype;
    float v[8], side[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[j] = e.alpha * __uint_as_float(raw[j]);
    }
    const long long ic = mi * e.c_sm + ni * e.c_sn;
    const bool c_vec = full8 && vec_ok(e.c, ct, ic, e.c_sn);
    if (e.beta != 0.0f) {
        load8(e.c, ct, ic, e.c_sn, c_vec, valid, side);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] += e.beta * side[j];
        }
    }
    if (e.has_bias) {
        const long long ib = mi * e.bias_sm + ni * e.bias_sn;
        load8(e.bias, e.bias_dtype, ib, e.bias_sn, full8 && vec_ok(e.bias, e.bias_dtype, ib, e.bias_sn), valid, side);
    }
    if (e.half_chain != 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = __half2float(__float2half_rn(v[j]));
        }
        if (e.has_bias) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = __half2float(__float2half_rn(v[j] + side[j]));
            }
        }
    } else {
        if (e.has_bias) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] += side[j];
            }
        }
        if (ct == KUDNN_B200_BF16) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
            }
        } else if (ct == KUDNN_B200_F16) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = __half2float(__float2half_rn(v[j]));
            }
        }
    }
    if (kAct != KUDNN_B200_ACT_NONE) {
        if (kAct < 0) {
            if (e.act != KUDNN_B200_ACT_NONE) {
                for (int j = 0; j < 8; ++j) {
                    v[j] = activation_any(v[j], e.act, e.act_alpha, ct == KUDNN_B200_F32 ? 1 : 0);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = activation<kPrecise == 1>(v[j], kAct, e.act_alpha);
            }
        }
        if (ct == KUDNN_B200_F16) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = __half2float(__float2half_rn(v[j]));
            }
        } else if (ct == KUDNN_B200_BF16) {
            if ((kAct < 0 ? e.act : kAct) == KUDNN_B200_ACT_RELU && e.act_alpha != 0.0f) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[j] = relu_bf16_overflow(v[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = __uint_as_float(__float_as_uint(v[j]) & 0xffff0000u);
            }
        }
    }
    if (e.c != nullptr) {
        store8(e.c, ct, ic, e.c_sn, c_vec, valid, v);
        for (int i = 0; i < e.n_mirrors; ++i) {
            store8(static_cast<char *>(e.c) + e.c_delta[i], ct, ic, e.c_sn, c_vec, valid, v);
        }
    }
    if (e.res_op != KUDNN_B200_RES_NONE) {
        const long long ir = mi * e.res_sm + ni * e.res_sn;
        load8(e.res, e.res_dtype, ir, e.res_sn, full8 && vec_ok(e.res, e.res_dtype, ir, e.res_sn), valid, side);
        if (e.res_op == KUDNN_B200_RES_IDENTICAL) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] += side[j];
            }
        } else if (e.res_op == KUDNN_B200_RES_EXT) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = fmaf(side[j], e.gamma, v[j]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] *= side[j];
            }
        }
        const int ot = e.out_dtype;
        if (ot == KUDNN_B200_F16) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = __half2float(__float2half_rn(v[j]));
            }
        } else if (ot == KUDNN_B200_BF16) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
            }
        }
        const long long io = mi * e.out_sm + ni * e.out_sn;
        const bool out_vec = full8 && vec_ok(e.out, ot, io, e.out_sn);
        store8(e.out, ot, io, e.out_sn, out_vec, valid, v);
        for (int i = 0; i < e.n_mirrors; ++i) {
            store8(static_cast<char *>(e.out) + e.out_delta[i], ot, io, e.out_sn, out_vec, valid, v);
        }
    }
}

// Per-row state of the fast path: byte pointers to the first column this thread handles.
struct RowPointers {
    char *c;
    const char *bias;
    const char *res;
    char *out;
    float bias_scalar;  // bias that does not vary along the row (column vector or single value)
    int bias_mode;      // 0 none, 1 per-column values read from `bias`, 2 bias_scalar, 3 fp32 values in bias_smem
    const float *bias_smem;  // the warp's slice of pre-loaded bias values, 8 per column group
};

__device__ __forceinline__ void load8_vec(const char *p, int dtype, float (&o)[8])
{
    if (dtype == KUDNN_B200_F32) {
        const float4 v0 = reinterpret_cast<const float4 *>(p)[0], v1 = reinterpret_cast<const float4 *>(p)[1];
        o[0] = v0.x; o[1] = v0.y; o[2] = v0.z; o[3] = v0.w;
        o[4] = v1.x; o[5] = v1.y; o[6] = v1.z; o[7] = v1.w;
    } else {
        const uint4 v = *reinterpret_cast<const uint4 *>(p);
        const unsigned w[4] = {v.x, v.y, v.z, v.w};
        if (dtype == KUDNN_B200_BF16) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                o[2 * j] = __uint_as_float(w[j] << 16);
                o[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
                o[2 * j] = f.x;
                o[2 * j + 1] = f.y;
            }
        }
    }
}

// v holds values exactly representable in dtype
__device__ __forceinline__ void store8_vec(char *p, int dtype, const float (&v)[8])
{
    if (dtype == KUDNN_B200_F32) {
        reinterpret_cast<float4 *>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4 *>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        unsigned w[4];
        if (dtype == KUDNN_B200_BF16) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w[j] = (__float_as_uint(v[2 * j]) >> 16) | (__float_as_uint(v[2 * j + 1]) & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                w[j] = *reinterpret_cast<const unsigned *>(&h);
            }
        }
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

template <int kDt>
__device__ __forceinline__ void round_rne8(float (&v)[8])
{
    if (kDt == KUDNN_B200_F16) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = __half2float(__float2half_rn(v[j]));
        }
    } else if (kDt == KUDNN_B200_BF16) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
        }
    }
}

// Arithmetic of the fast form of epilogue_group8 (beta == 0, side inputs contiguous along the row and 16-byte
// aligned at this group, all 8 columns in range), first half: v receives the 8 values of c, exactly representable
// in c's type.
// kDt: element type of c, bias, res and out when they all equal the kernel's input type (the common case: every
// type test below is then decided at compile time), or -1 when the types are read from the descriptor.
template <int kAct, int kDt>
__device__ __forceinline__ void compute_c8_fast(const EpiParams &e, const uint32_t (&raw)[8], const RowPointers &rp,
                                                int byte_off_bias, int g, float (&v)[8])
{
    const int ct = kDt > 0 ? kDt : e.c_dtype;
    float side[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[j] = __uint_as_float(raw[j]);
    }
    if (e.alpha != 1.0f) {  // multiplying by exactly 1 changes nothing, so the common case skips the pass
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] *= e.alpha;
        }
    }
    if (rp.bias_mode == 3) {
        const float4 b0 = *reinterpret_cast<const float4 *>(rp.bias_smem + g * 8);
        const float4 b1 = *reinterpret_cast<const float4 *>(rp.bias_smem + g * 8 + 4);
        side[0] = b0.x; side[1] = b0.y; side[2] = b0.z; side[3] = b0.w;
        side[4] = b1.x; side[5] = b1.y; side[6] = b1.z; side[7] = b1.w;
    } else if (rp.bias_mode == 1) {
        load8_vec(rp.bias + byte_off_bias, kDt > 0 ? kDt : e.bias_dtype, side);
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            side[j] = rp.bias_scalar;
        }
    }
    if (ct == KUDNN_B200_F16 && e.half_chain != 0) {
        round_rne8<KUDNN_B200_F16>(v);
        if (rp.bias_mode != 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] += side[j];
            }
            round_rne8<KUDNN_B200_F16>(v);
        }
    } else {
        if (rp.bias_mode != 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] += side[j];
            }
        }
        if (ct == KUDNN_B200_BF16) {
            round_rne8<KUDNN_B200_BF16>(v);
        } else if (ct == KUDNN_B200_F16) {
            round_rne8<KUDNN_B200_F16>(v);
        }
    }
    if (kAct != KUDNN_B200_ACT_NONE) {
        if (kAct < 0) {
            if (e.act != KUDNN_B200_ACT_NONE) {
                for (int j = 0; j < 8; ++j) {
                    v[j] = activation_any(v[j], e.act, e.act_alpha, ct == KUDNN_B200_F32 ? 1 : 0);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = activation<kDt == KUDNN_B200_F32>(v[j], kAct, e.act_alpha);
            }
        }
        if (ct == KUDNN_B200_F16) {
            round_rne8<KUDNN_B200_F16>(v);
        } else if (ct == KUDNN_B200_BF16) {
            if ((kAct < 0 ? e.act : kAct) == KUDNN_B200_ACT_RELU && e.act_alpha != 0.0f) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[j] = relu_bf16_overflow(v[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = __uint_as_float(__float_as_uint(v[j]) & 0xffff0000u);
            }
        }
    }
}

// Second half: v holds the values of c and is replaced by those of the second output (c (+) res).
template <int kDt>
__device__ __forceinline__ void compute_out8_fast(const EpiParams &e, const RowPointers &rp, int byte_off_res, float (&v)[8])
{
    float side[8];
    load8_vec(rp.res + byte_off_res, kDt > 0 ? kDt : e.res_dtype, side);
    if (e.res_op == KUDNN_B200_RES_IDENTICAL) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] += side[j];
        }
    } else if (e.res_op == KUDNN_B200_RES_EXT) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = fmaf(side[j], e.gamma, v[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] *= side[j];
        }
    }
    const int ot = kDt > 0 ? kDt : e.out_dtype;
    if (ot == KUDNN_B200_F16) {
        round_rne8<KUDNN_B200_F16>(v);
    } else if (ot == KUDNN_B200_BF16) {
        round_rne8<KUDNN_B200_BF16>(v);
    }
}

// Fast form of epilogue_group8: same arithmetic, no address arithmetic beyond pointer bumps, one 16-byte (fp32: two)
// store per tensor and mirror.
template <int kAct, int kDt>
__device__ __forceinline__ void epilogue_group8_fast(const EpiParams &e, const uint32_t (&raw)[8], const RowPointers &rp,
                                                     int byte_off_c, int byte_off_bias, int byte_off_res, int byte_off_out,
                                                     int g)
{
    float v[8];
    compute_c8_fast<kAct, kDt>(e, raw, rp, byte_off_bias, g, v);
    if (rp.c != nullptr) {
        store8_vec(rp.c + byte_off_c, kDt > 0 ? kDt : e.c_dtype, v);
        for (int i = 0; i < e.n_mirrors; ++i) {
            store8_vec(rp.c + e.c_delta[i] + byte_off_c, kDt > 0 ? kDt : e.c_dtype, v);
        }
    }
    if (e.res_op != KUDNN_B200_RES_NONE) {
        compute_out8_fast<kDt>(e, rp, byte_off_res, v);
        store8_vec(rp.out + byte_off_out, kDt > 0 ? kDt : e.out_dtype, v);
        for (int i = 0; i < e.n_mirrors; ++i) {
            store8_vec(rp.out + e.out_delta[i] + byte_off_out, kDt > 0 ? kDt : e.out_dtype, v);
        }
    }
}

__device__ __forceinline__ bool row_contiguous_aligned(const void *base, int dtype, long long idx0, long long sn)
{
    return sn == 1 && ((reinterpret_cast<uintptr_t>(base) + static_cast<uintptr_t>(idx0) * dtype_size(dtype)) & 15u) == 0;
}

// One thread's share of a tile: its row, `groups` groups of 8 columns starting at column n0, read from TMEM at
// taddr.  The loop is rolled to keep the code small (a fully unrolled epilogue does not fit the instruction cache
// and runs an order of magnitude slower); the TMEM load of the next group is in flight while the current one is
// processed.  Rows whose tensors are contiguous and 16-byte aligned take the pointer-bumping fast path.
// ---- row-coalesced output ---------------------------------------------------------------------------------------
// A TMEM lane is a row, so a thread's natural store is 16 bytes of its own row and a warp's store instruction touches
// 32 rows.  When a whole warp takes the vector path and one output tensor is written, the warp instead collects 128
// bytes per row (8 column groups of a 16-bit type, 4 of fp32) in 4 KiB of shared memory of its own and writes them
// out with every instruction covering 4 rows x 128 contiguous bytes.  That is what memory, and above all a peer GPU
// behind NVLink (mirrors), wants to see.  Chunks of 16 bytes are swizzled with the row index so that both the
// row-wise writes and the chunk-wise reads are free of bank conflicts.  No barrier beyond __syncwarp is involved.
__device__ __forceinline__ void pack8_to_chunks(const float (&v)[8], int dtype, uint4 &lo, uint4 &hi)
{
    if (dtype == KUDNN_B200_F32) {
        lo = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
        hi = make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7]));
    } else {
        unsigned w[4];
        if (dtype == KUDNN_B200_BF16) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w[j] = (__float_as_uint(v[2 * j]) >> 16) | (__float_as_uint(v[2 * j + 1]) & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                w[j] = *reinterpret_cast<const unsigned *>(&h);
            }
        }
        lo = make_uint4(w[0], w[1], w[2], w[3]);
        hi = lo;
    }
}

// The one 16-bit output of this thread for a group of 8 columns, packed into 16 bytes: c, or the second output when c
// is not written.
template <int kAct, int kDt>
__device__ __forceinline__ uint4 epilogue_group8_packed(const EpiParams &e, const uint32_t (&raw)[8], const RowPointers &rp,
                                                        int byte_off_bias, int byte_off_res, int g)
{
    float v[8];
    compute_c8_fast<kAct, kDt>(e, raw, rp, byte_off_bias, g, v);
    int dt = kDt > 0 ? kDt : e.c_dtype;
    if (rp.c == nullptr) {
        compute_out8_fast<kDt>(e, rp, byte_off_res, v);
        dt = kDt > 0 ? kDt : e.out_dtype;
    }
    uint4 lo, hi;
    pack8_to_chunks(v, dt, lo, hi);
    return lo;
}

// 32 bytes = one whole sector of the row: L2 takes it as it is, where a 16-byte store makes it merge the bytes into the
// sector it holds (measured: a thread's 16-byte stores cost the epilogue about 1000 cycles per column group)
__device__ __forceinline__ void store_32(char *p, const uint4 &a, const uint4 &b)
{
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
                 "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

template <int kAct, int kDt>
__device__ __noinline__ void epilogue_rows_coalesced(const EpiParams &e, uint32_t taddr, int groups, const RowPointers rp,
                                                        unsigned char *stage, int lane)
{
    // the one output tensor that is written: c, or the second output when c is not requested
    const bool second = rp.c == nullptr;
    const int odt = kDt > 0 ? kDt : (second ? e.out_dtype : e.c_dtype);
    const int chunks_per_group = (odt == KUDNN_B200_F32) ? 2 : 1;
    const int groups_per_pass = 8 / chunks_per_group;
    const long long pitch = (second ? e.out_sm : e.c_sm) * dtype_size(odt);  // bytes between rows
    char *row0 = (second ? rp.out : rp.c) - static_cast<long long>(lane) * pitch;  // row of lane 0
    const long long *delta = second ? e.out_delta : e.c_delta;
    const long long mc_delta = second ? e.out_mc_delta : e.c_mc_delta;
    const int step_bias = 8 * dtype_size(kDt > 0 ? kDt : e.bias_dtype), step_res = 8 * dtype_size(kDt > 0 ? kDt : e.res_dtype);
    const uint32_t stage_addr = smem_u32(stage);
    const uint32_t my_row = stage_addr + static_cast<uint32_t>(lane * 128);

    uint32_t next[8], cur[8];
    tmem_load_8_issue(taddr, next);
    for (int g0 = 0; g0 < groups; g0 += groups_per_pass) {
        const int pass_groups = (groups - g0 < groups_per_pass) ? groups - g0 : groups_per_pass;
#pragma unroll 1
        for (int gi = 0; gi < pass_groups; ++gi) {
            const int g = g0 + gi;
            tmem_load_wait(next);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                cur[j] = next[j];
            }
            if (g + 1 < groups) {
                tmem_load_8_issue(taddr + static_cast<uint32_t>((g + 1) * 8), next);
            }
            float v[8];
            compute_c8_fast<kAct, kDt>(e, cur, rp, g * step_bias, g, v);
            if (second) {
                compute_out8_fast<kDt>(e, rp, g * step_res, v);
            }
            uint4 lo, hi;
            pack8_to_chunks(v, odt, lo, hi);
            const int c0 = gi * chunks_per_group;
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + static_cast<uint32_t>(((c0 ^ (lane & 7)) << 4))),
                         "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w)
                         : "memory");
            if (chunks_per_group == 2) {
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(
                                 my_row + static_cast<uint32_t>((((c0 + 1) ^ (lane & 7)) << 4))),
                             "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                             : "memory");
            }
        }
        __syncwarp();
        // 8 lanes per row, 4 rows per instruction
        const int chunk = lane & 7;
        const int valid_chunks = pass_groups * chunks_per_group;
        const long long col_bytes = static_cast<long long>(g0) * 8 * dtype_size(odt) + chunk * 16;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int r = j * 4 + (lane >> 3);
            if (chunk < valid_chunks) {
                uint4 v;
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                             : "r"(stage_addr + static_cast<uint32_t>(r * 128 + ((chunk ^ (r & 7)) << 4))));
                char *dst = row0 + r * pitch + col_bytes;
                if (e.use_multicast != 0) {
                    // one store through the multicast mapping: the switch writes every rank's copy, this one included
                    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + mc_delta),
                                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                                 : "memory");
                } else {
                    *reinterpret_cast<uint4 *>(dst) = v;
                    for (int i = 0; i < e.n_mirrors; ++i) {
                        *reinterpret_cast<uint4 *>(dst + delta[i]) = v;
                    }
                }
            }
        }
        __syncwarp();  // the rows are reused by the next pass
    }
}

// Row-base pointers for the vector path of the epilogue.  Returns whether that path applies to the `groups` groups
// of 8 columns starting at (mi, n0): whole groups inside n, no beta term, every tensor involved contiguous along n
// and 16-byte aligned there.
__device__ __forceinline__ bool setup_row_pointers(const EpiParams &e, bool row_ok, long long mi, long long n0, int groups,
                                                   RowPointers &rp)
{
    rp.c = nullptr;
    rp.bias = nullptr;
    rp.res = nullptr;
    rp.out = nullptr;
    rp.bias_scalar = 0.0f;
    rp.bias_mode = 0;
    rp.bias_smem = nullptr;
    bool fast = row_ok && e.beta == 0.0f && (n0 + static_cast<long long>(groups) * 8 <= e.n);
    if (fast) {
        if (e.c != nullptr) {
            const long long ic = mi * e.c_sm + n0 * e.c_sn;
            fast = fast && row_contiguous_aligned(e.c, e.c_dtype, ic, e.c_sn);
            rp.c = static_cast<char *>(e.c) + ic * dtype_size(e.c_dtype);
        }
        if (e.has_bias) {
            const long long ib = mi * e.bias_sm + n0 * e.bias_sn;
            if (e.bias_sn == 0) {
                rp.bias_mode = 2;
                rp.bias_scalar = load_as_f32(e.bias, e.bias_dtype, ib);
            } else {
                rp.bias_mode = 1;
                fast = fast && row_contiguous_aligned(e.bias, e.bias_dtype, ib, e.bias_sn);
                rp.bias = static_cast<const char *>(e.bias) + ib * dtype_size(e.bias_dtype);
            }
        }
        if (e.res_op != KUDNN_B200_RES_NONE) {
            const long long ir = mi * e.res_sm + n0 * e.res_sn;
            const long long io = mi * e.out_sm + n0 * e.out_sn;
            fast = fast && row_contiguous_aligned(e.res, e.res_dtype, ir, e.res_sn) &&
                   row_contiguous_aligned(e.out, e.out_dtype, io, e.out_sn);
            rp.res = static_cast<const char *>(e.res) + ir * dtype_size(e.res_dtype);
            rp.out = static_cast<char *>(e.out) + io * dtype_size(e.out_dtype);
        }
    }
    return fast;
}

template <int kAct, int kDt>
__device__ __forceinline__ void epilogue_row(const EpiParams &e, uint32_t taddr, bool row_ok, long long mi, long long n0,
                                             int groups, const float *staged_bias, unsigned char *stage, int lane)
{
    if (groups <= 0) {
        return;
    }
    RowPointers rp;
    const bool fast = setup_row_pointers(e, row_ok, mi, n0, groups, rp);
    if (staged_bias != nullptr && rp.bias_mode == 1) {
        rp.bias_mode = 3;
        rp.bias_smem = staged_bias;
    }
    // all 32 rows on the vector path and a single output tensor: collect 128-byte row pieces and store those
    const bool one_output = (rp.c != nullptr) != (e.res_op != KUDNN_B200_RES_NONE);
    if (stage != nullptr && __all_sync(0xffffffffu, fast && one_output)) {
        epilogue_rows_coalesced<kAct, kDt>(e, taddr, groups, rp, stage, lane);
        return;
    }
    const int step_c = 8 * dtype_size(kDt > 0 ? kDt : e.c_dtype), step_bias = 8 * dtype_size(kDt > 0 ? kDt : e.bias_dtype);
    const int step_res = 8 * dtype_size(kDt > 0 ? kDt : e.res_dtype), step_out = 8 * dtype_size(kDt > 0 ? kDt : e.out_dtype);

    // One 16-bit output and no mirrors: two neighbouring column groups leave as one 32-byte store wherever the first of
    // them starts a sector (the groups of a part are consecutive, so all but a ragged first or last one pair up).
    const int odt = rp.c != nullptr ? (kDt > 0 ? kDt : e.c_dtype) : (kDt > 0 ? kDt : e.out_dtype);
    const bool pairs = fast && one_output && e.n_mirrors == 0 && dtype_size(odt) == 2;
    char *obase = rp.c != nullptr ? rp.c : rp.out;
    uint4 held = make_uint4(0u, 0u, 0u, 0u);
    bool have_held = false;

    uint32_t next[8], cur[8];
    tmem_load_8_issue(taddr, next);
#pragma unroll 1
    for (int g = 0; g < groups; ++g) {
        __syncwarp();  // rows of a warp may have taken different paths below; the TMEM instructions need them together
        tmem_load_wait(next);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            cur[j] = next[j];
        }
        if (g + 1 < groups) {
            tmem_load_8_issue(taddr + static_cast<uint32_t>((g + 1) * 8), next);
        }
        if (pairs) {
            const uint4 pk = epilogue_group8_packed<kAct, kDt>(e, cur, rp, g * step_bias, g * step_res, g);
            char *dst = obase + g * 16;
            if (have_held) {
                store_32(dst - 16, held, pk);
                have_held = false;
            } else if ((reinterpret_cast<uintptr_t>(dst) & 31u) == 0 && g + 1 < groups) {
                held = pk;
                have_held = true;
            } else {
                *reinterpret_cast<uint4 *>(dst) = pk;
            }
        } else if (fast) {
            epilogue_group8_fast<kAct, kDt>(e, cur, rp, g * step_c, g * step_bias, g * step_res, g * step_out, g);
        } else if (row_ok) {
            epilogue_group8<kAct, (kDt < 0 ? -1 : (kDt == KUDNN_B200_F32 ? 1 : 0))>(e, cur, mi, n0 + g * 8);
        }
    }
}

// 8-bit integer products: the accumulator holds exact 32-bit sums; c = acc (+ bias, 32-bit integers), clamped to the
// 32-bit range like the general kernel does.  alpha = 1 and beta = 0 (the host sends anything else elsewhere).
__device__ __forceinline__ void epilogue_row_int(const EpiParams &e, uint32_t taddr, bool row_ok, long long mi, long long n0,
                                                 int groups)
{
    if (groups <= 0) {
        return;
    }
    int *crow = static_cast<int *>(e.c) + (row_ok ? mi * e.c_sm + n0 * e.c_sn : 0);
    const int *brow = e.has_bias ? static_cast<const int *>(e.bias) + (row_ok ? mi * e.bias_sm + n0 * e.bias_sn : 0) : nullptr;
    const bool vec = row_ok && e.c_sn == 1 && (reinterpret_cast<uintptr_t>(crow) & 15u) == 0;
    uint32_t next[8], cur[8];
    tmem_load_8_issue(taddr, next);
#pragma unroll 1
    for (int g = 0; g < groups; ++g) {
        __syncwarp();  // rows past m skip the stores below; the TMEM instructions need the whole warp
        tmem_load_wait(next);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            cur[j] = next[j];
        }
        if (g + 1 < groups) {
            tmem_load_8_issue(taddr + static_cast<uint32_t>((g + 1) * 8), next);
        }
        if (!row_ok) {
            continue;
        }
        const long long left = e.n - (n0 + g * 8);
        const int valid = left >= 8 ? 8 : static_cast<int>(left);
        int v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            long long r = static_cast<int>(cur[j]);
            if (brow != nullptr && j < valid) {
                r += brow[(g * 8 + j) * e.bias_sn];
            }
            r = r > 2147483647ll ? 2147483647ll : (r < -2147483648ll ? -2147483648ll : r);
            v[j] = static_cast<int>(r);
        }
        if (vec && valid == 8) {
            int4 *dst = reinterpret_cast<int4 *>(crow + g * 8);
            dst[0] = make_int4(v[0], v[1], v[2], v[3]);
            dst[1] = make_int4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (j < valid) {
                    crow[(g * 8 + j) * e.c_sn] = v[j];
                }
            }
        }
    }
}

// ---- split-K through a thread-block cluster
// Every CTA of the cluster leaves its partial tile in its own shared memory as [128 rows][BN + 4 floats] (the four
// extra floats put the 16-byte stores of 8 consecutive rows on distinct banks).  After a cluster barrier, CTA r adds,
// for its 128 / splits rows, the partial tiles of all ranks in rank order (the result does not depend on timing) and
// runs the post-GEMM chain for those rows.
constexpr int kMaxSplits = 8;

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ float4 ld_cluster_f4(uint32_t local_smem_addr, uint32_t rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(remote)
                 : "memory");
    return v;
}

// Copies `groups` groups of 8 accumulator columns of this thread's row from TMEM to `dst` (shared memory).  The
// loads are issued three groups at a time before the wait.
__device__ __forceinline__ void dump_partial_row(uint32_t taddr, float *dst, int groups)
{
    for (int g0 = 0; g0 < groups; g0 += 3) {
        uint32_t r[3][8];
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 3; ++u) {
            if (g0 + u < groups) {
                tmem_load_8_issue(taddr + static_cast<uint32_t>((g0 + u) * 8), r[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < 3; ++u) {
            if (g0 + u < groups) {
                tmem_load_wait(r[u]);
                float4 *out = reinterpret_cast<float4 *>(dst + (g0 + u) * 8);
                out[0] = make_float4(__uint_as_float(r[u][0]), __uint_as_float(r[u][1]), __uint_as_float(r[u][2]),
                                     __uint_as_float(r[u][3]));
                out[1] = make_float4(__uint_as_float(r[u][4]), __uint_as_float(r[u][5]), __uint_as_float(r[u][6]),
                                     __uint_as_float(r[u][7]));
            }
        }
    }
}

// The epilogue threads of cluster rank `rank` finish rows [rank * 128 / splits, (rank + 1) * 128 / splits) of the tile.
template <int kAct, int kDt, int kBN>
__device__ __forceinline__ void finish_split_rows(const EpiParams &e, const float *part, int splits, uint32_t rank, int tm,
                                                  int tn, int m, int n, int epi_tid)
{
    constexpr int kPitch = kBN + 4;
    constexpr int kGroups = kBN / 8;
    const int rows_per = kBM / splits;
    const uint32_t part_addr = smem_u32(part);
    for (int u = epi_tid; u < rows_per * kGroups; u += kEpiWarps * 32) {
        const int r_local = u / kGroups, g = u - r_local * kGroups;
        const int row = static_cast<int>(rank) * rows_per + r_local;
        const long long mi = static_cast<long long>(tm) * kBM + row;
        const long long ni = static_cast<long long>(tn) * kBN + g * 8;
        if (mi >= m || ni >= n) {
            continue;
        }
        const uint32_t addr = part_addr + static_cast<uint32_t>((row * kPitch + g * 8) * 4);
        float4 lo[kMaxSplits], hi[kMaxSplits];
#pragma unroll
        for (int s = 0; s < kMaxSplits; ++s) {
            if (s < splits) {
                lo[s] = ld_cluster_f4(addr, static_cast<uint32_t>(s));
                hi[s] = ld_cluster_f4(addr + 16, static_cast<uint32_t>(s));
            }
        }
        float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int s = 0; s < kMaxSplits; ++s) {
            if (s < splits) {
                acc[0] += lo[s].x; acc[1] += lo[s].y; acc[2] += lo[s].z; acc[3] += lo[s].w;
                acc[4] += hi[s].x; acc[5] += hi[s].y; acc[6] += hi[s].z; acc[7] += hi[s].w;
            }
        }
        uint32_t raw[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            raw[j] = __float_as_uint(acc[j]);
        }
        RowPointers rp;
        if (setup_row_pointers(e, true, mi, ni, 1, rp)) {
            epilogue_group8_fast<kAct, kDt>(e, raw, rp, 0, 0, 0, 0, 0);
        } else {
            epilogue_group8<kAct, (kDt < 0 ? -1 : (kDt == KUDNN_B200_F32 ? 1 : 0))>(e, raw, mi, ni);
        }
    }
}

// Work item -> tile index, column offset inside the tile and width of the piece.
template <bool kPair, int kBN>
__device__ __forceinline__ void decode_item(const TcParams &p, int item, int &tile, int &n_off, int &width, int &batch,
                                            int &split)
{
    batch = 0;
    split = 0;
    if (!kPair) {
        const int unit = item / p.splits;  // (batch entry, tile)
        split = item - unit * p.splits;
        batch = unit / p.num_tiles;
        tile = unit - batch * p.num_tiles;
        n_off = 0;
        width = kBN;
    } else if (item < p.narrow_from) {
        tile = item;
        n_off = 0;
        width = kBN;
    } else {
        const int j = item - p.narrow_from;
        tile = p.narrow_from + (j >> 1);
        n_off = (j & 1) * (kBN / 2);
        width = kBN / 2;
    }
}

// kPair: two CTAs (a cluster of two SMs) work on a 256 x kBN tile with cta_group::2 MMAs.  Each CTA loads its 128
// rows of A and half of the B rows, so a k-block costs an SM 32 KiB of L2 traffic instead of the 48 KiB of the
// single-CTA 128 x 256 tile; the single-CTA kernel is limited by exactly that traffic.  Rank 0 of the pair (the
// leader) owns the "full" barriers, issues all MMAs and releases the stages of both CTAs.
template <int kKind, int kBN, bool kPair>
__global__ void __launch_bounds__(kTcThreads, 1)
    tc_linear_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ TcParams p)
{
    constexpr int kBRows = kPair ? kBN / 2 : kBN;  // rows of B this CTA loads per k-block
    constexpr int kBBytes = kBRows * kStageRowBytes;
    constexpr int kStageBytes = kABytes + kBBytes;
    const int kStages = p.stages;  // 3-6, what fits beside the tail (and the output staging when mirrors are written)
    constexpr int kTmemCols = 2 * kBN;
    constexpr int kElemsPerRow = (kKind == KUDNN_B200_F32) ? 32 : (kKind == KUDNN_B200_S8 ? 128 : 64);  // per 128-byte k-block row

    extern __shared__ unsigned char smem_dyn[];
    // stage buffers need 1024-byte alignment for the 128-byte swizzle pattern
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023u) &
                                                            ~static_cast<uintptr_t>(1023u));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes);
    uint64_t *full_bar = bars;
    uint64_t *empty_bar = bars + kMaxStages;
    uint64_t *tmem_full = bars + 2 * kMaxStages;
    uint64_t *tmem_empty = bars + 2 * kMaxStages + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kMaxStages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tmem_full + a, 1);
            mbar_init(tmem_empty + a, kPair ? 2 * p.epi_warps : p.epi_warps);  // pair: the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        if (kPair) {
            // executed by the same warp of both CTAs with the same destination offset
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"(kTmemCols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"(kTmemCols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (kPair) {
        cluster_sync_all();  // the peer's barriers are initialised before anything is signalled on them
    }
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // work items: tiles (x splits) over CTAs, or pair tiles over clusters of two
    const uint32_t pair_rank = kPair ? cluster_rank() : 0u;
    const int first_item = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int item_stride = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
            int stage = 0;
            uint32_t phase = 0;
            bool alive = true;
            for (int item = first_item; alive && item < p.num_items; item += item_stride) {
                int tile, n_off, width, batch, split;
                decode_item<kPair, kBN>(p, item, tile, n_off, width, batch, split);
                const int kb_begin = split * p.kb_per_split;
                const int kb_end = (kb_begin + p.kb_per_split < p.num_kb) ? kb_begin + p.kb_per_split : p.num_kb;
                const int per_group = p.group_m * p.tiles_n;
                const int group = tile / per_group;
                const int first_m = group * p.group_m;
                const int gsize = (p.tiles_m - first_m < p.group_m) ? (p.tiles_m - first_m) : p.group_m;
                const int in_group = tile - group * per_group;
                const int tn = in_group / gsize;
                // row of 128-row blocks this CTA loads: the pair's tile is 256 rows tall
                const int tm = kPair ? 2 * (first_m + in_group % gsize) + static_cast<int>(pair_rank)
                                     : first_m + in_group % gsize;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(empty_bar + stage, phase ^ 1u, abort_flag, p.status, 1, p.wait_limit)) {
                        alive = false;
                        break;
                    }
                    unsigned char *sa = smem + stage * kStageBytes;
                    unsigned char *sb = sa + kABytes;
                    if (kb == p.skip_kb && blockIdx.x == 0 && item == first_item) {
                        // test hook: this stage is never filled
                    } else if (kPair) {
                        // both CTAs' bytes are counted on the leader's barrier; only the leader announces them
                        if (pair_rank == 0) {
                            mbar_expect_tx(full_bar + stage, 2 * kStageBytes);
                        }
                        const uint32_t leader_bar = map_to_rank(smem_u32(full_bar + stage), 0u);
                        tma_load_2d_pair(sa, &tmap_a, leader_bar, kb * kElemsPerRow, tm * kBM);
                        // this CTA's half of the piece's B rows (a narrow piece uses the first half of the box only)
                        tma_load_2d_pair(sb, &tmap_b, leader_bar, kb * kElemsPerRow,
                                         tn * kBN + n_off + static_cast<int>(pair_rank) * (width / 2));
                    } else {
                        mbar_expect_tx(full_bar + stage, kStageBytes);
                        if (p.batch > 1) {
                            tma_load_3d(sa, &tmap_a, full_bar + stage, kb * kElemsPerRow, tm * kBM, p.a_bz != 0 ? batch : 0);
                            tma_load_3d(sb, &tmap_b, full_bar + stage, kb * kElemsPerRow, tn * kBN, p.b_bz != 0 ? batch : 0);
                        } else {
                            tma_load_2d(sa, &tmap_a, full_bar + stage, kb * kElemsPerRow, tm * kBM);
                            tma_load_2d(sb, &tmap_b, full_bar + stage, kb * kElemsPerRow, tn * kBN);
                        }
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && pair_rank == 0) {  // in a pair, the leader issues for both CTAs
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool alive = true;
            for (int item = first_item; alive && item < p.num_items; item += item_stride) {
                int tile, n_off, width, batch, split;
                decode_item<kPair, kBN>(p, item, tile, n_off, width, batch, split);
                const uint32_t idesc = (width == kBN) ? p.idesc : p.idesc_narrow;
                const int kb_begin = split * p.kb_per_split;
                const int kb_end = (kb_begin + p.kb_per_split < p.num_kb) ? kb_begin + p.kb_per_split : p.num_kb;
                if (!mbar_wait(tmem_empty + acc, acc_phase ^ 1u, abort_flag, p.status, 2, p.wait_limit)) {
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kBN);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(full_bar + stage, phase, abort_flag, p.status, 3, p.wait_limit)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * kStageBytes);
                    const uint64_t adesc = make_smem_desc(sa);
                    const uint64_t bdesc = make_smem_desc(sa + kABytes);
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        // 32 bytes along k inside the swizzle row = 2 units of the 16-byte address field
                        if (kPair) {
                            umma_pair<kKind>(tmem_d, adesc + static_cast<uint64_t>(2 * ks),
                                             bdesc + static_cast<uint64_t>(2 * ks), idesc,
                                             (kb != kb_begin || ks != 0) ? 1u : 0u);
                        } else {
                            umma<kKind>(tmem_d, adesc + static_cast<uint64_t>(2 * ks), bdesc + static_cast<uint64_t>(2 * ks),
                                        idesc, (kb != kb_begin || ks != 0) ? 1u : 0u);
                        }
                    }
                    if (kPair) {
                        umma_commit_pair(empty_bar + stage);  // frees the stage in both CTAs
                    } else {
                        umma_commit(empty_bar + stage);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!alive) {
                    break;
                }
                if (kPair) {
                    umma_commit_pair(tmem_full + acc);  // both CTAs' epilogue warps wait on their own copy
                } else {
                    umma_commit(tmem_full + acc);
                }
                acc ^= 1;
                if (acc == 0) {
                    acc_phase ^= 1u;
                }
            }
        }
    } else if (warp < 2 + p.epi_warps) {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;  // TMEM lanes this warp may touch: [32 * quarter, 32 * quarter + 32)
        const int row_in_tile = quarter * 32 + lane;
        const int part = (warp - 2) / 4;  // warps sharing a quarter split the tile's columns between them
        EpiParams e_batch;  // the epilogue tensors of the current batch entry (batched launches only)
        // the bias slices of the working warps share the space laid out for kEpiWarps slices of kWarpBiasFloats
        float *warp_bias = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(bars) + 256) +
                           (warp - 2) * (kEpiWarps * kWarpBiasFloats / p.epi_warps);
        // Rows are collected into 128-byte pieces before they are stored only when peers receive copies: for local
        // memory alone the 16-byte stores straight from registers are faster (measured both ways).
        unsigned char *warp_stage = p.epi.n_mirrors > 0 ? reinterpret_cast<unsigned char *>(bars) + kTailBytes +
                                                          (warp - 2) * kWarpStageBytes
                                                    : nullptr;
        int acc = 0;
        uint32_t acc_phase = 0;
        // "accumulator drained" goes to the MMA thread, which in a pair lives in the leader CTA
        const uint32_t tmem_empty_remote = kPair ? map_to_rank(smem_u32(tmem_empty), 0u) : 0u;
        for (int item = first_item; item < p.num_items; item += item_stride) {
            int tile, n_off, width, batch, split;
            decode_item<kPair, kBN>(p, item, tile, n_off, width, batch, split);
            if (p.batch > 1) {
                e_batch = epi_for_batch(p.epi, p.bp, batch);
            }
            const EpiParams &e = p.batch > 1 ? e_batch : p.epi;
            const int per_group = p.group_m * p.tiles_n;
            const int group = tile / per_group;
            const int first_m = group * p.group_m;
            const int gsize = (p.tiles_m - first_m < p.group_m) ? (p.tiles_m - first_m) : p.group_m;
            const int in_group = tile - group * per_group;
            const int tm = kPair ? 2 * (first_m + in_group % gsize) + static_cast<int>(pair_rank) : first_m + in_group % gsize;
            const int tn = in_group / gsize;
            // the warps that share a lane quarter split the tile's 8-column groups between them
            const int kParts = p.epi_warps / 4;
            const int piece_groups = width / 8;
            const int g_begin = part * piece_groups / kParts, g_end = (part + 1) * piece_groups / kParts;
            const long long n0 = static_cast<long long>(tn) * kBN + n_off + g_begin * 8;
            long long cols = p.n - n0;
            const long long part_cols = static_cast<long long>(g_end - g_begin) * 8;
            cols = cols < 0 ? 0 : (cols < part_cols ? cols : part_cols);
            const int groups = static_cast<int>((cols + 7) / 8);
            // A bias that is one value per column is fetched once per tile into the warp's slice of shared memory,
            // before the accumulator is awaited: the loop over column groups then has no global load on its path.
            const float *staged_bias = nullptr;
            if (kKind != KUDNN_B200_S8 && e.has_bias != 0 && e.bias_sm == 0 && e.bias_sn == 1) {
                __syncwarp();  // every lane is done with the previous tile's values
                for (int i = lane; i < groups * 8; i += 32) {
                    const long long col = n0 + i;
                    warp_bias[i] = col < p.n ? load_as_f32(e.bias, e.bias_dtype, col) : 0.0f;
                }
                __syncwarp();
                staged_bias = warp_bias;
            }
            // every lane waits on its own and may see the abort flag at a different poll: agree on one answer before
            // the warp-wide tensor-memory instructions below
            const bool arrived =
                __all_sync(0xffffffffu, mbar_wait(tmem_full + acc, acc_phase, abort_flag, p.status, 4, p.wait_limit));
            if (!arrived && p.splits == 1) {
                break;
            }
            tc_fence_after();
            const long long mi = static_cast<long long>(tm) * kBM + row_in_tile;
            const bool row_ok = mi < p.m;
            const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(acc * kBN);
            const uint32_t taddr_part = taddr_row + static_cast<uint32_t>(g_begin * 8);
            if (kKind != KUDNN_B200_S8 && p.splits > 1) {
                // partial tile -> this CTA's shared memory (the stage buffers: every load into them has landed and
                // every MMA that read them has completed once the accumulator barrier has fired); it is added to
                // the other ranks' tiles after the role branches, where all warps of the cluster meet
                if (arrived) {
                    float *part = reinterpret_cast<float *>(smem);
                    dump_partial_row(taddr_part, part + row_in_tile * (kBN + 4) + g_begin * 8, g_end - g_begin);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(tmem_empty + acc);
                    }
                }
                break;  // one work item per CTA in this mode
            }
            if constexpr (kKind == KUDNN_B200_S8) {
                epilogue_row_int(e, taddr_part, row_ok, mi, n0, groups);
            } else {
                // All output-side tensors in the kernel's input type (the usual case): the epilogue variants with the
                // element type fixed at compile time.  Any other mix, or a rarer activation: the variant that reads the
                // types and the activation from the descriptor.
                const bool typed = e.c_dtype == kKind && (e.has_bias == 0 || e.bias_dtype == kKind) &&
                                   (e.res_op == KUDNN_B200_RES_NONE || (e.res_dtype == kKind && e.out_dtype == kKind));
                const int act_case = typed ? e.act : -1;
                switch (act_case) {
                    case KUDNN_B200_ACT_NONE:
                        epilogue_row<KUDNN_B200_ACT_NONE, kKind>(e, taddr_part, row_ok, mi, n0, groups, staged_bias, warp_stage, lane);
                        break;
                    case KUDNN_B200_ACT_RELU:
                        epilogue_row<KUDNN_B200_ACT_RELU, kKind>(e, taddr_part, row_ok, mi, n0, groups, staged_bias, warp_stage, lane);
                        break;
                    case KUDNN_B200_ACT_SWISH:
                        epilogue_row<KUDNN_B200_ACT_SWISH, kKind>(e, taddr_part, row_ok, mi, n0, groups, staged_bias, warp_stage, lane);
                        break;
                    case KUDNN_B200_ACT_GELU_TANH:
                        epilogue_row<KUDNN_B200_ACT_GELU_TANH, kKind>(e, taddr_part, row_ok, mi, n0, groups, staged_bias, warp_stage, lane);
                        break;
                    default:
                        epilogue_row<-1, -1>(e, taddr_part, row_ok, mi, n0, groups, staged_bias, warp_stage, lane);
                        break;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (kPair) {
                    mbar_arrive_cluster(tmem_empty_remote + static_cast<uint32_t>(acc * sizeof(uint64_t)));
                } else {
                    mbar_arrive(tmem_empty + acc);
                }
            }
            acc ^= 1;
            if (acc == 0) {
                acc_phase ^= 1u;
            }
        }
    }

    if constexpr (kKind != KUDNN_B200_S8) {  // integer launches never split K
        if (p.splits > 1) {
            // ------------------------------------------------------------------ split-K: add the cluster's partial tiles
            __syncwarp();
            cluster_sync_all();  // all partial tiles are in place (a hardware barrier over every thread of the cluster)
            if (warp >= 2 && *abort_flag == 0) {
                const int unit = static_cast<int>(blockIdx.x) / p.splits;
                const int batch = unit / p.num_tiles;
                const int tile = unit - batch * p.num_tiles;
                const int per_group = p.group_m * p.tiles_n;
                const int group = tile / per_group;
                const int first_m = group * p.group_m;
                const int gsize = (p.tiles_m - first_m < p.group_m) ? (p.tiles_m - first_m) : p.group_m;
                const int in_group = tile - group * per_group;
                const int tm = first_m + in_group % gsize;
                const int tn = in_group / gsize;
                const float *part = reinterpret_cast<const float *>(smem);
                EpiParams e_batch;
                if (p.batch > 1) {
                    e_batch = epi_for_batch(p.epi, p.bp, batch);
                }
                const EpiParams &e = p.batch > 1 ? e_batch : p.epi;
                const uint32_t rank = cluster_rank();
                const int epi_tid = static_cast<int>(threadIdx.x) - 64;
                const bool typed = e.c_dtype == kKind && (e.has_bias == 0 || e.bias_dtype == kKind) &&
                                   (e.res_op == KUDNN_B200_RES_NONE || (e.res_dtype == kKind && e.out_dtype == kKind));
                switch (typed ? e.act : -1) {
                    case KUDNN_B200_ACT_NONE:
                        finish_split_rows<KUDNN_B200_ACT_NONE, kKind, kBN>(e, part, p.splits, rank, tm, tn, p.m, p.n, epi_tid);
                        break;
                    case KUDNN_B200_ACT_RELU:
                        finish_split_rows<KUDNN_B200_ACT_RELU, kKind, kBN>(e, part, p.splits, rank, tm, tn, p.m, p.n, epi_tid);
                        break;
                    case KUDNN_B200_ACT_SWISH:
                        finish_split_rows<KUDNN_B200_ACT_SWISH, kKind, kBN>(e, part, p.splits, rank, tm, tn, p.m, p.n, epi_tid);
                        break;
                    case KUDNN_B200_ACT_GELU_TANH:
                        finish_split_rows<KUDNN_B200_ACT_GELU_TANH, kKind, kBN>(e, part, p.splits, rank, tm, tn, p.m, p.n, epi_tid);
                        break;
                    default:
                        finish_split_rows<-1, -1, kBN>(e, part, p.splits, rank, tm, tn, p.m, p.n, epi_tid);
                        break;
                }
            }
            __syncwarp();
            cluster_sync_all();  // no CTA leaves while another still reads its shared memory
        }
    }

    // ---------------------------------------------------------------------- teardown
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag != 0) {
        // give copies and MMAs that were already issued time to land before the memory is handed back
        const long long t0 = clock64();
        while (clock64() - t0 < 400000ll) {
            __nanosleep(1000);
        }
        __syncthreads();
    }
    if (kPair) {
        // neither CTA frees tensor memory or leaves while the other may still signal its barriers or, through the
        // leader's MMAs, use its shared and tensor memory
        cluster_sync_all();
    }
    if (warp == 1) {
        if (kPair) {
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
        } else {
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
        }
    }
}

// ------------------------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::once_flag g_encode_once;
EncodeTiledFn g_encode = nullptr;
char g_tc_reason[160] = "";

void resolve_encode()
{
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
        std::snprintf(g_tc_reason, sizeof(g_tc_reason), "cuTensorMapEncodeTiled is not available from the driver (%s)",
                      cudaGetErrorString(e));
        (void)cudaGetLastError();
        return;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
}

cudaError_t encode_kmajor(CUtensorMap *map, const void *base, int kind, long long rows, long long k_total,
                          long long ld_elems, int box_rows, long long batch = 1, long long batch_stride = 0)
{
    if (batch > 1) {
        // [batch][rows][k]: a box is one batch entry deep.  An operand all entries share is encoded with one entry.
        const int es3 = dtype_size(kind);
        const CUtensorMapDataType dt3 = (kind == KUDNN_B200_F32)   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                        : (kind == KUDNN_B200_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                   : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        const bool shared = batch_stride == 0;
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(k_total), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(shared ? 1 : batch)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld_elems) * es3,
                                 static_cast<cuuint64_t>(shared ? rows * ld_elems : batch_stride) * es3};
        cuuint32_t box[3] = {static_cast<cuuint32_t>(kStageRowBytes / es3), static_cast<cuuint32_t>(box_rows), 1};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = g_encode(map, dt3, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
    }
    const int es = dtype_size(kind);
    const CUtensorMapDataType dt = (kind == KUDNN_B200_F32)   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : (kind == KUDNN_B200_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                   : (kind == KUDNN_B200_S8)  ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                              : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(k_total), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_elems) * es};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kStageRowBytes / es), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <int kKind, int kBN, bool kPair>
cudaError_t launch_one(const TcPlan &plan, const TcParams &p, cudaStream_t stream)
{
    auto kernel = tc_linear_kernel<kKind, kBN, kPair>;
    cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem_bytes));
    if (e != cudaSuccess) {
        return e;
    }
    CUtensorMap ta, tb;
    std::memcpy(&ta, plan.tmap_a, sizeof(ta));
    std::memcpy(&tb, plan.tmap_b, sizeof(tb));
    const int cluster = kPair ? 2 : plan.splits;
    if (cluster > 1) {
        // split-K: the CTAs that share a tile form a cluster, blockIdx.x = tile * splits + rank;
        // pair mode: clusters of two, blockIdx.x = 2 * cluster + rank
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(plan.grid), 1, 1);
        cfg.blockDim = dim3(kTcThreads, 1, 1);
        cfg.dynamicSmemBytes = plan.smem_bytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = static_cast<unsigned>(cluster);
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, kernel, ta, tb, p);
    }
    kernel<<<plan.grid, kTcThreads, plan.smem_bytes, stream>>>(ta, tb, p);
    return cudaGetLastError();
}

// How many clusters of two CTAs of the pair kernel the device runs at once (SMs pair up inside a GPC, so this can be
// fewer than half the SM count).  Queried once per kernel instance.
template <int kKind>
int max_pair_clusters(size_t smem_bytes)
{
    auto kernel = tc_linear_kernel<kKind, 256, true>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes)) !=
        cudaSuccess) {
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(kTcThreads, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return clusters;
}

}  // namespace

bool tc_available()
{
    std::call_once(g_encode_once, resolve_encode);
    return g_encode != nullptr;
}

const char *tc_unavailable_reason()
{
    return g_tc_reason;
}

cudaError_t tc_encode_kmajor(void *map128, const void *base, int kind, long long rows, long long k_total, long long ld_elems,
                             int box_rows)
{
    if (!tc_available()) {
        return cudaErrorNotSupported;
    }
    CUtensorMap m;
    cudaError_t e = encode_kmajor(&m, base, kind, rows, k_total, ld_elems, box_rows);
    if (e == cudaSuccess) {
        std::memcpy(map128, &m, sizeof(m));
    }
    return e;
}

cudaError_t tc_make_plan(const TcOperands &ops, long long m, long long n, int sm_count, bool with_staging, TcPlan *plan)
{
    static_assert(sizeof(CUtensorMap) <= 128, "tensor map storage too small");
    if (!tc_available()) {
        return cudaErrorNotSupported;
    }
    const long long tiles_m = (m + kBM - 1) / kBM;
    const long long tiles256 = ops.batch * tiles_m * ((n + 255) / 256);
    const int bn = (tiles256 >= sm_count || n > 128 * 64) ? 256 : 128;
    const long long tiles = ops.batch * tiles_m * ((n + bn - 1) / bn);  // over all batch entries
    if (tiles > (1ll << 30)) {
        return cudaErrorInvalidValue;
    }
    // CTA pairs for the large-problem shape (256-wide tiles): 256 x 256 tiles over clusters of two.  Not for launches
    // that run for many milliseconds: those are limited by the board's power cap, and the pair shape, which needs
    // fewer cycles, draws enough more power per cycle to end up slower there (bf16 n = 28672, k = 8192, ms per call,
    // pair / single CTA: 4096 rows 1.385 / 1.396, 8192 rows 2.84 / 2.85, 16384 rows 6.10 / 5.96, 32768 rows
    // 13.3 / 12.4).
    const double flops = 2.0 * static_cast<double>(m) * static_cast<double>(n) * static_cast<double>(ops.k_total);
    // batched launches use single CTAs
    bool pair = bn == 256 && m > kBM && flops < 6.0e12 && ops.batch == 1;
    if (const char *env = std::getenv("KUDNN_B200_TC_PAIR")) {
        pair = pair && std::atoi(env) != 0;
    }
    int pair_clusters = 0;
    if (pair) {
        const size_t smem = static_cast<size_t>(with_staging ? 5 : 6) * (kABytes + 128 * kStageRowBytes) + 1024 + kTailBytes +
                            (with_staging ? kStagingBytes : 0);
        pair_clusters = ops.kind == KUDNN_B200_F32   ? max_pair_clusters<KUDNN_B200_F32>(smem)
                        : ops.kind == KUDNN_B200_F16 ? max_pair_clusters<KUDNN_B200_F16>(smem)
                        : ops.kind == KUDNN_B200_S8  ? max_pair_clusters<KUDNN_B200_S8>(smem)
                                                     : max_pair_clusters<KUDNN_B200_BF16>(smem);
        pair = pair_clusters > 0;
    }
    plan->pair = pair ? 1 : 0;
    plan->narrow_from = 0;
    plan->block_n = bn;
    plan->stages = ((bn == 256 && !pair) ? 4 : 6) - (with_staging ? 1 : 0);
    // Split-K: with at most half the SMs busy and a long K, the CTAs of a cluster share a tile and cut K between
    // them (2, 4 or 8 ways: the rows of the tile are divided among the ranks for the final pass).  Each split keeps
    // at least four k-blocks so that the pipeline still fills, and no split may be empty.
    const int elems_per_row = kStageRowBytes / dtype_size(ops.kind);
    const long long num_kb = (ops.k_total + elems_per_row - 1) / elems_per_row;
    long long splits = 1;
    if (!pair && tiles * 2 <= sm_count && num_kb >= 8 && ops.kind != KUDNN_B200_S8) {
        long long want = std::min<long long>(sm_count / tiles, num_kb / 4);
        if (const char *env = std::getenv("KUDNN_B200_TC_SPLITS")) {
            const long long v = std::atoll(env);
            if (v >= 1 && v <= num_kb) {
                want = v;
            }
        }
        while (splits * 2 <= want && splits * 2 <= kMaxSplits) {
            splits *= 2;
        }
        while (splits > 1 && (num_kb + (num_kb + splits - 1) / splits - 1) / ((num_kb + splits - 1) / splits) != splits) {
            splits /= 2;
        }
    }
    plan->splits = static_cast<int>(splits);
    plan->kb_per_split = static_cast<int>((num_kb + splits - 1) / splits);
    const long long items = tiles * splits;
    plan->grid = splits > 1 ? static_cast<int>(items) : static_cast<int>(tiles < sm_count ? tiles : sm_count);
    const int b_rows = pair ? bn / 2 : bn;  // rows of the weight operand one CTA loads per k-block
    plan->smem_bytes = static_cast<size_t>(plan->stages) * (kABytes + b_rows * kStageRowBytes) + 1024 + kTailBytes +
                       (with_staging ? kStagingBytes : 0);
    if (pair) {
        const long long pair_tiles = ((m + 2 * kBM - 1) / (2 * kBM)) * ((n + bn - 1) / bn);
        plan->grid = 2 * static_cast<int>(pair_tiles < pair_clusters ? pair_tiles : pair_clusters);
        // Tiles left over after the last full wave: if they would keep at most half of the pairs busy, each of them
        // is processed as two pieces of half the width, which shortens that wave to a little more than half.
        const long long rem = pair_tiles % pair_clusters;
        bool narrow = pair_tiles > pair_clusters && rem > 0 && 2 * rem <= pair_clusters;
        plan->narrow_from = static_cast<int>(narrow ? pair_tiles - rem : pair_tiles);
    }
    CUtensorMap ta, tb;
    cudaError_t e = encode_kmajor(&ta, ops.a, ops.kind, m, ops.k_total, ops.lda, kBM, ops.batch, ops.a_bstride);
    if (e != cudaSuccess) {
        return e;
    }
    e = encode_kmajor(&tb, ops.b, ops.kind, n, ops.k_total, ops.ldb, b_rows, ops.batch, ops.b_bstride);
    if (e != cudaSuccess) {
        return e;
    }
    std::memcpy(plan->tmap_a, &ta, sizeof(ta));
    std::memcpy(plan->tmap_b, &tb, sizeof(tb));
    return cudaSuccess;
}

cudaError_t launch_tc(const TcOperands &ops, const TcPlan &plan, const EpiParams &epi, long long m, long long n,
                      DeviceStatus *status, cudaStream_t stream, long long wait_limit_cycles, int skip_kblock,
                      const BatchParams *bp)
{
    TcParams p;
    p.epi = epi;
    p.batch = static_cast<int>(ops.batch);
    p.a_bz = ops.a_bstride != 0 ? 1 : 0;
    p.b_bz = ops.b_bstride != 0 ? 1 : 0;
    std::memset(&p.bp, 0, sizeof(p.bp));
    p.bp.n1 = p.bp.n2 = 1;
    if (ops.batch > 1) {
        if (bp == nullptr || plan.pair != 0) {
            return cudaErrorInvalidValue;
        }
        p.bp = *bp;
    }
    p.wait_limit = wait_limit_cycles > 0 ? wait_limit_cycles : kDefaultWaitLimitCycles;
    // the test hook is honoured by the plain single-CTA shape only (no cluster partner is left half-signalled)
    p.skip_kb = (plan.pair == 0 && plan.splits == 1) ? skip_kblock : -1;
    {
        const bool sixteen = ops.kind == KUDNN_B200_F16 || ops.kind == KUDNN_B200_BF16;
        const bool light = sixteen && plan.splits == 1 && ops.batch == 1 && epi.n_mirrors == 0 && epi.beta == 0.0f &&
                           epi.res_op == KUDNN_B200_RES_NONE && epi.c_dtype == ops.kind &&
                           (epi.has_bias == 0 || epi.bias_dtype == ops.kind) &&
                           (epi.act == KUDNN_B200_ACT_NONE || epi.act == KUDNN_B200_ACT_RELU || epi.act == KUDNN_B200_ACT_SWISH);
        p.epi_warps = light ? 4 : kEpiWarps;
    }
    p.m = static_cast<int>(m);
    p.n = static_cast<int>(n);
    const int elems_per_row = kStageRowBytes / dtype_size(ops.kind);
    p.num_kb = static_cast<int>((ops.k_total + elems_per_row - 1) / elems_per_row);
    const int tile_rows = plan.pair ? 2 * kBM : kBM;
    p.tiles_m = static_cast<int>((m + tile_rows - 1) / tile_rows);
    p.tiles_n = static_cast<int>((n + plan.block_n - 1) / plan.block_n);
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.idesc = ops.kind == KUDNN_B200_S8
                  ? make_idesc_i8(ops.a_signed != 0, ops.b_signed != 0, plan.block_n, plan.pair ? 2 * kBM : kBM)
                  : make_idesc(ops.kind, plan.block_n, plan.pair ? 2 * kBM : kBM);
    p.status = status;
    p.splits = plan.splits;
    p.kb_per_split = plan.kb_per_split;
    p.stages = plan.stages;
    {
        // The A rows of one raster group are re-read for every tile column and should stay in L2 next to the
        // streaming weights: at most about 64 MB of them (16 tile rows of 256 x 8192 bf16).  Measured on the 32768-row
        // layer, ms per call for 8 / 12 / 16 tile rows per group: 13.05 / 12.84 / 12.72; DRAM traffic is the same
        // within 3 % (the wave's working set exceeds what L2 retains either way).
        const long long tile_bytes = static_cast<long long>(tile_rows) * ops.k_total * dtype_size(ops.kind);
        long long gm = (64ll << 20) / (tile_bytes > 0 ? tile_bytes : 1);
        gm = gm < 2 ? 2 : (gm > kMaxGroupM ? kMaxGroupM : gm);
        p.group_m = static_cast<int>(gm);
    }
    p.num_items = plan.pair ? plan.narrow_from + 2 * (p.num_tiles - plan.narrow_from)
                            : p.num_tiles * plan.splits * static_cast<int>(ops.batch);
    p.narrow_from = plan.pair ? plan.narrow_from : p.num_tiles;
    p.idesc_narrow = ops.kind == KUDNN_B200_S8
                         ? make_idesc_i8(ops.a_signed != 0, ops.b_signed != 0, plan.block_n / 2, plan.pair ? 2 * kBM : kBM)
                         : make_idesc(ops.kind, plan.block_n / 2, plan.pair ? 2 * kBM : kBM);
    if (plan.pair) {
        switch (ops.kind) {
            case KUDNN_B200_S8:
                return launch_one<KUDNN_B200_S8, 256, true>(plan, p, stream);
            case KUDNN_B200_F32:
                return launch_one<KUDNN_B200_F32, 256, true>(plan, p, stream);
            case KUDNN_B200_F16:
                return launch_one<KUDNN_B200_F16, 256, true>(plan, p, stream);
            default:
                return launch_one<KUDNN_B200_BF16, 256, true>(plan, p, stream);
        }
    }
    if (ops.kind == KUDNN_B200_S8) {
        if (plan.splits != 1 || ops.batch != 1) {
            return cudaErrorInvalidValue;
        }
        return plan.block_n == 256 ? launch_one<KUDNN_B200_S8, 256, false>(plan, p, stream)
                                   : launch_one<KUDNN_B200_S8, 128, false>(plan, p, stream);
    }
    if (plan.block_n == 256) {
        switch (ops.kind) {
            case KUDNN_B200_F32:
                return launch_one<KUDNN_B200_F32, 256, false>(plan, p, stream);
            case KUDNN_B200_F16:
                return launch_one<KUDNN_B200_F16, 256, false>(plan, p, stream);
            default:
                return launch_one<KUDNN_B200_BF16, 256, false>(plan, p, stream);
        }
    }
    switch (ops.kind) {
        case KUDNN_B200_F32:
            return launch_one<KUDNN_B200_F32, 128, false>(plan, p, stream);
        case KUDNN_B200_F16:
            return launch_one<KUDNN_B200_F16, 128, false>(plan, p, stream);
        default:
            return launch_one<KUDNN_B200_BF16, 128, false>(plan, p, stream);
    }
}

}  // namespace kb
