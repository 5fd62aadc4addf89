// Tensor-core Linear kernel for sm_100a: tcgen05.mma with the accumulator in tensor memory, operands brought
// into a multi-stage shared-memory ring by TMA, bias / activation / second output fused into the
// TMEM -> register epilogue.  It replaces the blocked, packed GEMM of the reference's JIT backend
// (src/dnn/src/matmul_jit/MatrixComputation/kudnn_default_impl_fp16fp16f32f32.cpp:900-983) and the BLAS calls of
// src/dnn/src/kudnn_gemm.cpp:157-227.
//
// Shape of one CTA (192 threads, persistent over output tiles, one CTA per SM):
//   warp 0      producer: one lane issues the TMA loads of the A tile [128 x 128 B] and the B tile [BN x 128 B]
//               of every k-block into the ring (4 or 6 stages), 128-byte swizzle, completion on an mbarrier
//   warp 1      one lane issues tcgen05.mma (M=128, N=BN, K=32 bytes per instruction, four per k-block) into one
//               of two TMEM accumulators and commits to the stage's "empty" barrier / the tile's "full" barrier;
//               the warp also owns TMEM allocation
//   warps 2..5  epilogue: each warp reads its 32 TMEM lanes (= 32 output rows) 32 columns at a time, applies the
//               post-GEMM chain and stores 16-byte vectors; the second accumulator lets this overlap the next
//               tile's main loop
// Operands are K-major ([rows, k], k contiguous).  16-bit inputs run as kind::f16 with fp32 accumulation.  fp32
// inputs run as kind::tf32 on split planes: x = hi + lo with hi = tf32(x), and the packed operands
// A' = [a_lo | a_hi | a_hi], B' = [b_hi | b_lo | b_hi] make one pass over 3k compute a_lo.b_hi + a_hi.b_lo + a_hi.b_hi.
//
// Every wait on an mbarrier is bounded: after about two seconds the waiting thread records a timeout in the
// handle's status block, raises a CTA-wide abort flag that all other waits poll, and the CTA drains and frees its
// tensor memory before returning.
#include "kernels.cuh"

#include <cuda.h>

#include <cstdio>
#include <cstring>
#include <mutex>

namespace kb {

namespace {

constexpr int kBM = 128;
constexpr int kTcThreads = 192;
constexpr int kStageRowBytes = 128;  // one swizzle row: 64 16-bit or 32 32-bit elements
constexpr int kABytes = kBM * kStageRowBytes;
constexpr int kGroupM = 16;  // tile rows per raster group
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

struct TcParams {
    EpiParams epi;
    int m, n;
    int num_kb;
    int tiles_m, tiles_n, num_tiles;
    unsigned idesc;
    DeviceStatus *status;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false when the CTA is aborting (this wait timed out, or another one did).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          DeviceStatus *status, int where)
{
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if (*abort_flag != 0) {
            return false;
        }
        if ((++spins & 0x3ffu) == 0u && global_timer_ns() - t0 > kWaitLimitNs) {
            *abort_flag = 1;
            if (atomicCAS(&status->code, kErrNone, kErrTimeout) == kErrNone) {
                status->where = where;
                status->block = static_cast<int>(blockIdx.x);
            }
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *tmap, uint64_t *bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major tile stored as rows of 128 bytes with the 128-byte swizzle:
// 8-row groups are 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

template <int kKind>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    if (kKind == KUDNN_B200_F32) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
            "}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

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

template <int kKind, int kBN>
__global__ void __launch_bounds__(kTcThreads, 1)
    tc_linear_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const TcParams p)
{
    constexpr int kBBytes = kBN * kStageRowBytes;
    constexpr int kStageBytes = kABytes + kBBytes;
    constexpr int kStages = (kBN == 256) ? 4 : 6;
    constexpr int kTmemCols = 2 * kBN;
    constexpr int kElemsPerRow = (kKind == KUDNN_B200_F32) ? 32 : 64;  // elements per 128-byte k-block row

    extern __shared__ unsigned char smem_dyn[];
    // stage buffers need 1024-byte alignment for the 128-byte swizzle pattern
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023u) &
                                                            ~static_cast<uintptr_t>(1023u));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes);
    uint64_t *full_bar = bars;
    uint64_t *empty_bar = bars + kStages;
    uint64_t *tmem_full = bars + 2 * kStages;
    uint64_t *tmem_empty = bars + 2 * kStages + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 4);
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
            mbar_init(tmem_empty + a, 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
            int stage = 0;
            uint32_t phase = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < p.num_tiles; tile += gridDim.x) {
                const int per_group = kGroupM * p.tiles_n;
                const int group = tile / per_group;
                const int first_m = group * kGroupM;
                const int gsize = (p.tiles_m - first_m < kGroupM) ? (p.tiles_m - first_m) : kGroupM;
                const int in_group = tile - group * per_group;
                const int tm = first_m + in_group % gsize;
                const int tn = in_group / gsize;
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (!mbar_wait(empty_bar + stage, phase ^ 1u, abort_flag, p.status, 1)) {
                        alive = false;
                        break;
                    }
                    unsigned char *sa = smem + stage * kStageBytes;
                    unsigned char *sb = sa + kABytes;
                    mbar_expect_tx(full_bar + stage, kStageBytes);
                    tma_load_2d(sa, &tmap_a, full_bar + stage, kb * kElemsPerRow, tm * kBM);
                    tma_load_2d(sb, &tmap_b, full_bar + stage, kb * kElemsPerRow, tn * kBN);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < p.num_tiles; tile += gridDim.x) {
                if (!mbar_wait(tmem_empty + acc, acc_phase ^ 1u, abort_flag, p.status, 2)) {
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kBN);
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (!mbar_wait(full_bar + stage, phase, abort_flag, p.status, 3)) {
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
                        umma<kKind>(tmem_d, adesc + static_cast<uint64_t>(2 * ks), bdesc + static_cast<uint64_t>(2 * ks),
                                    p.idesc, (kb | ks) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar + stage);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!alive) {
                    break;
                }
                umma_commit(tmem_full + acc);
                acc ^= 1;
                if (acc == 0) {
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;  // TMEM lanes this warp may touch: [32 * quarter, 32 * quarter + 32)
        const int row_in_tile = quarter * 32 + lane;
        const EpiParams &e = p.epi;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
            const int per_group = kGroupM * p.tiles_n;
            const int group = tile / per_group;
            const int first_m = group * kGroupM;
            const int gsize = (p.tiles_m - first_m < kGroupM) ? (p.tiles_m - first_m) : kGroupM;
            const int in_group = tile - group * per_group;
            const int tm = first_m + in_group % gsize;
            const int tn = in_group / gsize;
            if (!mbar_wait(tmem_full + acc, acc_phase, abort_flag, p.status, 4)) {
                break;
            }
            tc_fence_after();
            const long long mi = static_cast<long long>(tm) * kBM + row_in_tile;
            const bool row_ok = mi < p.m;
            const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(acc * kBN);
#pragma unroll 1
            for (int chunk = 0; chunk < kBN / 32; ++chunk) {
                const long long nc = static_cast<long long>(tn) * kBN + chunk * 32;
                if (nc >= p.n) {
                    break;  // warp-uniform: the rest of the tile is out of range
                }
                uint32_t raw[32];
                tmem_load_32(taddr_row + static_cast<uint32_t>(chunk * 32), raw);
                if (row_ok) {
#pragma unroll
                    for (int j8 = 0; j8 < 4; ++j8) {
                        const long long ni = nc + j8 * 8;
                        const int valid = (p.n - ni >= 8) ? 8 : static_cast<int>(p.n - ni);
                        if (valid <= 0) {
                            break;
                        }
                        const bool full8 = valid == 8;
                        float bias[8], res[8], cold[8], vc[8], vo[8];
                        const long long ic = mi * e.c_sm + ni * e.c_sn;
                        const bool c_vec = full8 && vec_ok(e.c, e.c_dtype, ic, e.c_sn);
                        if (e.has_bias) {
                            const long long ib = mi * e.bias_sm + ni * e.bias_sn;
                            load8(e.bias, e.bias_dtype, ib, e.bias_sn, full8 && vec_ok(e.bias, e.bias_dtype, ib, e.bias_sn),
                                  valid, bias);
                        }
                        if (e.beta != 0.0f && e.c != nullptr) {
                            load8(e.c, e.c_dtype, ic, e.c_sn, c_vec, valid, cold);
                        }
                        long long io = 0;
                        bool o_vec = false;
                        if (e.res_op != KUDNN_B200_RES_NONE) {
                            const long long ir = mi * e.res_sm + ni * e.res_sn;
                            load8(e.res, e.res_dtype, ir, e.res_sn, full8 && vec_ok(e.res, e.res_dtype, ir, e.res_sn),
                                  valid, res);
                            io = mi * e.out_sm + ni * e.out_sn;
                            o_vec = full8 && vec_ok(e.out, e.out_dtype, io, e.out_sn);
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const EpiResult r =
                                finish_element(e, __uint_as_float(raw[j8 * 8 + j]), (e.beta != 0.0f) ? cold[j] : 0.0f,
                                               e.has_bias ? bias[j] : 0.0f,
                                               (e.res_op != KUDNN_B200_RES_NONE) ? res[j] : 0.0f);
                            vc[j] = r.c;
                            vo[j] = r.out;
                        }
                        if (e.c != nullptr) {
                            store8(e.c, e.c_dtype, ic, e.c_sn, c_vec, valid, vc);
                        }
                        if (e.res_op != KUDNN_B200_RES_NONE) {
                            store8(e.out, e.out_dtype, io, e.out_sn, o_vec, valid, vo);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(tmem_empty + acc);
            }
            acc ^= 1;
            if (acc == 0) {
                acc_phase ^= 1u;
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag != 0) {
        // give copies and MMAs that were already issued time to land before the memory is handed back
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
            __nanosleep(1000);
        }
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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
                          long long ld_elems, int box_rows)
{
    const int es = dtype_size(kind);
    const CUtensorMapDataType dt = (kind == KUDNN_B200_F32)   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : (kind == KUDNN_B200_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
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

unsigned make_idesc(int kind, int n)
{
    const unsigned fmt = (kind == KUDNN_B200_F32) ? 2u : (kind == KUDNN_B200_BF16 ? 1u : 0u);
    unsigned d = 0;
    d |= 1u << 4;                              // accumulator format: fp32
    d |= fmt << 7;                             // A format
    d |= fmt << 10;                            // B format
    d |= static_cast<unsigned>(n >> 3) << 17;  // N / 8
    d |= static_cast<unsigned>(kBM >> 4) << 24;  // M / 16
    return d;                                  // both operands K-major, no negation, dense
}

template <int kKind, int kBN>
cudaError_t launch_one(const TcPlan &plan, const TcParams &p, cudaStream_t stream)
{
    auto kernel = tc_linear_kernel<kKind, kBN>;
    cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem_bytes));
    if (e != cudaSuccess) {
        return e;
    }
    CUtensorMap ta, tb;
    std::memcpy(&ta, plan.tmap_a, sizeof(ta));
    std::memcpy(&tb, plan.tmap_b, sizeof(tb));
    kernel<<<plan.grid, kTcThreads, plan.smem_bytes, stream>>>(ta, tb, p);
    return cudaGetLastError();
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

cudaError_t tc_make_plan(const TcOperands &ops, long long m, long long n, int sm_count, TcPlan *plan)
{
    static_assert(sizeof(CUtensorMap) <= 128, "tensor map storage too small");
    if (!tc_available()) {
        return cudaErrorNotSupported;
    }
    const long long tiles_m = (m + kBM - 1) / kBM;
    const long long tiles256 = tiles_m * ((n + 255) / 256);
    const int bn = (tiles256 >= sm_count || n > 128 * 64) ? 256 : 128;
    const long long tiles = tiles_m * ((n + bn - 1) / bn);
    if (tiles > (1ll << 30)) {
        return cudaErrorInvalidValue;
    }
    plan->block_n = bn;
    plan->stages = (bn == 256) ? 4 : 6;
    plan->grid = static_cast<int>(tiles < sm_count ? tiles : sm_count);
    plan->smem_bytes = static_cast<size_t>(plan->stages) * (kABytes + bn * kStageRowBytes) + 1024 + 256;
    CUtensorMap ta, tb;
    cudaError_t e = encode_kmajor(&ta, ops.a, ops.kind, m, ops.k_total, ops.lda, kBM);
    if (e != cudaSuccess) {
        return e;
    }
    e = encode_kmajor(&tb, ops.b, ops.kind, n, ops.k_total, ops.ldb, bn);
    if (e != cudaSuccess) {
        return e;
    }
    std::memcpy(plan->tmap_a, &ta, sizeof(ta));
    std::memcpy(plan->tmap_b, &tb, sizeof(tb));
    return cudaSuccess;
}

cudaError_t launch_tc(const TcOperands &ops, const TcPlan &plan, const EpiParams &epi, long long m, long long n,
                      DeviceStatus *status, cudaStream_t stream)
{
    TcParams p;
    p.epi = epi;
    p.m = static_cast<int>(m);
    p.n = static_cast<int>(n);
    const int elems_per_row = kStageRowBytes / dtype_size(ops.kind);
    p.num_kb = static_cast<int>((ops.k_total + elems_per_row - 1) / elems_per_row);
    p.tiles_m = static_cast<int>((m + kBM - 1) / kBM);
    p.tiles_n = static_cast<int>((n + plan.block_n - 1) / plan.block_n);
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.idesc = make_idesc(ops.kind, plan.block_n);
    p.status = status;
    if (plan.block_n == 256) {
        switch (ops.kind) {
            case KUDNN_B200_F32:
                return launch_one<KUDNN_B200_F32, 256>(plan, p, stream);
            case KUDNN_B200_F16:
                return launch_one<KUDNN_B200_F16, 256>(plan, p, stream);
            default:
                return launch_one<KUDNN_B200_BF16, 256>(plan, p, stream);
        }
    }
    switch (ops.kind) {
        case KUDNN_B200_F32:
            return launch_one<KUDNN_B200_F32, 128>(plan, p, stream);
        case KUDNN_B200_F16:
            return launch_one<KUDNN_B200_F16, 128>(plan, p, stream);
        default:
            return launch_one<KUDNN_B200_BF16, 128>(plan, p, stream);
    }
}

}  // namespace kb
