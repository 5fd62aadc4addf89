// Decode-shaped Linear (m <= 16, 16-bit types) with the weights streamed through a shared-memory ring.
//
// Why a second streaming kernel: the register-fed kernels of gemv.cu read the weights 64 bytes per row per warp
// instruction (the mma.sync fragment layout wants 8 different rows in one load), and HBM delivers about 12 % less for
// that access shape than for long runs.  Here one producer thread copies whole row segments (4 KiB contiguous per row)
// with bulk asynchronous copies into a ring of stages, completion on mbarriers; the fragment layout is produced on
// the way out of shared memory by ldmatrix, so the access shape in HBM no longer depends on it, and the bytes in
// flight per SM (the ring, up to 160 KiB) no longer depend on registers.
//
// Shape of one CTA (672 threads, one CTA per SM, persistent):
//   warp 16     producer: one lane issues, per stage, 8 bulk copies (8 weight rows x 2048 k) and waits on the stage's
//               "empty" barrier before reusing it
//   warps 0-15  consumers: every warp owns the same 32-wide k blocks of every stage (blocks w, w+16, w+32, w+48), so
//               its activation fragments never change and live in registers for the whole kernel; per stage it
//               issues 4 ldmatrix.x4 + 8 mma.sync.m16n8k16 (activations as the 16-row operand, fp32 accumulate)
//   warps 17-20 finishing warps: combine the consumers' partial tiles and run the fused epilogue
// A group of 8 weight rows spans `spg` consecutive stages (k chunk of the CTA / 2048).  When a group is complete the
// 16 consumer warps leave their 16x8 partial tiles in one of four shared-memory buffers (mbarrier hand-off, no
// CTA-wide barrier) and go on; finishing warp b owns buffer b, adds the 16 tiles in warp order and runs the epilogue,
// so the latency of the epilogue's loads, stores and atomics stays off the streaming warps.
// Work is the flat sequence of (group, stage) pairs, cut into equal contiguous ranges, one per CTA, so every SM
// streams the same number of bytes.  A group cut by a range boundary, or by the split of K across CTAs that keeps
// the activation fragments within the register budget, is finished through the slot/counter scheme of gemv.cu:
// partial tiles in global scratch, an arrival counter per group, the last arrival adds the slots in slot order.
//
// Waits on mbarriers are bounded; after a time-out the CTA records it, stops waiting and runs to its end (the
// results of that launch are then undefined and the host reports KUDNN_B200_TIMEOUT).
#include "kernels.cuh"

#include <algorithm>
#include <cstdlib>

namespace kb {

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kFinishWarps = 4;                   // warps that combine the consumers' partial tiles and run the epilogue
constexpr int kRingThreads = 32 * (kConsumerWarps + 1 + kFinishWarps);
constexpr int kStageK = 2048;                     // k elements per row per stage
constexpr int kRowPitch = kStageK * 2 + 16;       // bytes; the 16-byte skew keeps the 8 rows of an ldmatrix on distinct banks
constexpr int kStageBytes = 8 * kRowPitch;
constexpr int kRingStages = 5;
constexpr int kBlocksPerWarp = kStageK / 32 / kConsumerWarps;  // 4
constexpr long long kRingWaitCycles = 4000000000ll;

struct RingParams {
    const unsigned short *x;  // [m, k]
    const unsigned short *w;  // [n, k]
    long long x_ld, w_ld;
    int m, n, k;
    int ksplit, kc;           // K chunks over CTAs, chunk length
    int ctas_per_chunk;
    long long range;          // (group, stage) pairs per CTA
    long long total;          // pairs per chunk = groups * spg
    float *partials;          // [group][ksplit * 2][128]
    unsigned int *counters;   // [group]
    DeviceStatus *status;
    EpiParams epi;
};

__device__ __forceinline__ uint32_t ring_smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool ring_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(ring_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait; once any wait of the CTA has timed out, all of them return at once.
__device__ __forceinline__ void ring_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, DeviceStatus *status,
                                          int where)
{
    if (*abort_flag != 0) {
        return;
    }
    for (int i = 0; i < 64; ++i) {
        if (ring_try_wait(bar, parity)) {
            return;
        }
    }
    const long long t0 = clock64();
    unsigned spins = 0;
    while (!ring_try_wait(bar, parity)) {
        if ((++spins & 0x3fu) == 0u) {
            if (*abort_flag != 0) {
                return;
            }
            if (clock64() - t0 > kRingWaitCycles) {
                *abort_flag = 1;
                if (atomicCAS(&status->code, kErrNone, kErrTimeout) == kErrNone) {
                    status->where = where;
                    status->block = static_cast<int>(blockIdx.x);
                }
                return;
            }
        }
    }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

template <int kDtype>
__device__ __forceinline__ void ring_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1)
{
    if (kDtype == KUDNN_B200_BF16) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

__device__ __forceinline__ unsigned ld_x_pair(const unsigned short *x, long long ld, int row, int m, int k, int kmax)
{
    if (row >= m || k >= kmax) {
        return 0u;
    }
    return *reinterpret_cast<const unsigned *>(x + static_cast<long long>(row) * ld + k);
}

template <int kDtype, bool kRows16, int kSpg>
__global__ void __launch_bounds__(kRingThreads, 1) gemv_ring_kernel(const RingParams p)
{
    extern __shared__ __align__(128) unsigned char ring_smem[];
    unsigned char *stages = ring_smem;
    float *red = reinterpret_cast<float *>(ring_smem + kRingStages * kStageBytes);  // [kFinishWarps][16 warps][128]
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(red + kFinishWarps * kConsumerWarps * 128);
    uint64_t *empty_bar = full_bar + kRingStages;
    uint64_t *red_full = empty_bar + kRingStages;
    uint64_t *red_empty = red_full + kFinishWarps;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(red_empty + kFinishWarps);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kRingStages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ring_smem_u32(full_bar + s)), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ring_smem_u32(empty_bar + s)), "r"(kConsumerWarps)
                         : "memory");
        }
        for (int b = 0; b < kFinishWarps; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ring_smem_u32(red_full + b)), "r"(kConsumerWarps)
                         : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ring_smem_u32(red_empty + b)), "r"(1) : "memory");
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const int chunk = blockIdx.x % p.ksplit;
    const int cta = blockIdx.x / p.ksplit;
    const int kc0 = chunk * p.kc;
    const long long f0 = static_cast<long long>(cta) * p.range;
    const long long f1 = (f0 + p.range < p.total) ? f0 + p.range : p.total;

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer
        if (lane == 0 && cta < p.ctas_per_chunk) {
            int stage = 0;
            uint32_t phase = 0;
            for (long long f = f0; f < f1; ++f) {
                const long long group = f / kSpg;
                const int s = static_cast<int>(f - group * kSpg);
                ring_wait(empty_bar + stage, phase ^ 1u, abort_flag, p.status, 11);
                const long long row0 = group * 8;
                const int valid_rows = (p.n - row0 >= 8) ? 8 : static_cast<int>(p.n - row0);
                const uint32_t bar = ring_smem_u32(full_bar + stage);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                             "r"(static_cast<uint32_t>(valid_rows * kStageK * 2))
                             : "memory");
                unsigned char *dst = stages + stage * kStageBytes;
                const unsigned short *src = p.w + row0 * p.w_ld + kc0 + s * kStageK;
                for (int r = 0; r < valid_rows; ++r) {
                    asm volatile(
                        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                            ring_smem_u32(dst + r * kRowPitch)),
                        "l"(src + r * p.w_ld), "r"(static_cast<uint32_t>(kStageK * 2)), "r"(bar)
                        : "memory");
                }
                if (++stage == kRingStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp < kConsumerWarps && cta < p.ctas_per_chunk) {
        // ------------------------------------------------------------------ consumers
        const int gid = lane >> 2, tig = lane & 3;
        // activation fragments of this warp's k blocks, for every stage of a group
        constexpr int kRegsPerStep = kRows16 ? 4 : 2;
        unsigned xf[kSpg][kBlocksPerWarp][2][kRegsPerStep];
#pragma unroll
        for (int s = 0; s < kSpg; ++s) {
#pragma unroll
            for (int j = 0; j < kBlocksPerWarp; ++j) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int kb = kc0 + s * kStageK + (warp + kConsumerWarps * j) * 32 + h * 16 + tig * 2;
                    if (kRows16) {
                        xf[s][j][h][0] = ld_x_pair(p.x, p.x_ld, gid, p.m, kb, p.k);
                        xf[s][j][h][1] = ld_x_pair(p.x, p.x_ld, gid + 8, p.m, kb, p.k);
                        xf[s][j][h][2] = ld_x_pair(p.x, p.x_ld, gid, p.m, kb + 8, p.k);
                        xf[s][j][h][3] = ld_x_pair(p.x, p.x_ld, gid + 8, p.m, kb + 8, p.k);
                    } else {
                        xf[s][j][h][0] = ld_x_pair(p.x, p.x_ld, gid, p.m, kb, p.k);
                        xf[s][j][h][1] = ld_x_pair(p.x, p.x_ld, gid, p.m, kb + 8, p.k);
                    }
                }
            }
        }
        // ldmatrix row address of this lane inside a stage: matrix (lane / 8) covers k [8 * (lane / 8), +8) of a block
        const uint32_t lane_off = static_cast<uint32_t>((lane & 7) * kRowPitch + (lane >> 3) * 16);
        int stage = 0;
        uint32_t phase = 0;
        long long flushes = 0;
        // one accumulator per k block of a stage: four independent mma chains instead of one of depth eight
        float acc[kBlocksPerWarp][4];
#pragma unroll
        for (int j = 0; j < kBlocksPerWarp; ++j) {
            acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
        }
        for (long long f = f0; f < f1; ++f) {
            const long long group = f / kSpg;
            const int s = static_cast<int>(f - group * kSpg);
            ring_wait(full_bar + stage, phase, abort_flag, p.status, 12);
            const uint32_t base = ring_smem_u32(stages + stage * kStageBytes) + lane_off;
#pragma unroll
            for (int ss = 0; ss < kSpg; ++ss) {
                if (ss == s) {
#pragma unroll
                    for (int j = 0; j < kBlocksPerWarp; ++j) {
                        unsigned b0, b1, b2, b3;
                        ldmatrix_x4(base + static_cast<uint32_t>((warp + kConsumerWarps * j) * 64), b0, b1, b2, b3);
                        if (kRows16) {
                            ring_mma<kDtype>(acc[j], xf[ss][j][0][0], xf[ss][j][0][1], xf[ss][j][0][2], xf[ss][j][0][3], b0, b1);
                            ring_mma<kDtype>(acc[j], xf[ss][j][1][0], xf[ss][j][1][1], xf[ss][j][1][2], xf[ss][j][1][3], b2, b3);
                        } else {
                            ring_mma<kDtype>(acc[j], xf[ss][j][0][0], 0u, xf[ss][j][0][1], 0u, b0, b1);
                            ring_mma<kDtype>(acc[j], xf[ss][j][1][0], 0u, xf[ss][j][1][1], 0u, b2, b3);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ring_smem_u32(empty_bar + stage)) : "memory");
            }
            if (++stage == kRingStages) {
                stage = 0;
                phase ^= 1u;
            }
            if (s == kSpg - 1 || f == f1 - 1) {
                // the CTA's share of this group is complete: hand the partial tile to a finishing warp
                const int b = static_cast<int>(flushes % kFinishWarps);
                const uint32_t use = static_cast<uint32_t>(flushes / kFinishWarps);
                ring_wait(red_empty + b, (use & 1u) ^ 1u, abort_flag, p.status, 13);
                float *mine = red + (b * kConsumerWarps + warp) * 128;
                float tot[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    tot[e] = (acc[0][e] + acc[1][e]) + (acc[2][e] + acc[3][e]);
                }
                *reinterpret_cast<float4 *>(mine + lane * 4) = make_float4(tot[0], tot[1], tot[2], tot[3]);
#pragma unroll
                for (int j = 0; j < kBlocksPerWarp; ++j) {
                    acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
                }
                __syncwarp();
                if (lane == 0) {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ring_smem_u32(red_full + b)) : "memory");
                }
                ++flushes;
            }
        }
    } else if (warp > kConsumerWarps && cta < p.ctas_per_chunk && f0 < f1) {
        // ------------------------------------------------------------------ finishing warps
        const int b = warp - kConsumerWarps - 1;  // buffer b carries the CTA's flushes b, b + 4, b + 8, ...
        const int gid = lane >> 2, tig = lane & 3;
        const long long group0 = f0 / kSpg;
        const long long count = (f1 - 1) / kSpg - group0 + 1;
        for (long long i = b; i < count; i += kFinishWarps) {
            const long long group = group0 + i;
            const uint32_t use = static_cast<uint32_t>(i / kFinishWarps);
            ring_wait(red_full + b, use & 1u, abort_flag, p.status, 14);
            float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int w2 = 0; w2 < kConsumerWarps; ++w2) {
                const float4 v = *reinterpret_cast<const float4 *>(red + (b * kConsumerWarps + w2) * 128 + lane * 4);
                sum[0] += v.x;
                sum[1] += v.y;
                sum[2] += v.z;
                sum[3] += v.w;
            }
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ring_smem_u32(red_empty + b)) : "memory");
            }
            // which CTAs of this chunk touch the group, and is it whole here?
            const long long g_first = group * kSpg, g_last = g_first + kSpg - 1;
            const int c_first = static_cast<int>(g_first / p.range), c_last = static_cast<int>(g_last / p.range);
            const int pieces = c_last - c_first + 1;
            bool finish = (p.ksplit == 1 && pieces == 1);
            if (!finish) {
                const int slot = chunk * 2 + (cta - c_first);
                float *unit = p.partials + group * (static_cast<long long>(p.ksplit) * 2 * 128);
                *reinterpret_cast<float4 *>(unit + slot * 128 + lane * 4) = make_float4(sum[0], sum[1], sum[2], sum[3]);
                __threadfence();
                __syncwarp();
                unsigned old = 0u;
                if (lane == 0) {
                    old = atomicAdd(p.counters + group, 1u);
                }
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old == static_cast<unsigned>(p.ksplit * pieces - 1)) {
                    __threadfence();
                    sum[0] = sum[1] = sum[2] = sum[3] = 0.0f;
                    for (int c = 0; c < p.ksplit; ++c) {
                        for (int j = 0; j < pieces; ++j) {
                            const float4 v = __ldcg(reinterpret_cast<const float4 *>(unit + (c * 2 + j) * 128 + lane * 4));
                            sum[0] += v.x;
                            sum[1] += v.y;
                            sum[2] += v.z;
                            sum[3] += v.w;
                        }
                    }
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
                    const long long ni = group * 8 + tig * 2 + (e & 1);
                    if (mi < p.m && ni < p.n) {
                        epilogue_scalar(p.epi, sum[e], mi, ni);
                    }
                }
            }
        }
    }
    __syncthreads();
    if (*abort_flag != 0) {
        // copies already issued may still be landing in this CTA's shared memory
        const long long t0 = clock64();
        while (clock64() - t0 < 400000ll) {
            __nanosleep(1000);
        }
    }
}

}  // namespace

// Decides whether the ring kernel can take a problem, and how it is cut.  Pure host arithmetic.
bool gemv_ring_plan(const LinearProblem &pr, int sm_count, RingPlan *plan)
{
    if (pr.batch_count != 1 || pr.m < 1 || pr.m > 16 || pr.a_dtype != pr.b_dtype || pr.a_dtype == KUDNN_B200_F32) {
        return false;
    }
    if (pr.a_sk != 1 || pr.b_sk != 1 || pr.k % kStageK != 0 || pr.n < 8 || pr.n > (1 << 28)) {
        return false;
    }
    if ((pr.m > 1 && pr.a_sm % 8 != 0) || pr.b_sn % 8 != 0 || (reinterpret_cast<uintptr_t>(pr.a) & 15u) != 0 ||
        (reinterpret_cast<uintptr_t>(pr.b) & 15u) != 0) {
        return false;
    }
    const bool rows16 = pr.m > 8;
    int max_spg = rows16 ? 2 : 4;  // register budget of the activation fragments
    if (const char *env = std::getenv("KUDNN_B200_RING_MAX_SPG")) {
        const int v = std::atoi(env);
        if (v == 1 || v == 2 || v == 4) {
            max_spg = std::min(max_spg, v);
        }
    }
    const int stages_in_k = static_cast<int>(pr.k / kStageK);
    int ksplit = 1;
    while (stages_in_k / ksplit > max_spg) {
        ksplit *= 2;
    }
    if (stages_in_k % ksplit != 0) {
        return false;
    }
    const int spg = stages_in_k / ksplit;
    if (spg != 1 && spg != 2 && spg != 4) {
        return false;
    }
    const long long groups = (pr.n + 7) / 8;
    int ctas_per_chunk = std::max(sm_count / ksplit, 1);
    ctas_per_chunk = static_cast<int>(std::min<long long>(ctas_per_chunk, groups));  // a range covers at least one group
    const long long total = groups * spg;
    const long long range = (total + ctas_per_chunk - 1) / ctas_per_chunk;
    ctas_per_chunk = static_cast<int>((total + range - 1) / range);
    plan->rows16 = rows16;
    plan->ksplit = ksplit;
    plan->spg = spg;
    plan->kc = spg * kStageK;
    plan->ctas_per_chunk = ctas_per_chunk;
    plan->grid = ctas_per_chunk * ksplit;
    plan->range = range;
    plan->total = total;
    plan->smem_bytes = static_cast<size_t>(kRingStages) * kStageBytes + kFinishWarps * kConsumerWarps * 128 * sizeof(float) +
                       (2 * kRingStages + 2 * kFinishWarps) * sizeof(uint64_t) + 16;
    plan->partial_floats = groups * ksplit * 2 * 128;
    plan->counter_count = groups;
    return true;
}

namespace {

template <int kDtype, bool kRows16, int kSpg>
cudaError_t launch_ring_one(const RingParams &p, const RingPlan &plan, cudaStream_t stream)
{
    auto kernel = gemv_ring_kernel<kDtype, kRows16, kSpg>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem_bytes));
    if (e != cudaSuccess) {
        return e;
    }
    kernel<<<plan.grid, kRingThreads, plan.smem_bytes, stream>>>(p);
    return cudaGetLastError();
}

template <int kDtype>
cudaError_t launch_ring_dtype(const RingParams &p, const RingPlan &plan, cudaStream_t stream)
{
    if (plan.rows16) {
        return plan.spg == 1 ? launch_ring_one<kDtype, true, 1>(p, plan, stream) : launch_ring_one<kDtype, true, 2>(p, plan, stream);
    }
    switch (plan.spg) {
        case 1:
            return launch_ring_one<kDtype, false, 1>(p, plan, stream);
        case 2:
            return launch_ring_one<kDtype, false, 2>(p, plan, stream);
        default:
            return launch_ring_one<kDtype, false, 4>(p, plan, stream);
    }
}

}  // namespace

cudaError_t launch_gemv_ring(const LinearProblem &pr, const RingPlan &plan, const GemvWorkspace &ws, DeviceStatus *status,
                             cudaStream_t stream)
{
    if (ws.partial_floats < plan.partial_floats || ws.counter_count < plan.counter_count) {
        return cudaErrorInvalidValue;
    }
    RingParams p;
    p.x = static_cast<const unsigned short *>(pr.a);
    p.w = static_cast<const unsigned short *>(pr.b);
    p.x_ld = pr.a_sm;
    p.w_ld = pr.b_sn;
    p.m = static_cast<int>(pr.m);
    p.n = static_cast<int>(pr.n);
    p.k = static_cast<int>(pr.k);
    p.ksplit = plan.ksplit;
    p.kc = plan.kc;
    p.ctas_per_chunk = plan.ctas_per_chunk;
    p.range = plan.range;
    p.total = plan.total;
    p.partials = ws.partials;
    p.counters = ws.counters;
    p.status = status;
    p.epi = pr.epi;
    return pr.a_dtype == KUDNN_B200_F16 ? launch_ring_dtype<KUDNN_B200_F16>(p, plan, stream)
                                        : launch_ring_dtype<KUDNN_B200_BF16>(p, plan, stream);
}

}  // namespace kb
