// Thin wrappers over the sm_100a instructions the tensor-core kernels are built from: mbarriers, TMA tile loads,
// tcgen05 matrix multiply-accumulate with its shared-memory / instruction descriptors, tensor-memory loads.
// Every wait is bounded (see mbar_wait).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace kb {

constexpr long long kDefaultWaitLimitCycles = 4000000000ll;  // about two seconds at 2 GHz

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
// Bounded wait.  Returns false when the CTA is aborting (this wait timed out, or another one did).  The limit is
// counted on the SM's own cycle counter, which is cheap to read; the wall-clock timer is not (a read costs about a
// microsecond, which would sit on the critical path of every k-block).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          DeviceStatus *status, int where, long long limit)
{
#pragma unroll 1
    for (int i = 0; i < 128; ++i) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
    }
    const long long t0 = clock64();
    unsigned spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((++spins & 0x3fu) == 0u) {
            if (*abort_flag != 0) {
                return false;
            }
            if (clock64() - t0 > limit) {
                *abort_flag = 1;
                if (atomicCAS(&status->code, kErrNone, kErrTimeout) == kErrNone) {
                    status->where = where;
                    status->block = static_cast<int>(blockIdx.x);
                }
                return false;
            }
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

// the same with a third coordinate (batch entry); the box is one entry deep
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *tmap, uint64_t *bar, int x, int y, int z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// ---- CTA pair (cluster of two, tcgen05 cta_group::2) -----------------------------------------------------------
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_smem_addr, uint32_t rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
    return remote;
}

// Tile load of one CTA of a pair: the data lands in this CTA's shared memory, the bytes are counted on the leader's
// barrier (a cluster address).  No data is shared between CTAs by this copy.
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *tmap, uint32_t leader_bar_addr, int x,
                                                 int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
        "[%2];" ::"r"(smem_u32(smem_dst)),
        "l"(tmap), "r"(leader_bar_addr), "r"(x), "r"(y)
        : "memory");
}

// Arrival on a barrier of another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
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
    if (kKind == KUDNN_B200_S8) {
        // 8-bit integer operands (signedness of each in the instruction descriptor), 32-bit integer accumulator,
        // 32 elements of K per instruction
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
            "}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else if (kKind == KUDNN_B200_F32) {
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

// One MMA over both CTAs of a pair: M = 256 (128 rows of A and of the accumulator per CTA), B = N / 2 rows from
// each CTA's shared memory at the same offsets.  Issued by one thread of the leader CTA.
template <int kKind>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    if (kKind == KUDNN_B200_S8) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
            "}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else if (kKind == KUDNN_B200_F32) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
            "}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Completion of all MMAs issued so far by this thread, signalled on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"(static_cast<unsigned short>(3))
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 8 consecutive fp32 columns of this thread's TMEM lane; completion is awaited separately so that the next load
// can be in flight while the current values are processed
__device__ __forceinline__ void tmem_load_8_issue(uint32_t taddr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
// Waits for the outstanding TMEM loads.  The registers of the load are passed through so that the compiler cannot
// schedule a use of them ahead of the wait.
__device__ __forceinline__ void tmem_load_wait(uint32_t (&r)[8])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
                 :
                 : "memory");
}

// Instruction descriptor of tcgen05.mma kind::f16 / kind::tf32: fp32 accumulator, both operands K-major, dense.
inline unsigned make_idesc(int kind, int n, int m_rows)
{
    const unsigned fmt = (kind == KUDNN_B200_F32) ? 2u : (kind == KUDNN_B200_BF16 ? 1u : 0u);
    unsigned d = 0;
    d |= 1u << 4;                              // accumulator format: fp32
    d |= fmt << 7;                             // A format
    d |= fmt << 10;                            // B format
    d |= static_cast<unsigned>(n >> 3) << 17;  // N / 8
    d |= static_cast<unsigned>(m_rows >> 4) << 24;  // M / 16 (256 for a CTA pair)
    return d;
}

// Instruction descriptor of tcgen05.mma kind::i8: 32-bit integer accumulator, operands signed or unsigned 8-bit
// integers, both K-major, dense, no saturation.
inline unsigned make_idesc_i8(bool a_signed, bool b_signed, int n, int m_rows)
{
    unsigned d = 0;
    d |= 2u << 4;                               // accumulator format: s32
    d |= (a_signed ? 1u : 0u) << 7;             // A format: 0 = u8, 1 = s8
    d |= (b_signed ? 1u : 0u) << 10;            // B format
    d |= static_cast<unsigned>(n >> 3) << 17;   // N / 8
    d |= static_cast<unsigned>(m_rows >> 4) << 24;  // M / 16
    return d;
}

}  // namespace kb
