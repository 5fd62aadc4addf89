// C-ABI of the Linear(+post-op) path: descriptor validation, handle life cycle, weight pre-packing, kernel
// selection and launch, host-pointer staging.  The entry points are declared in include/kudnn_b200.h.
#include "kernels.cuh"

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <vector>

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int fail_cuda(cudaError_t e, const char *what)
{
    (void)cudaGetLastError();
    if (e == cudaErrorMemoryAllocation) {
        return fail(KUDNN_B200_ALLOC_FAILED, "%s: device allocation failed", what);
    }
    return fail(KUDNN_B200_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
}

bool is_float_dtype(int dt)
{
    return dt == KUDNN_B200_F32 || dt == KUDNN_B200_F16 || dt == KUDNN_B200_BF16;
}

bool is_int8_dtype(int dt)
{
    return dt == KUDNN_B200_S8 || dt == KUDNN_B200_U8;
}

long long batch_extent(const kudnn_b200_linear_desc &d, int i)
{
    return d.batch[i] > 0 ? d.batch[i] : 1;
}

// number of elements spanned by a tensor with the given extents and strides
long long span_elems(long long e0, long long s0, long long e1, long long s1, const kudnn_b200_linear_desc &d,
                     const int64_t sb[3])
{
    long long last = (e0 - 1) * s0 + (e1 - 1) * s1;
    for (int i = 0; i < 3; ++i) {
        last += (batch_extent(d, i) - 1) * sb[i];
    }
    return last + 1;
}

// Test hook (kudnn_b200_debug_fail_allocation): the n-th device allocation the library attempts from now on fails
// with cudaErrorMemoryAllocation instead of reaching cudaMalloc; negative = off.
std::atomic<int> g_alloc_fail_countdown{-1};

cudaError_t device_malloc(void **ptr, size_t bytes)
{
    int left = g_alloc_fail_countdown.load();
    while (left >= 0) {
        if (g_alloc_fail_countdown.compare_exchange_weak(left, left - 1)) {
            if (left == 0) {
                *ptr = nullptr;
                return cudaErrorMemoryAllocation;
            }
            break;
        }
    }
    return cudaMalloc(ptr, bytes);
}

struct DeviceBuffer {
    void *ptr = nullptr;
    size_t bytes = 0;
    cudaError_t reserve(size_t need)
    {
        if (need <= bytes) {
            return cudaSuccess;
        }
        if (ptr != nullptr) {
            cudaFree(ptr);
            ptr = nullptr;
            bytes = 0;
        }
        cudaError_t e = device_malloc(&ptr, need);
        if (e == cudaSuccess) {
            bytes = need;
        }
        return e;
    }
    void release()
    {
        if (ptr != nullptr) {
            cudaFree(ptr);
        }
        ptr = nullptr;
        bytes = 0;
    }
};

}  // namespace

namespace kb {

// Lets the other translation units of the library report through kudnn_b200_last_error().
int set_last_error(int code, const char *message)
{
    return fail(code, "%s", message);
}

}  // namespace kb

struct kudnn_b200_linear_s {
    kudnn_b200_linear_desc d;
    int forced_kernel = KUDNN_B200_KERNEL_AUTO;
    int last_kernel = 0;
    int last_launches = 0;
    int device = -1;
    int sm_count = 0;
    std::mutex lock;

    // output mirrors (kudnn_b200_linear_set_mirrors): device pointers to further copies of c / out
    int n_mirrors = 0;
    void *c_mirror[kb::kMaxMirrors] = {};
    void *out_mirror[kb::kMaxMirrors] = {};
    void *c_multicast = nullptr, *out_multicast = nullptr;  // the outputs as mapped through a multicast object, or null
    bool packed_int8 = false;  // the packed weights are the 8-bit values themselves, K-major (decode-shaped W8A16)

    // device-side waits: limit in SM cycles (0 = default) and the timeout test hook (kudnn_b200_debug_set_wait)
    long long wait_limit = 0;
    int skip_kblock = -1;
    cudaStream_t counters_stream = nullptr;  // stream the arrival counters were last zeroed or used on
    bool counters_dirty = false;             // a kernel that gave up may have left arrival counters set

    DeviceBuffer status;        // kb::DeviceStatus
    DeviceBuffer gemv_partials, gemv_counters;
    DeviceBuffer a_scratch;     // per-call packed activations
    DeviceBuffer b_scratch;     // per-call packed weights (when not pre-packed)
    DeviceBuffer b_packed;      // pre-packed weights
    DeviceBuffer b_blocked;     // decode-shaped handles: the weights once more in 8-row x 64-k blocks
    DeviceBuffer q_scratch;     // 8-bit weights widened to fp16 per call (when not pre-packed)
    DeviceBuffer stage[6];      // host-pointer staging: a, b, c, bias, res, out

    // pre-pack state
    const void *packed_key = nullptr;  // the caller's weight pointer the packed copy stands for
    const void *packed_ptr = nullptr;  // what the tensor-core kernel reads (b_packed.ptr, or the caller's device
                                       // pointer when that already is K-major); fp32: the three TF32 planes
    const void *packed_raw = nullptr;  // K-major copy in the original element type (what the other kernels read)
    long long packed_ld = 0, packed_ktotal = 0;
    long long blocked_kpad = 0;  // columns per row of b_blocked (k rounded up to 256); 0 = no blocked copy

    // tensor-map cache of the last tensor-core launch
    kb::TcPlan tc_plan;
    const void *plan_a = nullptr, *plan_b = nullptr;
    long long plan_m = 0;
    bool plan_staging = false;
    bool plan_valid = false;

    // kudnn_b200_linear_run_sharded: one child primitive per shard, each on its own device with its own copy (or
    // slab) of the weights
    struct Shard {
        kudnn_b200_linear_s *child = nullptr;
        int device = 0;
        long long begin = 0, count = 0;
        const void *weights = nullptr;  // host pointer the child's packed weights were made from
        DeviceBuffer buf[5];            // column shards: a, bias slice, c slab, res slab, out slab
    };
    std::vector<Shard> shards;
    int shard_mode = -1, shard_count = 0;

    // host-pointer path: copy-in, compute and copy-out streams with one event pair per row chunk
    static constexpr int kMaxChunks = 16;
    bool pipe_ready = false;
    cudaStream_t pipe_stream[3] = {nullptr, nullptr, nullptr};
    cudaEvent_t pipe_in[kMaxChunks], pipe_done[kMaxChunks];
};

namespace {

using Handle = kudnn_b200_linear_s;

int ensure_device(Handle *h)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(KUDNN_B200_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    }
    if (h->device == dev) {
        return KUDNN_B200_OK;
    }
    if (h->device != -1) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "handle was first used on device %d, current device is %d", h->device, dev);
    }
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) {
        return fail_cuda(e, "cudaGetDeviceProperties");
    }
    if (prop.major != 10) {
        return fail(KUDNN_B200_NO_DEVICE, "device %d is sm_%d%d; this library carries sm_100a code only", dev, prop.major,
                    prop.minor);
    }
    e = h->status.reserve(sizeof(kb::DeviceStatus));
    if (e != cudaSuccess) {
        return fail_cuda(e, "status block");
    }
    e = cudaMemset(h->status.ptr, 0, sizeof(kb::DeviceStatus));
    if (e != cudaSuccess) {
        return fail_cuda(e, "status block");
    }
    h->device = dev;
    h->sm_count = prop.multiProcessorCount;
    return KUDNN_B200_OK;
}

void fill_epi(const kudnn_b200_linear_desc &d, const kudnn_b200_linear_args &a, kb::EpiParams *e)
{
    e->c = a.c;
    e->bias = a.bias;
    e->res = a.res;
    e->out = a.out;
    e->c_sm = d.c_sm;
    e->c_sn = d.c_sn;
    e->bias_sm = d.bias_sm;
    e->bias_sn = d.bias_sn;
    e->res_sm = d.res_sm;
    e->res_sn = d.res_sn;
    e->out_sm = d.out_sm;
    e->out_sn = d.out_sn;
    e->alpha = a.alpha;
    e->beta = a.beta;
    if (d.a_dtype == KUDNN_B200_BF16 && d.b_dtype == KUDNN_B200_BF16 && d.c_dtype == KUDNN_B200_BF16 && d.has_bias == 0) {
        // the reference's bias-free bf16 product is cblas_bgemm, which takes its scalars as bf16
        // (src/dnn/src/kudnn_gemm.cpp:222-226)
        e->alpha = __bfloat162float(__float2bfloat16_rn(a.alpha));
        e->beta = __bfloat162float(__float2bfloat16_rn(a.beta));
    }
    e->gamma = a.gamma;
    e->act_alpha = d.act_alpha;
    e->c_dtype = d.c_dtype;
    e->bias_dtype = d.bias_dtype;
    e->res_dtype = d.res_dtype;
    e->out_dtype = d.out_dtype;
    e->has_bias = d.has_bias;
    // d.reserved != 0: the weights of this (internal) descriptor were widened from 8 bits
    e->half_chain = (d.c_dtype == KUDNN_B200_F16 && d.a_dtype == KUDNN_B200_F16 && d.b_dtype == KUDNN_B200_F16 &&
                     d.reserved == 0 && (d.has_bias == 0 || d.bias_dtype == KUDNN_B200_F16))
                        ? 1
                        : 0;
    e->act = d.act;
    e->res_op = d.res_op;
    e->m = static_cast<int>(d.m);
    e->n = static_cast<int>(d.n);
    e->n_mirrors = 0;
    e->use_multicast = 0;
    e->c_mc_delta = e->out_mc_delta = 0;
}

void fill_problem(const kudnn_b200_linear_desc &d, const kudnn_b200_linear_args &a, kb::LinearProblem *p)
{
    p->a = a.a;
    p->b = a.b;
    p->m = d.m;
    p->n = d.n;
    p->k = d.k;
    p->a_sm = d.a_sm;
    p->a_sk = d.a_sk;
    p->b_sk = d.b_sk;
    p->b_sn = d.b_sn;
    p->a_dtype = d.a_dtype;
    p->b_dtype = d.b_dtype;
    fill_epi(d, a, &p->epi);
    p->batch.n1 = batch_extent(d, 1);
    p->batch.n2 = batch_extent(d, 2);
    for (int i = 0; i < 3; ++i) {
        p->batch.a_sb[i] = d.a_sb[i];
        p->batch.b_sb[i] = d.b_sb[i];
        p->batch.c_sb[i] = d.c_sb[i];
        p->batch.bias_sb[i] = d.bias_sb[i];
        p->batch.res_sb[i] = d.res_sb[i];
        p->batch.out_sb[i] = d.out_sb[i];
    }
    p->batch_count = batch_extent(d, 0) * batch_extent(d, 1) * batch_extent(d, 2);
}

bool aligned16(const void *p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// K-major with rows that start on 16-byte boundaries: usable by TMA and by the streaming kernels as is
bool kmajor_ready(const void *p, int dtype, long long s_row, long long s_k, long long rows)
{
    const int vec = 16 / kb::dtype_size(dtype);
    return s_k == 1 && aligned16(p) && (rows == 1 || s_row % vec == 0);
}

long long round_up(long long v, long long a)
{
    return (v + a - 1) / a * a;
}

// Packs the weight operand into `buf`.  16-bit: [n, k_pad] K-major.  fp32: rows of [hi | lo | hi | raw] planes
// (raw only when with_raw), each k_pad floats; the tensor-core kernel contracts over the first three.
int pack_weights(Handle *h, const void *b_dev, DeviceBuffer *buf, bool with_raw, cudaStream_t stream, long long *ld,
                 long long *ktotal, const void **raw, int *launches)
{
    const kudnn_b200_linear_desc &d = h->d;
    if (d.b_dtype == KUDNN_B200_F32) {
        const long long k_pad = round_up(d.k, 32);
        const long long pitch = (with_raw ? 4 : 3) * k_pad;
        cudaError_t e = buf->reserve(static_cast<size_t>(d.n) * pitch * sizeof(float));
        if (e != cudaSuccess) {
            return fail_cuda(e, "packed weights");
        }
        float *base = static_cast<float *>(buf->ptr);
        e = kb::launch_split_tf32(b_dev, d.n, d.k, d.b_sn, d.b_sk, base, pitch, k_pad, 1, stream);
        if (e != cudaSuccess) {
            return fail_cuda(e, "weight split kernel");
        }
        *launches += 1;
        *raw = nullptr;
        if (with_raw) {
            e = kb::launch_pack_kmajor(b_dev, KUDNN_B200_F32, d.n, d.k, d.b_sn, d.b_sk, base + 3 * k_pad, KUDNN_B200_F32,
                                       pitch, k_pad, stream);
            if (e != cudaSuccess) {
                return fail_cuda(e, "weight pack kernel");
            }
            *launches += 1;
            *raw = base + 3 * k_pad;
        }
        *ld = pitch;
        *ktotal = 3 * k_pad;
    } else {
        const long long k_pad = round_up(d.k, 8);
        const long long pitch = k_pad;
        cudaError_t e = buf->reserve(static_cast<size_t>(d.n) * pitch * 2);
        if (e != cudaSuccess) {
            return fail_cuda(e, "packed weights");
        }
        // 8-bit weights are widened to fp16 here (exact), the type of the activations they meet
        e = kb::launch_pack_kmajor(b_dev, d.b_dtype, d.n, d.k, d.b_sn, d.b_sk, buf->ptr,
                                   is_int8_dtype(d.b_dtype) ? KUDNN_B200_F16 : d.b_dtype, pitch, k_pad, stream);
        if (e != cudaSuccess) {
            return fail_cuda(e, "weight pack kernel");
        }
        *launches += 1;
        *ld = pitch;
        *ktotal = d.k;
        *raw = buf->ptr;
    }
    return KUDNN_B200_OK;
}

// A batched problem whose weights are shared by all batch entries and whose other tensors are laid out so that
// (batch index, row) is one linear row index is a 2-D problem with batch * m rows: [B, S, K] x [K, N], the way a
// linear layer is applied to a batch of sequences.  Writes that 2-D descriptor and returns true when this holds.
bool collapse_batch(const kudnn_b200_linear_desc &d, kudnn_b200_linear_desc *out)
{
    const long long e[3] = {batch_extent(d, 0), batch_extent(d, 1), batch_extent(d, 2)};
    const long long nb = e[0] * e[1] * e[2];
    if (nb == 1 || nb * d.m > 0x7fffffffll) {
        return false;
    }
    for (int i = 0; i < 3; ++i) {
        if (e[i] > 1 && d.b_sb[i] != 0) {
            return false;
        }
    }
    auto linear_rows = [&](const int64_t sb[3], long long s_m) {
        long long expect = d.m * s_m;  // stride of the innermost batch dimension
        for (int i = 2; i >= 0; --i) {
            if (e[i] > 1 && sb[i] != expect) {
                return false;
            }
            expect *= e[i];
        }
        return true;
    };
    if (!linear_rows(d.a_sb, d.a_sm) || !linear_rows(d.c_sb, d.c_sm)) {
        return false;
    }
    if (d.has_bias != 0 && !linear_rows(d.bias_sb, d.bias_sm)) {
        return false;
    }
    if (d.res_op != KUDNN_B200_RES_NONE && (!linear_rows(d.res_sb, d.res_sm) || !linear_rows(d.out_sb, d.out_sm))) {
        return false;
    }
    *out = d;
    out->m = nb * d.m;
    for (int i = 0; i < 3; ++i) {
        out->batch[i] = 1;
        out->a_sb[i] = out->b_sb[i] = out->c_sb[i] = out->bias_sb[i] = out->res_sb[i] = out->out_sb[i] = 0;
    }
    return true;
}

// Split-K scratch of the streaming kernels: partial sums and arrival counters, grown on demand.
int reserve_gemv_scratch(Handle *h, long long partial_floats, long long counter_count, cudaStream_t stream,
                         kb::GemvWorkspace *ws)
{
    cudaError_t e = h->gemv_partials.reserve(static_cast<size_t>(partial_floats) * sizeof(float));
    if (e != cudaSuccess) {
        return fail_cuda(e, "streaming-kernel scratch");
    }
    const bool grow = h->gemv_counters.bytes < static_cast<size_t>(counter_count) * sizeof(unsigned);
    if (grow) {
        e = h->gemv_counters.reserve(static_cast<size_t>(counter_count) * sizeof(unsigned));
        if (e != cudaSuccess) {
            return fail_cuda(e, "streaming-kernel counters");
        }
    }
    // The kernels leave the counters at zero, so they are cleared only when they are new, after a run that gave
    // up, or when the caller moved to another stream (the clear is then ordered in front of this launch).
    if (grow || h->counters_dirty || h->counters_stream != stream) {
        e = cudaMemsetAsync(h->gemv_counters.ptr, 0, h->gemv_counters.bytes, stream);
        if (e != cudaSuccess) {
            return fail_cuda(e, "streaming-kernel counters");
        }
        h->counters_dirty = false;
        h->counters_stream = stream;
    }
    ws->partials = static_cast<float *>(h->gemv_partials.ptr);
    ws->counters = static_cast<unsigned *>(h->gemv_counters.ptr);
    ws->partial_floats = static_cast<long long>(h->gemv_partials.bytes / sizeof(float));
    ws->counter_count = static_cast<long long>(h->gemv_counters.bytes / sizeof(unsigned));
    return KUDNN_B200_OK;
}

// `d_in` is the handle's descriptor, or a copy of it restricted to a block of rows (host-pointer pipeline)
int run_device(Handle *h, const kudnn_b200_linear_desc &d_in, const kudnn_b200_linear_args &args, cudaStream_t stream)
{
    kudnn_b200_linear_desc collapsed;
    const kudnn_b200_linear_desc &d = collapse_batch(d_in, &collapsed) ? collapsed : d_in;
    if (args.a == nullptr || args.b == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run: a and b must not be null");
    }
    if ((d.has_bias != 0) != (args.bias != nullptr)) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run: bias pointer does not match the descriptor");
    }
    if (d.res_op != KUDNN_B200_RES_NONE) {
        if (args.res == nullptr || args.out == nullptr) {
            return fail(KUDNN_B200_BAD_ARGUMENTS, "run: res and out must not be null for this descriptor");
        }
    } else if (args.c == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run: c must not be null");
    }
    if (args.beta != 0.0f && args.c == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run: beta != 0 needs c");
    }
    int rc = ensure_device(h);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }

    // ---- 8-bit integer product, exact 32-bit sums: tcgen05 kind::i8 for problems worth a tensor-core launch (2-D,
    // alpha = 1, beta = 0), the general integer kernel for the rest
    if (d.c_dtype == KUDNN_B200_S32) {
        kb::LinearProblem ip;
        fill_problem(d, args, &ip);
        const int forced_int = h->forced_kernel;
        const bool packed = h->packed_key != nullptr && h->packed_key == args.b;
        if (packed) {
            ip.b = h->packed_raw;  // the caller's pointer (possibly host memory) is only the key
            ip.b_sk = 1;
            ip.b_sn = h->packed_ld;
        }
        const bool int_worth = static_cast<double>(d.m) * d.n * d.k >= 1.0e6 * 8 && d.k >= 32;
        if (ip.batch_count == 1 && args.alpha == 1.0f && args.beta == 0.0f && ip.epi.n_mirrors == 0 && kb::tc_available() &&
            (forced_int == KUDNN_B200_KERNEL_TC || (forced_int == KUDNN_B200_KERNEL_AUTO && int_worth))) {
            kb::TcOperands ops;
            ops.kind = KUDNN_B200_S8;
            ops.a_signed = d.a_dtype == KUDNN_B200_S8 ? 1 : 0;
            ops.b_signed = d.b_dtype == KUDNN_B200_S8 ? 1 : 0;
            ops.k_total = d.k;
            int launches = 0;
            const long long k_pad = round_up(d.k, 16);
            if (packed) {
                ops.b = h->packed_ptr;
                ops.ldb = h->packed_ld;
            } else if (kmajor_ready(args.b, d.b_dtype, d.b_sn, d.b_sk, d.n)) {
                ops.b = args.b;
                ops.ldb = d.b_sn;
            } else {
                cudaError_t e = h->b_scratch.reserve(static_cast<size_t>(d.n) * k_pad);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "packed weights");
                }
                e = kb::launch_pack_kmajor(args.b, d.b_dtype, d.n, d.k, d.b_sn, d.b_sk, h->b_scratch.ptr, d.b_dtype, k_pad, k_pad, stream);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "weight pack kernel");
                }
                launches += 1;
                ops.b = h->b_scratch.ptr;
                ops.ldb = k_pad;
            }
            if (kmajor_ready(args.a, d.a_dtype, d.a_sm, d.a_sk, d.m)) {
                ops.a = args.a;
                ops.lda = d.a_sm;
            } else {
                cudaError_t e = h->a_scratch.reserve(static_cast<size_t>(d.m) * k_pad);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "packed activations");
                }
                e = kb::launch_pack_kmajor(args.a, d.a_dtype, d.m, d.k, d.a_sm, d.a_sk, h->a_scratch.ptr, d.a_dtype, k_pad, k_pad, stream);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "activation pack kernel");
                }
                launches += 1;
                ops.a = h->a_scratch.ptr;
                ops.lda = k_pad;
            }
            if (!(h->plan_valid && h->plan_a == ops.a && h->plan_b == ops.b && h->plan_m == d.m && !h->plan_staging)) {
                cudaError_t e = kb::tc_make_plan(ops, d.m, d.n, h->sm_count, false, &h->tc_plan);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "tensor map encoding");
                }
                h->plan_a = ops.a;
                h->plan_b = ops.b;
                h->plan_m = d.m;
                h->plan_staging = false;
                h->plan_valid = true;
            }
            cudaError_t e = kb::launch_tc(ops, h->tc_plan, ip.epi, d.m, d.n, static_cast<kb::DeviceStatus *>(h->status.ptr), stream,
                                          h->wait_limit, -1, nullptr);
            if (e != cudaSuccess) {
                return fail_cuda(e, "tensor-core kernel launch");
            }
            h->last_kernel = KUDNN_B200_KERNEL_TC;
            h->last_launches = launches + 1;
            return KUDNN_B200_OK;
        }
        if (forced_int == KUDNN_B200_KERNEL_TC) {
            return fail(KUDNN_B200_UNSUPPORTED, "the tensor-core kernel takes 2-D integer products with alpha = 1 and beta = 0 only");
        }
        if (ip.batch_count > 65535) {
            return fail(KUDNN_B200_UNSUPPORTED, "more than 65535 batch entries");
        }
        cudaError_t e = kb::launch_int_gemm(ip, stream);
        if (e != cudaSuccess) {
            return fail_cuda(e, "integer kernel launch");
        }
        h->last_kernel = KUDNN_B200_KERNEL_SIMT;
        h->last_launches = 1;
        return KUDNN_B200_OK;
    }
    // ---- fp16 activations with 8-bit weights: the weights are widened to fp16, K-major, once when they are pre-packed
    // or else per call, and the problem continues as fp16 x fp16 whose fp16 result is rounded once
    if (is_int8_dtype(d.b_dtype)) {
        const bool nb1 = batch_extent(d, 0) * batch_extent(d, 1) * batch_extent(d, 2) == 1;
        // where the 8-bit weights are read from: the K-major copy (or the caller's own buffer) that pre-packing of a
        // decode-shaped primitive left, else the caller's pointer with its strides
        const bool packed8 = h->packed_int8 && h->packed_key != nullptr && h->packed_key == args.b;
        const void *w8 = packed8 ? h->packed_raw : args.b;
        const long long w8_sn = packed8 ? h->packed_ld : d.b_sn, w8_sk = packed8 ? 1 : d.b_sk;
        // decode shapes: the streaming kernels read the 8-bit weights as they are, half the bytes of their fp16 form
        const int forced8 = h->forced_kernel;
        if (nb1 && d.m <= 16 && h->n_mirrors == 0 &&
            (forced8 == KUDNN_B200_KERNEL_AUTO || forced8 == KUDNN_B200_KERNEL_GEMV_FMA || forced8 == KUDNN_B200_KERNEL_GEMV_MMA)) {
            kudnn_b200_linear_desc d8 = d;
            d8.b_sn = w8_sn;
            d8.b_sk = w8_sk;
            kudnn_b200_linear_args a8 = args;
            a8.b = w8;
            kb::LinearProblem p8;
            fill_problem(d8, a8, &p8);
            kb::GemvPlan plan8;
            if (kb::gemv_plan(p8, h->sm_count, forced8, &plan8)) {
                kb::GemvWorkspace ws8;
                rc = reserve_gemv_scratch(h, plan8.partial_floats, plan8.counter_count, stream, &ws8);
                if (rc != KUDNN_B200_OK) {
                    return rc;
                }
                cudaError_t e = kb::launch_gemv(p8, plan8, ws8, stream);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "streaming kernel launch");
                }
                h->last_kernel = plan8.kernel;
                h->last_launches = 1;
                return KUDNN_B200_OK;
            }
        }
        kudnn_b200_linear_desc dq = d;
        dq.b_dtype = KUDNN_B200_F16;
        dq.reserved = 1;
        dq.b_sk = 1;
        kudnn_b200_linear_args aq = args;
        if (!packed8 && h->packed_key != nullptr && h->packed_key == args.b) {
            dq.b_sn = h->packed_ld;  // the packed state stands for args.b: the inner call finds it by the same key
        } else {
            if (!nb1) {
                return fail(KUDNN_B200_UNSUPPORTED, "8-bit weights of batched problems are not supported");
            }
            const long long k_pad = round_up(d.k, 8);
            cudaError_t e = h->q_scratch.reserve(static_cast<size_t>(d.n) * k_pad * 2);
            if (e != cudaSuccess) {
                return fail_cuda(e, "widened weights");
            }
            e = kb::launch_pack_kmajor(w8, d.b_dtype, d.n, d.k, w8_sn, w8_sk, h->q_scratch.ptr, KUDNN_B200_F16, k_pad, k_pad, stream);
            if (e != cudaSuccess) {
                return fail_cuda(e, "weight widening kernel");
            }
            dq.b_sn = k_pad;
            aq.b = h->q_scratch.ptr;
        }
        const int rcq = run_device(h, dq, aq, stream);
        if (rcq == KUDNN_B200_OK && aq.b != args.b) {
            h->last_launches += 1;
        }
        return rcq;
    }

    kb::LinearProblem pr;
    fill_problem(d, args, &pr);
    if (h->n_mirrors > 0) {
        // the kernels address a mirror as "primary pointer + byte distance", which also survives batch offsets
        pr.epi.n_mirrors = h->n_mirrors;
        for (int i = 0; i < h->n_mirrors; ++i) {
            pr.epi.c_delta[i] = args.c != nullptr ? static_cast<char *>(h->c_mirror[i]) - static_cast<char *>(args.c) : 0;
            pr.epi.out_delta[i] =
                args.out != nullptr ? static_cast<char *>(h->out_mirror[i]) - static_cast<char *>(args.out) : 0;
            if ((args.c != nullptr && (h->c_mirror[i] == nullptr || pr.epi.c_delta[i] % 16 != 0)) ||
                (d.res_op != KUDNN_B200_RES_NONE && (h->out_mirror[i] == nullptr || pr.epi.out_delta[i] % 16 != 0))) {
                return fail(KUDNN_B200_BAD_ARGUMENTS,
                            "run: every mirror needs a pointer for each output that is written, at a distance from "
                            "the primary output that is a multiple of 16 bytes");
            }
        }
        if (h->c_multicast != nullptr || h->out_multicast != nullptr) {
            const long long dc = args.c != nullptr && h->c_multicast != nullptr
                                     ? static_cast<char *>(h->c_multicast) - static_cast<char *>(args.c) : 0;
            const long long dout = args.out != nullptr && h->out_multicast != nullptr
                                       ? static_cast<char *>(h->out_multicast) - static_cast<char *>(args.out) : 0;
            const bool c_ok = args.c == nullptr || (h->c_multicast != nullptr && dc % 16 == 0);
            const bool out_ok = d.res_op == KUDNN_B200_RES_NONE || (h->out_multicast != nullptr && dout % 16 == 0);
            if (!c_ok || !out_ok) {
                return fail(KUDNN_B200_BAD_ARGUMENTS,
                            "run: the multicast mapping needs a pointer for each output that is written, 16-byte congruent "
                            "with the primary output");
            }
            pr.epi.use_multicast = 1;
            pr.epi.c_mc_delta = dc;
            pr.epi.out_mc_delta = dout;
        }
    }
    int launches = 0;
    const int forced = h->forced_kernel;
    const bool use_packed = (h->packed_key != nullptr && h->packed_key == args.b);
    const bool two_d = pr.batch_count == 1;
    if (use_packed) {
        // every kernel reads the packed copy; the caller's pointer (possibly host memory) is only the key
        pr.b = h->packed_raw;
        pr.b_sk = 1;
        pr.b_sn = h->packed_ld;
        if (h->blocked_kpad > 0) {
            pr.b_blocked = h->b_blocked.ptr;
            pr.b_blocked_kpad = h->blocked_kpad;
        }
    }

    // ---- streaming kernels (m <= 16)
    if (two_d && d.m <= 16 &&
        (forced == KUDNN_B200_KERNEL_AUTO || forced == KUDNN_B200_KERNEL_GEMV_FMA || forced == KUDNN_B200_KERNEL_GEMV_MMA)) {
        kb::GemvPlan plan;
        if (kb::gemv_plan(pr, h->sm_count, forced, &plan)) {
            kb::GemvWorkspace ws;
            rc = reserve_gemv_scratch(h, plan.partial_floats, plan.counter_count, stream, &ws);
            if (rc != KUDNN_B200_OK) {
                return rc;
            }
            cudaError_t e = kb::launch_gemv(pr, plan, ws, stream);
            if (e != cudaSuccess) {
                return fail_cuda(e, "streaming kernel launch");
            }
            h->last_kernel = plan.kernel;
            h->last_launches = 1;
            return KUDNN_B200_OK;
        }
        if (forced != KUDNN_B200_KERNEL_AUTO) {
            return fail(KUDNN_B200_UNSUPPORTED, "the forced streaming kernel cannot take this problem");
        }
    }

    // ---- tensor-core kernel
    // Batched problems take it too: the batch entry is a third coordinate of the tile scheduler and of the tensor
    // maps.  An operand is read in place when its matrices are K-major and its batch entries lie a single stride
    // apart (or are one shared matrix); anything else is packed first, all entries in one launch.
    const long long nb = pr.batch_count;
    const bool tc_types = d.a_dtype == d.b_dtype;
    const bool tc_worth = static_cast<double>(d.m) * d.n * d.k * static_cast<double>(nb) >= 1.0e6 * 8 && d.k >= 32;
    const bool tc_batch_ok = nb == 1 || (nb <= 65535 && pr.epi.n_mirrors == 0);
    if (tc_batch_ok && tc_types && (forced == KUDNN_B200_KERNEL_TC || (forced == KUDNN_B200_KERNEL_AUTO && tc_worth))) {
        if (!kb::tc_available()) {
            if (forced == KUDNN_B200_KERNEL_TC) {
                return fail(KUDNN_B200_UNSUPPORTED, "tensor-core kernel unavailable: %s", kb::tc_unavailable_reason());
            }
        } else {
            kb::TcOperands ops;
            ops.kind = d.a_dtype;
            ops.batch = nb;
            const bool f32 = d.a_dtype == KUDNN_B200_F32;
            const int es = kb::dtype_size(d.a_dtype);
            const long long e3[3] = {batch_extent(d, 0), batch_extent(d, 1), batch_extent(d, 2)};
            // single stride between consecutive flat batch entries, 0 when all entries share the matrix; false when
            // the three batch strides do not reduce to one
            auto flat_stride = [&](const int64_t sb[3], long long *stride) {
                long long unit = -1;
                long long inner = 1;
                bool any = false, all_zero = true;
                for (int i = 2; i >= 0; --i) {
                    if (e3[i] > 1) {
                        any = true;
                        if (sb[i] != 0) {
                            all_zero = false;
                        }
                    }
                }
                if (!any || all_zero) {
                    *stride = 0;
                    return true;
                }
                for (int i = 2; i >= 0; --i) {
                    if (e3[i] > 1) {
                        if (sb[i] == 0 || sb[i] % inner != 0) {
                            return false;
                        }
                        const long long u = sb[i] / inner;
                        if (unit >= 0 && u != unit) {
                            return false;
                        }
                        unit = u;
                        inner *= e3[i];
                    }
                }
                *stride = unit;
                return (unit * es) % 16 == 0;
            };
            auto pack_batch = [&](const int64_t sb[3], bool shared, long long dst_batch) {
                kb::PackBatch pb;
                pb.count = shared ? 1 : nb;
                pb.n1 = e3[1];
                pb.n2 = e3[2];
                for (int i = 0; i < 3; ++i) {
                    pb.sb[i] = (e3[i] > 1) ? sb[i] : 0;
                }
                pb.dst_batch = dst_batch;
                return pb;
            };
            auto all_shared = [&](const int64_t sb[3]) {
                for (int i = 0; i < 3; ++i) {
                    if (e3[i] > 1 && sb[i] != 0) {
                        return false;
                    }
                }
                return true;
            };
            // weights
            long long bstride = 0;
            if (use_packed) {
                ops.b = h->packed_ptr;
                ops.ldb = h->packed_ld;
                ops.k_total = h->packed_ktotal;
            } else if (!f32 && kmajor_ready(args.b, d.b_dtype, d.b_sn, d.b_sk, d.n) && flat_stride(d.b_sb, &bstride)) {
                ops.b = args.b;
                ops.ldb = d.b_sn;
                ops.k_total = d.k;
                ops.b_bstride = bstride;
            } else if (nb == 1) {
                long long ld = 0, kt = 0;
                const void *raw = nullptr;
                rc = pack_weights(h, args.b, &h->b_scratch, false, stream, &ld, &kt, &raw, &launches);
                if (rc != KUDNN_B200_OK) {
                    return rc;
                }
                ops.b = h->b_scratch.ptr;
                ops.ldb = ld;
                ops.k_total = kt;
            } else {
                const bool shared = all_shared(d.b_sb);
                const long long k_pad = round_up(d.k, f32 ? 32 : 8);
                const long long pitch = f32 ? 3 * k_pad : k_pad;
                const long long per = d.n * pitch;
                cudaError_t e = h->b_scratch.reserve(static_cast<size_t>(shared ? 1 : nb) * per * es);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "packed weights");
                }
                const kb::PackBatch pb = pack_batch(d.b_sb, shared, per);
                e = f32 ? kb::launch_split_tf32(args.b, d.n, d.k, d.b_sn, d.b_sk, static_cast<float *>(h->b_scratch.ptr), pitch,
                                                k_pad, 1, stream, &pb)
                        : kb::launch_pack_kmajor(args.b, d.b_dtype, d.n, d.k, d.b_sn, d.b_sk, h->b_scratch.ptr, d.b_dtype, pitch,
                                                 k_pad, stream, &pb);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "weight pack kernel");
                }
                launches += 1;
                ops.b = h->b_scratch.ptr;
                ops.ldb = pitch;
                ops.k_total = f32 ? 3 * k_pad : d.k;
                ops.b_bstride = shared ? 0 : per;
            }
            // activations
            long long astride = 0;
            if (!f32 && kmajor_ready(args.a, d.a_dtype, d.a_sm, d.a_sk, d.m) && flat_stride(d.a_sb, &astride)) {
                ops.a = args.a;
                ops.lda = d.a_sm;
                ops.a_bstride = astride;
            } else {
                const bool shared = all_shared(d.a_sb);
                const long long k_pad = round_up(d.k, f32 ? 32 : 8);
                const long long pitch = f32 ? 3 * k_pad : k_pad;
                const long long per = d.m * pitch;
                cudaError_t e = h->a_scratch.reserve(static_cast<size_t>(shared ? 1 : nb) * per * es);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "packed activations");
                }
                const kb::PackBatch pb = pack_batch(d.a_sb, shared, per);
                e = f32 ? kb::launch_split_tf32(args.a, d.m, d.k, d.a_sm, d.a_sk, static_cast<float *>(h->a_scratch.ptr), pitch,
                                                k_pad, 0, stream, &pb)
                        : kb::launch_pack_kmajor(args.a, d.a_dtype, d.m, d.k, d.a_sm, d.a_sk, h->a_scratch.ptr, d.a_dtype, pitch,
                                                 k_pad, stream, &pb);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "activation pack kernel");
                }
                launches += 1;
                ops.a = h->a_scratch.ptr;
                ops.lda = pitch;
                ops.a_bstride = shared ? 0 : per;
            }
            const bool staging = pr.epi.n_mirrors > 0;
            if (nb > 1 || !(h->plan_valid && h->plan_a == ops.a && h->plan_b == ops.b && h->plan_m == d.m && h->plan_staging == staging)) {
                cudaError_t e = kb::tc_make_plan(ops, d.m, d.n, h->sm_count, staging, &h->tc_plan);
                if (e != cudaSuccess) {
                    return fail_cuda(e, "tensor map encoding");
                }
                h->plan_a = ops.a;
                h->plan_b = ops.b;
                h->plan_m = d.m;
                h->plan_staging = staging;
                h->plan_valid = nb == 1;
                if (const char *dbg = std::getenv("KUDNN_B200_DEBUG")) {
                    if (*dbg != '\0' && *dbg != '0') {
                        std::fprintf(stderr, "kudnn_b200: tensor-core plan batch=%lld m=%lld n=%lld k=%lld: tile %s x %d, %d stages, "
                                             "grid %d, k splits %d, narrow tail from tile %d, %zu bytes of shared memory\n",
                                     nb, static_cast<long long>(d.m), static_cast<long long>(d.n), static_cast<long long>(d.k),
                                     h->tc_plan.pair ? "256 (CTA pair)" : "128", h->tc_plan.block_n, h->tc_plan.stages,
                                     h->tc_plan.grid, h->tc_plan.splits, h->tc_plan.pair ? h->tc_plan.narrow_from : -1, h->tc_plan.smem_bytes);
                    }
                }
            }
            cudaError_t e = kb::launch_tc(ops, h->tc_plan, pr.epi, d.m, d.n,
                                          static_cast<kb::DeviceStatus *>(h->status.ptr), stream, h->wait_limit,
                                          h->skip_kblock, &pr.batch);
            if (e != cudaSuccess) {
                return fail_cuda(e, "tensor-core kernel launch");
            }
            h->last_kernel = KUDNN_B200_KERNEL_TC;
            h->last_launches = launches + 1;
            return KUDNN_B200_OK;
        }
    } else if (forced == KUDNN_B200_KERNEL_TC) {
        return fail(KUDNN_B200_UNSUPPORTED, "the tensor-core kernel takes problems with equal input types only");
    }

    // ---- general kernel
    if (pr.batch_count > 65535) {
        return fail(KUDNN_B200_UNSUPPORTED, "more than 65535 batch entries");
    }
    cudaError_t e = kb::launch_simt(pr, stream);
    if (e != cudaSuccess) {
        return fail_cuda(e, "general kernel launch");
    }
    h->last_kernel = KUDNN_B200_KERNEL_SIMT;
    h->last_launches = 1;
    return KUDNN_B200_OK;
}

// Host-pointer execution of a large 2-D problem as a pipeline over blocks of rows: while block i is computed, block
// i+1 is copied in and block i-1 is copied out, each on its own stream, so a call costs about the slowest of the
// three instead of their sum.  Rows of a, c, res and out must be contiguous along their second dimension.
bool pipeline_applies(const kudnn_b200_linear_desc &d, const kudnn_b200_linear_args &args)
{
    if (batch_extent(d, 0) * batch_extent(d, 1) * batch_extent(d, 2) != 1 || d.m < 1024 || args.beta != 0.0f) {
        return false;
    }
    if (d.a_sk != 1 || d.a_sm < d.k || d.c_sn != 1 || d.c_sm < d.n) {
        return false;
    }
    if (d.res_op != KUDNN_B200_RES_NONE && (d.res_sn != 1 || d.res_sm < d.n || d.out_sn != 1 || d.out_sm < d.n)) {
        return false;
    }
    if (d.has_bias && d.bias_sm != 0 && (d.bias_sn != 1 || d.bias_sm < d.n)) {
        return false;
    }
    // Only page-locked buffers overlap: with pageable memory the copy back of block i holds the host until it is
    // done, so block i+1 would be copied in only afterwards and the blocks would run strictly one after another,
    // each paying its own launch set-up.  Such callers get the single-shot path.
    auto pinned = [](const void *p) {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        return attr.type == cudaMemoryTypeHost;
    };
    if (!pinned(args.a) || !pinned(d.res_op != KUDNN_B200_RES_NONE ? args.out : args.c)) {
        return false;
    }
    const char *off = std::getenv("KUDNN_B200_HOST_PIPELINE");
    return !(off != nullptr && std::strcmp(off, "0") == 0);
}

int ensure_pipeline(Handle *h)
{
    if (h->pipe_ready) {
        return KUDNN_B200_OK;
    }
    for (auto &st : h->pipe_stream) {
        cudaError_t e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            return fail_cuda(e, "host pipeline streams");
        }
    }
    for (int i = 0; i < Handle::kMaxChunks; ++i) {
        cudaError_t e = cudaEventCreateWithFlags(&h->pipe_in[i], cudaEventDisableTiming);
        if (e == cudaSuccess) {
            e = cudaEventCreateWithFlags(&h->pipe_done[i], cudaEventDisableTiming);
        }
        if (e != cudaSuccess) {
            return fail_cuda(e, "host pipeline events");
        }
    }
    h->pipe_ready = true;
    return KUDNN_B200_OK;
}

int read_status(Handle *h)
{
    kb::DeviceStatus st;
    cudaError_t e = cudaMemcpy(&st, h->status.ptr, sizeof(st), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        return fail_cuda(e, "status read");
    }
    if (st.code != kb::kErrNone) {
        cudaMemset(h->status.ptr, 0, sizeof(st));
        h->counters_dirty = true;
        return fail(KUDNN_B200_TIMEOUT, "device-side wait gave up (site %d, block %d)", st.where, st.block);
    }
    return KUDNN_B200_OK;
}

int run_host_pipelined(Handle *h, const kudnn_b200_linear_args &args)
{
    const kudnn_b200_linear_desc &d = h->d;
    int rc = ensure_pipeline(h);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }
    cudaStream_t s_in = h->pipe_stream[0], s_run = h->pipe_stream[1], s_out = h->pipe_stream[2];
    const bool has_res = d.res_op != KUDNN_B200_RES_NONE;
    const size_t es_a = kb::dtype_size(d.a_dtype), es_c = kb::dtype_size(d.c_dtype);
    const size_t es_bias = kb::dtype_size(d.bias_dtype), es_res = kb::dtype_size(d.res_dtype), es_out = kb::dtype_size(d.out_dtype);
    const size_t bytes_a = (static_cast<size_t>(d.m - 1) * d.a_sm + d.k) * es_a;
    const size_t bytes_c = (static_cast<size_t>(d.m - 1) * d.c_sm + d.n) * es_c;
    const size_t bytes_b = static_cast<size_t>(span_elems(d.k, d.b_sk, d.n, d.b_sn, d, d.b_sb)) * kb::dtype_size(d.b_dtype);
    const size_t bytes_bias = d.has_bias ? static_cast<size_t>(span_elems(d.m, d.bias_sm, d.n, d.bias_sn, d, d.bias_sb)) * es_bias : 0;
    const size_t bytes_res = has_res ? (static_cast<size_t>(d.m - 1) * d.res_sm + d.n) * es_res : 0;
    const size_t bytes_out = has_res ? (static_cast<size_t>(d.m - 1) * d.out_sm + d.n) * es_out : 0;
    cudaError_t e = h->stage[0].reserve(bytes_a);
    if (e == cudaSuccess && args.c != nullptr) e = h->stage[2].reserve(bytes_c);
    if (e == cudaSuccess && d.has_bias) e = h->stage[3].reserve(bytes_bias);
    if (e == cudaSuccess && has_res) e = h->stage[4].reserve(bytes_res);
    if (e == cudaSuccess && has_res) e = h->stage[5].reserve(bytes_out);
    const bool b_cached = (h->packed_key != nullptr && h->packed_key == args.b);
    if (e == cudaSuccess && !b_cached) e = h->stage[1].reserve(bytes_b);
    if (e != cudaSuccess) {
        return fail_cuda(e, "host staging");
    }
    char *dev_a = static_cast<char *>(h->stage[0].ptr), *dev_c = static_cast<char *>(h->stage[2].ptr);
    char *dev_bias = static_cast<char *>(h->stage[3].ptr), *dev_res = static_cast<char *>(h->stage[4].ptr);
    char *dev_out = static_cast<char *>(h->stage[5].ptr);
    if (!b_cached) {
        e = cudaMemcpyAsync(h->stage[1].ptr, args.b, bytes_b, cudaMemcpyHostToDevice, s_in);
    }
    if (e == cudaSuccess && d.has_bias) {
        e = cudaMemcpyAsync(dev_bias, args.bias, bytes_bias, cudaMemcpyHostToDevice, s_in);
    }
    if (e != cudaSuccess) {
        return fail_cuda(e, "host to device copy");
    }
    long long rows = (d.m + 7) / 8;
    rows = std::max<long long>((rows + 127) / 128 * 128, 256);
    const int chunks = static_cast<int>((d.m + rows - 1) / rows);
    int launches = 0;
    for (int i = 0; i < chunks && i < Handle::kMaxChunks; ++i) {
        const long long r0 = i * rows, nr = std::min<long long>(rows, d.m - r0);
        const size_t off_a = static_cast<size_t>(r0) * d.a_sm * es_a;
        e = cudaMemcpyAsync(dev_a + off_a, static_cast<const char *>(args.a) + off_a,
                            (static_cast<size_t>(nr - 1) * d.a_sm + d.k) * es_a, cudaMemcpyHostToDevice, s_in);
        if (e == cudaSuccess && has_res) {
            const size_t off = static_cast<size_t>(r0) * d.res_sm * es_res;
            e = cudaMemcpyAsync(dev_res + off, static_cast<const char *>(args.res) + off,
                                (static_cast<size_t>(nr - 1) * d.res_sm + d.n) * es_res, cudaMemcpyHostToDevice, s_in);
        }
        if (e == cudaSuccess) e = cudaEventRecord(h->pipe_in[i], s_in);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(s_run, h->pipe_in[i], 0);
        if (e != cudaSuccess) {
            return fail_cuda(e, "host pipeline copy-in");
        }
        kudnn_b200_linear_desc sub = d;
        sub.m = nr;
        kudnn_b200_linear_args dev = args;
        dev.a = dev_a + off_a;
        dev.b = b_cached ? args.b : h->stage[1].ptr;
        dev.c = args.c != nullptr ? dev_c + static_cast<size_t>(r0) * d.c_sm * es_c : nullptr;
        dev.bias = d.has_bias ? dev_bias + static_cast<size_t>(r0) * d.bias_sm * es_bias : nullptr;
        dev.res = has_res ? dev_res + static_cast<size_t>(r0) * d.res_sm * es_res : nullptr;
        dev.out = has_res ? dev_out + static_cast<size_t>(r0) * d.out_sm * es_out : nullptr;
        rc = run_device(h, sub, dev, s_run);
        if (rc != KUDNN_B200_OK) {
            cudaDeviceSynchronize();
            return rc;
        }
        launches += h->last_launches;
        e = cudaEventRecord(h->pipe_done[i], s_run);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(s_out, h->pipe_done[i], 0);
        if (e == cudaSuccess && args.c != nullptr) {
            const size_t off = static_cast<size_t>(r0) * d.c_sm * es_c;
            e = cudaMemcpyAsync(static_cast<char *>(args.c) + off, dev_c + off, (static_cast<size_t>(nr - 1) * d.c_sm + d.n) * es_c,
                                cudaMemcpyDeviceToHost, s_out);
        }
        if (e == cudaSuccess && has_res) {
            const size_t off = static_cast<size_t>(r0) * d.out_sm * es_out;
            e = cudaMemcpyAsync(static_cast<char *>(args.out) + off, dev_out + off,
                                (static_cast<size_t>(nr - 1) * d.out_sm + d.n) * es_out, cudaMemcpyDeviceToHost, s_out);
        }
        if (e != cudaSuccess) {
            cudaDeviceSynchronize();
            return fail_cuda(e, "host pipeline copy-out");
        }
    }
    h->last_launches = launches;
    e = cudaStreamSynchronize(s_out);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s_run);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s_in);
    if (e != cudaSuccess) {
        return fail_cuda(e, "run_host");
    }
    return read_status(h);
}

}  // namespace

extern "C" {

int kudnn_b200_linear_validate(const kudnn_b200_linear_desc *desc)
{
    if (desc == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "validate: null descriptor");
    }
    const kudnn_b200_linear_desc &d = *desc;
    if (d.m <= 0 || d.n <= 0 || d.k <= 0) {
        return fail(KUDNN_B200_UNSUPPORTED, "validate: empty tensors are not supported");
    }
    if (d.m > 0x7fffffffll || d.n > 0x7fffffffll || d.k > 0x7fffffffll) {
        return fail(KUDNN_B200_UNSUPPORTED, "validate: extent exceeds 2^31-1");
    }
    for (int i = 0; i < 3; ++i) {
        if (d.batch[i] < 0) {
            return fail(KUDNN_B200_BAD_ARGUMENTS, "validate: negative batch extent");
        }
    }
    const bool int_gemm = is_int8_dtype(d.a_dtype) && is_int8_dtype(d.b_dtype) && d.c_dtype == KUDNN_B200_S32;
    const bool w8a16 = d.a_dtype == KUDNN_B200_F16 && is_int8_dtype(d.b_dtype) && d.c_dtype == KUDNN_B200_F16;
    if (int_gemm) {
        // <s8|u8, s8|u8, s32, s32> (src/dnn/src/kudnn_gemm.cpp:259-334): a plain product with an optional s32 bias
        if ((d.has_bias != 0 && d.bias_dtype != KUDNN_B200_S32) || d.act != KUDNN_B200_ACT_NONE || d.res_op != KUDNN_B200_RES_NONE) {
            return fail(KUDNN_B200_UNSUPPORTED, "validate: 8-bit integer products take an S32 bias and no post-operation");
        }
    } else if (!is_float_dtype(d.a_dtype) || !(is_float_dtype(d.b_dtype) || w8a16) || !is_float_dtype(d.c_dtype)) {
        return fail(KUDNN_B200_UNSUPPORTED, "validate: operands must be F32 / F16 / BF16, or F16 x S8/U8 -> F16, or S8/U8 x S8/U8 -> S32");
    }
    if (!int_gemm && d.has_bias != 0 && !is_float_dtype(d.bias_dtype)) {
        return fail(KUDNN_B200_UNSUPPORTED, "validate: bias type");
    }
    switch (d.act) {
        case KUDNN_B200_ACT_NONE:
        case KUDNN_B200_ACT_RELU:
        case KUDNN_B200_ACT_TANH:
        case KUDNN_B200_ACT_SIGMOID:
        case KUDNN_B200_ACT_GELU_TANH:
        case KUDNN_B200_ACT_SWISH:
        case KUDNN_B200_ACT_GELU_ERF:
            break;
        default:
            return fail(KUDNN_B200_UNSUPPORTED, "validate: activation %d is not implemented", d.act);
    }
    switch (d.res_op) {
        case KUDNN_B200_RES_NONE:
            break;
        case KUDNN_B200_RES_EXT:
        case KUDNN_B200_RES_IDENTICAL:
        case KUDNN_B200_RES_ELTWISE_MUL:
            if (!is_float_dtype(d.res_dtype) || !is_float_dtype(d.out_dtype)) {
                return fail(KUDNN_B200_UNSUPPORTED, "validate: res / out type");
            }
            break;
        default:
            return fail(KUDNN_B200_UNSUPPORTED, "validate: second-output operator %d", d.res_op);
    }
    if (d.a_sm < 0 || d.a_sk < 0 || d.b_sk < 0 || d.b_sn < 0 || d.c_sm < 0 || d.c_sn < 0) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "validate: negative stride");
    }
    if ((d.c_sm == 0 && d.m > 1) || (d.c_sn == 0 && d.n > 1)) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "validate: output strides must not broadcast");
    }
    return KUDNN_B200_OK;
}

int kudnn_b200_linear_create(const kudnn_b200_linear_desc *desc, kudnn_b200_linear_t *handle)
{
    if (handle == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "create: null handle pointer");
    }
    *handle = nullptr;
    int rc = kudnn_b200_linear_validate(desc);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }
    Handle *h = new (std::nothrow) Handle();
    if (h == nullptr) {
        return fail(KUDNN_B200_ALLOC_FAILED, "create: out of host memory");
    }
    h->d = *desc;
    const char *force = std::getenv("KUDNN_B200_FORCE_KERNEL");
    if (force != nullptr) {
        if (std::strcmp(force, "simt") == 0) {
            h->forced_kernel = KUDNN_B200_KERNEL_SIMT;
        } else if (std::strcmp(force, "tc") == 0) {
            h->forced_kernel = KUDNN_B200_KERNEL_TC;
        } else if (std::strcmp(force, "gemv_fma") == 0) {
            h->forced_kernel = KUDNN_B200_KERNEL_GEMV_FMA;
        } else if (std::strcmp(force, "gemv_mma") == 0) {
            h->forced_kernel = KUDNN_B200_KERNEL_GEMV_MMA;
        }
    }
    *handle = h;
    return KUDNN_B200_OK;
}

int kudnn_b200_linear_clone(kudnn_b200_linear_t src, kudnn_b200_linear_t *handle)
{
    if (src == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "clone: null handle");
    }
    int rc = kudnn_b200_linear_create(&src->d, handle);
    if (rc == KUDNN_B200_OK) {
        (*handle)->forced_kernel = src->forced_kernel;
    }
    return rc;
}

int kudnn_b200_linear_destroy(kudnn_b200_linear_t h)
{
    if (h == nullptr) {
        return KUDNN_B200_OK;
    }
    if (!h->shards.empty()) {
        int cur = -1;
        (void)cudaGetDevice(&cur);
        for (auto &sh : h->shards) {
            cudaSetDevice(sh.device);
            for (auto &b : sh.buf) {
                b.release();
            }
            kudnn_b200_linear_destroy(sh.child);
        }
        h->shards.clear();
        if (cur >= 0) {
            cudaSetDevice(cur);
        }
        (void)cudaGetLastError();
    }
    if (h->device >= 0) {
        int cur = 0;
        if (cudaGetDevice(&cur) == cudaSuccess && cur != h->device) {
            cudaSetDevice(h->device);
        } else {
            cur = -1;
        }
        h->status.release();
        h->gemv_partials.release();
        h->gemv_counters.release();
        h->a_scratch.release();
        h->b_scratch.release();
        h->b_packed.release();
        h->b_blocked.release();
        h->q_scratch.release();
        for (auto &s : h->stage) {
            s.release();
        }
        if (h->pipe_ready) {
            for (auto &st : h->pipe_stream) {
                cudaStreamDestroy(st);
            }
            for (int i = 0; i < kudnn_b200_linear_s::kMaxChunks; ++i) {
                cudaEventDestroy(h->pipe_in[i]);
                cudaEventDestroy(h->pipe_done[i]);
            }
        }
        if (cur >= 0) {
            cudaSetDevice(cur);
        }
        (void)cudaGetLastError();
    }
    delete h;
    return KUDNN_B200_OK;
}

int kudnn_b200_linear_prepack(kudnn_b200_linear_t h, const void *b, void *cuda_stream)
{
    if (h == nullptr || b == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "prepack: null argument");
    }
    std::lock_guard<std::mutex> guard(h->lock);
    int rc = ensure_device(h);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    const kudnn_b200_linear_desc &d = h->d;
    if (batch_extent(d, 0) * batch_extent(d, 1) * batch_extent(d, 2) != 1) {
        return fail(KUDNN_B200_UNSUPPORTED, "prepack: batched weights are not pre-packed");
    }
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, b);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        attr.type = cudaMemoryTypeUnregistered;
    }
    const bool on_device = attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
    const void *b_dev = b;
    if (!on_device) {
        const size_t bytes = static_cast<size_t>(span_elems(d.k, d.b_sk, d.n, d.b_sn, d, d.b_sb)) * kb::dtype_size(d.b_dtype);
        e = h->stage[1].reserve(bytes);
        if (e != cudaSuccess) {
            return fail_cuda(e, "prepack staging");
        }
        e = cudaMemcpyAsync(h->stage[1].ptr, b, bytes, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) {
            return fail_cuda(e, "prepack copy");
        }
        b_dev = h->stage[1].ptr;
    }
    h->plan_valid = false;
    if (d.c_dtype == KUDNN_B200_S32) {
        // 8-bit integer weights: K-major rows with a pitch of a multiple of 16 bytes, what the tensor maps of the
        // integer tensor-core launches read; already so on the device: used in place
        h->b_blocked.release();
        h->blocked_kpad = 0;
        if (on_device && kmajor_ready(b, d.b_dtype, d.b_sn, d.b_sk, d.n)) {
            h->b_packed.release();
            h->packed_ptr = b;
            h->packed_raw = b;
            h->packed_ld = d.b_sn;
        } else {
            const long long k_pad = round_up(d.k, 16);
            e = h->b_packed.reserve(static_cast<size_t>(d.n) * k_pad);
            if (e != cudaSuccess) {
                return fail_cuda(e, "packed weights");
            }
            e = kb::launch_pack_kmajor(b_dev, d.b_dtype, d.n, d.k, d.b_sn, d.b_sk, h->b_packed.ptr, d.b_dtype, k_pad, k_pad, stream);
            if (e != cudaSuccess) {
                return fail_cuda(e, "weight pack kernel");
            }
            h->packed_ptr = h->b_packed.ptr;
            h->packed_raw = h->b_packed.ptr;
            h->packed_ld = k_pad;
        }
        h->packed_ktotal = d.k;
        h->packed_key = b;
        e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) {
            return fail_cuda(e, "prepack");
        }
        return KUDNN_B200_OK;
    }
    h->packed_int8 = false;
    if (is_int8_dtype(d.b_dtype) && d.m <= 16 && d.k % 16 == 0) {
        // fp16 activations, 8-bit weights, decode shapes: the streaming kernels read the 8-bit values themselves.
        // K-major rows with a pitch of a multiple of 16 bytes: the caller's device buffer if it is so, else a copy.
        // Other kernels, when forced, widen from here per call.
        h->b_blocked.release();
        h->blocked_kpad = 0;
        if (on_device && kmajor_ready(b, d.b_dtype, d.b_sn, d.b_sk, d.n)) {
            h->b_packed.release();
            h->packed_ptr = b;
            h->packed_raw = b;
            h->packed_ld = d.b_sn;
        } else {
            e = h->b_packed.reserve(static_cast<size_t>(d.n) * d.k);
            if (e != cudaSuccess) {
                return fail_cuda(e, "packed weights");
            }
            e = kb::launch_pack_kmajor(b_dev, d.b_dtype, d.n, d.k, d.b_sn, d.b_sk, h->b_packed.ptr, d.b_dtype, d.k, d.k, stream);
            if (e != cudaSuccess) {
                return fail_cuda(e, "weight pack kernel");
            }
            h->packed_ptr = h->b_packed.ptr;
            h->packed_raw = h->b_packed.ptr;
            h->packed_ld = d.k;
        }
        h->packed_ktotal = d.k;
        h->packed_int8 = true;
        h->packed_key = b;
        e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) {
            return fail_cuda(e, "prepack");
        }
        return KUDNN_B200_OK;
    }
    if (on_device && d.b_dtype != KUDNN_B200_F32 && !is_int8_dtype(d.b_dtype) && kmajor_ready(b, d.b_dtype, d.b_sn, d.b_sk, d.n)) {
        // already in the streamed layout: the packed copy is the caller's buffer itself
        h->b_packed.release();
        h->packed_ptr = b;
        h->packed_raw = b;
        h->packed_ld = d.b_sn;
        h->packed_ktotal = d.k;
    } else {
        int launches = 0;
        long long ld = 0, kt = 0;
        const void *raw = nullptr;
        rc = pack_weights(h, b_dev, &h->b_packed, true, stream, &ld, &kt, &raw, &launches);
        if (rc != KUDNN_B200_OK) {
            return rc;
        }
        h->packed_ptr = h->b_packed.ptr;
        h->packed_raw = raw;
        h->packed_ld = ld;
        h->packed_ktotal = kt;
    }
    // Decode-shaped primitives (m <= 16, 16-bit types) stream the whole weight matrix on every call: they get a
    // second copy in blocks of 8 rows x 64 k, the unit their MMA kernels read, so that a warp's loads are one
    // contiguous piece of memory.  A single activation row stays on the FMA kernel, which reads plain rows.
    h->blocked_kpad = 0;
    if (d.m >= 2 && d.m <= 16 && d.b_dtype != KUDNN_B200_F32 &&
        (d.a_dtype == d.b_dtype || (d.a_dtype == KUDNN_B200_F16 && is_int8_dtype(d.b_dtype))) && d.k % 8 == 0) {
        const long long k_pad = round_up(d.k, 256);
        e = h->b_blocked.reserve(static_cast<size_t>(round_up(d.n, 8)) * k_pad * 2);
        if (e != cudaSuccess) {
            return fail_cuda(e, "decode-packed weights");
        }
        e = kb::launch_pack_blocks(h->packed_raw, d.n, d.k, h->packed_ld, h->b_blocked.ptr, k_pad, stream);
        if (e != cudaSuccess) {
            return fail_cuda(e, "decode pack kernel");
        }
        h->blocked_kpad = k_pad;
    } else {
        h->b_blocked.release();
    }
    h->packed_key = b;
    // one-time cost: later runs may use other streams (the host-pointer pipeline does) and the staging buffer is reused
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) {
        return fail_cuda(e, "prepack");
    }
    return KUDNN_B200_OK;
}

int kudnn_b200_linear_run(kudnn_b200_linear_t h, const kudnn_b200_linear_args *args, void *cuda_stream)
{
    if (h == nullptr || args == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run: null argument");
    }
    std::lock_guard<std::mutex> guard(h->lock);
    return run_device(h, h->d, *args, static_cast<cudaStream_t>(cuda_stream));
}

int kudnn_b200_linear_run_host(kudnn_b200_linear_t h, const kudnn_b200_linear_args *args)
{
    if (h == nullptr || args == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run_host: null argument");
    }
    std::lock_guard<std::mutex> guard(h->lock);
    int rc = ensure_device(h);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }
    const kudnn_b200_linear_desc &d = h->d;
    if (args->a == nullptr || args->b == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run_host: a and b must not be null");
    }
    if ((d.has_bias != 0) != (args->bias != nullptr)) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run_host: bias pointer does not match the descriptor");
    }
    if (d.res_op != KUDNN_B200_RES_NONE && (args->res == nullptr || args->out == nullptr)) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run_host: res and out must not be null for this descriptor");
    }
    if (d.res_op == KUDNN_B200_RES_NONE && args->c == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run_host: c must not be null");
    }
    if (pipeline_applies(d, *args)) {
        return run_host_pipelined(h, *args);
    }
    cudaStream_t stream = nullptr;
    const size_t bytes_a = static_cast<size_t>(span_elems(d.m, d.a_sm, d.k, d.a_sk, d, d.a_sb)) * kb::dtype_size(d.a_dtype);
    const size_t bytes_b = static_cast<size_t>(span_elems(d.k, d.b_sk, d.n, d.b_sn, d, d.b_sb)) * kb::dtype_size(d.b_dtype);
    const size_t bytes_c = static_cast<size_t>(span_elems(d.m, d.c_sm, d.n, d.c_sn, d, d.c_sb)) * kb::dtype_size(d.c_dtype);
    const size_t bytes_bias =
        d.has_bias ? static_cast<size_t>(span_elems(d.m, d.bias_sm, d.n, d.bias_sn, d, d.bias_sb)) * kb::dtype_size(d.bias_dtype)
                   : 0;
    const bool has_res = d.res_op != KUDNN_B200_RES_NONE;
    const size_t bytes_res =
        has_res ? static_cast<size_t>(span_elems(d.m, d.res_sm, d.n, d.res_sn, d, d.res_sb)) * kb::dtype_size(d.res_dtype) : 0;
    const size_t bytes_out =
        has_res ? static_cast<size_t>(span_elems(d.m, d.out_sm, d.n, d.out_sn, d, d.out_sb)) * kb::dtype_size(d.out_dtype) : 0;

    const bool b_cached = (h->packed_key != nullptr && h->packed_key == args->b);
    kudnn_b200_linear_args dev = *args;
    cudaError_t e;
#define KB_STAGE_IN(idx, host_ptr, nbytes, field)                                                        \
    do {                                                                                                 \
        e = h->stage[idx].reserve(nbytes);                                                               \
        if (e != cudaSuccess) return fail_cuda(e, "host staging");                                       \
        e = cudaMemcpyAsync(h->stage[idx].ptr, host_ptr, nbytes, cudaMemcpyHostToDevice, stream);        \
        if (e != cudaSuccess) return fail_cuda(e, "host to device copy");                                \
        dev.field = h->stage[idx].ptr;                                                                   \
    } while (0)
    KB_STAGE_IN(0, args->a, bytes_a, a);
    if (!b_cached) {
        KB_STAGE_IN(1, args->b, bytes_b, b);
    }
    if (d.has_bias) {
        KB_STAGE_IN(3, args->bias, bytes_bias, bias);
    }
    if (has_res) {
        KB_STAGE_IN(4, args->res, bytes_res, res);
        e = h->stage[5].reserve(bytes_out);
        if (e != cudaSuccess) return fail_cuda(e, "host staging");
        dev.out = h->stage[5].ptr;
    }
    if (args->c != nullptr) {
        if (args->beta != 0.0f) {
            KB_STAGE_IN(2, args->c, bytes_c, c);
        } else {
            e = h->stage[2].reserve(bytes_c);
            if (e != cudaSuccess) return fail_cuda(e, "host staging");
            dev.c = h->stage[2].ptr;
        }
    }
#undef KB_STAGE_IN
    rc = run_device(h, d, dev, stream);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }
    if (args->c != nullptr) {
        e = cudaMemcpyAsync(args->c, dev.c, bytes_c, cudaMemcpyDeviceToHost, stream);
        if (e != cudaSuccess) return fail_cuda(e, "device to host copy");
    }
    if (has_res) {
        e = cudaMemcpyAsync(args->out, dev.out, bytes_out, cudaMemcpyDeviceToHost, stream);
        if (e != cudaSuccess) return fail_cuda(e, "device to host copy");
    }
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) {
        return fail_cuda(e, "run_host");
    }
    return read_status(h);
}

int kudnn_b200_linear_run_sharded(kudnn_b200_linear_t h, const kudnn_b200_linear_args *args, int nshards, int mode)
{
    if (h == nullptr || args == nullptr || nshards < 1 || nshards > 64 ||
        (mode != KUDNN_B200_SHARD_ROWS && mode != KUDNN_B200_SHARD_COLS)) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run_sharded: bad argument");
    }
    std::lock_guard<std::mutex> guard(h->lock);
    const kudnn_b200_linear_desc &d = h->d;
    if (batch_extent(d, 0) * batch_extent(d, 1) * batch_extent(d, 2) != 1) {
        return fail(KUDNN_B200_UNSUPPORTED, "run_sharded: batched problems are not sharded");
    }
    if (args->a == nullptr || args->b == nullptr || (d.has_bias != 0) != (args->bias != nullptr) ||
        (d.res_op != KUDNN_B200_RES_NONE ? (args->res == nullptr || args->out == nullptr) : args->c == nullptr)) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run_sharded: pointers do not match the descriptor");
    }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, args->a) == cudaSuccess &&
        (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged)) {
        return fail(KUDNN_B200_UNSUPPORTED, "run_sharded takes host pointers (device-resident shards belong to one process per "
                                            "GPU, see kudnn_b200_shard_range and kudnn_b200_linear_set_mirrors)");
    }
    (void)cudaGetLastError();
    const int ndev = kudnn_b200_device_count();
    if (ndev <= 0) {
        return fail(KUDNN_B200_NO_DEVICE, "run_sharded: no CUDA device");
    }
    const bool cols = mode == KUDNN_B200_SHARD_COLS;
    const bool has_res = d.res_op != KUDNN_B200_RES_NONE;
    if (cols && (args->beta != 0.0f || d.a_sk != 1 || d.c_sn != 1 || (has_res && (d.res_sn != 1 || d.out_sn != 1)) ||
                 (d.has_bias != 0 && d.bias_sm != 0))) {
        return fail(KUDNN_B200_UNSUPPORTED, "run_sharded by columns needs beta = 0, row-major a / c / res / out and a bias that "
                                            "is one value per column");
    }
    // (re)build the children when the split changes
    if (h->shard_mode != mode || h->shard_count != nshards) {
        for (auto &sh : h->shards) {
            cudaSetDevice(sh.device);
            for (auto &b : sh.buf) {
                b.release();
            }
            kudnn_b200_linear_destroy(sh.child);
        }
        h->shards.clear();
        h->shards.resize(nshards);
        for (int i = 0; i < nshards; ++i) {
            Handle::Shard &sh = h->shards[i];
            int64_t begin = 0, count = 0;
            kudnn_b200_shard_range(cols ? d.n : d.m, nshards, i, cols ? 8 : 128, &begin, &count);
            sh.begin = begin;
            sh.count = count;
            sh.device = i % ndev;
            if (count == 0) {
                continue;
            }
            kudnn_b200_linear_desc sub = d;
            if (cols) {
                // on the device a shard is a compact problem: its slab of c / res / out has n_local columns
                sub.n = count;
                sub.c_sm = sub.res_sm = sub.out_sm = count;
                sub.a_sm = d.k;
            } else {
                sub.m = count;
            }
            int rc = kudnn_b200_linear_create(&sub, &sh.child);
            if (rc != KUDNN_B200_OK) {
                return rc;
            }
            sh.child->forced_kernel = h->forced_kernel;
        }
        h->shard_mode = mode;
        h->shard_count = nshards;
    }
    // one host thread per shard: set the device, stage, run, copy back
    std::vector<int> codes(nshards, KUDNN_B200_OK);
    std::vector<std::string> messages(nshards);
    auto work = [&](int i) {
        Handle::Shard &sh = h->shards[i];
        if (sh.count == 0) {
            return;
        }
        auto give_up = [&](int rc) {
            codes[i] = rc;
            messages[i] = g_error;
        };
        if (cudaSetDevice(sh.device) != cudaSuccess) {
            give_up(fail(KUDNN_B200_CUDA_ERROR, "run_sharded: cannot select device %d", sh.device));
            return;
        }
        const size_t es_b = kb::dtype_size(d.b_dtype);
        // the child's weights: the whole matrix (row shards) or its slab of columns, packed once per weight pointer
        const char *b_sub = static_cast<const char *>(args->b) + (cols ? sh.begin * d.b_sn * es_b : 0);
        if (sh.weights != b_sub) {
            int rc = kudnn_b200_linear_prepack(sh.child, b_sub, nullptr);
            if (rc != KUDNN_B200_OK) {
                give_up(rc);
                return;
            }
            sh.weights = b_sub;
        }
        kudnn_b200_linear_args sub = *args;
        sub.b = b_sub;
        if (!cols) {
            const long long r0 = sh.begin;
            sub.a = static_cast<const char *>(args->a) + r0 * d.a_sm * kb::dtype_size(d.a_dtype);
            sub.c = args->c != nullptr ? static_cast<char *>(args->c) + r0 * d.c_sm * kb::dtype_size(d.c_dtype) : nullptr;
            sub.bias = d.has_bias ? static_cast<const char *>(args->bias) + r0 * d.bias_sm * kb::dtype_size(d.bias_dtype) : nullptr;
            sub.res = has_res ? static_cast<const char *>(args->res) + r0 * d.res_sm * kb::dtype_size(d.res_dtype) : nullptr;
            sub.out = has_res ? static_cast<char *>(args->out) + r0 * d.out_sm * kb::dtype_size(d.out_dtype) : nullptr;
            int rc = kudnn_b200_linear_run_host(sh.child, &sub);
            if (rc != KUDNN_B200_OK) {
                give_up(rc);
            }
            return;
        }
        // column shard: x whole, the slabs of bias / res in, the slabs of c / out back, as strided copies
        const long long c0 = sh.begin, nl = sh.count;
        const size_t es_a = kb::dtype_size(d.a_dtype), es_c = kb::dtype_size(d.c_dtype), es_bias = kb::dtype_size(d.bias_dtype);
        const size_t es_r = kb::dtype_size(d.res_dtype), es_o = kb::dtype_size(d.out_dtype);
        cudaError_t e = sh.buf[0].reserve(static_cast<size_t>(d.m) * d.k * es_a);
        if (e == cudaSuccess && d.has_bias) e = sh.buf[1].reserve(static_cast<size_t>(nl) * es_bias);
        if (e == cudaSuccess && args->c != nullptr) e = sh.buf[2].reserve(static_cast<size_t>(d.m) * nl * es_c);
        if (e == cudaSuccess && has_res) e = sh.buf[3].reserve(static_cast<size_t>(d.m) * nl * es_r);
        if (e == cudaSuccess && has_res) e = sh.buf[4].reserve(static_cast<size_t>(d.m) * nl * es_o);
        cudaStream_t st = nullptr;
        if (e == cudaSuccess) {
            e = cudaMemcpy2DAsync(sh.buf[0].ptr, d.k * es_a, args->a, d.a_sm * es_a, d.k * es_a, d.m, cudaMemcpyHostToDevice, st);
        }
        if (e == cudaSuccess && d.has_bias) {
            e = cudaMemcpyAsync(sh.buf[1].ptr, static_cast<const char *>(args->bias) + c0 * d.bias_sn * es_bias, nl * es_bias,
                                cudaMemcpyHostToDevice, st);
        }
        if (e == cudaSuccess && has_res) {
            e = cudaMemcpy2DAsync(sh.buf[3].ptr, nl * es_r, static_cast<const char *>(args->res) + c0 * es_r, d.res_sm * es_r,
                                  nl * es_r, d.m, cudaMemcpyHostToDevice, st);
        }
        if (e != cudaSuccess) {
            give_up(fail_cuda(e, "run_sharded: staging"));
            return;
        }
        sub.a = sh.buf[0].ptr;
        sub.bias = d.has_bias ? sh.buf[1].ptr : nullptr;
        sub.c = args->c != nullptr ? sh.buf[2].ptr : nullptr;
        sub.res = has_res ? sh.buf[3].ptr : nullptr;
        sub.out = has_res ? sh.buf[4].ptr : nullptr;
        int rc = kudnn_b200_linear_run(sh.child, &sub, st);
        if (rc != KUDNN_B200_OK) {
            give_up(rc);
            return;
        }
        if (args->c != nullptr) {
            e = cudaMemcpy2DAsync(static_cast<char *>(args->c) + c0 * es_c, d.c_sm * es_c, sh.buf[2].ptr, nl * es_c, nl * es_c, d.m,
                                  cudaMemcpyDeviceToHost, st);
        }
        if (e == cudaSuccess && has_res) {
            e = cudaMemcpy2DAsync(static_cast<char *>(args->out) + c0 * es_o, d.out_sm * es_o, sh.buf[4].ptr, nl * es_o, nl * es_o,
                                  d.m, cudaMemcpyDeviceToHost, st);
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) {
            give_up(fail_cuda(e, "run_sharded: copy back"));
            return;
        }
        rc = kudnn_b200_linear_check(sh.child, st);
        if (rc != KUDNN_B200_OK) {
            give_up(rc);
        }
    };
    int cur = -1;
    (void)cudaGetDevice(&cur);
    std::vector<std::thread> threads;
    for (int i = 1; i < nshards; ++i) {
        threads.emplace_back(work, i);
    }
    work(0);
    for (auto &t : threads) {
        t.join();
    }
    if (cur >= 0) {
        cudaSetDevice(cur);
    }
    int launches = 0;
    for (int i = 0; i < nshards; ++i) {
        if (codes[i] != KUDNN_B200_OK) {
            return fail(codes[i], "shard %d: %s", i, messages[i].c_str());
        }
        if (h->shards[i].child != nullptr) {
            launches += h->shards[i].child->last_launches;
            h->last_kernel = h->shards[i].child->last_kernel;
        }
    }
    h->last_launches = launches;
    return KUDNN_B200_OK;
}

int kudnn_b200_linear_run_any(kudnn_b200_linear_t h, const kudnn_b200_linear_args *args, void *cuda_stream)
{
    if (h == nullptr || args == nullptr || args->a == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "run: null argument");
    }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, args->a) != cudaSuccess) {
        (void)cudaGetLastError();
        attr.type = cudaMemoryTypeUnregistered;
    }
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) {
        return kudnn_b200_linear_run(h, args, cuda_stream);
    }
    return kudnn_b200_linear_run_host(h, args);
}

int kudnn_b200_linear_check(kudnn_b200_linear_t h, void *cuda_stream)
{
    if (h == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "check: null handle");
    }
    std::lock_guard<std::mutex> guard(h->lock);
    if (h->device < 0) {
        return KUDNN_B200_OK;
    }
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) {
        return fail_cuda(e, "check");
    }
    return read_status(h);
}

int kudnn_b200_linear_force_kernel(kudnn_b200_linear_t h, int kernel)
{
    if (h == nullptr || kernel < KUDNN_B200_KERNEL_AUTO || kernel > KUDNN_B200_KERNEL_TC) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "force_kernel: bad argument");
    }
    h->forced_kernel = kernel;
    return KUDNN_B200_OK;
}

int kudnn_b200_linear_set_mirrors(kudnn_b200_linear_t h, int count, void *const *c_mirrors, void *const *out_mirrors)
{
    if (h == nullptr || count < 0 || count > kb::kMaxMirrors) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "set_mirrors: count must be between 0 and %d", kb::kMaxMirrors);
    }
    std::lock_guard<std::mutex> guard(h->lock);
    h->n_mirrors = count;
    for (int i = 0; i < count; ++i) {
        h->c_mirror[i] = c_mirrors != nullptr ? c_mirrors[i] : nullptr;
        h->out_mirror[i] = out_mirrors != nullptr ? out_mirrors[i] : nullptr;
    }
    return KUDNN_B200_OK;
}

int kudnn_b200_linear_set_multicast(kudnn_b200_linear_t h, void *c_multicast, void *out_multicast)
{
    if (h == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "set_multicast: null handle");
    }
    std::lock_guard<std::mutex> guard(h->lock);
    h->c_multicast = c_multicast;
    h->out_multicast = out_multicast;
    return KUDNN_B200_OK;
}

int kudnn_b200_linear_unpack(kudnn_b200_linear_t h)
{
    if (h == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "unpack: null handle");
    }
    std::lock_guard<std::mutex> guard(h->lock);
    h->packed_key = nullptr;
    h->packed_int8 = false;
    h->packed_ptr = nullptr;
    h->packed_raw = nullptr;
    h->packed_ld = h->packed_ktotal = 0;
    h->blocked_kpad = 0;
    h->plan_valid = false;
    if (h->device >= 0) {
        h->b_packed.release();
        h->b_blocked.release();
    }
    return KUDNN_B200_OK;
}

int kudnn_b200_debug_set_wait(kudnn_b200_linear_t h, long long wait_limit_cycles, int skip_kblock)
{
    if (h == nullptr || wait_limit_cycles < 0) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "debug_set_wait: bad argument");
    }
    std::lock_guard<std::mutex> guard(h->lock);
    h->wait_limit = wait_limit_cycles;
    h->skip_kblock = skip_kblock;
    return KUDNN_B200_OK;
}

int kudnn_b200_debug_fail_allocation(int nth)
{
    g_alloc_fail_countdown.store(nth);
    return KUDNN_B200_OK;
}

int kudnn_b200_linear_last_kernel(kudnn_b200_linear_t h)
{
    return h == nullptr ? 0 : h->last_kernel;
}

int kudnn_b200_linear_last_launches(kudnn_b200_linear_t h)
{
    return h == nullptr ? 0 : h->last_launches;
}

int64_t kudnn_b200_linear_workspace_bytes(kudnn_b200_linear_t h)
{
    if (h == nullptr) {
        return 0;
    }
    return static_cast<int64_t>(h->gemv_partials.bytes + h->gemv_counters.bytes + h->a_scratch.bytes + h->b_scratch.bytes +
                                h->b_packed.bytes + h->b_blocked.bytes);
}

int kudnn_b200_shard_range(int64_t total, int nparts, int part, int64_t align, int64_t *begin, int64_t *count)
{
    if (total < 0 || nparts <= 0 || part < 0 || part >= nparts || align <= 0 || begin == nullptr || count == nullptr) {
        return fail(KUDNN_B200_BAD_ARGUMENTS, "shard_range: bad argument");
    }
    const int64_t units = (total + align - 1) / align;
    const int64_t base = units / nparts, extra = units % nparts;
    const int64_t u0 = part * base + std::min<int64_t>(part, extra);
    const int64_t u1 = u0 + base + (part < extra ? 1 : 0);
    const int64_t b = std::min<int64_t>(u0 * align, total);
    const int64_t e = std::min<int64_t>(u1 * align, total);
    *begin = b;
    *count = e - b;
    return KUDNN_B200_OK;
}

const char *kudnn_b200_last_error(void)
{
    return g_error;
}

const char *kudnn_b200_version(void)
{
    return "kudnn_b200 0.1 (sm_100a)";
}

int kudnn_b200_device_count(void)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

}  // extern "C"
