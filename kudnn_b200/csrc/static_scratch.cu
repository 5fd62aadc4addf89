// Decode-shaped Linear for callers that must not allocate device memory.
//
// Some callers cannot reach cudaMalloc at the moment they need a result: code that runs under a memory budget
// fixed at start-up (every byte of HBM already handed to a serving engine's own pools), plug-ins whose host
// framework forbids allocation inside an operator call, and latency-critical decode loops that cannot afford the
// implicit device synchronisation an allocation may bring.  The regular entry points grow their scratch on demand
// with cudaMalloc; this one never does.  Its scratch (the partial sums and arrival counters of the streaming
// kernels' split-K reduction) lives in a fixed array inside this library's device image.
//
// Consequences a user has to know:
//   * the array is part of the library's device code: every GPU on which that code has been loaded holds it (about
//     8 MiB) until the process exits.  The CUDA runtime loads device code lazily by default, so the array appears
//     with the first call on a device, and each kernel variant (element type x row-count class) is loaded by the
//     first call that launches it; both take device memory from the driver, once.  Warm up one call per device and
//     variant before giving the rest of HBM away (or set CUDA_MODULE_LOADING=EAGER); later calls take none;
//   * problems whose scratch would not fit are refused with KUDNN_B200_UNSUPPORTED, nothing is launched;
//   * all calls on one device share the array.  Two calls that overlap on the GPU (different streams, or different
//     host threads on different streams) race on it and both results are undefined; serialise them on one stream;
//   * the first call on each device looks up the array's device address (no allocation, but a runtime query);
//     make that first call before starting any stream capture.
#include "kernels.cuh"

#include <mutex>

namespace {

constexpr long long kStaticPartialFloats = 2ll * 1024 * 1024;  // 8 MiB of partial sums
constexpr long long kStaticCounters = 16 * 1024;               // 64 KiB of arrival counters
constexpr size_t kStaticBytes = static_cast<size_t>(kStaticPartialFloats) * 4 + static_cast<size_t>(kStaticCounters) * 4;

// In host code this name is only a handle for the runtime; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

struct DeviceSlot {
    bool ready = false;
    unsigned char *scratch = nullptr;
    int sm_count = 0;
};

constexpr int kMaxDevices = 64;
DeviceSlot g_slots[kMaxDevices];
std::mutex g_slots_lock;

// Once per device, with that device current: resolve the scratch address and the SM count.
int prepare_device(int dev, DeviceSlot *out)
{
    std::lock_guard<std::mutex> guard(g_slots_lock);
    DeviceSlot &slot = g_slots[dev];
    if (!slot.ready) {
        int major = 0, sms = 0;
        cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e == cudaSuccess) {
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        }
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return kb::set_last_error(KUDNN_B200_CUDA_ERROR, "static-scratch run: cannot query the device");
        }
        if (major != 10) {
            return kb::set_last_error(KUDNN_B200_NO_DEVICE, "static-scratch run: the current device is not sm_100");
        }
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            (void)cudaGetLastError();
            return kb::set_last_error(KUDNN_B200_CUDA_ERROR, "static-scratch run: cudaGetSymbolAddress failed");
        }
        slot.scratch = static_cast<unsigned char *>(ptr);
        slot.sm_count = sms;
        slot.ready = true;
    }
    *out = slot;
    return KUDNN_B200_OK;
}

}  // namespace

extern "C" int kudnn_b200_linear_run_static_scratch(const kudnn_b200_linear_desc *desc,
                                                    const kudnn_b200_linear_args *args, void *cuda_stream)
{
    if (desc == nullptr || args == nullptr) {
        return kb::set_last_error(KUDNN_B200_BAD_ARGUMENTS, "static-scratch run: null argument");
    }
    int rc = kudnn_b200_linear_validate(desc);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }
    const kudnn_b200_linear_desc &d = *desc;
    for (int i = 0; i < 3; ++i) {
        if (d.batch[i] > 1) {
            return kb::set_last_error(KUDNN_B200_UNSUPPORTED, "static-scratch run: batched problems are not supported");
        }
    }
    if (d.m > 16) {
        return kb::set_last_error(KUDNN_B200_UNSUPPORTED, "static-scratch run: m must be at most 16 (decode shapes)");
    }
    if (args->a == nullptr || args->b == nullptr || (d.has_bias != 0) != (args->bias != nullptr)) {
        return kb::set_last_error(KUDNN_B200_BAD_ARGUMENTS, "static-scratch run: a / b / bias pointers do not match the descriptor");
    }
    if (d.res_op != KUDNN_B200_RES_NONE ? (args->res == nullptr || args->out == nullptr) : (args->c == nullptr)) {
        return kb::set_last_error(KUDNN_B200_BAD_ARGUMENTS, "static-scratch run: output pointers do not match the descriptor");
    }
    if (args->beta != 0.0f && args->c == nullptr) {
        return kb::set_last_error(KUDNN_B200_BAD_ARGUMENTS, "static-scratch run: beta != 0 needs c");
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        return kb::set_last_error(KUDNN_B200_NO_DEVICE, "static-scratch run: no usable CUDA device is current");
    }
    DeviceSlot slot;
    rc = prepare_device(dev, &slot);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }

    kb::LinearProblem pr;
    pr.a = args->a;
    pr.b = args->b;
    pr.m = d.m;
    pr.n = d.n;
    pr.k = d.k;
    pr.a_sm = d.a_sm;
    pr.a_sk = d.a_sk;
    pr.b_sk = d.b_sk;
    pr.b_sn = d.b_sn;
    pr.a_dtype = d.a_dtype;
    pr.b_dtype = d.b_dtype;
    kb::EpiParams &e = pr.epi;
    e.c = args->c;
    e.bias = args->bias;
    e.res = args->res;
    e.out = args->out;
    e.c_sm = d.c_sm;
    e.c_sn = d.c_sn;
    e.bias_sm = d.bias_sm;
    e.bias_sn = d.bias_sn;
    e.res_sm = d.res_sm;
    e.res_sn = d.res_sn;
    e.out_sm = d.out_sm;
    e.out_sn = d.out_sn;
    e.alpha = args->alpha;
    e.beta = args->beta;
    if (d.a_dtype == KUDNN_B200_BF16 && d.b_dtype == KUDNN_B200_BF16 && d.c_dtype == KUDNN_B200_BF16 && d.has_bias == 0) {
        // as in the handle-based entry points: the reference's bias-free bf16 product takes bf16 scalars
        e.alpha = __bfloat162float(__float2bfloat16_rn(args->alpha));
        e.beta = __bfloat162float(__float2bfloat16_rn(args->beta));
    }
    e.gamma = args->gamma;
    e.act_alpha = d.act_alpha;
    e.c_dtype = d.c_dtype;
    e.bias_dtype = d.bias_dtype;
    e.res_dtype = d.res_dtype;
    e.out_dtype = d.out_dtype;
    e.has_bias = d.has_bias;
    e.half_chain = (d.c_dtype == KUDNN_B200_F16 && d.a_dtype == KUDNN_B200_F16 && d.b_dtype == KUDNN_B200_F16 &&
                    (d.has_bias == 0 || d.bias_dtype == KUDNN_B200_F16))
                       ? 1
                       : 0;
    e.act = d.act;
    e.res_op = d.res_op;
    e.n_mirrors = 0;
    e.m = static_cast<int>(d.m);
    e.n = static_cast<int>(d.n);
    pr.batch.n1 = 1;
    pr.batch.n2 = 1;
    for (int i = 0; i < 3; ++i) {
        pr.batch.a_sb[i] = pr.batch.b_sb[i] = pr.batch.c_sb[i] = 0;
        pr.batch.bias_sb[i] = pr.batch.res_sb[i] = pr.batch.out_sb[i] = 0;
    }
    pr.batch_count = 1;

    kb::GemvPlan plan;
    if (!kb::gemv_plan(pr, slot.sm_count, KUDNN_B200_KERNEL_AUTO, &plan)) {
        return kb::set_last_error(KUDNN_B200_UNSUPPORTED,
                                  "static-scratch run: the streaming kernels need K-contiguous, 16-byte aligned a and b "
                                  "of one element type");
    }
    if (plan.partial_floats > kStaticPartialFloats || plan.counter_count > kStaticCounters) {
        return kb::set_last_error(KUDNN_B200_UNSUPPORTED,
                                  "static-scratch run: this problem needs more scratch than the built-in 8 MiB array holds "
                                  "(use kudnn_b200_linear_run, which allocates)");
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    kb::GemvWorkspace ws;
    ws.partials = reinterpret_cast<float *>(slot.scratch);
    ws.counters = reinterpret_cast<unsigned *>(slot.scratch + static_cast<size_t>(kStaticPartialFloats) * 4);
    ws.partial_floats = kStaticPartialFloats;
    ws.counter_count = kStaticCounters;
    // the counters must be zero when the kernel starts; an earlier call that was cut short may have left some set
    cudaError_t ce = cudaMemsetAsync(ws.counters, 0, static_cast<size_t>(plan.counter_count) * sizeof(unsigned), stream);
    if (ce == cudaSuccess) {
        ce = kb::launch_gemv(pr, plan, ws, stream);
    }
    if (ce != cudaSuccess) {
        (void)cudaGetLastError();
        return kb::set_last_error(KUDNN_B200_CUDA_ERROR, cudaGetErrorString(ce));
    }
    return KUDNN_B200_OK;
}
