// C-ABI of the stand-alone activation and RMS-normalisation operators (declared in include/kudnn_b200.h).  Pointers
// may be device memory (the kernels run on the caller's stream, asynchronously) or host memory, as the reference's
// callers pass it (the data is staged through temporary device buffers and the call returns when dst is complete).
#include "kernels.cuh"

namespace {

int device_sm_count(int *sms)
{
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return kb::set_last_error(KUDNN_B200_NO_DEVICE, "no usable CUDA device is current");
    }
    if (major != 10) {
        return kb::set_last_error(KUDNN_B200_NO_DEVICE, "the current device is not sm_100; this library carries sm_100a code only");
    }
    return KUDNN_B200_OK;
}

bool on_device(const void *p)
{
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

bool float_type(int dt)
{
    return dt == KUDNN_B200_F32 || dt == KUDNN_B200_F16 || dt == KUDNN_B200_BF16;
}

struct Temp {
    void *ptr = nullptr;
    ~Temp()
    {
        if (ptr != nullptr) {
            cudaFree(ptr);
        }
    }
    cudaError_t alloc(size_t bytes) { return cudaMalloc(&ptr, bytes); }
};

int cuda_fail(cudaError_t e, const char *what)
{
    (void)cudaGetLastError();
    return kb::set_last_error(e == cudaErrorMemoryAllocation ? KUDNN_B200_ALLOC_FAILED : KUDNN_B200_CUDA_ERROR, what);
}

}  // namespace

extern "C" {

int kudnn_b200_activation_validate(int64_t count, int src_dtype, int dst_dtype, int act)
{
    if (count <= 0) {
        return kb::set_last_error(KUDNN_B200_UNSUPPORTED, "activation: empty tensors are not supported");
    }
    if (!float_type(src_dtype) || !float_type(dst_dtype)) {
        return kb::set_last_error(KUDNN_B200_UNSUPPORTED, "activation: only F32 / F16 / BF16 tensors are implemented");
    }
    switch (act) {
        case KUDNN_B200_ACT_RELU:
        case KUDNN_B200_ACT_TANH:
        case KUDNN_B200_ACT_SIGMOID:
        case KUDNN_B200_ACT_GELU_TANH:
        case KUDNN_B200_ACT_SWISH:
        case KUDNN_B200_ACT_GELU_ERF:
            return KUDNN_B200_OK;
        default:
            return kb::set_last_error(KUDNN_B200_UNSUPPORTED, "activation: this function is not implemented");
    }
}

int kudnn_b200_activation_run(const void *src, void *dst, int64_t count, int src_dtype, int dst_dtype, int act, float alpha,
                              void *cuda_stream)
{
    int rc = kudnn_b200_activation_validate(count, src_dtype, dst_dtype, act);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }
    if (src == nullptr || dst == nullptr) {
        return kb::set_last_error(KUDNN_B200_BAD_ARGUMENTS, "activation: src and dst must not be null");
    }
    int sms = 0;
    rc = device_sm_count(&sms);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    const size_t src_bytes = static_cast<size_t>(count) * kb::dtype_size(src_dtype);
    const size_t dst_bytes = static_cast<size_t>(count) * kb::dtype_size(dst_dtype);
    if (on_device(src)) {
        if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) != 0) {
            return kb::set_last_error(KUDNN_B200_UNSUPPORTED, "activation: device tensors must start on 16-byte boundaries");
        }
        cudaError_t e = kb::launch_activation(src, src_dtype, dst, dst_dtype, count, act, alpha, sms, stream);
        return e == cudaSuccess ? KUDNN_B200_OK : cuda_fail(e, "activation kernel launch");
    }
    Temp d_src, d_dst;
    cudaError_t e = d_src.alloc(src_bytes);
    if (e == cudaSuccess) e = d_dst.alloc(dst_bytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_src.ptr, src, src_bytes, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = kb::launch_activation(d_src.ptr, src_dtype, d_dst.ptr, dst_dtype, count, act, alpha, sms, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dst, d_dst.ptr, dst_bytes, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    return e == cudaSuccess ? KUDNN_B200_OK : cuda_fail(e, "activation (host pointers)");
}

int kudnn_b200_rmsnorm_validate(int64_t rows, int64_t axis, int dtype, int flags)
{
    // USE_SHIFT is accepted and ignored, as in the reference (RMS normalisation has no shift term)
    if ((flags & KUDNN_B200_NORM_FUSE_RELU) != 0) {
        return kb::set_last_error(KUDNN_B200_UNSUPPORTED, "rmsnorm: fused relu is not supported");
    }
    if (rows <= 0 || axis <= 0) {
        return kb::set_last_error(KUDNN_B200_UNSUPPORTED, "rmsnorm: empty tensors are not supported");
    }
    if (axis > 0x7fffffffll) {
        return kb::set_last_error(KUDNN_B200_UNSUPPORTED, "rmsnorm: axis longer than 2^31-1");
    }
    if (!float_type(dtype)) {
        return kb::set_last_error(KUDNN_B200_UNSUPPORTED, "rmsnorm: only F32 / F16 / BF16 tensors are implemented");
    }
    return KUDNN_B200_OK;
}

int kudnn_b200_rmsnorm_run(const void *src, void *dst, const void *scale, float *variance, int64_t rows, int64_t axis,
                           int dtype, int flags, int save_stats, float eps, void *cuda_stream)
{
    int rc = kudnn_b200_rmsnorm_validate(rows, axis, dtype, flags);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }
    const int use_stats = (flags & KUDNN_B200_NORM_USE_GLOBAL_STATS) != 0 ? 1 : 0;
    const int use_scale = (flags & KUDNN_B200_NORM_USE_SCALE) != 0 ? 1 : 0;
    // the reference's null checks (src/dnn/src/kudnn_rms_normalization_fwd.cpp:213-226)
    if (src == nullptr || dst == nullptr || ((use_stats != 0 || save_stats != 0) && variance == nullptr) ||
        (use_scale != 0 && scale == nullptr)) {
        return kb::set_last_error(KUDNN_B200_BAD_ARGUMENTS, "rmsnorm: one of the tensors is null");
    }
    int sms = 0;
    rc = device_sm_count(&sms);
    if (rc != KUDNN_B200_OK) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    if (on_device(src)) {
        cudaError_t e = kb::launch_rmsnorm(src, dst, scale, variance, rows, axis, dtype, use_stats, use_scale, save_stats, eps,
                                           sms, stream);
        return e == cudaSuccess ? KUDNN_B200_OK : cuda_fail(e, "rmsnorm kernel launch");
    }
    const size_t es = kb::dtype_size(dtype);
    const size_t bytes = static_cast<size_t>(rows) * axis * es;
    Temp d_src, d_dst, d_scale, d_var;
    cudaError_t e = d_src.alloc(bytes);
    if (e == cudaSuccess) e = d_dst.alloc(bytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_src.ptr, src, bytes, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess && use_scale != 0) {
        e = d_scale.alloc(static_cast<size_t>(axis) * es);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d_scale.ptr, scale, static_cast<size_t>(axis) * es, cudaMemcpyHostToDevice, stream);
    }
    const bool stats = use_stats != 0 || save_stats != 0;
    if (e == cudaSuccess && stats) {
        e = d_var.alloc(static_cast<size_t>(rows) * sizeof(float));
        if (e == cudaSuccess && use_stats != 0) {
            e = cudaMemcpyAsync(d_var.ptr, variance, static_cast<size_t>(rows) * sizeof(float), cudaMemcpyHostToDevice, stream);
        }
    }
    if (e == cudaSuccess) {
        e = kb::launch_rmsnorm(d_src.ptr, d_dst.ptr, d_scale.ptr, static_cast<float *>(d_var.ptr), rows, axis, dtype, use_stats,
                               use_scale, save_stats, eps, sms, stream);
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(dst, d_dst.ptr, bytes, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess && use_stats == 0 && save_stats != 0) {
        e = cudaMemcpyAsync(variance, d_var.ptr, static_cast<size_t>(rows) * sizeof(float), cudaMemcpyDeviceToHost, stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    return e == cudaSuccess ? KUDNN_B200_OK : cuda_fail(e, "rmsnorm (host pointers)");
}

}  // extern "C"
