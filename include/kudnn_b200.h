/*
 * kudnn_b200 — C ABI of the B200 (sm_100a) Linear(+post-op) path.
 *
 * This is the boundary the C++ classes KuDNN::Gemm, KuDNN::LinearActivationLayerFWD and
 * KuDNN::LinearResFWD call into.  Plain pointers, sizes and PODs only; no exceptions cross it.
 * Every function returns one of the KUDNN_B200_* status codes; the text of the last error of
 * the calling thread is available from kudnn_b200_last_error().
 *
 * One descriptor covers what the three reference classes can express for this path:
 *     c   = act( alpha * a·b + beta * c + bias )              (rounded to c_dtype as the reference does)
 *     out = c (+) res                                          (optional second output)
 * with a [m,k], b [k,n], c / res / out [m,n], bias broadcastable to [m,n], up to three leading
 * batch dimensions (stride 0 = broadcast), every tensor addressed by element strides.
 */
#ifndef KUDNN_B200_H
#define KUDNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KUDNN_B200_API __attribute__((visibility("default")))

/* Status codes.  0..2 are KuDNN::Status (src/dnn/include/service/kudnn_err_codes.hpp:18-22);
 * the rest are appended for conditions a CPU library does not have. */
#define KUDNN_B200_OK 0
#define KUDNN_B200_UNSUPPORTED 1
#define KUDNN_B200_BAD_ARGUMENTS 2
#define KUDNN_B200_ALLOC_FAILED 3
#define KUDNN_B200_CUDA_ERROR 4
#define KUDNN_B200_TIMEOUT 5   /* a bounded device-side wait gave up; the context stays usable */
#define KUDNN_B200_NO_DEVICE 6 /* no sm_100 device, or the CUDA runtime could not be initialised */

/* Element types: the values of KuDNN::Element::TypeT (src/dnn/include/types/kudnn_data_type.hpp:31-39). */
#define KUDNN_B200_F32 1
#define KUDNN_B200_F16 2
#define KUDNN_B200_BF16 3
/* Integer types, accepted in two families of the reference's table (src/dnn/src/kudnn_gemm.cpp:590-601):
 *   a, b in {S8, U8}, c and bias S32 (:259-334): exact 32-bit integer sums, no activation, no second output;
 *   a F16, b in {S8, U8}, c F16 (:336-372, "W8A16"): the weights are widened to fp16 when they are packed. */
#define KUDNN_B200_S32 4
#define KUDNN_B200_S8 5
#define KUDNN_B200_U8 6

/* Activations: the values of KuDNN::ActivationFunction (src/dnn/include/operations/kudnn_eltwise.hpp:24-54);
 * 0 (UNIMPLEMENTED there) means "no activation" here. */
#define KUDNN_B200_ACT_NONE 0
#define KUDNN_B200_ACT_RELU 5
#define KUDNN_B200_ACT_TANH 9
#define KUDNN_B200_ACT_SIGMOID 10
#define KUDNN_B200_ACT_GELU_TANH 20
#define KUDNN_B200_ACT_SWISH 25
#define KUDNN_B200_ACT_GELU_ERF 27

/* Second-output operators.  EXT and IDENTICAL are KuDNN::ResOpsFunction::RES_EXT / RES_IDENTIAL
 * (src/dnn/include/operations/kudnn_linear_res.hpp:25-29, arithmetic in src/dnn/src/kudnn_linear_res.cpp:57-122).
 * The reference's RES_MUL is a second matrix product and is issued by the host as a second call.
 * ELTWISE_MUL (out = c * res element-wise) has no counterpart in the reference. */
#define KUDNN_B200_RES_NONE 0
#define KUDNN_B200_RES_EXT 1
#define KUDNN_B200_RES_IDENTICAL 2
#define KUDNN_B200_RES_ELTWISE_MUL 3

/* Kernel families, as reported by kudnn_b200_linear_last_kernel and accepted by ..._force_kernel. */
#define KUDNN_B200_KERNEL_AUTO 0
#define KUDNN_B200_KERNEL_SIMT 1     /* general strided FMA kernel: any layout, any size */
#define KUDNN_B200_KERNEL_GEMV_FMA 2 /* m <= 4 streaming kernel, fp32 FMA + warp-shuffle reduction */
#define KUDNN_B200_KERNEL_GEMV_MMA 3 /* m <= 16 streaming kernel, 16-bit inputs */
#define KUDNN_B200_KERNEL_TC 4       /* tcgen05 / TMEM tensor-core kernel fed by TMA */

/* Replaces the argument lists of the reference constructors:
 *   Gemm(aInfo,bInfo,cInfo,biasInfo,numThreads)                     src/dnn/include/operations/kudnn_gemm.hpp:36-39
 *   LinearActivationLayerFWD(a,b,c,bias,alpha,beta,kind,numThreads) .../kudnn_linear_activationlayer.hpp:44-52
 *   LinearResFWD(a,b,c,bias,res,linearRes,alpha,beta,gamma,kind,..) .../kudnn_linear_res.hpp:50-59
 * A TensorInfo (dims, type, layout, strides; src/dnn/include/types/kudnn_tensor_info.hpp:132-289) becomes a
 * dtype code plus element strides of the logical dimensions; layouts are folded into the strides. */
typedef struct kudnn_b200_linear_desc {
    int64_t m, n, k;
    int64_t batch[3]; /* leading batch extents, outermost first; 0 or 1 = absent */
    int32_t a_dtype, b_dtype, c_dtype, bias_dtype, res_dtype, out_dtype;
    int32_t has_bias, act, res_op, reserved;
    float act_alpha, act_beta; /* activation parameters (relu slope, swish beta); not GEMM scalars */
    int64_t a_sm, a_sk, a_sb[3];
    int64_t b_sk, b_sn, b_sb[3];
    int64_t c_sm, c_sn, c_sb[3];
    int64_t bias_sm, bias_sn, bias_sb[3]; /* 0 = broadcast along that dimension */
    int64_t res_sm, res_sn, res_sb[3];
    int64_t out_sm, out_sn, out_sb[3];
} kudnn_b200_linear_desc;

/* Replaces the pointer/scalar arguments of the reference Run methods
 * (kudnn_gemm.hpp:44-47, kudnn_linear_activationlayer.hpp:57-58, kudnn_linear_res.hpp:69-73). */
typedef struct kudnn_b200_linear_args {
    const void *a;
    const void *b;
    void *c;          /* may be NULL when res_op != NONE and only `out` is wanted */
    const void *bias; /* non-NULL iff has_bias */
    const void *res;  /* non-NULL iff res_op != NONE */
    void *out;        /* non-NULL iff res_op != NONE */
    float alpha, beta, gamma;
} kudnn_b200_linear_args;

typedef struct kudnn_b200_linear_s *kudnn_b200_linear_t;

/* Host-only check of a descriptor; replaces the kernel-facing part of Gemm::ValidateInput
 * (src/dnn/src/kudnn_gemm.cpp:384-476).  Touches no CUDA state. */
KUDNN_B200_API int kudnn_b200_linear_validate(const kudnn_b200_linear_desc *desc);

/* Primitive creation; replaces GemmImpl::GemmImpl (src/dnn/src/kudnn_gemm.cpp:830-857).  Host-only: device state is
 * created on first use, on the device that is current at that time. */
KUDNN_B200_API int kudnn_b200_linear_create(const kudnn_b200_linear_desc *desc, kudnn_b200_linear_t *handle);
KUDNN_B200_API int kudnn_b200_linear_clone(kudnn_b200_linear_t src, kudnn_b200_linear_t *handle);
KUDNN_B200_API int kudnn_b200_linear_destroy(kudnn_b200_linear_t handle);

/* Pre-packs the weight operand `b` (host or device memory) into the layout the chosen kernel streams (K-major,
 * 16-byte aligned rows; fp32 weights additionally split into TF32 hi/lo planes).  Later runs whose args->b equals
 * `b` use the packed copy and do not read `b` again: the packed copy is recognised by the ADDRESS alone.  After the
 * weights at that address have changed (an in-place update, or a new tensor the allocator placed where the old one
 * was) call prepack again, or kudnn_b200_linear_unpack to go back to reading `b` on every run; otherwise runs keep
 * using the old values.  Replaces the per-call packing inside the reference's BLAS/JIT
 * (src/dnn/src/matmul_jit/MatrixComputation/kudnn_default_impl_fp16fp16f32f32.cpp:929-962). */
KUDNN_B200_API int kudnn_b200_linear_prepack(kudnn_b200_linear_t handle, const void *b, void *cuda_stream);
/* Forgets (and frees) the packed copy.  No counterpart in the reference, which packs on every call. */
KUDNN_B200_API int kudnn_b200_linear_unpack(kudnn_b200_linear_t handle);

/* Execute with DEVICE pointers on `cuda_stream` (a cudaStream_t, NULL = default stream); asynchronous.
 * A handle owns device scratch (split-K partial sums and arrival counters, packed activations, the status block)
 * that all of its runs share: the handle's lock serialises the host side only, so runs of ONE handle must not overlap
 * on the GPU.  Keep a handle on one stream at a time; kudnn_b200_linear_clone gives every further stream a handle of
 * its own.
 * Replaces GemmImpl::Run / LinearActivationLayerFWDImpl::Run / LinearResFWDImpl::Run
 * (src/dnn/src/kudnn_gemm.cpp:859-877, kudnn_linear_activationlayer.cpp:40-56, kudnn_linear_res.cpp:184-202). */
KUDNN_B200_API int kudnn_b200_linear_run(kudnn_b200_linear_t handle, const kudnn_b200_linear_args *args,
                                         void *cuda_stream);

/* Execute with HOST pointers, as the reference's callers pass them: stages inputs to the device, runs, copies the
 * outputs back and synchronises.  A weight pointer that was pre-packed is not copied again.  Large 2-D problems
 * (m >= 1024) whose a and output buffers are page-locked (cudaHostAlloc / cudaHostRegister) are cut into blocks of
 * rows so that copy-in, kernel and copy-out overlap; pageable buffers take the single-shot path (copy everything in,
 * one run, copy everything out), because their copies hold the host and could not overlap anyway. */
KUDNN_B200_API int kudnn_b200_linear_run_host(kudnn_b200_linear_t handle, const kudnn_b200_linear_args *args);

/* Looks at where args->a lives and calls kudnn_b200_linear_run (device memory) or kudnn_b200_linear_run_host (anything
 * else).  All pointers of one call must be of the same kind.  This is what the C++ classes' Run methods use, so that
 * code written for the reference (host pointers) and GPU-resident callers share one signature. */
KUDNN_B200_API int kudnn_b200_linear_run_any(kudnn_b200_linear_t handle, const kudnn_b200_linear_args *args,
                                             void *cuda_stream);

/* Execute with HOST pointers on several GPUs of this machine from one process.  The rows of the layer
 * (KUDNN_B200_SHARD_ROWS: every device gets the whole weight matrix and a block of the rows of a, c, res, out) or its
 * columns (KUDNN_B200_SHARD_COLS: every device gets all of a and a slab of the columns of b, bias, c, res, out) are
 * cut into `nshards` pieces, boundaries at multiples of 128 rows / 8 columns; shard i runs on device
 * i modulo the device count, on a host thread of its own, through a child primitive that packs its weights on first
 * use and recognises the weight pointer afterwards.  Nothing crosses between devices: every shard's slab goes straight
 * back into the caller's host tensors, so no gather step is needed.  Returns when all outputs are complete.  No
 * counterpart in the reference, a single-socket CPU library. */
#define KUDNN_B200_SHARD_ROWS 0
#define KUDNN_B200_SHARD_COLS 1
KUDNN_B200_API int kudnn_b200_linear_run_sharded(kudnn_b200_linear_t handle, const kudnn_b200_linear_args *args,
                                                 int nshards, int mode);

/* Decode-shaped Linear (m <= 16, 2-D, K-contiguous a and b) that allocates no device memory, for callers that
 * cannot call cudaMalloc when they need the result: engines that have already handed all of HBM to their own pools,
 * plug-ins whose host forbids allocation inside an operator call, decode loops that cannot risk the device
 * synchronisation an allocation may cause.  This entry point has no counterpart in the reference.  It takes the
 * descriptor directly (no handle) and device pointers; the split-K scratch of the streaming kernels is a fixed
 * 8 MiB (+ 64 KiB of counters) array inside the library's device image, held by every GPU on which the library's
 * device code has been loaded, until the process exits.  Problems whose scratch does not fit return
 * KUDNN_B200_UNSUPPORTED and launch nothing.
 * All calls on a device share that array: calls that overlap on the GPU race and give undefined results, so keep
 * them on one stream.
 * Warm-up rule.  The CUDA runtime loads device code lazily (CUDA_MODULE_LOADING=LAZY is the default since 12.2): the
 * array comes into existence when the first call on a device resolves its address, and each kernel variant (element
 * type x row-count class m = 1 / 2..8 / 9..16) is loaded by the first call that launches it.  Both take device
 * memory from the driver, once.  So make one call per device and per variant you will use BEFORE handing the rest
 * of HBM to your pools and before any stream capture (or run with CUDA_MODULE_LOADING=EAGER); from then on a call
 * takes no device memory at all. */
KUDNN_B200_API int kudnn_b200_linear_run_static_scratch(const kudnn_b200_linear_desc *desc,
                                                        const kudnn_b200_linear_args *args, void *cuda_stream);

/* ---- the operators either side of Linear ---------------------------------------------------------------------------
 * Stand-alone activation pass over `count` elements of a dense tensor.  Replaces ActivationLayerFWD::Run
 * (src/dnn/include/operations/kudnn_eltwise.hpp:62-76, src/dnn/src/kudnn_eltwise.cpp:500-586): fp32 arithmetic; with
 * equal source and result types fp16 results are rounded to nearest even and bf16 results truncated, otherwise the
 * result is rounded once from fp32.  `act` is one of the KUDNN_B200_ACT_* codes (RELU, TANH, SIGMOID, GELU_TANH, SWISH,
 * GELU_ERF; the reference's other 16 functions return UNSUPPORTED), alpha the relu slope / swish factor.  src and dst
 * are both device memory (16-byte aligned; asynchronous on the stream) or both host memory (staged; synchronous). */
KUDNN_B200_API int kudnn_b200_activation_validate(int64_t count, int src_dtype, int dst_dtype, int act);
KUDNN_B200_API int kudnn_b200_activation_run(const void *src, void *dst, int64_t count, int src_dtype, int dst_dtype,
                                             int act, float alpha, void *cuda_stream);

/* RMS normalisation over the last axis of a dense [rows, axis] tensor: y = x * (scale * 1 / sqrt(variance + eps)),
 * variance = mean(x^2) per row in fp32, or the caller's `variance` with USE_GLOBAL_STATS; with save_stats the computed
 * variances are written to `variance`.  Replaces RMSNormalizationLayerFWD::Run
 * (src/dnn/include/operations/kudnn_rms_normalization.hpp:26-44, kernels/rmsnorm/kudnn_rmsnorm_fwd_last_def.hpp:128-180).
 * Flags are KuDNN::NormalizationFlags (src/dnn/include/types/kudnn_normalization.hpp:18-24).  The reference accepts
 * fp16 only; bf16 and fp32 are accepted here as well.  Device or host pointers, as for the activation. */
#define KUDNN_B200_NORM_USE_GLOBAL_STATS 0x1
#define KUDNN_B200_NORM_USE_SCALE 0x2
#define KUDNN_B200_NORM_USE_SHIFT 0x4
#define KUDNN_B200_NORM_FUSE_RELU 0x8
KUDNN_B200_API int kudnn_b200_rmsnorm_validate(int64_t rows, int64_t axis, int dtype, int flags);
KUDNN_B200_API int kudnn_b200_rmsnorm_run(const void *src, void *dst, const void *scale, float *variance, int64_t rows,
                                          int64_t axis, int dtype, int flags, int save_stats, float eps,
                                          void *cuda_stream);

/* Reads the device-side status word of the handle (bounded waits that gave up) after synchronising the stream. */
KUDNN_B200_API int kudnn_b200_linear_check(kudnn_b200_linear_t handle, void *cuda_stream);

/* ---- column-sharded layers: one kernel computes a slab of y and writes it into every rank's copy -------------------
 * No counterpart in the reference (a single-socket CPU library; its tensor-parallel users gather outside of it).
 *
 * set_mirrors: from now on every run of the handle stores c (and out) not only through args.c / args.out but also
 * through each mirror pointer, with the same strides.  A mirror is typically the same tensor in another GPU's
 * memory, opened with kudnn_b200_peer_buffer_open; the stores go over NVLink from the kernel's epilogue, tile by
 * tile, so there is no gather step afterwards.  Up to 7 mirrors; each must be 16-byte congruent with the primary
 * pointer.  Pass count = 0 to switch mirroring off.  When a launch has completed on a rank (stream synchronised),
 * its slab is complete in every mirror; the ranks still have to tell each other (a barrier) before they read. */
KUDNN_B200_API int kudnn_b200_linear_set_mirrors(kudnn_b200_linear_t handle, int count, void *const *c_mirrors,
                                                 void *const *out_mirrors);

/* set_multicast: on top of set_mirrors.  c_multicast / out_multicast are the addresses at which the same output
 * tensors are mapped through an NVLink multicast object that spans every rank's copy, this rank's included (created
 * by the host program: cuMulticastCreate / cuMulticastBindMem / cuMemMap, or a library that does so, e.g. PyTorch's
 * symmetric memory).  The tensor-core kernel then writes each finished 128-byte row piece with ONE multimem.st
 * instead of a local store plus one store per mirror: the switch replicates it, so a rank sends its slab over NVLink
 * once whatever the number of ranks.  Launches or rows that do not take that path (other kernels, unaligned rows) use
 * the plain mirror stores, so the mirrors must stay set.  Null pointers switch it off.  A process must not exit, and
 * its buffer must not be freed, while another rank may still store through the mapping. */
KUDNN_B200_API int kudnn_b200_linear_set_multicast(kudnn_b200_linear_t handle, void *c_multicast, void *out_multicast);

/* A device buffer other processes of this machine can map, and its 64-byte handle; open / close on the other side. */
#define KUDNN_B200_PEER_HANDLE_BYTES 64
KUDNN_B200_API int kudnn_b200_peer_buffer_create(size_t bytes, void **dev_ptr, unsigned char *handle_out);
KUDNN_B200_API int kudnn_b200_peer_buffer_open(const unsigned char *handle, void **dev_ptr);
KUDNN_B200_API int kudnn_b200_peer_buffer_close(void *dev_ptr);
KUDNN_B200_API int kudnn_b200_peer_buffer_destroy(void *dev_ptr);

/* Test hooks (no counterpart in the reference).  set_wait: device-side waits of this handle's tensor-core launches
 * give up after `wait_limit_cycles` SM cycles (0 = the default, about two seconds), and the producer of CTA 0 leaves
 * out the loads of k-block `skip_kblock` of its first tile (-1 = never), so that one bounded wait runs out, the
 * kernel drains, frees its tensor memory and the run reports KUDNN_B200_TIMEOUT; nothing faults or hangs.
 * fail_allocation: the nth (0 = next) device allocation the library attempts fails as if the device were out of
 * memory (KUDNN_B200_ALLOC_FAILED); negative = off. */
KUDNN_B200_API int kudnn_b200_debug_set_wait(kudnn_b200_linear_t handle, long long wait_limit_cycles, int skip_kblock);
KUDNN_B200_API int kudnn_b200_debug_fail_allocation(int nth);

/* Introspection used by tests and the benchmark. */
KUDNN_B200_API int kudnn_b200_linear_force_kernel(kudnn_b200_linear_t handle, int kernel);
KUDNN_B200_API int kudnn_b200_linear_last_kernel(kudnn_b200_linear_t handle);
KUDNN_B200_API int kudnn_b200_linear_last_launches(kudnn_b200_linear_t handle);
KUDNN_B200_API int64_t kudnn_b200_linear_workspace_bytes(kudnn_b200_linear_t handle);

/* Row partition used by the sharded launchers: part `part` of `nparts` gets rows [*begin, *begin + *count),
 * boundaries rounded to multiples of `align`.  Pure arithmetic. */
KUDNN_B200_API int kudnn_b200_shard_range(int64_t total, int nparts, int part, int64_t align, int64_t *begin,
                                          int64_t *count);

KUDNN_B200_API const char *kudnn_b200_last_error(void);
KUDNN_B200_API const char *kudnn_b200_version(void);
KUDNN_B200_API int kudnn_b200_device_count(void);

#ifdef __cplusplus
}
#endif

#endif /* KUDNN_B200_H */
