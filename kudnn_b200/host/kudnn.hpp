// KuDNN Linear API on B200: the value types and the three operator classes of the reference's public C++
// interface for the Linear path, implemented over the C ABI in include/kudnn_b200.h.
//
// Source-compatible with the reference headers for this path (namespaces, class and method names, argument order,
// defaults, exception types, enumerator order):
//   Shape / Layout / Element::Type / TensorInfo   src/dnn/include/types/*.hpp
//   Status, Service::LogicError / Unsupported / BadAlloc, Service::AlignedAlloc   src/dnn/include/service/*.hpp
//   Gemm                         src/dnn/include/operations/kudnn_gemm.hpp:29-51
//   LinearActivationLayerFWD     src/dnn/include/operations/kudnn_linear_activationlayer.hpp:31-63
//   LinearResFWD                 src/dnn/include/operations/kudnn_linear_res.hpp:25-77
//   ActivationFunction           src/dnn/include/operations/kudnn_eltwise.hpp:24-54
// Differences, all additive: data pointers may be device or host memory (host memory is staged through the GPU);
// PrepackWeights() and SetStream() exist on every operator; ResOpsFunction has a fourth value RES_ELTWISE_MUL;
// LinearActivationResFWD fuses an activation and a residual in one call; __fp16 / __bf16 are replaced by 2-byte
// storage structs so the header compiles on any host.
#ifndef KUDNN_B200_HOST_KUDNN_HPP
#define KUDNN_B200_HOST_KUDNN_HPP

#include <array>
#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <iterator>
#include <limits>
#include <memory>
#include <new>
#include <stdexcept>
#include <string>
#include <type_traits>

#define KUDNN_API_PUBLIC __attribute__((visibility("default")))

namespace KuDNN {

using SizeType = std::size_t;
using IntType = std::int64_t;

enum class Status { SUCCESS = 0, UNSUPPORTED, BAD_ARGUMENTS };

namespace Service {

struct BadAlloc : public std::bad_alloc {
    const char *what() const noexcept override { return "KuDNN allocation failed"; }
};
struct BadArrayNewLength : public std::bad_array_new_length {
    const char *what() const noexcept override { return "KuDNN bad array new length"; }
};
struct LogicError : public std::logic_error {
    using std::logic_error::logic_error;
};
struct Unsupported : public std::invalid_argument {
    using std::invalid_argument::invalid_argument;
};

constexpr SizeType ALIGNMENT = 128;

KUDNN_API_PUBLIC void ThrowOnStatus(Status s, const std::string &funcName) noexcept(false);
KUDNN_API_PUBLIC void *AlignedAlloc(SizeType n, SizeType alignment = ALIGNMENT) noexcept(false);
KUDNN_API_PUBLIC void Deallocate(void *p, SizeType n = 0) noexcept;

// true when the product of the range does not fit its integer type
template <typename It>
bool WillIntMultOverflow(It first, It last) noexcept
{
    using T = typename std::iterator_traits<It>::value_type;
    T prod = 1;
    for (It it = first; it != last; ++it) {
        const T v = *it;
        if (v != 0 && prod != 0) {
            volatile T next = prod * v;
            if (next / prod != v) {
                return true;
            }
        }
        prod *= v;
    }
    return false;
}

template <typename T, SizeType alignment = ALIGNMENT>
struct AlignedAllocator {
    using value_type = T;
    using size_type = ::KuDNN::SizeType;
    using difference_type = std::ptrdiff_t;
    template <typename U>
    struct rebind {
        using other = AlignedAllocator<U, alignment>;
    };
    AlignedAllocator() noexcept = default;
    template <typename U>
    AlignedAllocator(const AlignedAllocator<U, alignment> &) noexcept {}
    T *allocate(size_type n)
    {
        if (n > std::numeric_limits<size_type>::max() / sizeof(T)) {
            throw BadArrayNewLength();
        }
        return static_cast<T *>(AlignedAlloc(n * sizeof(T), alignment));
    }
    void deallocate(T *p, size_type n) noexcept { Deallocate(p, n * sizeof(T)); }
    bool operator==(const AlignedAllocator &) const noexcept { return true; }
    bool operator!=(const AlignedAllocator &) const noexcept { return false; }
};

}  // namespace Service

namespace Threading {

enum class EnvMode { KUDNN_THREAD_USE_ENV, KUDNN_THREAD_IGNORE_ENV };
enum class ThreadingControl { KUDNN_DEFAULT, KUDNN_MANUAL };

// Host threads do not take part in the computation here; the thread count is kept because every entry point
// validates its numThreads argument against it (src/dnn/src/kudnn_gemm.cpp:395-398).
KUDNN_API_PUBLIC int SetMaxNumThreads(int nThreads) noexcept;
KUDNN_API_PUBLIC int GetMaxNumThreads() noexcept;

}  // namespace Threading

// ------------------------------------------------------------------------------------------------ element types

namespace Element {

enum class TypeT { UNDEFINED = 0, F32, F16, BF16, S32, S8, U8 };

// 2-byte storage stand-ins for __fp16 and __bf16 (bit patterns only; arithmetic happens on the device)
struct Half {
    std::uint16_t bits;
};
struct BFloat16 {
    std::uint16_t bits;
};

struct Type final {
    using SizeType = ::KuDNN::SizeType;
    Type(const TypeT &t) noexcept(false) : type{t}, size{ByteSize(t)}
    {
        if (t == TypeT::UNDEFINED) {
            throw Service::LogicError{"Type: unsupported data type"};
        }
    }
    SizeType GetSize() const noexcept { return size; }
    SizeType GetBitwidth() const noexcept { return size * 8u; }
    operator TypeT() const noexcept { return type; }
    bool IsFP() const noexcept { return type == TypeT::F32 || type == TypeT::F16 || type == TypeT::BF16; }
    bool IsIntegral() const noexcept { return !IsFP(); }
    bool IsSigned() const noexcept { return type != TypeT::U8; }
    bool IsUnsigned() const noexcept { return !IsSigned(); }

private:
    static SizeType ByteSize(TypeT t) noexcept
    {
        switch (t) {
            case TypeT::F32:
            case TypeT::S32:
                return 4;
            case TypeT::F16:
            case TypeT::BF16:
                return 2;
            case TypeT::S8:
            case TypeT::U8:
                return 1;
            default:
                return 0;
        }
    }
    TypeT type;
    SizeType size;
};

template <typename T>
inline TypeT MatchType()
{
    if (std::is_same<T, float>::value) return TypeT::F32;
    if (std::is_same<T, Half>::value) return TypeT::F16;
    if (std::is_same<T, BFloat16>::value) return TypeT::BF16;
    if (std::is_same<T, std::int32_t>::value) return TypeT::S32;
    if (std::is_same<T, std::int8_t>::value) return TypeT::S8;
    if (std::is_same<T, std::uint8_t>::value) return TypeT::U8;
    return TypeT::UNDEFINED;
}

inline bool operator==(const Type &l, const TypeT &r) noexcept { return static_cast<TypeT>(l) == r; }
inline bool operator==(const TypeT &l, const Type &r) noexcept { return l == static_cast<TypeT>(r); }
inline bool operator==(const Type &l, const Type &r) noexcept { return static_cast<TypeT>(l) == static_cast<TypeT>(r); }
inline bool operator!=(const Type &l, const TypeT &r) noexcept { return !(l == r); }
inline bool operator!=(const TypeT &l, const Type &r) noexcept { return !(l == r); }
inline bool operator!=(const Type &l, const Type &r) noexcept { return !(l == r); }

}  // namespace Element

// ------------------------------------------------------------------------------------------------ shape, layout

constexpr SizeType MAX_DIMS = 5;

struct Shape final {
    using SizeType = ::KuDNN::SizeType;
    static constexpr SizeType NUM_MAX_DIMENSIONS = MAX_DIMS;

    Shape() noexcept : dimsArray{}, numDims{0} {}

    template <typename T>
    Shape(T *ptr, const SizeType size) noexcept(false) : dimsArray{}, numDims{0}
    {
        ResetShape(ptr, size);
    }
    // the variadic form also enforces the reference's 3 GiB-per-tensor guard (elements * 4 bytes)
    template <typename... Ts, typename = typename std::enable_if<(sizeof...(Ts) > 0) &&
                                                                 (std::is_arithmetic<Ts>::value && ...)>::type>
    Shape(Ts... dims) noexcept(false) : dimsArray{{static_cast<SizeType>(dims)...}}, numDims{sizeof...(dims)}
    {
        CheckRank(numDims);
        const long long total = static_cast<long long>(GetTotalDimsSize());
        if (total * 4 > 3LL * 1024 * 1024 * 1024) {
            throw Service::LogicError("Shape: exceeded available memory limit ");
        }
    }
    Shape(const std::initializer_list<SizeType> &list) noexcept(false) : dimsArray{}, numDims{0} { ResetShape(list); }

    template <typename... Ts, typename = typename std::enable_if<(std::is_arithmetic<Ts>::value && ...)>::type>
    Shape &ResetShape(Ts... dims) noexcept(false)
    {
        CheckRank(sizeof...(dims));
        dimsArray = {static_cast<SizeType>(dims)...};
        numDims = sizeof...(dims);
        return *this;
    }
    Shape &ResetShape(const std::initializer_list<SizeType> &list) noexcept(false)
    {
        CheckRank(list.size());
        dimsArray.fill(0);
        SizeType i = 0;
        for (SizeType v : list) {
            dimsArray[i++] = v;
        }
        numDims = list.size();
        return *this;
    }
    template <typename T>
    Shape &ResetShape(T *ptr, const SizeType size) noexcept(false)
    {
        if (ptr == nullptr) {
            throw Service::LogicError("Shape: ptr is nullptr");
        }
        CheckRank(size);
        dimsArray.fill(0);
        for (SizeType i = 0; i < size; ++i) {
            dimsArray[i] = static_cast<SizeType>(ptr[i]);
        }
        numDims = size;
        return *this;
    }

    Shape &operator+=(const Shape &adder) noexcept(false)
    {
        if (adder.numDims != numDims) {
            throw Service::LogicError("Shape: different size of base and adder shapes");
        }
        for (SizeType i = 0; i < numDims; ++i) {
            dimsArray[i] += adder.dimsArray[i];
        }
        return *this;
    }
    Shape operator+(const Shape &adder) const noexcept(false)
    {
        Shape r(*this);
        r += adder;
        return r;
    }
    SizeType operator[](SizeType id) const noexcept(false)
    {
        if (id >= numDims) {
            throw Service::LogicError("Shape: index >= num_dims");
        }
        return dimsArray[id];
    }
    SizeType &operator[](SizeType id) noexcept(false)
    {
        if (id >= numDims) {
            throw Service::LogicError("Shape: index >= num_dims");
        }
        return dimsArray[id];
    }
    SizeType GetNumDims() const noexcept { return numDims; }
    SizeType GetTotalDimsSize() const noexcept(false)
    {
        if (Service::WillIntMultOverflow(dimsArray.begin(), dimsArray.begin() + numDims)) {
            throw Service::LogicError("Shape: computing total size will cause overflow");
        }
        SizeType total = 1;
        for (SizeType i = 0; i < numDims; ++i) {
            total *= dimsArray[i];
        }
        return total;
    }

private:
    static void CheckRank(SizeType n) noexcept(false)
    {
        if (n > NUM_MAX_DIMENSIONS) {
            throw Service::LogicError("Shape: dims is greater than NUM_MAX_DIMENSIONS");
        }
    }
    std::array<SizeType, NUM_MAX_DIMENSIONS> dimsArray;
    SizeType numDims;
};

inline bool operator==(const Shape &l, const Shape &r) noexcept
{
    if (l.GetNumDims() != r.GetNumDims()) {
        return false;
    }
    for (SizeType i = 0; i < l.GetNumDims(); ++i) {
        if (l[i] != r[i]) {
            return false;
        }
    }
    return true;
}
inline bool operator!=(const Shape &l, const Shape &r) noexcept { return !(l == r); }

// A layout names the order of the logical dimensions in memory, slowest first: ACB = A outermost, B fastest.
enum class Layout {
    UNDEFINED = 0,
    A,
    AB, BA,
    ABC, ACB, BAC, BCA, CAB, CBA,
    ABCD, ABDC, ACBD, ACDB, ADBC, ADCB, BACD, BCDA, CDAB, CDBA, DCAB,
    ABCDE, ABCED, ABDEC, ACBDE, ACDEB, ADECB, BACDE, BCDEA, CDEAB, CDEBA, DECAB,
    ROW_MAJOR = AB, COL_MAJOR = BA,
    NCHW = ABCD, NHWC = ACDB, NCDHW = ABCDE, NDHWC = ACDEB,
    OIHW = ABCD, HWIO = CDBA, HWOI = CDAB, OHWI = ACDB, OHWO = BCDA, IOHW = BACD,
};

namespace Service {

// logical dimension stored at memory position idx (0 = slowest) of layout l
KUDNN_API_PUBLIC SizeType GetIdxForUserLayout(Layout l, SizeType idx) noexcept(false);
// rank of a layout, 0 for UNDEFINED
KUDNN_API_PUBLIC SizeType GetLayoutRank(Layout l) noexcept;
// strides of size-1 dimensions become 0 so that they broadcast
KUDNN_API_PUBLIC Shape FlushStrides(const Shape &dims, const Shape &strides) noexcept(false);

}  // namespace Service

struct KUDNN_API_PUBLIC TensorInfo final {
    using SizeType = ::KuDNN::SizeType;
    TensorInfo(const Shape &shape, const Element::Type &t, const Layout &l) noexcept(false);
    TensorInfo(const Shape &shape, const Element::Type &t, const Layout &l, const Shape &strides) noexcept(false);

    Shape GetDims() const noexcept { return dims; }
    SizeType GetNumDims() const noexcept { return dims.GetNumDims(); }
    SizeType GetTotalTensorSize() const noexcept { return dims.GetTotalDimsSize(); }
    Shape GetStrides() const noexcept { return stridesInfo; }
    Element::Type GetType() const noexcept { return type; }
    Layout GetLayout() const noexcept { return layout; }
    bool IsDense() const noexcept;
    bool HasStrideOverFastestDim() const noexcept;
    Layout GetStandardABXLayout() const;
    Layout GetStandardAXBLayout() const;
    Layout GetStandardBXALayout() const;
    SizeType GetAxisNumAccordingToLayout(SizeType axisNum) const noexcept(false);

    // kNoThrow = true: report through the returned Status; false: throw Service::LogicError
    template <bool kNoThrow = false>
    static typename std::conditional<kNoThrow, Status, void>::type ValidateElementType(Element::Type t) noexcept(kNoThrow);
    template <bool kNoThrow = false>
    static typename std::conditional<kNoThrow, Status, void>::type ValidateLayout(Shape d, Layout l) noexcept(kNoThrow);
    template <bool kNoThrow = false>
    static typename std::conditional<kNoThrow, Status, void>::type SetMinimumRequiredStrides(Shape d, Layout l,
                                                                                            Shape &s) noexcept(kNoThrow);
    template <bool kNoThrow = false>
    static typename std::conditional<kNoThrow, Status, void>::type ValidateDimsAndStrides(Shape d, Layout l,
                                                                                         Shape s) noexcept(kNoThrow);

private:
    Shape dims;
    Element::Type type;
    Layout layout;
    Shape stridesInfo;
};

inline bool operator==(const TensorInfo &l, const TensorInfo &r) noexcept
{
    return l.GetDims() == r.GetDims() && l.GetType() == r.GetType() && l.GetLayout() == r.GetLayout() &&
           l.GetStrides() == r.GetStrides();
}
inline bool operator!=(const TensorInfo &l, const TensorInfo &r) noexcept { return !(l == r); }

// ------------------------------------------------------------------------------------------------ operators

enum class ActivationFunction {
    UNIMPLEMENTED, ABS, EXP, LINEAR, LOG, RELU, ROUND, SQRT, SQUARE, TANH, SIGMOID, POW, CLIP, CLIP_V2, HARDSIGMOID,
    HARDSWISH, EXP_DST, LOGISTIC_DST, TANH_DST, ELU, GELU_TANH, CLIP_V2_DST, ELU_DST, RELU_DST, SQRT_DST, SWISH, SRELU,
    GELU_ERF, MISH
};

enum class ResOpsFunction {
    RES_EXT,
    RES_MUL,          // linearRes[m,o] = (a.b + bias)[m,n] . res[n,o] : a second matrix product
    RES_IDENTIAL,
    RES_ELTWISE_MUL   // extension: linearRes = (a.b + bias) * res, element by element
};

// flags of the normalisation layers (src/dnn/include/types/kudnn_normalization.hpp:18-29)
enum class NormalizationFlags : std::uint32_t {
    NONE = 0x0U,
    USE_GLOBAL_STATS = 0x1U,
    USE_SCALE = 0x2U,
    USE_SHIFT = 0x4U,
    FUSE_NORM_RELU = 0x8U
};
KUDNN_API_PUBLIC NormalizationFlags operator&(const NormalizationFlags &lhs, const NormalizationFlags &rhs);
KUDNN_API_PUBLIC NormalizationFlags operator|(const NormalizationFlags &lhs, const NormalizationFlags &rhs);
KUDNN_API_PUBLIC NormalizationFlags &operator&=(NormalizationFlags &lhs, const NormalizationFlags &rhs);
KUDNN_API_PUBLIC NormalizationFlags &operator|=(NormalizationFlags &lhs, const NormalizationFlags &rhs);

namespace Detail {
class LinearCore;
struct EltwiseState;
struct RmsNormState;
}

// Stand-alone activation pass (src/dnn/include/operations/kudnn_eltwise.hpp:62-76).  Forward functions implemented on
// the GPU: RELU, TANH, SIGMOID, GELU_TANH, SWISH, GELU_ERF; the others validate as UNSUPPORTED.  src and dst may be
// host memory, as in the reference, or device memory.
class KUDNN_API_PUBLIC ActivationLayerFWD final {
public:
    using SizeType = ::KuDNN::SizeType;
    static Status ValidateInput(const TensorInfo &srcInfo, const TensorInfo &dstInfo, ActivationFunction kind,
                                float alpha = 0.0f, float beta = 0.0f) noexcept(false);
    ActivationLayerFWD(const TensorInfo &srcInfo, const TensorInfo &dstInfo, ActivationFunction kind, float alpha = 0.0f,
                       float beta = 0.0f) noexcept(false);
    ActivationLayerFWD(const ActivationLayerFWD &other) noexcept(false);
    ActivationLayerFWD(ActivationLayerFWD &&other) noexcept;
    ActivationLayerFWD &operator=(const ActivationLayerFWD &other) noexcept(false);
    ActivationLayerFWD &operator=(ActivationLayerFWD &&other) noexcept;
    void Run(const void *src, void *dst) const noexcept(false);
    ~ActivationLayerFWD() noexcept;

    void SetStream(void *cudaStream) noexcept;  // extension: stream for device-pointer runs

private:
    std::unique_ptr<Detail::EltwiseState> pImpl;
};

// RMS normalisation over the last dimension (src/dnn/include/operations/kudnn_rms_normalization.hpp:26-44).  The
// reference accepts fp16 tensors only; bf16 and fp32 are accepted here as well.  The last logical dimension must be
// the innermost one in memory.
class KUDNN_API_PUBLIC RMSNormalizationLayerFWD final {
public:
    using SizeType = ::KuDNN::SizeType;
    static Status ValidateInput(const TensorInfo &srcInfo, const TensorInfo &statsInfo, const TensorInfo &scaleInfo,
                                const TensorInfo &dstInfo, NormalizationFlags flags) noexcept(false);
    RMSNormalizationLayerFWD(const TensorInfo &srcInfo, const TensorInfo &statsInfo, const TensorInfo &scaleInfo,
                             const TensorInfo &dstInfo, NormalizationFlags flags) noexcept(false);
    RMSNormalizationLayerFWD(const RMSNormalizationLayerFWD &other) noexcept(false);
    RMSNormalizationLayerFWD(RMSNormalizationLayerFWD &&other) noexcept;
    RMSNormalizationLayerFWD &operator=(const RMSNormalizationLayerFWD &other) noexcept(false);
    RMSNormalizationLayerFWD &operator=(RMSNormalizationLayerFWD &&other) noexcept;
    void Run(const void *src, void *dst, const void *scale, float *variance, bool saveStats, const float eps) const
        noexcept(false);
    ~RMSNormalizationLayerFWD() noexcept;

    void SetStream(void *cudaStream) noexcept;

private:
    std::unique_ptr<Detail::RmsNormState> pImpl;
};

class KUDNN_API_PUBLIC Gemm final {
public:
    using SizeType = ::KuDNN::SizeType;
    static Status ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                const TensorInfo &biasInfo, int numThreads = 0) noexcept;
    static Status ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                int numThreads = 0) noexcept;
    Gemm(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo, const TensorInfo &biasInfo,
         int numThreads = 0) noexcept(false);
    Gemm(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo, int numThreads = 0) noexcept(false);
    Gemm(const Gemm &other) noexcept(false);
    Gemm(Gemm &&other) noexcept;
    Gemm &operator=(const Gemm &other) noexcept(false);
    Gemm &operator=(Gemm &&other) noexcept;
    void Run(const void *a, const void *b, void *c, const void *bias, float alpha = 1.0f, float beta = 0.0f,
             int numThreads = 0) const noexcept(false);
    void Run(const void *a, const void *b, void *c, float alpha = 1.0f, float beta = 0.0f, int numThreads = 0) const
        noexcept(false);
    ~Gemm() noexcept;

    // extensions
    void PrepackWeights(const void *b) const noexcept(false);  // pack once; later Run(.., b, ..) reuses the packed copy
    void SetStream(void *cudaStream) noexcept;                 // stream for device-pointer runs (default: stream 0)
    int LastKernel() const noexcept;                           // KUDNN_B200_KERNEL_* of the most recent Run
    // Host-pointer runs are split over this machine's GPUs from now on: `shards` pieces of the rows (byColumns =
    // false) or of the columns of the layer, shard i on device i modulo the device count.  0 switches it off.
    void SetSharding(int shards, bool byColumns = false) noexcept;

private:
    std::unique_ptr<Detail::LinearCore> pImpl;
};

class KUDNN_API_PUBLIC LinearActivationLayerFWD final {
public:
    using SizeType = ::KuDNN::SizeType;
    static Status ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                const TensorInfo &biasInfo, float alpha = 1.0f, float beta = 0.0f,
                                ActivationFunction kind = KuDNN::ActivationFunction::RELU,
                                int numThreads = 0) noexcept(false);
    static Status ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                float alpha = 1.0f, float beta = 0.0f,
                                ActivationFunction kind = KuDNN::ActivationFunction::RELU,
                                int numThreads = 0) noexcept(false);
    LinearActivationLayerFWD(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                             const TensorInfo &biasInfo, float alpha = 1.0f, float beta = 0.0f,
                             ActivationFunction kind = KuDNN::ActivationFunction::RELU,
                             int numThreads = 0) noexcept(false);
    LinearActivationLayerFWD(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                             float alpha = 1.0f, float beta = 0.0f,
                             ActivationFunction kind = KuDNN::ActivationFunction::RELU,
                             int numThreads = 0) noexcept(false);
    LinearActivationLayerFWD(const LinearActivationLayerFWD &other) noexcept(false);
    LinearActivationLayerFWD(LinearActivationLayerFWD &&other) noexcept;
    LinearActivationLayerFWD &operator=(const LinearActivationLayerFWD &other) noexcept(false);
    LinearActivationLayerFWD &operator=(LinearActivationLayerFWD &&other) noexcept;
    void Run(const void *a, const void *b, void *c, const void *bias, int numThreads = 0) const noexcept(false);
    // declared by the reference but never defined there (link error); defined here
    void Run(const void *a, const void *b, void *c, int numThreads = 0) const noexcept(false);
    ~LinearActivationLayerFWD() noexcept;

    void PrepackWeights(const void *b) const noexcept(false);
    void SetStream(void *cudaStream) noexcept;
    int LastKernel() const noexcept;

private:
    std::unique_ptr<Detail::LinearCore> pImpl;
};

class KUDNN_API_PUBLIC LinearResFWD final {
public:
    using SizeType = ::KuDNN::SizeType;
    static Status ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                const TensorInfo &biasInfo, const TensorInfo &resInfo, const TensorInfo &linearResInfo,
                                float alpha = 1.0f, float beta = 0.0f, float gamma = 1.0f,
                                ResOpsFunction kind = ResOpsFunction::RES_IDENTIAL, int numThreads = 0) noexcept(false);
    static Status ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                const TensorInfo &res, const TensorInfo &linearRes, float alpha = 1.0f,
                                float beta = 0.0f, float gamma = 1.0f,
                                ResOpsFunction kind = ResOpsFunction::RES_IDENTIAL, int numThreads = 0) noexcept(false);
    LinearResFWD(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo, const TensorInfo &biasInfo,
                 const TensorInfo &res, const TensorInfo &linearRes, float alpha = 1.0f, float beta = 0.0f,
                 float gamma = 1.0f, ResOpsFunction kind = ResOpsFunction::RES_IDENTIAL,
                 int numThreads = 0) noexcept(false);
    LinearResFWD(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo, const TensorInfo &res,
                 const TensorInfo &linearRes, float alpha = 1.0f, float beta = 0.0f, float gamma = 1.0f,
                 ResOpsFunction kind = ResOpsFunction::RES_IDENTIAL, int numThreads = 0) noexcept(false);
    LinearResFWD(const LinearResFWD &other) noexcept(false);
    LinearResFWD(LinearResFWD &&other) noexcept;
    LinearResFWD &operator=(const LinearResFWD &other) noexcept(false);
    LinearResFWD &operator=(LinearResFWD &&other) noexcept;
    void Run(const void *a, const void *b, void *c, const void *bias, const void *res, void *linearRes,
             float gamma = 1.0f, int numThreads = 0) const noexcept(false);
    void Run(const void *a, const void *b, void *c, const void *res, void *linearRes, float gamma = 1.0f,
             int numThreads = 0) const noexcept(false);
    ~LinearResFWD() noexcept;

    void PrepackWeights(const void *b) const noexcept(false);
    void SetStream(void *cudaStream) noexcept;
    int LastKernel() const noexcept;

private:
    std::unique_ptr<Detail::LinearCore> pImpl;
    std::unique_ptr<Detail::LinearCore> pMul;  // second product of RES_MUL
};

// Extension: c = act(a.b + bias) and linearRes = c (+) res in one pass over the output.  The reference needs two
// operators (LinearActivationLayerFWD, then the residual half of LinearResFWD) and two more passes for this.
class KUDNN_API_PUBLIC LinearActivationResFWD final {
public:
    static Status ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                const TensorInfo &biasInfo, const TensorInfo &resInfo, const TensorInfo &linearResInfo,
                                float actAlpha, ActivationFunction actKind, float gamma, ResOpsFunction resKind,
                                int numThreads = 0) noexcept(false);
    LinearActivationResFWD(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                           const TensorInfo &biasInfo, const TensorInfo &resInfo, const TensorInfo &linearResInfo,
                           float actAlpha = 1.0f, ActivationFunction actKind = ActivationFunction::RELU,
                           float gamma = 1.0f, ResOpsFunction resKind = ResOpsFunction::RES_IDENTIAL,
                           int numThreads = 0) noexcept(false);
    LinearActivationResFWD(const LinearActivationResFWD &other) noexcept(false);
    LinearActivationResFWD(LinearActivationResFWD &&other) noexcept;
    ~LinearActivationResFWD() noexcept;
    // c may be nullptr when only linearRes is wanted; bias is nullptr iff biasInfo is empty
    void Run(const void *a, const void *b, void *c, const void *bias, const void *res, void *linearRes,
             float gamma = 1.0f, int numThreads = 0) const noexcept(false);
    void PrepackWeights(const void *b) const noexcept(false);
    void SetStream(void *cudaStream) noexcept;
    int LastKernel() const noexcept;

private:
    std::unique_ptr<Detail::LinearCore> pImpl;
};

}  // namespace KuDNN

#endif  // KUDNN_B200_HOST_KUDNN_HPP
