// Host side of the KuDNN Linear API over the C ABI of the CUDA library.
//
// What the reference does in src/dnn/src/kudnn_tensor_info.cpp, service.cpp, kudnn_gemm.cpp (validation and the
// public methods, :384-476, :884-942), kudnn_linear_activationlayer.cpp and kudnn_linear_res.cpp is restated here:
// descriptor arithmetic, validation in the reference's order with the reference's Status results, exceptions through
// ThrowOnStatus.  The arithmetic itself happens behind kudnn_b200_linear_run*.
#include "kudnn.hpp"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "kudnn_b200.h"

namespace KuDNN {

// ------------------------------------------------------------------------------------------------ Service

namespace Service {

void ThrowOnStatus(Status s, const std::string &funcName) noexcept(false)
{
    if (s == Status::UNSUPPORTED) {
        throw Unsupported{funcName + ": unsupported configuration of parameters"};
    }
    if (s == Status::BAD_ARGUMENTS) {
        throw LogicError{funcName + ": bad arguments' Shapes"};
    }
}

void *AlignedAlloc(SizeType n, SizeType alignment) noexcept(false)
{
    if (alignment == 0 || (alignment & (alignment - 1)) != 0) {
        throw LogicError("KuDNN alignment isn't a power of 2");
    }
    if (n > std::numeric_limits<std::size_t>::max() - alignment) {
        throw BadArrayNewLength();
    }
    const SizeType rounded = (n + alignment - 1) / alignment * alignment;
    void *p = ::aligned_alloc(alignment, rounded == 0 ? alignment : rounded);
    if (p == nullptr) {
        throw BadAlloc();
    }
    return p;
}

void Deallocate(void *p, SizeType) noexcept
{
    std::free(p);
}

namespace {

// memory order of the logical dimensions of every layout, slowest first, indexed by the enumerator value
const char *const kLayoutOrder[] = {
    "",      "A",     "AB",    "BA",    "ABC",   "ACB",   "BAC",   "BCA",   "CAB",   "CBA",   "ABCD",
    "ABDC",  "ACBD",  "ACDB",  "ADBC",  "ADCB",  "BACD",  "BCDA",  "CDAB",  "CDBA",  "DCAB",  "ABCDE",
    "ABCED", "ABDEC", "ACBDE", "ACDEB", "ADECB", "BACDE", "BCDEA", "CDEAB", "CDEBA", "DECAB",
};
constexpr int kNumLayouts = static_cast<int>(sizeof(kLayoutOrder) / sizeof(kLayoutOrder[0]));

const char *LayoutOrder(Layout l) noexcept
{
    const int v = static_cast<int>(l);
    return (v > 0 && v < kNumLayouts) ? kLayoutOrder[v] : "";
}

}  // namespace

SizeType GetLayoutRank(Layout l) noexcept
{
    return std::strlen(LayoutOrder(l));
}

SizeType GetIdxForUserLayout(Layout l, SizeType idx) noexcept(false)
{
    const char *order = LayoutOrder(l);
    if (idx >= std::strlen(order)) {
        throw LogicError("Shape: index >= layout size");
    }
    return static_cast<SizeType>(order[idx] - 'A');
}

Shape FlushStrides(const Shape &dims, const Shape &strides) noexcept(false)
{
    if (dims.GetNumDims() != strides.GetNumDims()) {
        throw LogicError{"FlushStrides: dims and strides have different dimensionality"};
    }
    Shape out = strides;
    for (SizeType i = 0; i < dims.GetNumDims(); ++i) {
        if (dims[i] == 1) {
            out[i] = 0;
        }
    }
    return out;
}

}  // namespace Service

// ------------------------------------------------------------------------------------------------ Threading

namespace Threading {

namespace {

int DefaultMaxThreads() noexcept
{
    int cores = static_cast<int>(std::thread::hardware_concurrency());
    if (cores <= 0) {
        cores = 1;
    }
    if (const char *env = std::getenv("KUDNN_MAX_NUM_THREADS")) {
        const long v = std::atol(env);
        if (v > 0) {
            return static_cast<int>(std::min<long>(v, cores));
        }
    }
    return cores;
}

std::atomic<int> g_maxThreads{DefaultMaxThreads()};

}  // namespace

int SetMaxNumThreads(int nThreads) noexcept
{
    const int old = g_maxThreads.load();
    const int cores = std::max(1, static_cast<int>(std::thread::hardware_concurrency()));
    if (nThreads > 0 && nThreads <= cores) {
        g_maxThreads.store(nThreads);
    }
    return old;
}

int GetMaxNumThreads() noexcept
{
    return g_maxThreads.load();
}

}  // namespace Threading

// ------------------------------------------------------------------------------------------------ TensorInfo

namespace {

template <bool kNoThrow>
typename std::conditional<kNoThrow, Status, void>::type Reject(const char *message) noexcept(kNoThrow)
{
    if constexpr (kNoThrow) {
        (void)message;
        return Status::BAD_ARGUMENTS;
    } else {
        throw Service::LogicError{message};
    }
}

}  // namespace

template <bool kNoThrow>
typename std::conditional<kNoThrow, Status, void>::type TensorInfo::ValidateElementType(Element::Type t) noexcept(kNoThrow)
{
    if (t == Element::TypeT::UNDEFINED) {
        return Reject<kNoThrow>("Tensor Info: Undefined data type of tensor");
    }
    if constexpr (kNoThrow) {
        return Status::SUCCESS;
    }
}

template <bool kNoThrow>
typename std::conditional<kNoThrow, Status, void>::type TensorInfo::ValidateLayout(Shape d, Layout l) noexcept(kNoThrow)
{
    const SizeType rank = d.GetNumDims();
    if (rank < 1 || rank > MAX_DIMS) {
        return Reject<kNoThrow>("Tensor Info: tensor dimensionality is incorrect");
    }
    if (Service::GetLayoutRank(l) != rank) {
        if constexpr (kNoThrow) {
            return Status::BAD_ARGUMENTS;
        } else {
            throw Service::LogicError{"Tensor Info: incorrect layout for " + std::to_string(rank) + "D tensor"};
        }
    }
    if constexpr (kNoThrow) {
        return Status::SUCCESS;
    }
}

template <bool kNoThrow>
typename std::conditional<kNoThrow, Status, void>::type TensorInfo::SetMinimumRequiredStrides(Shape d, Layout l,
                                                                                            Shape &s) noexcept(kNoThrow)
{
    const SizeType rank = d.GetNumDims();
    if (Service::GetLayoutRank(l) != rank || rank == 0) {
        return Reject<kNoThrow>("Tensor Info: layout wasn't processed");
    }
    SizeType strides[MAX_DIMS] = {0, 0, 0, 0, 0};
    SizeType running = 1;
    for (SizeType pos = rank; pos-- > 0;) {  // fastest dimension first
        const SizeType dim = Service::GetIdxForUserLayout(l, pos);
        strides[dim] = running;
        running *= d[dim];
    }
    for (SizeType i = 0; i < rank; ++i) {
        if (d[i] == 1) {
            strides[i] = 0;  // size-1 dimensions broadcast
        }
    }
    s.ResetShape(strides, rank);
    if constexpr (kNoThrow) {
        return Status::SUCCESS;
    }
}

template <bool kNoThrow>
typename std::conditional<kNoThrow, Status, void>::type TensorInfo::ValidateDimsAndStrides(Shape d, Layout l,
                                                                                         Shape s) noexcept(kNoThrow)
{
    if (d.GetNumDims() != s.GetNumDims()) {
        return Reject<kNoThrow>("Tensor Info: dims and strides have different dimensionality");
    }
    if constexpr (kNoThrow) {
        const Status st = ValidateLayout<true>(d, l);
        if (st != Status::SUCCESS) {
            return st;
        }
    } else {
        ValidateLayout<false>(d, l);
    }
    SizeType ext[MAX_DIMS] = {1, 1, 1, 1, 1};
    for (SizeType i = 0; i < d.GetNumDims(); ++i) {
        ext[i] = d[i];
    }
    if (Service::WillIntMultOverflow(ext, ext + d.GetNumDims())) {
        return Reject<kNoThrow>("TensorInfo: total size doesn't fit in SizeType");
    }
    Shape minimum;
    if constexpr (kNoThrow) {
        const Status st = SetMinimumRequiredStrides<true>(d, l, minimum);
        if (st != Status::SUCCESS) {
            return st;
        }
    } else {
        SetMinimumRequiredStrides<false>(d, l, minimum);
    }
    for (SizeType i = 0; i < d.GetNumDims(); ++i) {
        if (s[i] < minimum[i]) {
            return Reject<kNoThrow>("Tensor Info: incorrect strides");
        }
    }
    if constexpr (kNoThrow) {
        return Status::SUCCESS;
    }
}

template Status TensorInfo::ValidateElementType<true>(Element::Type) noexcept(true);
template void TensorInfo::ValidateElementType<false>(Element::Type) noexcept(false);
template Status TensorInfo::ValidateLayout<true>(Shape, Layout) noexcept(true);
template void TensorInfo::ValidateLayout<false>(Shape, Layout) noexcept(false);
template Status TensorInfo::SetMinimumRequiredStrides<true>(Shape, Layout, Shape &) noexcept(true);
template void TensorInfo::SetMinimumRequiredStrides<false>(Shape, Layout, Shape &) noexcept(false);
template Status TensorInfo::ValidateDimsAndStrides<true>(Shape, Layout, Shape) noexcept(true);
template void TensorInfo::ValidateDimsAndStrides<false>(Shape, Layout, Shape) noexcept(false);

TensorInfo::TensorInfo(const Shape &shape, const Element::Type &t, const Layout &l) noexcept(false)
    : dims(shape), type(t), layout(l), stridesInfo()
{
    ValidateElementType(type);
    ValidateLayout(dims, layout);
    SetMinimumRequiredStrides(dims, layout, stridesInfo);
}

TensorInfo::TensorInfo(const Shape &shape, const Element::Type &t, const Layout &l, const Shape &strides) noexcept(false)
    : dims(shape), type(t), layout(l), stridesInfo(strides)
{
    ValidateElementType(type);
    stridesInfo = Service::FlushStrides(dims, stridesInfo);
    ValidateDimsAndStrides(dims, layout, strides);
}

bool TensorInfo::IsDense() const noexcept
{
    Shape minimum;
    if (SetMinimumRequiredStrides<true>(dims, layout, minimum) != Status::SUCCESS) {
        return false;
    }
    return minimum == stridesInfo;
}

bool TensorInfo::HasStrideOverFastestDim() const noexcept
{
    const SizeType rank = dims.GetNumDims();
    if (rank == 0 || Service::GetLayoutRank(layout) != rank) {
        return false;
    }
    return stridesInfo[Service::GetIdxForUserLayout(layout, rank - 1)] > 1;
}

namespace {

Layout StandardLayout(SizeType rank, const Layout (&table)[5])
{
    if (rank < 1 || rank > 5) {
        throw Service::LogicError{"Tensor Info: tensor dimensionality is incorrect"};
    }
    return table[rank - 1];
}

}  // namespace

Layout TensorInfo::GetStandardABXLayout() const
{
    static const Layout t[5] = {Layout::A, Layout::AB, Layout::ABC, Layout::ABCD, Layout::ABCDE};
    return StandardLayout(dims.GetNumDims(), t);
}

Layout TensorInfo::GetStandardAXBLayout() const
{
    static const Layout t[5] = {Layout::A, Layout::AB, Layout::ACB, Layout::ACDB, Layout::ACDEB};
    return StandardLayout(dims.GetNumDims(), t);
}

Layout TensorInfo::GetStandardBXALayout() const
{
    static const Layout t[5] = {Layout::A, Layout::BA, Layout::BCA, Layout::BCDA, Layout::BCDEA};
    return StandardLayout(dims.GetNumDims(), t);
}

SizeType TensorInfo::GetAxisNumAccordingToLayout(SizeType axisNum) const noexcept(false)
{
    const SizeType rank = dims.GetNumDims();
    if (axisNum >= rank) {
        throw Service::LogicError{"Tensor Info: axisNum > tensor dimensionality"};
    }
    for (SizeType pos = 0; pos < rank; ++pos) {
        if (Service::GetIdxForUserLayout(layout, pos) == axisNum) {
            return pos;
        }
    }
    throw Service::LogicError{"Tensor Info: axisNum > tensor dimensionality"};
}

// ------------------------------------------------------------------------------------------------ validation

namespace {

bool IsEmpty(const TensorInfo &t) noexcept
{
    try {
        return t.GetTotalTensorSize() == 0;
    } catch (...) {
        return false;
    }
}

TensorInfo NoTensor(const TensorInfo &like)
{
    return TensorInfo(Shape{0}, like.GetType(), Layout::A);
}

SizeType FastestStride(const TensorInfo &t)
{
    const SizeType rank = t.GetNumDims();
    return t.GetStrides()[Service::GetIdxForUserLayout(t.GetLayout(), rank - 1)];
}

// src/dnn/src/kudnn_gemm.cpp:384-476, same checks in the same order
Status ValidateGemm(const TensorInfo &a, const TensorInfo &b, const TensorInfo &c, const TensorInfo &bias,
                    int numThreads) noexcept
{
    try {
        if (!c.IsDense()) {
            return Status::UNSUPPORTED;
        }
        if (a.GetType() == Element::TypeT::S32 || b.GetType() == Element::TypeT::S32) {
            return Status::UNSUPPORTED;
        }
        if (numThreads < 0 || numThreads > Threading::GetMaxNumThreads()) {
            return Status::BAD_ARGUMENTS;
        }
        const SizeType rank = a.GetNumDims();
        const bool noBias = IsEmpty(bias);
        if (rank != b.GetNumDims() || rank != c.GetNumDims() || (!noBias && rank != bias.GetNumDims()) || rank < 2) {
            return Status::BAD_ARGUMENTS;
        }
        const Shape ad = a.GetDims(), bd = b.GetDims(), cd = c.GetDims();
        if (ad[rank - 2] != cd[rank - 2] || ad[rank - 1] != bd[rank - 2] || bd[rank - 1] != cd[rank - 1]) {
            return Status::BAD_ARGUMENTS;
        }
        const Shape biasd = noBias ? Shape() : bias.GetDims();
        for (SizeType dim = 0; dim + 2 < rank; ++dim) {
            bool bad = false;
            if (ad[dim] != 1) {
                bad = bad || ad[dim] != cd[dim];
            }
            if (bd[dim] != 1 && ad[dim] != 1) {
                bad = bad || ad[dim] != bd[dim];
            }
            if (!noBias && biasd[dim] != 1) {
                bad = bad || biasd[dim] != cd[dim];
            }
            if (bad) {
                return Status::BAD_ARGUMENTS;
            }
        }
        if (!noBias && ((biasd[rank - 1] != 1 && biasd[rank - 1] != cd[rank - 1]) ||
                        (biasd[rank - 2] != 1 && biasd[rank - 2] != cd[rank - 2]))) {
            return Status::BAD_ARGUMENTS;
        }
        // the reference refuses only when every tensor has a non-unit stride on its fastest dimension
        auto strided = [](const TensorInfo &t) {
            const SizeType s = FastestStride(t);
            return s != 1 && s != 0;
        };
        if (strided(a) && strided(b) && strided(c) && !noBias && strided(bias)) {
            return Status::UNSUPPORTED;
        }
        if (a.GetTotalTensorSize() == 0 || b.GetTotalTensorSize() == 0 || c.GetTotalTensorSize() == 0) {
            return Status::UNSUPPORTED;
        }
        return Status::SUCCESS;
    } catch (...) {
        return Status::BAD_ARGUMENTS;
    }
}

bool IsOneOf(ActivationFunction k, std::initializer_list<ActivationFunction> set) noexcept
{
    return std::find(set.begin(), set.end(), k) != set.end();
}

// src/dnn/src/kudnn_eltwise.cpp:1479-1516 for src == dst == the Linear output
Status ValidateActivation(const TensorInfo &c, ActivationFunction kind, float alpha, float beta) noexcept
{
    using AF = ActivationFunction;
    const Element::TypeT t = c.GetType();
    const bool fp = t == Element::TypeT::F32 || t == Element::TypeT::F16 || t == Element::TypeT::BF16;
    if (!fp && !IsOneOf(kind, {AF::RELU, AF::LINEAR})) {
        return Status::UNSUPPORTED;
    }
    if (!IsOneOf(kind, {AF::ABS, AF::CLIP, AF::CLIP_V2, AF::ELU, AF::ELU_DST, AF::EXP, AF::GELU_ERF, AF::GELU_TANH,
                        AF::HARDSIGMOID, AF::HARDSWISH, AF::LINEAR, AF::LOG, AF::SIGMOID, AF::MISH, AF::POW, AF::RELU,
                        AF::ROUND, AF::SRELU, AF::SQRT, AF::SQUARE, AF::SWISH, AF::TANH})) {
        return Status::UNSUPPORTED;
    }
    if ((IsOneOf(kind, {AF::CLIP, AF::CLIP_V2}) && alpha > beta) || (kind == AF::SRELU && alpha == 0)) {
        return Status::UNSUPPORTED;
    }
    if (!c.IsDense() || IsEmpty(c)) {
        return Status::UNSUPPORTED;
    }
    // what the device epilogue implements; the rest of the reference's 22 functions is outside the Linear path
    if (!IsOneOf(kind, {AF::RELU, AF::SWISH, AF::GELU_TANH, AF::GELU_ERF, AF::SIGMOID, AF::TANH})) {
        return Status::UNSUPPORTED;
    }
    return Status::SUCCESS;
}

// src/dnn/src/kudnn_linear_res.cpp:136-166
Status ValidateRes(const TensorInfo &a, const TensorInfo &b, const TensorInfo &c, const TensorInfo &bias,
                   const TensorInfo &res, const TensorInfo &linearRes, ResOpsFunction kind, int numThreads) noexcept
{
    try {
        const Status st = ValidateGemm(a, b, c, bias, numThreads);
        if (st != Status::SUCCESS) {
            return st;
        }
        if (kind != ResOpsFunction::RES_EXT && kind != ResOpsFunction::RES_MUL && kind != ResOpsFunction::RES_IDENTIAL &&
            kind != ResOpsFunction::RES_ELTWISE_MUL) {
            return Status::UNSUPPORTED;
        }
        if (kind == ResOpsFunction::RES_MUL) {
            return ValidateGemm(c, res, linearRes, NoTensor(linearRes), numThreads);
        }
        const SizeType rank = c.GetNumDims();
        if (rank != res.GetNumDims() || rank != linearRes.GetNumDims()) {
            return Status::BAD_ARGUMENTS;
        }
        // the reference compares every dimension but the last; the device kernel also needs the last one to agree
        for (SizeType dim = 0; dim < rank; ++dim) {
            if (c.GetDims()[dim] != res.GetDims()[dim] || c.GetDims()[dim] != linearRes.GetDims()[dim]) {
                return Status::BAD_ARGUMENTS;
            }
        }
        return Status::SUCCESS;
    } catch (...) {
        return Status::BAD_ARGUMENTS;
    }
}

int DtypeCode(Element::TypeT t) noexcept
{
    switch (t) {
        case Element::TypeT::F32:
            return KUDNN_B200_F32;
        case Element::TypeT::F16:
            return KUDNN_B200_F16;
        case Element::TypeT::BF16:
            return KUDNN_B200_BF16;
        case Element::TypeT::S32:
            return KUDNN_B200_S32;
        case Element::TypeT::S8:
            return KUDNN_B200_S8;
        case Element::TypeT::U8:
            return KUDNN_B200_U8;
        default:
            return 100 + static_cast<int>(t);  // rejected by kudnn_b200_linear_validate as UNSUPPORTED
    }
}

int ActivationCode(ActivationFunction k) noexcept
{
    return static_cast<int>(k);  // the C ABI uses the enumerator values
}

struct Strides2 {
    int64_t row, col, batch[3];
};

// strides of the matrix dimensions (last two logical dims) and of up to three leading batch dims, right-aligned
Strides2 MatrixStrides(const TensorInfo &t)
{
    Strides2 s{};
    const SizeType rank = t.GetNumDims();
    const Shape st = t.GetStrides();
    s.row = static_cast<int64_t>(st[rank - 2]);
    s.col = static_cast<int64_t>(st[rank - 1]);
    for (SizeType i = 0; i + 2 < rank; ++i) {
        s.batch[3 - (rank - 2) + i] = static_cast<int64_t>(st[i]);
    }
    return s;
}

// TensorInfo quadruple (+ optional residual pair) -> C-ABI descriptor.  Layouts disappear into the strides.
kudnn_b200_linear_desc MakeDesc(const TensorInfo &a, const TensorInfo &b, const TensorInfo &c, const TensorInfo &bias,
                                const TensorInfo *res, const TensorInfo *out)
{
    kudnn_b200_linear_desc d;
    std::memset(&d, 0, sizeof(d));
    const SizeType rank = c.GetNumDims();
    const Shape cd = c.GetDims();
    d.m = static_cast<int64_t>(cd[rank - 2]);
    d.n = static_cast<int64_t>(cd[rank - 1]);
    d.k = static_cast<int64_t>(a.GetDims()[rank - 1]);
    for (SizeType i = 0; i + 2 < rank; ++i) {
        d.batch[3 - (rank - 2) + i] = static_cast<int64_t>(cd[i]);
    }
    d.a_dtype = DtypeCode(a.GetType());
    d.b_dtype = DtypeCode(b.GetType());
    d.c_dtype = DtypeCode(c.GetType());
    const Strides2 sa = MatrixStrides(a), sb = MatrixStrides(b), sc = MatrixStrides(c);
    d.a_sm = sa.row;
    d.a_sk = sa.col;
    d.b_sk = sb.row;
    d.b_sn = sb.col;
    d.c_sm = sc.row;
    d.c_sn = sc.col;
    // a dense 1 x n or m x 1 output has a flushed (0) stride on the size-1 dimension; give it its natural pitch
    if (d.c_sm == 0) {
        d.c_sm = d.n;
    }
    if (d.c_sn == 0) {
        d.c_sn = 1;
    }
    std::copy(sa.batch, sa.batch + 3, d.a_sb);
    std::copy(sb.batch, sb.batch + 3, d.b_sb);
    std::copy(sc.batch, sc.batch + 3, d.c_sb);
    d.bias_dtype = d.c_dtype;
    if (!IsEmpty(bias)) {
        d.has_bias = 1;
        d.bias_dtype = DtypeCode(bias.GetType());
        const Strides2 s = MatrixStrides(bias);
        d.bias_sm = s.row;
        d.bias_sn = s.col;
        std::copy(s.batch, s.batch + 3, d.bias_sb);
    }
    d.res_dtype = d.out_dtype = d.c_dtype;
    if (res != nullptr && out != nullptr) {
        d.res_dtype = DtypeCode(res->GetType());
        d.out_dtype = DtypeCode(out->GetType());
        const Strides2 sr = MatrixStrides(*res), so = MatrixStrides(*out);
        d.res_sm = sr.row;
        d.res_sn = sr.col;
        d.out_sm = so.row == 0 ? d.n : so.row;
        d.out_sn = so.col == 0 ? 1 : so.col;
        std::copy(sr.batch, sr.batch + 3, d.res_sb);
        std::copy(so.batch, so.batch + 3, d.out_sb);
    }
    d.act_alpha = 1.0f;
    return d;
}

[[noreturn]] void ThrowCabi(int status, const char *who)
{
    const std::string text = std::string(who) + ": " + kudnn_b200_last_error();
    switch (status) {
        case KUDNN_B200_UNSUPPORTED:
            throw Service::Unsupported{text};
        case KUDNN_B200_ALLOC_FAILED:
            throw Service::BadAlloc{};
        default:
            throw Service::LogicError{text};
    }
}

}  // namespace

// ------------------------------------------------------------------------------------------------ LinearCore

namespace Detail {

// One created C-ABI primitive plus what the public classes need to remember about it.
class LinearCore final {
public:
    LinearCore(const kudnn_b200_linear_desc &desc, bool hasBias, const char *who) : desc_(desc), hasBias_(hasBias), who_(who)
    {
        const int rc = kudnn_b200_linear_create(&desc_, &handle_);
        if (rc != KUDNN_B200_OK) {
            ThrowCabi(rc, who_);
        }
    }
    LinearCore(const LinearCore &other) : desc_(other.desc_), hasBias_(other.hasBias_), who_(other.who_), stream_(other.stream_)
    {
        const int rc = kudnn_b200_linear_clone(other.handle_, &handle_);
        if (rc != KUDNN_B200_OK) {
            ThrowCabi(rc, who_);
        }
    }
    LinearCore &operator=(const LinearCore &) = delete;
    ~LinearCore()
    {
        kudnn_b200_linear_destroy(handle_);
    }

    void CheckThreads(int numThreads) const
    {
        if (numThreads < 0 || numThreads > Threading::GetMaxNumThreads()) {
            throw Service::LogicError{std::string(who_) + ": numThreads is out of range"};
        }
    }

    void Run(const void *a, const void *b, void *c, const void *bias, const void *res, void *out, float alpha, float beta,
             float gamma) const
    {
        kudnn_b200_linear_args args;
        args.a = a;
        args.b = b;
        args.c = c;
        args.bias = bias;
        args.res = res;
        args.out = out;
        args.alpha = alpha;
        args.beta = beta;
        args.gamma = gamma;
        const int rc = shards_ > 0 ? kudnn_b200_linear_run_sharded(handle_, &args, shards_,
                                                                  shardColumns_ ? KUDNN_B200_SHARD_COLS : KUDNN_B200_SHARD_ROWS)
                                   : kudnn_b200_linear_run_any(handle_, &args, stream_);
        if (rc != KUDNN_B200_OK) {
            ThrowCabi(rc, who_);
        }
    }
    void SetSharding(int shards, bool byColumns) noexcept
    {
        shards_ = shards;
        shardColumns_ = byColumns;
    }

    void Prepack(const void *b) const
    {
        const int rc = kudnn_b200_linear_prepack(handle_, b, stream_);
        if (rc != KUDNN_B200_OK) {
            ThrowCabi(rc, who_);
        }
    }

    void SetStream(void *s) noexcept { stream_ = s; }
    int LastKernel() const noexcept { return kudnn_b200_linear_last_kernel(handle_); }
    bool HasBias() const noexcept { return hasBias_; }
    const kudnn_b200_linear_desc &Desc() const noexcept { return desc_; }

private:
    kudnn_b200_linear_desc desc_;
    kudnn_b200_linear_t handle_ = nullptr;
    bool hasBias_;
    const char *who_;
    void *stream_ = nullptr;
    int shards_ = 0;
    bool shardColumns_ = false;
};

}  // namespace Detail

namespace {

std::unique_ptr<Detail::LinearCore> CloneCore(const std::unique_ptr<Detail::LinearCore> &p)
{
    return p ? std::make_unique<Detail::LinearCore>(*p) : nullptr;
}

void CheckRunPointers(const Detail::LinearCore &core, const void *a, const void *b, const void *c, const void *bias,
                      const char *who)
{
    // src/dnn/src/kudnn_gemm.cpp:862-868
    if (a == nullptr || b == nullptr || c == nullptr || (core.HasBias() && bias == nullptr)) {
        throw Service::LogicError{std::string(who) + ": one of input matrices is nullptr"};
    }
    if (!core.HasBias() && bias != nullptr) {
        throw Service::LogicError{std::string(who) + ": bias isn't nullptr, but bias TensorInfo has 0 total size"};
    }
}

}  // namespace

// ------------------------------------------------------------------------------------------------ Gemm

Status Gemm::ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                           const TensorInfo &biasInfo, int numThreads) noexcept
{
    const Status st = ValidateGemm(aInfo, bInfo, cInfo, biasInfo, numThreads);
    if (st != Status::SUCCESS) {
        return st;
    }
    try {
        const kudnn_b200_linear_desc d = MakeDesc(aInfo, bInfo, cInfo, biasInfo, nullptr, nullptr);
        return static_cast<Status>(std::min(kudnn_b200_linear_validate(&d), 2));
    } catch (...) {
        return Status::BAD_ARGUMENTS;
    }
}

Status Gemm::ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                           int numThreads) noexcept
{
    try {
        return ValidateInput(aInfo, bInfo, cInfo, NoTensor(cInfo), numThreads);
    } catch (...) {
        return Status::BAD_ARGUMENTS;
    }
}

Gemm::Gemm(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo, const TensorInfo &biasInfo,
           int numThreads) noexcept(false)
{
    Service::ThrowOnStatus(ValidateInput(aInfo, bInfo, cInfo, biasInfo, numThreads), "GEMM");
    pImpl = std::make_unique<Detail::LinearCore>(MakeDesc(aInfo, bInfo, cInfo, biasInfo, nullptr, nullptr),
                                                 !IsEmpty(biasInfo), "Matmul Layer");
}

Gemm::Gemm(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo, int numThreads) noexcept(false)
    : Gemm(aInfo, bInfo, cInfo, NoTensor(cInfo), numThreads)
{
}

Gemm::Gemm(const Gemm &other) noexcept(false) : pImpl(CloneCore(other.pImpl)) {}
Gemm::Gemm(Gemm &&other) noexcept = default;
Gemm &Gemm::operator=(const Gemm &other) noexcept(false)
{
    if (this != &other) {
        pImpl = CloneCore(other.pImpl);
    }
    return *this;
}
Gemm &Gemm::operator=(Gemm &&other) noexcept = default;
Gemm::~Gemm() noexcept = default;

void Gemm::Run(const void *a, const void *b, void *c, const void *bias, float alpha, float beta, int numThreads) const
    noexcept(false)
{
    CheckRunPointers(*pImpl, a, b, c, bias, "Matmul Layer");
    pImpl->CheckThreads(numThreads);
    pImpl->Run(a, b, c, bias, nullptr, nullptr, alpha, beta, 1.0f);
}

void Gemm::Run(const void *a, const void *b, void *c, float alpha, float beta, int numThreads) const noexcept(false)
{
    Run(a, b, c, nullptr, alpha, beta, numThreads);
}

void Gemm::PrepackWeights(const void *b) const noexcept(false)
{
    pImpl->Prepack(b);
}
void Gemm::SetStream(void *cudaStream) noexcept
{
    pImpl->SetStream(cudaStream);
}
void Gemm::SetSharding(int shards, bool byColumns) noexcept
{
    pImpl->SetSharding(shards, byColumns);
}
int Gemm::LastKernel() const noexcept
{
    return pImpl->LastKernel();
}

// ------------------------------------------------------------------------------------------------ LinearActivationLayerFWD

Status LinearActivationLayerFWD::ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                               const TensorInfo &biasInfo, float alpha, float beta,
                                               ActivationFunction kind, int numThreads) noexcept(false)
{
    // Gemm first, then the activation: the order decides which Status a doubly wrong call reports
    const Status st = ValidateGemm(aInfo, bInfo, cInfo, biasInfo, numThreads);
    if (st != Status::SUCCESS) {
        return st;
    }
    const Status act = ValidateActivation(cInfo, kind, alpha, beta);
    if (act != Status::SUCCESS) {
        return act;
    }
    return Gemm::ValidateInput(aInfo, bInfo, cInfo, biasInfo, numThreads);
}

Status LinearActivationLayerFWD::ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                               float alpha, float beta, ActivationFunction kind,
                                               int numThreads) noexcept(false)
{
    return ValidateInput(aInfo, bInfo, cInfo, NoTensor(cInfo), alpha, beta, kind, numThreads);
}

LinearActivationLayerFWD::LinearActivationLayerFWD(const TensorInfo &aInfo, const TensorInfo &bInfo,
                                                   const TensorInfo &cInfo, const TensorInfo &biasInfo, float alpha,
                                                   float beta, ActivationFunction kind, int numThreads) noexcept(false)
{
    // the reference constructs its Gemm member first, so Gemm's message wins when both parts are wrong
    Service::ThrowOnStatus(ValidateGemm(aInfo, bInfo, cInfo, biasInfo, numThreads), "GEMM");
    Service::ThrowOnStatus(ValidateInput(aInfo, bInfo, cInfo, biasInfo, alpha, beta, kind, numThreads),
                           "LinearActivationLayerFWD");
    kudnn_b200_linear_desc d = MakeDesc(aInfo, bInfo, cInfo, biasInfo, nullptr, nullptr);
    d.act = ActivationCode(kind);
    d.act_alpha = alpha;  // the activation's parameter (relu slope, swish beta), not a GEMM scale
    d.act_beta = beta;
    pImpl = std::make_unique<Detail::LinearCore>(d, !IsEmpty(biasInfo), "LinearActivationLayerFWD");
}

LinearActivationLayerFWD::LinearActivationLayerFWD(const TensorInfo &aInfo, const TensorInfo &bInfo,
                                                   const TensorInfo &cInfo, float alpha, float beta,
                                                   ActivationFunction kind, int numThreads) noexcept(false)
    : LinearActivationLayerFWD(aInfo, bInfo, cInfo, NoTensor(cInfo), alpha, beta, kind, numThreads)
{
}

LinearActivationLayerFWD::LinearActivationLayerFWD(const LinearActivationLayerFWD &other) noexcept(false)
    : pImpl(CloneCore(other.pImpl))
{
}
LinearActivationLayerFWD::LinearActivationLayerFWD(LinearActivationLayerFWD &&other) noexcept = default;
LinearActivationLayerFWD &LinearActivationLayerFWD::operator=(const LinearActivationLayerFWD &other) noexcept(false)
{
    if (this != &other) {
        pImpl = CloneCore(other.pImpl);
    }
    return *this;
}
LinearActivationLayerFWD &LinearActivationLayerFWD::operator=(LinearActivationLayerFWD &&other) noexcept = default;
LinearActivationLayerFWD::~LinearActivationLayerFWD() noexcept = default;

void LinearActivationLayerFWD::Run(const void *a, const void *b, void *c, const void *bias, int numThreads) const
    noexcept(false)
{
    CheckRunPointers(*pImpl, a, b, c, bias, "Matmul Layer");
    pImpl->CheckThreads(numThreads);
    pImpl->Run(a, b, c, bias, nullptr, nullptr, 1.0f, 0.0f, 1.0f);  // the GEMM always runs with alpha 1, beta 0
}

void LinearActivationLayerFWD::Run(const void *a, const void *b, void *c, int numThreads) const noexcept(false)
{
    Run(a, b, c, nullptr, numThreads);
}

void LinearActivationLayerFWD::PrepackWeights(const void *b) const noexcept(false)
{
    pImpl->Prepack(b);
}
void LinearActivationLayerFWD::SetStream(void *cudaStream) noexcept
{
    pImpl->SetStream(cudaStream);
}
int LinearActivationLayerFWD::LastKernel() const noexcept
{
    return pImpl->LastKernel();
}

// ------------------------------------------------------------------------------------------------ LinearResFWD

Status LinearResFWD::ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                   const TensorInfo &biasInfo, const TensorInfo &resInfo, const TensorInfo &linearResInfo,
                                   float, float, float, ResOpsFunction kind, int numThreads) noexcept(false)
{
    const Status st = ValidateRes(aInfo, bInfo, cInfo, biasInfo, resInfo, linearResInfo, kind, numThreads);
    if (st != Status::SUCCESS) {
        return st;
    }
    try {
        kudnn_b200_linear_desc d = (kind == ResOpsFunction::RES_MUL)
                                       ? MakeDesc(aInfo, bInfo, cInfo, biasInfo, nullptr, nullptr)
                                       : MakeDesc(aInfo, bInfo, cInfo, biasInfo, &resInfo, &linearResInfo);
        if (kind != ResOpsFunction::RES_MUL) {
            d.res_op = KUDNN_B200_RES_IDENTICAL;
        }
        return static_cast<Status>(std::min(kudnn_b200_linear_validate(&d), 2));
    } catch (...) {
        return Status::BAD_ARGUMENTS;
    }
}

Status LinearResFWD::ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                   const TensorInfo &res, const TensorInfo &linearRes, float alpha, float beta,
                                   float gamma, ResOpsFunction kind, int numThreads) noexcept(false)
{
    return ValidateInput(aInfo, bInfo, cInfo, NoTensor(cInfo), res, linearRes, alpha, beta, gamma, kind, numThreads);
}

LinearResFWD::LinearResFWD(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                           const TensorInfo &biasInfo, const TensorInfo &res, const TensorInfo &linearRes, float alpha,
                           float beta, float gamma, ResOpsFunction kind, int numThreads) noexcept(false)
{
    Service::ThrowOnStatus(ValidateGemm(aInfo, bInfo, cInfo, biasInfo, numThreads), "GEMM");
    Service::ThrowOnStatus(ValidateInput(aInfo, bInfo, cInfo, biasInfo, res, linearRes, alpha, beta, gamma, kind, numThreads),
                           "LinearResFWD");
    const bool hasBias = !IsEmpty(biasInfo);
    if (kind == ResOpsFunction::RES_MUL) {
        // (a.b + bias)[m,n] . res[n,o]: two products; the second reads the rounded first output, as the reference does
        pImpl = std::make_unique<Detail::LinearCore>(MakeDesc(aInfo, bInfo, cInfo, biasInfo, nullptr, nullptr), hasBias,
                                                     "LinearResFWD");
        pMul = std::make_unique<Detail::LinearCore>(MakeDesc(cInfo, res, linearRes, NoTensor(linearRes), nullptr, nullptr),
                                                    false, "LinearResFWD");
        return;
    }
    kudnn_b200_linear_desc d = MakeDesc(aInfo, bInfo, cInfo, biasInfo, &res, &linearRes);
    d.res_op = kind == ResOpsFunction::RES_EXT        ? KUDNN_B200_RES_EXT
               : kind == ResOpsFunction::RES_IDENTIAL ? KUDNN_B200_RES_IDENTICAL
                                                      : KUDNN_B200_RES_ELTWISE_MUL;
    pImpl = std::make_unique<Detail::LinearCore>(d, hasBias, "LinearResFWD");
}

LinearResFWD::LinearResFWD(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                           const TensorInfo &res, const TensorInfo &linearRes, float alpha, float beta, float gamma,
                           ResOpsFunction kind, int numThreads) noexcept(false)
    : LinearResFWD(aInfo, bInfo, cInfo, NoTensor(cInfo), res, linearRes, alpha, beta, gamma, kind, numThreads)
{
}

LinearResFWD::LinearResFWD(const LinearResFWD &other) noexcept(false)
    : pImpl(CloneCore(other.pImpl)), pMul(CloneCore(other.pMul))
{
}
LinearResFWD::LinearResFWD(LinearResFWD &&other) noexcept = default;
LinearResFWD &LinearResFWD::operator=(const LinearResFWD &other) noexcept(false)
{
    if (this != &other) {
        pImpl = CloneCore(other.pImpl);
        pMul = CloneCore(other.pMul);
    }
    return *this;
}
LinearResFWD &LinearResFWD::operator=(LinearResFWD &&other) noexcept = default;
LinearResFWD::~LinearResFWD() noexcept = default;

void LinearResFWD::Run(const void *a, const void *b, void *c, const void *bias, const void *res, void *linearRes,
                       float gamma, int numThreads) const noexcept(false)
{
    CheckRunPointers(*pImpl, a, b, c, bias, "Matmul Layer");
    if (res == nullptr || linearRes == nullptr) {
        throw Service::LogicError{"Matmul Layer: one of input matrices is nullptr"};
    }
    pImpl->CheckThreads(numThreads);
    if (pMul) {
        pImpl->Run(a, b, c, bias, nullptr, nullptr, 1.0f, 0.0f, 1.0f);
        pMul->Run(c, res, linearRes, nullptr, nullptr, nullptr, 1.0f, 0.0f, 1.0f);
        return;
    }
    // gamma comes from this call, not from the constructor (src/dnn/src/kudnn_linear_res.cpp:184, :271)
    pImpl->Run(a, b, c, bias, res, linearRes, 1.0f, 0.0f, gamma);
}

void LinearResFWD::Run(const void *a, const void *b, void *c, const void *res, void *linearRes, float gamma,
                       int numThreads) const noexcept(false)
{
    Run(a, b, c, nullptr, res, linearRes, gamma, numThreads);
}

void LinearResFWD::PrepackWeights(const void *b) const noexcept(false)
{
    pImpl->Prepack(b);
}
void LinearResFWD::SetStream(void *cudaStream) noexcept
{
    pImpl->SetStream(cudaStream);
    if (pMul) {
        pMul->SetStream(cudaStream);
    }
}
int LinearResFWD::LastKernel() const noexcept
{
    return pImpl->LastKernel();
}

// ------------------------------------------------------------------------------------------------ LinearActivationResFWD

Status LinearActivationResFWD::ValidateInput(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                             const TensorInfo &biasInfo, const TensorInfo &resInfo,
                                             const TensorInfo &linearResInfo, float actAlpha, ActivationFunction actKind,
                                             float gamma, ResOpsFunction resKind, int numThreads) noexcept(false)
{
    if (resKind == ResOpsFunction::RES_MUL) {
        return Status::UNSUPPORTED;  // a second matrix product cannot be fused into the first one's epilogue
    }
    const Status st = LinearActivationLayerFWD::ValidateInput(aInfo, bInfo, cInfo, biasInfo, actAlpha, 0.0f, actKind, numThreads);
    if (st != Status::SUCCESS) {
        return st;
    }
    return LinearResFWD::ValidateInput(aInfo, bInfo, cInfo, biasInfo, resInfo, linearResInfo, 1.0f, 0.0f, gamma, resKind,
                                       numThreads);
}

LinearActivationResFWD::LinearActivationResFWD(const TensorInfo &aInfo, const TensorInfo &bInfo, const TensorInfo &cInfo,
                                               const TensorInfo &biasInfo, const TensorInfo &resInfo,
                                               const TensorInfo &linearResInfo, float actAlpha, ActivationFunction actKind,
                                               float gamma, ResOpsFunction resKind, int numThreads) noexcept(false)
{
    Service::ThrowOnStatus(ValidateInput(aInfo, bInfo, cInfo, biasInfo, resInfo, linearResInfo, actAlpha, actKind, gamma,
                                         resKind, numThreads),
                           "LinearActivationResFWD");
    kudnn_b200_linear_desc d = MakeDesc(aInfo, bInfo, cInfo, biasInfo, &resInfo, &linearResInfo);
    d.act = ActivationCode(actKind);
    d.act_alpha = actAlpha;
    d.res_op = resKind == ResOpsFunction::RES_EXT        ? KUDNN_B200_RES_EXT
               : resKind == ResOpsFunction::RES_IDENTIAL ? KUDNN_B200_RES_IDENTICAL
                                                         : KUDNN_B200_RES_ELTWISE_MUL;
    pImpl = std::make_unique<Detail::LinearCore>(d, !IsEmpty(biasInfo), "LinearActivationResFWD");
}

LinearActivationResFWD::LinearActivationResFWD(const LinearActivationResFWD &other) noexcept(false)
    : pImpl(CloneCore(other.pImpl))
{
}
LinearActivationResFWD::LinearActivationResFWD(LinearActivationResFWD &&other) noexcept = default;
LinearActivationResFWD::~LinearActivationResFWD() noexcept = default;

void LinearActivationResFWD::Run(const void *a, const void *b, void *c, const void *bias, const void *res, void *linearRes,
                                 float gamma, int numThreads) const noexcept(false)
{
    if (a == nullptr || b == nullptr || res == nullptr || linearRes == nullptr || (pImpl->HasBias() && bias == nullptr) ||
        (!pImpl->HasBias() && bias != nullptr)) {
        throw Service::LogicError{"Matmul Layer: one of input matrices is nullptr"};
    }
    pImpl->CheckThreads(numThreads);
    pImpl->Run(a, b, c, bias, res, linearRes, 1.0f, 0.0f, gamma);
}

void LinearActivationResFWD::PrepackWeights(const void *b) const noexcept(false)
{
    pImpl->Prepack(b);
}
void LinearActivationResFWD::SetStream(void *cudaStream) noexcept
{
    pImpl->SetStream(cudaStream);
}
int LinearActivationResFWD::LastKernel() const noexcept
{
    return pImpl->LastKernel();
}

// ------------------------------------------------------------------------------------------------ NormalizationFlags

NormalizationFlags operator&(const NormalizationFlags &lhs, const NormalizationFlags &rhs)
{
    return static_cast<NormalizationFlags>(static_cast<std::uint32_t>(lhs) & static_cast<std::uint32_t>(rhs));
}
NormalizationFlags operator|(const NormalizationFlags &lhs, const NormalizationFlags &rhs)
{
    return static_cast<NormalizationFlags>(static_cast<std::uint32_t>(lhs) | static_cast<std::uint32_t>(rhs));
}
NormalizationFlags &operator&=(NormalizationFlags &lhs, const NormalizationFlags &rhs)
{
    lhs = lhs & rhs;
    return lhs;
}
NormalizationFlags &operator|=(NormalizationFlags &lhs, const NormalizationFlags &rhs)
{
    lhs = lhs | rhs;
    return lhs;
}

// ------------------------------------------------------------------------------------------------ ActivationLayerFWD

namespace Detail {
struct EltwiseState {
    int64_t count;
    int srcType, dstType, kind;
    float alpha;
    void *stream = nullptr;
};
struct RmsNormState {
    int64_t rows, axis;
    int type, flags;
    void *stream = nullptr;
};
}  // namespace Detail

// The checks of the reference in its order (src/dnn/src/kudnn_eltwise.cpp:1479-1516); functions and element types the
// GPU path does not implement are UNSUPPORTED, the answer the reference gives for what it does not implement.
Status ActivationLayerFWD::ValidateInput(const TensorInfo &srcInfo, const TensorInfo &dstInfo, ActivationFunction kind,
                                         float alpha, float beta) noexcept(false)
{
    if (srcInfo.GetLayout() != dstInfo.GetLayout()) {
        return Status::BAD_ARGUMENTS;
    }
    const auto isFloat = [](Element::TypeT t) {
        return t == Element::TypeT::F32 || t == Element::TypeT::F16 || t == Element::TypeT::BF16;
    };
    if (!isFloat(srcInfo.GetType()) || !isFloat(dstInfo.GetType())) {
        return Status::UNSUPPORTED;  // the reference also takes S32 / S8 / U8 for RELU and LINEAR
    }
    switch (kind) {
        case ActivationFunction::RELU:
        case ActivationFunction::TANH:
        case ActivationFunction::SIGMOID:
        case ActivationFunction::GELU_TANH:
        case ActivationFunction::SWISH:
        case ActivationFunction::GELU_ERF:
            break;
        default:
            return Status::UNSUPPORTED;
    }
    (void)alpha;
    (void)beta;
    if (!srcInfo.IsDense() || !dstInfo.IsDense()) {
        return Status::UNSUPPORTED;
    }
    if (srcInfo.GetTotalTensorSize() == 0 || srcInfo.GetDims() != dstInfo.GetDims()) {
        return Status::UNSUPPORTED;
    }
    return Status::SUCCESS;
}

ActivationLayerFWD::ActivationLayerFWD(const TensorInfo &srcInfo, const TensorInfo &dstInfo, ActivationFunction kind,
                                       float alpha, float beta) noexcept(false)
{
    Service::ThrowOnStatus(ValidateInput(srcInfo, dstInfo, kind, alpha, beta), "Activation Layer");
    pImpl = std::make_unique<Detail::EltwiseState>();
    pImpl->count = static_cast<int64_t>(srcInfo.GetTotalTensorSize());
    pImpl->srcType = DtypeCode(srcInfo.GetType());
    pImpl->dstType = DtypeCode(dstInfo.GetType());
    pImpl->kind = ActivationCode(kind);
    pImpl->alpha = alpha;
}
ActivationLayerFWD::ActivationLayerFWD(const ActivationLayerFWD &other) noexcept(false)
    : pImpl(std::make_unique<Detail::EltwiseState>(*other.pImpl))
{
}
ActivationLayerFWD::ActivationLayerFWD(ActivationLayerFWD &&other) noexcept = default;
ActivationLayerFWD &ActivationLayerFWD::operator=(const ActivationLayerFWD &other) noexcept(false)
{
    if (this != &other) {
        pImpl = std::make_unique<Detail::EltwiseState>(*other.pImpl);
    }
    return *this;
}
ActivationLayerFWD &ActivationLayerFWD::operator=(ActivationLayerFWD &&other) noexcept = default;
ActivationLayerFWD::~ActivationLayerFWD() noexcept = default;

void ActivationLayerFWD::Run(const void *src, void *dst) const noexcept(false)
{
    if (src == nullptr || dst == nullptr) {
        throw Service::LogicError{"Activation Layer: one of input matrices is nullptr"};
    }
    const int rc = kudnn_b200_activation_run(src, dst, pImpl->count, pImpl->srcType, pImpl->dstType, pImpl->kind,
                                             pImpl->alpha, pImpl->stream);
    if (rc != KUDNN_B200_OK) {
        ThrowCabi(rc, "Activation Layer");
    }
}
void ActivationLayerFWD::SetStream(void *cudaStream) noexcept
{
    pImpl->stream = cudaStream;
}

// ------------------------------------------------------------------------------------------------ RMSNormalizationLayerFWD

// src/dnn/src/kudnn_rms_normalization_fwd.cpp:333-369, check for check; bf16 and fp32 pass the type checks as well.
Status RMSNormalizationLayerFWD::ValidateInput(const TensorInfo &srcInfo, const TensorInfo &statsInfo,
                                               const TensorInfo &scaleInfo, const TensorInfo &dstInfo,
                                               NormalizationFlags flags) noexcept(false)
{
    if (static_cast<bool>(flags & NormalizationFlags::FUSE_NORM_RELU)) {
        return Status::UNSUPPORTED;
    }
    if (srcInfo.GetDims() != dstInfo.GetDims()) {
        return Status::BAD_ARGUMENTS;
    }
    const Element::TypeT t = srcInfo.GetType();
    if ((t != Element::TypeT::F16 && t != Element::TypeT::BF16 && t != Element::TypeT::F32) || dstInfo.GetType() != t) {
        return Status::UNSUPPORTED;
    }
    if (static_cast<bool>(flags & NormalizationFlags::USE_SCALE) && scaleInfo.GetType() != t) {
        return Status::UNSUPPORTED;
    }
    if ((srcInfo.GetNumDims() - 1) != statsInfo.GetNumDims()) {
        return Status::BAD_ARGUMENTS;
    }
    if (srcInfo.GetTotalTensorSize() == 0) {
        return Status::UNSUPPORTED;
    }
    if (scaleInfo.GetNumDims() != 1) {
        return Status::BAD_ARGUMENTS;
    }
    if (srcInfo.GetDims()[srcInfo.GetNumDims() - 1] != scaleInfo.GetDims()[0]) {
        return Status::BAD_ARGUMENTS;
    }
    for (SizeType i = 0; i < statsInfo.GetNumDims(); ++i) {
        if (srcInfo.GetDims()[i] != statsInfo.GetDims()[i]) {
            return Status::BAD_ARGUMENTS;
        }
    }
    if (!srcInfo.IsDense() || !statsInfo.IsDense() || !scaleInfo.IsDense() || !dstInfo.IsDense()) {
        return Status::UNSUPPORTED;
    }
    // the GPU kernel normalises rows that are contiguous in memory: plain row-major tensors
    if (srcInfo.GetLayout() != srcInfo.GetStandardABXLayout() || dstInfo.GetLayout() != srcInfo.GetLayout() ||
        statsInfo.GetLayout() != statsInfo.GetStandardABXLayout()) {
        return Status::UNSUPPORTED;
    }
    return Status::SUCCESS;
}

RMSNormalizationLayerFWD::RMSNormalizationLayerFWD(const TensorInfo &srcInfo, const TensorInfo &statsInfo,
                                                   const TensorInfo &scaleInfo, const TensorInfo &dstInfo,
                                                   NormalizationFlags flags) noexcept(false)
{
    Service::ThrowOnStatus(ValidateInput(srcInfo, statsInfo, scaleInfo, dstInfo, flags), "Normalization Layer");
    pImpl = std::make_unique<Detail::RmsNormState>();
    pImpl->axis = static_cast<int64_t>(srcInfo.GetDims()[srcInfo.GetNumDims() - 1]);
    pImpl->rows = static_cast<int64_t>(srcInfo.GetTotalTensorSize()) / pImpl->axis;
    pImpl->type = DtypeCode(srcInfo.GetType());
    pImpl->flags = static_cast<int>(static_cast<std::uint32_t>(flags));
}
RMSNormalizationLayerFWD::RMSNormalizationLayerFWD(const RMSNormalizationLayerFWD &other) noexcept(false)
    : pImpl(std::make_unique<Detail::RmsNormState>(*other.pImpl))
{
}
RMSNormalizationLayerFWD::RMSNormalizationLayerFWD(RMSNormalizationLayerFWD &&other) noexcept = default;
RMSNormalizationLayerFWD &RMSNormalizationLayerFWD::operator=(const RMSNormalizationLayerFWD &other) noexcept(false)
{
    if (this != &other) {
        pImpl = std::make_unique<Detail::RmsNormState>(*other.pImpl);
    }
    return *this;
}
RMSNormalizationLayerFWD &RMSNormalizationLayerFWD::operator=(RMSNormalizationLayerFWD &&other) noexcept = default;
RMSNormalizationLayerFWD::~RMSNormalizationLayerFWD() noexcept = default;

void RMSNormalizationLayerFWD::Run(const void *src, void *dst, const void *scale, float *variance, bool saveStats,
                                   const float eps) const noexcept(false)
{
    // src/dnn/src/kudnn_rms_normalization_fwd.cpp:213-226
    if (src == nullptr || dst == nullptr) {
        throw Service::LogicError{"Normalization: one of input matrices is nullptr"};
    }
    if (((pImpl->flags & KUDNN_B200_NORM_USE_GLOBAL_STATS) != 0 || saveStats) && variance == nullptr) {
        throw Service::LogicError{"Normalization: one of input matrices is nullptr"};
    }
    if ((pImpl->flags & KUDNN_B200_NORM_USE_SCALE) != 0 && scale == nullptr) {
        throw Service::LogicError{"Normalization Layer: one of input matrices is nullptr"};
    }
    const int rc = kudnn_b200_rmsnorm_run(src, dst, scale, variance, pImpl->rows, pImpl->axis, pImpl->type, pImpl->flags,
                                          saveStats ? 1 : 0, eps, pImpl->stream);
    if (rc != KUDNN_B200_OK) {
        ThrowCabi(rc, "Normalization Layer");
    }
}
void RMSNormalizationLayerFWD::SetStream(void *cudaStream) noexcept
{
    pImpl->stream = cudaStream;
}

}  // namespace KuDNN
