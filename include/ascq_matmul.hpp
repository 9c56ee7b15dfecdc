// C++ host mirror of the Ascend C Matmul object (include/adv_api/matmul/matmul.h:79-398, MX form
// impl/adv_api/detail/matmul/mx_matmul_impl.h:135-171) on top of the C ABI (ascq.h).
//
// The reference object lives inside a device kernel and computes one core's singleCoreM x singleCoreN block of
// C = A . B (+ bias) from global-memory operands.  Here the same protocol
//     Init / SetOrgShape / SetSingleShape / SetTail / SetTensorA / SetTensorB / SetBias / SetQuantScalar / SetQuantVector /
//     SetAntiQuantScalar / SetAntiQuantVector / SetTensorScaleA / SetTensorScaleB / SetWorkspace ->
//     IterateAll  (or  while (Iterate()) GetTensorC(...))  -> End
// runs on the host and enqueues the matching library call on a CUDA stream; the whole single-core block is one
// "iteration".  Which call is taken follows from the operand types exactly as the reference picks its data path:
//
//   A x B -> C                                  what must be set                library call
//   int8 x int8 -> int32                        -                               ascq_matmul_w8a8 (accumulator output)
//   int8 x int8 -> half                         SetQuantScalar | SetQuantVector ascq_matmul_i8_quant   (DEQF16 / VDEQF16)
//   int8 x int8 -> int8 | uint8                 SetQuantScalar | SetQuantVector ascq_matmul_i8_requant (REQ8 / VREQ8)
//   half x half, bf16 x bf16 -> half|bf16|float -                               ascq_matmul_f16
//   half x half, bf16 x bf16 -> int8 | uint8    SetQuantScalar | SetQuantVector ascq_matmul_f16_quant  (QF322B8_PRE / VQF322B8_PRE)
//   half|bf16 x int8 -> half|bf16|float         SetAntiQuantScalar | ...Vector  ascq_matmul_w8a16 (needs SetWorkspace)
//   fp4x2_e2m1 x fp4x2_e2m1 (with scale) -> bf16     SetTensorScaleA / B        ascq_group_matmul_mxfp4 (one group; SetWorkspace)
//   fp8 x fp8 (with scale) -> bf16 | float           SetTensorScaleA / B        ascq_group_matmul_mxfp8 (one group; SetWorkspace)
//
// Layouts.  A is [M, Ka] row-major (isTransposeA = false).  B is taken K-major, [N, Kb], which is SetTensorB(gm, true);
// the reference's default [Kb, N] form is accepted for one-byte element types and for fp4 pairs when a workspace is
// set (it is turned once per IterateAll), and refused for 16-bit types.  scaleB likewise: [N, K/32] with
// isTransposeScaleB = true (the reference's default), the sample's [K/64, N, 2] form otherwise.
// Whatever the reference asserts, and every combination not listed above, throws ascq::Error.
//
// Header only; link against libascq.so.  No CUDA headers are needed: a stream is passed as void*.
#ifndef ASCQ_MATMUL_HPP_
#define ASCQ_MATMUL_HPP_

#include <cstring>
#include <type_traits>

#include "ascq_ascendc.hpp"

namespace ascq {
struct fp8_e4m3fn_t { uint8_t bits; };
struct fp8_e5m2_t { uint8_t bits; };
template <> struct DTypeOf<fp8_e4m3fn_t> { static constexpr ascq_dtype value = ASCQ_DT_FP8_E4M3; };
template <> struct DTypeOf<fp8_e5m2_t> { static constexpr ascq_dtype value = ASCQ_DT_FP8_E5M2; };
}  // namespace ascq

namespace AscendC {

using fp4x2_e2m1_t = ascq::fp4x2_e2m1_t;
using fp8_e8m0_t = ascq::fp8_e8m0_t;
using fp8_e4m3fn_t = ascq::fp8_e4m3fn_t;
using fp8_e5m2_t = ascq::fp8_e5m2_t;

// include/adv_api/matmul/matmul_tiling_base.h:101-145
enum class TPosition : int32_t { GM, A1, A2, B1, B2, C1, C2, CO1, CO2, VECIN, VECOUT, VECCALC, LCM = VECCALC, SPM, SHM = SPM, TSCM, MAX };
enum class CubeFormat : int32_t { ND = 0, NZ, ZN, ZZ, NN, ND_ALIGN, SCALAR, VECTOR, ROW_MAJOR = ND, COLUMN_MAJOR = 8 };

// impl/adv_api/detail/matmul/utils/matmul_type_def.h:36-46 and :110-117 (the members this mirror reads)
template <TPosition POSITION, CubeFormat FORMAT, typename TYPE, bool ISTRANS = false> struct MatmulType {
    constexpr static TPosition pos = POSITION;
    constexpr static CubeFormat format = FORMAT;
    using T = TYPE;
    constexpr static bool isTrans = ISTRANS;
    constexpr static bool hasScale = false;
};
template <TPosition POSITION, TPosition SCALE_POSITION, CubeFormat FORMAT, typename TYPE, bool ISTRANS = false>
struct MatmulTypeWithScale : MatmulType<POSITION, FORMAT, TYPE, ISTRANS> {
    constexpr static TPosition scalePosition = SCALE_POSITION;
    constexpr static bool hasScale = true;
};

// include/adv_api/matmul/matmul_tilingdata.h:21-72: the host-computed tiling blob, field for field.  The mirror reads
// M, N, Ka, Kb, singleCoreM / N / K and isBias; block sizes and buffer depths have no meaning on this hardware.
struct TCubeTiling {
    int32_t usedCoreNum = 1, M = 0, N = 0, Ka = 0, Kb = 0, singleCoreM = 0, singleCoreN = 0, singleCoreK = 0;
    int32_t baseM = 0, baseN = 0, baseK = 0, depthA1 = 0, depthB1 = 0, stepM = 0, stepN = 0, isBias = 0;
    int32_t transLength = 0, iterateOrder = 0, shareMode = 0, shareL1Size = 0, shareL0CSize = 0, shareUbSize = 0;
    int32_t batchM = 0, batchN = 0, singleBatchM = 0, singleBatchN = 0, stepKa = 0, stepKb = 0;
    int32_t depthAL1CacheUB = 0, depthBL1CacheUB = 0, dbL0A = 0, dbL0B = 0, dbL0C = 0;
    int32_t ALayoutInfoB = 0, ALayoutInfoS = 0, ALayoutInfoN = 0, ALayoutInfoG = 0, ALayoutInfoD = 0;
    int32_t BLayoutInfoB = 0, BLayoutInfoS = 0, BLayoutInfoN = 0, BLayoutInfoG = 0, BLayoutInfoD = 0;
    int32_t CLayoutInfoB = 0, CLayoutInfoS1 = 0, CLayoutInfoN = 0, CLayoutInfoG = 0, CLayoutInfoS2 = 0;
    int32_t BatchNum = 0, mxTypePara = 0;
};

template <class A_TYPE, class B_TYPE, class C_TYPE, class BIAS_TYPE = C_TYPE> class Matmul {
    using SrcAT = typename A_TYPE::T;
    using SrcBT = typename B_TYPE::T;
    using DstT = typename C_TYPE::T;
    using BiasT = typename BIAS_TYPE::T;
    using SrcT = SrcAT;

    template <typename X, typename... Ys> static constexpr bool one_of = (std::is_same<X, Ys>::value || ...);
    static constexpr bool kInt8 = std::is_same<SrcAT, int8_t>::value && std::is_same<SrcBT, int8_t>::value;
    static constexpr bool kFloat16 = one_of<SrcAT, half, bfloat16_t> && std::is_same<SrcAT, SrcBT>::value;
    static constexpr bool kWeightOnly = one_of<SrcAT, half, bfloat16_t> && std::is_same<SrcBT, int8_t>::value;
    static constexpr bool kMx = A_TYPE::hasScale && B_TYPE::hasScale;
    static constexpr bool kMxFp4 = kMx && std::is_same<SrcAT, fp4x2_e2m1_t>::value && std::is_same<SrcBT, fp4x2_e2m1_t>::value;
    static constexpr bool kMxFp8 = kMx && one_of<SrcAT, fp8_e4m3fn_t, fp8_e5m2_t> && one_of<SrcBT, fp8_e4m3fn_t, fp8_e5m2_t>;
    static_assert(A_TYPE::format == CubeFormat::ND && B_TYPE::format == CubeFormat::ND && C_TYPE::format == CubeFormat::ND,
                  "only row-major (ND) global-memory matrices are mirrored");
    static_assert(A_TYPE::hasScale == B_TYPE::hasScale, "both operands carry scales or neither does (isMxMatmul)");

public:
    Matmul() = default;

    // REGIST_MATMUL_OBJ(&pipe, workspace, obj, &tiling) of the reference boils down to Init(&tiling)
    void Init(const TCubeTiling* cubeTiling, void* /*tpipe*/ = nullptr)
    {
        if (!cubeTiling) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "Init: tiling is NULL");
        orgM_ = cubeTiling->M; orgN_ = cubeTiling->N; orgKa_ = cubeTiling->Ka; orgKb_ = cubeTiling->Kb; orgKc_ = 0;
        m_ = cubeTiling->singleCoreM ? cubeTiling->singleCoreM : cubeTiling->M;
        n_ = cubeTiling->singleCoreN ? cubeTiling->singleCoreN : cubeTiling->N;
        k_ = cubeTiling->singleCoreK ? cubeTiling->singleCoreK : cubeTiling->Ka;
        tilingBias_ = cubeTiling->isBias != 0;
        pending_ = true;
    }
    void SetOrgShape(int orgM, int orgN, int orgK) { SetOrgShape(orgM, orgN, orgK, orgK, 0); }
    void SetOrgShape(int orgM, int orgN, int orgKa, int orgKb, int orgKc = 0)
    {
        orgM_ = orgM; orgN_ = orgN; orgKa_ = orgKa; orgKb_ = orgKb; orgKc_ = orgKc;
        if (m_ <= 0) m_ = orgM;
        if (n_ <= 0) n_ = orgN;
        if (k_ <= 0) k_ = orgKa;
    }
    void SetSingleShape(int singleM, int singleN, int singleK) { SetTail(singleM, singleN, singleK); }
    void SetTail(int tailM = -1, int tailN = -1, int tailK = -1)
    {
        if (tailM != -1) m_ = tailM;
        if (tailN != -1) n_ = tailN;
        if (tailK != -1) k_ = tailK;
        pending_ = true;
    }
    void SetTensorA(const GlobalTensor<SrcAT>& gm, bool isTransposeA = false) { a_ = gm.ptr; transA_ = isTransposeA; pending_ = true; }
    void SetTensorB(const GlobalTensor<SrcBT>& gm, bool isTransposeB = false) { b_ = gm.ptr; transB_ = isTransposeB; pending_ = true; }
    void SetBias(const GlobalTensor<BiasT>& biasGlobal) { bias_ = biasGlobal.ptr; }
    void DisableBias() { bias_ = nullptr; }
    void ClearBias() { bias_ = nullptr; }
    void SetQuantScalar(const uint64_t quantScalar) { quantScalar_ = quantScalar; quantVector_ = nullptr; quantSet_ = true; }
    void SetQuantVector(const GlobalTensor<uint64_t>& quantTensor) { quantVector_ = quantTensor.ptr; quantSet_ = true; }
    // The scalars arrive as bit patterns of SrcT, as SetAntiQuantScalar(const SrcT, const SrcT) takes them
    void SetAntiQuantScalar(const SrcT offsetScalar, const SrcT scaleScalar)
    {
        aqOffsetScalar_ = to_float(offsetScalar); aqScaleScalar_ = to_float(scaleScalar);
        aqOffset_ = aqScale_ = nullptr; antiQuantSet_ = true;
    }
    void SetAntiQuantVector(const GlobalTensor<SrcT>& offsetTensor, const GlobalTensor<SrcT>& scaleTensor)
    {
        aqOffset_ = offsetTensor.ptr; aqScale_ = scaleTensor.ptr; antiQuantSet_ = true;
    }
    void SetTensorScaleA(const GlobalTensor<fp8_e8m0_t>& gm, bool isTransposeScaleA = false) { scaleA_ = gm.ptr; transScaleA_ = isTransposeScaleA; }
    void SetTensorScaleB(const GlobalTensor<fp8_e8m0_t>& gm, bool isTransposeScaleB = true) { scaleB_ = gm.ptr; transScaleB_ = isTransposeScaleB; }
    // Device scratch for the calls that need some (see the table above); stays with the caller.
    void SetWorkspace(GlobalTensor<uint8_t>& addr) { workspace_ = addr.ptr; workspaceBytes_ = addr.size; }
    template <class T> void SetWorkspace(const T* addr, int size) { workspace_ = reinterpret_cast<uint8_t*>(const_cast<T*>(addr)); workspaceBytes_ = size_t(size) * sizeof(T); }
    // Not part of the reference: the CUDA stream the calls are enqueued on (default stream when never set).
    void SetStream(void* stream) { stream_ = stream; }
    // How many bytes SetWorkspace must provide for the shapes and layouts set so far.
    size_t GetWorkspaceSize() const
    {
        size_t need = 0;
        if constexpr (kWeightOnly) need = ascq_matmul_w8a16_workspace_size(n_, k_);
        if constexpr (kMxFp4) need = ascq_group_matmul_mxfp4_workspace_size(m_, 1, k_, n_);
        if constexpr (kMxFp8) need = ascq_group_matmul_mxfp8_workspace_size(m_, 1, k_, n_);
        need = (need + 255) / 256 * 256;
        return need + turned_b_bytes() + turned_scale_b_bytes();
    }

    // One iteration covers the whole single-core block: true once after any Set*, then false.
    template <bool sync = true> bool Iterate(bool enPartialSum = false)
    {
        if (enPartialSum) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "Iterate: partial sums are not mirrored");
        const bool run = pending_;
        pending_ = false;
        haveBlock_ = run;
        return run;
    }
    template <bool sync = true>
    void GetTensorC(const GlobalTensor<DstT>& gm, uint8_t enAtomic = 0, bool enSequentialWrite = false)
    {
        if (!haveBlock_) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "GetTensorC without a preceding Iterate() that returned true");
        haveBlock_ = false;
        compute(gm, enAtomic, enSequentialWrite);
    }
    template <bool sync = true>
    void IterateAll(const GlobalTensor<DstT>& gm, uint8_t enAtomic = 0, bool enSequentialWrite = false, bool /*waitIterateAll*/ = false,
                    bool /*fakeMsg*/ = false)
    {
        pending_ = true;
        while (Iterate()) GetTensorC(gm, enAtomic, enSequentialWrite);
    }
    void End() { pending_ = false; haveBlock_ = false; }

private:
    static float to_float(half v)
    {
        const uint32_t s = (v.bits >> 15) & 1u, e = (v.bits >> 10) & 31u, m = v.bits & 1023u;
        uint32_t bits;
        if (e == 0) {
            if (m == 0) bits = s << 31;
            else {
                int sh = 0;
                uint32_t mm = m;
                while (!(mm & 1024u)) { mm <<= 1; ++sh; }
                bits = (s << 31) | (uint32_t(113 - sh) << 23) | ((mm & 1023u) << 13);
            }
        } else if (e == 31) bits = (s << 31) | 0x7F800000u | (m << 13);
        else bits = (s << 31) | ((e + 112u) << 23) | (m << 13);
        float f;
        std::memcpy(&f, &bits, 4);
        return f;
    }
    static float to_float(bfloat16_t v)
    {
        const uint32_t bits = uint32_t(v.bits) << 16;
        float f;
        std::memcpy(&f, &bits, 4);
        return f;
    }
    template <typename X> static float to_float(X) { return 0.f; }

    size_t turned_b_bytes() const
    {
        if (transB_) return 0;
        const size_t bytes = kMxFp4 ? size_t(n_) * k_ / 2 : size_t(n_) * k_ * sizeof(SrcBT);
        return (bytes + 255) / 256 * 256;
    }
    size_t turned_scale_b_bytes() const { return (kMx && !transScaleB_) ? (size_t(n_) * (k_ / 32) + 255) / 256 * 256 : 0; }

    void compute(const GlobalTensor<DstT>& gm, uint8_t enAtomic, bool enSequentialWrite)
    {
        using ascq::check;
        if (enAtomic != 0) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "atomic accumulation into C is not mirrored");
        if (!a_ || !b_ || !gm.ptr) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "SetTensorA, SetTensorB and a C tensor are needed");
        if (transA_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "A must be [M, K] row-major (isTransposeA = false)");
        if (m_ <= 0 || n_ <= 0 || k_ <= 0) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "set the shape first (Init, SetOrgShape or SetSingleShape)");
        if (orgKa_ > 0 && (orgKa_ != k_ || orgKb_ != k_))
            throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "splitting K between cores is not mirrored: singleCoreK must equal Ka and Kb");
        if (tilingBias_ && !bias_) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "the tiling says isBias but SetBias was not called");
        // rows of C start every orgKc (when given) or orgN elements, unless the block is written back to back
        const int ldc = enSequentialWrite ? n_ : (orgKc_ > 0 ? orgKc_ : (orgN_ > 0 ? orgN_ : n_));

        // B (and scaleB) in the reference's [K, N] form: turn them into the K-major form inside the workspace
        uint8_t* ws = workspace_;
        size_t wsLeft = workspaceBytes_;
        auto take = [&](size_t bytes) -> uint8_t* {
            if (bytes == 0) return nullptr;
            if (!ws || wsLeft < bytes) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "SetWorkspace: more scratch is needed (see GetWorkspaceSize)");
            uint8_t* p = ws;
            ws += bytes;
            wsLeft -= bytes;
            return p;
        };
        (void)take;
        const void* bNk = b_;
        if (!transB_ && orgN_ > 0 && n_ != orgN_)
            throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "a column block of a [K, N] matrix B is not contiguous: give B K-major (SetTensorB(gm, true))");
        if (!transB_) {
            if constexpr (kMxFp4) {
                uint8_t* t = take(turned_b_bytes());
                check(ascq_mx_repack_b_kn_to_nk(t, reinterpret_cast<const uint8_t*>(b_), k_, n_, stream_));
                bNk = t;
            } else if constexpr (sizeof(SrcBT) == 1) {
                uint8_t* t = take(turned_b_bytes());
                check(ascq_transpose_i8_kn_to_nk(reinterpret_cast<int8_t*>(t), reinterpret_cast<const int8_t*>(b_), k_, n_, stream_));
                bNk = t;
            } else {
                throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "16-bit B must be given K-major: SetTensorB(gm, true) with B stored [N, K]");
            }
        }
        const uint8_t* sB = reinterpret_cast<const uint8_t*>(scaleB_);
        (void)sB;
        if constexpr (kMx) {
            if (!scaleA_ || !scaleB_) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "SetTensorScaleA and SetTensorScaleB are needed");
            if (transScaleA_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "scaleA must be [M, K/32] (isTransposeScaleA = false)");
            if (!transScaleB_) {
                uint8_t* t = take(turned_scale_b_bytes());
                check(ascq_mx_repack_scale_b(t, sB, k_ / 32, n_, stream_));
                sB = t;
            }
        }

        if constexpr (kInt8 && std::is_same<DstT, int32_t>::value) {
            if (bias_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "int32 output: the bias is not added to the accumulator dump");
            if (ldc != n_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "int32 output is written densely: N of the block must equal the row pitch of C");
            check(ascq_matmul_w8a8(nullptr, a_ptr<int8_t>(), static_cast<const int8_t*>(bNk), nullptr, nullptr, nullptr, m_, n_, k_, n_,
                                   reinterpret_cast<int32_t*>(gm.ptr), stream_));
        } else if constexpr (kInt8 && std::is_same<DstT, half>::value) {
            static_assert(std::is_same<BiasT, int32_t>::value, "the bias of an int8 matmul is int32_t");
            if (!quantSet_) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "int8 -> half needs SetQuantScalar or SetQuantVector");
            float qs;
            const uint32_t lo = static_cast<uint32_t>(quantScalar_);
            std::memcpy(&qs, &lo, 4);
            check(ascq_matmul_i8_quant(gm.ptr, a_ptr<int8_t>(), static_cast<const int8_t*>(bNk), bias_ptr<int32_t>(), quantVector_, qs, m_,
                                       n_, k_, ldc, stream_));
        } else if constexpr (kInt8 && one_of<DstT, int8_t, uint8_t>) {
            static_assert(std::is_same<BiasT, int32_t>::value, "the bias of an int8 matmul is int32_t");
            if (!quantSet_) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "int8 -> int8 needs SetQuantScalar or SetQuantVector");
            check(ascq_matmul_i8_requant(gm.ptr, a_ptr<int8_t>(), static_cast<const int8_t*>(bNk), bias_ptr<int32_t>(), quantVector_,
                                         quantScalar_, m_, n_, k_, ldc, stream_));
        } else if constexpr (kFloat16 && !kMx && one_of<DstT, int8_t, uint8_t>) {
            if (bias_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "half / bfloat16 matmul: the bias is not mirrored");
            if (!quantSet_) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "half -> int8 needs SetQuantScalar or SetQuantVector");
            check(ascq_matmul_f16_quant(gm.ptr, a_, bNk, ascq::DTypeOf<SrcAT>::value, quantVector_, quantScalar_, m_, n_, k_, ldc, stream_));
        } else if constexpr (kFloat16 && !kMx && one_of<DstT, half, bfloat16_t, float>) {
            if (bias_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "half / bfloat16 matmul: the bias is not mirrored");
            check(ascq_matmul_f16(gm.ptr, ascq::DTypeOf<DstT>::value, a_, bNk, ascq::DTypeOf<SrcAT>::value, m_, n_, k_, ldc, stream_));
        } else if constexpr (kWeightOnly && one_of<DstT, half, bfloat16_t, float>) {
            if (bias_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "weight-only-quantised matmul: the bias is not mirrored");
            if (!antiQuantSet_) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "half x int8 needs SetAntiQuantScalar or SetAntiQuantVector");
            const size_t need = ascq_matmul_w8a16_workspace_size(n_, k_);
            uint8_t* scratch = take((need + 255) / 256 * 256);
            check(ascq_matmul_w8a16(gm.ptr, ascq::DTypeOf<DstT>::value, a_, ascq::DTypeOf<SrcAT>::value, static_cast<const int8_t*>(bNk),
                                    aqOffset_, aqScale_, aqOffsetScalar_, aqScaleScalar_, m_, n_, k_, ldc, scratch, need, stream_));
        } else if constexpr (kMxFp4 && std::is_same<DstT, bfloat16_t>::value) {
            if (bias_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "MX matmul: the bias is not mirrored");
            if (ldc != n_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "MX matmul writes C densely: N of the block must equal the row pitch of C");
            const int64_t rows[1] = {m_};
            const size_t need = ascq_group_matmul_mxfp4_workspace_size(m_, 1, k_, n_);
            uint8_t* scratch = take((need + 255) / 256 * 256);
            check(ascq_group_matmul_mxfp4(gm.ptr, a_ptr<uint8_t>(), reinterpret_cast<const uint8_t*>(scaleA_), static_cast<const uint8_t*>(bNk),
                                          sB, rows, 1, k_, n_, scratch, need, stream_));
        } else if constexpr (kMxFp8 && one_of<DstT, bfloat16_t, float>) {
            if (bias_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "MX matmul: the bias is not mirrored");
            if (ldc != n_) throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "MX matmul writes C densely: N of the block must equal the row pitch of C");
            const int64_t rows[1] = {m_};
            const size_t need = ascq_group_matmul_mxfp8_workspace_size(m_, 1, k_, n_);
            uint8_t* scratch = take((need + 255) / 256 * 256);
            check(ascq_group_matmul_mxfp8(gm.ptr, ascq::DTypeOf<DstT>::value, a_ptr<uint8_t>(), ascq::DTypeOf<SrcAT>::value,
                                          reinterpret_cast<const uint8_t*>(scaleA_), static_cast<const uint8_t*>(bNk),
                                          ascq::DTypeOf<SrcBT>::value, sB, rows, 1, k_, n_, scratch, need, stream_));
        } else {
            throw ascq::Error(ASCQ_ERR_UNSUPPORTED, "this combination of A, B and C types has no kernel here");
        }
    }
    template <typename X> const X* a_ptr() const { return reinterpret_cast<const X*>(a_); }
    template <typename X> const X* bias_ptr() const { return reinterpret_cast<const X*>(bias_); }

    int orgM_ = 0, orgN_ = 0, orgKa_ = 0, orgKb_ = 0, orgKc_ = 0;
    int m_ = 0, n_ = 0, k_ = 0;
    const SrcAT* a_ = nullptr;
    const SrcBT* b_ = nullptr;
    const BiasT* bias_ = nullptr;
    bool transA_ = false, transB_ = false, tilingBias_ = false;
    uint64_t quantScalar_ = 0;
    const uint64_t* quantVector_ = nullptr;
    bool quantSet_ = false;
    const SrcT* aqOffset_ = nullptr;
    const SrcT* aqScale_ = nullptr;
    float aqOffsetScalar_ = 0.f, aqScaleScalar_ = 1.f;
    bool antiQuantSet_ = false;
    const fp8_e8m0_t* scaleA_ = nullptr;
    const fp8_e8m0_t* scaleB_ = nullptr;
    bool transScaleA_ = false, transScaleB_ = true;
    uint8_t* workspace_ = nullptr;
    size_t workspaceBytes_ = 0;
    void* stream_ = nullptr;
    bool pending_ = false, haveBlock_ = false;
};

}  // namespace AscendC
#endif  // ASCQ_MATMUL_HPP_
