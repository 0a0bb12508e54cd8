// AscendC::Matmul for B200: the reference's operator object (include/adv_api/matmul/matmul.h:54-400,
// include/adv_api/matmul/matmul_intf.h:46-67) kept on the host.  Set* methods record state; IterateAll
// launches the tensor-core GEMM through ascb200_gemm.  Buffer-choreography settings of the Ascend
// implementation (L1/L0 depths, double-buffer switches, iterate order) are accepted and have no effect
// on results.
#pragma once
#include <type_traits>

#include "../kernel_operator.h"
#include "matmul_config.h"

namespace AscendC {

// impl/adv_api/detail/matmul/utils/matmul_type_def.h:37-49
template <TPosition POSITION, CubeFormat FORMAT, typename TYPE, bool ISTRANS = false>
struct MatmulType {
    constexpr static TPosition pos = POSITION;
    constexpr static CubeFormat format = FORMAT;
    using T = TYPE;
    constexpr static bool isTrans = ISTRANS;
};
// impl/adv_api/detail/matmul/utils/matmul_type_def.h:114-130: operand type that carries an e8m0 scale tensor
template <TPosition POSITION, TPosition SCALE_POSITION, CubeFormat FORMAT, typename TYPE, bool ISTRANS = false,
          TPosition SRCPOS = TPosition::GM, CubeFormat SCALE_FORMAT = FORMAT, bool SCALE_ISTRANS = ISTRANS>
struct MatmulTypeWithScale : public MatmulType<POSITION, FORMAT, TYPE, ISTRANS> {
    constexpr static TPosition scalePosition = SCALE_POSITION;
    constexpr static CubeFormat scaleFormat = SCALE_FORMAT;
    constexpr static bool isScaleTrans = SCALE_ISTRANS;
};

// impl/adv_api/detail/matmul/utils/matmul_call_back.h:26-39: only the all-default callback set is supported.
template <void* DataCopyOut = nullptr, void* CopyA1 = nullptr, void* CopyB1 = nullptr>
struct MatmulCallBackFunc {};
struct MatmulPolicyDefault {};
struct MatmulWithScalePolicy {};  // impl/adv_api/detail/matmul/policy/matmul_policy.h:66 (selects the MX scheduler)

namespace detail {
template <class T> struct KindOf;
template <> struct KindOf<half> { static constexpr int value = ASCB200_KIND_F16; };
template <> struct KindOf<bfloat16_t> { static constexpr int value = ASCB200_KIND_BF16; };
template <> struct KindOf<int8_t> { static constexpr int value = ASCB200_KIND_S8; };
template <> struct KindOf<fp4x2_e2m1_t> { static constexpr int value = ASCB200_KIND_MXFP4; };
// The fifth argument is a MatmulConfig or, for constant tiling, the MatmulApiStaticTiling made from one.
constexpr const MatmulConfig& ToMatmulConfig(const MatmulConfig& cfg) { return cfg; }
constexpr const MatmulConfig& ToMatmulConfig(const MatmulApiStaticTiling& tiling) { return tiling.cfg; }
}  // namespace detail

template <class A_TYPE, class B_TYPE, class C_TYPE, class BIAS_TYPE = C_TYPE, const auto& MM_CFG_OR_TILING = CFG_NORM,
          class MM_CB = MatmulCallBackFunc<>, class POLICY = MatmulPolicyDefault>
class Matmul {
public:
    static constexpr const MatmulConfig& MM_CFG = detail::ToMatmulConfig(MM_CFG_OR_TILING);
    static constexpr bool hasStaticTiling = std::is_same<std::decay_t<decltype(MM_CFG_OR_TILING)>, MatmulApiStaticTiling>::value;
    using SrcAT = typename A_TYPE::T;
    using SrcBT = typename B_TYPE::T;
    using DstT = typename C_TYPE::T;
    using BiasT = typename BIAS_TYPE::T;
    static_assert(std::is_same<SrcAT, SrcBT>::value, "A and B must have the same element type");
    static_assert(A_TYPE::format == CubeFormat::ND, "A must be ND (row-major); use isTrans for the other orientation");
    static_assert(B_TYPE::format == CubeFormat::ND || B_TYPE::format == CubeFormat::NZ, "B must be ND or the fractal NZ format");
    static_assert(C_TYPE::format == CubeFormat::ND || C_TYPE::format == CubeFormat::ND_ALIGN, "C must be ND or ND_ALIGN");
    static_assert(B_TYPE::format != CubeFormat::NZ || sizeof(SrcBT) <= 2, "NZ unpacking covers 1- and 2-byte elements");
    static constexpr bool isMx = std::is_same<SrcAT, fp4x2_e2m1_t>::value;
    static constexpr int elemsPerStorage = isMx ? 2 : 1;  // GlobalTensor offsets count storage units (bytes for packed fp4)

    Matmul() = default;
    Matmul(const Matmul&) = delete;  // the object may own the unpacked copy of an NZ operand
    Matmul& operator=(const Matmul&) = delete;

    void Init(const TCubeTiling* cubeTiling, TPipe* tpipe = nullptr)
    {
        if (cubeTiling) {
            tiling_ = *cubeTiling;
        } else {
            // constant tiling: the shapes are compile-time constants of the fifth template argument; SetOrgShape refines them
            tiling_ = TCubeTiling{};
            if constexpr (hasStaticTiling) {
                tiling_.M = MM_CFG_OR_TILING.M;
                tiling_.N = MM_CFG_OR_TILING.N;
                tiling_.Ka = MM_CFG_OR_TILING.Ka;
                tiling_.Kb = MM_CFG_OR_TILING.Kb;
                tiling_.singleCoreM = MM_CFG_OR_TILING.singleCoreM;
                tiling_.singleCoreN = MM_CFG_OR_TILING.singleCoreN;
                tiling_.singleCoreK = MM_CFG_OR_TILING.singleCoreK;
                tiling_.isBias = MM_CFG_OR_TILING.isBias;
            } else {
                AscendC::detail::Latch(ASCB200_EINVAL, "Matmul::Init (null tiling without a constant tiling)");
            }
        }
        stream_ = tpipe ? tpipe->GetStream() : AscendC::detail::CurrentStream();
        orgM_ = tiling_.M;
        orgN_ = tiling_.N;
        orgKa_ = tiling_.Ka;
        orgKb_ = tiling_.Kb;
        orgKc_ = 0;
        singleM_ = tiling_.singleCoreM;
        singleN_ = tiling_.singleCoreN;
        singleK_ = tiling_.singleCoreK;
        biasOn_ = false;
        quantVec_ = nullptr;
        quantScalar_ = 0;
        quantSet_ = false;
    }
    void SetSubBlockIdx(uint8_t) {}
    void SetOrgShape(int orgM, int orgN, int orgK) { SetOrgShape(orgM, orgN, orgK, orgK, 0); }
    void SetOrgShape(int orgM, int orgN, int orgKa, int orgKb, int orgKc = 0)
    {
        orgM_ = orgM;
        orgN_ = orgN;
        orgKa_ = orgKa;
        orgKb_ = orgKb;
        orgKc_ = orgKc;
    }
    void SetSingleShape(int singleM, int singleN, int singleK)
    {
        singleM_ = singleM;
        singleN_ = singleN;
        singleK_ = singleK;
    }
    void SetTail(int tailM = -1, int tailN = -1, int tailK = -1)
    {
        if (tailM != -1) singleM_ = tailM;
        if (tailN != -1) singleN_ = tailN;
        if (tailK != -1) singleK_ = tailK;
    }
    void SetTensorA(const GlobalTensor<SrcAT>& gm, bool isTransposeA = false)
    {
        a_ = gm.GetPhyAddr();
        transA_ = isTransposeA;
    }
    void SetTensorB(const GlobalTensor<SrcBT>& gm, bool isTransposeB = false)
    {
        if (b_ != gm.GetPhyAddr()) unpackedFor_ = nullptr;  // another NZ tensor: unpack again
        b_ = gm.GetPhyAddr();
        transB_ = isTransposeB;
    }
    void SetTensorScaleA(const GlobalTensor<fp8_e8m0_t>& gm, bool isTransposeScaleA = false)
    {
        scaleA_ = gm.GetPhyAddr();
        transScaleA_ = isTransposeScaleA;
    }
    void SetTensorScaleB(const GlobalTensor<fp8_e8m0_t>& gm, bool isTransposeScaleB = true)
    {
        scaleB_ = gm.GetPhyAddr();
        transScaleB_ = isTransposeScaleB;
    }
    void SetBias(const GlobalTensor<BiasT>& biasGlobal)
    {
        bias_ = biasGlobal.GetPhyAddr();
        biasOn_ = true;
    }
    void DisableBias() { biasOn_ = false; }
    void ClearBias() { biasOn_ = false; }
    void SetQuantScalar(const uint64_t quantScalar)
    {
        quantScalar_ = quantScalar;
        quantVec_ = nullptr;
        quantSet_ = true;
    }
    void SetQuantVector(const GlobalTensor<uint64_t>& quantTensor)
    {
        quantVec_ = quantTensor.GetPhyAddr();
        quantSet_ = true;
    }

    // The whole single-core block in one launch (impl/adv_api/detail/matmul/matmul_impl.h:119-139).
    template <bool sync = true>
    void IterateAll(const GlobalTensor<DstT>& gm, uint8_t enAtomic = 0, bool enSequentialWrite = false, bool waitIterateAll = false,
                    bool fakeMsg = false)
    {
        (void)waitIterateAll;
        (void)fakeMsg;
        if (enAtomic > 3 || enSequentialWrite) {  // enAtomic: 1 add, 2 max, 3 min; block-sequential output is not implemented
            AscendC::detail::Latch(ASCB200_EUNSUPPORTED, "Matmul::IterateAll (enAtomic > 3, enSequentialWrite)");
            return;
        }
        ascb200_gemm_desc d;
        std::memset(&d, 0, sizeof(d));
        d.kind = detail::KindOf<SrcAT>::value;
        d.m = singleM_;
        d.n = singleN_;
        d.k = singleK_;
        d.a_dev = a_;
        d.b_dev = b_;
        d.trans_a = transA_ ? 1 : 0;
        d.trans_b = transB_ ? 1 : 0;
        d.lda = transA_ ? orgM_ : orgKa_;
        d.ldb = transB_ ? orgKb_ : orgN_;
        if constexpr (B_TYPE::format == CubeFormat::NZ) {
            // A fractal B ([N/C0][Kb/16][16][C0] over the original shape) is unpacked once per tensor into a K-major copy
            // that the object owns; End() releases it.  Sub-blocks of an NZ tensor are not addressable by element offset.
            if (transB_ || singleN_ != orgN_ || singleK_ != orgKb_) {
                AscendC::detail::Latch(ASCB200_EUNSUPPORTED, "Matmul::IterateAll (NZ B: whole, untransposed tensor only)");
                return;
            }
            if (unpackedFor_ != b_) {
                const size_t bytes = static_cast<size_t>(orgN_) * orgKb_ * sizeof(SrcBT);
                if (bytes > unpackedBytes_) {
                    if (unpacked_) (void)ascb200_free(unpacked_);
                    unpacked_ = nullptr;
                    unpackedBytes_ = 0;
                    const int rc = ascb200_malloc(&unpacked_, bytes);
                    if (rc != ASCB200_OK) {
                        AscendC::detail::Latch(rc, "Matmul::IterateAll (NZ B buffer)");
                        return;
                    }
                    unpackedBytes_ = bytes;
                }
                const int rc = ascb200_nz_unpack(b_, unpacked_, 1, orgKb_, orgN_, static_cast<int32_t>(sizeof(SrcBT)), 1, stream_);
                if (rc != ASCB200_OK) {
                    AscendC::detail::Latch(rc, "Matmul::IterateAll (NZ B unpack)");
                    return;
                }
                unpackedFor_ = b_;
            }
            d.b_dev = unpacked_;
            d.trans_b = 1;
            d.ldb = orgKb_;
        }
        d.atomic = enAtomic;
        d.scale_a_dev = scaleA_;
        d.scale_b_dev = scaleB_;
        d.bias_dev = (biasOn_ && MM_CFG.enableSetBias) ? bias_ : nullptr;
        d.c_dev = gm.GetPhyAddr();
        d.ldc = orgKc_ > 0 ? orgKc_ : orgN_;
        if constexpr (C_TYPE::format == CubeFormat::ND_ALIGN) {
            // ND with every row padded to a multiple of 32 bytes
            constexpr int perBlock = 32 / static_cast<int>(sizeof(DstT));
            d.ldc = (d.ldc + perBlock - 1) / perBlock * perBlock;
        }
        d.c_dtype = AscendC::detail::DTypeOf<DstT>::value;
        d.relu = MM_CFG.enableRelu ? 1 : 0;
        if (quantSet_) {
            d.epilogue = ASCB200_EPI_FIXPIPE_QUANT;
            d.quant_dev = quantVec_;
            d.quant_scalar = quantScalar_;
        } else {
            d.epilogue = ASCB200_EPI_CAST;
        }
        if (isMx && (transScaleA_ || !transScaleB_)) {
            // scales must be [rows, K/32] with K contiguous for both operands
            AscendC::detail::Latch(ASCB200_EUNSUPPORTED, "Matmul::IterateAll (scale tensor orientation)");
            return;
        }
        AscendC::detail::Latch(ascb200_gemm(&d, stream_), "Matmul::IterateAll");
        if (sync) done_ = true;
    }

    // IterateBatch(gm, batchA, batchB, enSequentialWrite, matrixStrideA, matrixStrideB, matrixStrideC, enPartialSum, enAtomic)
    // (include/adv_api/matmul/matmul_client.h:1024-1027; use: examples/.../batch_matmul/batch_matmul.asc:193), NORMAL layout: A holds
    // batchA matrices [M, K] (or [K, M]), B batchB matrices, C max(batchA, batchB) matrices, each `matrixStride` elements
    // after the previous one (0 = densely packed); the smaller batch count is broadcast (it must divide the larger).
    // One launch per matrix pair; the bias is per batch when MM_CFG.isBiasBatch, else shared.
    void IterateBatch(const GlobalTensor<DstT>& gm, uint32_t batchA, uint32_t batchB, bool enSequentialWrite, const uint32_t matrixStrideA = 0,
                      const uint32_t matrixStrideB = 0, const uint32_t matrixStrideC = 0, const bool enPartialSum = false, const uint8_t enAtomic = 0)
    {
        (void)enPartialSum;
        if (batchA == 0 || batchB == 0 || enSequentialWrite) {
            AscendC::detail::Latch(batchA == 0 || batchB == 0 ? ASCB200_EINVAL : ASCB200_EUNSUPPORTED, "Matmul::IterateBatch");
            return;
        }
        const uint32_t batch = batchA > batchB ? batchA : batchB;
        if (batch % batchA != 0 || batch % batchB != 0) {
            AscendC::detail::Latch(ASCB200_EINVAL, "Matmul::IterateBatch (batch counts must divide each other)");
            return;
        }
        const size_t strideA = matrixStrideA ? matrixStrideA : static_cast<size_t>(singleM_) * singleK_ / elemsPerStorage;
        const size_t strideB = matrixStrideB ? matrixStrideB : static_cast<size_t>(singleK_) * singleN_ / elemsPerStorage;
        const size_t strideC = matrixStrideC ? matrixStrideC : static_cast<size_t>(singleM_) * singleN_;
        const SrcAT* a0 = a_;
        const SrcBT* b0 = b_;
        const BiasT* bias0 = bias_;
        for (uint32_t i = 0; i < batch; ++i) {
            a_ = a0 + (i / (batch / batchA)) * strideA;
            b_ = b0 + (i / (batch / batchB)) * strideB;
            if (biasOn_ && MM_CFG.isBiasBatch) bias_ = bias0 + static_cast<size_t>(i) * singleN_;
            IterateAll<false>(gm[i * strideC], enAtomic);
        }
        a_ = a0;
        b_ = b0;
        bias_ = bias0;
    }
    // Iterate / GetTensorC pair: the first Iterate() computes the whole block into the tensor that the
    // following GetTensorC names; later Iterate() calls report completion.
    template <bool sync = true>
    bool Iterate(bool enPartialSum = false)
    {
        (void)enPartialSum;
        if (iterPending_) {
            iterPending_ = false;
            return false;
        }
        iterPending_ = true;
        return true;
    }
    template <bool sync = true>
    void GetTensorC(const GlobalTensor<DstT>& gm, uint8_t enAtomic = 0, bool enSequentialWrite = false)
    {
        if (iterPending_) IterateAll<sync>(gm, enAtomic, enSequentialWrite);
    }
    void End()
    {
        if (unpacked_) {
            (void)ascb200_stream_sync(stream_);
            (void)ascb200_free(unpacked_);
        }
        unpacked_ = nullptr;
        unpackedBytes_ = 0;
        unpackedFor_ = nullptr;
    }
    ~Matmul() { End(); }
    void SetLocalWorkspace(const LocalTensor<uint8_t>&) {}
    int GetLastError() const { return AscendC::GetLastError(); }

private:
    TCubeTiling tiling_{};
    void* stream_ = nullptr;
    const SrcAT* a_ = nullptr;
    const SrcBT* b_ = nullptr;
    void* unpacked_ = nullptr;           // K-major copy of an NZ-format B
    size_t unpackedBytes_ = 0;
    const SrcBT* unpackedFor_ = nullptr;
    const fp8_e8m0_t* scaleA_ = nullptr;
    const fp8_e8m0_t* scaleB_ = nullptr;
    const BiasT* bias_ = nullptr;
    const uint64_t* quantVec_ = nullptr;
    uint64_t quantScalar_ = 0;
    bool transA_ = false, transB_ = false, transScaleA_ = false, transScaleB_ = true;
    bool biasOn_ = false, quantSet_ = false, done_ = false, iterPending_ = false;
    int orgM_ = 0, orgN_ = 0, orgKa_ = 0, orgKb_ = 0, orgKc_ = 0, singleM_ = 0, singleN_ = 0, singleK_ = 0;
};

}  // namespace AscendC

// include/adv_api/matmul/matmul_intf.h:40-41 / impl/adv_api/detail/kfc/kfc_register_obj.h:142-162
#define REGIST_MATMUL_OBJ(tpipe, workspace, obj, tiling) \
    do {                                                 \
        (void)(workspace);                               \
        (obj).SetSubBlockIdx(0);                         \
        (obj).Init((tiling), (tpipe));                   \
    } while (0)
