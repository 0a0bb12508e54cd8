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
template <TPosition POSITION, CubeFormat FORMAT, typename TYPE, bool ISTRANS = false, LayoutMode LAYOUT = LayoutMode::NONE, bool IBSHARE = false,
          TPosition SRCPOS = TPosition::GM>
struct MatmulType {
    constexpr static TPosition pos = POSITION;
    constexpr static CubeFormat format = FORMAT;
    using T = TYPE;
    constexpr static bool isTrans = ISTRANS;
    constexpr static LayoutMode layout = LAYOUT;   // batch layout of IterateBatch / IterateNBatch
    constexpr static bool ibShare = IBSHARE;       // L1 sharing between AI cores: accepted, no meaning here
    constexpr static TPosition srcPos = SRCPOS;
};
// impl/adv_api/detail/matmul/utils/matmul_type_def.h:114-130: operand type that carries an e8m0 scale tensor
template <TPosition POSITION, TPosition SCALE_POSITION, CubeFormat FORMAT, typename TYPE, bool ISTRANS = false,
          TPosition SRCPOS = TPosition::GM, CubeFormat SCALE_FORMAT = FORMAT, bool SCALE_ISTRANS = ISTRANS>
struct MatmulTypeWithScale : public MatmulType<POSITION, FORMAT, TYPE, ISTRANS, LayoutMode::NONE, false, SRCPOS> {
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
template <> struct KindOf<fp8_e4m3fn_t> { static constexpr int value = ASCB200_KIND_MXFP8_E4M3; };   // MX Matmul (with scale tensors) only
template <> struct KindOf<fp8_e5m2_t> { static constexpr int value = ASCB200_KIND_MXFP8_E5M2; };
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
    static_assert(C_TYPE::format == CubeFormat::ND || C_TYPE::format == CubeFormat::ND_ALIGN || C_TYPE::format == CubeFormat::NZ ||
                      C_TYPE::format == CubeFormat::COLUMN_MAJOR,
                  "C must be ND, ND_ALIGN, NZ or COLUMN_MAJOR");
    static_assert(A_TYPE::layout == B_TYPE::layout || A_TYPE::layout == LayoutMode::NONE || B_TYPE::layout == LayoutMode::NONE,
                  "A and B must have the same batch layout (IterateBatch.md)");
    static_assert(B_TYPE::format != CubeFormat::NZ || sizeof(SrcBT) <= 2, "NZ unpacking covers 1- and 2-byte elements");
    static constexpr bool isFp4 = std::is_same<SrcAT, fp4x2_e2m1_t>::value;
    static constexpr bool isMx = isFp4 || std::is_same<SrcAT, fp8_e4m3fn_t>::value || std::is_same<SrcAT, fp8_e5m2_t>::value;
    static constexpr int elemsPerStorage = isFp4 ? 2 : 1;  // GlobalTensor offsets count storage units (bytes for packed fp4)

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

    // The whole single-core block in one launch (impl/adv_api/detail/matmul/matmul_impl.h:119-139).  Like the reference's
    // IterateAll for output in global memory (`while (Iterate()) GetTensorC(gm, enAtomic)`), the blocks land at their places in
    // the [singleCoreM, singleCoreN] output whatever enSequentialWrite says; block-sequential output is GetTensorC's.
    template <bool sync = true>
    void IterateAll(const GlobalTensor<DstT>& gm, uint8_t enAtomic = 0, bool enSequentialWrite = false, bool waitIterateAll = false,
                    bool fakeMsg = false)
    {
        (void)enSequentialWrite;
        (void)waitIterateAll;
        (void)fakeMsg;
        Launch(gm.GetPhyAddr(), DefaultLdc(), enAtomic, 0, 0, singleM_, singleN_);
        if (sync) done_ = true;
    }

    // IterateBatch(gm, batchA, batchB, enSequentialWrite, matrixStrideA, matrixStrideB, matrixStrideC, enPartialSum, enAtomic)
    // (include/adv_api/matmul/matmul_client.h:1024-1027; use: examples/.../batch_matmul/batch_matmul.asc:166-193).  One launch per
    // matrix pair; the smaller batch count is broadcast (it must divide the larger); the bias is per batch when
    // MM_CFG.isBiasBatch, else shared.  Where matrix i of an operand starts and how far its rows are apart follows the
    // operand's LayoutMode (IterateBatch.md, "BSNGD / SBNGD / BNGS1S2"):
    //   NORMAL / NONE / BNGS1S2  matrices packed one after the other (`matrixStride` elements apart when given);
    //   BSNGD   [B][S][N][G][D]: matrix i starts i * D elements after the first, its rows are N * G * D elements apart;
    //   SBNGD   [S][B][N][G][D]: the same with rows B * N * G * D apart;
    // for C the inner extent is CLayoutInfoS2 instead of D.  The caller positions the tensors at the first matrix of the call.
    void IterateBatch(const GlobalTensor<DstT>& gm, uint32_t batchA, uint32_t batchB, bool enSequentialWrite, const uint32_t matrixStrideA = 0,
                      const uint32_t matrixStrideB = 0, const uint32_t matrixStrideC = 0, const bool enPartialSum = false, const uint8_t enAtomic = 0)
    {
        (void)enPartialSum;
        constexpr bool stridedIn = A_TYPE::layout == LayoutMode::BSNGD || A_TYPE::layout == LayoutMode::SBNGD;
        if (batchA == 0 || batchB == 0 || (enSequentialWrite && stridedIn)) {   // BSNGD / SBNGD have no sequential mode (IterateBatch.md)
            AscendC::detail::Latch(batchA == 0 || batchB == 0 ? ASCB200_EINVAL : ASCB200_EUNSUPPORTED, "Matmul::IterateBatch");
            return;
        }
        const uint32_t batch = batchA > batchB ? batchA : batchB;
        if (batch % batchA != 0 || batch % batchB != 0) {
            AscendC::detail::Latch(ASCB200_EINVAL, "Matmul::IterateBatch (batch counts must divide each other)");
            return;
        }
        size_t strideA = matrixStrideA ? matrixStrideA : static_cast<size_t>(singleM_) * singleK_ / elemsPerStorage;
        size_t strideB = matrixStrideB ? matrixStrideB : static_cast<size_t>(singleK_) * singleN_ / elemsPerStorage;
        size_t strideC = matrixStrideC ? matrixStrideC : static_cast<size_t>(singleM_) * singleN_;
        int64_t ldc = DefaultLdc();
        ldaBatch_ = ldbBatch_ = 0;
        if constexpr (A_TYPE::layout == LayoutMode::BSNGD || A_TYPE::layout == LayoutMode::SBNGD) {
            strideA = tiling_.ALayoutInfoD;
            ldaBatch_ = static_cast<int64_t>(tiling_.ALayoutInfoN) * tiling_.ALayoutInfoG * tiling_.ALayoutInfoD *
                        (A_TYPE::layout == LayoutMode::SBNGD ? tiling_.ALayoutInfoB : 1);
        }
        if constexpr (B_TYPE::layout == LayoutMode::BSNGD || B_TYPE::layout == LayoutMode::SBNGD) {
            strideB = tiling_.BLayoutInfoD;
            ldbBatch_ = static_cast<int64_t>(tiling_.BLayoutInfoN) * tiling_.BLayoutInfoG * tiling_.BLayoutInfoD *
                        (B_TYPE::layout == LayoutMode::SBNGD ? tiling_.BLayoutInfoB : 1);
        }
        if constexpr (C_TYPE::layout == LayoutMode::BSNGD || C_TYPE::layout == LayoutMode::SBNGD) {
            strideC = tiling_.CLayoutInfoS2;
            ldc = static_cast<int64_t>(tiling_.CLayoutInfoN) * tiling_.CLayoutInfoG * tiling_.CLayoutInfoS2 *
                  (C_TYPE::layout == LayoutMode::SBNGD ? tiling_.CLayoutInfoB : 1);
        }
        const SrcAT* a0 = a_;
        const SrcBT* b0 = b_;
        const BiasT* bias0 = bias_;
        for (uint32_t i = 0; i < batch; ++i) {
            a_ = a0 + (i / (batch / batchA)) * strideA;
            b_ = b0 + (i / (batch / batchB)) * strideB;
            if (biasOn_ && MM_CFG.isBiasBatch) bias_ = bias0 + static_cast<size_t>(i) * singleN_;
            Launch(gm.GetPhyAddr() + i * strideC, ldc, enAtomic, 0, 0, singleM_, singleN_);
        }
        a_ = a0;
        b_ = b0;
        bias_ = bias0;
        ldaBatch_ = ldbBatch_ = 0;
    }
    // SetWorkspace + IterateNBatch + GetBatchTensorC (include/adv_api/matmul/matmul_client.h:1121; IterateNBatch.md; use:
    // examples/.../batch_matmul_iterate_n_batch/batch_matmul_iterate_n_batch.asc:150-190): `batchLoop` IterateBatch calls in a
    // row, whose results go to the tensor SetWorkspace named.  Call i starts i * batchA matrices further in A (i * batchB in B,
    // i * max(batchA, batchB) in C and in the bias) - a matrix being D (S2 for C) elements in the strided layouts, or one
    // whole [S, D] block when a call covers all N * G matrices of a row block, as in the example's own loop
    // (batch_matmul.asc:172-190).
    void SetWorkspace(const GlobalTensor<DstT>& workspace) { workspace_ = workspace; }
    template <bool sync = true, bool waitIterateBatch = false>
    void IterateNBatch(const uint32_t batchLoop, uint32_t batchA, uint32_t batchB, bool enSequentialWrite, const uint32_t matrixStrideA = 0,
                       const uint32_t matrixStrideB = 0, const uint32_t matrixStrideC = 0)
    {
        if (!workspace_.GetPhyAddr()) {
            AscendC::detail::Latch(ASCB200_EINVAL, "Matmul::IterateNBatch (SetWorkspace first)");
            return;
        }
        const uint32_t batchC = batchA > batchB ? batchA : batchB;
        const SrcAT* a0 = a_;
        const SrcBT* b0 = b_;
        const BiasT* bias0 = bias_;
        constexpr bool normalA = !(A_TYPE::layout == LayoutMode::BSNGD || A_TYPE::layout == LayoutMode::SBNGD);
        constexpr bool normalB = !(B_TYPE::layout == LayoutMode::BSNGD || B_TYPE::layout == LayoutMode::SBNGD);
        constexpr bool normalC = !(C_TYPE::layout == LayoutMode::BSNGD || C_TYPE::layout == LayoutMode::SBNGD);
        for (uint32_t i = 0; i < batchLoop; ++i) {
            size_t offA = normalA ? static_cast<size_t>(i) * batchA * singleM_ * singleK_ / elemsPerStorage : static_cast<size_t>(i) * batchA * tiling_.ALayoutInfoD;
            size_t offB = normalB ? static_cast<size_t>(i) * batchB * singleK_ * singleN_ / elemsPerStorage : static_cast<size_t>(i) * batchB * tiling_.BLayoutInfoD;
            size_t offC = normalC ? static_cast<size_t>(i) * batchC * singleM_ * singleN_ : static_cast<size_t>(i) * batchC * tiling_.CLayoutInfoS2;
            if (!normalA && tiling_.BatchNum == tiling_.ALayoutInfoN * tiling_.ALayoutInfoG) offA *= tiling_.ALayoutInfoS;
            if (!normalB && tiling_.BatchNum == tiling_.BLayoutInfoN * tiling_.BLayoutInfoG) offB *= tiling_.BLayoutInfoS;
            if (!normalC && tiling_.BatchNum == tiling_.CLayoutInfoN * tiling_.CLayoutInfoG) offC *= tiling_.CLayoutInfoS1;
            a_ = a0 + offA;
            b_ = b0 + offB;
            if (biasOn_) bias_ = bias0 + (MM_CFG.isBiasBatch ? static_cast<size_t>(i) * batchC * singleN_ : 0);
            IterateBatch(workspace_[offC], batchA, batchB, enSequentialWrite, matrixStrideA, matrixStrideB, matrixStrideC);
        }
        a_ = a0;
        b_ = b0;
        bias_ = bias0;
        nBatchNext_ = 0;
        nBatchC_ = batchC;
    }
    // The result of the next IterateBatch of the preceding IterateNBatch: a view into the workspace.
    template <bool sync = true>
    GlobalTensor<DstT> GetBatchTensorC(uint32_t batchA, uint32_t batchB, bool enSequentialWrite = false)
    {
        (void)enSequentialWrite;
        const uint32_t batchC = batchA > batchB ? batchA : batchB;
        constexpr bool normalC = !(C_TYPE::layout == LayoutMode::BSNGD || C_TYPE::layout == LayoutMode::SBNGD);
        size_t offC = normalC ? static_cast<size_t>(nBatchNext_) * batchC * singleM_ * singleN_ : static_cast<size_t>(nBatchNext_) * batchC * tiling_.CLayoutInfoS2;
        if (!normalC && tiling_.BatchNum == tiling_.CLayoutInfoN * tiling_.CLayoutInfoG) offC *= tiling_.CLayoutInfoS1;
        ++nBatchNext_;
        return workspace_[offC];
    }
    // Iterate / GetTensorC (Iterate.md, GetTensorC.md): every Iterate() moves to the next baseM x baseN block of the
    // [singleCoreM, singleCoreN] output - along M first, along N first with iterateOrder == 1 (ORDER_N) - and returns false after
    // the last one; GetTensorC computes the current block (one launch on the block's rows of A and columns of B) and writes it at
    // its place in the output, or, with enSequentialWrite, as a compact [height, width] matrix at the tensor it is given (the
    // caller places the blocks: quant_group_matmul_custom.asc:320-328; CopyOutNZ2ND<enSequentialWrite>,
    // impl/adv_api/detail/matmul/stage/copy_cube_out/copy_cube_out_fixpipe.h:153-170: stride = baseWidth, offset 0).
    template <bool sync = true>
    bool Iterate(bool enPartialSum = false)
    {
        (void)enPartialSum;
        const int bm = BaseM(), bn = BaseN();
        const int mIter = (singleM_ + bm - 1) / bm, nIter = (singleN_ + bn - 1) / bn;
        iterIdx_ = iterActive_ ? iterIdx_ + 1 : 0;
        iterActive_ = iterIdx_ < mIter * nIter;
        return iterActive_;
    }
    template <bool sync = true>
    void GetTensorC(const GlobalTensor<DstT>& gm, uint8_t enAtomic = 0, bool enSequentialWrite = false)
    {
        if (!iterActive_) return;
        const int bm = BaseM(), bn = BaseN();
        const int mIter = (singleM_ + bm - 1) / bm, nIter = (singleN_ + bn - 1) / bn;
        const int curRow = tiling_.iterateOrder == 1 ? iterIdx_ / nIter : iterIdx_ % mIter;
        const int curCol = tiling_.iterateOrder == 1 ? iterIdx_ % nIter : iterIdx_ / mIter;
        const int h = singleM_ - curRow * bm < bm ? singleM_ - curRow * bm : bm;
        const int w = singleN_ - curCol * bn < bn ? singleN_ - curCol * bn : bn;
        if (enSequentialWrite) {
            if constexpr (C_TYPE::format == CubeFormat::NZ || C_TYPE::format == CubeFormat::COLUMN_MAJOR) {
                Launch(gm.GetPhyAddr(), h, enAtomic, curRow * bm, curCol * bn, h, w);   // a compact block: its own row count is the pitch
            } else {
                Launch(gm.GetPhyAddr(), AlignLdc(w), enAtomic, curRow * bm, curCol * bn, h, w);
            }
        } else {
            const int64_t ldc = DefaultLdc();
            DstT* at = gm.GetPhyAddr();
            if constexpr (C_TYPE::format == CubeFormat::COLUMN_MAJOR) at += static_cast<int64_t>(curCol) * bn * ldc + static_cast<int64_t>(curRow) * bm;
            else if constexpr (C_TYPE::format == CubeFormat::NZ) at += static_cast<int64_t>(curCol) * bn * ldc + static_cast<int64_t>(curRow) * bm * NzC0();
            else at += static_cast<int64_t>(curRow) * bm * ldc + static_cast<int64_t>(curCol) * bn;
            Launch(at, ldc, enAtomic, curRow * bm, curCol * bn, h, w);
        }
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
    int BaseM() const { return tiling_.baseM > 0 ? tiling_.baseM : singleM_; }
    int BaseN() const { return tiling_.baseN > 0 ? tiling_.baseN : singleN_; }
    static constexpr int NzC0() { return sizeof(DstT) == 1 ? 32 : 16; }
    // leading dimension of C in its format: row length for ND (padded to 32 bytes for ND_ALIGN), row count for the others
    int64_t AlignLdc(int64_t cols) const
    {
        if constexpr (C_TYPE::format == CubeFormat::ND_ALIGN) {
            constexpr int perBlock = 32 / static_cast<int>(sizeof(DstT));
            return (cols + perBlock - 1) / perBlock * perBlock;
        }
        return cols;
    }
    int64_t DefaultLdc() const
    {
        if constexpr (C_TYPE::format == CubeFormat::NZ || C_TYPE::format == CubeFormat::COLUMN_MAJOR) return orgM_;
        return AlignLdc(orgKc_ > 0 ? orgKc_ : orgN_);
    }
    // Owns a K-major copy of B made once per tensor (an NZ-format B, or the [K, N] fp4 B of an MX Matmul); End() releases it.
    bool EnsureCopyOfB(size_t bytes)
    {
        if (bytes > unpackedBytes_) {
            if (unpacked_) (void)ascb200_free(unpacked_);
            unpacked_ = nullptr;
            unpackedBytes_ = 0;
            const int rc = ascb200_malloc(&unpacked_, bytes);
            if (rc != ASCB200_OK) {
                AscendC::detail::Latch(rc, "Matmul (buffer for the re-laid-out B)");
                return false;
            }
            unpackedBytes_ = bytes;
        }
        return true;
    }
    // One launch: rows [rowOff, rowOff + h) x columns [colOff, colOff + w) of the single-core block, written to `c` with leading
    // dimension ldc in the format of C_TYPE.
    void Launch(DstT* c, int64_t ldc, uint8_t enAtomic, int rowOff, int colOff, int h, int w)
    {
        if (enAtomic > 3) {  // enAtomic: 1 add, 2 max, 3 min
            AscendC::detail::Latch(ASCB200_EUNSUPPORTED, "Matmul (enAtomic > 3)");
            return;
        }
        const bool whole = rowOff == 0 && colOff == 0 && h == singleM_ && w == singleN_;
        ascb200_gemm_desc d;
        std::memset(&d, 0, sizeof(d));
        d.kind = detail::KindOf<SrcAT>::value;
        d.m = h;
        d.n = w;
        d.k = singleK_;
        d.trans_a = transA_ ? 1 : 0;
        d.trans_b = transB_ ? 1 : 0;
        d.lda = ldaBatch_ ? ldaBatch_ : (transA_ ? orgM_ : orgKa_);
        d.ldb = ldbBatch_ ? ldbBatch_ : (transB_ ? orgKb_ : orgN_);
        // element offsets of the block's first row of A / first column of B (storage units: two fp4 values per unit)
        const int64_t offA = transA_ ? rowOff : static_cast<int64_t>(rowOff) * d.lda;
        const int64_t offB = transB_ ? static_cast<int64_t>(colOff) * d.ldb : colOff;
        d.a_dev = a_ + offA / elemsPerStorage;
        d.b_dev = b_ + offB / elemsPerStorage;
        if constexpr (B_TYPE::format == CubeFormat::NZ) {
            // A fractal B ([N/C0][Kb/16][16][C0] over the original shape) is unpacked once per tensor into a K-major copy
            // that the object owns.  Sub-blocks of an NZ tensor are not addressable by element offset.
            if (transB_ || singleN_ != orgN_ || singleK_ != orgKb_) {
                AscendC::detail::Latch(ASCB200_EUNSUPPORTED, "Matmul (NZ B: whole, untransposed tensor only)");
                return;
            }
            if (unpackedFor_ != b_) {
                if (!EnsureCopyOfB(static_cast<size_t>(orgN_) * orgKb_ * sizeof(SrcBT))) return;
                const int rc = ascb200_nz_unpack(b_, unpacked_, 1, orgKb_, orgN_, static_cast<int32_t>(sizeof(SrcBT)), 1, stream_);
                if (rc != ASCB200_OK) {
                    AscendC::detail::Latch(rc, "Matmul (NZ B unpack)");
                    return;
                }
                unpackedFor_ = b_;
            }
            d.b_dev = static_cast<const SrcBT*>(unpacked_) + static_cast<int64_t>(colOff) * orgKb_;
            d.trans_b = 1;
            d.ldb = orgKb_;
        }
        if constexpr (isMx) {
            // Scale tensors: [rows, K/32] or, for a transposed scaleA / a non-transposed scaleB, the reference's pair order
            // [K/64][rows][2] (SetTensorScaleA / SetTensorScaleB, impl/adv_api/detail/matmul/mx_matmul_impl.h:136-158).
            const int64_t sk = singleK_ / 32;
            d.scale_flags = (transScaleA_ ? ASCB200_SCALE_A_PAIRED : 0) | (!transScaleB_ ? ASCB200_SCALE_B_PAIRED : 0);
            if (!whole && (transScaleA_ || !transScaleB_ || (isFp4 && ((transA_ && (rowOff & 1)) || (!transB_ && (colOff & 1)))))) {
                AscendC::detail::Latch(ASCB200_EUNSUPPORTED, "Matmul (MX sub-block with pair-ordered scales or an odd offset)");
                return;
            }
            d.scale_a_dev = scaleA_ + static_cast<int64_t>(rowOff) * sk;
            d.scale_b_dev = scaleB_ + static_cast<int64_t>(colOff) * sk;
            if (isFp4 && !transB_ && whole && singleN_ == orgN_ && singleK_ == orgKb_) {
                // the reference's ND B ([K, N], two N-neighbours per byte): weights, transposed to K-major once per tensor
                if (unpackedFor_ != b_) {
                    if (!EnsureCopyOfB(static_cast<size_t>(orgN_) * orgKb_ / 2)) return;
                    const int rc = ascb200_fp4_transpose(b_, unpacked_, orgKb_, orgN_, stream_);
                    if (rc != ASCB200_OK) {
                        AscendC::detail::Latch(rc, "Matmul (fp4 B transpose)");
                        return;
                    }
                    unpackedFor_ = b_;
                }
                d.b_dev = unpacked_;
                d.trans_b = 1;
                d.ldb = orgKb_;
            }
        }
        d.atomic = enAtomic;
        d.bias_dev = (biasOn_ && MM_CFG.enableSetBias) ? bias_ + colOff : nullptr;
        d.c_dev = c;
        d.ldc = ldc;
        d.c_layout = C_TYPE::format == CubeFormat::NZ ? ASCB200_C_NZ : C_TYPE::format == CubeFormat::COLUMN_MAJOR ? ASCB200_C_COLUMN_MAJOR : ASCB200_C_ROW_MAJOR;
        d.c_dtype = AscendC::detail::DTypeOf<DstT>::value;
        d.relu = MM_CFG.enableRelu ? 1 : 0;
        if (quantSet_) {
            d.epilogue = ASCB200_EPI_FIXPIPE_QUANT;
            d.quant_dev = quantVec_ ? quantVec_ + colOff : nullptr;
            d.quant_scalar = quantScalar_;
        } else {
            d.epilogue = ASCB200_EPI_CAST;
        }
        AscendC::detail::Latch(ascb200_gemm(&d, stream_), "Matmul");
    }

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
    bool biasOn_ = false, quantSet_ = false, done_ = false, iterActive_ = false;
    int iterIdx_ = 0;                      // base block of the running Iterate / GetTensorC sequence
    int64_t ldaBatch_ = 0, ldbBatch_ = 0;  // row pitch of A / B inside IterateBatch for the strided layouts (0 = the usual one)
    GlobalTensor<DstT> workspace_;         // SetWorkspace: where IterateNBatch writes
    uint32_t nBatchNext_ = 0, nBatchC_ = 0;
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
