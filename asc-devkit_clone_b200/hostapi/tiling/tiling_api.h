// Host tiling API of the hot path for B200 (the reference's static library `tiling_api`):
//   matmul_tiling::MatmulApiTiling / MultiCoreMatmulTiling -> optiling::TCubeTiling
//       (include/adv_api/matmul/matmul_tiling_base.h:316-653, matmul_tiling.h:30-62, bmm_tiling.h)
//   AscendC::SoftMaxTilingFunc, GetSoftMaxMin/MaxTmpSize, IsBasicBlockInSoftMax
//       (impl/adv_api/tiling/activation/softmax_tiling.cpp:88-215,522-544)
//   AscendC::GetAscendQuantMaxMinTmpSize / GetAscendDequantMaxMinTmpSize (+ TmpBufferFactorSize)
//       (impl/adv_api/tiling/quantization/ascend_{quant,dequant}_tiling_impl.cpp)
//   platform_ascendc::PlatformAscendC: reports the B200 as one "core" per SM.
// The tiling structs keep the reference's field order and sizes so that host programs can keep
// serialising them; fields that describe Ascend on-chip buffer choreography are filled with
// plausible values and never read by the B200 kernels (the tile shape is chosen inside ascb200_gemm).
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

#include "../kernel_operator.h"

namespace ge {
class Shape {
public:
    Shape() = default;
    explicit Shape(std::vector<int64_t> dims) : dims_(std::move(dims)) {}
    const std::vector<int64_t>& GetDims() const { return dims_; }
    size_t GetDimNum() const { return dims_.size(); }
    int64_t GetShapeSize() const
    {
        if (dims_.empty()) return 0;
        int64_t s = 1;
        for (int64_t d : dims_) s *= d;
        return s;
    }

private:
    std::vector<int64_t> dims_;
};
}  // namespace ge

namespace platform_ascendc {
enum class CoreMemType { L0_A = 0, L0_B, L0_C, L1, L2, UB, HBM, FB, BT };
class PlatformAscendC {
public:
    // one Ascend "AI core" = one SM; the cube and vector counts are the same
    uint32_t GetCoreNumAic() const { return Sms(); }
    uint32_t GetCoreNumAiv() const { return Sms(); }
    uint32_t GetCoreNum() const { return Sms(); }
    void GetCoreMemSize(const CoreMemType& t, uint64_t& size) const
    {
        switch (t) {
            case CoreMemType::L1: size = 227 * 1024; break;        // shared memory per CTA
            case CoreMemType::L0_C: size = 256 * 1024; break;      // TMEM per SM
            case CoreMemType::UB: size = 256 * 1024; break;        // register file per SM
            case CoreMemType::L2: size = 126ull << 20; break;
            case CoreMemType::HBM: size = 180ull << 30; break;
            default: size = 64 * 1024; break;
        }
    }
    uint32_t GetLibApiWorkSpaceSize() const { return 0; }

private:
    static uint32_t Sms()
    {
        const int n = ascb200_sm_count();
        return n > 0 ? static_cast<uint32_t>(n) : 148u;
    }
};
class PlatformAscendCManager {
public:
    static PlatformAscendC* GetInstance(const char* /*socVersion*/ = nullptr)
    {
        static PlatformAscendC instance;
        return &instance;
    }
};
}  // namespace platform_ascendc

namespace optiling {
#define ASCB200_TCUBE_FIELDS(X)                                                                                                          \
    X(usedCoreNum) X(M) X(N) X(Ka) X(Kb) X(singleCoreM) X(singleCoreN) X(singleCoreK) X(baseM) X(baseN) X(baseK) X(depthA1) X(depthB1)    \
    X(stepM) X(stepN) X(isBias) X(transLength) X(iterateOrder) X(shareMode) X(shareL1Size) X(shareL0CSize) X(shareUbSize) X(batchM)      \
    X(batchN) X(singleBatchM) X(singleBatchN) X(stepKa) X(stepKb) X(depthAL1CacheUB) X(depthBL1CacheUB) X(dbL0A) X(dbL0B) X(dbL0C)       \
    X(ALayoutInfoB) X(ALayoutInfoS) X(ALayoutInfoN) X(ALayoutInfoG) X(ALayoutInfoD) X(BLayoutInfoB) X(BLayoutInfoS) X(BLayoutInfoN)      \
    X(BLayoutInfoG) X(BLayoutInfoD) X(CLayoutInfoB) X(CLayoutInfoS1) X(CLayoutInfoN) X(CLayoutInfoG) X(CLayoutInfoS2) X(BatchNum)        \
    X(mxTypePara)
// Serialisable tiling object with set_x / get_x accessors (the reference generates it with BEGIN_TILING_DATA_DEF).
class TCubeTiling {
public:
#define ASCB200_ACCESSOR(f)                     \
    void set_##f(int32_t v) { data_.f = v; }    \
    int32_t get_##f() const { return data_.f; }
    ASCB200_TCUBE_FIELDS(ASCB200_ACCESSOR)
#undef ASCB200_ACCESSOR
    size_t GetDataSize() const { return sizeof(::TCubeTiling); }
    void SaveToBuffer(void* buf, size_t capacity) const { std::memcpy(buf, &data_, std::min(capacity, sizeof(data_))); }
    const ::TCubeTiling& Data() const { return data_; }

private:
    ::TCubeTiling data_{};
};

#define ASCB200_SOFTMAX_FIELDS(X)                                                                                              \
    X(srcM) X(srcK) X(srcSize) X(outMaxM) X(outMaxK) X(outMaxSize) X(splitM) X(splitK) X(splitSize) X(reduceM) X(reduceK)        \
    X(reduceSize) X(rangeM) X(tailM) X(tailSplitSize) X(tailReduceSize)
class SoftMaxTiling {
public:
#define ASCB200_ACCESSOR(f)                      \
    void set_##f(uint32_t v) { data_.f = v; }    \
    uint32_t get_##f() const { return data_.f; }
    ASCB200_SOFTMAX_FIELDS(ASCB200_ACCESSOR)
#undef ASCB200_ACCESSOR
    size_t GetDataSize() const { return sizeof(::SoftMaxTiling); }
    void SaveToBuffer(void* buf, size_t capacity) const { std::memcpy(buf, &data_, std::min(capacity, sizeof(data_))); }
    const ::SoftMaxTiling& Data() const { return data_; }

private:
    ::SoftMaxTiling data_{};
};
}  // namespace optiling

namespace matmul_tiling {
// include/adv_api/matmul/matmul_tiling_base.h:35-182 (values kept)
enum class DataType : int32_t {
    DT_FLOAT = 0, DT_FLOAT16 = 1, DT_INT8 = 2, DT_INT32 = 3, DT_UINT8 = 4, DT_INT16 = 6, DT_UINT16 = 7, DT_UINT32 = 8, DT_INT64 = 9,
    DT_UINT64 = 10, DT_DOUBLE = 11, DT_BOOL = 12, DT_BF16 = 27, DT_UNDEFINED = 28, DT_INT4 = 29, DT_BFLOAT16 = 33, DT_HIFLOAT8 = 34,
    DT_FLOAT8_E4M3FN = 35, DT_FLOAT8_E5M2 = 36, DT_FLOAT4_E2M1 = 37, DT_FLOAT8_E8M0 = 38, DT_FLOAT4_E1M2 = 39, DT_MAX = 42
};
enum class TPosition : int32_t { GM, A1, A2, B1, B2, C1, C2, CO1, CO2, VECIN, VECOUT, VECCALC, LCM = VECCALC, SPM, SHM = SPM, TSCM, MAX };
enum class CubeFormat : int32_t { ND = 0, NZ, ZN, ZZ, NN, ND_ALIGN, SCALAR, VECTOR, ROW_MAJOR = ND, COLUMN_MAJOR = 8 };
enum class MatrixTraverse : int32_t { NOSET = 0, FIRSTM = 1, FIRSTN = 2 };
enum class MatrixMadType : int32_t { NORMAL = 0, HF32 = 1, MXMODE = 2 };
enum class DequantType : int32_t { SCALAR = 0, TENSOR = 1 };

struct MatmulTypeDesc {
    TPosition pos = TPosition::GM;
    CubeFormat format = CubeFormat::ND;
    DataType dtype = DataType::DT_UNDEFINED;
    bool isTrans = false;
    bool set = false;
};

class MatmulApiTilingBase {
public:
    MatmulApiTilingBase() = default;
    explicit MatmulApiTilingBase(const platform_ascendc::PlatformAscendC& platform) : cores_(static_cast<int32_t>(platform.GetCoreNumAic())) {}
    virtual ~MatmulApiTilingBase() = default;

    int32_t SetAType(TPosition pos, CubeFormat type, DataType dataType, bool isTrans = false) { return SetType(a_, pos, type, dataType, isTrans); }
    int32_t SetBType(TPosition pos, CubeFormat type, DataType dataType, bool isTrans = false) { return SetType(b_, pos, type, dataType, isTrans); }
    int32_t SetCType(TPosition pos, CubeFormat type, DataType dataType) { return SetType(c_, pos, type, dataType, false); }
    int32_t SetBiasType(TPosition pos, CubeFormat type, DataType dataType) { return SetType(bias_, pos, type, dataType, false); }
    int32_t SetScaleAType(TPosition, CubeFormat, bool isScaleTrans = false)
    {
        scaleATrans_ = isScaleTrans;
        return 0;
    }
    int32_t SetScaleBType(TPosition, CubeFormat, bool isScaleTrans = true)
    {
        scaleBTrans_ = isScaleTrans;
        return 0;
    }
    int32_t SetDequantType(DequantType t)
    {
        dequant_ = t;
        return 0;
    }
    virtual int32_t SetShape(int32_t m, int32_t n, int32_t k)
    {
        m_ = m;
        n_ = n;
        k_ = k;
        return 0;
    }
    int32_t SetOrgShape(int32_t orgM, int32_t orgN, int32_t orgK) { return SetOrgShape(orgM, orgN, orgK, orgK); }
    int32_t SetOrgShape(int32_t orgM, int32_t orgN, int32_t orgKa, int32_t orgKb)
    {
        orgM_ = orgM;
        orgN_ = orgN;
        orgKa_ = orgKa;
        orgKb_ = orgKb;
        return 0;
    }
    int32_t EnableBias(bool isBias = false)
    {
        isBias_ = isBias;
        return 0;
    }
    int32_t SetBias(bool isBias = false) { return EnableBias(isBias); }
    int32_t SetFixSplit(int32_t baseM = -1, int32_t baseN = -1, int32_t baseK = -1)
    {
        // the reference rejects values that are not multiples of the 16-element fractal
        if ((baseM != -1 && (baseM <= 0 || baseM % 16 != 0)) || (baseN != -1 && (baseN <= 0 || baseN % 16 != 0)) ||
            (baseK != -1 && baseK <= 0))
            return -1;
        fixM_ = baseM;
        fixN_ = baseN;
        fixK_ = baseK;
        return 0;
    }
    int32_t SetBufferSpace(int32_t = -1, int32_t = -1, int32_t = -1, int32_t = -1) { return 0; }
    // Batch layouts (include/adv_api/matmul/matmul_tiling_base.h:406-438): the B, S, N, G, D extents of each operand are
    // copied into the tiling (ALayoutInfoB ... CLayoutInfoS2, BatchNum) for IterateBatch to read.
    int32_t SetALayout(int32_t b, int32_t s, int32_t n, int32_t g, int32_t d) { return SetLayout(aLayout_, b, s, n, g, d); }
    int32_t SetBLayout(int32_t b, int32_t s, int32_t n, int32_t g, int32_t d) { return SetLayout(bLayout_, b, s, n, g, d); }
    int32_t SetCLayout(int32_t b, int32_t s, int32_t n, int32_t g, int32_t d) { return SetLayout(cLayout_, b, s, n, g, d); }
    // NORMAL layout: A [batchA, m, k], B [batchB, k, n] (or transposed), C [max(batchA, batchB), m, n]
    // (impl/adv_api/tiling/matmul/matmul_tiling_base.cpp:365-400).
    int32_t SetBatchInfoForNormal(int32_t batchA, int32_t batchB, int32_t m, int32_t n, int32_t k)
    {
        if (batchA <= 0 || batchB <= 0 || m <= 0 || n <= 0 || k <= 0) return -1;
        SetLayout(aLayout_, batchA, m, 1, 1, k);
        SetLayout(bLayout_, batchB, n, 1, 1, k);
        SetLayout(cLayout_, std::max(batchA, batchB), m, 1, 1, n);
        return 0;
    }
    int32_t SetBatchNum(int32_t batch)
    {
        if (batch <= 0) return -1;
        batchNum_ = batch;
        return 0;
    }
    int32_t SetTraverse(MatrixTraverse t)
    {
        traverse_ = t;
        return 0;
    }
    int32_t SetMadType(MatrixMadType t)
    {
        mad_ = t;
        return 0;
    }
    int32_t SetSplitRange(int32_t = -1, int32_t = -1, int32_t = -1, int32_t = -1, int32_t = -1, int32_t = -1) { return 0; }
    int32_t SetDoubleBuffer(bool, bool, bool, bool, bool = true, bool = true) { return 0; }
    int32_t SetSparse(bool = false) { return 0; }
    int32_t GetBaseM() const { return baseM_; }
    int32_t GetBaseN() const { return baseN_; }
    int32_t GetBaseK() const { return baseK_; }

    virtual int64_t GetTiling(optiling::TCubeTiling& tiling) = 0;
    int64_t GetTiling(::TCubeTiling& tiling)
    {
        optiling::TCubeTiling t;
        const int64_t rc = GetTiling(t);
        if (rc == 0) tiling = t.Data();
        return rc;
    }

protected:
    static int32_t SetType(MatmulTypeDesc& d, TPosition pos, CubeFormat f, DataType t, bool trans)
    {
        d.pos = pos;
        d.format = f;
        d.dtype = t;
        d.isTrans = trans;
        d.set = true;
        return 0;
    }
    static int32_t SetLayout(int32_t (&l)[5], int32_t b, int32_t s, int32_t n, int32_t g, int32_t d)
    {
        l[0] = b;
        l[1] = s;
        l[2] = n;
        l[3] = g;
        l[4] = d;
        return 0;
    }
    static bool IsBf16(DataType t) { return t == DataType::DT_BF16 || t == DataType::DT_BFLOAT16; }
    static int ElemBits(DataType t)
    {
        switch (t) {
            case DataType::DT_FLOAT: case DataType::DT_INT32: return 32;
            case DataType::DT_FLOAT16: case DataType::DT_BF16: case DataType::DT_BFLOAT16: return 16;
            case DataType::DT_INT8: case DataType::DT_FLOAT8_E4M3FN: case DataType::DT_FLOAT8_E5M2: case DataType::DT_HIFLOAT8: return 8;
            case DataType::DT_FLOAT4_E2M1: case DataType::DT_FLOAT4_E1M2: case DataType::DT_INT4: return 4;
            default: return 0;
        }
    }
    // Operand / result combinations of the Mmad data-type table (Mmad.md:186-237, MmadMx.md:160-171).
    bool TypesValid() const
    {
        if (!a_.set || !b_.set || !c_.set) return false;
        const DataType a = a_.dtype, b = b_.dtype, c = c_.dtype;
        const bool same = a == b || (IsBf16(a) && IsBf16(b));
        if (!same) return false;
        if (a == DataType::DT_FLOAT16 || IsBf16(a) || a == DataType::DT_FLOAT)
            return c == DataType::DT_FLOAT || c == DataType::DT_FLOAT16 || IsBf16(c) || c == DataType::DT_INT8;
        if (a == DataType::DT_INT8 || a == DataType::DT_INT4)
            return c == DataType::DT_INT32 || c == DataType::DT_FLOAT16 || c == DataType::DT_INT8 || IsBf16(c);
        if (ElemBits(a) == 4 || ElemBits(a) == 8)  // fp4 / fp8 need the MX mode
            return mad_ == MatrixMadType::MXMODE && (c == DataType::DT_FLOAT || c == DataType::DT_FLOAT16 || IsBf16(c) || c == DataType::DT_INT8);
        return false;
    }
    static int32_t Align16(int32_t v) { return (v + 15) / 16 * 16; }
    // Fills every field for a block of singleM x singleN x singleK computed by `cores` cores.
    int64_t Fill(optiling::TCubeTiling& t, int32_t cores, int32_t singleM, int32_t singleN, int32_t singleK)
    {
        if (m_ <= 0 || n_ <= 0 || k_ <= 0 || !TypesValid()) return -1;
        if (mad_ == MatrixMadType::MXMODE && k_ % 64 != 0) return -1;  // MmadMx.md:187
        const int bits = ElemBits(a_.dtype);
        // B200 tile: 128 rows x up to 256 columns x 128 bytes of K per pipeline stage
        const int32_t tileK = bits == 32 ? 32 : 128 * 8 / bits;
        baseM_ = fixM_ != -1 ? fixM_ : std::min(128, Align16(singleM));
        baseN_ = fixN_ != -1 ? fixN_ : std::min(256, Align16(singleN));
        baseK_ = fixK_ != -1 ? fixK_ : std::min(tileK, Align16(singleK));
        const int32_t orgM = orgM_ > 0 ? orgM_ : m_, orgN = orgN_ > 0 ? orgN_ : n_;
        const int32_t orgKa = orgKa_ > 0 ? orgKa_ : k_, orgKb = orgKb_ > 0 ? orgKb_ : k_;
        t = optiling::TCubeTiling();
        t.set_usedCoreNum(cores);
        t.set_M(orgM);
        t.set_N(orgN);
        t.set_Ka(orgKa);
        t.set_Kb(orgKb);
        t.set_singleCoreM(singleM);
        t.set_singleCoreN(singleN);
        t.set_singleCoreK(singleK);
        t.set_baseM(baseM_);
        t.set_baseN(baseN_);
        t.set_baseK(baseK_);
        const int32_t stages = 4;
        t.set_depthA1(stages);
        t.set_depthB1(stages);
        t.set_stepM(1);
        t.set_stepN(1);
        t.set_stepKa(stages);
        t.set_stepKb(stages);
        t.set_isBias(isBias_ ? 1 : 0);
        t.set_iterateOrder(traverse_ == MatrixTraverse::FIRSTN ? 1 : 0);
        t.set_dbL0A(2);
        t.set_dbL0B(2);
        t.set_dbL0C(2);
        const int64_t tileBytes = static_cast<int64_t>(baseM_ + baseN_) * baseK_ * bits / 8 * stages;
        t.set_shareL1Size(static_cast<int32_t>(std::min<int64_t>(tileBytes, 227 * 1024)));
        t.set_shareL0CSize(baseM_ * baseN_ * 4);
        t.set_transLength(0);
        t.set_batchM(1);
        t.set_batchN(1);
        t.set_singleBatchM(1);
        t.set_singleBatchN(1);
        t.set_BatchNum(batchNum_ > 0 ? batchNum_ : 1);
        t.set_ALayoutInfoB(aLayout_[0]);
        t.set_ALayoutInfoS(aLayout_[1]);
        t.set_ALayoutInfoN(aLayout_[2]);
        t.set_ALayoutInfoG(aLayout_[3]);
        t.set_ALayoutInfoD(aLayout_[4]);
        t.set_BLayoutInfoB(bLayout_[0]);
        t.set_BLayoutInfoS(bLayout_[1]);
        t.set_BLayoutInfoN(bLayout_[2]);
        t.set_BLayoutInfoG(bLayout_[3]);
        t.set_BLayoutInfoD(bLayout_[4]);
        t.set_CLayoutInfoB(cLayout_[0]);
        t.set_CLayoutInfoS1(cLayout_[1]);
        t.set_CLayoutInfoN(cLayout_[2]);
        t.set_CLayoutInfoG(cLayout_[3]);
        t.set_CLayoutInfoS2(cLayout_[4]);
        t.set_mxTypePara(mad_ == MatrixMadType::MXMODE ? 1 : 0);
        return 0;
    }

    MatmulTypeDesc a_, b_, c_, bias_;
    bool scaleATrans_ = false, scaleBTrans_ = true, isBias_ = false;
    DequantType dequant_ = DequantType::SCALAR;
    MatrixTraverse traverse_ = MatrixTraverse::NOSET;
    MatrixMadType mad_ = MatrixMadType::NORMAL;
    int32_t m_ = 0, n_ = 0, k_ = 0, orgM_ = 0, orgN_ = 0, orgKa_ = 0, orgKb_ = 0;
    int32_t aLayout_[5] = {0, 0, 0, 0, 0}, bLayout_[5] = {0, 0, 0, 0, 0}, cLayout_[5] = {0, 0, 0, 0, 0}, batchNum_ = 0;
    int32_t fixM_ = -1, fixN_ = -1, fixK_ = -1, baseM_ = 0, baseN_ = 0, baseK_ = 0;
    int32_t cores_ = 1;
};

// Single-core tiling: the whole SetShape block belongs to one operator object.
class MatmulApiTiling : public MatmulApiTilingBase {
public:
    using MatmulApiTilingBase::GetTiling;
    using MatmulApiTilingBase::MatmulApiTilingBase;
    int64_t GetTiling(optiling::TCubeTiling& tiling) override { return Fill(tiling, 1, m_, n_, k_); }
};

// Multi-core tiling: splits M x N over at most SetDim() blocks with 16-aligned single-core extents
// (the rule tests/api/adv_api/tiling/test_matmul_api_tiling.cpp:28-56 checks).  With SetDim(1) the one
// block is the whole problem, which is how a B200 launch should be driven.
class MultiCoreMatmulTiling : public MatmulApiTilingBase {
public:
    using MatmulApiTilingBase::GetTiling;
    using MatmulApiTilingBase::MatmulApiTilingBase;
    int32_t SetDim(int32_t dim)
    {
        if (dim <= 0) return -1;
        dim_ = dim;
        return 0;
    }
    int32_t SetSingleShape(int32_t singleM = -1, int32_t singleN = -1, int32_t singleK = -1)
    {
        userM_ = singleM;
        userN_ = singleN;
        userK_ = singleK;
        return 0;
    }
    int32_t SetSingleRange(int32_t = -1, int32_t = -1, int32_t = -1, int32_t = -1, int32_t = -1, int32_t = -1) { return 0; }
    int32_t GetSingleShape(int32_t& shapeM, int32_t& shapeN, int32_t& shapeK) const
    {
        shapeM = singleM_;
        shapeN = singleN_;
        shapeK = singleK_;
        return 0;
    }
    int32_t GetCoreNum(int32_t& dim, int32_t& mDim, int32_t& nDim) const
    {
        dim = mDim_ * nDim_;
        mDim = mDim_;
        nDim = nDim_;
        return 0;
    }
    int64_t GetTiling(optiling::TCubeTiling& tiling) override
    {
        if (m_ <= 0 || n_ <= 0 || k_ <= 0) return -1;
        int bestM = 1, bestN = 1;
        int64_t bestCost = -1;
        for (int dm = 1; dm <= dim_; ++dm) {
            const int dn = dim_ / dm;
            if (dn < 1) break;
            const int32_t sm = Align16((m_ + dm - 1) / dm), sn = Align16((n_ + dn - 1) / dn);
            const int usedM = (m_ + sm - 1) / sm, usedN = (n_ + sn - 1) / sn;
            // per-core work first, then operand traffic (sm + sn) as the tie-break
            const int64_t cost = static_cast<int64_t>(sm) * sn * 4096 + sm + sn - (usedM * usedN == dim_ ? 1 : 0);
            if (bestCost < 0 || cost < bestCost) {
                bestCost = cost;
                bestM = dm;
                bestN = dn;
            }
        }
        singleM_ = userM_ > 0 ? userM_ : (dim_ == 1 ? m_ : Align16((m_ + bestM - 1) / bestM));
        singleN_ = userN_ > 0 ? userN_ : (dim_ == 1 ? n_ : Align16((n_ + bestN - 1) / bestN));
        singleK_ = userK_ > 0 ? userK_ : k_;
        mDim_ = (m_ + singleM_ - 1) / singleM_;
        nDim_ = (n_ + singleN_ - 1) / singleN_;
        return Fill(tiling, mDim_ * nDim_, singleM_, singleN_, singleK_);
    }

private:
    int32_t dim_ = 1, userM_ = -1, userN_ = -1, userK_ = -1, singleM_ = 0, singleN_ = 0, singleK_ = 0, mDim_ = 1, nDim_ = 1;
};

// Batch tiling (include/adv_api/matmul/bmm_tiling.h:186-242): one block computes whole matrices of the batch; on a B200 the
// batch runs as one launch per matrix pair on one device, so the used core count is 1 and no batch axis is split.
class BatchMatmulTiling : public MatmulApiTilingBase {
public:
    using MatmulApiTilingBase::GetTiling;
    using MatmulApiTilingBase::MatmulApiTilingBase;
    int32_t GetCoreNum(int32_t& dim, int32_t& mDim, int32_t& nDim, int32_t& batchCoreM, int32_t& batchCoreN) const
    {
        dim = mDim = nDim = batchCoreM = batchCoreN = 1;
        return 0;
    }
    int64_t GetTiling(optiling::TCubeTiling& tiling) override { return Fill(tiling, 1, m_, n_, k_); }
};
}  // namespace matmul_tiling

namespace AscendC {
using TensorShape = ge::Shape;

namespace tiling_detail {
constexpr uint32_t kBlk = 32, kHalf = 2, kFloat = 4, kBasicTileNum = kBlk / kFloat, kBasicUnit = 64, kBasicMin = 256;
inline bool SoftmaxArgsOk(const TensorShape& s, uint32_t typeSize)
{
    return s.GetShapeSize() > 0 && (typeSize == kHalf || typeSize == kFloat);
}
inline void LastAxis(const TensorShape& s, uint32_t& m, uint32_t& k)
{
    k = static_cast<uint32_t>(s.GetDims().back());
    m = static_cast<uint32_t>(s.GetShapeSize() / k);
}
}  // namespace tiling_detail

// impl/adv_api/tiling/activation/softmax_tiling.cpp:88-148 (the formula of the non-"regbase" architectures;
// the sizes describe the reference's on-chip scratch and are informational on B200: the kernels need none)
inline uint32_t GetSoftMaxMaxTmpSize(const TensorShape& srcShape, const uint32_t dataTypeSize, const bool /*isReuseSource*/)
{
    using namespace tiling_detail;
    if (!SoftmaxArgsOk(srcShape, dataTypeSize)) return 0;
    uint32_t m, k;
    LastAxis(srcShape, m, k);
    return m * (kBlk / dataTypeSize + k + kBasicUnit) * kFloat;
}
inline uint32_t GetSoftMaxMinTmpSize(const TensorShape& srcShape, const uint32_t dataTypeSize, const bool /*isReuseSource*/)
{
    using namespace tiling_detail;
    if (!SoftmaxArgsOk(srcShape, dataTypeSize)) return 0;
    uint32_t m, k;
    LastAxis(srcShape, m, k);
    return (kBlk / dataTypeSize + k + kBasicUnit) * kFloat;
}
// impl/adv_api/tiling/activation/softmax_tiling.cpp:150-215
inline void SoftMaxTilingFunc(const TensorShape& srcShape, const uint32_t dataTypeSize, const uint32_t localWorkSpaceSize,
                              optiling::SoftMaxTiling& tiling)
{
    using namespace tiling_detail;
    if (!SoftmaxArgsOk(srcShape, dataTypeSize)) return;
    uint32_t rows, cols;
    LastAxis(srcShape, rows, cols);
    const uint32_t statCols = kBlk / dataTypeSize;  // one 32-byte block of max / sum values per row

    // Rows per pass: what the scratch holds (a row needs its cols values, its statistics block and one basic unit, all fp32),
    // in whole basic tiles when the matrix is split at all; shapes made of basic blocks get a divisor of the row count that
    // also keeps a pass under the basic-block size.
    uint32_t pass = std::min((localWorkSpaceSize / kFloat) / (statCols + cols + kBasicUnit), rows);
    const auto wholeTiles = [](uint32_t r) { return r - r % kBasicTileNum; };
    if (pass < rows && pass > kBasicTileNum) pass = wholeTiles(pass);
    const bool basicBlocks = rows % kBasicTileNum == 0 && cols % kBasicUnit == 0;
    if (basicBlocks && pass > kBasicTileNum) {
        for (pass = wholeTiles(pass); rows % pass != 0;) pass -= kBasicTileNum;
        while (pass * cols >= kBasicUnit * kBasicMin) pass >>= 1;
    }
    const uint32_t passes = pass ? rows / pass : 0, left = pass ? rows % pass : 0;

    // The structure describes three row ranges (whole source, one pass, the last partial pass), each as the data rectangle
    // rows x cols and the statistics rectangle rows x statCols.
    tiling.set_srcM(rows), tiling.set_srcK(cols), tiling.set_srcSize(rows * cols);
    tiling.set_outMaxM(rows), tiling.set_outMaxK(statCols), tiling.set_outMaxSize(rows * statCols);
    tiling.set_splitM(pass), tiling.set_splitK(cols), tiling.set_splitSize(pass * cols);
    tiling.set_reduceM(pass), tiling.set_reduceK(statCols), tiling.set_reduceSize(pass * statCols);
    if (pass) tiling.set_rangeM(passes);
    tiling.set_tailM(left), tiling.set_tailSplitSize(left * cols), tiling.set_tailReduceSize(left * statCols);
}
inline void SoftMaxTilingFunc(const TensorShape& srcShape, const uint32_t dataTypeSize, const uint32_t localWorkSpaceSize, ::SoftMaxTiling& tiling)
{
    optiling::SoftMaxTiling t;
    SoftMaxTilingFunc(srcShape, dataTypeSize, localWorkSpaceSize, t);
    tiling = t.Data();
}
// impl/adv_api/tiling/activation/softmax_tiling.cpp:522-544
inline bool IsBasicBlockInSoftMax(optiling::SoftMaxTiling& tiling, const uint32_t dataTypeSize = 2)
{
    if (dataTypeSize == 0) return false;
    const uint32_t srcK = tiling.get_srcK();
    return tiling.get_tailM() == 0 && srcK >= (tiling_detail::kBasicMin / dataTypeSize) && srcK < 2048 && srcK % tiling_detail::kBasicUnit == 0;
}
inline bool IsBasicBlockInSoftMax(::SoftMaxTiling& tiling, const uint32_t dataTypeSize = 2)
{
    optiling::SoftMaxTiling t;
    t.set_srcK(tiling.srcK);
    t.set_tailM(tiling.tailM);
    return IsBasicBlockInSoftMax(t, dataTypeSize);
}

// impl/adv_api/tiling/quantization/ascend_quant_tiling_impl.cpp:25-70
inline void GetAscendQuantMaxMinTmpSize(const TensorShape& srcShape, const uint32_t /*typeSize*/, uint32_t& maxValue, uint32_t& minValue)
{
    const uint32_t inputSize = static_cast<uint32_t>(srcShape.GetShapeSize());
    const uint32_t maxVal = std::max(inputSize * 2u, 2u * 256u);
    maxValue = (maxVal + 31u) / 32u * 32u;
    minValue = 2u * 256u;
}
inline void GetAscendQuantTmpBufferFactorSize(uint32_t& maxLiveNodeCount, uint32_t& extraBuf)
{
    extraBuf = 0u;
    maxLiveNodeCount = 2u;
}
// impl/adv_api/tiling/quantization/ascend_dequant_tiling_impl.cpp:27-105
inline void GetAscendDequantMaxMinTmpSize(const TensorShape& srcShape, const uint32_t /*typeSize*/, uint32_t& maxValue, uint32_t& minValue)
{
    const std::vector<int64_t>& dims = srcShape.GetDims();
    uint32_t outer = 1, inner = 0;
    if (dims.size() == 2) {
        outer = static_cast<uint32_t>(dims[0]);
        inner = static_cast<uint32_t>(dims[1]);
    } else if (dims.size() == 1) {
        inner = static_cast<uint32_t>(dims[0]);
    } else {
        return;
    }
    const uint32_t deqScaleSize = inner + 8u;
    maxValue = (64u + outer * inner + deqScaleSize) * 4u;
    minValue = (64u + inner + deqScaleSize) * 4u;
}
inline void GetAscendDequantTmpBufferFactorSize(const TensorShape& srcShape, uint32_t& maxLiveNodeCount, uint32_t& extraBuf)
{
    const std::vector<int64_t>& dims = srcShape.GetDims();
    extraBuf = 8u + 64u;
    if (dims.size() == 2) {
        extraBuf += static_cast<uint32_t>(dims[1]);
        maxLiveNodeCount = 1u;
    } else if (dims.size() == 1) {
        maxLiveNodeCount = 2u;
    } else {
        extraBuf = 0u;
        maxLiveNodeCount = 0u;
    }
}
}  // namespace AscendC
