// Host tiling known-answer tests.  The expected numbers are those the reference's own tiling tests
// assert (tests/api/adv_api/tiling/test_tiling.cpp:3441-3462,3799-3864,6589-6660 and
// tests/api/adv_api/tiling/test_matmul_api_tiling.cpp:28-56), minus the ones that size Ascend L1.
#include <cstdio>
#include <vector>

#include "tiling/tiling_api.h"

static int g_fail = 0;
#define EXPECT_EQ(a, b)                                                                                     \
    do {                                                                                                    \
        const long long va = static_cast<long long>(a), vb = static_cast<long long>(b);                     \
        if (va != vb) {                                                                                     \
            std::printf("FAIL %s:%d: %s = %lld, expected %s = %lld\n", __FILE__, __LINE__, #a, va, #b, vb); \
            ++g_fail;                                                                                       \
        }                                                                                                   \
    } while (0)

int main()
{
    using namespace AscendC;
    {   // SoftMax, shape [128,128] half
        ge::Shape shape(std::vector<int64_t>{128, 128});
        EXPECT_EQ(GetSoftMaxMinTmpSize(shape, 2, true), (16 + 128 + 64) * 4);
        EXPECT_EQ(GetSoftMaxMaxTmpSize(shape, 2, true), 128 * (16 + 128 + 64) * 4);
        EXPECT_EQ(GetSoftMaxMaxTmpSize(shape, 1, true), 0);
        optiling::SoftMaxTiling t;
        SoftMaxTilingFunc(shape, 2, 100 * 1024 * 4, t);
        EXPECT_EQ(t.get_reduceM(), 64);
        EXPECT_EQ(IsBasicBlockInSoftMax(t), true);
        EXPECT_EQ(t.get_srcM(), 128);
        EXPECT_EQ(t.get_srcK(), 128);
        EXPECT_EQ(t.get_outMaxK(), 16);
        EXPECT_EQ(t.get_rangeM(), 2);
        EXPECT_EQ(t.get_tailM(), 0);
        ::SoftMaxTiling pod;
        SoftMaxTilingFunc(shape, 2, 100 * 1024 * 4, pod);
        EXPECT_EQ(pod.reduceM, 64);
        EXPECT_EQ(t.GetDataSize(), 64);
        // the baseline row-op shape: every row in one pass
        ge::Shape big(std::vector<int64_t>{4096, 2048});
        SoftMaxTilingFunc(big, 2, GetSoftMaxMaxTmpSize(big, 2, false), t);
        EXPECT_EQ(t.get_srcM(), 4096);
        EXPECT_EQ(t.get_srcK(), 2048);
        EXPECT_EQ(t.get_splitM() * t.get_rangeM() + t.get_tailM(), 4096);
    }
    {   // AscendQuant / AscendDequant scratch sizes
        uint32_t maxV = 0, minV = 0, live = 0, extra = 0;
        GetAscendQuantMaxMinTmpSize(ge::Shape(std::vector<int64_t>{512}), 2, maxV, minV);
        EXPECT_EQ(minV, 2 * 256);
        EXPECT_EQ(maxV, 2 * 512);
        GetAscendQuantTmpBufferFactorSize(live, extra);
        EXPECT_EQ(live, 2);
        EXPECT_EQ(extra, 0);
        GetAscendDequantMaxMinTmpSize(ge::Shape(std::vector<int64_t>{10, 32}), 4, maxV, minV);
        EXPECT_EQ(minV, 4 * (64 + 32 + 40));
        EXPECT_EQ(maxV, 4 * (64 + 32 * 10 + 40));
        GetAscendDequantTmpBufferFactorSize(ge::Shape(std::vector<int64_t>{10, 32}), live, extra);
        EXPECT_EQ(live, 1);
        EXPECT_EQ(extra, 104);
        GetAscendDequantMaxMinTmpSize(ge::Shape(std::vector<int64_t>{320}), 4, maxV, minV);
        EXPECT_EQ(minV, 4 * (64 + 320 + 328));
        EXPECT_EQ(maxV, 4 * (64 + 320 + 328));
        GetAscendDequantTmpBufferFactorSize(ge::Shape(std::vector<int64_t>{320}), live, extra);
        EXPECT_EQ(live, 2);
        EXPECT_EQ(extra, 72);
        GetAscendDequantTmpBufferFactorSize(ge::Shape(std::vector<int64_t>{2, 3, 4}), live, extra);
        EXPECT_EQ(live, 0);
        EXPECT_EQ(extra, 0);
    }
    {   // Matmul: SetFixSplit is echoed
        using namespace matmul_tiling;
        MatmulApiTiling tiling;
        tiling.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT16);
        tiling.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT16);
        tiling.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT);
        tiling.SetBiasType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT);
        tiling.SetShape(1024, 1024, 1024);
        tiling.SetOrgShape(1024, 1024, 1024);
        tiling.EnableBias(true);
        tiling.SetBufferSpace(-1, 128 * 1024, -1);
        tiling.SetDoubleBuffer(false, false, false, false, false, false);
        tiling.SetTraverse(MatrixTraverse::FIRSTM);
        tiling.SetMadType(MatrixMadType::NORMAL);
        tiling.SetSplitRange(128, 128, 128);
        EXPECT_EQ(tiling.SetFixSplit(16, 16, 16), 0);
        optiling::TCubeTiling data;
        EXPECT_EQ(tiling.GetTiling(data), 0);
        EXPECT_EQ(data.get_baseM(), 16);
        EXPECT_EQ(data.get_baseN(), 16);
        EXPECT_EQ(data.get_isBias(), 1);
        EXPECT_EQ(data.get_M(), 1024);
        EXPECT_EQ(data.GetDataSize(), 200);
        EXPECT_EQ(tiling.SetFixSplit(17, 16, 16), -1);
        ::TCubeTiling pod;
        uint8_t buf[200];
        data.SaveToBuffer(buf, sizeof(buf));
        std::memcpy(&pod, buf, sizeof(pod));
        EXPECT_EQ(pod.baseM, 16);
        EXPECT_EQ(pod.singleCoreK, 1024);
    }
    {   // Matmul: return codes
        using namespace matmul_tiling;
        optiling::TCubeTiling data;
        MatmulApiTiling bad;
        bad.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT16);
        bad.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_INT8);  // operand types differ
        bad.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT);
        bad.SetShape(64, 64, 64);
        EXPECT_EQ(bad.GetTiling(data), -1);
        MatmulApiTiling noShape;
        noShape.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_INT8);
        noShape.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_INT8);
        noShape.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_INT32);
        EXPECT_EQ(noShape.GetTiling(data), -1);
        noShape.SetShape(64, 64, 64);
        EXPECT_EQ(noShape.GetTiling(data), 0);
        MatmulApiTiling mx;  // fp4 needs the MX mode and K % 64 == 0
        mx.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT4_E2M1);
        mx.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT4_E2M1, true);
        mx.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_BF16);
        mx.SetShape(256, 256, 256);
        EXPECT_EQ(mx.GetTiling(data), -1);
        mx.SetMadType(MatrixMadType::MXMODE);
        EXPECT_EQ(mx.GetTiling(data), 0);
        EXPECT_EQ(data.get_mxTypePara(), 1);
        mx.SetShape(256, 256, 96);
        EXPECT_EQ(mx.GetTiling(data), -1);
    }
    {   // Multi-core: single-core extents are multiples of 16 and cover the problem
        using namespace matmul_tiling;
        optiling::TCubeTiling data;
        MultiCoreMatmulTiling api;
        api.SetDim(10);
        api.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::NZ, DataType::DT_FLOAT, true);
        api.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::NZ, DataType::DT_FLOAT);
        api.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::NZ, DataType::DT_FLOAT);
        api.SetBiasType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT16);
        api.SetOrgShape(736, 7168, 4096);
        api.SetShape(736, 7168, 4096);
        api.EnableBias(true);
        api.SetBufferSpace(-1, -1, -1);
        EXPECT_EQ(api.GetTiling(data), 0);
        int32_t sm = 1, sn = 1, sk = 1;
        api.GetSingleShape(sm, sn, sk);
        EXPECT_EQ(sm % 16, 0);
        EXPECT_EQ(sn % 16, 0);
        EXPECT_EQ(sk, 4096);
        int32_t dim, mDim, nDim;
        api.GetCoreNum(dim, mDim, nDim);
        EXPECT_EQ(dim <= 10, true);
        EXPECT_EQ(static_cast<long long>(sm) * mDim >= 736 && static_cast<long long>(sn) * nDim >= 7168, true);
        EXPECT_EQ(data.get_usedCoreNum(), dim);
        // one core = the whole problem, unaligned extents kept as they are
        MultiCoreMatmulTiling one(*platform_ascendc::PlatformAscendCManager::GetInstance());
        one.SetDim(1);
        one.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT16);
        one.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT16);
        one.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, DataType::DT_FLOAT);
        one.SetShape(512, 1024, 512);
        EXPECT_EQ(one.GetTiling(data), 0);
        EXPECT_EQ(data.get_singleCoreM(), 512);
        EXPECT_EQ(data.get_singleCoreN(), 1024);
        EXPECT_EQ(data.get_usedCoreNum(), 1);
    }
    std::printf(g_fail ? "%d checks failed\n" : "tiling ok\n", g_fail);
    return g_fail ? 1 : 0;
}
