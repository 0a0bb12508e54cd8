// Drives the C++ mirror of the reference operator API on a B200, following the call sequences of the
// reference examples (Matmul: examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul/matmul.asc:95-184;
// matmul_quant; SoftMax; AscendQuant; AscendDequant) and checks the results on the host.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <random>
#include <vector>

#include "lib/matmul_intf.h"
#include "tiling/tiling_api.h"

static int g_fail = 0;
#define CHECK(cond, ...)                      \
    do {                                      \
        if (!(cond)) {                        \
            std::printf("FAIL %s:%d: ", __FILE__, __LINE__); \
            std::printf(__VA_ARGS__);         \
            std::printf("\n");                \
            ++g_fail;                         \
        }                                     \
    } while (0)

template <class T>
struct DevBuf {
    T* p = nullptr;
    size_t n = 0;
    explicit DevBuf(size_t count) : n(count) { ascb200_malloc(reinterpret_cast<void**>(&p), count * sizeof(T)); }
    explicit DevBuf(const std::vector<T>& h) : DevBuf(h.size()) { Upload(h); }
    ~DevBuf() { ascb200_free(p); }
    void Upload(const std::vector<T>& h)
    {
        ascb200_memcpy_h2d(p, h.data(), h.size() * sizeof(T), nullptr);
        ascb200_stream_sync(nullptr);
    }
    std::vector<T> Download() const
    {
        std::vector<T> h(n);
        ascb200_memcpy_d2h(h.data(), p, n * sizeof(T), nullptr);
        ascb200_stream_sync(nullptr);
        return h;
    }
};

// The example's kernel class, as host code (matmul.asc:41-141): one "core" owns the whole problem.
template <typename AType, typename BType, typename CType, typename BiasType>
class MatmulKernel {
public:
    void Init(GM_ADDR a, GM_ADDR b, GM_ADDR bias, GM_ADDR c, const TCubeTiling& tiling)
    {
        this->tiling = tiling;
        aGlobal.SetGlobalBuffer(reinterpret_cast<AType*>(a), tiling.M * tiling.Ka);
        bGlobal.SetGlobalBuffer(reinterpret_cast<BType*>(b), tiling.Kb * tiling.N);
        cGlobal.SetGlobalBuffer(reinterpret_cast<CType*>(c), tiling.M * tiling.N);
        biasGlobal.SetGlobalBuffer(reinterpret_cast<BiasType*>(bias), tiling.N);
        const int64_t blockIdx = AscendC::GetBlockIdx();
        const auto mSingleBlocks = (tiling.M + tiling.singleCoreM - 1) / tiling.singleCoreM;
        const auto mCoreIndx = blockIdx % mSingleBlocks, nCoreIndx = blockIdx / mSingleBlocks;
        aGlobal = aGlobal[mCoreIndx * tiling.Ka * tiling.singleCoreM];
        bGlobal = bGlobal[nCoreIndx * tiling.singleCoreN];
        cGlobal = cGlobal[mCoreIndx * tiling.N * tiling.singleCoreM + nCoreIndx * tiling.singleCoreN];
        biasGlobal = biasGlobal[nCoreIndx * tiling.singleCoreN];
    }
    void Process(AscendC::TPipe* pipe)
    {
        (void)pipe;
        matmulObj.SetTensorA(aGlobal, false);
        matmulObj.SetTensorB(bGlobal, false);
        if (tiling.isBias) matmulObj.SetBias(biasGlobal);
        matmulObj.IterateAll(cGlobal);
        matmulObj.End();
    }
    AscendC::Matmul<AscendC::MatmulType<AscendC::TPosition::GM, CubeFormat::ND, AType>, AscendC::MatmulType<AscendC::TPosition::GM, CubeFormat::ND, BType>,
                    AscendC::MatmulType<AscendC::TPosition::GM, CubeFormat::ND, CType>, AscendC::MatmulType<AscendC::TPosition::GM, CubeFormat::ND, BiasType>,
                    CFG_NORM>
        matmulObj;

private:
    AscendC::GlobalTensor<AType> aGlobal;
    AscendC::GlobalTensor<BType> bGlobal;
    AscendC::GlobalTensor<CType> cGlobal;
    AscendC::GlobalTensor<BiasType> biasGlobal;
    TCubeTiling tiling;
};

static void TestMatmulFp16()
{
    const int M = 512, N = 1024, K = 512;  // the baseline fp16 configuration
    std::mt19937 rng(0xA5C0);
    std::uniform_real_distribution<float> u(-1.f, 1.f);
    std::vector<half> a(M * K), b(K * N);
    std::vector<float> bias(N);
    for (auto& v : a) v = half(u(rng));
    for (auto& v : b) v = half(u(rng));
    for (auto& v : bias) v = u(rng);

    // host tiling exactly as the example's GenerateTiling (matmul.asc:158-184)
    auto* platform = platform_ascendc::PlatformAscendCManager::GetInstance();
    optiling::TCubeTiling tilingData;
    matmul_tiling::MultiCoreMatmulTiling tilingApi(*platform);
    tilingApi.SetDim(1);
    tilingApi.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_FLOAT16, false);
    tilingApi.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_FLOAT16, false);
    tilingApi.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_FLOAT);
    tilingApi.SetBiasType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_FLOAT);
    tilingApi.SetOrgShape(M, N, K);
    tilingApi.SetShape(M, N, K);
    tilingApi.EnableBias(true);
    tilingApi.SetBufferSpace(-1, -1, -1);
    CHECK(tilingApi.GetTiling(tilingData) == 0, "GetTiling");
    std::vector<uint8_t> tilingBuf(tilingData.GetDataSize());
    tilingData.SaveToBuffer(tilingBuf.data(), tilingBuf.size());

    DevBuf<half> dA(a), dB(b);
    DevBuf<float> dBias(bias), dC(static_cast<size_t>(M) * N);
    {   // the example's kernel body (matmul.asc:144-156)
        TCubeTiling tiling;
        std::memcpy(&tiling, tilingBuf.data(), sizeof(tiling));
        AscendC::TPipe pipe;
        MatmulKernel<half, half, float, float> kernel;
        REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), kernel.matmulObj, &tiling);
        kernel.Init(reinterpret_cast<GM_ADDR>(dA.p), reinterpret_cast<GM_ADDR>(dB.p), reinterpret_cast<GM_ADDR>(dBias.p),
                    reinterpret_cast<GM_ADDR>(dC.p), tiling);
        kernel.Process(&pipe);
    }
    CHECK(AscendC::GetLastError() == 0, "operator error %d", AscendC::GetLastError());
    const std::vector<float> c = dC.Download();
    std::vector<float> af(a.begin(), a.end()), bf(b.begin(), b.end());
    double worst = 0;
    for (int m = 0; m < M; m += 7)
        for (int n = 0; n < N; n += 5) {
            float acc = bias[n];
            for (int k = 0; k < K; ++k) acc += af[m * K + k] * bf[k * N + n];
            const double err = std::fabs(c[static_cast<size_t>(m) * N + n] - acc);
            worst = std::max(worst, err);
            if (err > 1e-3 + 1e-2 * std::fabs(acc)) {
                CHECK(false, "C[%d,%d] = %f, expected %f", m, n, c[static_cast<size_t>(m) * N + n], acc);
                return;
            }
        }
    std::printf("matmul fp16 512x512x1024+bias: max abs err %.3g\n", worst);
}

static void TestMatmulQuant()
{
    // matmul_quant example flow: int8 x int8 -> half through SetQuantVector (per-channel DEQF16) and SetQuantScalar
    const int M = 256, N = 384, K = 256;
    std::mt19937 rng(7);
    std::uniform_int_distribution<int> ui(-10, 9);
    std::uniform_real_distribution<float> us(0.1f, 2.0f);
    std::vector<int8_t> a(M * K), b(K * N);
    for (auto& v : a) v = static_cast<int8_t>(ui(rng));
    for (auto& v : b) v = static_cast<int8_t>(ui(rng));
    std::vector<uint64_t> q(N);
    std::vector<float> alpha(N);
    for (int n = 0; n < N; ++n) {
        float s = us(rng);
        uint32_t bits;
        std::memcpy(&bits, &s, 4);
        q[n] = bits;  // the unit keeps bits [31:13]
        bits &= 0xFFFFE000u;
        std::memcpy(&alpha[n], &bits, 4);
    }
    matmul_tiling::MatmulApiTiling api;
    api.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT8);
    api.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT8);
    api.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_FLOAT16);
    api.SetShape(M, N, K);
    api.SetOrgShape(M, N, K);
    api.SetDequantType(matmul_tiling::DequantType::TENSOR);
    TCubeTiling tiling;
    CHECK(api.GetTiling(tiling) == 0, "GetTiling");

    DevBuf<int8_t> dA(a), dB(b);
    DevBuf<uint64_t> dQ(q);
    DevBuf<half> dC(static_cast<size_t>(M) * N);
    AscendC::TPipe pipe;
    using A = AscendC::MatmulType<AscendC::TPosition::GM, CubeFormat::ND, int8_t>;
    using C = AscendC::MatmulType<AscendC::TPosition::GM, CubeFormat::ND, half>;
    using B32 = AscendC::MatmulType<AscendC::TPosition::GM, CubeFormat::ND, int32_t>;
    AscendC::Matmul<A, A, C, B32> mm;
    REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
    AscendC::GlobalTensor<int8_t> ga, gb;
    AscendC::GlobalTensor<uint64_t> gq;
    AscendC::GlobalTensor<half> gc;
    ga.SetGlobalBuffer(dA.p, a.size());
    gb.SetGlobalBuffer(dB.p, b.size());
    gq.SetGlobalBuffer(dQ.p, q.size());
    gc.SetGlobalBuffer(dC.p, dC.n);
    for (int pass = 0; pass < 2; ++pass) {
        mm.SetTensorA(ga);
        mm.SetTensorB(gb);
        if (pass == 0) mm.SetQuantVector(gq);
        else mm.SetQuantScalar(q[3]);
        mm.IterateAll(gc);
        mm.End();
        ascb200_stream_sync(nullptr);
        const std::vector<half> c = dC.Download();
        int bad = 0;
        for (int m = 0; m < M; m += 3)
            for (int n = 0; n < N; ++n) {
                int32_t acc = 0;
                for (int k = 0; k < K; ++k) acc += static_cast<int32_t>(a[m * K + k]) * b[k * N + n];
                const half expect(static_cast<float>(acc) * (pass == 0 ? alpha[n] : alpha[3]));
                if (c[static_cast<size_t>(m) * N + n].bits != expect.bits) ++bad;
            }
        CHECK(bad == 0, "quant matmul pass %d: %d mismatches", pass, bad);
    }
    CHECK(AscendC::GetLastError() == 0, "operator error %d", AscendC::GetLastError());
}

static void TestSoftmaxQuantDequant()
{
    const uint32_t M = 64, K = 2048;
    std::mt19937 rng(11);
    std::normal_distribution<float> nd(0.f, 3.f);
    std::vector<half> x(M * K);
    for (auto& v : x) v = half(nd(rng));
    DevBuf<half> dX(x), dY(M * K);
    DevBuf<float> dSum(M * 8), dMax(M * 8);
    ::SoftMaxTiling tiling;
    ge::Shape shape(std::vector<int64_t>{M, K});
    AscendC::SoftMaxTilingFunc(shape, sizeof(half), AscendC::GetSoftMaxMaxTmpSize(shape, sizeof(half), false), tiling);
    AscendC::TPipe pipe;
    AscendC::LocalTensor<half> src(dX.p, M * K), dst(dY.p, M * K);
    AscendC::LocalTensor<float> sum(dSum.p, M * 8), mx(dMax.p, M * 8);
    AscendC::SoftMaxShapeInfo info{M, K, M, K};
    AscendC::SoftMax<half>(dst, sum, mx, src, tiling, info);
    // per-channel AscendQuant of the result
    std::vector<half> scale(K);
    std::uniform_real_distribution<float> u(0.5f, 2.0f);
    for (auto& s : scale) s = half(127.0f / u(rng));
    DevBuf<half> dScale(scale);
    DevBuf<int8_t> dQ(M * K);
    AscendC::LocalTensor<half> scaleT(dScale.p, K);
    AscendC::LocalTensor<int8_t> qT(dQ.p, M * K);
    AscendC::AscendQuant<half>(qT, dst, scaleT, half(0.0f), K, M * K);
    ascb200_stream_sync(nullptr);
    CHECK(AscendC::GetLastError() == 0, "operator error %d", AscendC::GetLastError());
    const auto y = dY.Download();
    const auto s = dSum.Download();
    const auto mxh = dMax.Download();
    const auto q = dQ.Download();
    int bad = 0, badq = 0;
    for (uint32_t r = 0; r < M; ++r) {
        float m = -INFINITY;
        for (uint32_t k = 0; k < K; ++k) m = std::max(m, static_cast<float>(x[r * K + k]));
        double tot = 0;
        for (uint32_t k = 0; k < K; ++k) tot += std::exp(static_cast<double>(static_cast<float>(x[r * K + k]) - m));
        if (mxh[r * 8] != m || mxh[r * 8 + 7] != m || std::fabs(s[r * 8] - tot) > 1e-5 * tot) ++bad;
        for (uint32_t k = 0; k < K; ++k) {
            const double ref = std::exp(static_cast<double>(static_cast<float>(x[r * K + k]) - m)) / tot;
            const float got = y[r * K + k];
            if (std::fabs(got - ref) > 1e-3 * ref + 6e-8) ++bad;
            // AscendQuant in fp16: half(y * scale) then round to nearest even, saturating
            const half prod(static_cast<float>(y[r * K + k]) * static_cast<float>(scale[k]));
            const float pf = prod;
            const int expect = static_cast<int>(std::max(-128.0f, std::min(127.0f, std::nearbyint(pf))));
            if (q[r * K + k] != expect) ++badq;
        }
    }
    CHECK(bad == 0, "softmax: %d bad values", bad);
    CHECK(badq == 0, "AscendQuant: %d mismatches", badq);

    // AscendDequant: int32 [m, n] x fp32 scale[n] -> fp32, the dequant example's shape
    const uint32_t dm = 128, dn = 32;
    std::vector<int32_t> src32(dm * dn);
    std::vector<float> dscale(dn);
    std::uniform_int_distribution<int> ui(-10, 9);
    std::uniform_real_distribution<float> us(-100.f, 100.f);
    for (auto& v : src32) v = ui(rng);
    for (auto& v : dscale) v = us(rng);
    DevBuf<int32_t> dSrc(src32);
    DevBuf<float> dDs(dscale), dOut(dm * dn);
    AscendC::LocalTensor<int32_t> srcT(dSrc.p, dm * dn);
    AscendC::LocalTensor<float> scT(dDs.p, dn), outT(dOut.p, dm * dn);
    AscendC::AscendDequant<float, float>(outT, srcT, scT, AscendC::DequantParams{dm, dn, dn});
    ascb200_stream_sync(nullptr);
    const auto out = dOut.Download();
    int badd = 0;
    for (uint32_t i = 0; i < dm * dn; ++i)
        if (out[i] != static_cast<float>(src32[i]) * dscale[i % dn]) ++badd;
    CHECK(badd == 0, "AscendDequant: %d mismatches", badd);
}

// B in the fractal NZ format of the grouped example's weights, result added into C (enAtomic = 1), and an
// ND_ALIGN output whose rows are padded to 32 bytes.
static void TestMatmulNzAtomicAlign()
{
    using namespace AscendC;
    const int M = 200, N = 96, K = 160;
    std::mt19937 rng(7);
    std::uniform_int_distribution<int> u(-10, 9);
    std::vector<int8_t> a(M * K), b(K * N), bNz(K * N);
    for (auto& v : a) v = static_cast<int8_t>(u(rng));
    for (auto& v : b) v = static_cast<int8_t>(u(rng));
    for (int k = 0; k < K; ++k)
        for (int n = 0; n < N; ++n) bNz[((static_cast<size_t>(n / 32) * (K / 16) + k / 16) * 16 + k % 16) * 32 + n % 32] = b[k * N + n];
    std::vector<int32_t> c0(M * N);
    for (auto& v : c0) v = u(rng) * 100;
    DevBuf<int8_t> dA(a), dB(bNz);
    DevBuf<int32_t> dC(c0);
    TCubeTiling tiling{};
    tiling.M = tiling.singleCoreM = M;
    tiling.N = tiling.singleCoreN = N;
    tiling.Ka = tiling.Kb = tiling.singleCoreK = K;
    {
        TPipe pipe;
        Matmul<MatmulType<TPosition::GM, CubeFormat::ND, int8_t>, MatmulType<TPosition::GM, CubeFormat::NZ, int8_t>,
               MatmulType<TPosition::GM, CubeFormat::ND, int32_t>, MatmulType<TPosition::GM, CubeFormat::ND, int32_t>>
            mm;
        REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
        GlobalTensor<int8_t> ga, gb;
        GlobalTensor<int32_t> gc;
        ga.SetGlobalBuffer(dA.p, a.size());
        gb.SetGlobalBuffer(dB.p, bNz.size());
        gc.SetGlobalBuffer(dC.p, c0.size());
        mm.SetTensorA(ga);
        mm.SetTensorB(gb);
        mm.IterateAll(gc, 1);
        mm.IterateAll(gc, 1);  // second call reuses the unpacked copy
        mm.End();
    }
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<int32_t> c = dC.Download();
    int bad = 0;
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            int32_t acc = 0;
            for (int k = 0; k < K; ++k) acc += static_cast<int32_t>(a[m * K + k]) * b[k * N + n];
            if (c[m * N + n] != c0[m * N + n] + 2 * acc) ++bad;
        }
    CHECK(bad == 0, "NZ B + atomic add: %d wrong", bad);

    const int N2 = 520, LD = 528;  // 520 halves = 1040 bytes -> padded to 1056
    std::vector<half> ah(M * K), bh(K * N2);
    std::uniform_real_distribution<float> uf(-1.f, 1.f);
    for (auto& v : ah) v = half(uf(rng));
    for (auto& v : bh) v = half(uf(rng));
    std::vector<half> cInit(static_cast<size_t>(M) * LD, half(-77.0f));
    DevBuf<half> dAh(ah), dBh(bh), dCh(cInit);
    tiling.N = tiling.singleCoreN = N2;
    {
        TPipe pipe;
        Matmul<MatmulType<TPosition::GM, CubeFormat::ND, half>, MatmulType<TPosition::GM, CubeFormat::ND, half>,
               MatmulType<TPosition::GM, CubeFormat::ND_ALIGN, half>, MatmulType<TPosition::GM, CubeFormat::ND, float>>
            mm;
        REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
        GlobalTensor<half> ga, gb, gc;
        ga.SetGlobalBuffer(dAh.p, ah.size());
        gb.SetGlobalBuffer(dBh.p, bh.size());
        gc.SetGlobalBuffer(dCh.p, cInit.size());
        mm.SetTensorA(ga);
        mm.SetTensorB(gb);
        mm.IterateAll(gc);
        mm.End();
    }
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<half> ch = dCh.Download();
    bad = 0;
    for (int m = 0; m < M; m += 3) {
        for (int n = 0; n < N2; n += 7) {
            float acc = 0;
            for (int k = 0; k < K; ++k) acc += static_cast<float>(ah[m * K + k]) * static_cast<float>(bh[k * N2 + n]);
            if (std::fabs(static_cast<float>(ch[static_cast<size_t>(m) * LD + n]) - acc) > 1e-3 + 1e-2 * std::fabs(acc)) ++bad;
        }
        for (int n = N2; n < LD; ++n)
            if (static_cast<float>(ch[static_cast<size_t>(m) * LD + n]) != -77.0f) ++bad;  // padding stays untouched
    }
    CHECK(bad == 0, "ND_ALIGN output: %d wrong", bad);
    std::printf("matmul NZ B + enAtomic, ND_ALIGN C: ok\n");
}

// AscendQuant<dstT, srcT, scaleT, isReuseSource, config, policy> with PER_TOKEN and PER_GROUP (fp4 destination).
static constexpr AscendC::AscendQuantConfig kQuantCfgOffset = {0, 0, 0, 0, true, 1, AscendC::RoundMode::CAST_RINT};
static constexpr AscendC::AscendQuantConfig kQuantCfgGroup = {0, 0, 0, 0, false, 1, AscendC::RoundMode::CAST_RINT};
static constexpr AscendC::AscendQuantPolicy kPerToken = AscendC::AscendQuantPolicy::PER_TOKEN;
static constexpr AscendC::AscendQuantPolicy kPerGroup = AscendC::AscendQuantPolicy::PER_GROUP;
static void TestQuantPolicies()
{
    using namespace AscendC;
    const uint32_t M = 24, N = 128;
    std::mt19937 rng(11);
    std::uniform_real_distribution<float> u(-4.f, 4.f);
    std::vector<half> x(M * N);
    for (auto& v : x) v = half(u(rng));
    std::vector<float> scale(M), offset(M);
    for (uint32_t i = 0; i < M; ++i) {
        scale[i] = 5.0f + 0.5f * i;
        offset[i] = static_cast<float>(i) - 10.0f;
    }
    DevBuf<half> dX(x);
    DevBuf<float> dS(scale), dO(offset);
    DevBuf<int8_t> dQ(M * N);
    TPipe pipe;
    AscendQuantParam para{M, N, M * N, 0};
    AscendQuant<int8_t, half, float, false, kQuantCfgOffset, kPerToken>(LocalTensor<int8_t>(dQ.p, dQ.n), LocalTensor<half>(dX.p, dX.n),
                                                                         LocalTensor<float>(dS.p, dS.n), LocalTensor<float>(dO.p, dO.n), para);
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<int8_t> q = dQ.Download();
    int bad = 0;
    for (uint32_t i = 0; i < M; ++i)
        for (uint32_t j = 0; j < N; ++j) {
            const float v = static_cast<float>(x[i * N + j]) * scale[i] + offset[i];
            const float r = std::nearbyint(std::fmin(std::fmax(v, -128.f), 127.f));
            if (q[i * N + j] != static_cast<int8_t>(r)) ++bad;
        }
    CHECK(bad == 0, "PER_TOKEN int8: %d wrong", bad);

    // PER_GROUP, groups of 32 columns, fp4 e2m1 destination (two values per byte): spot-check the decoded values
    std::vector<float> gscale(M * (N / 32), 0.5f);
    DevBuf<float> dGs(gscale);
    DevBuf<fp4x2_e2m1_t> dF(M * N / 2);
    AscendQuantParam gpara{M, N, M * N, 32};
    AscendQuant<fp4x2_e2m1_t, half, float, false, kQuantCfgGroup, kPerGroup>(LocalTensor<fp4x2_e2m1_t>(dF.p, dF.n), LocalTensor<half>(dX.p, dX.n),
                                                                               LocalTensor<float>(dGs.p, dGs.n), 0.0f, gpara);
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<fp4x2_e2m1_t> f = dF.Download();
    static const float grid[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    bad = 0;
    for (uint32_t e = 0; e < M * N; ++e) {
        const uint8_t code = (f[e / 2].bits >> (4 * (e & 1))) & 0xF;
        const float got = (code & 8 ? -1.f : 1.f) * grid[code & 7];
        const float want = static_cast<float>(x[e]) * 0.5f;  // |want| <= 2: the nearest grid point is within 0.25
        if (std::fabs(got - want) > 0.25f + 0.004f) ++bad;  // + half a bfloat16 step: the value passes through bfloat16 first
    }
    CHECK(bad == 0, "PER_GROUP fp4: %d values off the nearest grid point", bad);
    // AscendDequant PER_TOKEN: int32 -> float with one scale per row
    static constexpr AscendDeQuantConfig kDeqCfg = {false, 1};
    static constexpr AscendDeQuantPolicy kDeqPerToken = AscendDeQuantPolicy::PER_TOKEN;
    std::vector<int32_t> acc(M * N);
    for (uint32_t e = 0; e < M * N; ++e) acc[e] = static_cast<int32_t>(e * 37u % 20011u) - 10000;
    DevBuf<int32_t> dAcc(acc);
    DevBuf<float> dDeq(M * N);
    AscendDequant<float, int32_t, float, kDeqCfg, kDeqPerToken>(LocalTensor<float>(dDeq.p, dDeq.n), LocalTensor<int32_t>(dAcc.p, dAcc.n),
                                                                 LocalTensor<float>(dS.p, dS.n), LocalTensor<float>(dO.p, dO.n),
                                                                 AscendDeQuantParam{M, N, M * N, 0});
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<float> deq = dDeq.Download();
    bad = 0;
    for (uint32_t e = 0; e < M * N; ++e)
        if (deq[e] != static_cast<float>(acc[e]) * scale[e / N]) ++bad;
    CHECK(bad == 0, "AscendDequant PER_TOKEN: %d wrong", bad);
    std::printf("AscendQuant PER_TOKEN / PER_GROUP, AscendDequant PER_TOKEN: ok\n");
}

// SoftmaxFlashV2 over two K tiles (half data, float statistics), checked through the online-softmax identity.
static void TestSoftmaxFlashV2()
{
    using namespace AscendC;
    const uint32_t M = 16, K = 256;
    std::mt19937 rng(5);
    std::normal_distribution<float> nd(0.f, 2.f);
    std::vector<half> x1(M * K), x2(M * K);
    for (auto& v : x1) v = half(nd(rng));
    for (auto& v : x2) v = half(nd(rng) + 1.0f);
    DevBuf<half> d1(x1), d2(x2), dY(M * K), dEm(M * 16);
    DevBuf<float> dSum(M * 8), dMax(M * 8), dSum2(M * 8), dMax2(M * 8);
    SoftMaxTiling tiling{};
    tiling.srcM = M;
    tiling.srcK = K;
    TPipe pipe;
    SoftmaxFlashV2<half, false>(LocalTensor<half>(dY.p, dY.n), LocalTensor<float>(dSum.p, dSum.n), LocalTensor<float>(dMax.p, dMax.n),
                                LocalTensor<half>(d1.p, d1.n), LocalTensor<half>(dEm.p, dEm.n), LocalTensor<float>(dSum.p, dSum.n),
                                LocalTensor<float>(dMax.p, dMax.n), tiling);
    SoftmaxFlashV2<half, true>(LocalTensor<half>(dY.p, dY.n), LocalTensor<float>(dSum2.p, dSum2.n), LocalTensor<float>(dMax2.p, dMax2.n),
                               LocalTensor<half>(d2.p, d2.n), LocalTensor<half>(dEm.p, dEm.n), LocalTensor<float>(dSum.p, dSum.n),
                               LocalTensor<float>(dMax.p, dMax.n), tiling);
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<float> sum2 = dSum2.Download(), max2 = dMax2.Download();
    int bad = 0;
    for (uint32_t i = 0; i < M; ++i) {
        float mx = -1e30f;
        for (uint32_t j = 0; j < K; ++j) mx = std::fmax(mx, std::fmax(static_cast<float>(x1[i * K + j]), static_cast<float>(x2[i * K + j])));
        double s = 0;
        for (uint32_t j = 0; j < K; ++j) s += std::exp(static_cast<float>(x1[i * K + j]) - mx) + std::exp(static_cast<float>(x2[i * K + j]) - mx);
        if (max2[i * 8] != mx || max2[i * 8 + 7] != mx || std::fabs(sum2[i * 8] - s) > 2e-3 * s) ++bad;
    }
    CHECK(bad == 0, "SoftmaxFlashV2: %d rows wrong", bad);
    std::printf("SoftmaxFlashV2 two tiles: ok\n");
    // the first version (SoftmaxFlash) normalises: without update every row of dst sums to 1
    DevBuf<half> dY1(M * K);
    SoftmaxFlash<half>(LocalTensor<half>(dY1.p, dY1.n), LocalTensor<float>(dSum.p, dSum.n), LocalTensor<float>(dMax.p, dMax.n),
                       LocalTensor<half>(d1.p, d1.n), LocalTensor<half>(dEm.p, dEm.n), LocalTensor<float>(dSum.p, dSum.n),
                       LocalTensor<float>(dMax.p, dMax.n), tiling, false);
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<half> yn = dY1.Download();
    bad = 0;
    for (uint32_t i = 0; i < M; ++i) {
        double tot = 0;
        for (uint32_t j = 0; j < K; ++j) tot += static_cast<float>(yn[i * K + j]);
        if (std::fabs(tot - 1.0) > 2e-3) ++bad;
    }
    CHECK(bad == 0, "SoftmaxFlash: %d rows do not sum to 1", bad);
    std::printf("SoftmaxFlash (first version): ok\n");
}

// LogSoftMax as in the reference's logsoftmax example: statistics are LocalTensor<T>, one 32-byte block per row.
static void TestLogSoftMax()
{
    using namespace AscendC;
    const uint32_t M = 24, K = 512;
    std::mt19937 rng(21);
    std::normal_distribution<float> nd(0.f, 2.f);
    std::vector<float> x(M * K);
    for (auto& v : x) v = nd(rng);
    DevBuf<float> dX(x), dY(M * K), dSum(M * 8), dMax(M * 8);
    DevBuf<uint8_t> dTmp(32);
    LogSoftMaxTiling tiling{};
    tiling.srcM = M;
    tiling.srcK = K;
    TPipe pipe;
    LogSoftMax<float>(LocalTensor<float>(dY.p, dY.n), LocalTensor<float>(dSum.p, dSum.n), LocalTensor<float>(dMax.p, dMax.n),
                      LocalTensor<float>(dX.p, dX.n), LocalTensor<uint8_t>(dTmp.p, dTmp.n), tiling);
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<float> y = dY.Download(), sum = dSum.Download(), mxv = dMax.Download();
    int bad = 0;
    for (uint32_t i = 0; i < M; ++i) {
        float mx = -1e30f;
        for (uint32_t j = 0; j < K; ++j) mx = std::fmax(mx, x[i * K + j]);
        double s = 0;
        for (uint32_t j = 0; j < K; ++j) s += std::exp(static_cast<double>(x[i * K + j] - mx));
        if (mxv[i * 8] != mx || mxv[i * 8 + 7] != mx || std::fabs(sum[i * 8 + 3] - s) > 1e-5 * s) ++bad;
        for (uint32_t j = 0; j < K; ++j) {
            const double want = std::log10(std::exp(static_cast<double>(x[i * K + j] - mx)) / s);
            if (std::fabs(y[i * K + j] - want) > 1e-3 + 1e-3 * std::fabs(want)) ++bad;
        }
    }
    CHECK(bad == 0, "LogSoftMax: %d values wrong", bad);
    std::printf("LogSoftMax: ok\n");
    // SimpleSoftMax with the statistics LogSoftMax just wrote: 10^y_log must equal its result
    DevBuf<float> dY2(M * K);
    SimpleSoftMax<float>(LocalTensor<float>(dY2.p, dY2.n), LocalTensor<float>(dSum.p, dSum.n), LocalTensor<float>(dMax.p, dMax.n),
                         LocalTensor<float>(dX.p, dX.n), SoftMaxTiling{M, K});
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<float> y2 = dY2.Download();
    bad = 0;
    for (uint32_t i = 0; i < M * K; ++i)
        if (std::fabs(y2[i] - std::pow(10.0, static_cast<double>(y[i]))) > 1e-3 * y2[i] + 1e-9) ++bad;
    CHECK(bad == 0, "SimpleSoftMax: %d values wrong", bad);
    std::printf("SimpleSoftMax: ok\n");
    // SoftmaxGrad of that softmax output with grad = x, then SoftmaxGradFront: the row sums
    DevBuf<float> dG(M * K), dF(M * 8);
    SoftmaxGrad<float>(LocalTensor<float>(dG.p, dG.n), LocalTensor<float>(dX.p, dX.n), LocalTensor<float>(dY2.p, dY2.n), SoftMaxTiling{M, K});
    SoftmaxGradFront<float>(LocalTensor<float>(dF.p, dF.n), LocalTensor<float>(dX.p, dX.n), LocalTensor<float>(dY2.p, dY2.n), SoftMaxTiling{M, K});
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<float> gr = dG.Download(), fr = dF.Download();
    bad = 0;
    for (uint32_t i = 0; i < M; ++i) {
        double s = 0;
        for (uint32_t j = 0; j < K; ++j) s += static_cast<double>(x[i * K + j]) * y2[i * K + j];
        if (std::fabs(fr[i * 8] - s) > 1e-4 * (1 + std::fabs(s)) || fr[i * 8 + 7] != fr[i * 8]) ++bad;
        for (uint32_t j = 0; j < K; ++j)
            if (std::fabs(gr[i * K + j] - (x[i * K + j] - s) * y2[i * K + j]) > 1e-4) ++bad;
    }
    CHECK(bad == 0, "SoftmaxGrad: %d values wrong", bad);
    std::printf("SoftmaxGrad: ok\n");
}

// AscendAntiQuant as in the reference's antiquant example: int8 [8, 128] -> half with one (scale, offset) pair per column.
static void TestAntiQuant()
{
    using namespace AscendC;
    const uint32_t K = 8, N = 128;
    std::mt19937 rng(33);
    std::uniform_int_distribution<int> ui(-10, 10);
    std::uniform_real_distribution<float> uf(-10.f, 10.f);
    std::vector<int8_t> src(K * N);
    std::vector<half> off(N), sc(N);
    for (auto& v : src) v = static_cast<int8_t>(ui(rng));
    for (auto& v : off) v = half(uf(rng));
    for (auto& v : sc) v = half(uf(rng));
    DevBuf<int8_t> dS(src);
    DevBuf<half> dO(off), dC(sc), dD(K * N), dT(K * N);
    DevBuf<uint8_t> tmp(32);
    AscendAntiQuant<int8_t, half, false>(LocalTensor<half>(dD.p, dD.n), LocalTensor<int8_t>(dS.p, dS.n), LocalTensor<half>(dO.p, dO.n),
                                         LocalTensor<half>(dC.p, dC.n), LocalTensor<uint8_t>(tmp.p, tmp.n), K);
    AscendAntiQuant<int8_t, half, false>(LocalTensor<half>(dT.p, dT.n), LocalTensor<int8_t>(dS.p, dS.n), half(1.5f), half(0.5f),
                                         LocalTensor<uint8_t>(tmp.p, tmp.n), K);
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<half> d = dD.Download(), t = dT.Download();
    int bad = 0;
    for (uint32_t i = 0; i < K; ++i)
        for (uint32_t j = 0; j < N; ++j) {
            const half sum = half(static_cast<float>(src[i * N + j]) + static_cast<float>(off[j]));  // half add
            const half want = half(static_cast<float>(sum) * static_cast<float>(sc[j]));            // half multiply
            if (static_cast<float>(d[i * N + j]) != static_cast<float>(want)) ++bad;
            if (static_cast<float>(t[i * N + j]) != (src[i * N + j] + 1.5f) * 0.5f) ++bad;
        }
    CHECK(bad == 0, "AscendAntiQuant: %d values wrong", bad);
    std::printf("AscendAntiQuant: ok\n");
}

// Constant tiling as in the reference's matmul_constant_tiling example: the shapes are template constants
// (GetMMConfig + GetMatmulApiTiling), the object is initialised without a TCubeTiling.
static constexpr MatmulShapeParams kConstShape = {256, 384, 128, 128, 256, 64};
static constexpr MatmulApiStaticTiling GetCustomConstantCFG()
{
    using A_TYPE = AscendC::MatmulType<AscendC::TPosition::GM, CubeFormat::ND, half>;
    using C_TYPE = AscendC::MatmulType<AscendC::TPosition::GM, CubeFormat::ND, float>;
    MatmulConfig mmCFG = GetMMConfig<MatmulConfigMode::CONFIG_MDL>(kConstShape, MatmulFuncParams{false, false, false, false, 0,
                                                                                                   IterateOrder::UNDEF, ScheduleType::INNER_PRODUCT,
                                                                                                   true, false, false, false, false, false, false,
                                                                                                   /*enableRelu=*/true});
    mmCFG.enUnitFlag = true;
    auto constantCFG = AscendC::GetMatmulApiTiling<A_TYPE, A_TYPE, C_TYPE, C_TYPE>(mmCFG);
    constantCFG.depthA1 = 8;
    constantCFG.depthB1 = 8;
    return constantCFG;
}
static constexpr MatmulApiStaticTiling kConstantCfg = GetCustomConstantCFG();
static_assert(kConstantCfg.singleCoreM == 256 && kConstantCfg.N == 384 && kConstantCfg.baseK == 64 && kConstantCfg.cfg.doMultiDataLoad &&
                  kConstantCfg.cfg.enableRelu && kConstantCfg.depthA1 == 8,
              "constant tiling is evaluated at compile time");
static void TestConstantTiling()
{
    using namespace AscendC;
    const int M = 256, N = 384, K = 128;
    std::mt19937 rng(3);
    std::uniform_real_distribution<float> u(-1.f, 1.f);
    std::vector<half> a(M * K), b(K * N);
    for (auto& v : a) v = half(u(rng));
    for (auto& v : b) v = half(u(rng));
    DevBuf<half> dA(a), dB(b);
    DevBuf<float> dC(static_cast<size_t>(M) * N);
    {
        TPipe pipe;
        using A_TYPE = MatmulType<TPosition::GM, CubeFormat::ND, half>;
        using C_TYPE = MatmulType<TPosition::GM, CubeFormat::ND, float>;
        Matmul<A_TYPE, A_TYPE, C_TYPE, C_TYPE, kConstantCfg> mm;
        REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, static_cast<TCubeTiling*>(nullptr));
        GlobalTensor<half> ga, gb;
        GlobalTensor<float> gc;
        ga.SetGlobalBuffer(dA.p, a.size());
        gb.SetGlobalBuffer(dB.p, b.size());
        gc.SetGlobalBuffer(dC.p, dC.n);
        mm.SetOrgShape(M, N, K);
        mm.SetTensorA(ga);
        mm.SetTensorB(gb);
        mm.IterateAll(gc);
        mm.End();
    }
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<float> c = dC.Download();
    int bad = 0;
    for (int m = 0; m < M; m += 5)
        for (int n = 0; n < N; n += 3) {
            float acc = 0;
            for (int k = 0; k < K; ++k) acc += static_cast<float>(a[m * K + k]) * static_cast<float>(b[k * N + n]);
            acc = std::fmax(acc, 0.0f);  // enableRelu of the config
            if (std::fabs(c[static_cast<size_t>(m) * N + n] - acc) > 1e-3 + 1e-2 * std::fabs(acc)) ++bad;
        }
    CHECK(bad == 0, "constant tiling + ReLU: %d wrong", bad);
    std::printf("constant tiling (GetMMConfig / GetMatmulApiTiling): ok\n");
}

// IterateBatch, NORMAL layout: four A matrices against one shared (broadcast) B, transposed B as in the batch example.
static void TestIterateBatch()
{
    using namespace AscendC;
    const int BATCH = 4, M = 96, N = 160, K = 64;
    std::mt19937 rng(9);
    std::uniform_int_distribution<int> u(-5, 5);
    std::vector<int8_t> a(BATCH * M * K), b(N * K);
    for (auto& v : a) v = static_cast<int8_t>(u(rng));
    for (auto& v : b) v = static_cast<int8_t>(u(rng));
    DevBuf<int8_t> dA(a), dB(b);
    DevBuf<int32_t> dC(static_cast<size_t>(BATCH) * M * N);
    // tiling as in the reference's batch_matmul_bias_reuse example (BatchMatmulTiling + SetBatchInfoForNormal + SetBatchNum)
    matmul_tiling::BatchMatmulTiling api;
    api.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT8, false);
    api.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT8, true);
    api.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT32);
    api.SetOrgShape(M, N, K);
    api.SetShape(M, N, K);
    api.SetBatchInfoForNormal(BATCH, 1, M, N, K);
    api.SetBatchNum(BATCH);
    TCubeTiling tiling{};
    CHECK(api.GetTiling(tiling) == 0, "BatchMatmulTiling::GetTiling");
    CHECK(tiling.BatchNum == BATCH && tiling.ALayoutInfoB == BATCH && tiling.ALayoutInfoS == M && tiling.ALayoutInfoD == K &&
              tiling.BLayoutInfoB == 1 && tiling.BLayoutInfoS == N && tiling.CLayoutInfoB == BATCH && tiling.CLayoutInfoS1 == M &&
              tiling.CLayoutInfoS2 == N && tiling.ALayoutInfoN == 1 && tiling.CLayoutInfoG == 1,
          "batch layout fields of the tiling");
    int32_t dim = 0, mDim = 0, nDim = 0, bM = 0, bN = 0;
    api.GetCoreNum(dim, mDim, nDim, bM, bN);
    CHECK(dim == 1 && mDim == 1 && nDim == 1 && bM == 1 && bN == 1, "BatchMatmulTiling::GetCoreNum");
    CHECK(api.SetBatchNum(0) == -1 && api.SetBatchInfoForNormal(0, 1, M, N, K) == -1, "batch setters refuse non-positive extents");
    {
        TPipe pipe;
        using T8 = MatmulType<TPosition::GM, CubeFormat::ND, int8_t>;
        using T8T = MatmulType<TPosition::GM, CubeFormat::ND, int8_t, true>;
        using T32 = MatmulType<TPosition::GM, CubeFormat::ND, int32_t>;
        Matmul<T8, T8T, T32, T32> mm;
        REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
        GlobalTensor<int8_t> ga, gb;
        GlobalTensor<int32_t> gc;
        ga.SetGlobalBuffer(dA.p, a.size());
        gb.SetGlobalBuffer(dB.p, b.size());
        gc.SetGlobalBuffer(dC.p, dC.n);
        mm.SetTensorA(ga, false);
        mm.SetTensorB(gb, true);  // B stored [N, K]
        mm.IterateBatch(gc, BATCH, 1, false);
        mm.End();
    }
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<int32_t> c = dC.Download();
    int bad = 0;
    for (int i = 0; i < BATCH; ++i)
        for (int m = 0; m < M; ++m)
            for (int n = 0; n < N; ++n) {
                int32_t acc = 0;
                for (int k = 0; k < K; ++k) acc += static_cast<int32_t>(a[(i * M + m) * K + k]) * b[n * K + k];
                if (c[(static_cast<size_t>(i) * M + m) * N + n] != acc) ++bad;
            }
    CHECK(bad == 0, "IterateBatch: %d wrong", bad);
    std::printf("IterateBatch (4 x A, shared B): ok\n");
}

// Batch layouts BSNGD / SBNGD with the shapes and the loop of the reference's batch_matmul example (batch_matmul.asc:166-193,
// scripts/gen_data.py:19-66: A [B, S, N, G, D], B [B, S', N, G, D] used transposed, C [B, S, N, G, S']): every (b, n, g) is one
// [S, D] x [D, S'] product whose rows lie N * G * D elements apart.  int8 data, int32 results compared exactly.
template <LayoutMode LAYOUT>
static void TestBatchLayout(const char* name)
{
    using namespace AscendC;
    const int B = 2, SA = 32, SB = 96, N = 1, G = 3, D = 64;
    std::mt19937 rng(11);
    std::uniform_int_distribution<int> u(-6, 6);
    const bool sb = LAYOUT == LayoutMode::SBNGD;
    // element (b, s, n, g, d) of a tensor with inner extent `in`: BSNGD [B][S][N][G][in], SBNGD [S][B][N][G][in]
    auto at = [&](int b, int s, int n, int g, int d, int S, int in) -> size_t {
        return sb ? ((((static_cast<size_t>(s) * B + b) * N + n) * G + g) * in + d) : ((((static_cast<size_t>(b) * S + s) * N + n) * G + g) * in + d);
    };
    std::vector<int8_t> a(static_cast<size_t>(B) * SA * N * G * D), b(static_cast<size_t>(B) * SB * N * G * D);
    for (auto& v : a) v = static_cast<int8_t>(u(rng));
    for (auto& v : b) v = static_cast<int8_t>(u(rng));
    DevBuf<int8_t> dA(a), dB(b);
    DevBuf<int32_t> dC(static_cast<size_t>(B) * SA * N * G * SB);
    matmul_tiling::BatchMatmulTiling api;
    api.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT8, false);
    api.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT8, true);
    api.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT32);
    api.SetShape(SA, SB, D);
    api.SetOrgShape(SA, SB, D);
    api.SetALayout(B, SA, N, G, D);
    api.SetBLayout(B, SB, N, G, D);
    api.SetCLayout(B, SA, N, G, SB);
    api.SetBatchNum(N * G);
    TCubeTiling tiling{};
    CHECK(api.GetTiling(tiling) == 0, "BatchMatmulTiling::GetTiling");
    {
        TPipe pipe;
        using TA = MatmulType<TPosition::GM, CubeFormat::ND, int8_t, false, LAYOUT>;
        using TB = MatmulType<TPosition::GM, CubeFormat::ND, int8_t, true, LAYOUT>;
        using TC = MatmulType<TPosition::GM, CubeFormat::ND, int32_t, false, LAYOUT>;
        Matmul<TA, TB, TC, TC> mm;
        REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
        GlobalTensor<int8_t> ga, gb;
        GlobalTensor<int32_t> gc;
        ga.SetGlobalBuffer(dA.p, a.size());
        gb.SetGlobalBuffer(dB.p, b.size());
        gc.SetGlobalBuffer(dC.p, dC.n);
        const int batchA = N * G, batchB = N * G;
        for (int i = 0; i < B; ++i) {   // one call per b: all N * G matrices of that row block
            const size_t offA = sb ? static_cast<size_t>(i) * N * G * D : static_cast<size_t>(i) * D * SA * batchA;
            const size_t offB = sb ? static_cast<size_t>(i) * N * G * D : static_cast<size_t>(i) * D * SB * batchB;
            const size_t offC = sb ? static_cast<size_t>(i) * N * G * SB : static_cast<size_t>(i) * batchA * SB * SA;
            mm.SetTensorA(ga[offA], false);
            mm.SetTensorB(gb[offB], true);
            mm.IterateBatch(gc[offC], batchA, batchB, false);
        }
        mm.End();
    }
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<int32_t> c = dC.Download();
    int bad = 0;
    for (int bi = 0; bi < B; ++bi)
        for (int g = 0; g < G; ++g)
            for (int s1 = 0; s1 < SA; ++s1)
                for (int s2 = 0; s2 < SB; ++s2) {
                    int32_t acc = 0;
                    for (int d = 0; d < D; ++d) acc += static_cast<int32_t>(a[at(bi, s1, 0, g, d, SA, D)]) * b[at(bi, s2, 0, g, d, SB, D)];
                    if (c[at(bi, s1, 0, g, s2, SA, SB)] != acc) ++bad;
                }
    CHECK(bad == 0, "IterateBatch %s: %d wrong", name, bad);
    std::printf("IterateBatch %s: ok\n", name);
}

// IterateNBatch + GetBatchTensorC as in batch_matmul_iterate_n_batch.asc:150-190 (A [1, M, 1, b, K], B [1, N, 1, b, K], C
// [1, M, 1, b, N], BatchNum = 1 per call): three calls of one matrix each, results in the workspace.
static void TestIterateNBatch()
{
    using namespace AscendC;
    const int M = 32, N = 64, K = 64, NB = 3;
    std::mt19937 rng(12);
    std::uniform_int_distribution<int> u(-6, 6);
    std::vector<int8_t> a(static_cast<size_t>(M) * NB * K), b(static_cast<size_t>(N) * NB * K);
    for (auto& v : a) v = static_cast<int8_t>(u(rng));
    for (auto& v : b) v = static_cast<int8_t>(u(rng));
    DevBuf<int8_t> dA(a), dB(b);
    DevBuf<int32_t> dC(static_cast<size_t>(M) * NB * N);
    matmul_tiling::BatchMatmulTiling api;
    api.SetAType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT8, false);
    api.SetBType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT8, true);
    api.SetCType(matmul_tiling::TPosition::GM, matmul_tiling::CubeFormat::ND, matmul_tiling::DataType::DT_INT32);
    api.SetShape(M, N, K);
    api.SetOrgShape(M, N, K);
    api.SetALayout(1, M, 1, NB, K);
    api.SetBLayout(1, N, 1, NB, K);
    api.SetCLayout(1, M, 1, NB, N);
    api.SetBatchNum(1);
    TCubeTiling tiling{};
    CHECK(api.GetTiling(tiling) == 0, "BatchMatmulTiling::GetTiling");
    {
        TPipe pipe;
        using TA = MatmulType<TPosition::GM, CubeFormat::ND, int8_t, false, LayoutMode::BSNGD>;
        using TB = MatmulType<TPosition::GM, CubeFormat::ND, int8_t, true, LayoutMode::BSNGD>;
        using TC = MatmulType<TPosition::GM, CubeFormat::ND, int32_t, false, LayoutMode::BSNGD>;
        Matmul<TA, TB, TC, TC> mm;
        REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
        GlobalTensor<int8_t> ga, gb;
        GlobalTensor<int32_t> gc;
        ga.SetGlobalBuffer(dA.p, a.size());
        gb.SetGlobalBuffer(dB.p, b.size());
        gc.SetGlobalBuffer(dC.p, dC.n);
        mm.SetTensorA(ga, false);
        mm.SetTensorB(gb, true);
        const int nNum = tiling.ALayoutInfoB * tiling.ALayoutInfoN * tiling.ALayoutInfoG / tiling.BatchNum;
        CHECK(nNum == NB, "nNum %d", nNum);
        mm.SetWorkspace(gc);
        mm.template IterateNBatch<false>(nNum, 1, 1, false);
        for (int j = 0; j < nNum; ++j) {
            GlobalTensor<int32_t> t = mm.template GetBatchTensorC<false>(1, 1, false);
            CHECK(t.GetPhyAddr() == dC.p + static_cast<size_t>(j) * N, "GetBatchTensorC %d", j);
        }
        mm.End();
    }
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<int32_t> c = dC.Download();
    int bad = 0;
    for (int g = 0; g < NB; ++g)
        for (int m = 0; m < M; ++m)
            for (int n = 0; n < N; ++n) {
                int32_t acc = 0;
                for (int k = 0; k < K; ++k) acc += static_cast<int32_t>(a[(static_cast<size_t>(m) * NB + g) * K + k]) * b[(static_cast<size_t>(n) * NB + g) * K + k];
                if (c[(static_cast<size_t>(m) * NB + g) * N + n] != acc) ++bad;
            }
    CHECK(bad == 0, "IterateNBatch: %d wrong", bad);
    std::printf("IterateNBatch (BSNGD, three calls of one matrix): ok\n");
}

// Iterate / GetTensorC over base blocks: in place (each block at its position in C) and block-sequential (each block a compact
// matrix in its own slot, as the grouped example collects them: quant_group_matmul_custom.asc:320-328), both iteration orders;
// then the column-major and fractal output formats of IterateAll.
static void TestBaseBlocksAndOutputFormats()
{
    using namespace AscendC;
    const int M = 200, N = 328, K = 128, BM = 96, BN = 128;
    std::mt19937 rng(13);
    std::uniform_int_distribution<int> u(-7, 7);
    std::vector<int8_t> a(static_cast<size_t>(M) * K), b(static_cast<size_t>(N) * K);
    for (auto& v : a) v = static_cast<int8_t>(u(rng));
    for (auto& v : b) v = static_cast<int8_t>(u(rng));
    std::vector<int32_t> ref(static_cast<size_t>(M) * N);
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            int32_t acc = 0;
            for (int k = 0; k < K; ++k) acc += static_cast<int32_t>(a[static_cast<size_t>(m) * K + k]) * b[static_cast<size_t>(n) * K + k];
            ref[static_cast<size_t>(m) * N + n] = acc;
        }
    DevBuf<int8_t> dA(a), dB(b);
    TCubeTiling tiling{};
    tiling.usedCoreNum = 1;
    tiling.M = tiling.singleCoreM = M;
    tiling.N = tiling.singleCoreN = N;
    tiling.Ka = tiling.Kb = tiling.singleCoreK = K;
    tiling.baseM = BM;
    tiling.baseN = BN;
    tiling.baseK = 64;
    using T8 = MatmulType<TPosition::GM, CubeFormat::ND, int8_t>;
    using T8T = MatmulType<TPosition::GM, CubeFormat::ND, int8_t, true>;
    const int mIter = (M + BM - 1) / BM, nIter = (N + BN - 1) / BN;
    for (int order = 0; order < 2; ++order) {
        tiling.iterateOrder = order;
        DevBuf<int32_t> dC(static_cast<size_t>(M) * N), dSlots(static_cast<size_t>(mIter) * nIter * BM * BN);
        {
            TPipe pipe;
            using T32 = MatmulType<TPosition::GM, CubeFormat::ND, int32_t>;
            Matmul<T8, T8T, T32, T32> mm;
            REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
            GlobalTensor<int8_t> ga, gb;
            GlobalTensor<int32_t> gc, gs;
            ga.SetGlobalBuffer(dA.p, a.size());
            gb.SetGlobalBuffer(dB.p, b.size());
            gc.SetGlobalBuffer(dC.p, dC.n);
            gs.SetGlobalBuffer(dSlots.p, dSlots.n);
            mm.SetTensorA(ga, false);
            mm.SetTensorB(gb, true);
            int blocks = 0;
            while (mm.Iterate()) {
                mm.GetTensorC(gc);                                                      // at its place in [M, N]
                mm.GetTensorC(gs[static_cast<size_t>(blocks) * BM * BN], 0, true);      // compact, in slot `blocks`
                ++blocks;
            }
            CHECK(blocks == mIter * nIter, "Iterate returned %d blocks", blocks);
            mm.End();
        }
        CHECK(GetLastError() == 0, "operator error %d", GetLastError());
        const std::vector<int32_t> c = dC.Download(), slots = dSlots.Download();
        int bad = 0;
        for (size_t i = 0; i < c.size(); ++i) bad += c[i] != ref[i];
        for (int blk = 0; blk < mIter * nIter; ++blk) {
            const int row = order == 1 ? blk / nIter : blk % mIter, col = order == 1 ? blk % nIter : blk / mIter;
            const int h = std::min(BM, M - row * BM), w = std::min(BN, N - col * BN);
            for (int i = 0; i < h; ++i)
                for (int j = 0; j < w; ++j)
                    bad += slots[static_cast<size_t>(blk) * BM * BN + static_cast<size_t>(i) * w + j] != ref[static_cast<size_t>(row * BM + i) * N + col * BN + j];
        }
        CHECK(bad == 0, "base blocks, iterateOrder %d: %d wrong", order, bad);
    }
    // output formats
    {
        DevBuf<int32_t> dCm(static_cast<size_t>(M) * N), dNz(static_cast<size_t>((N + 15) / 16) * M * 16);
        TPipe pipe;
        using TCM = MatmulType<TPosition::GM, CubeFormat::COLUMN_MAJOR, int32_t>;
        using TNZ = MatmulType<TPosition::GM, CubeFormat::NZ, int32_t>;
        GlobalTensor<int8_t> ga, gb;
        ga.SetGlobalBuffer(dA.p, a.size());
        gb.SetGlobalBuffer(dB.p, b.size());
        {
            Matmul<T8, T8T, TCM, TCM> mm;
            REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
            GlobalTensor<int32_t> gc;
            gc.SetGlobalBuffer(dCm.p, dCm.n);
            mm.SetTensorA(ga, false);
            mm.SetTensorB(gb, true);
            mm.IterateAll(gc);
            mm.End();
        }
        {
            Matmul<T8, T8T, TNZ, TNZ> mm;
            REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
            GlobalTensor<int32_t> gc;
            gc.SetGlobalBuffer(dNz.p, dNz.n);
            mm.SetTensorA(ga, false);
            mm.SetTensorB(gb, true);
            while (mm.Iterate()) mm.GetTensorC(gc);   // block by block into the fractal matrix
            mm.End();
        }
        CHECK(GetLastError() == 0, "operator error %d", GetLastError());
        const std::vector<int32_t> cm = dCm.Download(), nz = dNz.Download();
        int bad = 0;
        for (int m = 0; m < M; ++m)
            for (int n = 0; n < N; ++n) {
                bad += cm[static_cast<size_t>(n) * M + m] != ref[static_cast<size_t>(m) * N + n];
                bad += nz[(static_cast<size_t>(n / 16) * M + m) * 16 + n % 16] != ref[static_cast<size_t>(m) * N + n];
            }
        CHECK(bad == 0, "COLUMN_MAJOR / NZ outputs: %d wrong", bad);
    }
    std::printf("Iterate / GetTensorC base blocks (in place, sequential), COLUMN_MAJOR and NZ outputs: ok\n");
}

// MX Matmul through the mirror with the reference's layouts of an untransposed B ([K, N] fp4, scaleB [K/64][N][2]) against the
// K-major form of the same operands: identical bits.
static void TestMxLayouts()
{
    using namespace AscendC;
    const int M = 128, N = 192, K = 256, SK = K / 32;
    std::mt19937 rng(14);
    std::uniform_int_distribution<int> code(0, 15), sc(124, 130);
    std::vector<uint8_t> ca(static_cast<size_t>(M) * K), cb(static_cast<size_t>(K) * N);   // fp4 codes, A [M, K], B [K, N]
    for (auto& v : ca) v = static_cast<uint8_t>(code(rng));
    for (auto& v : cb) v = static_cast<uint8_t>(code(rng));
    std::vector<uint8_t> sa(static_cast<size_t>(M) * SK), sbT(static_cast<size_t>(N) * SK);     // scaleA [M, SK], scaleB^T [N, SK]
    for (auto& v : sa) v = static_cast<uint8_t>(sc(rng));
    for (auto& v : sbT) v = static_cast<uint8_t>(sc(rng));
    std::vector<fp4x2_e2m1_t> a(static_cast<size_t>(M) * K / 2), bNd(static_cast<size_t>(K) * N / 2), bKm(static_cast<size_t>(N) * K / 2);
    for (int m = 0; m < M; ++m)
        for (int k = 0; k < K; k += 2) a[(static_cast<size_t>(m) * K + k) / 2].bits = static_cast<uint8_t>(ca[static_cast<size_t>(m) * K + k] | (ca[static_cast<size_t>(m) * K + k + 1] << 4));
    for (int k = 0; k < K; ++k)
        for (int n = 0; n < N; n += 2) bNd[(static_cast<size_t>(k) * N + n) / 2].bits = static_cast<uint8_t>(cb[static_cast<size_t>(k) * N + n] | (cb[static_cast<size_t>(k) * N + n + 1] << 4));
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; k += 2) bKm[(static_cast<size_t>(n) * K + k) / 2].bits = static_cast<uint8_t>(cb[static_cast<size_t>(k) * N + n] | (cb[static_cast<size_t>(k + 1) * N + n] << 4));
    std::vector<fp8_e8m0_t> vsa(sa.size()), vsbT(sbT.size()), vsbP(sbT.size());
    for (size_t i = 0; i < sa.size(); ++i) vsa[i].bits = sa[i];
    for (size_t i = 0; i < sbT.size(); ++i) vsbT[i].bits = sbT[i];
    for (int p = 0; p < SK / 2; ++p)
        for (int n = 0; n < N; ++n)
            for (int j = 0; j < 2; ++j) vsbP[(static_cast<size_t>(p) * N + n) * 2 + j].bits = sbT[static_cast<size_t>(n) * SK + 2 * p + j];
    DevBuf<fp4x2_e2m1_t> dA(a), dBnd(bNd), dBkm(bKm);
    DevBuf<fp8_e8m0_t> dSa(vsa), dSbT(vsbT), dSbP(vsbP);
    DevBuf<float> dC1(static_cast<size_t>(M) * N), dC2(static_cast<size_t>(M) * N);
    TCubeTiling tiling{};
    tiling.usedCoreNum = 1;
    tiling.M = tiling.singleCoreM = M;
    tiling.N = tiling.singleCoreN = N;
    tiling.Ka = tiling.Kb = tiling.singleCoreK = K;
    tiling.baseM = 128;
    tiling.baseN = 256;
    tiling.baseK = 256;
    {
        TPipe pipe;
        using TA = MatmulTypeWithScale<TPosition::GM, TPosition::GM, CubeFormat::ND, fp4x2_e2m1_t, false>;
        using TBT = MatmulTypeWithScale<TPosition::GM, TPosition::GM, CubeFormat::ND, fp4x2_e2m1_t, true>;
        using TBN = MatmulTypeWithScale<TPosition::GM, TPosition::GM, CubeFormat::ND, fp4x2_e2m1_t, false>;
        using TC = MatmulType<TPosition::GM, CubeFormat::ND, float>;
        GlobalTensor<fp4x2_e2m1_t> ga, gbn, gbk;
        GlobalTensor<fp8_e8m0_t> gsa, gsbt, gsbp;
        GlobalTensor<float> gc1, gc2;
        ga.SetGlobalBuffer(dA.p, a.size());
        gbn.SetGlobalBuffer(dBnd.p, bNd.size());
        gbk.SetGlobalBuffer(dBkm.p, bKm.size());
        gsa.SetGlobalBuffer(dSa.p, vsa.size());
        gsbt.SetGlobalBuffer(dSbT.p, vsbT.size());
        gsbp.SetGlobalBuffer(dSbP.p, vsbP.size());
        gc1.SetGlobalBuffer(dC1.p, dC1.n);
        gc2.SetGlobalBuffer(dC2.p, dC2.n);
        {
            Matmul<TA, TBT, TC, TC, CFG_MDL, MatmulCallBackFunc<>, MatmulWithScalePolicy> mm;
            REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
            mm.SetTensorA(ga, false);
            mm.SetTensorB(gbk, true);
            mm.SetTensorScaleA(gsa, false);
            mm.SetTensorScaleB(gsbt, true);
            mm.IterateAll(gc1);
            mm.End();
        }
        {
            Matmul<TA, TBN, TC, TC, CFG_MDL, MatmulCallBackFunc<>, MatmulWithScalePolicy> mm;
            REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
            mm.SetTensorA(ga, false);
            mm.SetTensorB(gbn, false);          // [K, N]
            mm.SetTensorScaleA(gsa, false);
            mm.SetTensorScaleB(gsbp, false);    // [K/64][N][2]
            mm.IterateAll(gc2);
            mm.IterateAll(gc2);                 // the transposed copy of B is kept between calls
            mm.End();
        }
    }
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<float> c1 = dC1.Download(), c2 = dC2.Download();
    int bad = 0, nonzero = 0;
    for (size_t i = 0; i < c1.size(); ++i) {
        bad += std::memcmp(&c1[i], &c2[i], sizeof(float)) != 0;
        nonzero += c1[i] != 0.0f;
    }
    CHECK(bad == 0 && nonzero > 0, "MX layouts: %d differ, %d non-zero", bad, nonzero);
    std::printf("MX Matmul, [K, N] B with pair-ordered scaleB == K-major form: ok\n");
}

// MX Matmul with fp8 e5m2 operands as in the reference's matmul_mx example (A [M, K], B [K, N] not transposed, scaleB in the pair
// order): small integers and power-of-two scales, so the expected fp32 result is exact.
static void TestMxFp8()
{
    using namespace AscendC;
    const int M = 64, N = 128, K = 128, SK = K / 32;
    static const uint8_t kCode[5] = {0x00, 0x3C, 0x40, 0x42, 0x44};   // e5m2 encodings of 0, 1, 2, 3, 4
    std::mt19937 rng(15);
    std::uniform_int_distribution<int> u(-4, 4), sc(126, 129);
    std::vector<int> va(static_cast<size_t>(M) * K), vb(static_cast<size_t>(K) * N);
    for (auto& v : va) v = u(rng);
    for (auto& v : vb) v = u(rng);
    std::vector<fp8_e5m2_t> a(va.size()), b(vb.size());
    for (size_t i = 0; i < va.size(); ++i) a[i].bits = static_cast<uint8_t>(kCode[std::abs(va[i])] | (va[i] < 0 ? 0x80 : 0));
    for (size_t i = 0; i < vb.size(); ++i) b[i].bits = static_cast<uint8_t>(kCode[std::abs(vb[i])] | (vb[i] < 0 ? 0x80 : 0));
    std::vector<uint8_t> sa(static_cast<size_t>(M) * SK), sb(static_cast<size_t>(SK) * N);   // scaleA [M, SK], scaleB [SK, N]
    for (auto& v : sa) v = static_cast<uint8_t>(sc(rng));
    for (auto& v : sb) v = static_cast<uint8_t>(sc(rng));
    std::vector<fp8_e8m0_t> vsa(sa.size()), vsbP(sb.size());
    for (size_t i = 0; i < sa.size(); ++i) vsa[i].bits = sa[i];
    for (int p = 0; p < SK / 2; ++p)
        for (int n = 0; n < N; ++n)
            for (int j = 0; j < 2; ++j) vsbP[(static_cast<size_t>(p) * N + n) * 2 + j].bits = sb[static_cast<size_t>(2 * p + j) * N + n];
    DevBuf<fp8_e5m2_t> dA(a), dB(b);
    DevBuf<fp8_e8m0_t> dSa(vsa), dSb(vsbP);
    DevBuf<float> dC(static_cast<size_t>(M) * N);
    TCubeTiling tiling{};
    tiling.usedCoreNum = 1;
    tiling.M = tiling.singleCoreM = M;
    tiling.N = tiling.singleCoreN = N;
    tiling.Ka = tiling.Kb = tiling.singleCoreK = K;
    tiling.baseM = 64;
    tiling.baseN = 128;
    tiling.baseK = 128;
    {
        TPipe pipe;
        using TA = MatmulTypeWithScale<TPosition::GM, TPosition::GM, CubeFormat::ND, fp8_e5m2_t, false>;
        using TB = MatmulTypeWithScale<TPosition::GM, TPosition::GM, CubeFormat::ND, fp8_e5m2_t, false>;
        using TC = MatmulType<TPosition::GM, CubeFormat::ND, float>;
        Matmul<TA, TB, TC, TC, CFG_MDL, MatmulCallBackFunc<>, MatmulWithScalePolicy> mm;
        REGIST_MATMUL_OBJ(&pipe, GetSysWorkSpacePtr(), mm, &tiling);
        GlobalTensor<fp8_e5m2_t> ga, gb;
        GlobalTensor<fp8_e8m0_t> gsa, gsb;
        GlobalTensor<float> gc;
        ga.SetGlobalBuffer(dA.p, a.size());
        gb.SetGlobalBuffer(dB.p, b.size());
        gsa.SetGlobalBuffer(dSa.p, vsa.size());
        gsb.SetGlobalBuffer(dSb.p, vsbP.size());
        gc.SetGlobalBuffer(dC.p, dC.n);
        mm.SetTensorA(ga, false);
        mm.SetTensorB(gb, false);
        mm.SetTensorScaleA(gsa, false);
        mm.SetTensorScaleB(gsb, false);
        mm.IterateAll(gc);
        mm.End();
    }
    CHECK(GetLastError() == 0, "operator error %d", GetLastError());
    const std::vector<float> c = dC.Download();
    int bad = 0;
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            double acc = 0.0;
            for (int k = 0; k < K; ++k)
                acc += std::ldexp(static_cast<double>(va[static_cast<size_t>(m) * K + k]), sa[static_cast<size_t>(m) * SK + k / 32] - 127) *
                       std::ldexp(static_cast<double>(vb[static_cast<size_t>(k) * N + n]), sb[static_cast<size_t>(k / 32) * N + n] - 127);
            bad += c[static_cast<size_t>(m) * N + n] != static_cast<float>(acc);
        }
    CHECK(bad == 0, "MX fp8 Matmul: %d wrong", bad);
    std::printf("MX Matmul fp8 e5m2, [K, N] B, pair-ordered scaleB: ok\n");
}

static void TestErrorLatch()
{
    AscendC::ClearLastError();
    AscendC::LocalTensor<half> none;
    AscendC::LocalTensor<float> nonef;
    ::SoftMaxTiling tiling{};
    tiling.srcM = 4;
    tiling.srcK = 64;
    AscendC::SoftMax<half>(none, nonef, nonef, none, tiling);  // null tensors: latched, no crash, no launch
    CHECK(AscendC::GetLastError() == ASCB200_EINVAL, "expected EINVAL, got %d", AscendC::GetLastError());
    AscendC::ClearLastError();
}

int main()
{
    if (ascb200_init(0) != 0) {
        std::printf("no B200 available\n");
        return 2;
    }
    TestMatmulFp16();
    TestMatmulQuant();
    TestSoftmaxQuantDequant();
    TestMatmulNzAtomicAlign();
    TestQuantPolicies();
    TestSoftmaxFlashV2();
    TestLogSoftMax();
    TestAntiQuant();
    TestConstantTiling();
    TestIterateBatch();
    TestBatchLayout<LayoutMode::BSNGD>("BSNGD");
    TestBatchLayout<LayoutMode::SBNGD>("SBNGD");
    TestIterateNBatch();
    TestBaseBlocksAndOutputFormats();
    TestMxLayouts();
    TestMxFp8();
    TestErrorLatch();
    std::printf(g_fail ? "%d checks failed\n" : "hostapi ok\n", g_fail);
    return g_fail ? 1 : 0;
}
