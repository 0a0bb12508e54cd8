// MatmulConfig, its template presets and the constant-tiling entry points of the reference
// (include/adv_api/matmul/matmul_config.h:38-330, include/adv_api/matmul/tiling.h:36-600,
// include/adv_api/matmul/constant_tiling.h:37-92), for host code that was written against them.
//
// On Ascend these settings choose a scheduler template and its buffer choreography (Norm / MDL / basic block / IBShare,
// L1 depths, preloads ...).  The B200 kernels schedule themselves, so only the settings that can change results are
// consumed (enableRelu, enableSetBias, enableQuantVector, isBiasBatch and the shapes of a constant tiling); everything else
// is carried so that existing code compiles and round-trips unchanged.
#pragma once
#include <cstdint>

enum class LayoutMode { NONE = 0, BSNGD, SBNGD, BNGS1S2, NORMAL };
enum class BatchMode { NONE = 0, BATCH_LESS_THAN_L1, BATCH_LARGE_THAN_L1, SINGLE_LARGE_THAN_L1 };
enum BatchOutMode { SINGLE_BATCH = 0, MULTI_BATCH, DYNAMIC };
enum class IterateOrder { ORDER_M = 0, ORDER_N, UNDEF };
enum class ScheduleType { INNER_PRODUCT = 0, OUTER_PRODUCT };
enum IterateMode : uint8_t {
    ITERATE_MODE_NORMAL = 0b00000001,
    ITERATE_MODE_ALL = 0b00000010,
    ITERATE_MODE_BATCH = 0b00000100,
    ITERATE_MODE_N_BATCH = 0b00001000,
    ITERATE_MODE_DEFAULT = 0b11111111,
};
enum class DecompressionMode { DECOMP_NONE = 0 };
enum PreallocationMode : uint8_t { PREALLOCATION_ENABLE_NONE = 0, PREALLOCATION_ENABLE_ALL = 0b00111111 };
enum class MatmulConfigMode { CONFIG_NORM, CONFIG_MDL, CONFIG_SPECIALMDL, CONFIG_IBSHARE };

struct MatmulConfig {
    bool doNorm = true;
    bool doBasicBlock = false;
    bool doMultiDataLoad = false;
    uint32_t basicM = 0, basicN = 0, basicK = 0;
    bool intrinsicsCheck = false;
    bool isNBatch = false;
    bool enVecND2NZ = false;
    bool doSpecialBasicBlock = false;
    uint32_t doMTE2Preload = 0;
    uint32_t singleCoreM = 0, singleCoreN = 0, singleCoreK = 0;
    uint32_t stepM = 0, stepN = 0;
    uint32_t baseMN = 0, singleCoreMN = 0;
    bool enUnitFlag = true;
    bool isPerTensor = false;
    bool hasAntiQuantOffset = false;
    bool doIBShareNorm = false;
    bool doSpecialMDL = false;
    bool enableInit = true;
    BatchMode batchMode = BatchMode::NONE;
    bool enableEnd = true;
    bool enableGetTensorC = true;
    bool enableSetOrgShape = true;
    bool enableSetBias = true;        // consumed: SetBias has an effect only when true
    bool enableSetTail = true;
    bool enableQuantVector = true;
    bool enableSetDefineData = true;
    uint8_t iterateMode = ITERATE_MODE_DEFAULT;
    bool enableReuse = true;
    bool enableUBReuse = false;
    bool enableL1CacheUB = false;
    bool intraBlockPartSum = false;
    IterateOrder iterateOrder = IterateOrder::UNDEF;
    ScheduleType scheduleType = ScheduleType::INNER_PRODUCT;
    bool enableDoubleCache = false;
    bool isBiasBatch = true;
    bool enableStaticPadZeros = false;
    bool isPartialOutput = false;
    bool enableMixDualMaster = false;
    bool isA2B2Shared = false;
    bool isEnableChannelSplit = false;
    bool enableKdimReorderLoad = false;
    bool isCO1Shared = false;
    uint32_t sharedCO1BufferSize = 64 * 1024;
    BatchOutMode bmmOutMode = BatchOutMode::SINGLE_BATCH;
    bool enableL1BankConflictOptimise = false;
    bool enableRelu = false;          // consumed: ReLU in the output stage
    DecompressionMode decompMode = DecompressionMode::DECOMP_NONE;
    PreallocationMode preAllocationMode = PreallocationMode::PREALLOCATION_ENABLE_ALL;
};

struct MatmulShapeParams {
    uint32_t singleCoreM, singleCoreN, singleCoreK;
    uint32_t basicM, basicN, basicK;
};
struct MatmulQuantParams {
    bool isPerTensor;
    bool hasAntiQuantOffset;
};
struct MatmulBatchParams {
    bool isNBatch;
    BatchMode batchMode;
    bool isBiasBatch = true;
    BatchOutMode bmmOutMode = BatchOutMode::SINGLE_BATCH;
};
struct MatmulFuncParams {
    bool intrinsicsCheck;
    bool enVecND2NZ;
    bool enableDoubleCache;
    bool enableL1CacheUB;
    uint32_t doMTE2Preload;
    IterateOrder iterateOrder;
    ScheduleType scheduleType;
    bool enableReuse = true;
    bool enableUBReuse = false;
    bool isPartialOutput = false;
    bool isA2B2Shared = false;
    bool isEnableChannelSplit = false;
    bool enableKdimReorderLoad = false;
    bool enableL1BankConflictOptimise = false;
    bool enableRelu = false;
    DecompressionMode decompMode = DecompressionMode::DECOMP_NONE;
};
struct MatmulBiasParams {
    bool enableSetBias = true;
};

// ---- template presets (include/adv_api/matmul/tiling.h:36-492): same parameter lists, same defaults -----------------------
constexpr MatmulConfig GetNormalConfig(const bool intrinsicsLimit = false, const bool batchLoop = false, const bool isVecND2NZ = false,
                                       const BatchMode bmmMode = BatchMode::BATCH_LESS_THAN_L1, const bool isMsgReuse = true,
                                       const IterateOrder iterateOrder = IterateOrder::UNDEF,
                                       const ScheduleType scheduleType = ScheduleType::INNER_PRODUCT, const bool enUnitFlag = true,
                                       const bool enableMixDualMaster = false, const BatchOutMode bmmOutMode = BatchOutMode::SINGLE_BATCH,
                                       const PreallocationMode preAllocationMode = PreallocationMode::PREALLOCATION_ENABLE_ALL)
{
    MatmulConfig c;
    c.doNorm = true;
    c.intrinsicsCheck = intrinsicsLimit;
    c.isNBatch = batchLoop;
    c.enVecND2NZ = isVecND2NZ;
    c.batchMode = bmmMode;
    c.enableReuse = isMsgReuse;
    c.iterateOrder = iterateOrder;
    c.scheduleType = scheduleType;
    c.enUnitFlag = enUnitFlag;
    c.enableMixDualMaster = enableMixDualMaster;
    c.bmmOutMode = bmmOutMode;
    c.preAllocationMode = preAllocationMode;
    return c;
}
constexpr MatmulConfig GetMDLConfig(const bool intrinsicsLimit = false, const bool batchLoop = false, const uint32_t doMTE2Preload = 0,
                                    const bool isVecND2NZ = false, bool isPerTensor = false, bool hasAntiQuantOffset = false,
                                    const bool enUnitFlag = false, const bool isMsgReuse = true, const bool enableUBReuse = true,
                                    const bool enableL1CacheUB = false, const bool enableMixDualMaster = false,
                                    const bool enableKdimReorderLoad = false, const bool enableL1BankConflictOptimise = false,
                                    const PreallocationMode preAllocationMode = PreallocationMode::PREALLOCATION_ENABLE_ALL)
{
    MatmulConfig c;
    c.doNorm = false;
    c.doMultiDataLoad = true;
    c.intrinsicsCheck = intrinsicsLimit;
    c.isNBatch = batchLoop;
    c.doMTE2Preload = doMTE2Preload;
    c.enVecND2NZ = isVecND2NZ;
    c.isPerTensor = isPerTensor;
    c.hasAntiQuantOffset = hasAntiQuantOffset;
    c.enUnitFlag = enUnitFlag;
    c.enableReuse = isMsgReuse;
    c.enableUBReuse = enableUBReuse;
    c.enableL1CacheUB = enableL1CacheUB;
    c.enableMixDualMaster = enableMixDualMaster;
    c.enableKdimReorderLoad = enableKdimReorderLoad;
    c.enableL1BankConflictOptimise = enableL1BankConflictOptimise;
    c.preAllocationMode = preAllocationMode;
    return c;
}
constexpr MatmulConfig GetSpecialMDLConfig(const bool intrinsicsLimit = false, const bool batchLoop = false, const uint32_t doMTE2Preload = 0,
                                           const bool isVecND2NZ = false, bool isPerTensor = false, bool hasAntiQuantOffset = false,
                                           const PreallocationMode preAllocationMode = PreallocationMode::PREALLOCATION_ENABLE_ALL)
{
    MatmulConfig c = GetMDLConfig(intrinsicsLimit, batchLoop, doMTE2Preload, isVecND2NZ, isPerTensor, hasAntiQuantOffset);
    c.doMultiDataLoad = false;
    c.doSpecialMDL = true;
    c.preAllocationMode = preAllocationMode;
    return c;
}
constexpr MatmulConfig GetBasicConfig(const uint32_t basicM, const uint32_t basicN, const uint32_t basicK, const bool intrinsicsLimit = false,
                                      const bool batchLoop = false, const BatchMode bmmMode = BatchMode::BATCH_LESS_THAN_L1,
                                      const PreallocationMode preAllocationMode = PreallocationMode::PREALLOCATION_ENABLE_ALL)
{
    MatmulConfig c;
    c.doNorm = false;
    c.doBasicBlock = true;
    c.basicM = basicM;
    c.basicN = basicN;
    c.basicK = basicK;
    c.intrinsicsCheck = intrinsicsLimit;
    c.isNBatch = batchLoop;
    c.batchMode = bmmMode;
    c.preAllocationMode = preAllocationMode;
    return c;
}
constexpr MatmulConfig GetSpecialBasicConfig(const uint32_t basicM, const uint32_t basicN, const uint32_t basicK, const uint32_t singleCoreM,
                                             const uint32_t singleCoreN, const uint32_t singleCoreK, const uint32_t stepM, const uint32_t stepN,
                                             const bool intrinsicsLimit = false, const bool batchLoop = false,
                                             const BatchMode bmmMode = BatchMode::BATCH_LESS_THAN_L1,
                                             const PreallocationMode preAllocationMode = PreallocationMode::PREALLOCATION_ENABLE_ALL)
{
    MatmulConfig c = GetBasicConfig(basicM, basicN, basicK, intrinsicsLimit, batchLoop, bmmMode, preAllocationMode);
    c.doBasicBlock = false;
    c.doSpecialBasicBlock = true;
    c.singleCoreM = singleCoreM;
    c.singleCoreN = singleCoreN;
    c.singleCoreK = singleCoreK;
    c.stepM = stepM;
    c.stepN = stepN;
    c.baseMN = basicM * basicN;
    c.singleCoreMN = singleCoreM * singleCoreN;
    return c;
}
constexpr MatmulConfig GetIBShareNormConfig(const bool intrinsicsLimit = false, const bool batchLoop = false, const bool isVecND2NZ = false,
                                            const BatchMode bmmMode = BatchMode::BATCH_LESS_THAN_L1, const bool isDoubleCache = false,
                                            const bool enUnitFlag = true,
                                            const PreallocationMode preAllocationMode = PreallocationMode::PREALLOCATION_ENABLE_ALL)
{
    MatmulConfig c;
    c.doNorm = false;
    c.doIBShareNorm = true;
    c.intrinsicsCheck = intrinsicsLimit;
    c.isNBatch = batchLoop;
    c.enVecND2NZ = isVecND2NZ;
    c.batchMode = bmmMode;
    c.enableDoubleCache = isDoubleCache;
    c.enUnitFlag = enUnitFlag;
    c.preAllocationMode = preAllocationMode;
    return c;
}
constexpr MatmulConfig CFG_NORM = GetNormalConfig();
constexpr MatmulConfig CFG_MDL = GetMDLConfig();
constexpr MatmulConfig MM_CFG_BB = GetBasicConfig(128, 128, 128);
constexpr MatmulConfig CFG_IBSHARE_NORM = GetIBShareNormConfig();

// GetMMConfig<mode>(params...): a preset with any of the parameter structs applied, in any order (tiling.h:495-516).
namespace matmul_config_detail {
constexpr void Apply(MatmulConfig& c, const MatmulShapeParams& p)
{
    c.singleCoreM = p.singleCoreM;
    c.singleCoreN = p.singleCoreN;
    c.singleCoreK = p.singleCoreK;
    c.basicM = p.basicM;
    c.basicN = p.basicN;
    c.basicK = p.basicK;
}
constexpr void Apply(MatmulConfig& c, const MatmulQuantParams& p)
{
    c.isPerTensor = p.isPerTensor;
    c.hasAntiQuantOffset = p.hasAntiQuantOffset;
}
constexpr void Apply(MatmulConfig& c, const MatmulBatchParams& p)
{
    c.isNBatch = p.isNBatch;
    c.batchMode = p.batchMode;
    c.isBiasBatch = p.isBiasBatch;
    c.bmmOutMode = p.bmmOutMode;
}
constexpr void Apply(MatmulConfig& c, const MatmulFuncParams& p)
{
    c.intrinsicsCheck = p.intrinsicsCheck;
    c.enVecND2NZ = p.enVecND2NZ;
    c.enableDoubleCache = p.enableDoubleCache;
    c.enableL1CacheUB = p.enableL1CacheUB;
    c.doMTE2Preload = p.doMTE2Preload;
    c.iterateOrder = p.iterateOrder;
    c.scheduleType = p.scheduleType;
    c.enableReuse = p.enableReuse;
    c.enableUBReuse = p.enableUBReuse;
    c.isPartialOutput = p.isPartialOutput;
    c.isA2B2Shared = p.isA2B2Shared;
    c.isEnableChannelSplit = p.isEnableChannelSplit;
    c.enableKdimReorderLoad = p.enableKdimReorderLoad;
    c.enableL1BankConflictOptimise = p.enableL1BankConflictOptimise;
    c.enableRelu = p.enableRelu;
    c.decompMode = p.decompMode;
}
constexpr void Apply(MatmulConfig& c, const MatmulBiasParams& p) { c.enableSetBias = p.enableSetBias; }
constexpr void ApplyAll(MatmulConfig&) {}
template <typename First, typename... Rest>
constexpr void ApplyAll(MatmulConfig& c, const First& first, const Rest&... rest)
{
    Apply(c, first);
    ApplyAll(c, rest...);
}
}  // namespace matmul_config_detail

template <MatmulConfigMode configMode, typename... ArgTypes>
constexpr MatmulConfig GetMMConfig(const ArgTypes&... args)
{
    MatmulConfig c = CFG_NORM;
    if (configMode == MatmulConfigMode::CONFIG_MDL) c = CFG_MDL;
    else if (configMode == MatmulConfigMode::CONFIG_SPECIALMDL) c = GetSpecialMDLConfig();
    else if (configMode == MatmulConfigMode::CONFIG_IBSHARE) c = CFG_IBSHARE_NORM;
    matmul_config_detail::ApplyAll(c, args...);
    return c;
}

// Constant tiling (include/adv_api/matmul/tiling.h:518-600): the TCubeTiling fields as compile-time constants plus the config.
struct MatmulApiStaticTiling {
    int32_t usedCoreNum = -1, M = -1, N = -1, Ka = -1, Kb = -1, singleCoreM = -1, singleCoreN = -1, singleCoreK = -1, baseM = -1, baseN = -1,
            baseK = -1, depthA1 = -1, depthB1 = -1, stepM = -1, stepN = -1, isBias = -1, transLength = -1, iterateOrder = -1, shareMode = -1,
            shareL1Size = -1, shareL0CSize = -1, shareUbSize = -1, stepKa = -1, stepKb = -1, depthAL1CacheUB = -1, depthBL1CacheUB = -1,
            dbL0A = -1, dbL0B = -1, dbL0C = -1, ALayoutInfoB = -1, ALayoutInfoS = -1, ALayoutInfoN = -1, ALayoutInfoG = -1, ALayoutInfoD = -1,
            BLayoutInfoB = -1, BLayoutInfoS = -1, BLayoutInfoN = -1, BLayoutInfoG = -1, BLayoutInfoD = -1, CLayoutInfoB = -1,
            CLayoutInfoS1 = -1, CLayoutInfoN = -1, CLayoutInfoG = -1, CLayoutInfoS2 = -1, BatchNum = -1, mxTypePara = -1;
    MatmulConfig cfg = CFG_NORM;
};

namespace AscendC {
// the reference declares the config symbols at global scope; qualified uses keep working
using ::CFG_IBSHARE_NORM;
using ::CFG_MDL;
using ::CFG_NORM;
using ::MM_CFG_BB;
using ::MatmulApiStaticTiling;
using ::MatmulConfig;

// GetMatmulApiTiling<A_TYPE, B_TYPE, C_TYPE, BIAS_TYPE>(mmCFG, l1Size) (constant_tiling.h:37-90): the shape fields follow the
// config exactly like the reference; the L1 / L0 choreography fields (depths, steps, double-buffer switches) are set to the
// smallest valid values, since the B200 kernels do not read them.
template <class A_TYPE, class B_TYPE, class C_TYPE, class BIAS_TYPE>
constexpr MatmulApiStaticTiling GetMatmulApiTiling(const MatmulConfig& mmCFG, int32_t /*l1Size*/ = 512 * 1024)
{
    MatmulApiStaticTiling t;
    t.cfg = mmCFG;
    if (mmCFG.singleCoreM == 0 || mmCFG.singleCoreN == 0 || mmCFG.singleCoreK == 0) {
        if (mmCFG.basicM != 0 && mmCFG.basicN != 0 && mmCFG.basicK != 0) {
            t.baseM = static_cast<int32_t>(mmCFG.basicM);
            t.baseN = static_cast<int32_t>(mmCFG.basicN);
            t.baseK = static_cast<int32_t>(mmCFG.basicK);
            t.dbL0A = 1;
            t.dbL0B = 1;
            t.isBias = mmCFG.enableSetBias ? 1 : 0;
        }
        return t;
    }
    t.M = t.singleCoreM = static_cast<int32_t>(mmCFG.singleCoreM);
    t.N = t.singleCoreN = static_cast<int32_t>(mmCFG.singleCoreN);
    t.Ka = t.Kb = t.singleCoreK = static_cast<int32_t>(mmCFG.singleCoreK);
    t.baseM = static_cast<int32_t>(mmCFG.basicM);
    t.baseN = static_cast<int32_t>(mmCFG.basicN);
    t.baseK = static_cast<int32_t>(mmCFG.basicK);
    t.isBias = mmCFG.enableSetBias ? 1 : 0;
    t.stepM = t.stepN = t.stepKa = t.stepKb = 1;
    t.depthA1 = t.depthB1 = 1;
    t.dbL0A = t.dbL0B = t.dbL0C = 1;
    t.iterateOrder = 0;
    t.usedCoreNum = 1;
    return t;
}
}  // namespace AscendC
