// SoftMax, AscendQuant and AscendDequant with the reference's argument lists, forwarding to the C ABI.
// Included by kernel_operator.h.  Tensors are device memory holding the whole operand; sharedTmpBuffer
// arguments are accepted and ignored (the B200 kernels keep their working set in registers).
#pragma once

namespace AscendC {

// include/adv_api/activation/softmax_utils.h:33-78
enum class SoftmaxMode { SOFTMAX_NORMAL = 0, SOFTMAX_OUTPUT_WITHOUT_BRC = 1 };
struct SoftmaxConfig {
    constexpr SoftmaxConfig(bool isCheckTilingIn = true, uint32_t oriSrcMIn = 0, uint32_t oriSrcKIn = 0,
                            SoftmaxMode modeIn = SoftmaxMode::SOFTMAX_NORMAL)
        : isCheckTiling(isCheckTilingIn), oriSrcM(oriSrcMIn), oriSrcK(oriSrcKIn), mode(modeIn)
    {}
    bool isCheckTiling;
    uint32_t oriSrcM, oriSrcK;
    SoftmaxMode mode;
};
constexpr SoftmaxConfig SOFTMAX_DEFAULT_CFG = {true, 0, 0, SoftmaxMode::SOFTMAX_NORMAL};
struct SoftMaxShapeInfo {
    uint32_t srcM{0};
    uint32_t srcK{0};
    uint32_t oriSrcM{0};
    uint32_t oriSrcK{0};
};

// SoftMax<T>(dst, sum, max, src, tiling, shapeInfo)  (include/adv_api/activation/softmax.h:92-109).
// The shape comes from shapeInfo when given, else from the tiling, like the reference; sum / max are
// [srcM, 8] fp32 (one 32-byte block per row) unless config.mode is SOFTMAX_OUTPUT_WITHOUT_BRC.
template <typename T, bool isReuseSource = false, bool isBasicBlock = false, bool isDataFormatNZ = false,
          const SoftmaxConfig& config = SOFTMAX_DEFAULT_CFG>
inline void SoftMax(const LocalTensor<T>& dstTensor, const LocalTensor<float>& sumTensor, const LocalTensor<float>& maxTensor,
                    const LocalTensor<T>& srcTensor, const SoftMaxTiling& tiling, const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    static_assert(!isDataFormatNZ, "NZ-format SoftMax is not part of the B200 path");
    const uint32_t m = softmaxShapeInfo.srcM ? softmaxShapeInfo.srcM : tiling.srcM;
    const uint32_t k = softmaxShapeInfo.srcK ? softmaxShapeInfo.srcK : tiling.srcK;
    const int brc = config.mode == SoftmaxMode::SOFTMAX_OUTPUT_WITHOUT_BRC ? 0 : 1;
    detail::Latch(ascb200_softmax(srcTensor.GetPhyAddr(), dstTensor.GetPhyAddr(), sumTensor.GetPhyAddr(), maxTensor.GetPhyAddr(),
                                  static_cast<int32_t>(m), static_cast<int32_t>(k), detail::DTypeOf<T>::value, brc, detail::CurrentStream()),
                  "SoftMax");
}
template <typename T, bool isReuseSource = false, bool isBasicBlock = false, bool isDataFormatNZ = false,
          const SoftmaxConfig& config = SOFTMAX_DEFAULT_CFG>
inline void SoftMax(const LocalTensor<T>& dstTensor, const LocalTensor<float>& sumTensor, const LocalTensor<float>& maxTensor,
                    const LocalTensor<T>& srcTensor, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const SoftMaxTiling& tiling,
                    const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    SoftMax<T, isReuseSource, isBasicBlock, isDataFormatNZ, config>(dstTensor, sumTensor, maxTensor, srcTensor, tiling, softmaxShapeInfo);
}

// LogSoftMax<T>(dst, sum, max, src, sharedTmpBuffer, tiling, shapeInfo)  (include/adv_api/activation/logsoftmax.h:56-71).
// y = log10(softmax(x)); sum / max are LocalTensor<T> holding one 32-byte block per row ([srcM, 16] half or [srcM, 8] float).
template <typename T, bool isReuseSource = false, bool isDataFormatNZ = false>
inline void LogSoftMax(const LocalTensor<T>& dst, const LocalTensor<T>& sum, const LocalTensor<T>& max, const LocalTensor<T>& src,
                       const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const LogSoftMaxTiling& tiling,
                       const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    static_assert(!isDataFormatNZ, "NZ-format LogSoftMax is not part of the B200 path");
    const uint32_t m = softmaxShapeInfo.srcM ? softmaxShapeInfo.srcM : tiling.srcM;
    const uint32_t k = softmaxShapeInfo.srcK ? softmaxShapeInfo.srcK : tiling.srcK;
    detail::Latch(ascb200_log_softmax(src.GetPhyAddr(), dst.GetPhyAddr(), sum.GetPhyAddr(), max.GetPhyAddr(), static_cast<int32_t>(m),
                                      static_cast<int32_t>(k), detail::DTypeOf<T>::value, 1, detail::CurrentStream()),
                  "LogSoftMax");
}

// SimpleSoftMax<T>(dst, inSum, inMax, src, tiling, shapeInfo)  (include/adv_api/activation/simplesoftmax.h:55-190):
// the all-T form, the half-data / float-statistics form, and both again with a sharedTmpBuffer.
namespace detail {
template <typename T, typename ST>
inline void SimpleSoftMaxCall(const LocalTensor<T>& dst, const LocalTensor<ST>& inSum, const LocalTensor<ST>& inMax, const LocalTensor<T>& src,
                              const SoftMaxTiling& tiling, const SoftMaxShapeInfo& info, const SoftmaxConfig& config)
{
    const uint32_t m = info.srcM ? info.srcM : tiling.srcM;
    const uint32_t k = info.srcK ? info.srcK : tiling.srcK;
    const int brc = config.mode == SoftmaxMode::SOFTMAX_OUTPUT_WITHOUT_BRC ? 0 : 1;
    Latch(ascb200_simple_softmax(src.GetPhyAddr(), dst.GetPhyAddr(), inSum.GetPhyAddr(), inMax.GetPhyAddr(), static_cast<int32_t>(m),
                                 static_cast<int32_t>(k), DTypeOf<T>::value, DTypeOf<ST>::value, brc, CurrentStream()),
          "SimpleSoftMax");
}
}  // namespace detail
template <typename T, bool isReuseSource = false, bool isBasicBlock = false, bool isDataFormatNZ = false,
          const SoftmaxConfig& config = SOFTMAX_DEFAULT_CFG>
inline void SimpleSoftMax(const LocalTensor<T>& dstTensor, const LocalTensor<T>& inSumTensor, const LocalTensor<T>& inMaxTensor,
                          const LocalTensor<T>& srcTensor, const SoftMaxTiling& tiling, const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    static_assert(!isDataFormatNZ, "NZ-format SimpleSoftMax is not part of the B200 path");
    detail::SimpleSoftMaxCall(dstTensor, inSumTensor, inMaxTensor, srcTensor, tiling, softmaxShapeInfo, config);
}
template <typename T, bool isReuseSource = false, bool isBasicBlock = false, bool isDataFormatNZ = false,
          const SoftmaxConfig& config = SOFTMAX_DEFAULT_CFG>
inline void SimpleSoftMax(const LocalTensor<half>& dstTensor, const LocalTensor<float>& inSumTensor, const LocalTensor<float>& inMaxTensor,
                          const LocalTensor<half>& srcTensor, const SoftMaxTiling& tiling, const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    static_assert(!isDataFormatNZ, "NZ-format SimpleSoftMax is not part of the B200 path");
    detail::SimpleSoftMaxCall(dstTensor, inSumTensor, inMaxTensor, srcTensor, tiling, softmaxShapeInfo, config);
}
template <typename T, bool isReuseSource = false, bool isBasicBlock = false, bool isDataFormatNZ = false,
          const SoftmaxConfig& config = SOFTMAX_DEFAULT_CFG>
inline void SimpleSoftMax(const LocalTensor<T>& dstTensor, const LocalTensor<T>& inSumTensor, const LocalTensor<T>& inMaxTensor,
                          const LocalTensor<T>& srcTensor, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const SoftMaxTiling& tiling,
                          const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    SimpleSoftMax<T, isReuseSource, isBasicBlock, isDataFormatNZ, config>(dstTensor, inSumTensor, inMaxTensor, srcTensor, tiling, softmaxShapeInfo);
}
template <typename T, bool isReuseSource = false, bool isBasicBlock = false, bool isDataFormatNZ = false,
          const SoftmaxConfig& config = SOFTMAX_DEFAULT_CFG>
inline void SimpleSoftMax(const LocalTensor<half>& dstTensor, const LocalTensor<float>& inSumTensor, const LocalTensor<float>& inMaxTensor,
                          const LocalTensor<half>& srcTensor, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const SoftMaxTiling& tiling,
                          const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    SimpleSoftMax<T, isReuseSource, isBasicBlock, isDataFormatNZ, config>(dstTensor, inSumTensor, inMaxTensor, srcTensor, tiling, softmaxShapeInfo);
}

// SoftmaxGrad<T>(dst, grad, src, [sharedTmpBuffer,] tiling, isFront, shapeInfo) and SoftmaxGradFront<T>(dst, grad, src,
// [sharedTmpBuffer,] tiling, shapeInfo)  (include/adv_api/activation/softmaxgrad.h:57-175).  src is the softmax output y.
template <typename T, bool isReuseSource = false, bool isDataFormatNZ = false>
inline void SoftmaxGrad(const LocalTensor<T>& dstTensor, const LocalTensor<T>& gradTensor, const LocalTensor<T>& srcTensor,
                        const SoftMaxTiling& tiling, bool isFront = false, const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    static_assert(!isDataFormatNZ, "NZ-format SoftmaxGrad is not part of the B200 path");
    const uint32_t m = softmaxShapeInfo.srcM ? softmaxShapeInfo.srcM : tiling.srcM;
    const uint32_t k = softmaxShapeInfo.srcK ? softmaxShapeInfo.srcK : tiling.srcK;
    detail::Latch(ascb200_softmax_grad(gradTensor.GetPhyAddr(), srcTensor.GetPhyAddr(), dstTensor.GetPhyAddr(), static_cast<int32_t>(m),
                                       static_cast<int32_t>(k), detail::DTypeOf<T>::value, isFront ? 1 : 0, detail::CurrentStream()),
                  "SoftmaxGrad");
}
template <typename T, bool isReuseSource = false, bool isDataFormatNZ = false>
inline void SoftmaxGrad(const LocalTensor<T>& dstTensor, const LocalTensor<T>& gradTensor, const LocalTensor<T>& srcTensor,
                        const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const SoftMaxTiling& tiling, bool isFront = false,
                        const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    SoftmaxGrad<T, isReuseSource, isDataFormatNZ>(dstTensor, gradTensor, srcTensor, tiling, isFront, softmaxShapeInfo);
}
template <typename T, bool isBasicBlock = false, bool isDataFormatNZ = false>
inline void SoftmaxGradFront(const LocalTensor<T>& dstTensor, const LocalTensor<T>& gradTensor, const LocalTensor<T>& srcTensor,
                             const SoftMaxTiling& tiling, const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    SoftmaxGrad<T, false, isDataFormatNZ>(dstTensor, gradTensor, srcTensor, tiling, true, softmaxShapeInfo);
}
template <typename T, bool isBasicBlock = false, bool isDataFormatNZ = false>
inline void SoftmaxGradFront(const LocalTensor<T>& dstTensor, const LocalTensor<T>& gradTensor, const LocalTensor<T>& srcTensor,
                             const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const SoftMaxTiling& tiling,
                             const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    SoftmaxGrad<T, false, isDataFormatNZ>(dstTensor, gradTensor, srcTensor, tiling, true, softmaxShapeInfo);
}

// AscendAntiQuant<InputDataType, OutputDataType, isTranspose>(dst, src, [offset,] scale, [sharedTmpBuffer,] k, shapeInfo)
// (include/adv_api/quantization/ascend_antiquant.h:47-200), int8 source, half / bfloat16 output: dst = scale * (src + offset).
// Per channel: src is [k, n] with one (scale, offset) pair per column (isTranspose = false) or [n, k] with one pair per row
// (isTranspose = true); n = src.GetSize() / k.  Per tensor: scalar scale / offset in the output type.
struct AntiQuantShapeInfo {  // include/adv_api/quantization/ascend_antiquant_utils.h:27-32
    uint32_t offsetHeight{0};
    uint32_t offsetWidth{0};
    uint32_t scaleHeight{0};
    uint32_t scaleWidth{0};
};
namespace detail {
template <typename OutputDataType, bool isTranspose>
inline void AntiQuantChannel(const LocalTensor<OutputDataType>& dst, const LocalTensor<int8_t>& src, const void* offset,
                             const LocalTensor<OutputDataType>& scale, uint32_t k)
{
    const uint32_t n = k ? static_cast<uint32_t>(src.GetSize() / k) : 0;
    Latch(ascb200_antiquant(src.GetPhyAddr(), dst.GetPhyAddr(), static_cast<int32_t>(isTranspose ? n : k), static_cast<int32_t>(isTranspose ? k : n),
                            DTypeOf<OutputDataType>::value, isTranspose ? 2 : 1, scale.GetPhyAddr(), offset, 1.0f, 0.0f, CurrentStream()),
          "AscendAntiQuant");
}
template <typename OutputDataType>
inline void AntiQuantTensor(const LocalTensor<OutputDataType>& dst, const LocalTensor<int8_t>& src, OutputDataType offset, OutputDataType scale,
                            uint32_t k)
{
    const uint32_t n = k ? static_cast<uint32_t>(src.GetSize() / k) : 0;
    Latch(ascb200_antiquant(src.GetPhyAddr(), dst.GetPhyAddr(), static_cast<int32_t>(k), static_cast<int32_t>(n), DTypeOf<OutputDataType>::value, 0,
                            nullptr, nullptr, static_cast<float>(scale), static_cast<float>(offset), CurrentStream()),
          "AscendAntiQuant");
}
}  // namespace detail
template <typename InputDataType, typename OutputDataType, bool isTranspose>
inline void AscendAntiQuant(const LocalTensor<OutputDataType>& dst, const LocalTensor<InputDataType>& src, const LocalTensor<OutputDataType>& offset,
                            const LocalTensor<OutputDataType>& scale, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const uint32_t k,
                            const AntiQuantShapeInfo& = {})
{
    static_assert(std::is_same<InputDataType, int8_t>::value, "the B200 path anti-quantises int8 sources");
    detail::AntiQuantChannel<OutputDataType, isTranspose>(dst, src, offset.GetPhyAddr(), scale, k);
}
template <typename InputDataType, typename OutputDataType, bool isTranspose>
inline void AscendAntiQuant(const LocalTensor<OutputDataType>& dst, const LocalTensor<InputDataType>& src, const LocalTensor<OutputDataType>& scale,
                            const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const uint32_t k, const AntiQuantShapeInfo& = {})
{
    static_assert(std::is_same<InputDataType, int8_t>::value, "the B200 path anti-quantises int8 sources");
    detail::AntiQuantChannel<OutputDataType, isTranspose>(dst, src, nullptr, scale, k);
}
template <typename InputDataType, typename OutputDataType, bool isTranspose>
inline void AscendAntiQuant(const LocalTensor<OutputDataType>& dst, const LocalTensor<InputDataType>& src, const LocalTensor<OutputDataType>& offset,
                            const LocalTensor<OutputDataType>& scale, const uint32_t k, const AntiQuantShapeInfo& = {})
{
    static_assert(std::is_same<InputDataType, int8_t>::value, "the B200 path anti-quantises int8 sources");
    detail::AntiQuantChannel<OutputDataType, isTranspose>(dst, src, offset.GetPhyAddr(), scale, k);
}
template <typename InputDataType, typename OutputDataType, bool isTranspose>
inline void AscendAntiQuant(const LocalTensor<OutputDataType>& dst, const LocalTensor<InputDataType>& src, const OutputDataType offset,
                            const OutputDataType scale, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const uint32_t k,
                            const AntiQuantShapeInfo& = {})
{
    static_assert(std::is_same<InputDataType, int8_t>::value, "the B200 path anti-quantises int8 sources");
    detail::AntiQuantTensor<OutputDataType>(dst, src, offset, scale, k);
}
template <typename InputDataType, typename OutputDataType, bool isTranspose>
inline void AscendAntiQuant(const LocalTensor<OutputDataType>& dst, const LocalTensor<InputDataType>& src, const OutputDataType scale,
                            const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const uint32_t k, const AntiQuantShapeInfo& = {})
{
    static_assert(std::is_same<InputDataType, int8_t>::value, "the B200 path anti-quantises int8 sources");
    detail::AntiQuantTensor<OutputDataType>(dst, src, OutputDataType(0.0f), scale, k);
}
template <typename InputDataType, typename OutputDataType, bool isTranspose>
inline void AscendAntiQuant(const LocalTensor<OutputDataType>& dst, const LocalTensor<InputDataType>& src, const OutputDataType offset,
                            const OutputDataType scale, const uint32_t k, const AntiQuantShapeInfo& = {})
{
    static_assert(std::is_same<InputDataType, int8_t>::value, "the B200 path anti-quantises int8 sources");
    detail::AntiQuantTensor<OutputDataType>(dst, src, offset, scale, k);
}

// SoftmaxFlash<T>(dst, sum, max, src, expMax, inSum, inMax, [sharedTmpBuffer,] tiling, isUpdate, shapeInfo)
// (include/adv_api/activation/softmaxflash.h:65-215; deprecated by the reference in favour of SoftmaxFlashV2, kept for existing callers).
namespace detail {
template <typename T, typename ST>
inline void SoftmaxFlashCall(const LocalTensor<T>& dst, const LocalTensor<ST>& sum, const LocalTensor<ST>& max, const LocalTensor<T>& src,
                             const LocalTensor<T>& expMax, const LocalTensor<ST>& inSum, const LocalTensor<ST>& inMax, const SoftMaxTiling& tiling,
                             bool isUpdate, const SoftMaxShapeInfo& info)
{
    const uint32_t m = info.srcM ? info.srcM : tiling.srcM;
    const uint32_t k = info.srcK ? info.srcK : tiling.srcK;
    Latch(ascb200_softmax_flash(src.GetPhyAddr(), dst.GetPhyAddr(), sum.GetPhyAddr(), max.GetPhyAddr(), expMax.GetPhyAddr(), inSum.GetPhyAddr(),
                                inMax.GetPhyAddr(), static_cast<int32_t>(m), static_cast<int32_t>(k), DTypeOf<T>::value, DTypeOf<ST>::value,
                                isUpdate ? 1 : 0, 1, CurrentStream()),
          "SoftmaxFlash");
}
}  // namespace detail
template <typename T, bool isReuseSource = false, bool isBasicBlock = false>
inline void SoftmaxFlash(const LocalTensor<T>& dstTensor, const LocalTensor<T>& sumTensor, const LocalTensor<T>& maxTensor,
                         const LocalTensor<T>& srcTensor, const LocalTensor<T>& expMaxTensor, const LocalTensor<T>& inSumTensor,
                         const LocalTensor<T>& inMaxTensor, const SoftMaxTiling& tiling, bool isUpdate = false,
                         const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    detail::SoftmaxFlashCall(dstTensor, sumTensor, maxTensor, srcTensor, expMaxTensor, inSumTensor, inMaxTensor, tiling, isUpdate, softmaxShapeInfo);
}
template <typename T, bool isReuseSource = false, bool isBasicBlock = false>
inline void SoftmaxFlash(const LocalTensor<half>& dstTensor, const LocalTensor<float>& sumTensor, const LocalTensor<float>& maxTensor,
                         const LocalTensor<half>& srcTensor, const LocalTensor<half>& expMaxTensor, const LocalTensor<float>& inSumTensor,
                         const LocalTensor<float>& inMaxTensor, const SoftMaxTiling& tiling, bool isUpdate = false,
                         const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    detail::SoftmaxFlashCall(dstTensor, sumTensor, maxTensor, srcTensor, expMaxTensor, inSumTensor, inMaxTensor, tiling, isUpdate, softmaxShapeInfo);
}
template <typename T, bool isReuseSource = false, bool isBasicBlock = false>
inline void SoftmaxFlash(const LocalTensor<T>& dstTensor, const LocalTensor<T>& sumTensor, const LocalTensor<T>& maxTensor,
                         const LocalTensor<T>& srcTensor, const LocalTensor<T>& expMaxTensor, const LocalTensor<T>& inSumTensor,
                         const LocalTensor<T>& inMaxTensor, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const SoftMaxTiling& tiling,
                         bool isUpdate = false, const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    detail::SoftmaxFlashCall(dstTensor, sumTensor, maxTensor, srcTensor, expMaxTensor, inSumTensor, inMaxTensor, tiling, isUpdate, softmaxShapeInfo);
}
template <typename T, bool isReuseSource = false, bool isBasicBlock = false>
inline void SoftmaxFlash(const LocalTensor<half>& dstTensor, const LocalTensor<float>& sumTensor, const LocalTensor<float>& maxTensor,
                         const LocalTensor<half>& srcTensor, const LocalTensor<half>& expMaxTensor, const LocalTensor<float>& inSumTensor,
                         const LocalTensor<float>& inMaxTensor, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const SoftMaxTiling& tiling,
                         bool isUpdate = false, const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    detail::SoftmaxFlashCall(dstTensor, sumTensor, maxTensor, srcTensor, expMaxTensor, inSumTensor, inMaxTensor, tiling, isUpdate, softmaxShapeInfo);
}

// SoftmaxFlashV2<T, isUpdate>(dst, expSum, max, src, expMax, inExpSum, inMax, tiling, shapeInfo)
// (include/adv_api/activation/softmaxflashv2.h:93-260): the all-T overloads and the half data / float statistics overloads,
// each with and without sharedTmpBuffer.
namespace detail {
template <typename T, typename ST, bool isUpdate, const SoftmaxConfig& config>
inline void SoftmaxFlashV2Call(const LocalTensor<T>& dst, const LocalTensor<ST>& expSum, const LocalTensor<ST>& max, const LocalTensor<T>& src,
                               const LocalTensor<T>& expMax, const LocalTensor<ST>& inExpSum, const LocalTensor<ST>& inMax,
                               const SoftMaxTiling& tiling, const SoftMaxShapeInfo& shape)
{
    const uint32_t m = shape.srcM ? shape.srcM : tiling.srcM;
    const uint32_t k = shape.srcK ? shape.srcK : tiling.srcK;
    const int brc = config.mode == SoftmaxMode::SOFTMAX_OUTPUT_WITHOUT_BRC ? 0 : 1;
    Latch(ascb200_softmax_flash_v2(src.GetPhyAddr(), dst.GetPhyAddr(), expSum.GetPhyAddr(), max.GetPhyAddr(), expMax.GetPhyAddr(),
                                   inExpSum.GetPhyAddr(), inMax.GetPhyAddr(), static_cast<int32_t>(m), static_cast<int32_t>(k), DTypeOf<T>::value,
                                   DTypeOf<ST>::value, isUpdate ? 1 : 0, brc, CurrentStream()),
          "SoftmaxFlashV2");
}
}  // namespace detail
template <typename T, bool isUpdate = false, bool isReuseSource = false, bool isBasicBlock = false, bool isDataFormatNZ = false,
          const SoftmaxConfig& config = SOFTMAX_DEFAULT_CFG>
inline void SoftmaxFlashV2(const LocalTensor<T>& dstTensor, const LocalTensor<T>& expSumTensor, const LocalTensor<T>& maxTensor,
                           const LocalTensor<T>& srcTensor, const LocalTensor<T>& expMaxTensor, const LocalTensor<T>& inExpSumTensor,
                           const LocalTensor<T>& inMaxTensor, const SoftMaxTiling& tiling, const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    static_assert(!isDataFormatNZ, "NZ-format SoftmaxFlashV2 is not part of the B200 path");
    detail::SoftmaxFlashV2Call<T, T, isUpdate, config>(dstTensor, expSumTensor, maxTensor, srcTensor, expMaxTensor, inExpSumTensor, inMaxTensor,
                                                       tiling, softmaxShapeInfo);
}
template <typename T, bool isUpdate = false, bool isReuseSource = false, bool isBasicBlock = false, bool isDataFormatNZ = false,
          const SoftmaxConfig& config = SOFTMAX_DEFAULT_CFG>
inline void SoftmaxFlashV2(const LocalTensor<half>& dstTensor, const LocalTensor<float>& expSumTensor, const LocalTensor<float>& maxTensor,
                           const LocalTensor<half>& srcTensor, const LocalTensor<half>& expMaxTensor, const LocalTensor<float>& inExpSumTensor,
                           const LocalTensor<float>& inMaxTensor, const SoftMaxTiling& tiling, const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    static_assert(!isDataFormatNZ, "NZ-format SoftmaxFlashV2 is not part of the B200 path");
    detail::SoftmaxFlashV2Call<half, float, isUpdate, config>(dstTensor, expSumTensor, maxTensor, srcTensor, expMaxTensor, inExpSumTensor,
                                                              inMaxTensor, tiling, softmaxShapeInfo);
}
template <typename T, bool isUpdate = false, bool isReuseSource = false, bool isBasicBlock = false, bool isDataFormatNZ = false,
          const SoftmaxConfig& config = SOFTMAX_DEFAULT_CFG>
inline void SoftmaxFlashV2(const LocalTensor<T>& dstTensor, const LocalTensor<T>& expSumTensor, const LocalTensor<T>& maxTensor,
                           const LocalTensor<T>& srcTensor, const LocalTensor<T>& expMaxTensor, const LocalTensor<T>& inExpSumTensor,
                           const LocalTensor<T>& inMaxTensor, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const SoftMaxTiling& tiling,
                           const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    SoftmaxFlashV2<T, isUpdate, isReuseSource, isBasicBlock, isDataFormatNZ, config>(dstTensor, expSumTensor, maxTensor, srcTensor, expMaxTensor,
                                                                                      inExpSumTensor, inMaxTensor, tiling, softmaxShapeInfo);
}
template <typename T, bool isUpdate = false, bool isReuseSource = false, bool isBasicBlock = false, bool isDataFormatNZ = false,
          const SoftmaxConfig& config = SOFTMAX_DEFAULT_CFG>
inline void SoftmaxFlashV2(const LocalTensor<half>& dstTensor, const LocalTensor<float>& expSumTensor, const LocalTensor<float>& maxTensor,
                           const LocalTensor<half>& srcTensor, const LocalTensor<half>& expMaxTensor, const LocalTensor<float>& inExpSumTensor,
                           const LocalTensor<float>& inMaxTensor, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const SoftMaxTiling& tiling,
                           const SoftMaxShapeInfo& softmaxShapeInfo = {})
{
    SoftmaxFlashV2<T, isUpdate, isReuseSource, isBasicBlock, isDataFormatNZ, config>(dstTensor, expSumTensor, maxTensor, srcTensor, expMaxTensor,
                                                                                      inExpSumTensor, inMaxTensor, tiling, softmaxShapeInfo);
}

// include/adv_api/quantization/ascend_quant_utils.h:31-73
struct AscendQuantConfig {
    constexpr AscendQuantConfig(uint32_t calcCountIn, uint32_t offsetCountIn, uint32_t scaleCountIn, uint32_t workLocalSizeIn,
                                bool hasOffsetIn = false, int32_t kDimIn = 1, RoundMode roundModeIn = RoundMode::CAST_RINT)
        : calcCount(calcCountIn), offsetCount(offsetCountIn), scaleCount(scaleCountIn), workLocalSize(workLocalSizeIn),
          hasOffset(hasOffsetIn), kDim(kDimIn), roundMode(roundModeIn)
    {}
    uint32_t calcCount, offsetCount, scaleCount, workLocalSize;
    bool hasOffset;
    int32_t kDim;
    RoundMode roundMode;
};
constexpr AscendQuantConfig ASCEND_QUANT_DEFAULT_CFG = {0, 0, 0, 0, false, 1, RoundMode::CAST_RINT};

namespace detail {
template <typename T>
inline void QuantPerTensor(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, float scale, float offset, uint64_t calCount)
{
    Latch(ascb200_quant_per_tensor(src.GetPhyAddr(), dst.GetPhyAddr(), static_cast<int64_t>(calCount), DTypeOf<T>::value, scale, offset,
                                   CurrentStream()),
          "AscendQuant");
}
template <typename T>
inline void QuantPerChannel(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const LocalTensor<T>& scale, const T* offsetTensor,
                            float offsetScalar, uint64_t scaleCount, uint64_t calCount)
{
    if (scaleCount == 0 || calCount % scaleCount != 0) {
        Latch(ASCB200_EINVAL, "AscendQuant (calCount must be a multiple of scaleCount)");
        return;
    }
    Latch(ascb200_quant_per_channel(src.GetPhyAddr(), dst.GetPhyAddr(), static_cast<int32_t>(calCount / scaleCount),
                                    static_cast<int32_t>(scaleCount), DTypeOf<T>::value, scale.GetPhyAddr(), offsetTensor, offsetScalar,
                                    CurrentStream()),
          "AscendQuant");
}
}  // namespace detail

// per tensor (include/adv_api/quantization/ascend_quant.h:63-136)
template <typename T, bool isReuseSource = false, const AscendQuantConfig& config = ASCEND_QUANT_DEFAULT_CFG>
inline void AscendQuant(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const float scale, const float offset, const uint32_t calCount)
{
    static_assert(config.roundMode == RoundMode::CAST_RINT, "only CAST_RINT is implemented");
    detail::QuantPerTensor<T>(dst, src, scale, offset, calCount);
}
template <typename T, bool isReuseSource = false, const AscendQuantConfig& config = ASCEND_QUANT_DEFAULT_CFG>
inline void AscendQuant(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/,
                        const float scale, const float offset, const uint32_t calCount)
{
    detail::QuantPerTensor<T>(dst, src, scale, offset, calCount);
}
template <typename T, bool isReuseSource = false, const AscendQuantConfig& config = ASCEND_QUANT_DEFAULT_CFG>
inline void AscendQuant(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const float scale, const float offset)
{
    detail::QuantPerTensor<T>(dst, src, scale, offset, src.GetSize());
}
template <typename T, bool isReuseSource = false, const AscendQuantConfig& config = ASCEND_QUANT_DEFAULT_CFG>
inline void AscendQuant(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/,
                        const float scale, const float offset)
{
    detail::QuantPerTensor<T>(dst, src, scale, offset, src.GetSize());
}
// per channel, scalar offset (ascend_quant.h:159-236)
template <typename T, bool isReuseSource = false, const AscendQuantConfig& config = ASCEND_QUANT_DEFAULT_CFG>
inline void AscendQuant(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const LocalTensor<T>& scaleTensor, const T offset,
                        const uint32_t scaleCount, const uint32_t calCount)
{
    detail::QuantPerChannel<T>(dst, src, scaleTensor, nullptr, static_cast<float>(offset), scaleCount, calCount);
}
template <typename T, bool isReuseSource = false, const AscendQuantConfig& config = ASCEND_QUANT_DEFAULT_CFG>
inline void AscendQuant(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/,
                        const LocalTensor<T>& scaleTensor, const T offset, const uint32_t scaleCount, const uint32_t calCount)
{
    detail::QuantPerChannel<T>(dst, src, scaleTensor, nullptr, static_cast<float>(offset), scaleCount, calCount);
}
template <typename T, bool isReuseSource = false, const AscendQuantConfig& config = ASCEND_QUANT_DEFAULT_CFG>
inline void AscendQuant(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const LocalTensor<T>& scaleTensor, const T offset)
{
    detail::QuantPerChannel<T>(dst, src, scaleTensor, nullptr, static_cast<float>(offset), scaleTensor.GetSize(), src.GetSize());
}
// per channel, offset tensor (ascend_quant.h:261-342)
template <typename T, bool isReuseSource = false, const AscendQuantConfig& config = ASCEND_QUANT_DEFAULT_CFG>
inline void AscendQuant(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const LocalTensor<T>& scaleTensor,
                        const LocalTensor<T>& offsetTensor, const uint32_t scaleCount, const uint32_t offsetCount, const uint32_t calCount)
{
    if (offsetCount != scaleCount) {
        detail::Latch(ASCB200_EINVAL, "AscendQuant (offsetCount must equal scaleCount)");
        return;
    }
    detail::QuantPerChannel<T>(dst, src, scaleTensor, offsetTensor.GetPhyAddr(), 0.0f, scaleCount, calCount);
}
template <typename T, bool isReuseSource = false, const AscendQuantConfig& config = ASCEND_QUANT_DEFAULT_CFG>
inline void AscendQuant(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/,
                        const LocalTensor<T>& scaleTensor, const LocalTensor<T>& offsetTensor, const uint32_t scaleCount,
                        const uint32_t offsetCount, const uint32_t calCount)
{
    AscendQuant<T, isReuseSource, config>(dst, src, scaleTensor, offsetTensor, scaleCount, offsetCount, calCount);
}
template <typename T, bool isReuseSource = false, const AscendQuantConfig& config = ASCEND_QUANT_DEFAULT_CFG>
inline void AscendQuant(const LocalTensor<int8_t>& dst, const LocalTensor<T>& src, const LocalTensor<T>& scaleTensor,
                        const LocalTensor<T>& offsetTensor)
{
    detail::QuantPerChannel<T>(dst, src, scaleTensor, offsetTensor.GetPhyAddr(), 0.0f, scaleTensor.GetSize(), src.GetSize());
}

// ---- AscendQuant with a policy (include/adv_api/quantization/ascend_quant.h:682-790) ---------------------------
// include/adv_api/quantization/ascend_quant_utils.h:75-89
enum class AscendQuantPolicy : int32_t { PER_TENSOR, PER_CHANNEL, PER_TOKEN, PER_GROUP, PER_CHANNEL_PER_GROUP, PER_TOKEN_PER_GROUP };
struct AscendQuantParam {
    uint32_t m;
    uint32_t n;
    uint32_t calCount;
    uint32_t groupSize = 0;
};

namespace detail {
template <typename dstT, typename srcT, typename scaleT, const AscendQuantConfig& config, const AscendQuantPolicy& policy>
inline void QuantPolicy(const LocalTensor<dstT>& dst, const LocalTensor<srcT>& src, const LocalTensor<scaleT>& scale, const scaleT* offsetTensor,
                        float offsetScalar, const AscendQuantParam& para)
{
    static_assert(policy == AscendQuantPolicy::PER_TOKEN || policy == AscendQuantPolicy::PER_GROUP,
                  "unsupported policy for AscendQuant in current device!");  // the reference's own restriction
    static_assert(config.roundMode == RoundMode::CAST_NONE || config.roundMode == RoundMode::CAST_RINT || config.roundMode == RoundMode::CAST_FLOOR ||
                      config.roundMode == RoundMode::CAST_CEIL || config.roundMode == RoundMode::CAST_ROUND || config.roundMode == RoundMode::CAST_TRUNC,
                  "CAST_ODD and the hybrid rounding modes are not implemented");
    static_assert(config.roundMode == RoundMode::CAST_NONE || config.roundMode == RoundMode::CAST_RINT || std::is_same<dstT, int8_t>::value,
                  "fp8 / fp4 destinations round to nearest even only");
    if (para.n == 0 || para.calCount % para.n != 0) {
        Latch(ASCB200_EINVAL, "AscendQuant (calCount must be an integer multiple of n)");
        return;
    }
    Latch(ascb200_quant_policy_rm(src.GetPhyAddr(), dst.GetPhyAddr(), static_cast<int32_t>(para.calCount / para.n), static_cast<int32_t>(para.n),
                                  DTypeOf<srcT>::value, DTypeOf<scaleT>::value, DTypeOf<dstT>::value, static_cast<int32_t>(policy), config.kDim,
                                  static_cast<int32_t>(para.groupSize), scale.GetPhyAddr(), offsetTensor, offsetScalar, config.hasOffset ? 1 : 0,
                                  static_cast<int32_t>(config.roundMode), CurrentStream()),
          "AscendQuant (policy)");
}
}  // namespace detail

template <typename dstT, typename srcT, typename scaleT, bool isReuseSource = false, const AscendQuantConfig& config,
          const AscendQuantPolicy& policy>
inline void AscendQuant(const LocalTensor<dstT>& dstTensor, const LocalTensor<srcT>& srcTensor, const LocalTensor<scaleT>& scaleTensor,
                        const LocalTensor<scaleT>& offsetTensor, const AscendQuantParam& para)
{
    detail::QuantPolicy<dstT, srcT, scaleT, config, policy>(dstTensor, srcTensor, scaleTensor, offsetTensor.GetPhyAddr(), 0.0f, para);
}
template <typename dstT, typename srcT, typename scaleT, bool isReuseSource = false, const AscendQuantConfig& config,
          const AscendQuantPolicy& policy>
inline void AscendQuant(const LocalTensor<dstT>& dstTensor, const LocalTensor<srcT>& srcTensor, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/,
                        const LocalTensor<scaleT>& scaleTensor, const LocalTensor<scaleT>& offsetTensor, const AscendQuantParam& para)
{
    detail::QuantPolicy<dstT, srcT, scaleT, config, policy>(dstTensor, srcTensor, scaleTensor, offsetTensor.GetPhyAddr(), 0.0f, para);
}
template <typename dstT, typename srcT, typename scaleT, bool isReuseSource = false, const AscendQuantConfig& config,
          const AscendQuantPolicy& policy>
inline void AscendQuant(const LocalTensor<dstT>& dstTensor, const LocalTensor<srcT>& srcTensor, const LocalTensor<scaleT>& scaleTensor,
                        const scaleT offset, const AscendQuantParam& para)
{
    detail::QuantPolicy<dstT, srcT, scaleT, config, policy>(dstTensor, srcTensor, scaleTensor, nullptr, static_cast<float>(offset), para);
}
template <typename dstT, typename srcT, typename scaleT, bool isReuseSource = false, const AscendQuantConfig& config,
          const AscendQuantPolicy& policy>
inline void AscendQuant(const LocalTensor<dstT>& dstTensor, const LocalTensor<srcT>& srcTensor, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/,
                        const LocalTensor<scaleT>& scaleTensor, const scaleT offset, const AscendQuantParam& para)
{
    detail::QuantPolicy<dstT, srcT, scaleT, config, policy>(dstTensor, srcTensor, scaleTensor, nullptr, static_cast<float>(offset), para);
}

// include/adv_api/quantization/ascend_dequant_utils.h:26-30
struct DequantParams {
    uint32_t m;         // rows of src
    uint32_t n;         // int32 elements per src row (a multiple of 8: 32 bytes)
    uint32_t calCount;  // leading elements of each row that are dequantised
};

namespace detail {
template <typename dstT>
inline uint32_t DequantDstRow(uint32_t n)
{
    const uint32_t perBlock = 32 / sizeof(dstT);  // dst rows are padded to a 32-byte multiple like in the reference
    return (n + perBlock - 1) / perBlock * perBlock;
}
template <DeQuantMode mode>
inline DequantParams DequantShape(DequantParams p)
{
    // {1, m*n, n} means {m, n, n} in single-row mode (include/adv_api/quantization/ascend_dequant.h, mode description)
    if (mode == DeQuantMode::DEQUANT_WITH_SINGLE_ROW && p.m == 1 && p.calCount > 0 && p.n > p.calCount && p.n % p.calCount == 0)
        return DequantParams{p.n / p.calCount, p.calCount, p.calCount};
    return p;
}
}  // namespace detail

// AscendDequant<dstT, scaleT, mode>(dst, src, deqScale, params)  (include/adv_api/quantization/ascend_dequant.h).
// scaleT float or bfloat16_t for a tensor scale; a uint64_t tensor carries the fp32 scale in its low 32 bits
// and is not supported here (convert once on the host).
template <typename dstT, typename scaleT, DeQuantMode mode = DeQuantMode::DEQUANT_WITH_SINGLE_ROW>
inline void AscendDequant(const LocalTensor<dstT>& dst, const LocalTensor<int32_t>& src, const LocalTensor<scaleT>& deqScale, DequantParams params)
{
    static_assert(sizeof(scaleT) != 8, "uint64_t deqScale tensors are not supported: pass the fp32 scales");
    const DequantParams p = detail::DequantShape<mode>(params);
    detail::Latch(ascb200_dequant(src.GetPhyAddr(), dst.GetPhyAddr(), static_cast<int32_t>(p.m), static_cast<int32_t>(p.n),
                                  static_cast<int32_t>(p.calCount), static_cast<int32_t>(detail::DequantDstRow<dstT>(p.n)),
                                  detail::DTypeOf<dstT>::value, deqScale.GetPhyAddr(), detail::DTypeOf<scaleT>::value, 0.0f,
                                  detail::CurrentStream()),
                  "AscendDequant");
}
template <typename dstT, typename scaleT, DeQuantMode mode = DeQuantMode::DEQUANT_WITH_SINGLE_ROW>
inline void AscendDequant(const LocalTensor<dstT>& dst, const LocalTensor<int32_t>& src, const LocalTensor<scaleT>& deqScale,
                          const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, DequantParams params)
{
    AscendDequant<dstT, scaleT, mode>(dst, src, deqScale, params);
}
// scalar scale overload
template <typename dstT, typename scaleT, DeQuantMode mode = DeQuantMode::DEQUANT_WITH_SINGLE_ROW>
inline void AscendDequant(const LocalTensor<dstT>& dst, const LocalTensor<int32_t>& src, const scaleT deqScale, DequantParams params)
{
    const DequantParams p = detail::DequantShape<mode>(params);
    detail::Latch(ascb200_dequant(src.GetPhyAddr(), dst.GetPhyAddr(), static_cast<int32_t>(p.m), static_cast<int32_t>(p.n),
                                  static_cast<int32_t>(p.calCount), static_cast<int32_t>(detail::DequantDstRow<dstT>(p.n)),
                                  detail::DTypeOf<dstT>::value, nullptr, ASCB200_F32, static_cast<float>(deqScale), detail::CurrentStream()),
                  "AscendDequant");
}

// ---- AscendDequant with a policy (include/adv_api/quantization/ascend_dequant.h:293-318) ----------------------------
// include/adv_api/quantization/ascend_dequant_utils.h:32-44
struct AscendDeQuantConfig {
    bool hasOffset;
    int32_t kDim = 1;
};
enum class AscendDeQuantPolicy : int32_t { PER_TOKEN, PER_GROUP, PER_CHANNEL_PER_GROUP, PER_TOKEN_PER_GROUP };
struct AscendDeQuantParam {
    uint32_t m;
    uint32_t n;
    uint32_t calCount;
    uint32_t groupSize = 0;
};
template <typename dstT, typename srcT, typename scaleT, const AscendDeQuantConfig& config, const AscendDeQuantPolicy& policy>
inline void AscendDequant(const LocalTensor<dstT>& dstTensor, const LocalTensor<srcT>& srcTensor, const LocalTensor<scaleT>& scaleTensor,
                          const LocalTensor<scaleT>& /*offsetTensor: not used by the reference's arithmetic*/, const AscendDeQuantParam& para)
{
    static_assert(policy == AscendDeQuantPolicy::PER_TOKEN || policy == AscendDeQuantPolicy::PER_GROUP,
                  "unsupported policy for AscendDequant in current device!");
    if (para.n == 0 || para.calCount % para.n != 0) {
        detail::Latch(ASCB200_EINVAL, "AscendDequant (calCount must be an integer multiple of n)");
        return;
    }
    detail::Latch(ascb200_dequant_policy(srcTensor.GetPhyAddr(), dstTensor.GetPhyAddr(), static_cast<int32_t>(para.calCount / para.n),
                                         static_cast<int32_t>(para.n), detail::DTypeOf<srcT>::value, detail::DTypeOf<scaleT>::value,
                                         detail::DTypeOf<dstT>::value, static_cast<int32_t>(policy), config.kDim,
                                         static_cast<int32_t>(para.groupSize), scaleTensor.GetPhyAddr(), detail::CurrentStream()),
                  "AscendDequant (policy)");
}
template <typename dstT, typename srcT, typename scaleT, const AscendDeQuantConfig& config, const AscendDeQuantPolicy& policy>
inline void AscendDequant(const LocalTensor<dstT>& dstTensor, const LocalTensor<srcT>& srcTensor, const LocalTensor<scaleT>& scaleTensor,
                          const LocalTensor<scaleT>& offsetTensor, const LocalTensor<uint8_t>& /*sharedTmpBuffer*/, const AscendDeQuantParam& para)
{
    AscendDequant<dstT, srcT, scaleT, config, policy>(dstTensor, srcTensor, scaleTensor, offsetTensor, para);
}

}  // namespace AscendC
