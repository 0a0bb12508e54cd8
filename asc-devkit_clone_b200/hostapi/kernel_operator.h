// Host-side mirror of the Ascend C kernel-side vocabulary for the hot path, for B200.
//
// In the reference these types live inside an NPU kernel (kernel_operator.h); here the same names
// describe device memory of a CUDA GPU and are used from ordinary host code: a GlobalTensor /
// LocalTensor is a non-owning view of device memory, TPipe carries the CUDA stream, and the
// operators (Matmul, SoftMax, AscendQuant, AscendDequant) launch kernels through the C ABI of
// ascb200.h.  "Single core" of the reference = the whole GPU: GetBlockIdx() is 0, GetBlockNum() is 1.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "ascb200.h"

#ifndef __CUDACC__
#ifndef __global__
#define __global__
#endif
#endif
#define __aicore__
#define __gm__
#define __cube__
#define __vector__
#define __mix__(c, v)
#define GM_ADDR uint8_t*

// ---- element types (bit-pattern wrappers; arithmetic happens on the GPU) --------------------------
struct half {
    uint16_t bits = 0;
    half() = default;
    half(float f) { bits = FromFloat(f); }  // CAST_RINT, IEEE overflow to inf
    operator float() const
    {
        const uint32_t sign = static_cast<uint32_t>(bits & 0x8000u) << 16, exp = (bits >> 10) & 0x1Fu, man = bits & 0x3FFu;
        uint32_t u;
        if (exp == 0) {
            if (man == 0) {
                u = sign;
            } else {
                float v = std::ldexp(static_cast<float>(man), -24);
                std::memcpy(&u, &v, 4);
                u |= sign;
            }
        } else if (exp == 31) {
            u = sign | 0x7F800000u | (man << 13);
        } else {
            u = sign | ((exp + 112u) << 23) | (man << 13);
        }
        float f;
        std::memcpy(&f, &u, 4);
        return f;
    }
    static uint16_t FromFloat(float f)
    {
        uint32_t u;
        std::memcpy(&u, &f, 4);
        const uint16_t sign = static_cast<uint16_t>((u >> 16) & 0x8000u);
        const uint32_t a = u & 0x7FFFFFFFu;
        if (a > 0x7F800000u) return sign | 0x7E00u;
        if (a >= 0x477FF000u) return sign | 0x7C00u;
        if (a < 0x33000001u) return sign;
        const int32_t e = static_cast<int32_t>(a >> 23) - 127;
        uint32_t m = (a & 0x7FFFFFu) | 0x800000u, base = 0;
        int shift = 13;
        if (e < -14) {
            shift = 13 + (-14 - e);
        } else {
            base = static_cast<uint32_t>(e + 15) << 10;
            m &= 0x7FFFFFu;
        }
        uint32_t q = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (q & 1u))) q++;
        return static_cast<uint16_t>(sign | (base + q));
    }
};
struct bfloat16_t {
    uint16_t bits = 0;
    bfloat16_t() = default;
    bfloat16_t(float f)
    {
        uint32_t u;
        std::memcpy(&u, &f, 4);
        if ((u & 0x7FFFFFFFu) > 0x7F800000u) {
            bits = static_cast<uint16_t>((u >> 16) | 0x40u);
        } else {
            u += 0x7FFFu + ((u >> 16) & 1u);
            bits = static_cast<uint16_t>(u >> 16);
        }
    }
    operator float() const
    {
        const uint32_t u = static_cast<uint32_t>(bits) << 16;
        float f;
        std::memcpy(&f, &u, 4);
        return f;
    }
};
struct fp4x2_e2m1_t { uint8_t bits = 0; };  // two e2m1 values, even index in the low nibble
struct fp4x2_e1m2_t { uint8_t bits = 0; };  // declared for completeness; B200 tensor cores have no e1m2 path
struct fp8_e8m0_t { uint8_t bits = 0; };    // 2^(bits-127)
struct fp8_e4m3fn_t { uint8_t bits = 0; };  // Matmul output of the QF322FP8_PRE fixpipe mode (no infinities, largest finite 448)
struct fp8_e5m2_t { uint8_t bits = 0; };    // largest finite 57344

// include/adv_api/matmul/matmul_config.h:26-37
enum class CubeFormat { ND = 0, NZ, ZN, ZZ, NN, ND_ALIGN, SCALAR, VECTOR, ROW_MAJOR = ND, COLUMN_MAJOR = 8 };

// 50 x int32, the order of include/adv_api/matmul/matmul_tilingdata.h:20-72
struct TCubeTiling {
    int32_t usedCoreNum, M, N, Ka, Kb, singleCoreM, singleCoreN, singleCoreK, baseM, baseN, baseK, depthA1, depthB1, stepM, stepN, isBias,
        transLength, iterateOrder, shareMode, shareL1Size, shareL0CSize, shareUbSize, batchM, batchN, singleBatchM, singleBatchN, stepKa,
        stepKb, depthAL1CacheUB, depthBL1CacheUB, dbL0A, dbL0B, dbL0C, ALayoutInfoB, ALayoutInfoS, ALayoutInfoN, ALayoutInfoG, ALayoutInfoD,
        BLayoutInfoB, BLayoutInfoS, BLayoutInfoN, BLayoutInfoG, BLayoutInfoD, CLayoutInfoB, CLayoutInfoS1, CLayoutInfoN, CLayoutInfoG,
        CLayoutInfoS2, BatchNum, mxTypePara;
};
static_assert(sizeof(TCubeTiling) == 200, "TCubeTiling is 50 int32 fields");

// 16 x uint32, include/adv_api/activation/softmax_tilingdata.h:20-38
struct SoftMaxTiling {
    uint32_t srcM, srcK, srcSize, outMaxM, outMaxK, outMaxSize, splitM, splitK, splitSize, reduceM, reduceK, reduceSize, rangeM, tailM,
        tailSplitSize, tailReduceSize;
};
static_assert(sizeof(SoftMaxTiling) == 64, "SoftMaxTiling is 16 uint32 fields");
// include/adv_api/activation/logsoftmax_tilingdata.h:20-37: the same 16 fields under its own name.
struct LogSoftMaxTiling {
    uint32_t srcM, srcK, srcSize, outMaxM, outMaxK, outMaxSize, splitM, splitK, splitSize, reduceM, reduceK, reduceSize, rangeM, tailM,
        tailSplitSize, tailReduceSize;
};

namespace AscendC {

// impl/basic_api/common_types.h:27-50
enum class TPosition : uint8_t { GM, A1, A2, B1, B2, C1, C2, CO1, CO2, VECIN, VECOUT, VECCALC, LCM = VECCALC, SPM, SHM = SPM, TSCM, C2PIPE2GM, C2PIPE2LOCAL, MAX };
// impl/basic_api/utils/kernel_utils_mode.h:103-120,193-196
enum class RoundMode : uint8_t { CAST_NONE = 0, CAST_RINT, CAST_FLOOR, CAST_CEIL, CAST_ROUND, CAST_TRUNC, CAST_ODD, CAST_HYBRID, CAST_EVEN, CAST_ZERO, UNKNOWN = 0xFF };
enum class DeQuantMode : uint8_t { DEQUANT_WITH_SINGLE_ROW = 0, DEQUANT_WITH_MULTI_ROW };

namespace detail {
template <class T> struct DTypeOf;
template <> struct DTypeOf<float> { static constexpr int value = ASCB200_F32; };
template <> struct DTypeOf<half> { static constexpr int value = ASCB200_F16; };
template <> struct DTypeOf<bfloat16_t> { static constexpr int value = ASCB200_BF16; };
template <> struct DTypeOf<int8_t> { static constexpr int value = ASCB200_S8; };
template <> struct DTypeOf<int32_t> { static constexpr int value = ASCB200_S32; };
template <> struct DTypeOf<fp4x2_e2m1_t> { static constexpr int value = ASCB200_FP4_E2M1; };
template <> struct DTypeOf<fp8_e4m3fn_t> { static constexpr int value = ASCB200_FP8_E4M3; };
template <> struct DTypeOf<fp8_e5m2_t> { static constexpr int value = ASCB200_FP8_E5M2; };

// First failing C-ABI code of the calling thread's operator calls (kernel-side APIs return void).
inline int& LastError()
{
    static thread_local int code = ASCB200_OK;
    return code;
}
inline void Latch(int code, const char* what)
{
    if (code != ASCB200_OK) {
        if (LastError() == ASCB200_OK) LastError() = code;
        std::fprintf(stderr, "[ascb200] %s failed: %d (%s)\n", what, code, ascb200_strerror(code));
    }
}
inline void*& CurrentStream()
{
    static thread_local void* stream = nullptr;
    return stream;
}
}  // namespace detail

inline int GetLastError() { return detail::LastError(); }
inline void ClearLastError() { detail::LastError() = ASCB200_OK; }
inline int64_t GetBlockIdx() { return 0; }
inline int64_t GetBlockNum() { return 1; }

// Non-owning view of device memory (include/basic_api/kernel_tensor.h:256-289).
template <class T>
class GlobalTensor {
public:
    using PrimType = T;
    void SetGlobalBuffer(T* buffer, uint64_t bufferSize)
    {
        ptr_ = buffer;
        size_ = bufferSize;
    }
    void SetGlobalBuffer(T* buffer) { ptr_ = buffer; }
    T* GetPhyAddr() const { return ptr_; }
    T* GetPhyAddr(uint64_t offset) const { return ptr_ + offset; }
    uint64_t GetSize() const { return size_; }
    GlobalTensor operator[](uint64_t offset) const
    {
        GlobalTensor t;
        t.ptr_ = ptr_ + offset;
        t.size_ = size_ > offset ? size_ - offset : 0;
        return t;
    }
    // Element access goes through a synchronous copy: meant for a few scalars (e.g. a group list), not for bulk data.
    T GetValue(uint64_t offset) const
    {
        T v{};
        detail::Latch(ascb200_memcpy_d2h(&v, ptr_ + offset, sizeof(T), detail::CurrentStream()), "GlobalTensor::GetValue");
        detail::Latch(ascb200_stream_sync(detail::CurrentStream()), "GlobalTensor::GetValue");
        return v;
    }
    void SetValue(uint64_t offset, T v)
    {
        detail::Latch(ascb200_memcpy_h2d(ptr_ + offset, &v, sizeof(T), detail::CurrentStream()), "GlobalTensor::SetValue");
        detail::Latch(ascb200_stream_sync(detail::CurrentStream()), "GlobalTensor::SetValue");
    }

private:
    T* ptr_ = nullptr;
    uint64_t size_ = 0;
};

// "Unified buffer" tensors of the reference are on-chip; here a LocalTensor is a view of device
// global memory that holds the whole operand of the operator call.
template <class T>
class LocalTensor {
public:
    using PrimType = T;
    LocalTensor() = default;
    LocalTensor(T* devicePtr, uint64_t size) : ptr_(devicePtr), size_(size) {}
    void SetAddr(T* devicePtr, uint64_t size)
    {
        ptr_ = devicePtr;
        size_ = size;
    }
    T* GetPhyAddr() const { return ptr_; }
    uint64_t GetSize() const { return size_; }
    LocalTensor operator[](uint64_t offset) const { return LocalTensor(ptr_ + offset, size_ > offset ? size_ - offset : 0); }
    template <class U>
    LocalTensor<U> ReinterpretCast() const
    {
        return LocalTensor<U>(reinterpret_cast<U*>(ptr_), size_ * sizeof(T) / sizeof(U));
    }

private:
    T* ptr_ = nullptr;
    uint64_t size_ = 0;
};

// Carries the CUDA stream the operators of this thread launch on (the reference's TPipe manages on-chip buffers).
class TPipe {
public:
    TPipe() { detail::CurrentStream() = nullptr; }
    explicit TPipe(void* cudaStream) : stream_(cudaStream) { detail::CurrentStream() = stream_; }
    ~TPipe() { Destroy(); }
    void* GetStream() const { return stream_; }
    void Destroy()
    {
        if (!destroyed_) {
            (void)ascb200_stream_sync(stream_);
            destroyed_ = true;
        }
    }

private:
    void* stream_ = nullptr;
    bool destroyed_ = false;
};

}  // namespace AscendC

inline uint8_t* GetSysWorkSpacePtr()
{
    static uint8_t dummy;  // the B200 kernels need no system workspace; non-null like a configured one
    return &dummy;
}

#include "adv_api_ops.h"
