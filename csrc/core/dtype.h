// dtype.h - element sizes, names, and host-side arithmetic for every HcclDataType.
// The host simulator reduces fp16 / bf16 / fp8 by widening to float, applying the operator and
// narrowing with round-to-nearest-even, which is also what the CUDA kernels do per element.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

#include "hccl/hccl_types.h"

namespace hc {

inline uint32_t DtypeSize(HcclDataType t)
{
    switch (t) {
        case HCCL_DATA_TYPE_INT8: case HCCL_DATA_TYPE_UINT8: case HCCL_DATA_TYPE_HIF8:
        case HCCL_DATA_TYPE_FP8E4M3: case HCCL_DATA_TYPE_FP8E5M2: case HCCL_DATA_TYPE_FP8E8M0: return 1;
        case HCCL_DATA_TYPE_INT16: case HCCL_DATA_TYPE_UINT16: case HCCL_DATA_TYPE_FP16: case HCCL_DATA_TYPE_BFP16: return 2;
        case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_UINT32: case HCCL_DATA_TYPE_FP32: return 4;
        case HCCL_DATA_TYPE_INT64: case HCCL_DATA_TYPE_UINT64: case HCCL_DATA_TYPE_FP64: return 8;
        case HCCL_DATA_TYPE_INT128: return 16;
        default: return 0;
    }
}

inline const char *DtypeName(HcclDataType t)
{
    switch (t) {
        case HCCL_DATA_TYPE_INT8: return "int8"; case HCCL_DATA_TYPE_INT16: return "int16";
        case HCCL_DATA_TYPE_INT32: return "int32"; case HCCL_DATA_TYPE_FP16: return "fp16";
        case HCCL_DATA_TYPE_FP32: return "fp32"; case HCCL_DATA_TYPE_INT64: return "int64";
        case HCCL_DATA_TYPE_UINT64: return "uint64"; case HCCL_DATA_TYPE_UINT8: return "uint8";
        case HCCL_DATA_TYPE_UINT16: return "uint16"; case HCCL_DATA_TYPE_UINT32: return "uint32";
        case HCCL_DATA_TYPE_FP64: return "fp64"; case HCCL_DATA_TYPE_BFP16: return "bf16";
        case HCCL_DATA_TYPE_INT128: return "int128"; case HCCL_DATA_TYPE_HIF8: return "hif8";
        case HCCL_DATA_TYPE_FP8E4M3: return "fp8e4m3"; case HCCL_DATA_TYPE_FP8E5M2: return "fp8e5m2";
        case HCCL_DATA_TYPE_FP8E8M0: return "fp8e8m0"; default: return "invalid";
    }
}

// Reductions are defined for the arithmetic types; the opaque ones (int128, hif8, fp8*) only copy.
inline bool DtypeReducible(HcclDataType t)
{
    switch (t) {
        case HCCL_DATA_TYPE_INT8: case HCCL_DATA_TYPE_INT16: case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_INT64:
        case HCCL_DATA_TYPE_UINT8: case HCCL_DATA_TYPE_UINT16: case HCCL_DATA_TYPE_UINT32: case HCCL_DATA_TYPE_UINT64:
        case HCCL_DATA_TYPE_FP16: case HCCL_DATA_TYPE_BFP16: case HCCL_DATA_TYPE_FP32: case HCCL_DATA_TYPE_FP64:
            return true;
        default: return false;
    }
}

inline const char *ReduceOpName(HcclReduceOp op)
{
    switch (op) {
        case HCCL_REDUCE_SUM: return "sum"; case HCCL_REDUCE_PROD: return "prod";
        case HCCL_REDUCE_MAX: return "max"; case HCCL_REDUCE_MIN: return "min"; default: return "invalid";
    }
}

// ---- 16-bit float conversions (round to nearest even) ----
inline float Bf16ToFloat(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
inline uint16_t FloatToBf16(float f)
{
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
    uint32_t lsb = (u >> 16) & 1;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}
inline float HalfToFloat(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ff, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else { int e = -1; do { ++e; man <<= 1; } while (!(man & 0x400)); u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13); }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp + 112) << 23) | (man << 13);
    float f; memcpy(&f, &u, 4); return f;
}
inline uint16_t FloatToHalf(float f)
{
    uint32_t u; memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000; int32_t exp = (int32_t)((u >> 23) & 0xff) - 127 + 15; uint32_t man = u & 0x7fffff;
    if (((u >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00 | (man ? 0x200 : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7c00);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000; int shift = 14 - exp; uint32_t half = man >> shift; uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) ++half;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)exp << 10) | (man >> 13); uint32_t rem = man & 0x1fff;
    if (rem > 0x1000 || (rem == 0x1000 && (half & 1))) ++half;
    return (uint16_t)(sign | half);
}

template <typename T>
inline T ApplyOp(HcclReduceOp op, T a, T b)
{
    switch (op) {
        case HCCL_REDUCE_SUM: return (T)(a + b);
        case HCCL_REDUCE_PROD: return (T)(a * b);
        case HCCL_REDUCE_MAX: return a > b ? a : b;
        case HCCL_REDUCE_MIN: return a < b ? a : b;
        default: return a;
    }
}

// dst[i] = dst[i] op src[i] on the host.  Returns false for a type that cannot be reduced.
inline bool HostReduce(void *dst, const void *src, uint64_t count, HcclDataType t, HcclReduceOp op)
{
#define HC_RED_CASE(E, T)                                                                     \
    case E: { T *d = (T *)dst; const T *s = (const T *)src;                                  \
              for (uint64_t i = 0; i < count; ++i) { d[i] = ApplyOp<T>(op, d[i], s[i]); }                \
              return true; }
    switch (t) {
        HC_RED_CASE(HCCL_DATA_TYPE_INT8, int8_t) HC_RED_CASE(HCCL_DATA_TYPE_INT16, int16_t)
        HC_RED_CASE(HCCL_DATA_TYPE_INT32, int32_t) HC_RED_CASE(HCCL_DATA_TYPE_INT64, int64_t)
        HC_RED_CASE(HCCL_DATA_TYPE_UINT8, uint8_t) HC_RED_CASE(HCCL_DATA_TYPE_UINT16, uint16_t)
        HC_RED_CASE(HCCL_DATA_TYPE_UINT32, uint32_t) HC_RED_CASE(HCCL_DATA_TYPE_UINT64, uint64_t)
        HC_RED_CASE(HCCL_DATA_TYPE_FP32, float) HC_RED_CASE(HCCL_DATA_TYPE_FP64, double)
        case HCCL_DATA_TYPE_FP16: { uint16_t *d = (uint16_t *)dst; const uint16_t *s = (const uint16_t *)src;
            for (uint64_t i = 0; i < count; ++i) { d[i] = FloatToHalf(ApplyOp<float>(op, HalfToFloat(d[i]), HalfToFloat(s[i]))); }
            return true; }
        case HCCL_DATA_TYPE_BFP16: { uint16_t *d = (uint16_t *)dst; const uint16_t *s = (const uint16_t *)src;
            for (uint64_t i = 0; i < count; ++i) { d[i] = FloatToBf16(ApplyOp<float>(op, Bf16ToFloat(d[i]), Bf16ToFloat(s[i]))); }
            return true; }
        default: return false;
    }
#undef HC_RED_CASE
}

}  // namespace hc
