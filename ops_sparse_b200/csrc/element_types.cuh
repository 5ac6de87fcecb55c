/*
 * Element types of the narrow-storage products (fp16, bf16 and int8 matrices and dense operands), shared
 * by the SpMV and SpMM kernels.  The supported combinations are the reference's tables
 * (sparse/spmv/arch35/spmv_host.cpp:44-66, sparse/spmm/arch35/host/spmm_host.cpp:379-387) without the
 * complex rows.
 *
 * A product of two fp16, bf16 or int8 numbers is exact in fp32 (22, 16 and 14 significant bits) and in
 * fp64, so sums of them in fp64 carry no product error; a sum of int8 products is an exact integer below
 * 2^45.  Results are rounded once: alpha * sum + beta * old is formed in fp64 and converted to the output
 * type to nearest even (the reference rounds its fp32 accumulator the same way,
 * sparse/spmv/arch35/spmv_kernel.cpp:104-160); with the integer compute type the value
 * alpha * sum + beta * old is formed exactly in 128 bits and saturated to the int32 range, which is the
 * value the reference's case analysis produces (sparse/spmv/arch35/spmv_kernel.cpp:347-375).
 */
#ifndef ACLSPARSE_B200_ELEMENT_TYPES_CUH_
#define ACLSPARSE_B200_ELEMENT_TYPES_CUH_

#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "aclsparse_b200_kernels.h"

namespace aclsp {

constexpr int kF32 = static_cast<int>(ACLSP_TYPE_F32);
constexpr int kF16 = static_cast<int>(ACLSP_TYPE_F16);
constexpr int kBF16 = static_cast<int>(ACLSP_TYPE_BF16);
constexpr int kI8 = static_cast<int>(ACLSP_TYPE_I8);

// Element i of an array of the input type kIn, as fp32 (exact), through the read-only path.
template <int kIn>
__device__ __forceinline__ float LoadIn(const void* base, int64_t i)
{
    if constexpr (kIn == kF16) {
        return __half2float(__ldg(static_cast<const __half*>(base) + i));
    } else if constexpr (kIn == kBF16) {
        return __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(base) + i));
    } else if constexpr (kIn == kI8) {
        return static_cast<float>(__ldg(static_cast<const signed char*>(base) + i));
    } else {
        return __ldg(static_cast<const float*>(base) + i);
    }
}

// The scalars of a product in both forms; only one is used, by computeInt.
struct TypedScalars {
    double alpha;
    double beta;
    bool betaZero;
    long long alphaInt;
    long long betaInt;
};

__device__ __forceinline__ TypedScalars LoadTypedScalars(uint32_t computeInt, const void* alphaPtr, const void* betaPtr,
                                                         float alpha, float beta, int32_t alphaInt, int32_t betaInt)
{
    TypedScalars s;
    if (computeInt != 0) {
        s.alphaInt = alphaPtr != nullptr ? *static_cast<const int32_t*>(alphaPtr) : alphaInt;
        s.betaInt = betaPtr != nullptr ? *static_cast<const int32_t*>(betaPtr) : betaInt;
        s.alpha = static_cast<double>(s.alphaInt);
        s.beta = static_cast<double>(s.betaInt);
        s.betaZero = s.betaInt == 0;
        return s;
    }
    const float a = alphaPtr != nullptr ? *static_cast<const float*>(alphaPtr) : alpha;
    const float b = betaPtr != nullptr ? *static_cast<const float*>(betaPtr) : beta;
    s.alpha = static_cast<double>(a);
    s.beta = static_cast<double>(b);
    s.betaZero = b == 0.0f;
    s.alphaInt = 0;
    s.betaInt = 0;
    return s;
}

// out[at] = alpha * sum + beta * from[fromAt], both arrays of element type `type` (ACLSP_TYPE_*).
// beta == 0 does not read `from`.
__device__ __forceinline__ void StoreScaled(uint32_t type, void* out, int64_t at, const void* from, int64_t fromAt,
                                            double sum, const TypedScalars& s)
{
    if (type == ACLSP_TYPE_I32) {
        const long long old = s.betaZero ? 0 : static_cast<const int32_t*>(from)[fromAt];
        __int128 r = static_cast<__int128>(s.alphaInt) * static_cast<long long>(sum) +
                     static_cast<__int128>(s.betaInt) * old;
        const __int128 hi = 2147483647;
        const __int128 lo = -hi - 1;
        r = r > hi ? hi : (r < lo ? lo : r);
        static_cast<int32_t*>(out)[at] = static_cast<int32_t>(r);
        return;
    }
    double r = s.alpha * sum;
    if (type == ACLSP_TYPE_F16) {
        if (!s.betaZero) {
            r += s.beta * static_cast<double>(__half2float(static_cast<const __half*>(from)[fromAt]));
        }
        static_cast<__half*>(out)[at] = __double2half(r);
    } else if (type == ACLSP_TYPE_BF16) {
        if (!s.betaZero) {
            r += s.beta * static_cast<double>(__bfloat162float(static_cast<const __nv_bfloat16*>(from)[fromAt]));
        }
        static_cast<__nv_bfloat16*>(out)[at] = __double2bfloat16(r);
    } else {
        if (!s.betaZero) {
            r += s.beta * static_cast<double>(static_cast<const float*>(from)[fromAt]);
        }
        static_cast<float*>(out)[at] = static_cast<float>(r);
    }
}

}  // namespace aclsp

#endif  // ACLSPARSE_B200_ELEMENT_TYPES_CUH_
