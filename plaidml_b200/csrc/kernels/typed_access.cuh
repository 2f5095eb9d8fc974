// Typed element access shared by the general kernels: tensors are addressed through an element-type code, values
// travel in one of a few compute classes (float, double, 64-bit integers).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "pmlb_kernels.h"

namespace pmlb {

template <class T>
__device__ __forceinline__ T load_as(const void* base, int dtype, long long i) {
  switch (dtype) {
    case PMLB_BOOL:
    case PMLB_U8: return static_cast<T>(static_cast<const uint8_t*>(base)[i]);
    case PMLB_I8: return static_cast<T>(static_cast<const int8_t*>(base)[i]);
    case PMLB_I16: return static_cast<T>(static_cast<const int16_t*>(base)[i]);
    case PMLB_U16: return static_cast<T>(static_cast<const uint16_t*>(base)[i]);
    case PMLB_I32: return static_cast<T>(static_cast<const int32_t*>(base)[i]);
    case PMLB_U32: return static_cast<T>(static_cast<const uint32_t*>(base)[i]);
    case PMLB_I64: return static_cast<T>(static_cast<const long long*>(base)[i]);
    case PMLB_U64: return static_cast<T>(static_cast<const unsigned long long*>(base)[i]);
    case PMLB_F16: return static_cast<T>(__half2float(static_cast<const __half*>(base)[i]));
    case PMLB_BF16:
      return static_cast<T>(__bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]));
    case PMLB_F32: return static_cast<T>(static_cast<const float*>(base)[i]);
    case PMLB_F64: return static_cast<T>(static_cast<const double*>(base)[i]);
    default: return T(0);
  }
}

// Float -> integer conversions saturate in CUDA; the reference's fptosi is undefined out
// of range, so any choice is conforming.
template <class T>
__device__ __forceinline__ void store_as(void* base, int dtype, long long i, T v) {
  switch (dtype) {
    case PMLB_BOOL: static_cast<uint8_t*>(base)[i] = (v != T(0)) ? 1 : 0; break;
    case PMLB_U8: static_cast<uint8_t*>(base)[i] = static_cast<uint8_t>(static_cast<long long>(v)); break;
    case PMLB_I8: static_cast<int8_t*>(base)[i] = static_cast<int8_t>(static_cast<long long>(v)); break;
    case PMLB_I16: static_cast<int16_t*>(base)[i] = static_cast<int16_t>(static_cast<long long>(v)); break;
    case PMLB_U16: static_cast<uint16_t*>(base)[i] = static_cast<uint16_t>(static_cast<long long>(v)); break;
    case PMLB_I32: static_cast<int32_t*>(base)[i] = static_cast<int32_t>(static_cast<long long>(v)); break;
    case PMLB_U32: static_cast<uint32_t*>(base)[i] = static_cast<uint32_t>(static_cast<long long>(v)); break;
    case PMLB_I64: static_cast<long long*>(base)[i] = static_cast<long long>(v); break;
    case PMLB_U64: static_cast<unsigned long long*>(base)[i] = static_cast<unsigned long long>(v); break;
    case PMLB_F16: static_cast<__half*>(base)[i] = __float2half_rn(static_cast<float>(v)); break;
    case PMLB_BF16: static_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(static_cast<float>(v)); break;
    case PMLB_F32: static_cast<float*>(base)[i] = static_cast<float>(v); break;
    case PMLB_F64: static_cast<double*>(base)[i] = static_cast<double>(v); break;
    default: break;
  }
}

__device__ __forceinline__ bool dtype_is_float(int dt) {
  return dt == PMLB_F16 || dt == PMLB_BF16 || dt == PMLB_F32 || dt == PMLB_F64;
}

// Rounds / wraps a value of the compute class to what the element type can hold.
template <class T>
__device__ __forceinline__ T narrow(T v, int dtype) {
  if constexpr (sizeof(T) == 4) {  // float class
    if (dtype == PMLB_F16) return __half2float(__float2half_rn(v));
    if (dtype == PMLB_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
  } else if constexpr (static_cast<T>(0.5) != T(0)) {  // double
    return v;
  } else {
    switch (dtype) {
      case PMLB_BOOL: return (v != 0) ? T(1) : T(0);
      case PMLB_I8: return static_cast<T>(static_cast<int8_t>(v));
      case PMLB_U8: return static_cast<T>(static_cast<uint8_t>(v));
      case PMLB_I16: return static_cast<T>(static_cast<int16_t>(v));
      case PMLB_U16: return static_cast<T>(static_cast<uint16_t>(v));
      case PMLB_I32: return static_cast<T>(static_cast<int32_t>(v));
      case PMLB_U32: return static_cast<T>(static_cast<uint32_t>(v));
      default: return v;
    }
  }
}

}  // namespace pmlb
