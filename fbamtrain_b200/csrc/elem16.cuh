// The 16-bit element type of the kernels in this directory.  Every source file is compiled twice: as is (elements
// are bf16, library libfbam_kernels.so) and with -DFBAM_ELEM_FP16 (elements are IEEE half, library
// libfbam_kernels_fp16.so).  Both libraries export the same entry points; the Python side picks the library from
// the tensors' dtype.  Accumulation is fp32 in both.  Everything that depends on the element type goes through the
// names below: the types, the conversions, the type field of a tensor map, the operand-format field of the tcgen05
// instruction descriptor, and the type suffix in inline PTX.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#ifdef FBAM_ELEM_FP16
typedef __half elem_t;
typedef __half2 elem2_t;
#define ELEM_PTX "f16"
#define ELEM_TMAP CU_TENSOR_MAP_DATA_TYPE_FLOAT16
#define ELEM_IDESC_FORMAT 0u          // tcgen05 kind::f16 operand format: 0 = f16, 1 = bf16
#define ELEM_IS_FP16 1
__host__ __device__ __forceinline__ float e2f(elem_t x) { return __half2float(x); }
__host__ __device__ __forceinline__ elem_t f2e(float x) { return __float2half_rn(x); }
__host__ __device__ __forceinline__ elem2_t ff2e2(float a, float b) { return __floats2half2_rn(a, b); }
__host__ __device__ __forceinline__ elem2_t f22e2(float2 v) { return __float22half2_rn(v); }
__host__ __device__ __forceinline__ float2 e22ff(elem2_t v) { return __half22float2(v); }
#else
typedef __nv_bfloat16 elem_t;
typedef __nv_bfloat162 elem2_t;
#define ELEM_PTX "bf16"
#define ELEM_TMAP CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
#define ELEM_IDESC_FORMAT 1u
#define ELEM_IS_FP16 0
__host__ __device__ __forceinline__ float e2f(elem_t x) { return __bfloat162float(x); }
__host__ __device__ __forceinline__ elem_t f2e(float x) { return __float2bfloat16(x); }
__host__ __device__ __forceinline__ elem2_t ff2e2(float a, float b) { return __floats2bfloat162_rn(a, b); }
__host__ __device__ __forceinline__ elem2_t f22e2(float2 v) { return __float22bfloat162_rn(v); }
__host__ __device__ __forceinline__ float2 e22ff(elem2_t v) { return __bfloat1622float2(v); }
#endif
