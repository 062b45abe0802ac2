// Shared helpers for the sm_100a kernels behind the C ABI in include/inquant_b200.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/inquant_b200.h"

namespace inq {

// Thread-local text of the last CUDA failure, exposed through inq_last_error().
char* last_error_buffer();
int fail_cuda(cudaError_t err, const char* where);

#define INQ_CUDA_CHECK(expr)                                        \
  do {                                                              \
    cudaError_t inq_err__ = (expr);                                 \
    if (inq_err__ != cudaSuccess) return inq::fail_cuda(inq_err__, #expr); \
  } while (0)

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ bool finite_f32(float v) { return (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u; }

// Destination of one output field for row (outer slot, inner index).
struct FieldRef {
  char* base;
  long long so, si;
  __host__ __device__ char* at(long long slot, long long h) const { return base + slot * so + h * si; }
};
inline FieldRef make_field(const inq_field_t& f) { return FieldRef{(char*)f.base, f.outer_stride, f.inner_stride}; }

struct InputRef {
  const void* x;
  long long n_outer, n_inner, s_outer, s_inner, s_token;
  int tokens, channels;
  const void* page_ids;
  int page_ids_i64;
  long long num_slots;
  // false for a page id outside the destination the caller described (the row is then skipped)
  __device__ bool slot_ok(long long slot) const { return num_slots <= 0 || (slot >= 0 && slot < num_slots); }
  __device__ long long slot(long long p) const {
    if (!page_ids) return p;
    return page_ids_i64 ? ((const long long*)page_ids)[p] : (long long)((const int*)page_ids)[p];
  }
};
inline InputRef make_input(const inq_input_t& in) {
  return InputRef{in.x, in.n_outer, in.n_inner, in.stride_outer, in.stride_inner, in.stride_token,
                  in.tokens, in.channels, in.page_ids, in.page_ids_i64, in.num_slots};
}
inline int dtype_size(int dtype) { return dtype == INQ_F32 ? 4 : 2; }
inline bool valid_dtype(int dtype) { return dtype == INQ_F32 || dtype == INQ_F16 || dtype == INQ_BF16; }

}  // namespace inq
