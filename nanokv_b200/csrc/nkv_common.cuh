// Shared host/device helpers of the nanokv_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nanokv_b200.h"

namespace nkv {

// ---- host-side status plumbing -------------------------------------------
int fail(int status, const char* fmt, ...);  // records the message, returns status

#define NKV_REQUIRE(cond, status, ...)                       \
  do {                                                       \
    if (!(cond)) return ::nkv::fail((status), __VA_ARGS__);  \
  } while (0)

#define NKV_CUDA(expr)                                                          \
  do {                                                                          \
    cudaError_t err__ = (expr);                                                 \
    if (err__ != cudaSuccess)                                                   \
      return ::nkv::fail(NKV_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(err__)); \
  } while (0)

#define NKV_LAUNCH_CHECK(name)                                                  \
  do {                                                                          \
    cudaError_t err__ = cudaGetLastError();                                     \
    if (err__ != cudaSuccess)                                                   \
      return ::nkv::fail(NKV_ERR_CUDA, "launch of %s: %s", name, cudaGetErrorString(err__)); \
  } while (0)

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline size_t dtype_bytes(int dtype) { return dtype == NKV_F32 ? 4 : 2; }

// test / triage hook: route bf16 work through the fp32 CUDA-core kernels.
bool simt_forced();

// ---- device helpers ---------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_float(uint16_t bits) {
  return __uint_as_float(static_cast<uint32_t>(bits) << 16);
}

__device__ __forceinline__ float round_to_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ uint16_t float_to_bf16_bits(float v) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// INT4 code (0..14, i.e. the signed code plus 7) of coefficient z for a group scale, with the
// reference's rounding points.  IN_BF16: the quotient is rounded to bf16 before rint (LingBot's
// form).  Otherwise rint(z / scale) in fp32, taken through the reciprocal: z * inv is within 2 ulp
// of the IEEE quotient, so the two can only round to different integers when z * inv lies within
// ~1e-6 of a half; exactly those values take the IEEE division.
template <bool IN_BF16>
__device__ __forceinline__ int quant_code(float z, float scale, float inv) {
  float q;
  if (IN_BF16) {
    q = round_to_bf16(__fdiv_rn(z, scale));
  } else {
    q = z * inv;
    if (fabsf(q - rintf(q)) > 0.49999f && fabsf(q) < 8.5f) q = __fdiv_rn(z, scale);
  }
  return static_cast<int>(fminf(fmaxf(rintf(q), -7.f), 7.f)) + 7;
}

// element i of an array of the given element type, as float (exact)
__device__ __forceinline__ float load_float(const void* base, int dtype, size_t i) {
  if (dtype == NKV_F32) return static_cast<const float*>(base)[i];
  uint16_t bits = static_cast<const uint16_t*>(base)[i];
  if (dtype == NKV_BF16) return bf16_bits_to_float(bits);
  return __half2float(__ushort_as_half(bits));
}

__device__ __forceinline__ void store_float(void* base, int dtype, size_t i, float v) {
  if (dtype == NKV_F32) {
    static_cast<float*>(base)[i] = v;
  } else if (dtype == NKV_BF16) {
    static_cast<uint16_t*>(base)[i] = float_to_bf16_bits(v);
  } else {
    static_cast<uint16_t*>(base)[i] = __half_as_ushort(__float2half_rn(v));
  }
}

__device__ __forceinline__ int load_id(const void* ids, int id_bytes, size_t t) {
  return id_bytes == 1 ? static_cast<const uint8_t*>(ids)[t]
                       : static_cast<const uint16_t*>(ids)[t];
}

// Segment of token t: largest s with seg_start[s] <= t (binary search).
__device__ __forceinline__ int find_segment(const int32_t* seg_start, int segments, int t) {
  int lo = 0, hi = segments - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (seg_start[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Row of the stacked centre table that token t was assigned to.
__device__ __forceinline__ int center_row_of(const nkv_history& h, int t) {
  int s = find_segment(h.seg_start, h.segments, t);
  return h.seg_center_row[s] + load_id(h.ids, h.id_bytes, t);
}

// latent coefficient j of token t: code * stored scale (exact in fp32).
__device__ __forceinline__ float latent_value(const nkv_history& h, int t, int j) {
  uint8_t byte = h.codes[static_cast<size_t>(t) * (h.rank >> 1) + (j >> 1)];
  int nibble = (j & 1) ? (byte >> 4) : (byte & 15);
  float scale = load_float(h.scales, h.scale_dtype,
                           static_cast<size_t>(t) * (h.rank / h.group) + j / h.group);
  return static_cast<float>(nibble - 7) * scale;
}

}  // namespace nkv
