// HBM-bound kernels: INT4 quantise + pack (+ append) and the LSE merge.
#include "nkv_internal.h"

namespace nkv {
namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// One warp per (token, group).  Lane p owns coefficient pairs p, p+32, ... of
// the group, so each lane forms whole bytes.
template <bool IN_BF16>
__global__ void __launch_bounds__(256)
quant_pack_kernel(const void* coeff, int dtype, int S, int r, int group, float eps,
                  int scale_dtype, uint8_t* codes, void* scales) {
  const int lane = threadIdx.x & 31;
  const int groups = r / group;
  const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= static_cast<long long>(S) * groups) return;
  const int t = static_cast<int>(unit / groups), g = static_cast<int>(unit % groups);
  const size_t base = static_cast<size_t>(t) * r + static_cast<size_t>(g) * group;
  const int pairs = group >> 1;
  float amax = 0.f;
  for (int p = lane; p < pairs; p += 32) {
    amax = fmaxf(amax, fabsf(load_float(coeff, dtype, base + 2 * p)));
    amax = fmaxf(amax, fabsf(load_float(coeff, dtype, base + 2 * p + 1)));
  }
  amax = warp_max(amax);
  float scale;
  if (IN_BF16) scale = round_to_bf16(__fdiv_rn(fmaxf(amax, round_to_bf16(eps)), 7.0f));
  else scale = __fdiv_rn(fmaxf(amax, eps), 7.0f);
  uint8_t* dst = codes + (base >> 1);
  for (int p = lane; p < pairs; p += 32) {
    float q0 = __fdiv_rn(load_float(coeff, dtype, base + 2 * p), scale);
    float q1 = __fdiv_rn(load_float(coeff, dtype, base + 2 * p + 1), scale);
    if (IN_BF16) { q0 = round_to_bf16(q0); q1 = round_to_bf16(q1); }
    int c0 = static_cast<int>(fminf(fmaxf(rintf(q0), -7.f), 7.f)) + 7;
    int c1 = static_cast<int>(fminf(fmaxf(rintf(q1), -7.f), 7.f)) + 7;
    dst[p] = static_cast<uint8_t>(c0 | (c1 << 4));
  }
  if (lane == 0) store_float(scales, scale_dtype, static_cast<size_t>(t) * groups + g, scale);
}

constexpr int MAX_PARTS = 16;
struct MergeArgs {
  const void* outs[MAX_PARTS];
  const float* lses[MAX_PARTS];
};

__device__ __forceinline__ float logaddexp(float a, float b) {
  if (isinf(a) && a == b) return a;
  float m = fmaxf(a, b);
  return m + log1pf(expf(-fabsf(a - b)));
}

// thread = (row, 4 consecutive columns)
__global__ void __launch_bounds__(256)
lse_merge_kernel(MergeArgs args, int parts, long long rows, int d, int dtype, void* out,
                 float* lse_out) {
  const int per_row = d >> 2;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * per_row) return;
  const long long row = idx / per_row;
  const int col = static_cast<int>(idx % per_row) * 4;
  float lse = args.lses[0][row];
  for (int p = 1; p < parts; ++p) lse = logaddexp(lse, args.lses[p][row]);
  const float origin = isfinite(lse) ? lse : 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int p = 0; p < parts; ++p) {
    float w = expf(args.lses[p][row] - origin);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float v = __fmul_rn(load_float(args.outs[p], dtype, static_cast<size_t>(row) * d + col + c), w);
      acc[c] = p == 0 ? v : __fadd_rn(acc[c], v);
    }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) store_float(out, dtype, static_cast<size_t>(row) * d + col + c, acc[c]);
  if (col == 0) lse_out[row] = lse;
}

}  // namespace

int quant_pack(const void* coeff, int coeff_dtype, int S, int r, int group, float eps,
               int quant_mode, int scale_dtype, uint8_t* codes, void* scales,
               cudaStream_t stream) {
  if (S == 0) return NKV_OK;
  long long units = static_cast<long long>(S) * (r / group);
  unsigned blocks = static_cast<unsigned>((units + 7) / 8);
  if (quant_mode == NKV_QUANT_IN_BF16)
    quant_pack_kernel<true><<<blocks, 256, 0, stream>>>(coeff, coeff_dtype, S, r, group, eps,
                                                        scale_dtype, codes, scales);
  else
    quant_pack_kernel<false><<<blocks, 256, 0, stream>>>(coeff, coeff_dtype, S, r, group, eps,
                                                         scale_dtype, codes, scales);
  NKV_LAUNCH_CHECK("quant_pack_kernel");
  return NKV_OK;
}

int lse_merge(const void* const* outs, const float* const* lses, int parts, int64_t rows, int d,
              int dtype, void* out, float* lse_out, cudaStream_t stream) {
  NKV_REQUIRE(parts >= 1 && parts <= MAX_PARTS, NKV_ERR_TOO_LARGE,
              "lse merge takes 1..%d partitions, got %d", MAX_PARTS, parts);
  NKV_REQUIRE(d % 4 == 0, NKV_ERR_INVALID, "merge width %d must be a multiple of 4", d);
  if (rows == 0) return NKV_OK;
  MergeArgs args{};
  for (int p = 0; p < parts; ++p) { args.outs[p] = outs[p]; args.lses[p] = lses[p]; }
  long long total = rows * (d >> 2);
  lse_merge_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      args, parts, rows, d, dtype, out, lse_out);
  NKV_LAUNCH_CHECK("lse_merge_kernel");
  return NKV_OK;
}

}  // namespace nkv
