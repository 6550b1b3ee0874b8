// nkv_encode_append_static: the encoder entry point for callers that must not
// allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc where they call the
// encoder: a serving loop that has handed the whole device to its own pool
// and forbids allocations after start-up, or a plugin called from a context
// where an allocation could synchronise the device or fail under memory
// pressure halfway through a rollout.  nkv_encode_append needs scratch for
// the projected coefficients (S x r values) between its projection and its
// quantiser; here that scratch is a fixed array in the library's own device
// image, so the caller passes inputs and outputs only.
#include <mutex>

#include "nkv_internal.h"

namespace {

// Holds S * r coefficients of one call.  4 MiB covers the largest chunk the
// reference commits at once (1560 tokens) at rank 640 in fp32.
// Every GPU that loads the library keeps this array until the process exits.
static __device__ __align__(256) unsigned char g_coeff_scratch[NKV_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_mutex;
void* g_scratch_address[MAX_DEVICES] = {};

// In host code `g_coeff_scratch` is only a handle for the runtime, not a device
// address; the address a kernel can use comes from cudaGetSymbolAddress, asked
// once per device with that device current.
int scratch_for_current_device(void** address) {
  int device = 0;
  NKV_CUDA(cudaGetDevice(&device));
  NKV_REQUIRE(device >= 0 && device < MAX_DEVICES, NKV_ERR_UNSUPPORTED,
              "device ordinal %d beyond the %d this entry point tracks", device, MAX_DEVICES);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* resolved = nullptr;
    NKV_CUDA(cudaGetSymbolAddress(&resolved, g_coeff_scratch));
    NKV_REQUIRE(resolved != nullptr, NKV_ERR_CUDA, "static scratch has no device address");
    g_scratch_address[device] = resolved;
  }
  *address = g_scratch_address[device];
  return NKV_OK;
}

}  // namespace

extern "C" int nkv_encode_append_static(const void* x, int x_dtype, const void* centers_bf16, int C,
                                        const float* mean, const void* encoder, int encoder_dtype,
                                        int S, int J, int r, int group, float eps, int quant_mode,
                                        int scale_dtype, int id_bytes, int offset, uint8_t* codes,
                                        void* scales, void* ids, void* stream) {
  NKV_REQUIRE(S >= 0 && r > 0, NKV_ERR_INVALID, "encode_append_static: S=%d r=%d", S, r);
  NKV_REQUIRE(encoder_dtype == NKV_F32 || encoder_dtype == NKV_BF16, NKV_ERR_INVALID,
              "encode_append_static: encoder dtype");
  const size_t needed = static_cast<size_t>(S) * r * nkv::dtype_bytes(encoder_dtype);
  NKV_REQUIRE(needed <= NKV_STATIC_SCRATCH_BYTES, NKV_ERR_TOO_LARGE,
              "encode_append_static: %d tokens x rank %d need %zu bytes of coefficient scratch, "
              "the built-in array holds %d; split the chunk or use nkv_encode_append",
              S, r, needed, NKV_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != NKV_OK) return rc;
  // The projection overwrites every coefficient the quantiser will read, so the
  // previous call's contents never matter and nothing needs clearing.
  return nkv_encode_append(x, x_dtype, centers_bf16, C, mean, encoder, encoder_dtype, S, J, r,
                           group, eps, quant_mode, scale_dtype, id_bytes, offset, codes, scales,
                           ids, scratch, NKV_STATIC_SCRATCH_BYTES, stream);
}
