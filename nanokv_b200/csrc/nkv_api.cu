// extern "C" surface of libnanokv_b200: argument checks and kernel dispatch.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "nkv_internal.h"
#include "nkv_tc.cuh"

namespace nkv {

static thread_local char g_error[512] = "";
static std::atomic<int> g_bf16_path{NKV_PATH_TENSOR_CORES};

int fail(int status, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return status;
}

bool simt_forced() { return g_bf16_path.load(std::memory_order_relaxed) == NKV_PATH_CUDA_CORES; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_tensor_map(CUtensorMap* map, int elem_bytes, const void* base, int rank,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      int swizzle_bytes) {
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult query;
    NKV_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query));
    NKV_REQUIRE(fn != nullptr && query == cudaDriverEntryPointSuccess, NKV_ERR_CUDA,
                "driver does not export cuTensorMapEncodeTiled");
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  NKV_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, NKV_ERR_INVALID,
              "TMA source %p is not 16-byte aligned", base);
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5], estrides[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estrides[i] = 1;
    if (i > 0) {
      NKV_REQUIRE(strides_bytes[i - 1] % 16 == 0, NKV_ERR_INVALID,
                  "TMA stride %llu is not a multiple of 16 bytes",
                  static_cast<unsigned long long>(strides_bytes[i - 1]));
      gstrides[i - 1] = strides_bytes[i - 1];
    }
  }
  CUresult rc = encode(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                       static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides, gbox,
                       estrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                       : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NKV_REQUIRE(rc == CUDA_SUCCESS, NKV_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d",
              static_cast<int>(rc));
  return NKV_OK;
}

static int check_history(const nkv_history* h, const char* name) {
  NKV_REQUIRE(h != nullptr, NKV_ERR_INVALID, "%s history is NULL", name);
  NKV_REQUIRE(h->tokens >= 0 && h->rank > 0 && h->rank % 2 == 0, NKV_ERR_INVALID,
              "%s history: tokens=%d rank=%d", name, h->tokens, h->rank);
  NKV_REQUIRE(h->group > 0 && h->rank % h->group == 0 && h->group % 2 == 0, NKV_ERR_INVALID,
              "%s history: group %d must be even and divide rank %d", name, h->group, h->rank);
  NKV_REQUIRE(h->scale_dtype == NKV_BF16 || h->scale_dtype == NKV_F16, NKV_ERR_INVALID,
              "%s history: scales must be bf16 or fp16", name);
  NKV_REQUIRE(h->id_bytes == 1 || h->id_bytes == 2, NKV_ERR_INVALID,
              "%s history: id_bytes must be 1 or 2", name);
  if (h->tokens > 0)
    NKV_REQUIRE(h->segments >= 1 && h->seg_start && h->seg_center_row && h->codes && h->scales &&
                    h->ids && h->centers,
                NKV_ERR_INVALID, "%s history: missing arrays or segment table", name);
  return NKV_OK;
}

}  // namespace nkv

using namespace nkv;

extern "C" {

const char* nkv_status_string(int status) {
  switch (status) {
    case NKV_OK: return "ok";
    case NKV_ERR_INVALID: return "invalid argument";
    case NKV_ERR_CUDA: return "CUDA error";
    case NKV_ERR_UNSUPPORTED: return "unsupported shape";
    case NKV_ERR_DEVICE_WAIT: return "device-side wait gave up";
    case NKV_ERR_TOO_LARGE: return "fixed capacity exceeded";
    default: return "unknown status";
  }
}

const char* nkv_last_error(void) { return g_error; }

int nkv_version(void) { return NKV_ABI_VERSION; }

int nkv_set_bf16_path(int path) {
  NKV_REQUIRE(path == NKV_PATH_TENSOR_CORES || path == NKV_PATH_CUDA_CORES, NKV_ERR_INVALID,
              "set_bf16_path: %d", path);
  g_bf16_path.store(path, std::memory_order_relaxed);
  return NKV_OK;
}

int nkv_selftest_bounded_wait(int kind, long long budget_cycles, int32_t* status_word, void* stream) {
  return tc_wait_expiry_selftest(kind, budget_cycles, status_word, static_cast<cudaStream_t>(stream));
}

int nkv_assign(const void* x, int x_dtype, const void* centers, int centers_dtype, int S, int J,
               int C, void* ids, int id_bytes, void* stream) {
  NKV_REQUIRE(S >= 0 && J > 0 && C > 0, NKV_ERR_INVALID, "assign: S=%d J=%d C=%d", S, J, C);
  NKV_REQUIRE(id_bytes == 1 || id_bytes == 2, NKV_ERR_INVALID, "assign: id_bytes=%d", id_bytes);
  NKV_REQUIRE(C <= (id_bytes == 1 ? 256 : 65536), NKV_ERR_INVALID,
              "assign: %d centres do not fit %d-byte ids", C, id_bytes);
  NKV_REQUIRE(x_dtype == NKV_F32 || x_dtype == NKV_BF16, NKV_ERR_INVALID, "assign: x dtype");
  NKV_REQUIRE(centers_dtype == NKV_F32 || centers_dtype == NKV_BF16, NKV_ERR_INVALID,
              "assign: centres dtype");
  auto s = static_cast<cudaStream_t>(stream);
  if (x_dtype == NKV_BF16 && centers_dtype == NKV_BF16 && !simt_forced() &&
      tc_assign_supported(J, C))
    return tc_assign(x, centers, S, J, C, ids, id_bytes, s);
  return simt_assign(x, x_dtype, centers, centers_dtype, S, J, C, ids, id_bytes, nullptr, s);
}

// fp32 centres, 32-bit labels, and (for the tensor-core assignment of bf16 rows) the centres' three
// bf16 planes with their squared norms
static size_t kmeans_planes_offset(int S, int J, int C) {
  const size_t head = sizeof(float) * static_cast<size_t>(C) * J + sizeof(int32_t) * static_cast<size_t>(S);
  return (head + 255) / 256 * 256;
}
size_t nkv_kmeans_workspace_bytes(int S, int J, int C) {
  return kmeans_planes_offset(S, J, C) + tc_assign_f32_workspace_bytes(J, C) + 256;
}

int nkv_kmeans(const void* x, int x_dtype, int S, int J, int C, int iters,
               const int32_t* init_rows, void* centers_bf16, void* ids, int id_bytes,
               void* workspace, size_t workspace_bytes, void* stream) {
  NKV_REQUIRE(S > 0 && J > 0 && C > 0 && C <= S, NKV_ERR_INVALID,
              "kmeans: clusters must be in [1, S]; got C=%d S=%d", C, S);
  NKV_REQUIRE(iters >= 0, NKV_ERR_INVALID, "kmeans: iters=%d", iters);
  NKV_REQUIRE(id_bytes == 1 || id_bytes == 2, NKV_ERR_INVALID, "kmeans: id_bytes=%d", id_bytes);
  NKV_REQUIRE(C <= (id_bytes == 1 ? 256 : 65536), NKV_ERR_INVALID,
              "kmeans: %d centres do not fit %d-byte ids", C, id_bytes);
  NKV_REQUIRE(workspace && workspace_bytes >= nkv_kmeans_workspace_bytes(S, J, C), NKV_ERR_INVALID,
              "kmeans: workspace of %zu bytes is too small", workspace_bytes);
  auto s = static_cast<cudaStream_t>(stream);
  float* centers = static_cast<float*>(workspace);
  int32_t* labels = reinterpret_cast<int32_t*>(centers + static_cast<size_t>(C) * J);
  int rc = kmeans_gather_init(x, x_dtype, J, C, init_rows, centers, s);
  if (rc != NKV_OK) return rc;
  NKV_CUDA(cudaMemsetAsync(labels, 0, sizeof(int32_t) * S, s));
  // bf16 rows: the assignment runs on the tensor cores against the fp32 centres split into bf16
  // planes (fp32-accurate distances); anything else on the fp32 CUDA-core kernel
  const bool planes = x_dtype == NKV_BF16 && !simt_forced() && tc_assign_supported(J, C) &&
                      (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  uint8_t* plane_space = static_cast<uint8_t*>(workspace) + kmeans_planes_offset(S, J, C);
  plane_space += (256 - (reinterpret_cast<uintptr_t>(plane_space) & 255)) & 255;
  for (int it = 0; it < iters; ++it) {
    rc = planes ? tc_assign_f32(x, centers, S, J, C, labels, plane_space, s)
                : simt_assign(x, x_dtype, centers, NKV_F32, S, J, C, nullptr, id_bytes, labels, s);
    if (rc != NKV_OK) return rc;
    rc = kmeans_update(x, x_dtype, S, J, C, labels, centers, s);
    if (rc != NKV_OK) return rc;
  }
  return kmeans_store(centers, labels, S, J, C, centers_bf16, ids, id_bytes, s);
}

int nkv_project(const void* x, int x_dtype, const void* centers_bf16, const void* ids,
                int id_bytes, const float* mean, const void* encoder, int encoder_dtype, int S,
                int J, int r, void* coeff, void* stream) {
  NKV_REQUIRE(S >= 0 && J > 0 && r > 0, NKV_ERR_INVALID, "project: S=%d J=%d r=%d", S, J, r);
  NKV_REQUIRE(encoder_dtype == NKV_F32 || encoder_dtype == NKV_BF16, NKV_ERR_INVALID,
              "project: encoder dtype");
  auto s = static_cast<cudaStream_t>(stream);
  if (encoder_dtype == NKV_BF16 && x_dtype == NKV_BF16 && !simt_forced() &&
      tc_project_supported(J, r))
    return tc_project(x, centers_bf16, ids, id_bytes, mean, encoder, S, J, r, coeff, s);
  return simt_project(x, x_dtype, centers_bf16, ids, id_bytes, mean, encoder, encoder_dtype, S, J,
                      r, coeff, s);
}

int nkv_quant_pack(const void* coeff, int coeff_dtype, int S, int r, int group, float eps,
                   int quant_mode, int scale_dtype, uint8_t* codes, void* scales, void* stream) {
  NKV_REQUIRE(S >= 0 && r > 0 && group > 0 && r % group == 0 && group % 2 == 0, NKV_ERR_INVALID,
              "quant_pack: S=%d r=%d group=%d (group must be even and divide r)", S, r, group);
  NKV_REQUIRE(coeff_dtype == NKV_F32 || coeff_dtype == NKV_BF16, NKV_ERR_INVALID,
              "quant_pack: coefficient dtype");
  NKV_REQUIRE(scale_dtype == NKV_BF16 || scale_dtype == NKV_F16, NKV_ERR_INVALID,
              "quant_pack: scale dtype");
  NKV_REQUIRE(quant_mode == NKV_QUANT_F32 || quant_mode == NKV_QUANT_IN_BF16, NKV_ERR_INVALID,
              "quant_pack: quant_mode=%d", quant_mode);
  NKV_REQUIRE(quant_mode != NKV_QUANT_IN_BF16 || coeff_dtype == NKV_BF16, NKV_ERR_INVALID,
              "quant_pack: NKV_QUANT_IN_BF16 needs bf16 coefficients");
  return quant_pack(coeff, coeff_dtype, S, r, group, eps, quant_mode, scale_dtype, codes, scales,
                    static_cast<cudaStream_t>(stream));
}

int nkv_project_quant(const void* x, int x_dtype, const void* centers_bf16, const void* ids, int id_bytes,
                      const float* mean, const void* encoder, int encoder_dtype, int S, int J, int r,
                      int group, float eps, int quant_mode, int scale_dtype, uint8_t* codes,
                      void* scales, void* workspace, size_t workspace_bytes, void* stream) {
  NKV_REQUIRE(S >= 0 && J > 0 && r > 0 && group > 0 && r % group == 0, NKV_ERR_INVALID,
              "project_quant: S=%d J=%d r=%d group=%d", S, J, r, group);
  NKV_REQUIRE(encoder_dtype == NKV_F32 || encoder_dtype == NKV_BF16, NKV_ERR_INVALID,
              "project_quant: encoder dtype");
  NKV_REQUIRE(scale_dtype == NKV_BF16 || scale_dtype == NKV_F16, NKV_ERR_INVALID,
              "project_quant: scale dtype");
  NKV_REQUIRE(quant_mode == NKV_QUANT_F32 || quant_mode == NKV_QUANT_IN_BF16, NKV_ERR_INVALID,
              "project_quant: quant_mode=%d", quant_mode);
  NKV_REQUIRE(quant_mode != NKV_QUANT_IN_BF16 || encoder_dtype == NKV_BF16, NKV_ERR_INVALID,
              "project_quant: NKV_QUANT_IN_BF16 needs bf16 coefficients");
  // bf16 operands with one scale per token: projection, quantiser and packing in one kernel, the
  // coefficients stay on chip
  if (encoder_dtype == NKV_BF16 && x_dtype == NKV_BF16 && !simt_forced() &&
      tc_project_quant_supported(J, r, group) && (reinterpret_cast<uintptr_t>(codes) & 15) == 0)
    return tc_project_quant(x, centers_bf16, ids, id_bytes, mean, encoder, S, J, r, eps, quant_mode,
                            scale_dtype, codes, scales, static_cast<cudaStream_t>(stream));
  NKV_REQUIRE(workspace && workspace_bytes >= static_cast<size_t>(S) * r * dtype_bytes(encoder_dtype),
              NKV_ERR_INVALID, "project_quant: workspace of %zu bytes is too small", workspace_bytes);
  int rc = nkv_project(x, x_dtype, centers_bf16, ids, id_bytes, mean, encoder, encoder_dtype, S, J, r,
                       workspace, stream);
  if (rc != NKV_OK) return rc;
  return nkv_quant_pack(workspace, encoder_dtype, S, r, group, eps, quant_mode, scale_dtype, codes,
                        scales, stream);
}

int nkv_encode_append(const void* x, int x_dtype, const void* centers_bf16, int C,
                      const float* mean, const void* encoder, int encoder_dtype, int S, int J,
                      int r, int group, float eps, int quant_mode, int scale_dtype, int id_bytes,
                      int offset, uint8_t* codes, void* scales, void* ids, void* workspace,
                      size_t workspace_bytes, void* stream) {
  NKV_REQUIRE(offset >= 0, NKV_ERR_INVALID, "encode_append: offset=%d", offset);
  NKV_REQUIRE(r > 0 && group > 0 && r % group == 0, NKV_ERR_INVALID,
              "encode_append: r=%d group=%d", r, group);
  NKV_REQUIRE(workspace && workspace_bytes >= static_cast<size_t>(S) * r * dtype_bytes(encoder_dtype),
              NKV_ERR_INVALID, "encode_append: workspace of %zu bytes is too small", workspace_bytes);
  void* ids_at = static_cast<uint8_t*>(ids) + static_cast<size_t>(offset) * id_bytes;
  uint8_t* codes_at = codes + static_cast<size_t>(offset) * (r / 2);
  void* scales_at = static_cast<uint8_t*>(scales) + static_cast<size_t>(offset) * (r / group) * 2;
  int rc = nkv_assign(x, x_dtype, centers_bf16, NKV_BF16, S, J, C, ids_at, id_bytes, stream);
  if (rc != NKV_OK) return rc;
  return nkv_project_quant(x, x_dtype, centers_bf16, ids_at, id_bytes, mean, encoder, encoder_dtype, S,
                           J, r, group, eps, quant_mode, scale_dtype, codes_at, scales_at, workspace,
                           workspace_bytes, stream);
}

int nkv_decode_rows(const nkv_history* hist, const int32_t* rows_index, int n,
                    const void* decoder, int decoder_dtype, const float* mean, int J, void* out,
                    int out_dtype, void* stream) {
  int rc = check_history(hist, "decode");
  if (rc != NKV_OK) return rc;
  NKV_REQUIRE(n >= 0 && J > 0, NKV_ERR_INVALID, "decode_rows: n=%d J=%d", n, J);
  NKV_REQUIRE(rows_index != nullptr || n <= hist->tokens, NKV_ERR_INVALID,
              "decode_rows: %d rows requested from %d tokens", n, hist->tokens);
  NKV_REQUIRE(decoder_dtype == NKV_F32 || decoder_dtype == NKV_BF16, NKV_ERR_INVALID,
              "decode_rows: decoder dtype");
  return simt_decode_rows(*hist, rows_index, n, decoder, decoder_dtype, mean, J, out, out_dtype,
                          static_cast<cudaStream_t>(stream));
}

size_t nkv_attn_codec_workspace_bytes(int Q, int heads, int dv, int splits) {
  if (splits <= 1) return 0;
  return static_cast<size_t>(splits) * Q * heads * (static_cast<size_t>(dv) * 2 + 4);
}

static int check_rope(const nkv_rope* rope, int d, int64_t rows) {
  NKV_REQUIRE(rope->cos_sin != nullptr && rope->table_rows > 0 &&
                  (rope->frame_seqlen == 0 ||
                   (rope->frame_seqlen > 0 && rope->width > 0 && rope->frame_seqlen % rope->width == 0)),
              NKV_ERR_INVALID, "rope: table_rows=%d frame_seqlen=%d width=%d", rope->table_rows,
              rope->frame_seqlen, rope->width);
  NKV_REQUIRE(rope->positions != nullptr || rows == 0, NKV_ERR_INVALID, "rope: positions are NULL");
  NKV_REQUIRE(d % 4 == 0 && (reinterpret_cast<uintptr_t>(rope->cos_sin) & 7) == 0, NKV_ERR_INVALID,
              "rope: head width %d / table alignment", d);
  NKV_REQUIRE(rope->table_half > 0 && (rope->pair_index != nullptr || rope->table_half == d / 2),
              NKV_ERR_INVALID, "rope: table_half=%d for head width %d without a pair index",
              rope->table_half, d);
  return NKV_OK;
}

int nkv_rope_rows(const void* x, int dtype, int64_t stride_row, int64_t stride_head, int S, int heads,
                  int d, const nkv_rope* rope, void* out, void* stream) {
  NKV_REQUIRE(x && out && rope && S >= 0 && heads >= 0 && d > 0 && d % 2 == 0, NKV_ERR_INVALID,
              "rope_rows: S=%d heads=%d d=%d", S, heads, d);
  NKV_REQUIRE(dtype == NKV_F32 || dtype == NKV_BF16, NKV_ERR_INVALID, "rope_rows: dtype");
  NKV_REQUIRE(d % 4 == 0, NKV_ERR_INVALID, "rope_rows: head width %d", d);
  int rc = check_rope(rope, d, S);
  if (rc != NKV_OK) return rc;
  return rope_rows(x, dtype, stride_row, stride_head, S, heads, d, *rope, out,
                   static_cast<cudaStream_t>(stream));
}

static int check_camera(const nkv_camera* cam, int d) {
  NKV_REQUIRE(cam->matrices != nullptr && cam->cam_index != nullptr && cam->frames > 0 &&
                  cam->tokens_per_frame > 0,
              NKV_ERR_INVALID, "camera: frames=%d tokens_per_frame=%d", cam->frames, cam->tokens_per_frame);
  NKV_REQUIRE(d % 8 == 0 && (reinterpret_cast<uintptr_t>(cam->matrices) & 15) == 0, NKV_ERR_INVALID,
              "camera: head width %d must be a multiple of 8 and the matrices 16-byte aligned", d);
  return NKV_OK;
}

int nkv_decoder_prepare(const void* w_bf16, int64_t rows, int rank, void* out_bf16, void* stream) {
  NKV_REQUIRE(w_bf16 && out_bf16 && rows >= 0 && rank > 0, NKV_ERR_INVALID,
              "decoder_prepare: rows=%lld rank=%d", static_cast<long long>(rows), rank);
  return tc_prepare_decoder(w_bf16, rows, rank, out_bf16, static_cast<cudaStream_t>(stream));
}

int nkv_camera_rows(const void* x, int dtype, int64_t stride_row, int64_t stride_head, int S,
                    int heads, int d, const nkv_camera* camera, void* out, void* stream) {
  NKV_REQUIRE(x && out && camera && S >= 0 && heads >= 0 && d > 0, NKV_ERR_INVALID,
              "camera_rows: S=%d heads=%d d=%d", S, heads, d);
  NKV_REQUIRE(dtype == NKV_F32 || dtype == NKV_BF16, NKV_ERR_INVALID, "camera_rows: dtype");
  int rc = check_camera(camera, d);
  if (rc != NKV_OK) return rc;
  return camera_rows(x, dtype, stride_row, stride_head, S, heads, d, *camera, out,
                     static_cast<cudaStream_t>(stream));
}

int nkv_attn_codec_rope(const void* q, int dtype, int64_t q_stride_token, int64_t q_stride_head,
                        int Q, int heads, int dk, int dv, const nkv_history* hist_k,
                        const nkv_history* hist_v, const void* wk, const float* bias_k,
                        const void* wv, const float* bias_v, const nkv_rope* rope, float scale,
                        void* out, float* lse, int32_t* status_word, int splits, void* workspace,
                        size_t workspace_bytes, void* stream) {
  return nkv_attn_codec_pos(q, dtype, q_stride_token, q_stride_head, Q, heads, dk, dv, hist_k, hist_v,
                            wk, bias_k, wv, bias_v, NKV_WEIGHTS_NATURAL, rope, nullptr, nullptr, scale,
                            out, lse, status_word, splits, workspace, workspace_bytes, stream);
}

int nkv_attn_codec_pos(const void* q, int dtype, int64_t q_stride_token, int64_t q_stride_head,
                       int Q, int heads, int dk, int dv, const nkv_history* hist_k,
                       const nkv_history* hist_v, const void* wk, const float* bias_k,
                       const void* wv, const float* bias_v, int weight_order, const nkv_rope* rope,
                       const nkv_camera* camera_k, const nkv_camera* camera_v, float scale,
                       void* out, float* lse, int32_t* status_word, int splits, void* workspace,
                       size_t workspace_bytes, void* stream) {
  int rc = check_history(hist_k, "K");
  if (rc != NKV_OK) return rc;
  rc = check_history(hist_v, "V");
  if (rc != NKV_OK) return rc;
  NKV_REQUIRE(hist_k->tokens == hist_v->tokens && hist_k->rank == hist_v->rank &&
                  hist_k->group == hist_v->group && hist_k->scale_dtype == hist_v->scale_dtype,
              NKV_ERR_INVALID, "K and V histories differ in tokens / rank / group / scale dtype");
  NKV_REQUIRE(dtype == NKV_F32 || dtype == NKV_BF16, NKV_ERR_INVALID, "attn_codec: dtype");
  NKV_REQUIRE(Q >= 0 && heads >= 0, NKV_ERR_INVALID, "attn_codec: Q=%d heads=%d", Q, heads);
  NKV_REQUIRE(splits >= 1 && splits <= 16, NKV_ERR_INVALID, "attn_codec: splits=%d (1..16)", splits);
  NKV_REQUIRE(workspace_bytes >= nkv_attn_codec_workspace_bytes(Q, heads, dv, splits),
              NKV_ERR_INVALID, "attn_codec: workspace of %zu bytes is too small for %d splits",
              workspace_bytes, splits);
  const bool prepared = weight_order == NKV_WEIGHTS_KERNEL_ORDER;
  NKV_REQUIRE(weight_order == NKV_WEIGHTS_NATURAL || prepared, NKV_ERR_INVALID,
              "attn_codec: weight_order=%d", weight_order);
  NKV_REQUIRE(!prepared || (dtype == NKV_BF16 && !simt_forced() && tc_attn_supported(dk, dv, hist_k->rank)),
              NKV_ERR_INVALID,
              "attn_codec: kernel-order weights are only valid on the bf16 tensor-core path");
  if (rope != nullptr) {
    rc = check_rope(rope, dk, hist_k->tokens);
    if (rc != NKV_OK) return rc;
  }
  if (camera_k != nullptr) {
    rc = check_camera(camera_k, dk);
    if (rc != NKV_OK) return rc;
  }
  if (camera_v != nullptr) {
    rc = check_camera(camera_v, dv);
    if (rc != NKV_OK) return rc;
  }
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == NKV_BF16 && !simt_forced())
    return tc_attn_codec(q, q_stride_token, q_stride_head, Q, heads, dk, dv, hist_k, hist_v, wk,
                         bias_k, wv, bias_v, scale, out, lse, status_word, splits, workspace, s,
                         rope, camera_k, camera_v, prepared);
  return simt_attn(q, dtype, q_stride_token, q_stride_head, Q, heads, dk, dv, hist_k, hist_v, wk,
                   bias_k, wv, bias_v, nullptr, nullptr, 0, 0, hist_k->tokens, scale, out, lse, s,
                   rope, camera_k, camera_v);
}

int nkv_attn_codec_split(const void* q, int dtype, int64_t q_stride_token, int64_t q_stride_head,
                         int Q, int heads, int dk, int dv, const nkv_history* hist_k,
                         const nkv_history* hist_v, const void* wk, const float* bias_k,
                         const void* wv, const float* bias_v, float scale, void* out, float* lse,
                         int32_t* status_word, int splits, void* workspace, size_t workspace_bytes,
                         void* stream) {
  return nkv_attn_codec_rope(q, dtype, q_stride_token, q_stride_head, Q, heads, dk, dv, hist_k,
                             hist_v, wk, bias_k, wv, bias_v, nullptr, scale, out, lse, status_word,
                             splits, workspace, workspace_bytes, stream);
}

int nkv_attn_codec(const void* q, int dtype, int64_t q_stride_token, int64_t q_stride_head, int Q,
                   int heads, int dk, int dv, const nkv_history* hist_k,
                   const nkv_history* hist_v, const void* wk, const float* bias_k, const void* wv,
                   const float* bias_v, float scale, void* out, float* lse, int32_t* status_word,
                   void* stream) {
  return nkv_attn_codec_split(q, dtype, q_stride_token, q_stride_head, Q, heads, dk, dv, hist_k,
                              hist_v, wk, bias_k, wv, bias_v, scale, out, lse, status_word, 1,
                              nullptr, 0, stream);
}

int nkv_attention_lse(const void* q, const void* k, const void* v, int dtype,
                      int64_t q_stride_token, int64_t q_stride_head, int64_t kv_stride_token,
                      int64_t kv_stride_head, int Q, int N, int heads, int d, int dv, float scale,
                      void* out, float* lse, void* stream) {
  NKV_REQUIRE(dtype == NKV_F32 || dtype == NKV_BF16, NKV_ERR_INVALID, "attention_lse: dtype");
  NKV_REQUIRE(Q >= 0 && N >= 0 && heads >= 0, NKV_ERR_INVALID, "attention_lse: Q=%d N=%d heads=%d",
              Q, N, heads);
  return simt_attn(q, dtype, q_stride_token, q_stride_head, Q, heads, d, dv, nullptr, nullptr,
                   nullptr, nullptr, nullptr, nullptr, k, v, kv_stride_token, kv_stride_head, N,
                   scale, out, lse, static_cast<cudaStream_t>(stream));
}

int nkv_lse_merge(const void* const* outs, const float* const* lses, int parts, int64_t rows,
                  int d, int dtype, void* out, float* lse_out, void* stream) {
  NKV_REQUIRE(outs && lses && rows >= 0 && d > 0, NKV_ERR_INVALID, "lse_merge: rows=%lld d=%d",
              static_cast<long long>(rows), d);
  NKV_REQUIRE(dtype == NKV_F32 || dtype == NKV_BF16, NKV_ERR_INVALID, "lse_merge: dtype");
  return lse_merge(outs, lses, parts, rows, d, dtype, out, lse_out,
                   static_cast<cudaStream_t>(stream));
}

int nkv_peer_alloc(int64_t bytes, void** ptr, uint8_t* handle) {
  NKV_REQUIRE(bytes > 0 && ptr && handle, NKV_ERR_INVALID, "peer_alloc: bytes=%lld",
              static_cast<long long>(bytes));
  static_assert(sizeof(cudaIpcMemHandle_t) == NKV_PEER_HANDLE_BYTES, "handle size");
  void* base = nullptr;
  NKV_CUDA(cudaMalloc(&base, static_cast<size_t>(bytes)));
  cudaIpcMemHandle_t ipc;
  cudaError_t err = cudaIpcGetMemHandle(&ipc, base);
  if (err != cudaSuccess) {
    cudaFree(base);
    return fail(NKV_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(err));
  }
  memcpy(handle, &ipc, sizeof(ipc));
  *ptr = base;
  return NKV_OK;
}

int nkv_peer_open(const uint8_t* handle, void** ptr) {
  NKV_REQUIRE(handle && ptr, NKV_ERR_INVALID, "peer_open: null argument");
  cudaIpcMemHandle_t ipc;
  memcpy(&ipc, handle, sizeof(ipc));
  void* mapped = nullptr;
  NKV_CUDA(cudaIpcOpenMemHandle(&mapped, ipc, cudaIpcMemLazyEnablePeerAccess));
  *ptr = mapped;
  return NKV_OK;
}

int nkv_peer_close(void* ptr) {
  NKV_REQUIRE(ptr, NKV_ERR_INVALID, "peer_close: null pointer");
  NKV_CUDA(cudaIpcCloseMemHandle(ptr));
  return NKV_OK;
}

int nkv_peer_free(void* ptr) {
  NKV_REQUIRE(ptr, NKV_ERR_INVALID, "peer_free: null pointer");
  NKV_CUDA(cudaFree(ptr));
  return NKV_OK;
}

int nkv_cp_merge_peer(const void* const* part_out, const float* const* part_lse,
                      void* const* dst_out, float* const* dst_lse, int world, int64_t rows,
                      int d, int64_t row_begin, int64_t row_end, int dtype, void* stream) {
  NKV_REQUIRE(part_out && part_lse && dst_out && dst_lse && rows >= 0 && d > 0, NKV_ERR_INVALID,
              "cp_merge_peer: rows=%lld d=%d", static_cast<long long>(rows), d);
  NKV_REQUIRE(dtype == NKV_F32 || dtype == NKV_BF16, NKV_ERR_INVALID, "cp_merge_peer: dtype");
  return cp_merge_peer(part_out, part_lse, dst_out, dst_lse, world, rows, d, row_begin, row_end,
                       dtype, static_cast<cudaStream_t>(stream));
}

int nkv_cp_exchange_peer(const void* const* part_out, const float* const* part_lse,
                         void* const* dst_out, float* const* dst_lse, int32_t* const* flags, int world,
                         int rank, int64_t rows, int d, int64_t row_begin, int64_t row_end, int dtype,
                         int epoch, long long budget_cycles, int32_t* status_word, void* stream) {
  NKV_REQUIRE(part_out && part_lse && dst_out && dst_lse && flags && rows >= 0 && d > 0, NKV_ERR_INVALID,
              "cp_exchange_peer: rows=%lld d=%d", static_cast<long long>(rows), d);
  NKV_REQUIRE(dtype == NKV_F32 || dtype == NKV_BF16, NKV_ERR_INVALID, "cp_exchange_peer: dtype");
  if (budget_cycles <= 0) budget_cycles = 1ll << 31;
  return cp_merge_peer(part_out, part_lse, dst_out, dst_lse, world, rows, d, row_begin, row_end, dtype,
                       static_cast<cudaStream_t>(stream), flags, rank, epoch, budget_cycles, status_word);
}

int nkv_operator_unpack_int8(const int8_t* qweight, const void* scale_bf16, int64_t rows, int cols,
                             int group, void* out_bf16, void* stream) {
  NKV_REQUIRE(qweight && scale_bf16 && out_bf16 && rows >= 0, NKV_ERR_INVALID,
              "operator_unpack_int8: null argument or rows=%lld", static_cast<long long>(rows));
  return unpack_int8(qweight, scale_bf16, rows, cols, group, out_bf16,
                     static_cast<cudaStream_t>(stream));
}

int nkv_head_linear(const void* x, int dtype, int64_t stride_row, int64_t stride_head,
                    const int32_t* heads, const void* w, int64_t rows, int group_heads, int din, int dout,
                    int dout_pad, void* out, void* stream) {
  NKV_REQUIRE(x && w && out && rows >= 0, NKV_ERR_INVALID, "head_linear: null argument or rows=%lld",
              static_cast<long long>(rows));
  return head_linear(x, dtype, stride_row, stride_head, heads, w, rows, group_heads, din, dout, dout_pad,
                     out, static_cast<cudaStream_t>(stream));
}

int nkv_fast_finish(const void* native, const float* native_lse, const void* lifted, const float* low_lse,
                    const int32_t* heads, const float* value_mean, const float* projected_mean,
                    int64_t rows, int total_heads, int group_heads, int d, int dtype, void* out,
                    float* out_lse, void* stream) {
  NKV_REQUIRE(native && native_lse && lifted && low_lse && heads && out && rows >= 0, NKV_ERR_INVALID,
              "fast_finish: null argument or rows=%lld", static_cast<long long>(rows));
  return fast_finish(native, native_lse, lifted, low_lse, heads, value_mean, projected_mean, rows,
                     total_heads, group_heads, d, dtype, out, out_lse, static_cast<cudaStream_t>(stream));
}

size_t nkv_history_moments_workspace_bytes(int tokens, int rank) {
  return history_moments_workspace_bytes(tokens, rank);
}

int nkv_history_moments(const nkv_history* hist, float* latent_sum, int32_t* center_counts,
                        void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_history(hist, "moments");
  if (rc != NKV_OK) return rc;
  NKV_REQUIRE(latent_sum && center_counts, NKV_ERR_INVALID, "history_moments: null output");
  NKV_REQUIRE(workspace_bytes >= history_moments_workspace_bytes(hist->tokens, hist->rank) &&
                  (workspace != nullptr || hist->tokens == 0),
              NKV_ERR_INVALID, "history_moments: workspace of %zu bytes is too small", workspace_bytes);
  return history_moments(*hist, latent_sum, center_counts, workspace,
                         static_cast<cudaStream_t>(stream));
}

}  // extern "C"
