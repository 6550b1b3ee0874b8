// Launchers shared between the translation units of libnanokv_b200.
#pragma once

#include "nkv_common.cuh"

namespace nkv {

// ---- fp32 CUDA-core kernels (nkv_simt.cu): the arithmetic of the fp32 path,
// and with emulate_bf16 the rounding points of the bf16 path (triage hook).
int simt_assign(const void* x, int x_dtype, const void* centers, int c_dtype, int S, int J,
                int C, void* ids, int id_bytes, int32_t* labels32, cudaStream_t stream);
int simt_project(const void* x, int x_dtype, const void* centers_bf16, const void* ids,
                 int id_bytes, const float* mean, const void* encoder, int enc_dtype, int S,
                 int J, int r, void* coeff, cudaStream_t stream);
int simt_decode_rows(const nkv_history& hist, const int32_t* rows_index, int n,
                     const void* decoder, int dec_dtype, const float* mean, int J, void* out,
                     int out_dtype, cudaStream_t stream);
int simt_attn(const void* q, int dtype, int64_t q_stride_token, int64_t q_stride_head, int Q,
              int heads, int dk, int dv, const nkv_history* hist_k, const nkv_history* hist_v,
              const void* wk, const float* bias_k, const void* wv, const float* bias_v,
              const void* k_plain, const void* v_plain, int64_t kv_stride_token,
              int64_t kv_stride_head, int N, float scale, void* out, float* lse,
              cudaStream_t stream, const nkv_rope* rope = nullptr, const nkv_camera* cam_k = nullptr,
              const nkv_camera* cam_v = nullptr);
int camera_rows(const void* x, int dtype, int64_t stride_row, int64_t stride_head, int S, int heads,
                int d, const nkv_camera& camera, void* out, cudaStream_t stream);
int rope_rows(const void* x, int dtype, int64_t stride_row, int64_t stride_head, int S, int heads,
              int d, const nkv_rope& rope, void* out, cudaStream_t stream);
int kmeans_gather_init(const void* x, int x_dtype, int J, int C, const int32_t* init_rows,
                       float* centers, cudaStream_t stream);
int kmeans_update(const void* x, int x_dtype, int S, int J, int C, const int32_t* labels,
                  float* centers, cudaStream_t stream);
int kmeans_store(const float* centers, const int32_t* labels, int S, int J, int C,
                 void* centers_bf16, void* ids, int id_bytes, cudaStream_t stream);

// ---- HBM-bound elementwise kernels (nkv_elementwise.cu)
int quant_pack(const void* coeff, int coeff_dtype, int S, int r, int group, float eps,
               int quant_mode, int scale_dtype, uint8_t* codes, void* scales,
               cudaStream_t stream);
int lse_merge(const void* const* outs, const float* const* lses, int parts, int64_t rows,
              int d, int dtype, void* out, float* lse_out, cudaStream_t stream);
int fast_finish(const void* native, const float* native_lse, const void* lifted, const float* low_lse,
                const int32_t* heads, const float* mean, const float* projected, int64_t rows,
                int total_heads, int group_heads, int d, int dtype, void* out, float* out_lse,
                cudaStream_t stream);
int head_linear(const void* x, int dtype, int64_t stride_row, int64_t stride_head, const int32_t* heads,
                const void* w, int64_t rows, int group_heads, int din, int dout, int dout_pad, void* out,
                cudaStream_t stream);
size_t history_moments_workspace_bytes(int tokens, int rank);
int history_moments(const nkv_history& h, float* latent_sum, int32_t* center_counts, void* workspace,
                    cudaStream_t stream);
int unpack_int8(const int8_t* q, const void* scale_bf16, int64_t rows, int cols, int group,
                void* out_bf16, cudaStream_t stream);
int cp_merge_peer(const void* const* part_out, const float* const* part_lse, void* const* dst_out,
                  float* const* dst_lse, int world, int64_t rows, int d, int64_t row_begin,
                  int64_t row_end, int dtype, cudaStream_t stream, int32_t* const* flags = nullptr,
                  int rank = 0, int epoch = 0, long long budget_cycles = 0, int32_t* status = nullptr);

// ---- tcgen05 / TMA kernels (nkv_tc_*.cu), bf16 operands, fp32 accumulation
int tc_assign(const void* x_bf16, const void* centers_bf16, int S, int J, int C, void* ids,
              int id_bytes, cudaStream_t stream);
int tc_project(const void* x_bf16, const void* centers_bf16, const void* ids, int id_bytes,
               const float* mean, const void* encoder_bf16, int S, int J, int r, void* coeff,
               cudaStream_t stream);
int tc_attn_codec(const void* q, int64_t q_stride_token, int64_t q_stride_head, int Q,
                  int heads, int dk, int dv, const nkv_history* hist_k,
                  const nkv_history* hist_v, const void* wk, const float* bias_k,
                  const void* wv, const float* bias_v, float scale, void* out, float* lse,
                  int32_t* status_word, int splits, void* workspace, cudaStream_t stream,
                  const nkv_rope* rope = nullptr, const nkv_camera* cam_k = nullptr,
                  const nkv_camera* cam_v = nullptr, bool prepared_weights = false);
int tc_prepare_decoder(const void* w_bf16, int64_t rows, int rank, void* out_bf16, cudaStream_t stream);
bool tc_attn_supported(int dk, int dv, int rank);
int tc_wait_expiry_selftest(int kind, long long budget_cycles, int32_t* status_word, cudaStream_t stream);
bool tc_project_supported(int J, int r);
bool tc_project_quant_supported(int J, int r, int group);
int tc_project_quant(const void* x_bf16, const void* centers_bf16, const void* ids, int id_bytes,
                     const float* mean, const void* encoder_bf16, int S, int J, int r, float eps,
                     int quant_mode, int scale_dtype, uint8_t* codes, void* scales, cudaStream_t stream);
bool tc_assign_supported(int J, int C);
size_t tc_assign_f32_workspace_bytes(int J, int C);
int tc_assign_f32(const void* x_bf16, const float* centers_f32, int S, int J, int C, int32_t* labels,
                  void* workspace, cudaStream_t stream);

}  // namespace nkv
