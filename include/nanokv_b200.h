/*
 * nanokv_b200 -- C ABI of the B200 (sm_100a) compressed-KV hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (a cudaStream_t passed as void*), enqueues its kernels on that stream and
 * returns NKV_OK or a negative status; nothing here allocates device memory
 * at call time (the scratch the library owns -- the fused read's staging ring,
 * the static encoder scratch -- is __device__ storage inside the library; only
 * nkv_peer_alloc allocates, by name), synchronises the device, or traps.
 * nkv_last_error() gives the detail text of the calling thread's last failure.
 *
 * "Reference" citations name the function of the NanoKV project that each
 * entry point replaces, by path inside that project:
 *   MGM/ = models/Matrix-Game-3.5/fast/diffsynth/models/
 *   MGC/ = models/Matrix-Game-3.5/fast/codec_native/
 *   LB/  = models/LingBot-World-2.0/fast/wan/modules/
 *   HY/  = models/HY-WorldPlay/fast/hyvideo/models/transformers/modules/
 *
 * Symbols: J = heads * head_dim (joint width), r = rank, C = centres of one
 * segment, G = quantisation group (G == r is the reference's per-token scale),
 * S = tokens encoded by a call, N = history tokens read, Q = query tokens.
 */
#ifndef NANOKV_B200_H
#define NANOKV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NKV_ABI_VERSION 1

/* status codes */
#define NKV_OK               0
#define NKV_ERR_INVALID     (-1)  /* bad shape / argument          -> ValueError   */
#define NKV_ERR_CUDA        (-2)  /* CUDA runtime reported an error -> RuntimeError */
#define NKV_ERR_UNSUPPORTED (-3)  /* shape outside the built kernels -> RuntimeError */
#define NKV_ERR_DEVICE_WAIT (-4)  /* a bounded device-side wait gave up             */
#define NKV_ERR_TOO_LARGE   (-5)  /* exceeds a stated fixed capacity                */

/* element types */
#define NKV_F32  0
#define NKV_BF16 1
#define NKV_F16  2

/* quantiser arithmetic (nkv_quant_pack / nkv_encode_append) */
#define NKV_QUANT_F32      0  /* upcast to fp32 first: LB/lingbot_v2_kv_codec.py:285-287, HY/kv_codecs.py:237-255 */
#define NKV_QUANT_IN_BF16  1  /* amax, /7 and z/scale rounded to bf16: MGM/nanokv_codec.py:349-350 with a bf16 operator */

const char* nkv_status_string(int status);
const char* nkv_last_error(void);
int nkv_version(void);

/*
 * One compressed history tensor (K or V of one layer), struct-of-arrays in
 * HBM.  Token t belongs to segment s with seg_start[s] <= t < seg_start[s+1];
 * its centre is row seg_center_row[s] + ids[t] of `centers`.
 * Reference payloads: MGM/nanokv_codec.py:352-365 (packed_codes, scale,
 * centers, ids per segment; segments concatenated by concat_values :600-609),
 * LB/lingbot_v2_kv_codec.py:288-297.
 */
typedef struct nkv_history {
  const uint8_t* codes;          /* [tokens, rank/2]  two INT4 per byte, even index in the low nibble */
  const void*    scales;         /* [tokens, rank/group]  bf16 or fp16 */
  const void*    ids;            /* [tokens]  uint8 or uint16 centre id inside the token's segment */
  const void*    centers;        /* [center_rows, center_width]  bf16, all segments' tables stacked */
  const int32_t* seg_start;      /* [segments + 1] device array of token offsets */
  const int32_t* seg_center_row; /* [segments]     device array of first centre row per segment */
  int32_t tokens;
  int32_t segments;
  int32_t rank;
  int32_t group;
  int32_t scale_dtype;           /* NKV_BF16 | NKV_F16 */
  int32_t id_bytes;              /* 1 | 2 */
  int32_t center_rows;
  int32_t center_width;          /* row pitch of `centers` in elements */
} nkv_history;

/*
 * Which kernels serve bf16 inputs, process-wide: the tcgen05 tensor-core kernels (default) or the
 * fp32 CUDA-core kernels run with the bf16 path's rounding points.  The second form is the
 * triage aid for a suspected tensor-core discrepancy (same arithmetic contract, independent
 * code) and is what the parity tests cross-check the tensor-core kernels against at sizes a CPU
 * oracle cannot reach; it is far slower.  No counterpart in the reference.
 */
#define NKV_PATH_TENSOR_CORES 0
#define NKV_PATH_CUDA_CORES   1
int nkv_set_bf16_path(int path);

/*
 * Self-test of the bounded device-side waits: launches one tiny kernel whose only thread waits
 * on (kind 0) a shared-memory barrier on which nobody arrives, or (kind 1) a global counter that
 * nobody advances.  After `budget_cycles` SM cycles (1 .. 2^28) the wait must give up, exactly as
 * the waits inside the fused read do after their budget of about a second; the wait-site code
 * (990 / 991) is then stored in *status_word (device int32, cleared by the caller) and the kernel
 * returns.  Nothing faults or hangs: this exercises the give-up path, not an error of the GPU.
 * No counterpart in the reference.
 */
int nkv_selftest_bounded_wait(int kind, long long budget_cycles, int32_t* status_word, void* stream);

/* ------------------------------------------------------------------ encode */

/*
 * ids[t] = argmin_c ||x[t] - centers[c]||^2 evaluated as
 * ||x||^2 + ||c||^2 - 2 x.c in fp32, lowest index on ties.
 * Reference: the assignment step of semantic_residual,
 * MGM/nanokv_codec.py:316-321, LB/lingbot_v2_kv_codec.py:226-230.
 * x [S,J] (f32|bf16), centers [C,J] (f32|bf16), ids [S] of id_bytes each.
 */
int nkv_assign(const void* x, int x_dtype, const void* centers, int centers_dtype,
               int S, int J, int C, void* ids, int id_bytes, void* stream);

/*
 * Online C-means over one chunk: `iters` rounds of assign + deterministic
 * centre update (empty clusters keep their centre); ids are those of the last
 * assignment; stored centres are rounded to bf16.
 * Reference: semantic_residual, MGM/nanokv_codec.py:302-330,
 * LB/lingbot_v2_kv_codec.py:210-239 (the seeded randperm that picks
 * init_rows stays on the host, as it does there).
 * workspace: nkv_kmeans_workspace_bytes(S, J, C) bytes of device scratch.
 */
size_t nkv_kmeans_workspace_bytes(int S, int J, int C);
int nkv_kmeans(const void* x, int x_dtype, int S, int J, int C, int iters,
               const int32_t* init_rows, void* centers_bf16, void* ids, int id_bytes,
               void* workspace, size_t workspace_bytes, void* stream);

/*
 * coeff[t] = ((x[t] - centers[ids[t]]) - mean) @ encoder^T.
 * bf16 encoder: the residual is formed in fp32, rounded to bf16, multiplied
 * with fp32 accumulation and stored as bf16; f32 encoder: fp32 throughout.
 * Reference: MGM/nanokv_codec.py:326-330,345-348 with _operator_linear
 * :134-141; LB/lingbot_v2_kv_codec.py:236-239,280 with _linear :102-106.
 * x [S,J], centers bf16 [C,J], mean f32 [J], encoder [r,J], coeff [S,r] in
 * the encoder's dtype.
 */
int nkv_project(const void* x, int x_dtype, const void* centers_bf16, const void* ids,
                int id_bytes, const float* mean, const void* encoder, int encoder_dtype,
                int S, int J, int r, void* coeff, void* stream);

/*
 * Per-group symmetric INT4: scale = max(amax, eps) / 7, code =
 * clamp(rint(z / scale), -7, 7) with round-half-even, bytes = (code+7) pairs
 * with the even coefficient in the low nibble; the stored scale is rounded
 * to scale_dtype after the codes were formed.
 * Reference: MGM/nanokv_codec.py:349-351 + _pack_int4 :282-292;
 * LB/lingbot_v2_kv_codec.py:285-287 + :242-247 (Triton twins
 * LB/lingbot_v2_kv_codec_triton.py:12-67); HY/kv_codecs.py:237-255.
 * coeff [S,r] (f32|bf16) -> codes [S,r/2], scales [S,r/group].
 * Writing at an offset into a history cache is the append (E5).
 */
int nkv_quant_pack(const void* coeff, int coeff_dtype, int S, int r, int group, float eps,
                   int quant_mode, int scale_dtype, uint8_t* codes, void* scales,
                   void* stream);

/*
 * Projection, quantiser and packing of one chunk whose centre ids are known (after nkv_kmeans or
 * nkv_assign): coeff = ((x - centre[id]) - mean) @ encoder^T rounded once to the encoder dtype, then
 * nkv_quant_pack of those coefficients, written to codes [S,r/2] and scales [S,r/group].
 * Reference: the second half of encode_tensor, MGM/nanokv_codec.py:345-351, LB/lingbot_v2_kv_codec.py:280-287.
 * With bf16 operands and one scale per token (group == r, r a multiple of 64 that tiles over at most
 * two column parts) one kernel does all of it: the coefficients stay in tensor memory, the per-token
 * maximum crosses the two column-half thread blocks through their shared memory, and `workspace`
 * is not touched.  Otherwise it runs nkv_project into `workspace` (S * r elements of the encoder
 * dtype) followed by nkv_quant_pack.  Same bytes either way.
 */
int nkv_project_quant(const void* x, int x_dtype, const void* centers_bf16, const void* ids, int id_bytes,
                      const float* mean, const void* encoder, int encoder_dtype, int S, int J, int r,
                      int group, float eps, int quant_mode, int scale_dtype, uint8_t* codes,
                      void* scales, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Whole encoder of one chunk against given (stored, bf16) centres: assign,
 * project, quantise, pack, and write codes / scales / ids at token `offset`
 * of the destination arrays (the append).
 * Reference: encode_tensor, MGM/nanokv_codec.py:334-365,
 * LB/lingbot_v2_kv_codec.py:256-297.
 * workspace: S * r elements of the encoder dtype (unused when nkv_project_quant's single-kernel
 * form applies).
 */
int nkv_encode_append(const void* x, int x_dtype, const void* centers_bf16, int C,
                      const float* mean, const void* encoder, int encoder_dtype,
                      int S, int J, int r, int group, float eps, int quant_mode,
                      int scale_dtype, int id_bytes, int offset,
                      uint8_t* codes, void* scales, void* ids,
                      void* workspace, size_t workspace_bytes, void* stream);

/*
 * nkv_encode_append without caller-provided scratch and without any device
 * allocation.  (No counterpart in the reference: its encoder allocates
 * temporaries freely through PyTorch.)
 * For hosts that may not allocate where they encode -- a server that gave the
 * whole GPU to its own memory pool at start-up, a plugin that must not risk a
 * synchronising or failing cudaMalloc in the middle of a rollout.  The
 * coefficient scratch (S * r values of the encoder dtype) lives in a fixed
 * array of NKV_STATIC_SCRATCH_BYTES inside the library's device image; every
 * GPU that loads the library holds that array until the process exits.
 * Limits and rules:
 *  - S * r * sizeof(encoder element) must not exceed NKV_STATIC_SCRATCH_BYTES,
 *    else NKV_ERR_TOO_LARGE (split the chunk, or use nkv_encode_append);
 *  - the first call on each device looks the array's address up
 *    (cudaGetSymbolAddress, with that device current); make that first call
 *    before any stream capture;
 *  - all calls on a device share the one array, so two calls whose kernels can
 *    overlap on the GPU (different streams) race: keep calls stream-ordered.
 *    Nothing has to be cleared between calls: each call overwrites every
 *    coefficient it later reads.
 * Arguments and results are those of nkv_encode_append.
 */
#define NKV_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
int nkv_encode_append_static(const void* x, int x_dtype, const void* centers_bf16, int C,
                             const float* mean, const void* encoder, int encoder_dtype,
                             int S, int J, int r, int group, float eps, int quant_mode,
                             int scale_dtype, int id_bytes, int offset,
                             uint8_t* codes, void* scales, void* ids, void* stream);

/* ------------------------------------------------------------------- decode */

/*
 * rows = latent @ decoder^T + mean, then + centre, for tokens
 * rows_index[0..n) (or 0..n when rows_index is NULL) of a history tensor.
 * bf16 decoder: latent = bf16(code * scale), bf16(acc + bf16(mean)), then the
 * bf16 centre is added and the sum rounded to bf16; f32 decoder: fp32.
 * Reference: decode_tensor MGM/nanokv_codec.py:369-390, _decode_method_segments
 * :393-455, LB/lingbot_v2_kv_codec.py:301-326,404-437 (row / slice forms).
 * decoder [J,r], mean f32 [J], out [n,J] (f32|bf16).
 */
int nkv_decode_rows(const nkv_history* hist, const int32_t* rows_index, int n,
                    const void* decoder, int decoder_dtype, const float* mean, int J,
                    void* out, int out_dtype, void* stream);

/* ---------------------------------------------------------------- attention */

/*
 * Fused codec-attention over a compressed history.  For every head h and
 * history token t the kernel rebuilds, on chip,
 *     K[t,h,:] = bf16( bf16(latent_k[t] @ wk[h]^T + bias_k[h]) + centers_k[row(t), h*dk : (h+1)*dk] )
 *     V[t,h,:] likewise with wv / bias_v / centers_v,
 * and computes O = softmax(q K^T * scale) V with an online softmax, returning
 * O and the natural-log LSE.  On the tensor-core path every K / V tile of 128 tokens is rebuilt ONCE
 * per head by producer thread blocks and handed to the blocks that attend it through a staging ring
 * the library owns (24 MiB of __device__ storage per GPU, reused tile after tile, so it stays in
 * L2): no K or V row of the history is stored in HBM as a tensor, and none outlives the launch.
 * Launches on one device are serialised on that ring (an event orders streams).  `status_word`
 * (int32 on the device, zeroed by the caller, mandatory) receives a site code if a bounded
 * device-side wait gave up or the score range guard tripped; the affected lse rows are NaN.
 * With wk / wv = the decoder viewed as [heads, head_dim, r] and bias = mean
 * this is the full-dimensional read (decode + attention); with reader
 * matrices and projected centre tables it is the NanoKV-Fast low-width read.
 * Reference: decode (above) + attention_lse MGC/core.py:45-72 /
 * LB/codec_native_attention.py:53-104; reader read MGC/core.py:168-200.
 * q [Q, heads, dk] with strides (elements); wk [heads, dk, r]; wv [heads, dv, r];
 * bias_k f32 [heads, dk]; bias_v f32 [heads, dv]; out [Q, heads, dv] in the
 * dtype of q; lse f32 [Q, heads].  dtype NKV_BF16 runs on tcgen05 tensor
 * cores; NKV_F32 is the fp32 CUDA-core path.  An empty history yields
 * (0, -inf).
 */
int nkv_attn_codec(const void* q, int dtype, int64_t q_stride_token, int64_t q_stride_head,
                   int Q, int heads, int dk, int dv,
                   const nkv_history* hist_k, const nkv_history* hist_v,
                   const void* wk, const float* bias_k, const void* wv, const float* bias_v,
                   float scale, void* out, float* lse, int32_t* status_word, void* stream);

/*
 * nkv_attn_codec with the history cut into AT MOST `splits` (1..16) contiguous runs of tiles that
 * are attended by separate groups of thread blocks of ONE launch (the library picks the count, up
 * to this bound, that fills the GPU's SMs for the given Q, heads and history); their partial
 * (O, lse) go to `workspace` (nkv_attn_codec_workspace_bytes(…, splits) bytes) and are merged by
 * log-sum-exp (the merge of MGC/core.py:33-42).  Results equal nkv_attn_codec up to the rounding of
 * the partials to the output dtype.  The fp32 path ignores `splits`.
 */
size_t nkv_attn_codec_workspace_bytes(int Q, int heads, int dv, int splits);
int nkv_attn_codec_split(const void* q, int dtype, int64_t q_stride_token, int64_t q_stride_head,
                         int Q, int heads, int dk, int dv,
                         const nkv_history* hist_k, const nkv_history* hist_v,
                         const void* wk, const float* bias_k, const void* wv, const float* bias_v,
                         float scale, void* out, float* lse, int32_t* status_word,
                         int splits, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Positional restore of the reconstructed keys inside the read: 3-D RoPE by
 * the absolute position of every history token.  A rolling cache is "sink +
 * recent", not one contiguous interval, so positions travel with the tokens.
 * position -> frame = pos / frame_seqlen, row = (pos % frame_seqlen) / width,
 * column = (pos % frame_seqlen) % width; of the head_dim/2 adjacent-element
 * pairs of a key row, the first half - 2*(half/3) are rotated by the table
 * row of the frame, the next half/3 by that of the row, the last half/3 by
 * that of the column (half = head_dim/2).  The reference multiplies in complex
 * float64 and rounds once to the key dtype; here the table holds f32 (cos, sin)
 * and the rotation runs in fp32 on the twice-rounded key, then rounds once.
 * Coordinates beyond table_rows - 1 are clamped.
 * Reference: rope_pre_key_by_positions
 * models/LingBot-World-2.0/fast/wan/modules/lingbot_v2_cache_runtime.py:19-76
 * (fused form codec_native_rope_triton.py:10-46); table rope_params
 * wan/modules/model.py:29-36, bands :426-430.
 */
typedef struct nkv_rope {
  const int32_t* positions;  /* [history tokens] absolute token positions (device) */
  const float* cos_sin;      /* [table_rows][table_half][2] (cos, sin) (device) */
  int32_t table_rows;
  int32_t frame_seqlen;      /* tokens per frame = height * width; 0: the table has one row per
                                token position (every band reads row `position`), the form in which
                                Matrix-Game hands its multipliers over (rope_selected
                                models/Matrix-Game-3.5/fast/codec_native/core.py:75-91) */
  int32_t width;
  int32_t table_half;        /* pairs per table row = native head_dim / 2; the bands are cut on it */
  const int32_t* pair_index; /* NULL: pair p of the key row is native pair p (table_half = dk/2).
                                Else [heads][dk/2]: the native pair each pair of a low-width row
                                retains (selected RoPE of the NanoKV-Fast readers, _rope_low /
                                _selected_multiplier wan/modules/codec_native_attention.py:416-438,
                                rope_selected codec_native_rope_triton.py:31-47) (device) */
} nkv_rope;

/*
 * nkv_attn_codec_split with the keys rotated as above before Q K^T (queries
 * arrive already rotated, as at the reference call site
 * wan/modules/codec_native_attention.py:713-716).  rope == NULL is
 * nkv_attn_codec_split.
 */
int nkv_attn_codec_rope(const void* q, int dtype, int64_t q_stride_token, int64_t q_stride_head,
                        int Q, int heads, int dk, int dv,
                        const nkv_history* hist_k, const nkv_history* hist_v,
                        const void* wk, const float* bias_k, const void* wv, const float* bias_v,
                        const nkv_rope* rope, float scale, void* out, float* lse,
                        int32_t* status_word, int splits, void* workspace, size_t workspace_bytes,
                        void* stream);

/*
 * PRoPE camera transform of the rebuilt rows (Matrix-Game / HY): a row is made of 8-wide blocks,
 * a block of four two-element slots; output slot i of a block is sum_j M[i][j] * input slot j,
 * with M = matrices[frame][camera] (4 x 4), camera = cam_index[head][block] (the native block id
 * modulo 4 for the blocks a low-width reader retains) and frame = token / tokens_per_frame
 * (equal-sized frames, clamped to frames - 1).  Operands are bf16 values (the matrices are
 * rounded to bf16 on load), fp32 accumulation, one rounding; it follows the rotation.
 * Reference: camera_selected models/Matrix-Game-3.5/fast/codec_native/core.py:110-137, fused
 * form codec_native/camera_kernel.py:9-80; call sites codec_native/mg35.py:321, :339-346.
 */
typedef struct nkv_camera {
  const float* matrices;     /* [frames][4][4][4] f32 (device) */
  const int32_t* cam_index;  /* [heads][head_dim / 8] camera 0..3 of every block (device) */
  int32_t frames;
  int32_t tokens_per_frame;
} nkv_camera;

/*
 * Decoder / reader rows in the order the tensor-core kernel expands a code word: within every
 * group of 8 latent columns, 0 2 4 6 1 3 5 7 (even elements are the low nibbles of four code
 * bytes, odd ones the high nibbles, so each bf16 pair comes from one byte permute).  Done once
 * per operator at load time, like the INT8 expansion; w [rows, rank] bf16 -> out [rows, rank].
 * The result is only valid as wk / wv of nkv_attn_codec_pos with NKV_WEIGHTS_KERNEL_ORDER and
 * dtype NKV_BF16.  No counterpart in the reference.
 */
#define NKV_WEIGHTS_NATURAL 0
#define NKV_WEIGHTS_KERNEL_ORDER 1
int nkv_decoder_prepare(const void* w_bf16, int64_t rows, int rank, void* out_bf16, void* stream);

/*
 * nkv_attn_codec_rope plus the camera transform of the rebuilt keys (camera_k) and values
 * (camera_v); any of rope / camera_k / camera_v may be NULL.  weight_order says whether wk / wv
 * are as stored (NKV_WEIGHTS_NATURAL) or came from nkv_decoder_prepare.
 */
int nkv_attn_codec_pos(const void* q, int dtype, int64_t q_stride_token, int64_t q_stride_head,
                       int Q, int heads, int dk, int dv,
                       const nkv_history* hist_k, const nkv_history* hist_v,
                       const void* wk, const float* bias_k, const void* wv, const float* bias_v,
                       int weight_order,
                       const nkv_rope* rope, const nkv_camera* camera_k, const nkv_camera* camera_v,
                       float scale, void* out, float* lse, int32_t* status_word, int splits,
                       void* workspace, size_t workspace_bytes, void* stream);

/* The camera transform applied to explicit rows x [S, heads, d] (reduced queries with P^T,
 * attention outputs with P): out [S, heads, d] contiguous, same dtype. */
int nkv_camera_rows(const void* x, int dtype, int64_t stride_row, int64_t stride_head, int S,
                    int heads, int d, const nkv_camera* camera, void* out, void* stream);

/*
 * The same rotation applied to explicit rows (queries, the current chunk's keys):
 * x [S, heads, d] with strides in elements -> out [S, heads, d] contiguous, same dtype;
 * rope->positions holds the S row positions.  fp32 arithmetic, one rounding.
 */
int nkv_rope_rows(const void* x, int dtype, int64_t stride_row, int64_t stride_head, int S, int heads,
                  int d, const nkv_rope* rope, void* out, void* stream);

/*
 * Plain attention with LSE over K / V rows that are already full width (the
 * protected / current-chunk partition): O = softmax(q K^T * scale) V.
 * Reference: attention_lse, MGC/core.py:45-72;
 * _attention_lse LB/codec_native_attention.py:53-104.
 * q [Q, heads, d], k [N, heads, d], v [N, heads, dv] (token-major, strides in
 * elements), out [Q, heads, dv], lse f32 [Q, heads].
 */
int nkv_attention_lse(const void* q, const void* k, const void* v, int dtype,
                      int64_t q_stride_token, int64_t q_stride_head,
                      int64_t kv_stride_token, int64_t kv_stride_head,
                      int Q, int N, int heads, int d, int dv, float scale,
                      void* out, float* lse, void* stream);

/*
 * P-way log-sum-exp merge of attention partials: lse = logsumexp_p lse_p,
 * O = sum_p O_p * exp(lse_p - lse) in fp32 with one final rounding; a row
 * whose partials are all empty (-inf) gives (0, -inf).
 * Reference: merge MGC/core.py:33-42, _merge LB/codec_native_attention.py:43-50,
 * LB/codec_native_merge_triton.py:7-18 (two-way; folded here over P).
 * outs: P pointers (host array) to [rows, d] tensors; lses: P pointers to
 * f32 [rows]; out [rows, d]; lse_out f32 [rows].
 */
int nkv_lse_merge(const void* const* outs, const float* const* lses, int parts,
                  int64_t rows, int d, int dtype, void* out, float* lse_out, void* stream);

/*
 * Context-parallel exchange over peer memory (one process per GPU on one
 * NVSwitch box).  The reference has no history-sharded mode -- its only
 * multi-GPU mode shards heads by all-to-all
 * (models/LingBot-World-2.0/fast/wan/distributed/util.py:20-30,
 * sequence_parallel.py:464-468) -- so these entry points have no counterpart there; the arithmetic is the
 * reference's two-way merge (MGC/core.py:33-42) folded over the ranks, the
 * same as nkv_lse_merge.
 *
 * nkv_peer_alloc: device buffer on the current device plus a 64-byte handle
 * another process of the box passes to nkv_peer_open to map the buffer
 * (peer access is enabled on first use).  nkv_peer_close unmaps, nkv_peer_free
 * releases the owner's buffer once every peer has closed it.
 *
 * nkv_cp_merge_peer: this rank merges rows [row_begin, row_end) of the
 * `world` partials (part_out[p]: [rows, d] of dtype, part_lse[p]: f32 [rows];
 * host arrays of device pointers, one per rank, peers' buffers as mapped by
 * nkv_peer_open) and stores the merged rows into every rank's dst_out[p] /
 * dst_lse[p].  Plain loads and stores only (no multicast).  The caller orders
 * the ranks: every partial complete before the call, every rank's call complete
 * before any result is read or any partial overwritten.
 */
#define NKV_PEER_HANDLE_BYTES 64
int nkv_peer_alloc(int64_t bytes, void** ptr, uint8_t* handle);
int nkv_peer_open(const uint8_t* handle, void** ptr);
int nkv_peer_close(void* ptr);
int nkv_peer_free(void* ptr);
int nkv_cp_merge_peer(const void* const* part_out, const float* const* part_lse,
                      void* const* dst_out, float* const* dst_lse, int world, int64_t rows,
                      int d, int64_t row_begin, int64_t row_end, int dtype, void* stream);

/*
 * nkv_cp_merge_peer with the ordering of the ranks inside the kernel, so that the exchange of a
 * layer is ONE launch per rank and no collective: every rank owns NKV_PEER_FLAG_WORDS int32 of
 * peer-visible memory, zero at the start (flags[p]: rank p's words as mapped on this rank).  The
 * kernel tells every rank that this rank's partial of `epoch` is complete (a release store at
 * system scope; the partial was written by earlier work of the same stream), waits until every rank
 * has said so here, merges and stores this rank's row slice into every rank's result, tells every
 * rank that the slice has landed and waits until all slices have landed here -- after which every
 * result row is in place and nobody still reads this rank's partial.  `epoch` counts the calls of a
 * communicator from 1 upwards, the same on every rank.  Waits are bounded by `budget_cycles` SM
 * cycles (<= 0: about a second); one that runs out stores its site (980: a partial never came,
 * 981: a slice never landed) in *status_word and ends the kernel -- NKV_ERR_DEVICE_WAIT for the host
 * that checks the word.  Plain loads and stores over peer mappings only (no multicast); the ranks'
 * kernels run on different GPUs.  No counterpart in the reference.
 */
#define NKV_PEER_FLAG_WORDS 64
int nkv_cp_exchange_peer(const void* const* part_out, const float* const* part_lse,
                         void* const* dst_out, float* const* dst_lse, int32_t* const* flags,
                         int world, int rank, int64_t rows, int d, int64_t row_begin,
                         int64_t row_end, int dtype, int epoch, long long budget_cycles,
                         int32_t* status_word, void* stream);

/*
 * INT8 operator storage -> resident bf16 weights, once at load time:
 *     out[r, c] = bf16( bf16(qweight[r, c]) * scale[r, c / group] )
 * the expression the reference evaluates before every projection
 * (_operator_linear MGM/nanokv_codec.py:134-152, _pack_operator :108-131,
 * unpack_int8_weight MGM/nanokv_codec_kernels.py:76-82; LingBot per-row form
 * _linear LB/lingbot_v2_kv_codec.py:104-108).  A B200 keeps every layer's
 * operators resident in bf16 (about 0.5 GB for 40 layers at H 40 x D 128,
 * rank 640), so the kernels read bf16 and nothing is dequantised per call.
 * qweight i8 [rows, cols]; scale bf16 [rows, cols / group]; cols % 16 == 0.
 */
int nkv_operator_unpack_int8(const int8_t* qweight, const void* scale_bf16, int64_t rows, int cols,
                             int group, void* out_bf16, void* stream);

/*
 * First moments of a compressed history, without decoding it:
 *   latent_sum[j]      = sum over tokens of the bf16 latent coefficient j (f32 [rank])
 *   center_counts[row] = tokens assigned to centre row `row` (i32 [center_rows])
 * from which the mean decoded value follows by linearity,
 *   mean V = decoder (latent_sum / n) + bf16(mean) + (counts^T centres) / n,
 * as the reference forms it for the value-mean residual of the NanoKV-Fast read
 * (_compressed_value_mean wan/modules/codec_native_attention.py:465-501).
 * Deterministic (fixed summation order).  workspace:
 * nkv_history_moments_workspace_bytes(tokens, rank) bytes.
 */
size_t nkv_history_moments_workspace_bytes(int tokens, int rank);
int nkv_history_moments(const nkv_history* hist, float* latent_sum, int32_t* center_counts,
                        void* workspace, size_t workspace_bytes, void* stream);

/*
 * The two small per-head linear maps of a reader group of the mixed-dimensional read:
 *     out[n, g, e] = sum_d x[n, head(g), d] * w[g, d, e],   head(g) = heads[g] (g when heads is NULL)
 * fp32 accumulation, one rounding to `dtype`; columns [dout, dout_pad) of out are zero.  With
 * w = q_reduce [h, D, d] and x the pre-positional queries [Q, H, D] this is the reduced query
 * (query MGC/core.py:164-166, LB/codec_native_attention.py:115-116), with w = lift [h, d, D] and x
 * the low-width attention output the lifted value (lift_value MGC/core.py:202-204,
 * LB/codec_native_attention.py:210-211).  x strides in elements; w [group_heads, din, dout] and
 * out [rows, group_heads, dout_pad] contiguous; dtype NKV_BF16 | NKV_F32 for x, w and out.
 */
int nkv_head_linear(const void* x, int dtype, int64_t stride_row, int64_t stride_head,
                    const int32_t* heads, const void* w, int64_t rows, int group_heads, int din,
                    int dout, int dout_pad, void* out, void* stream);

/*
 * Finish of the mixed-dimensional (NanoKV-Fast) read for one head group, one launch:
 * the value-mean correction, the log-sum-exp merge of the full-width partial with the
 * lifted low-width partial, and the scatter of the group's heads to their places
 * (finish wan/modules/codec_native_finish_triton.py:10-46, LingBot fast tree):
 *     l      = logaddexp(native_lse[n, head], low_lse[n, g]),  origin = l if finite else 0
 *     low    = (lifted[n, g, :] + value_mean[head, :]) - projected_mean[g, :]
 *     out[n, head, :] = native[n, head, :] * exp(native_lse - origin) + low * exp(low_lse - origin)
 * fp32 in this order, one rounding to `dtype`; head = heads[g].
 * native, out [rows, total_heads, d]; lifted [rows, group_heads, d] in `dtype` (NKV_BF16 /
 * NKV_F32); native_lse [rows, total_heads], low_lse [rows, group_heads] f32; heads i32
 * [group_heads]; value_mean f32 [total_heads, d] and projected_mean f32 [group_heads, d]
 * both NULL to skip the correction; out_lse f32 [rows, total_heads] or NULL.  out may alias
 * native (each element is read and written by the same thread).  d % 8 == 0.
 */
int nkv_fast_finish(const void* native, const float* native_lse, const void* lifted, const float* low_lse,
                    const int32_t* heads, const float* value_mean, const float* projected_mean,
                    int64_t rows, int total_heads, int group_heads, int d, int dtype, void* out,
                    float* out_lse, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NANOKV_B200_H */
