// fp32 CUDA-core kernels of the compressed-KV path.
//
// These carry the fp32 configuration (operators stored in fp32, where the
// reference runs true IEEE fp32 GEMMs and tensor cores have no matching
// mode) and the online C-means, whose centres are fp32 running means.  With
// `emulate_bf16` they reproduce the rounding points of the bf16 path, which
// the test-suite uses to cross-check the tensor-core kernels at full size.
#include "nkv_internal.h"

namespace nkv {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;
constexpr int THREADS = 256;

// acc[4][4] += A[64 x K] * B[64 x K]^T for the calling block's tile.
// loadA(m, k) / loadB(n, k) return the operand element (0 outside bounds).
// As / Bs: BK * (64 + PAD) floats each.
template <class FA, class FB>
__device__ __forceinline__ void gemm_tile(float (&acc)[4][4], int K, FA loadA, FB loadB,
                                          float* As, float* Bs) {
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int idx = tid + i * THREADS;
      int m = idx / BK, kk = idx % BK;
      int k = k0 + kk;
      As[kk * (BM + PAD) + m] = k < K ? loadA(m, k) : 0.f;
      Bs[kk * (BN + PAD) + m] = k < K ? loadB(m, k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk * (BM + PAD) + ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk * (BN + PAD) + tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
}

// squared norm of `rows` consecutive rows (<= 64) into out[0..64), 4 threads per row
__device__ __forceinline__ void row_sqnorms(const void* base, int dtype, int first, int count,
                                            int total, int J, float* out) {
  const int tid = threadIdx.x, row = tid >> 2, part = tid & 3;
  float sum = 0.f;
  if (row < count && first + row < total) {
    size_t off = static_cast<size_t>(first + row) * J;
    for (int j = part; j < J; j += 4) {
      float v = load_float(base, dtype, off + j);
      sum = fmaf(v, v, sum);
    }
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  if (part == 0) out[row] = sum;
}

// ---------------------------------------------------------------- assignment
__global__ void __launch_bounds__(THREADS)
assign_kernel(const void* x, int x_dtype, const void* centers, int c_dtype, int S, int J, int C,
              void* ids, int id_bytes, int32_t* labels32) {
  __shared__ float As[BK * (BM + PAD)], Bs[BK * (BN + PAD)];
  __shared__ float xn[BM], cn[BN];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int m0 = blockIdx.x * BM;
  row_sqnorms(x, x_dtype, m0, BM, S, J, xn);
  float best_d[4];
  int best_i[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { best_d[i] = INFINITY; best_i[i] = 0; }
  for (int n0 = 0; n0 < C; n0 += BN) {
    __syncthreads();
    row_sqnorms(centers, c_dtype, n0, BN, C, J, cn);
    float acc[4][4] = {};
    auto loadA = [&](int m, int k) {
      int t = m0 + m;
      return t < S ? load_float(x, x_dtype, static_cast<size_t>(t) * J + k) : 0.f;
    };
    auto loadB = [&](int n, int k) {
      int c = n0 + n;
      return c < C ? load_float(centers, c_dtype, static_cast<size_t>(c) * J + k) : 0.f;
    };
    gemm_tile(acc, J, loadA, loadB, As, Bs);  // ends with __syncthreads: xn / cn visible
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float d = INFINITY;
      int idx = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int c = n0 + tx * 4 + j;
        if (c < C) {
          // (||x||^2 + ||c||^2) - 2 x.c, in that association, in fp32
          float dist = __fsub_rn(__fadd_rn(xn[ty * 4 + i], cn[tx * 4 + j]),
                                 __fmul_rn(2.0f, acc[i][j]));
          if (dist < d) { d = dist; idx = c; }
        }
      }
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) {
        float od = __shfl_xor_sync(0xffffffffu, d, off);
        int oi = __shfl_xor_sync(0xffffffffu, idx, off);
        if (od < d || (od == d && oi < idx)) { d = od; idx = oi; }
      }
      if (d < best_d[i]) { best_d[i] = d; best_i[i] = idx; }
    }
  }
  if (tx == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int t = m0 + ty * 4 + i;
      if (t < S) {
        if (ids) {
          if (id_bytes == 1) static_cast<uint8_t*>(ids)[t] = static_cast<uint8_t>(best_i[i]);
          else static_cast<uint16_t*>(ids)[t] = static_cast<uint16_t>(best_i[i]);
        }
        if (labels32) labels32[t] = best_i[i];
      }
    }
  }
}

// ---------------------------------------------------------------- projection
template <bool BF16>
__global__ void __launch_bounds__(THREADS)
project_kernel(const void* x, int x_dtype, const uint16_t* centers, const void* ids, int id_bytes,
               const float* mean, const void* encoder, int S, int J, int r, void* coeff) {
  __shared__ float As[BK * (BM + PAD)], Bs[BK * (BN + PAD)];
  __shared__ int crow[BM];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  if (tid < BM) crow[tid] = (m0 + tid < S) ? load_id(ids, id_bytes, m0 + tid) : 0;
  __syncthreads();
  float acc[4][4] = {};
  auto loadA = [&](int m, int k) {
    int t = m0 + m;
    if (t >= S) return 0.f;
    float v = load_float(x, x_dtype, static_cast<size_t>(t) * J + k);
    float c = bf16_bits_to_float(centers[static_cast<size_t>(crow[m]) * J + k]);
    float res = __fsub_rn(__fsub_rn(v, c), mean[k]);
    return BF16 ? round_to_bf16(res) : res;
  };
  auto loadB = [&](int n, int k) {
    int c = n0 + n;
    return c < r ? load_float(encoder, BF16 ? NKV_BF16 : NKV_F32, static_cast<size_t>(c) * J + k)
                 : 0.f;
  };
  gemm_tile(acc, J, loadA, loadB, As, Bs);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int t = m0 + ty * 4 + i;
    if (t >= S) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int c = n0 + tx * 4 + j;
      if (c < r) store_float(coeff, BF16 ? NKV_BF16 : NKV_F32, static_cast<size_t>(t) * r + c,
                             acc[i][j]);
    }
  }
}

// -------------------------------------------------------------------- decode
template <bool BF16>
__global__ void __launch_bounds__(THREADS)
decode_rows_kernel(nkv_history h, const int32_t* rows_index, int n, const void* decoder,
                   const float* mean, int J, void* out, int out_dtype) {
  __shared__ float As[BK * (BM + PAD)], Bs[BK * (BN + PAD)];
  __shared__ int tok[BM], crow[BM];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  if (tid < BM) {
    int t = -1, row = 0;
    if (m0 + tid < n) {
      t = rows_index ? rows_index[m0 + tid] : m0 + tid;
      if (t < 0 || t >= h.tokens) t = -1; else row = center_row_of(h, t);
    }
    tok[tid] = t;
    crow[tid] = row;
  }
  __syncthreads();
  float acc[4][4] = {};
  auto loadA = [&](int m, int k) {
    int t = tok[m];
    if (t < 0) return 0.f;
    float v = latent_value(h, t, k);
    return BF16 ? round_to_bf16(v) : v;
  };
  auto loadB = [&](int nn, int k) {
    int c = n0 + nn;
    return c < J ? load_float(decoder, BF16 ? NKV_BF16 : NKV_F32,
                              static_cast<size_t>(c) * h.rank + k) : 0.f;
  };
  gemm_tile(acc, h.rank, loadA, loadB, As, Bs);
  const uint16_t* centers = static_cast<const uint16_t*>(h.centers);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = ty * 4 + i;
    if (m0 + m >= n || tok[m] < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int c = n0 + tx * 4 + j;
      if (c >= J) continue;
      float center = bf16_bits_to_float(centers[static_cast<size_t>(crow[m]) * h.center_width + c]);
      float v;
      if (BF16) {
        v = round_to_bf16(__fadd_rn(acc[i][j], round_to_bf16(mean[c])));
        v = round_to_bf16(__fadd_rn(v, center));
      } else {
        v = __fadd_rn(__fadd_rn(acc[i][j], mean[c]), center);
      }
      store_float(out, out_dtype, static_cast<size_t>(m0 + m) * J + c, v);
    }
  }
}

// ----------------------------------------------------------------- attention
// One block = 64 queries of one head; K/V tiles of 64 tokens are either read
// from memory (CODEC = false) or rebuilt from the compressed history into
// shared memory (CODEC = true).  Online softmax in fp32.
struct AttnArgs {
  const void* q; int dtype; int64_t q_stride_token, q_stride_head;
  int Q, heads, N; float scale;
  nkv_history hk, hv;
  const void* wk; const float* bias_k; const void* wv; const float* bias_v;
  const void* k_plain; const void* v_plain; int64_t kv_stride_token, kv_stride_head;
  void* out; float* lse;
  nkv_rope rope;   // cos_sin == nullptr: no positional restore
  nkv_camera cam_k, cam_v;   // matrices == nullptr: no camera transform
};

template <int DK, int DV, bool CODEC>
__global__ void __launch_bounds__(THREADS)
attn_kernel(AttnArgs a) {
  extern __shared__ float smem[];
  float* Qs = smem;                 // [DK][64]
  float* Ks = Qs + DK * 64;         // [DK][64]
  float* Vs = Ks + DK * 64;         // [64][DV]
  float* Ps = Vs + 64 * DV;         // [64][64]
  float* As = Ps + 64 * 64;         // staging for the decode GEMM
  float* Bs = As + BK * (BM + PAD);
  __shared__ int crow_k[64], crow_v[64];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int q0 = blockIdx.x * 64, head = blockIdx.y;
  const bool bf16 = a.dtype == NKV_BF16;
  for (int idx = tid; idx < 64 * DK; idx += THREADS) {
    int i = idx / DK, d = idx % DK;
    float v = 0.f;
    if (q0 + i < a.Q)
      v = load_float(a.q, a.dtype, static_cast<size_t>(q0 + i) * a.q_stride_token +
                                       static_cast<size_t>(head) * a.q_stride_head + d);
    Qs[d * 64 + i] = v;
  }
  constexpr int OC = DV / 16;
  float o[4][OC] = {};
  float m_run[4], l_run[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }

  for (int t0 = 0; t0 < a.N; t0 += 64) {
    __syncthreads();  // previous tile fully consumed (also orders the Qs fill)
    if (CODEC) {
      if (tid < 64) {
        int t = t0 + tid;
        crow_k[tid] = t < a.N ? center_row_of(a.hk, t) : 0;
        crow_v[tid] = t < a.N ? center_row_of(a.hv, t) : 0;
      }
      __syncthreads();
      // K and V tiles: [64 tok x D] = latent [64 x r] * W_head [D x r]^T, 64 columns at a time
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const nkv_history& h = which == 0 ? a.hk : a.hv;
        const void* w = which == 0 ? a.wk : a.wv;
        const float* bias = which == 0 ? a.bias_k : a.bias_v;
        const int* crow = which == 0 ? crow_k : crow_v;
        const int D = which == 0 ? DK : DV;
        const uint16_t* centers = static_cast<const uint16_t*>(h.centers);
        for (int n0 = 0; n0 < D; n0 += 64) {
          float acc[4][4] = {};
          auto loadA = [&](int m, int k) {
            int t = t0 + m;
            if (t >= a.N) return 0.f;
            float v = latent_value(h, t, k);
            return bf16 ? round_to_bf16(v) : v;
          };
          auto loadB = [&](int nn, int k) {
            int c = n0 + nn;
            return c < D ? load_float(w, a.dtype,
                                      (static_cast<size_t>(head) * D + c) * h.rank + k) : 0.f;
          };
          gemm_tile(acc, h.rank, loadA, loadB, As, Bs);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            int m = ty * 4 + i;
            float vals[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              int c = n0 + tx * 4 + j;
              float v = 0.f;
              if (c < D && t0 + m < a.N) {
                float center = bf16_bits_to_float(
                    centers[static_cast<size_t>(crow[m]) * h.center_width +
                            static_cast<size_t>(head) * D + c]);
                float b = bias[head * D + c];
                if (bf16) {
                  v = round_to_bf16(__fadd_rn(acc[i][j], b));
                  v = round_to_bf16(__fadd_rn(v, center));
                } else {
                  v = __fadd_rn(__fadd_rn(acc[i][j], b), center);
                }
              }
              vals[j] = v;
            }
            if (which == 0 && a.rope.cos_sin != nullptr && t0 + m < a.N) {
              // rotate the adjacent pairs (c, c+1) by the token's frame / row / column
              const int half = D / 2, th = a.rope.table_half, third = th / 3;
              const int band_a = th - 2 * third, band_b = band_a + third;
              const int pos = max(a.rope.positions[t0 + m], 0);
              int frame = pos, prow = pos, pcol = pos;   // frame_seqlen 0: one table row per token
              if (a.rope.frame_seqlen > 0) {
                frame = pos / a.rope.frame_seqlen;
                const int spatial = pos - frame * a.rope.frame_seqlen;
                prow = spatial / a.rope.width;
                pcol = spatial - prow * a.rope.width;
              }
#pragma unroll
              for (int pr = 0; pr < 2; ++pr) {
                const int pl = (n0 + tx * 4) / 2 + pr;
                if (pl >= half) continue;
                const int pg = a.rope.pair_index ? a.rope.pair_index[head * half + pl] : pl;
                int coord = pg < band_a ? frame : (pg < band_b ? prow : pcol);
                coord = min(coord, a.rope.table_rows - 1);
                const float2 cs = reinterpret_cast<const float2*>(a.rope.cos_sin)[static_cast<size_t>(coord) * th + pg];
                const float x0 = vals[2 * pr], x1 = vals[2 * pr + 1];
                float y0 = fmaf(x0, cs.x, -(x1 * cs.y)), y1 = fmaf(x0, cs.y, x1 * cs.x);
                vals[2 * pr] = bf16 ? round_to_bf16(y0) : y0;
                vals[2 * pr + 1] = bf16 ? round_to_bf16(y1) : y1;
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              int c = n0 + tx * 4 + j;
              if (c >= D) continue;
              if (which == 0) Ks[c * 64 + m] = vals[j]; else Vs[m * DV + c] = vals[j];
            }
          }
        }
      }
    } else {
      for (int idx = tid; idx < 64 * DK; idx += THREADS) {
        int j = idx / DK, d = idx % DK;
        float v = 0.f;
        if (t0 + j < a.N)
          v = load_float(a.k_plain, a.dtype, static_cast<size_t>(t0 + j) * a.kv_stride_token +
                                                 static_cast<size_t>(head) * a.kv_stride_head + d);
        Ks[d * 64 + j] = v;
      }
      for (int idx = tid; idx < 64 * DV; idx += THREADS) {
        int j = idx / DV, d = idx % DV;
        float v = 0.f;
        if (t0 + j < a.N)
          v = load_float(a.v_plain, a.dtype, static_cast<size_t>(t0 + j) * a.kv_stride_token +
                                                 static_cast<size_t>(head) * a.kv_stride_head + d);
        Vs[j * DV + d] = v;
      }
    }
    if (CODEC && (a.cam_k.matrices != nullptr || a.cam_v.matrices != nullptr)) {
      // camera transform of the finished tiles: thread = one (token, 8-wide block)
      __syncthreads();
      for (int which = 0; which < 2; ++which) {
        const nkv_camera& cam = which == 0 ? a.cam_k : a.cam_v;
        if (cam.matrices == nullptr) continue;
        const int D = which == 0 ? DK : DV;
        for (int idx = tid; idx < 64 * (D / 8); idx += THREADS) {
          const int m = idx % 64, g = idx / 64;
          if (t0 + m >= a.N) continue;
          const int frame = min((t0 + m) / cam.tokens_per_frame, cam.frames - 1);
          const float* mat = cam.matrices + (static_cast<size_t>(frame) * 4 + (cam.cam_index[head * (D / 8) + g] & 3)) * 16;
          float x[8], y[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) x[k] = which == 0 ? Ks[(g * 8 + k) * 64 + m] : Vs[m * DV + g * 8 + k];
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              float acc = 0.f;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float mij = bf16 ? round_to_bf16(mat[i * 4 + j]) : mat[i * 4 + j];
                acc = fmaf(mij, x[2 * j + r], acc);
              }
              y[2 * i + r] = bf16 ? round_to_bf16(acc) : acc;
            }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (which == 0) Ks[(g * 8 + k) * 64 + m] = y[k]; else Vs[m * DV + g * 8 + k] = y[k];
          }
        }
      }
    }
    __syncthreads();
    // S = Q K^T
    float s[4][4] = {};
#pragma unroll 8
    for (int d = 0; d < DK; ++d) {
      float qa[4], kb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qa[i] = Qs[d * 64 + ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) kb[j] = Ks[d * 64 + tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = fmaf(qa[i], kb[j], s[i][j]);
    }
    float alpha[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s[i][j] = (t0 + tx * 4 + j < a.N) ? s[i][j] * a.scale : -INFINITY;
        mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      float m_new = fmaxf(m_run[i], mx);  // finite: every processed tile has a valid token
      alpha[i] = expf(m_run[i] - m_new);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float p = expf(s[i][j] - m_new);
        Ps[(ty * 4 + i) * 64 + tx * 4 + j] = p;
        sum += p;
      }
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      l_run[i] = l_run[i] * alpha[i] + sum;
      m_run[i] = m_new;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < OC; ++c) o[i][c] *= alpha[i];
#pragma unroll 4
    for (int t = 0; t < 64; ++t) {
      float p[4], vv[OC];
#pragma unroll
      for (int i = 0; i < 4; ++i) p[i] = Ps[(ty * 4 + i) * 64 + t];
#pragma unroll
      for (int c = 0; c < OC; ++c) vv[c] = Vs[t * DV + tx + 16 * c];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < OC; ++c) o[i][c] = fmaf(p[i], vv[c], o[i][c]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int qi = q0 + ty * 4 + i;
    if (qi >= a.Q) continue;
    float inv = l_run[i] > 0.f ? 1.0f / l_run[i] : 0.f;
    size_t row = static_cast<size_t>(qi) * a.heads + head;
#pragma unroll
    for (int c = 0; c < OC; ++c)
      store_float(a.out, a.dtype, row * DV + tx + 16 * c, o[i][c] * inv);
    if (tx == 0) a.lse[row] = l_run[i] > 0.f ? m_run[i] + logf(l_run[i]) : -INFINITY;
  }
}

template <int DK, int DV, bool CODEC>
int launch_attn(const AttnArgs& a, cudaStream_t stream) {
  size_t smem = sizeof(float) * (2 * DK * 64 + 64 * DV + 64 * 64 + 2 * BK * (BM + PAD));
  auto kernel = attn_kernel<DK, DV, CODEC>;
  NKV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem)));
  dim3 grid(ceil_div(a.Q, 64), a.heads);
  kernel<<<grid, THREADS, smem, stream>>>(a);
  NKV_LAUNCH_CHECK("attn_kernel");
  return NKV_OK;
}

// -------------------------------------------------------------------- k-means
__global__ void gather_init_kernel(const void* x, int x_dtype, int J, const int32_t* init_rows,
                                   float* centers) {
  int c = blockIdx.x;
  size_t src = static_cast<size_t>(init_rows[c]) * J;
  for (int j = threadIdx.x; j < J; j += blockDim.x)
    centers[static_cast<size_t>(c) * J + j] = load_float(x, x_dtype, src + j);
}

// centre c, column j: sum of member rows in token order / member count;
// an empty cluster keeps its centre.
__global__ void __launch_bounds__(256)
kmeans_update_kernel(const void* x, int x_dtype, int S, int J, const int32_t* labels,
                     float* centers) {
  // Block (c, column block): the mean of the rows labelled c, summed in increasing token order (one
  // fp32 addition per row, the order a sequential scatter-add takes) so that the result does not
  // depend on the launch shape.  Labels are taken 2,048 at a time: every thread looks at eight of
  // them, a block-wide exclusive scan turns the match counts into positions, and the matching
  // tokens land in shared memory in order; the columns are then summed over that short list only,
  // four loads in flight at a time.
  __shared__ int list[2048];
  __shared__ int warp_total[8];
  const int c = blockIdx.x, j = blockIdx.y * 256 + threadIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float sum = 0.f;
  int count = 0;
  for (int s0 = 0; s0 < S; s0 += 2048) {
    const int len = min(2048, S - s0);
    int mine[8], n = 0;
    const int first = threadIdx.x * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int i = first + k;
      mine[k] = (i < len && __ldg(labels + s0 + i) == c) ? 1 : 0;
      n += mine[k];
    }
    int scan = n;                                           // inclusive scan inside the warp
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, scan, off);
      if (lane >= off) scan += v;
    }
    __syncthreads();                                        // the previous list has been consumed
    if (lane == 31) warp_total[warp] = scan;
    __syncthreads();
    int base = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < warp) base += warp_total[w];
      total += warp_total[w];
    }
    int at = base + scan - n;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (mine[k]) list[at++] = s0 + first + k;
    __syncthreads();
    count += total;
    if (j < J) {
      int i = 0;
      for (; i + 4 <= total; i += 4) {
        const float a = load_float(x, x_dtype, static_cast<size_t>(list[i]) * J + j);
        const float b = load_float(x, x_dtype, static_cast<size_t>(list[i + 1]) * J + j);
        const float d = load_float(x, x_dtype, static_cast<size_t>(list[i + 2]) * J + j);
        const float e = load_float(x, x_dtype, static_cast<size_t>(list[i + 3]) * J + j);
        sum = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(sum, a), b), d), e);
      }
      for (; i < total; ++i) sum = __fadd_rn(sum, load_float(x, x_dtype, static_cast<size_t>(list[i]) * J + j));
    }
  }
  if (j < J && count > 0) centers[static_cast<size_t>(c) * J + j] = __fdiv_rn(sum, static_cast<float>(count));
}

__global__ void kmeans_store_kernel(const float* centers, const int32_t* labels, int S, size_t CJ,
                                    uint16_t* centers_bf16, void* ids, int id_bytes) {
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < CJ) centers_bf16[i] = float_to_bf16_bits(centers[i]);
  if (i < static_cast<size_t>(S)) {
    if (id_bytes == 1) static_cast<uint8_t*>(ids)[i] = static_cast<uint8_t>(labels[i]);
    else static_cast<uint16_t*>(ids)[i] = static_cast<uint16_t>(labels[i]);
  }
}

}  // namespace

int simt_assign(const void* x, int x_dtype, const void* centers, int c_dtype, int S, int J,
                int C, void* ids, int id_bytes, int32_t* labels32, cudaStream_t stream) {
  if (S == 0) return NKV_OK;
  assign_kernel<<<ceil_div(S, BM), THREADS, 0, stream>>>(x, x_dtype, centers, c_dtype, S, J, C,
                                                        ids, id_bytes, labels32);
  NKV_LAUNCH_CHECK("assign_kernel");
  return NKV_OK;
}

int simt_project(const void* x, int x_dtype, const void* centers_bf16, const void* ids,
                 int id_bytes, const float* mean, const void* encoder, int enc_dtype, int S,
                 int J, int r, void* coeff, cudaStream_t stream) {
  if (S == 0) return NKV_OK;
  dim3 grid(ceil_div(S, BM), ceil_div(r, BN));
  const uint16_t* centers = static_cast<const uint16_t*>(centers_bf16);
  if (enc_dtype == NKV_BF16)
    project_kernel<true><<<grid, THREADS, 0, stream>>>(x, x_dtype, centers, ids, id_bytes, mean,
                                                       encoder, S, J, r, coeff);
  else
    project_kernel<false><<<grid, THREADS, 0, stream>>>(x, x_dtype, centers, ids, id_bytes, mean,
                                                        encoder, S, J, r, coeff);
  NKV_LAUNCH_CHECK("project_kernel");
  return NKV_OK;
}

int simt_decode_rows(const nkv_history& hist, const int32_t* rows_index, int n,
                     const void* decoder, int dec_dtype, const float* mean, int J, void* out,
                     int out_dtype, cudaStream_t stream) {
  if (n == 0) return NKV_OK;
  dim3 grid(ceil_div(n, BM), ceil_div(J, BN));
  if (dec_dtype == NKV_BF16)
    decode_rows_kernel<true><<<grid, THREADS, 0, stream>>>(hist, rows_index, n, decoder, mean, J,
                                                           out, out_dtype);
  else
    decode_rows_kernel<false><<<grid, THREADS, 0, stream>>>(hist, rows_index, n, decoder, mean, J,
                                                            out, out_dtype);
  NKV_LAUNCH_CHECK("decode_rows_kernel");
  return NKV_OK;
}

int simt_attn(const void* q, int dtype, int64_t q_stride_token, int64_t q_stride_head, int Q,
              int heads, int dk, int dv, const nkv_history* hist_k, const nkv_history* hist_v,
              const void* wk, const float* bias_k, const void* wv, const float* bias_v,
              const void* k_plain, const void* v_plain, int64_t kv_stride_token,
              int64_t kv_stride_head, int N, float scale, void* out, float* lse,
              cudaStream_t stream, const nkv_rope* rope, const nkv_camera* cam_k,
              const nkv_camera* cam_v) {
  if (Q == 0 || heads == 0) return NKV_OK;
  AttnArgs a{};
  if (rope != nullptr) a.rope = *rope;
  if (cam_k != nullptr) a.cam_k = *cam_k;
  if (cam_v != nullptr) a.cam_v = *cam_v;
  a.q = q; a.dtype = dtype; a.q_stride_token = q_stride_token; a.q_stride_head = q_stride_head;
  a.Q = Q; a.heads = heads; a.N = N; a.scale = scale;
  const bool codec = hist_k != nullptr;
  if (codec) { a.hk = *hist_k; a.hv = *hist_v; }
  a.wk = wk; a.bias_k = bias_k; a.wv = wv; a.bias_v = bias_v;
  a.k_plain = k_plain; a.v_plain = v_plain;
  a.kv_stride_token = kv_stride_token; a.kv_stride_head = kv_stride_head;
  a.out = out; a.lse = lse;
#define NKV_ATTN_CASE(DK_, DV_)                                            \
  if (dk == DK_ && dv == DV_)                                              \
    return codec ? launch_attn<DK_, DV_, true>(a, stream) : launch_attn<DK_, DV_, false>(a, stream);
  NKV_ATTN_CASE(128, 128)
  NKV_ATTN_CASE(64, 64)
  NKV_ATTN_CASE(32, 32)
  NKV_ATTN_CASE(16, 16)
#undef NKV_ATTN_CASE
  return fail(NKV_ERR_UNSUPPORTED, "attention head widths dk=%d dv=%d (built: 16, 32, 64, 128 with dk == dv)", dk, dv);
}

// camera transform of explicit rows: thread = one (row, head, 8-wide block)
__global__ void __launch_bounds__(256)
camera_rows_kernel(const void* x, int dtype, long long stride_row, long long stride_head, int S,
                   int heads, int d, nkv_camera cam, void* out) {
  const int blocks = d / 8;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(S) * heads * blocks) return;
  const int g = static_cast<int>(idx % blocks);
  const int head = static_cast<int>((idx / blocks) % heads);
  const int row = static_cast<int>(idx / (static_cast<long long>(blocks) * heads));
  const int frame = min(row / cam.tokens_per_frame, cam.frames - 1);
  const float* mat = cam.matrices + (static_cast<size_t>(frame) * 4 + (cam.cam_index[head * blocks + g] & 3)) * 16;
  const bool bf16 = dtype == NKV_BF16;
  const size_t src = static_cast<size_t>(row) * stride_row + static_cast<size_t>(head) * stride_head + g * 8;
  const size_t dst = (static_cast<size_t>(row) * heads + head) * d + g * 8;
  float v[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = load_float(x, dtype, src + k);
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        acc = fmaf(bf16 ? round_to_bf16(mat[i * 4 + j]) : mat[i * 4 + j], v[2 * j + r], acc);
      store_float(out, dtype, dst + 2 * i + r, acc);
    }
}

int camera_rows(const void* x, int dtype, int64_t stride_row, int64_t stride_head, int S, int heads,
                int d, const nkv_camera& camera, void* out, cudaStream_t stream) {
  const long long total = static_cast<long long>(S) * heads * (d / 8);
  if (total == 0) return NKV_OK;
  camera_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      x, dtype, stride_row, stride_head, S, heads, d, camera, out);
  NKV_LAUNCH_CHECK("camera_rows_kernel");
  return NKV_OK;
}

// rotation of explicit rows: thread = four adjacent pairs (8 elements) of one (row, head)
__global__ void __launch_bounds__(256)
rope_rows_kernel(const void* x, int dtype, long long stride_row, long long stride_head, int S,
                 int heads, int d, nkv_rope rope, void* out, int vector) {
  const int half = d / 2, quads = half / 4 + (half % 4 ? 1 : 0);
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(S) * heads * quads) return;
  const int pl0 = static_cast<int>(idx % quads) * 4;
  const int head = static_cast<int>((idx / quads) % heads);
  const int row = static_cast<int>(idx / (static_cast<long long>(quads) * heads));
  const int th = rope.table_half, third = th / 3, band_a = th - 2 * third, band_b = band_a + third;
  const int pos = max(rope.positions[row], 0);
  int frame = pos, prow = pos, pcol = pos;   // frame_seqlen 0: one table row per token
  if (rope.frame_seqlen > 0) {
    frame = pos / rope.frame_seqlen;
    const int spatial = pos - frame * rope.frame_seqlen;
    prow = spatial / rope.width;
    pcol = spatial - prow * rope.width;
  }
  const size_t src = static_cast<size_t>(row) * stride_row + static_cast<size_t>(head) * stride_head + 2 * pl0;
  const size_t dst = (static_cast<size_t>(row) * heads + head) * d + 2 * pl0;
  float v[8];
  const int count = min(4, half - pl0);
  if (vector && dtype == NKV_BF16) {
    const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + src);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[2 * k] = __uint_as_float(w[k] << 16);
      v[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
    }
  } else {
    for (int k = 0; k < 2 * count; ++k) v[k] = load_float(x, dtype, src + k);
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (k >= count) break;
    const int pl = pl0 + k;
    const int pg = rope.pair_index ? rope.pair_index[head * half + pl] : pl;
    int coord = pg < band_a ? frame : (pg < band_b ? prow : pcol);
    coord = min(coord, rope.table_rows - 1);
    const float2 cs = reinterpret_cast<const float2*>(rope.cos_sin)[static_cast<size_t>(coord) * th + pg];
    const float x0 = v[2 * k], x1 = v[2 * k + 1];
    v[2 * k] = fmaf(x0, cs.x, -(x1 * cs.y));
    v[2 * k + 1] = fmaf(x0, cs.y, x1 * cs.x);
  }
  if (vector && dtype == NKV_BF16) {
    uint4 packed;
    packed.x = float_to_bf16_bits(v[0]) | (static_cast<uint32_t>(float_to_bf16_bits(v[1])) << 16);
    packed.y = float_to_bf16_bits(v[2]) | (static_cast<uint32_t>(float_to_bf16_bits(v[3])) << 16);
    packed.z = float_to_bf16_bits(v[4]) | (static_cast<uint32_t>(float_to_bf16_bits(v[5])) << 16);
    packed.w = float_to_bf16_bits(v[6]) | (static_cast<uint32_t>(float_to_bf16_bits(v[7])) << 16);
    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(out) + dst) = packed;
  } else {
    for (int k = 0; k < 2 * count; ++k) store_float(out, dtype, dst + k, v[k]);
  }
}

int rope_rows(const void* x, int dtype, int64_t stride_row, int64_t stride_head, int S, int heads,
              int d, const nkv_rope& rope, void* out, cudaStream_t stream) {
  const int half = d / 2, quads = half / 4 + (half % 4 ? 1 : 0);
  const long long total = static_cast<long long>(S) * heads * quads;
  if (total == 0) return NKV_OK;
  // 16-byte path: whole groups of 8 elements, every row and head start 16-byte aligned
  const int vector = d % 8 == 0 && stride_row % 8 == 0 && stride_head % 8 == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  rope_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      x, dtype, stride_row, stride_head, S, heads, d, rope, out, vector);
  NKV_LAUNCH_CHECK("rope_rows_kernel");
  return NKV_OK;
}

int kmeans_gather_init(const void* x, int x_dtype, int J, int C, const int32_t* init_rows,
                       float* centers, cudaStream_t stream) {
  gather_init_kernel<<<C, 256, 0, stream>>>(x, x_dtype, J, init_rows, centers);
  NKV_LAUNCH_CHECK("gather_init_kernel");
  return NKV_OK;
}

int kmeans_update(const void* x, int x_dtype, int S, int J, int C, const int32_t* labels,
                  float* centers, cudaStream_t stream) {
  dim3 grid(C, ceil_div(J, 256));
  kmeans_update_kernel<<<grid, 256, 0, stream>>>(x, x_dtype, S, J, labels, centers);
  NKV_LAUNCH_CHECK("kmeans_update_kernel");
  return NKV_OK;
}

int kmeans_store(const float* centers, const int32_t* labels, int S, int J, int C,
                 void* centers_bf16, void* ids, int id_bytes, cudaStream_t stream) {
  size_t CJ = static_cast<size_t>(C) * J;
  size_t total = CJ > static_cast<size_t>(S) ? CJ : static_cast<size_t>(S);
  kmeans_store_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      centers, labels, S, CJ, static_cast<uint16_t*>(centers_bf16), ids, id_bytes);
  NKV_LAUNCH_CHECK("kmeans_store_kernel");
  return NKV_OK;
}

}  // namespace nkv
