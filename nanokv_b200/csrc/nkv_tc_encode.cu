// Encoder GEMMs on tcgen05: nearest-centre assignment and residual projection.
//
// Both are [128 tokens x K=J] x [N x K]^T tiles with fp32 accumulators in TMEM,
// K streamed 64 columns at a time through a shared-memory ring of up to four stages.
//   assign : A = token rows (TMA), B = centre rows (TMA), N = C <= 512.  While
//            a stage is resident the compute warps accumulate ||x||^2 and
//            ||c||^2 from the same tiles; the epilogue evaluates
//            (||x||^2 + ||c||^2) - 2 x.c in fp32 and keeps the first minimum.
//   project: A = bf16((x - centre[id]) - mean), formed by the compute warps in
//            the swizzled operand layout; B = encoder rows (TMA); the epilogue
//            rounds once to bf16.
//   project + quantise: the same GEMM, but the epilogue keeps the coefficients in TMEM, takes the
//            token's absolute maximum over the whole rank row (the two column-half CTAs of a token
//            tile form a cluster and swap their half-row maxima through each other's shared
//            memory), quantises to INT4, packs two codes per byte and writes codes and scale to
//            their place in the history: the bf16 coefficients never travel to HBM.
// A CTA covers up to 512 output columns as 1 or 2 accumulators of NB <= 256.
// Warps 0-7 compute, warp 8 lane 0 issues TMA, warp 9 lane 0 issues MMA.
#include <atomic>

#include "nkv_internal.h"
#include "nkv_tc.cuh"

namespace nkv {
namespace {

using namespace tc;

constexpr int TM = 128;
constexpr int COMPUTE_THREADS = 256;
constexpr int THREADS = COMPUTE_THREADS + 64;
constexpr int A_BYTES = 128 * 128;

constexpr int MAX_STAGES = 4;
enum Bar { TMA_FULL = 0, A_FULL = 4, STAGE_FREE = 8, ACC_DONE = 12, SIDE_READY = 13, CAND_READY = 14,
           PEER_READY = 15, NUM_BARS = 16 };
enum Mode { PROJECT = 0, ASSIGN_IDS = 1, PROJECT_QUANT = 2 };
constexpr int META_HEAD = 256;      // barriers, TMEM slot, abort flag

struct Params {
  int S, J, NB, NACC, n_total;      // n_total = r (project) or C (assign)
  int nstages;                      // depth of the shared-memory operand ring (2..4)
  int rows;                         // tokens owned by one CTA (<= TM)
  // project
  const uint16_t* x; const uint16_t* centers; const void* ids; int id_bytes;
  const float* mean; uint16_t* coeff;
  // assign
  void* ids_out;
  int32_t* labels_out;              // optional 32-bit copy of the ids (the C-means update reads it)
  int a_chunks;                     // 64-column chunks of a token row; K runs over planes * a_chunks chunks
  const float* cnorm;               // squared norms of the centres when B holds bf16 planes of fp32 centres
  // project + quantise: codes u8 [S, r/2] and scales [S] at the history's token offset
  uint8_t* codes; void* scales; float eps; int in_bf16; int scale_dtype; int column_parts;
};

__device__ __forceinline__ float sumsq8(uint4 w) {
  const uint32_t words[4] = {w.x, w.y, w.z, w.w};
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float a = __uint_as_float(words[i] << 16), b = __uint_as_float(words[i] & 0xFFFF0000u);
    s = fmaf(a, a, s);
    s = fmaf(b, b, s);
  }
  return s;
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
encode_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                   const __grid_constant__ CUtensorMap map_b, Params p) {
  constexpr bool ASSIGN = MODE == ASSIGN_IDS;
  constexpr bool QUANT = MODE == PROJECT_QUANT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int b_bytes = p.NB * 128;                       // one accumulator's B tile
  const int stage_bytes = A_BYTES + p.NACC * b_bytes;
  const int nst = p.nstages;
  uint8_t* meta = smem + nst * stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(meta);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(meta + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(meta + NUM_BARS * 8 + 4);
  float* xn_part = reinterpret_cast<float*>(meta + META_HEAD);    // [128][2]
  float* cand_d = xn_part + 256;                                  // [128]
  int* cand_i = reinterpret_cast<int*>(cand_d + 128);             // [128]
  float* cn_part = reinterpret_cast<float*>(cand_i + 128);        // [C][2]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * p.rows;                   // this CTA's tokens: [m0, m_end)
  const int m_end = min(p.S, m0 + p.rows);
  const int n_base = blockIdx.y * p.NACC * p.NB;
  // assign against fp32 centres: B is the centres split into bf16 planes laid side by side along
  // K, A (the token rows) is walked once per plane
  const int nchunks = ASSIGN ? p.a_chunks * (p.cnorm != nullptr ? 3 : 1) : p.J / 64;

  if (tid == 0) {
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(&bars[TMA_FULL + s], 1);
      mbar_init(&bars[A_FULL + s], COMPUTE_THREADS);
      mbar_init(&bars[STAGE_FREE + s], ASSIGN ? 1 + COMPUTE_THREADS : 1);
    }
    mbar_init(&bars[ACC_DONE], 1);
    mbar_init(&bars[SIDE_READY], COMPUTE_THREADS);
    mbar_init(&bars[CAND_READY], 128);
    mbar_init(&bars[PEER_READY], 128);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 9) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // the column-half CTAs of one token tile write into each other's shared memory: nobody may do so
  // before the peer's barriers exist
  const bool paired = QUANT && p.column_parts == 2;
  if (paired) cluster_sync_all();

  if (warp == 8) {
    if (lane == 0) {
      prefetch_tensormap(&map_b);
      if (ASSIGN) prefetch_tensormap(&map_a);
      bool ok = true;
      for (int c = 0; c < nchunks && ok; ++c) {
        const int s = c % nst, u = c / nst;
        if (u >= 1) ok = mbar_wait(&bars[STAGE_FREE + s], (u - 1) & 1, abort_flag, 400 + s);
        if (!ok) break;
        uint8_t* stage = smem + s * stage_bytes;
        mbar_arrive_expect_tx(&bars[TMA_FULL + s], p.NACC * b_bytes + (ASSIGN ? A_BYTES : 0));
        if (ASSIGN) tma_load_2d(stage, &map_a, (c % p.a_chunks) * 64, m0, &bars[TMA_FULL + s]);
        for (int a = 0; a < p.NACC; ++a)
          tma_load_2d(stage + A_BYTES + a * b_bytes, &map_b, c * 64, n_base + a * p.NB,
                      &bars[TMA_FULL + s]);
      }
      if (!ok) {
        const long long start = clock64();
        while (clock64() - start < (1ll << 21)) {}
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // The whole warp walks the uniform control flow; one elected lane issues.
    const bool leader = elect_one();
    const uint32_t idesc = make_idesc_bf16(128, p.NB);
    const uint32_t smem_base = smem_u32(smem);
    bool ok = true;
    for (int c = 0; c < nchunks && ok; ++c) {
      const int s = c % nst, u = c / nst;
      ok = mbar_wait(&bars[TMA_FULL + s], u & 1, abort_flag, 410 + s);
      if (ok && !ASSIGN) ok = mbar_wait(&bars[A_FULL + s], u & 1, abort_flag, 412 + s);
      if (!ok) break;
      tc_fence_after();
      const uint32_t stage = smem_base + s * stage_bytes;
      const uint64_t a_desc = make_smem_desc_sw128(stage);
      for (int a = 0; a < p.NACC; ++a) {
        const uint64_t b_desc = make_smem_desc_sw128(stage + A_BYTES + a * b_bytes);
        if (leader) {
          mma_bf16(tmem_base + a * 256, a_desc, b_desc, idesc, c > 0);
          mma_bf16(tmem_base + a * 256, a_desc + 2, b_desc + 2, idesc, true);
          mma_bf16(tmem_base + a * 256, a_desc + 4, b_desc + 4, idesc, true);
          mma_bf16(tmem_base + a * 256, a_desc + 6, b_desc + 6, idesc, true);
        }
      }
      if (leader) mma_commit(&bars[STAGE_FREE + s]);
      __syncwarp();
    }
    if (ok && leader) mma_commit(&bars[ACC_DONE]);
    __syncwarp();
  } else {
    const int row = tid & 127, wg = tid >> 7;
    const uint32_t lane_sel = static_cast<uint32_t>(32 * (warp & 3)) << 16;
    bool ok = true;
    if (ASSIGN) {
      // ---- squared norms from the resident tiles
      const int C = p.n_total;
      float xs = 0.f, cs[4] = {0.f, 0.f, 0.f, 0.f};
      for (int c = 0; c < nchunks && ok; ++c) {
        const int s = c % nst, u = c / nst;
        ok = mbar_wait(&bars[TMA_FULL + s], u & 1, abort_flag, 420 + s);
        if (!ok) break;
        const uint8_t* stage = smem + s * stage_bytes;
        if (c < p.a_chunks) {
          const uint4* src = reinterpret_cast<const uint4*>(stage + (tid >> 1) * 128 + (tid & 1) * 64);
#pragma unroll
          for (int j = 0; j < 4; ++j) xs += sumsq8(src[j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int item = tid + i * COMPUTE_THREADS;
          if (p.cnorm == nullptr && item < 2 * C) {
            const uint4* src = reinterpret_cast<const uint4*>(stage + A_BYTES + (item >> 1) * 128 + (item & 1) * 64);
#pragma unroll
            for (int j = 0; j < 4; ++j) cs[i] += sumsq8(src[j]);
          }
        }
        mbar_arrive(&bars[STAGE_FREE + s]);
      }
      if (ok) {
        xn_part[tid] = xs;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int item = tid + i * COMPUTE_THREADS;
          if (item < 2 * C) cn_part[item] = cs[i];
        }
        mbar_arrive(&bars[SIDE_READY]);
        ok = mbar_wait(&bars[SIDE_READY], 0, abort_flag, 430) &&
             mbar_wait(&bars[ACC_DONE], 0, abort_flag, 431);
      }
      if (ok) {
        tc_fence_after();
        const float xn = xn_part[2 * row] + xn_part[2 * row + 1];
        const int chunks = (C + 31) / 32, split = (chunks + 1) / 2;
        const int first = wg == 0 ? 0 : split, last = wg == 0 ? split : chunks;
        float best = INFINITY;
        int best_i = 0x7fffffff;
#pragma unroll 1
        for (int cc = first; cc < last; ++cc) {
          const int col = cc * 32, acc = col / p.NB;
          float v[32];
          tmem_ld32(tmem_base + lane_sel + acc * 256 + (col - acc * p.NB), v);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int cidx = col + j;
            if (cidx < C) {
              const float cn = p.cnorm != nullptr ? __ldg(p.cnorm + cidx) : cn_part[2 * cidx] + cn_part[2 * cidx + 1];
              const float dist = __fsub_rn(__fadd_rn(xn, cn), __fmul_rn(2.0f, v[j]));
              if (dist < best) { best = dist; best_i = cidx; }
            }
          }
        }
        if (wg == 1) {
          cand_d[row] = best;
          cand_i[row] = best_i;
          mbar_arrive(&bars[CAND_READY]);
        } else {
          ok = mbar_wait(&bars[CAND_READY], 0, abort_flag, 432);
          if (ok) {
            if (cand_d[row] < best) { best = cand_d[row]; best_i = cand_i[row]; }
            const int t = m0 + row;
            if (t < m_end) {
              if (p.ids_out != nullptr) {
                if (p.id_bytes == 1) static_cast<uint8_t*>(p.ids_out)[t] = static_cast<uint8_t>(best_i);
                else static_cast<uint16_t*>(p.ids_out)[t] = static_cast<uint16_t>(best_i);
              }
              if (p.labels_out != nullptr) p.labels_out[t] = best_i;
            }
          }
        }
      }
    } else {
      // ---- residual operand: bf16((x - centre[id]) - mean), 32 columns per thread
      const int r = tid >> 1, half = tid & 1;
      const int t = m0 + r;
      const bool in = t < m_end;
      const uint16_t* xrow = p.x + static_cast<size_t>(in ? t : 0) * p.J;
      const uint16_t* crow = p.centers + static_cast<size_t>(in ? load_id(p.ids, p.id_bytes, t) : 0) * p.J;
      // raw operands of one chunk for this thread: 32 columns of x and of the centre row
      uint4 xn[4], cn[4];
      auto fetch = [&](int c) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          xn[j] = make_uint4(0, 0, 0, 0);
          cn[j] = make_uint4(0, 0, 0, 0);
          if (in && c < nchunks) {
            xn[j] = __ldg(reinterpret_cast<const uint4*>(xrow + c * 64 + half * 32) + j);
            cn[j] = __ldg(reinterpret_cast<const uint4*>(crow + c * 64 + half * 32) + j);
          }
        }
      };
      fetch(0);
      for (int c = 0; c < nchunks && ok; ++c) {
        const int s = c % nst, u = c / nst;
        uint4 xc[4], cc4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { xc[j] = xn[j]; cc4[j] = cn[j]; }
        fetch(c + 1);                       // in flight while this chunk is formed
        if (u >= 1) ok = mbar_wait(&bars[STAGE_FREE + s], (u - 1) & 1, abort_flag, 440 + s);
        if (!ok) break;
        uint8_t* stage = smem + s * stage_bytes;
        const int j0 = c * 64 + half * 32;
        const float4* ms = reinterpret_cast<const float4*>(p.mean + j0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 out = make_uint4(0, 0, 0, 0);
          if (in) {
            const uint4 xw = xc[j], cw = cc4[j];
            const float4 m0v = __ldg(ms + 2 * j), m1v = __ldg(ms + 2 * j + 1);
            const uint32_t xwords[4] = {xw.x, xw.y, xw.z, xw.w};
            const uint32_t cwords[4] = {cw.x, cw.y, cw.z, cw.w};
            const float mv[8] = {m0v.x, m0v.y, m0v.z, m0v.w, m1v.x, m1v.y, m1v.z, m1v.w};
            uint32_t* o = &out.x;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              float lo = __fsub_rn(__fsub_rn(__uint_as_float(xwords[w] << 16),
                                             __uint_as_float(cwords[w] << 16)), mv[2 * w]);
              float hi = __fsub_rn(__fsub_rn(__uint_as_float(xwords[w] & 0xFFFF0000u),
                                             __uint_as_float(cwords[w] & 0xFFFF0000u)), mv[2 * w + 1]);
              o[w] = pack_bf16x2(lo, hi);
            }
          }
          *reinterpret_cast<uint4*>(stage + sw128_offset(r, half * 32 + j * 8)) = out;
        }
        fence_proxy_async();
        mbar_arrive(&bars[A_FULL + s]);
      }
      if (ok) ok = mbar_wait(&bars[ACC_DONE], 0, abort_flag, 450);
      if (ok && QUANT) {
        // ---- quantise + pack from TMEM.  Pass 1: |max| of the bf16-rounded coefficients of this
        // thread's column chunks; the two warpgroups, then the two column-half CTAs, combine.
        tc_fence_after();
        const int nc = p.NACC * p.NB;
        const int tok = m0 + row;
        float amax = 0.f;
#pragma unroll 1
        for (int cc = wg; cc < nc / 32; cc += 2) {
          const int col = cc * 32, acc = col / p.NB;
          float v[32];
          tmem_ld32(tmem_base + lane_sel + acc * 256 + (col - acc * p.NB), v);
#pragma unroll
          for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(round_to_bf16(v[j])));
        }
        xn_part[wg * 128 + row] = amax;
        mbar_arrive(&bars[SIDE_READY]);
        ok = mbar_wait(&bars[SIDE_READY], 0, abort_flag, 451);
        if (ok) {
          amax = fmaxf(xn_part[row], xn_part[128 + row]);
          if (paired) {
            if (wg == 0) {
              const uint32_t peer = cluster_ctarank() ^ 1u;
              st_cluster_b32(map_to_cta(smem_u32(&cand_d[row]), peer), __float_as_uint(amax));
              mbar_arrive_cluster(map_to_cta(smem_u32(&bars[PEER_READY]), peer));
            }
            ok = mbar_wait_cluster(&bars[PEER_READY], 0, abort_flag, 452);
            if (ok) amax = fmaxf(amax, cand_d[row]);
          }
        }
        if (ok) {
          float scale;
          if (p.in_bf16) scale = round_to_bf16(__fdiv_rn(fmaxf(amax, round_to_bf16(p.eps)), 7.0f));
          else scale = __fdiv_rn(fmaxf(amax, p.eps), 7.0f);
          const float inv = __frcp_rn(scale);
#pragma unroll 1
          for (int cc = wg; cc < nc / 32; cc += 2) {
            const int col = cc * 32, acc = col / p.NB;
            float v[32];
            tmem_ld32(tmem_base + lane_sel + acc * 256 + (col - acc * p.NB), v);
            uint32_t words[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              uint32_t out = 0;
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float z0 = round_to_bf16(v[w * 8 + 2 * k]), z1 = round_to_bf16(v[w * 8 + 2 * k + 1]);
                const int c0 = p.in_bf16 ? quant_code<true>(z0, scale, inv) : quant_code<false>(z0, scale, inv);
                const int c1 = p.in_bf16 ? quant_code<true>(z1, scale, inv) : quant_code<false>(z1, scale, inv);
                out |= static_cast<uint32_t>(c0 | (c1 << 4)) << (8 * k);
              }
              words[w] = out;
            }
            if (tok < m_end)
              *reinterpret_cast<uint4*>(p.codes + static_cast<size_t>(tok) * (p.n_total >> 1) +
                                        ((n_base + col) >> 1)) = make_uint4(words[0], words[1], words[2], words[3]);
          }
          if (wg == 0 && blockIdx.y == 0 && tok < m_end) store_float(p.scales, p.scale_dtype, tok, scale);
        }
      } else if (ok) {
        tc_fence_after();
        const int nc = p.NACC * p.NB;
        const int tok = m0 + row;
#pragma unroll 1
        for (int cc = wg; cc < nc / 32; cc += 2) {
          const int col = cc * 32, acc = col / p.NB;
          float v[32];
          tmem_ld32(tmem_base + lane_sel + acc * 256 + (col - acc * p.NB), v);
          if (tok < m_end) {
            uint16_t* dst = p.coeff + static_cast<size_t>(tok) * p.n_total + n_base + col;
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              uint4 w;
              w.x = pack_bf16x2(v[j4 * 8 + 0], v[j4 * 8 + 1]);
              w.y = pack_bf16x2(v[j4 * 8 + 2], v[j4 * 8 + 3]);
              w.z = pack_bf16x2(v[j4 * 8 + 4], v[j4 * 8 + 5]);
              w.w = pack_bf16x2(v[j4 * 8 + 6], v[j4 * 8 + 7]);
              *reinterpret_cast<uint4*>(dst + j4 * 8) = w;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
  // neither CTA of a pair leaves while the other may still write into its shared memory
  if (paired) cluster_sync_all();
}

// split n_total columns into grid.y CTAs x NACC accumulators x NB columns
bool plan_columns(int n_total, int* gy, int* nacc, int* nb) {
  for (int g = 1; g <= 16; ++g) {
    if (n_total % g) continue;
    int nc = n_total / g;
    if (nc <= 256 && nc % 32 == 0) { *gy = g; *nacc = 1; *nb = nc; return true; }
    if (nc <= 512 && nc % 64 == 0) { *gy = g; *nacc = 2; *nb = nc / 2; return true; }
  }
  return false;
}

size_t smem_bytes(int nacc, int nb, int n_total, int stages = 2) {
  return stages * static_cast<size_t>(A_BYTES + nacc * nb * 128) + META_HEAD + 4 * (256 + 128 + 128) +
         8 * static_cast<size_t>(n_total) + 1024;
}

int pick_stages(int nacc, int nb, int n_total) {
  int stages = MAX_STAGES;
  while (stages > 2 && smem_bytes(nacc, nb, n_total, stages) > 232448) --stages;
  return stages;
}

}  // namespace

bool tc_project_supported(int J, int r) {
  int gy, nacc, nb;
  return J % 64 == 0 && plan_columns(r, &gy, &nacc, &nb) &&
         smem_bytes(nacc, nb, 0) <= 232448;
}

// Tokens per CTA (<= TM): the MMA always spans TM rows, but the operand build, the loads and the
// epilogue scale with the rows a CTA owns, so the token tiles are sized to fill whole rounds of the
// SMs instead of leaving the last round mostly empty (12,480 tokens: 147 CTAs of 85 rows instead
// of 98 of 128).  Not below 64 rows: every CTA streams the whole B operand from L2.
int pick_rows(int S, int column_parts) {
  // SM count of the current device, cached per device ordinal
  static std::atomic<int> cached[64];
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) device = -1;
  if (device >= 0) sms = cached[device].load(std::memory_order_relaxed);
  if (sms == 0) {
    if (device < 0 ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      sms = 148;
    if (device >= 0) cached[device].store(sms, std::memory_order_relaxed);
  }
  const long long units = static_cast<long long>(ceil_div(S, TM)) * column_parts;
  const long long waves = (units + sms - 1) / sms;
  const long long tiles = waves * sms / column_parts;
  long long rows = (S + tiles - 1) / (tiles > 0 ? tiles : 1);
  rows = rows < 64 ? 64 : (rows > TM ? TM : rows);
  return static_cast<int>(rows);
}

bool tc_assign_supported(int J, int C) {
  if (J % 64 || C % 16 || C > 512) return false;
  return C <= 256 || C % 64 == 0;
}

int tc_project(const void* x_bf16, const void* centers_bf16, const void* ids, int id_bytes,
               const float* mean, const void* encoder_bf16, int S, int J, int r, void* coeff,
               cudaStream_t stream) {
  if (S == 0) return NKV_OK;
  Params p{};
  int gy;
  NKV_REQUIRE(plan_columns(r, &gy, &p.NACC, &p.NB), NKV_ERR_UNSUPPORTED,
              "projection rank %d cannot be tiled", r);
  NKV_REQUIRE((reinterpret_cast<uintptr_t>(x_bf16) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(centers_bf16) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(mean) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(coeff) & 15) == 0,
              NKV_ERR_INVALID, "projection operands must be 16-byte aligned");
  p.S = S; p.J = J; p.n_total = r;
  p.x = static_cast<const uint16_t*>(x_bf16);
  p.centers = static_cast<const uint16_t*>(centers_bf16);
  p.ids = ids; p.id_bytes = id_bytes; p.mean = mean;
  p.coeff = static_cast<uint16_t*>(coeff);
  CUtensorMap map_b;
  uint64_t dims[2] = {static_cast<uint64_t>(J), static_cast<uint64_t>(r)};
  uint64_t strides[1] = {static_cast<uint64_t>(J) * 2};
  uint32_t box[2] = {64, static_cast<uint32_t>(p.NB)};
  int rc = encode_tensor_map(&map_b, 2, encoder_bf16, 2, dims, strides, box, 128);
  if (rc != NKV_OK) return rc;
  p.nstages = pick_stages(p.NACC, p.NB, 0);
  size_t smem = smem_bytes(p.NACC, p.NB, 0, p.nstages);
  auto kernel = encode_gemm_kernel<PROJECT>;
  NKV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem)));
  p.rows = pick_rows(S, gy);
  dim3 grid(ceil_div(S, p.rows), gy);
  kernel<<<grid, THREADS, smem, stream>>>(map_b, map_b, p);
  NKV_LAUNCH_CHECK("encode_gemm_kernel<project>");
  return NKV_OK;
}

bool tc_project_quant_supported(int J, int r, int group) {
  int gy, nacc, nb;
  return group == r && r % 64 == 0 && tc_project_supported(J, r) && plan_columns(r, &gy, &nacc, &nb) && gy <= 2;
}

int tc_project_quant(const void* x_bf16, const void* centers_bf16, const void* ids, int id_bytes,
                     const float* mean, const void* encoder_bf16, int S, int J, int r, float eps,
                     int quant_mode, int scale_dtype, uint8_t* codes, void* scales, cudaStream_t stream) {
  if (S == 0) return NKV_OK;
  Params p{};
  int gy;
  NKV_REQUIRE(plan_columns(r, &gy, &p.NACC, &p.NB) && gy <= 2, NKV_ERR_UNSUPPORTED,
              "fused projection: rank %d cannot be tiled over at most two column parts", r);
  NKV_REQUIRE((reinterpret_cast<uintptr_t>(x_bf16) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(centers_bf16) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(mean) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(codes) & 15) == 0 && (r / 2) % 16 == 0,
              NKV_ERR_INVALID, "fused projection operands must be 16-byte aligned");
  p.S = S; p.J = J; p.n_total = r;
  p.x = static_cast<const uint16_t*>(x_bf16);
  p.centers = static_cast<const uint16_t*>(centers_bf16);
  p.ids = ids; p.id_bytes = id_bytes; p.mean = mean;
  p.codes = codes; p.scales = scales; p.eps = eps;
  p.in_bf16 = quant_mode == NKV_QUANT_IN_BF16 ? 1 : 0;
  p.scale_dtype = scale_dtype;
  p.column_parts = gy;
  CUtensorMap map_b;
  uint64_t dims[2] = {static_cast<uint64_t>(J), static_cast<uint64_t>(r)};
  uint64_t strides[1] = {static_cast<uint64_t>(J) * 2};
  uint32_t box[2] = {64, static_cast<uint32_t>(p.NB)};
  int rc = encode_tensor_map(&map_b, 2, encoder_bf16, 2, dims, strides, box, 128);
  if (rc != NKV_OK) return rc;
  p.nstages = pick_stages(p.NACC, p.NB, 0);
  size_t smem = smem_bytes(p.NACC, p.NB, 0, p.nstages);
  auto kernel = encode_gemm_kernel<PROJECT_QUANT>;
  NKV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem)));
  p.rows = pick_rows(S, gy);
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(ceil_div(S, p.rows), gy);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 1;
  attribute.val.clusterDim.y = gy;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  NKV_CUDA(cudaLaunchKernelEx(&config, kernel, map_b, map_b, p));
  NKV_LAUNCH_CHECK("encode_gemm_kernel<project + quantise>");
  return NKV_OK;
}

int tc_assign(const void* x_bf16, const void* centers_bf16, int S, int J, int C, void* ids,
              int id_bytes, cudaStream_t stream) {
  if (S == 0) return NKV_OK;
  Params p{};
  p.S = S; p.J = J; p.n_total = C;
  p.NACC = C > 256 ? 2 : 1;
  p.NB = C / p.NACC;
  p.ids_out = ids; p.id_bytes = id_bytes;
  p.a_chunks = J / 64;
  CUtensorMap map_a, map_b;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(J), static_cast<uint64_t>(S)};
    uint64_t strides[1] = {static_cast<uint64_t>(J) * 2};
    uint32_t box[2] = {64, TM};
    int rc = encode_tensor_map(&map_a, 2, x_bf16, 2, dims, strides, box, 128);
    if (rc != NKV_OK) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(J), static_cast<uint64_t>(C)};
    uint64_t strides[1] = {static_cast<uint64_t>(J) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(p.NB)};
    int rc = encode_tensor_map(&map_b, 2, centers_bf16, 2, dims, strides, box, 128);
    if (rc != NKV_OK) return rc;
  }
  p.nstages = pick_stages(p.NACC, p.NB, C);
  size_t smem = smem_bytes(p.NACC, p.NB, C, p.nstages);
  auto kernel = encode_gemm_kernel<ASSIGN_IDS>;
  NKV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem)));
  p.rows = pick_rows(S, 1);
  dim3 grid(ceil_div(S, p.rows), 1);
  kernel<<<grid, THREADS, smem, stream>>>(map_a, map_b, p);
  NKV_LAUNCH_CHECK("encode_gemm_kernel<assign>");
  return NKV_OK;
}

namespace {

// fp32 centre rows -> three bf16 planes side by side ([C, 3 J]: c = hi + mid + lo exactly, up to the
// last bit of the third term) and the rows' squared norms in fp32
__global__ void __launch_bounds__(256)
split_centers_kernel(const float* centers, int J, uint16_t* planes, float* cnorm) {
  __shared__ float part[256];
  const int c = blockIdx.x;
  const float* row = centers + static_cast<size_t>(c) * J;
  uint16_t* out = planes + static_cast<size_t>(c) * 3 * J;
  float sum = 0.f;
  for (int j = threadIdx.x; j < J; j += 256) {
    const float v = row[j];
    sum = fmaf(v, v, sum);
    const uint16_t hi = float_to_bf16_bits(v);
    const float r1 = __fsub_rn(v, bf16_bits_to_float(hi));
    const uint16_t mid = float_to_bf16_bits(r1);
    const float r2 = __fsub_rn(r1, bf16_bits_to_float(mid));
    out[j] = hi;
    out[J + j] = mid;
    out[2 * J + j] = float_to_bf16_bits(r2);
  }
  part[threadIdx.x] = sum;
  __syncthreads();
  for (int width = 128; width >= 1; width >>= 1) {
    if (threadIdx.x < width) part[threadIdx.x] += part[threadIdx.x + width];
    __syncthreads();
  }
  if (threadIdx.x == 0) cnorm[c] = part[0];
}

}  // namespace

size_t tc_assign_f32_workspace_bytes(int J, int C) {
  return static_cast<size_t>(C) * 3 * J * 2 + static_cast<size_t>(C) * 4 + 256;
}

// Nearest centre against fp32 centres on the tensor cores: every bf16 x bf16 product is exact in the
// fp32 accumulator, and the three planes restore the centres' 24 mantissa bits, so the distances
// carry fp32 accuracy (the accumulation order is the tensor core's).  Writes 32-bit labels.
int tc_assign_f32(const void* x_bf16, const float* centers_f32, int S, int J, int C, int32_t* labels,
                  void* workspace, cudaStream_t stream) {
  if (S == 0) return NKV_OK;
  NKV_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, NKV_ERR_INVALID,
              "assign: plane workspace must be 256-byte aligned");
  uint16_t* planes = static_cast<uint16_t*>(workspace);
  float* cnorm = reinterpret_cast<float*>(planes + static_cast<size_t>(C) * 3 * J);
  split_centers_kernel<<<C, 256, 0, stream>>>(centers_f32, J, planes, cnorm);
  NKV_LAUNCH_CHECK("split_centers_kernel");
  Params p{};
  p.S = S; p.J = J; p.n_total = C;
  p.NACC = C > 256 ? 2 : 1;
  p.NB = C / p.NACC;
  p.labels_out = labels; p.id_bytes = 1;
  p.a_chunks = J / 64;
  p.cnorm = cnorm;
  CUtensorMap map_a, map_b;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(J), static_cast<uint64_t>(S)};
    uint64_t strides[1] = {static_cast<uint64_t>(J) * 2};
    uint32_t box[2] = {64, TM};
    int rc = encode_tensor_map(&map_a, 2, x_bf16, 2, dims, strides, box, 128);
    if (rc != NKV_OK) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(J) * 3, static_cast<uint64_t>(C)};
    uint64_t strides[1] = {static_cast<uint64_t>(J) * 3 * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(p.NB)};
    int rc = encode_tensor_map(&map_b, 2, planes, 2, dims, strides, box, 128);
    if (rc != NKV_OK) return rc;
  }
  p.nstages = pick_stages(p.NACC, p.NB, C);
  size_t smem = smem_bytes(p.NACC, p.NB, C, p.nstages);
  auto kernel = encode_gemm_kernel<ASSIGN_IDS>;
  NKV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem)));
  p.rows = pick_rows(S, 1);
  dim3 grid(ceil_div(S, p.rows), 1);
  kernel<<<grid, THREADS, smem, stream>>>(map_a, map_b, p);
  NKV_LAUNCH_CHECK("encode_gemm_kernel<assign, fp32 centres>");
  return NKV_OK;
}

}  // namespace nkv
