// Fused codec-attention on tcgen05 tensor cores (bf16 operands, fp32 TMEM
// accumulators).
//
// One CTA owns one head and up to 256 queries (two 128-row query tiles) and
// walks the compressed history in tiles of 128 tokens.  Per tile:
//   1. TMA streams the packed INT4 codes of the tile and the head's slice of
//      the decoder (or reader) matrix, 64 latent columns at a time, through a
//      ring of NW slots that is never aliased, so the producer runs ahead
//      across tile boundaries; the compute warps expand the codes to bf16
//      latent rows (code * stored scale, one rounding) straight into the
//      128-byte-swizzled operand layout of a two-slot latent ring,
//   2. tcgen05.mma rebuilds K[128 tok x D] and V[128 tok x D] for this head in
//      TMEM; the compute warps add bias and the token's centre row with the
//      reference's two bf16 roundings and park K (row-major) and V (transposed)
//      in shared memory -- K and V never exist in global memory,
//   3. S = Q K^T per query tile in TMEM, online softmax in registers (exp2,
//      lazy rescaling of the O accumulator), P to shared memory as bf16 (over
//      the K tile and the latent ring, both dead by then),
//   4. O += P V in TMEM.
// Warp roles: warps 0-7 compute (dequantise / epilogue / softmax), warp 8 lane 0
// issues TMA, warp 9 lane 0 issues MMA, warp 10 prefetches per-token metadata
// (centre row, scales) two tiles ahead.  All hand-offs are mbarriers with
// bounded waits (see nkv_tc.cuh).
//
// TMEM columns: [0,128) K accumulator then S of query tile 0; [128,256) V
// accumulator then S of tile 1; [256,384) O tile 0; [384,512) O tile 1.
#include "nkv_internal.h"
#include "nkv_tc.cuh"

namespace nkv {
namespace {

using namespace tc;

constexpr int TOK = 128;          // history tokens per tile
constexpr int QT = 128;           // queries per query tile
constexpr int NQ = 2;             // query tiles per CTA
constexpr int COMPUTE_THREADS = 256;
constexpr int THREADS = COMPUTE_THREADS + 96;
constexpr int CHUNK = 64;         // latent columns per pipeline step
constexpr int TILE_BYTES = 128 * 128;  // one [128 rows x 64 bf16] swizzled tile
constexpr int MAX_NW = 4;
constexpr float RESCALE_THRESHOLD = 8.0f;

enum Bar {
  Q_FULL = 0, W_FULL = 1, W_FREE = 5, LAT_FULL = 9, LAT_FREE = 13, ACC_DONE = 17,
  META_FULL = 19, META_FREE = 21, KV_READY = 23, S_FULL = 24, P_READY = 26, PV_DONE = 28,
  KEPI_DONE = 30, NUM_BARS = 31
};

struct Params {
  int Q, heads, N, rank, nchunks, ngroups, group;
  int scale_dtype, nw;
  float scale_log2;
  nkv_history hk, hv;
  const float* bias_k;
  const float* bias_v;
  uint16_t* out;
  float* lse;
  int32_t* status;
  long long* prof;   // optional: cycle buckets of CTA (0,0), see nkv_debug_attn_profile
};

// Same result with bf16 pair arithmetic and no int->float conversions, for bf16 scales:
// the bit pattern 0x4300 | n is the bf16 number 128 + n; (128 + n) - 135 = n - 7 exactly, and the
// bf16 product of two bf16 numbers is the exact product rounded once, as the reference computes it.
__device__ __forceinline__ uint4 dequant8_bf16(uint32_t word, __nv_bfloat162 scale2) {
  const uint32_t lo = word & 0x0F0F0F0Fu, hi = (word >> 4) & 0x0F0F0F0Fu;
  const uint32_t t[4] = {__byte_perm(lo, hi, 0x4400), __byte_perm(lo, hi, 0x5511),
                         __byte_perm(lo, hi, 0x6622), __byte_perm(lo, hi, 0x7733)};
  const uint32_t bias_bits = 0x43074307u;   // bf16 pair (135, 135)
  const __nv_bfloat162 bias2 = *reinterpret_cast<const __nv_bfloat162*>(&bias_bits);
  uint4 r;
  uint32_t* o = &r.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t bits = (t[i] & 0x00FF00FFu) | 0x43004300u;
    const __nv_bfloat162 v = __hmul2(__hsub2(*reinterpret_cast<const __nv_bfloat162*>(&bits), bias2), scale2);
    o[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  return r;
}

template <int D>
struct Layout {
  static constexpr int DCH = D / 64;                     // 64-column chunks of a head row
  static constexpr int Q_OFF = 0;                        // [NQ][DCH] tiles
  static constexpr int K_OFF = Q_OFF + NQ * DCH * TILE_BYTES;   // [DCH] tiles [128 tok x 64]
  static constexpr int VT_OFF = K_OFF + DCH * TILE_BYTES;       // [2] tiles [D rows x 64 tok]
  static constexpr int VT_TILE = D * 128;
  static constexpr int SCRATCH_OFF = VT_OFF + 2 * VT_TILE;      // 8 warps x 4 KB: centre-row staging
  static constexpr int RING_OFF = SCRATCH_OFF + 2 * TILE_BYTES;
  static constexpr int SLOT_W = 0;
  static constexpr int SLOT_CODES = D * 128;
  static constexpr int SLOT_BYTES = SLOT_CODES + TOK * 32;
  __host__ __device__ static int meta_off(int nw) { return RING_OFF + nw * SLOT_BYTES; }
  // meta: bars, tmem slot, abort, bias_k/v [D] floats, then per meta buffer (x2):
  // crow [2][128] ints and scales [2][128][ngroups] u16
  static constexpr int BARS = 0;
  static constexpr int SLOT = NUM_BARS * 8;
  static constexpr int ABORT = SLOT + 4;
  static constexpr int BIAS = ((ABORT + 4 + 15) / 16) * 16;
  static constexpr int CROW = BIAS + 2 * D * 4;
  static constexpr int SCALES = CROW + 2 * 2 * TOK * 4;
  static size_t bytes(int nw, int ngroups) {
    return meta_off(nw) + SCALES + 2 * 2 * TOK * ngroups * 2 + 1024;
  }
};

__device__ __forceinline__ float scale_to_float(uint16_t bits, int dtype) {
  return dtype == NKV_BF16 ? bf16_bits_to_float(bits) : __half2float(__ushort_as_half(bits));
}

// 4 code bytes (8 nibbles, even element in the low nibble) -> 8 bf16 latents
__device__ __forceinline__ uint4 dequant8(uint32_t word, float scale) {
  uint4 r;
  uint32_t* o = &r.x;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    uint32_t byte = (word >> (8 * b)) & 0xFFu;
    float lo = static_cast<float>(static_cast<int>(byte & 15u) - 7) * scale;
    float hi = static_cast<float>(static_cast<int>(byte >> 4) - 7) * scale;
    o[b] = pack_bf16x2(lo, hi);
  }
  return r;
}

// Lap timer of one thread: adds the cycles since the previous lap to a bucket.
struct Laps {
  long long* out;
  long long last;
  __device__ __forceinline__ void start(long long* dst, bool on) { out = on ? dst : nullptr; last = clock64(); }
  __device__ __forceinline__ void lap(int bucket) {
    if (out) { long long now = clock64(); out[bucket] += now - last; last = now; }
  }
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attn_codec_kernel(const __grid_constant__ CUtensorMap map_q,
                  const __grid_constant__ CUtensorMap map_wk,
                  const __grid_constant__ CUtensorMap map_wv,
                  const __grid_constant__ CUtensorMap map_ck,
                  const __grid_constant__ CUtensorMap map_cv, Params p) {
  using L = Layout<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int nw = p.nw;
  uint8_t* meta = smem + L::meta_off(nw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(meta + L::BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(meta + L::SLOT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(meta + L::ABORT);
  float* bias = reinterpret_cast<float*>(meta + L::BIAS);            // [2][D]
  int* crow = reinterpret_cast<int*>(meta + L::CROW);                // [2 buf][2][128]
  uint16_t* scales = reinterpret_cast<uint16_t*>(meta + L::SCALES);  // [2 buf][2][128][ngroups]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y;
  const int q0 = blockIdx.x * (NQ * QT);
  const int nq = (q0 + QT < p.Q) ? 2 : 1;
  const int ntiles = (p.N + TOK - 1) / TOK;
  const int nchunks = p.nchunks;
  const int ng = p.ngroups;

  if (tid == 0) {
    mbar_init(&bars[Q_FULL], 1);
    for (int s = 0; s < MAX_NW; ++s) {
      mbar_init(&bars[W_FULL + s], 1);
      mbar_init(&bars[W_FREE + s], 1);
      mbar_init(&bars[LAT_FULL + s], COMPUTE_THREADS);
      mbar_init(&bars[LAT_FREE + s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[ACC_DONE + s], 1);
      mbar_init(&bars[META_FULL + s], 32);
      mbar_init(&bars[META_FREE + s], COMPUTE_THREADS);
      mbar_init(&bars[S_FULL + s], 1);
      mbar_init(&bars[P_READY + s], QT);
      mbar_init(&bars[PV_DONE + s], 1);
    }
    mbar_init(&bars[KV_READY], COMPUTE_THREADS);
    mbar_init(&bars[KEPI_DONE], COMPUTE_THREADS);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  for (int i = tid; i < 2 * D; i += THREADS)
    bias[i] = i < D ? p.bias_k[head * D + i] : p.bias_v[head * D + (i - D)];
  if (warp == 9) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_wk);
      prefetch_tensormap(&map_wv);
      prefetch_tensormap(&map_ck);
      prefetch_tensormap(&map_cv);
      mbar_arrive_expect_tx(&bars[Q_FULL], nq * L::DCH * TILE_BYTES);
      for (int i = 0; i < nq; ++i)
        for (int c = 0; c < L::DCH; ++c)
          tma_load_3d(smem + L::Q_OFF + (i * L::DCH + c) * TILE_BYTES, &map_q, c * 64, head,
                      q0 + i * QT, &bars[Q_FULL]);
      bool ok = true;
      int slot = 0, use = 0;             // ring position of chunk g = it * 2 * nchunks + ...
      for (int it = 0; it < ntiles && ok; ++it) {
        for (int which = 0; which < 2 && ok; ++which) {
          for (int c = 0; c < nchunks && ok; ++c) {
            if (use >= 1) ok = mbar_wait(&bars[W_FREE + slot], (use - 1) & 1, abort_flag, 110 + slot);
            if (!ok) break;
            uint8_t* dst = smem + L::RING_OFF + slot * L::SLOT_BYTES;
            mbar_arrive_expect_tx(&bars[W_FULL + slot], TOK * 32 + D * 128);
            tma_load_2d(dst + L::SLOT_CODES, which ? &map_cv : &map_ck, c * 32, it * TOK,
                        &bars[W_FULL + slot]);
            tma_load_2d(dst + L::SLOT_W, which ? &map_wv : &map_wk, c * CHUNK, head * D,
                        &bars[W_FULL + slot]);
            if (++slot == nw) { slot = 0; ++use; }
          }
        }
      }
      if (!ok) {  // let copies already in flight land before the CTA goes away
        const long long start = clock64();
        while (clock64() - start < (1ll << 21)) {}
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_dec = make_idesc_bf16(128, D);    // [128 tok] x [D]
      const uint32_t idesc_s = make_idesc_bf16(128, TOK);    // [128 q] x [128 tok]
      const uint32_t idesc_pv = make_idesc_bf16(128, D);     // [128 q] x [D]
      const uint32_t smem_base = smem_u32(smem);
      Laps laps;
      laps.start(p.prof + 16, p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0);
      bool ok = mbar_wait(&bars[Q_FULL], 0, abort_flag, 200);
      int slot = 0, use = 0, g = 0;
      for (int it = 0; it < ntiles && ok; ++it) {
        for (int which = 0; which < 2 && ok; ++which) {
          for (int c = 0; c < nchunks && ok; ++c, ++g) {
            const int ls = g & 3, lu = g >> 2;   // four latent staging slots in TMEM
            ok = mbar_wait(&bars[W_FULL + slot], use & 1, abort_flag, 210 + slot);
            laps.lap(0);
            ok = ok && mbar_wait(&bars[LAT_FULL + ls], lu & 1, abort_flag, 214 + ls);
            laps.lap(1);
            if (!ok) break;
            tc_fence_after();
            const uint32_t w = smem_base + L::RING_OFF + slot * L::SLOT_BYTES + L::SLOT_W;
            // latent chunk: 32 TMEM columns in the other tensor's (idle) accumulator region
            const uint32_t lat = tmem_base + (which == 0 ? 128 : 0) + ls * 32;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_bf16_ts(tmem_base + which * 128, lat + k * 8, make_smem_desc_sw128(w + k * 32),
                          idesc_dec, c > 0 || k > 0);
            mma_commit(&bars[W_FREE + slot]);
            mma_commit(&bars[LAT_FREE + ls]);
            if (c == nchunks - 1) mma_commit(&bars[ACC_DONE + which]);
            if (++slot == nw) { slot = 0; ++use; }
            laps.lap(2);
          }
        }
        if (!ok) break;
        ok = mbar_wait(&bars[KV_READY], it & 1, abort_flag, 220);
        laps.lap(3);
        if (!ok) break;
        tc_fence_after();
        for (int i = 0; i < nq; ++i) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t a = smem_base + L::Q_OFF + (i * L::DCH + (k >> 2)) * TILE_BYTES + (k & 3) * 32;
            const uint32_t b = smem_base + L::K_OFF + (k >> 2) * TILE_BYTES + (k & 3) * 32;
            mma_bf16(tmem_base + i * 128, make_smem_desc_sw128(a), make_smem_desc_sw128(b),
                     idesc_s, k > 0);
          }
          mma_commit(&bars[S_FULL + i]);
        }
        for (int i = 0; i < nq && ok; ++i) {
          laps.lap(4);
          ok = mbar_wait(&bars[P_READY + i], it & 1, abort_flag, 230 + i);
          laps.lap(5);
          if (!ok) break;
          tc_fence_after();
          // P (bf16 pairs) sits in the first 64 columns of the S region it was computed from
#pragma unroll
          for (int k = 0; k < TOK / 16; ++k) {
            const uint32_t b = smem_base + L::VT_OFF + (k >> 2) * L::VT_TILE + (k & 3) * 32;
            mma_bf16_ts(tmem_base + 256 + i * 128, tmem_base + i * 128 + k * 8,
                        make_smem_desc_sw128(b), idesc_pv, it > 0 || k > 0);
          }
          mma_commit(&bars[PV_DONE + i]);
        }
        laps.lap(6);
      }
    }
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------------------------- per-token metadata, two tiles ahead
    bool ok = true;
    for (int it = 0; it < ntiles && ok; ++it) {
      const int b = it & 1, u = it >> 1;
      if (u >= 1) ok = mbar_wait(&bars[META_FREE + b], (u - 1) & 1, abort_flag, 240 + b);
      if (!ok) break;
      const int t0 = it * TOK;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const nkv_history& h = which ? p.hv : p.hk;
        for (int r = lane; r < TOK; r += 32) {
          const int t = t0 + r;
          const bool in = t < p.N;
          crow[(b * 2 + which) * TOK + r] = in ? center_row_of(h, t) : 0;
          const uint16_t* src = static_cast<const uint16_t*>(h.scales) + static_cast<size_t>(t) * ng;
          uint16_t* dst = scales + static_cast<size_t>((b * 2 + which) * TOK + r) * ng;
          for (int gi = 0; gi < ng; ++gi) dst[gi] = in ? src[gi] : 0;
        }
      }
      mbar_arrive(&bars[META_FULL + b]);
    }
  } else {
    // ------------------------------------------------------------ compute warps
    const int wg = tid >> 7;                    // query tile this thread's softmax serves
    const int row = tid & 127;                  // TMEM lane == token row == query row
    const uint32_t lane_sel = static_cast<uint32_t>(32 * (warp & 3)) << 16;
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    int slot = 0, use = 0, g = 0;
    Laps laps;
    laps.start(p.prof, p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0);
    for (int it = 0; it < ntiles && ok; ++it) {
      const int t0 = it * TOK;
      const int valid = min(TOK, p.N - t0);
      const int mb = it & 1;
      if (it > 0) {  // P of the previous tile lives in the K tile and the latent ring
        for (int i = 0; i < nq && ok; ++i)
          ok = mbar_wait(&bars[PV_DONE + i], (it - 1) & 1, abort_flag, 300 + i);
        if (!ok) break;
        tc_fence_after();
      }
      laps.lap(0);
      ok = mbar_wait(&bars[META_FULL + mb], (it >> 1) & 1, abort_flag, 310);
      laps.lap(1);
      if (!ok) break;
      // ---- per tensor: expand codes to bf16 latent chunks in tensor memory (the A operand of
      // the decode MMA), then the epilogue: bias, centre, two bf16 roundings, park in shared memory
      for (int which = 0; which < 2 && ok; ++which) {
        if (which == 1) {
          // V's latent staging reuses K-accumulator columns: every thread must have read them
          ok = mbar_wait(&bars[KEPI_DONE], it & 1, abort_flag, 326);
          if (!ok) break;
        }
        for (int c = 0; c < nchunks && ok; ++c, ++g) {
          const int ls = g & 3, lu = g >> 2;   // four latent staging slots in TMEM
          ok = mbar_wait(&bars[W_FULL + slot], use & 1, abort_flag, 320 + slot);
          laps.lap(2);
          if (ok && lu >= 1) ok = mbar_wait(&bars[LAT_FREE + ls], (lu - 1) & 1, abort_flag, 324 + ls);
          laps.lap(3);
          if (!ok) break;
          tc_fence_after();
          const uint8_t* codes = smem + L::RING_OFF + slot * L::SLOT_BYTES + L::SLOT_CODES;
          const int half = wg;        // this thread: token `row`, latent columns half*32 .. +32
          const uint4 code = *reinterpret_cast<const uint4*>(codes + row * 32 + half * 16);
          const int col0 = c * CHUNK + half * 32;
          const uint16_t sbits =
              scales[static_cast<size_t>((mb * 2 + which) * TOK + row) * p.ngroups + col0 / p.group];
          const uint32_t words[4] = {code.x, code.y, code.z, code.w};
          uint32_t packed[16];
          if (p.scale_dtype == NKV_BF16) {
            const uint32_t pair = static_cast<uint32_t>(sbits) * 0x00010001u;
            const __nv_bfloat162 scale2 = *reinterpret_cast<const __nv_bfloat162*>(&pair);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 v = dequant8_bf16(words[j], scale2);
              packed[4 * j] = v.x; packed[4 * j + 1] = v.y; packed[4 * j + 2] = v.z; packed[4 * j + 3] = v.w;
            }
          } else {
            const float sc = scale_to_float(sbits, p.scale_dtype);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 v = dequant8(words[j], sc);
              packed[4 * j] = v.x; packed[4 * j + 1] = v.y; packed[4 * j + 2] = v.z; packed[4 * j + 3] = v.w;
            }
          }
          tmem_st16(tmem_base + lane_sel + (which == 0 ? 128 : 0) + ls * 32 + half * 16, packed);
          tmem_wait_st();
          laps.lap(4);
          tc_fence_before();
          mbar_arrive(&bars[LAT_FULL + ls]);
          laps.lap(5);
          if (++slot == nw) { slot = 0; ++use; }
        }
        if (!ok) break;
        const nkv_history& h = which ? p.hv : p.hk;
        const bool in = row < valid;
        const int colhalf = warp >> 2;
        const int colbase = colhalf * (D / 2);
        // Centre rows of this warp's 32 tokens (D/2 columns each), gathered cooperatively: PIECES
        // lanes read one row's 16-byte pieces, so a load instruction touches 32/PIECES lines
        // instead of 32; the rows are then redistributed through a swizzled staging area in the
        // scratch area of shared memory.
        constexpr int PIECES = D / 16, RPI = 32 / PIECES;
        const int wrow0 = 32 * (warp & 3);
        const uint16_t* cbase = static_cast<const uint16_t*>(h.centers) +
                                static_cast<size_t>(head) * D + colbase;
        uint4 cen[PIECES];
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
          const int rloc = i * RPI + lane / PIECES, piece = lane % PIECES;
          const int crow_i = crow[(mb * 2 + which) * TOK + wrow0 + rloc];
          cen[i] = __ldg(reinterpret_cast<const uint4*>(
              cbase + static_cast<size_t>(crow_i) * h.center_width + piece * 8));
        }
        laps.lap(6);
        ok = mbar_wait(&bars[ACC_DONE + which], it & 1, abort_flag, 330 + which);
        if (!ok) break;
        tc_fence_after();
        laps.lap(7);
        {
          uint8_t* stage = smem + L::SCRATCH_OFF + warp * (32 * PIECES * 16);
#pragma unroll
          for (int i = 0; i < PIECES; ++i) {
            const int rloc = i * RPI + lane / PIECES, piece = lane % PIECES;
            *reinterpret_cast<uint4*>(stage + rloc * (PIECES * 16) +
                                      ((piece ^ (rloc & (PIECES - 1))) << 4)) = cen[i];
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < PIECES; ++j)
            cen[j] = *reinterpret_cast<const uint4*>(stage + lane * (PIECES * 16) +
                                                     ((j ^ (lane & (PIECES - 1))) << 4));
          __syncwarp();
        }
#pragma unroll
        for (int cc = 0; cc < D / 64; ++cc) {
          const int col = colbase + cc * 32;
          float v[32];
          tmem_ld32(tmem_base + lane_sel + which * 128 + col, v);
          uint32_t packed[16];
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            const uint4 cw = cen[cc * 4 + j4];
            const uint32_t cwords[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const int j = j4 * 8 + w * 2;
              float x0 = round_to_bf16(v[j] + bias[which * D + col + j]);
              float x1 = round_to_bf16(v[j + 1] + bias[which * D + col + j + 1]);
              x0 += __uint_as_float(cwords[w] << 16);
              x1 += __uint_as_float(cwords[w] & 0xFFFF0000u);
              packed[j4 * 4 + w] = in ? pack_bf16x2(x0, x1) : 0u;
            }
          }
          if (which == 0) {
            uint8_t* tile = smem + L::K_OFF + (col >> 6) * TILE_BYTES;
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4)
              *reinterpret_cast<uint4*>(tile + sw128_offset(row, (col & 63) + j4 * 8)) =
                  make_uint4(packed[j4 * 4], packed[j4 * 4 + 1], packed[j4 * 4 + 2], packed[j4 * 4 + 3]);
          } else {
            uint8_t* tile = smem + L::VT_OFF + (row >> 6) * L::VT_TILE;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const uint32_t wv = packed[j >> 1];
              const uint16_t bits = (j & 1) ? static_cast<uint16_t>(wv >> 16) : static_cast<uint16_t>(wv & 0xFFFFu);
              *reinterpret_cast<uint16_t*>(tile + sw128_offset(col + j, row & 63)) = bits;
            }
          }
        }
        if (which == 0) {
          tc_fence_before();
          mbar_arrive(&bars[KEPI_DONE]);
        }
      }
      if (!ok) break;
      laps.lap(8);
      mbar_arrive(&bars[META_FREE + mb]);
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(&bars[KV_READY]);
      laps.lap(9);
      // ---- online softmax of this thread's query row
      if (wg < nq) {
        ok = mbar_wait(&bars[S_FULL + wg], it & 1, abort_flag, 340 + wg);
        laps.lap(10);
        if (!ok) break;
        tc_fence_after();
        const uint32_t s_addr = tmem_base + lane_sel + wg * 128;
        float mx = -INFINITY;
#pragma unroll 1
        for (int cc = 0; cc < TOK / 32; ++cc) {
          if (cc * 32 >= valid) break;
          float v[32];
          tmem_ld32(s_addr + cc * 32, v);
          if (valid == TOK) {
#pragma unroll
            for (int j = 0; j < 32; ++j) mx = fmaxf(mx, v[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (cc * 32 + j < valid) mx = fmaxf(mx, v[j]);
          }
        }
        const float m_new = mx * p.scale_log2;
        const bool need = m_new > m_used + RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, need)) {
          const float m_next = fmaxf(m_used, m_new);
          const float alpha = exp2f(m_used - m_next);   // 0 on the first tile (m_used = -inf)
          if (it > 0) {
            const uint32_t o_addr = tmem_base + lane_sel + 256 + wg * 128;
#pragma unroll 1
            for (int cc = 0; cc < D / 32; ++cc) {
              float v[32];
              tmem_ld32(o_addr + cc * 32, v);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= alpha;
              tmem_st32(o_addr + cc * 32, v);
            }
          }
          l_run *= alpha;
          m_used = m_next;
        }
        // P (bf16 pairs) replaces S in place: the 16 cells written per step lie below the 32 read
        float sum = 0.f;
#pragma unroll 1
        for (int cc = 0; cc < TOK / 32; ++cc) {
          float v[32];
          tmem_ld32(s_addr + cc * 32, v);
          uint32_t packed[16];
          if (valid == TOK) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float p0 = exp2f(fmaf(v[j], p.scale_log2, -m_used));
              const float p1 = exp2f(fmaf(v[j + 1], p.scale_log2, -m_used));
              sum += p0 + p1;
              packed[j >> 1] = pack_bf16x2(p0, p1);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float p0 = (cc * 32 + j < valid) ? exp2f(fmaf(v[j], p.scale_log2, -m_used)) : 0.f;
              float p1 = (cc * 32 + j + 1 < valid) ? exp2f(fmaf(v[j + 1], p.scale_log2, -m_used)) : 0.f;
              sum += p0 + p1;
              packed[j >> 1] = pack_bf16x2(p0, p1);
            }
          }
          tmem_st16(s_addr + cc * 16, packed);
        }
        tmem_wait_st();
        l_run += sum;
        laps.lap(11);
        tc_fence_before();
        mbar_arrive(&bars[P_READY + wg]);
        laps.lap(12);
      }
    }
    // ---- write O / l and the natural-log LSE
    if (ok && wg < nq && ntiles > 0) {
      ok = mbar_wait(&bars[PV_DONE + wg], (ntiles - 1) & 1, abort_flag, 350 + wg);
      if (ok) {
        tc_fence_after();
        const int qrow = q0 + wg * QT + row;
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        const uint32_t o_addr = tmem_base + lane_sel + 256 + wg * 128;
        uint16_t* dst = p.out + (static_cast<size_t>(qrow) * p.heads + head) * D;
#pragma unroll 1
        for (int cc = 0; cc < D / 32; ++cc) {
          float v[32];
          tmem_ld32(o_addr + cc * 32, v);
          if (qrow < p.Q) {
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              uint4 w;
              w.x = pack_bf16x2(v[j4 * 8 + 0] * inv, v[j4 * 8 + 1] * inv);
              w.y = pack_bf16x2(v[j4 * 8 + 2] * inv, v[j4 * 8 + 3] * inv);
              w.z = pack_bf16x2(v[j4 * 8 + 4] * inv, v[j4 * 8 + 5] * inv);
              w.w = pack_bf16x2(v[j4 * 8 + 6] * inv, v[j4 * 8 + 7] * inv);
              *reinterpret_cast<uint4*>(dst + cc * 32 + j4 * 8) = w;
            }
          }
        }
        if (qrow < p.Q)
          p.lse[static_cast<size_t>(qrow) * p.heads + head] =
              l_run > 0.f ? (m_used + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
  if (tid == 0 && *abort_flag && p.status) atomicCAS(p.status, 0, *abort_flag);
}

__global__ void fill_empty_kernel(uint16_t* out, float* lse, size_t rows, int d) {
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < rows * d) out[i] = 0;
  if (i < rows) lse[i] = -INFINITY;
}

constexpr size_t SMEM_LIMIT = 232448;  // 227 KB per CTA
long long* g_profile = nullptr;

template <int D>
int launch(const CUtensorMap maps[5], Params& p, cudaStream_t stream) {
  int nw = MAX_NW;
  while (nw > 2 && Layout<D>::bytes(nw, p.ngroups) > SMEM_LIMIT) --nw;
  size_t smem = Layout<D>::bytes(nw, p.ngroups);
  NKV_REQUIRE(smem <= SMEM_LIMIT, NKV_ERR_UNSUPPORTED,
              "codec attention needs %zu bytes of shared memory (rank/group = %d too fine)", smem,
              p.ngroups);
  p.nw = nw;
  p.prof = g_profile;
  auto kernel = attn_codec_kernel<D>;
  NKV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem)));
  dim3 grid(ceil_div(p.Q, NQ * QT), p.heads);
  kernel<<<grid, THREADS, smem, stream>>>(maps[0], maps[1], maps[2], maps[3], maps[4], p);
  NKV_LAUNCH_CHECK("attn_codec_kernel");
  return NKV_OK;
}

}  // namespace

// Development aid: 32 device int64 cycle buckets filled by CTA (0,0) of later launches
// (compute thread 0: buckets 0-12, MMA thread: 16-22); nullptr switches it off.
void tc_attn_set_profile(long long* device_buckets) { g_profile = device_buckets; }

bool tc_attn_supported(int dk, int dv, int rank) {
  return dk == dv && (dk == 64 || dk == 128) && rank % 64 == 0 && rank > 0;
}

int tc_attn_codec(const void* q, int64_t q_stride_token, int64_t q_stride_head, int Q, int heads,
                  int dk, int dv, const nkv_history* hist_k, const nkv_history* hist_v,
                  const void* wk, const float* bias_k, const void* wv, const float* bias_v,
                  float scale, void* out, float* lse, int32_t* status_word,
                  cudaStream_t stream) {
  const nkv_history& hk = *hist_k;
  const nkv_history& hv = *hist_v;
  const int N = hk.tokens, rank = hk.rank, group = hk.group;
  NKV_REQUIRE(tc_attn_supported(dk, dv, rank), NKV_ERR_UNSUPPORTED,
              "tensor-core codec attention is built for dk == dv in {64, 128} and rank %% 64 == 0 "
              "(got dk=%d dv=%d rank=%d)", dk, dv, rank);
  NKV_REQUIRE(group % 32 == 0 && rank % group == 0 && (group == 32 || group % 64 == 0),
              NKV_ERR_UNSUPPORTED, "quantisation group %d (need 32 or a multiple of 64 dividing the rank)", group);
  NKV_REQUIRE(hk.center_width % 8 == 0 && hv.center_width % 8 == 0, NKV_ERR_INVALID,
              "centre row pitch must be a multiple of 8 elements");
  NKV_REQUIRE(q_stride_head % 8 == 0 && q_stride_token % 8 == 0, NKV_ERR_INVALID,
              "query strides must be multiples of 8 elements (16 bytes)");
  if (Q == 0 || heads == 0) return NKV_OK;
  if (N == 0) {
    size_t rows = static_cast<size_t>(Q) * heads;
    fill_empty_kernel<<<static_cast<unsigned>((rows * dv + 255) / 256), 256, 0, stream>>>(
        static_cast<uint16_t*>(out), lse, rows, dv);
    NKV_LAUNCH_CHECK("fill_empty_kernel");
    return NKV_OK;
  }
  CUtensorMap maps[5];
  {
    uint64_t dims[3] = {static_cast<uint64_t>(dk), static_cast<uint64_t>(heads), static_cast<uint64_t>(Q)};
    uint64_t strides[2] = {static_cast<uint64_t>(q_stride_head) * 2, static_cast<uint64_t>(q_stride_token) * 2};
    uint32_t box[3] = {64, 1, QT};
    int rc = encode_tensor_map(&maps[0], 2, q, 3, dims, strides, box, true);
    if (rc != NKV_OK) return rc;
  }
  const void* weights[2] = {wk, wv};
  for (int w = 0; w < 2; ++w) {
    uint64_t dims[2] = {static_cast<uint64_t>(rank), static_cast<uint64_t>(heads) * dk};
    uint64_t strides[1] = {static_cast<uint64_t>(rank) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(dk)};
    int rc = encode_tensor_map(&maps[1 + w], 2, weights[w], 2, dims, strides, box, true);
    if (rc != NKV_OK) return rc;
  }
  const nkv_history* hists[2] = {&hk, &hv};
  for (int w = 0; w < 2; ++w) {
    uint64_t dims[2] = {static_cast<uint64_t>(rank / 2), static_cast<uint64_t>(N)};
    uint64_t strides[1] = {static_cast<uint64_t>(rank / 2)};
    uint32_t box[2] = {32, TOK};
    int rc = encode_tensor_map(&maps[3 + w], 1, hists[w]->codes, 2, dims, strides, box, false);
    if (rc != NKV_OK) return rc;
  }
  Params p{};
  p.Q = Q; p.heads = heads; p.N = N; p.rank = rank; p.nchunks = rank / CHUNK;
  p.group = group; p.ngroups = rank / group; p.scale_dtype = hk.scale_dtype;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.hk = hk; p.hv = hv; p.bias_k = bias_k; p.bias_v = bias_v;
  p.out = static_cast<uint16_t*>(out); p.lse = lse; p.status = status_word;
  return dk == 128 ? launch<128>(maps, p, stream) : launch<64>(maps, p, stream);
}

}  // namespace nkv
