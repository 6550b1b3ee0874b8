// Fused codec-attention on tcgen05 tensor cores (bf16 operands, fp32 TMEM
// accumulators), with the K/V reconstruction shared inside a thread-block cluster.
//
// A CTA owns one head and up to 256 queries (two 128-row query tiles) and walks
// the compressed history in tiles of 128 tokens.  The CL CTAs of a cluster serve
// CL consecutive query blocks of the SAME head, so they all need the same K and
// V tile.  Each of them rebuilds one 64-column part of it (CL = 4: K columns
// 0-63 / 64-127, V columns 0-63 / 64-127) and stores that part into the shared
// memory of every CTA of the cluster (distributed shared memory), which divides
// the decode GEMM, the dequantisation and the decoder-matrix traffic by CL.
// Per tile and CTA:
//   1. TMA streams the packed INT4 codes of the tile (of this CTA's tensor) and
//      64 rows of the head's decoder (or reader) slice, 64 latent columns at a
//      time, through a ring of NW slots; the compute warps expand the codes to
//      bf16 latent rows (code * stored scale, one rounding) into tensor memory,
//      where they are the A operand of the decode MMA,
//   2. tcgen05.mma rebuilds the [128 tok x 64] part in TMEM; the compute warps
//      add bias and the token's centre row with the reference's two bf16
//      roundings and store K (row-major) or V (transposed) into all CL CTAs --
//      K and V never exist in global memory,
//   3. S = Q K^T per query tile in TMEM, online softmax in registers (exp2, lazy
//      rescaling of the O accumulator); P replaces S in TMEM as bf16 pairs,
//   4. O += P V (P from TMEM, V from shared memory) in TMEM.
// Warp roles: warps 0-7 compute (dequantise / epilogue / softmax), warp 8 lane 0
// issues TMA, warp 9 lane 0 issues MMA, warp 10 prefetches per-token metadata
// (centre row, scales) two tiles ahead.  All hand-offs are mbarriers with
// bounded waits (see nkv_tc.cuh); peers signal each other with cluster-scope
// arrivals and multicast commits.  No TMA load uses multicast.
//
// TMEM columns: [0,128) S of query tile 0 (decode accumulator in [0,64));
// [128,256) S of tile 1; latent staging slots of 32 columns at 64, 96, 192, 224; [256,384) O
// tile 0; [384,512) O tile 1.
#include <type_traits>

#include "nkv_internal.h"
#include "nkv_tc.cuh"

namespace nkv {
namespace {

using namespace tc;

constexpr int TOK = 128;          // history tokens per tile
constexpr int QT = 128;           // queries per query tile
constexpr int NQ = 2;             // query tiles per CTA
constexpr int COMPUTE_THREADS = 256;
constexpr int COMPUTE_WARPS = COMPUTE_THREADS / 32;
constexpr int THREADS = COMPUTE_THREADS + 96;
constexpr int CHUNK = 64;         // latent columns per pipeline step
constexpr int PART = 64;          // K/V columns rebuilt by one CTA
constexpr int TILE_BYTES = 128 * 128;  // one [128 rows x 64 bf16] swizzled tile
constexpr int MAX_NW = 4;         // decoder-row ring slots in shared memory; a slot holds the rows of a
                                  // PAIR of 64-column latent chunks (as many slots as fit, at least 2)
#ifndef NKV_NSTAGE
#define NKV_NSTAGE 2              // 3 (third slot in P1's columns) measured 2 % slower on H 40 x D 128, r 640
#endif
constexpr int NSTAGE = NKV_NSTAGE;  // latent staging slots in tensor memory (a pair of chunks each);
                                    // pair i of a tile uses slot i % NSTAGE
constexpr int NDONE = 8;          // "MMAs of pair g are complete" barriers, indexed by g % 8
constexpr float RESCALE_THRESHOLD = 8.0f;

enum Bar {
  Q_FULL = 0, W_FULL = 1, PAIR_DONE = 5, LAT_FULL = 13,
  META_FULL = 22, META_FREE = 24, KV_READY = 26, KV_FREE = 27, S_FULL = 28, P_READY = 30,
  PV_DONE = 32, EPI_LOCAL = 34, CODES_FULL = 35, CODES_FREE = 36, NUM_BARS = 37
};

struct Params {
  int Q, heads, N, rank, nchunks, ngroups, group;
  int scale_dtype, nw;
  int w_perm;            // decoder rows are in kernel order (tc_prepare_decoder)
  int tiles_per_split;   // grid.z splits the history; split z writes partial (O, lse) number z
  float scale_log2;
  nkv_history hk, hv;
  const float* bias_k;
  const float* bias_v;
  uint16_t* out;
  float* lse;
  int32_t* status;
  nkv_rope rope;     // cos_sin == nullptr: keys are used as rebuilt
  nkv_camera cam_k, cam_v;   // matrices == nullptr: no camera transform of that tensor
  long long* prof;   // optional: cycle buckets of CTA (0,0), see nkv_debug_attn_profile
};

template <int D>
struct Layout {
  static constexpr int CL = D / PART * 2;                // CTAs per cluster: 4 (D 128) or 2 (D 64)
  static constexpr int DCH = D / 64;                     // 64-column chunks of a head row
  static constexpr int Q_OFF = 0;                        // [NQ][DCH] tiles
  static constexpr int K_OFF = Q_OFF + NQ * DCH * TILE_BYTES;   // [DCH] tiles [128 tok x 64]
  static constexpr int VT_OFF = K_OFF + DCH * TILE_BYTES;       // V: [DCH] tiles [128 tok x 64], like K
  static constexpr int VT_TILE = D * 128;                       // (2 * VT_TILE == DCH * TILE_BYTES)
  // codes of the tile: one [128 tok x 64 byte] block per pair of latent chunks, 64-byte swizzle
  // (rows 64 bytes apart would put a quarter-warp's 16-byte reads on two bank groups)
  static constexpr int CODES_OFF = VT_OFF + 2 * VT_TILE;
  static constexpr int CODE_BLOCK = TOK * 64;
  // centre staging of the epilogue (8 warps x 2 KB) reuses the head of the code buffer: the codes
  // of a tile are all expanded before its epilogue starts, and the next tile's codes are only
  // requested (CODES_FREE) after the staging has been read back
  static constexpr int SCRATCH_OFF = CODES_OFF;
  __host__ __device__ static int codes_bytes(int rank) {
    const int bytes = ((rank / CHUNK + 1) / 2) * CODE_BLOCK;
    return bytes < TILE_BYTES ? TILE_BYTES : bytes;
  }
  __host__ __device__ static int ring_off(int rank) { return CODES_OFF + codes_bytes(rank); }
  static constexpr int CHUNK_BYTES = PART * 128;         // [64 decoder rows x 64 latent cols]
  static constexpr int SLOT_BYTES = 2 * CHUNK_BYTES;     // a pair of chunks
  __host__ __device__ static int meta_off(int nw, int rank) { return ring_off(rank) + nw * SLOT_BYTES; }
  // meta: bars, tmem slot, abort, bias [64] floats, then two metadata buffers of
  // crow [128] ints and scales [128][ngroups] u16
  static constexpr int BARS = 0;
  static constexpr int SLOT = NUM_BARS * 8;
  static constexpr int ABORT = SLOT + 4;
  static constexpr int BIAS = ((ABORT + 4 + 15) / 16) * 16;
  static constexpr int PAIRS = BIAS + PART * 4;          // [PART / 2] native pair of each pair of the part
  static constexpr int CAMS = PAIRS + (PART / 2) * 4;   // [PART / 8] camera of each block of the part
  static constexpr int CROW = CAMS + (PART / 8) * 4;
  static constexpr int SCALES = CROW + 2 * TOK * 4;
  static size_t bytes(int nw, int ngroups, int rank) {
    return meta_off(nw, rank) + SCALES + 2 * TOK * ngroups * 2 + 1024;
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

// One arrival per warp: 32 lanes arriving on the same mbarrier are 32 serialised shared-memory
// atomics; the lanes synchronise (which orders their earlier accesses and fences before lane 0's
// releasing arrive) and lane 0 arrives for the warp.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// Kernel-order variants: the decoder rows were prepared (tc_prepare_decoder) so that within every
// group of 8 latent columns the order is e0 e2 e4 e6 e1 e3 e5 e7.  The even elements are the low
// nibbles of a code word and the odd ones its high nibbles, so a byte permute against the constant
// 0x43 builds each bf16 pair directly (4 PRMT per 8 elements instead of 4 PRMT + 4 LOP3: the
// integer pipe is what bounds the expansion).
__device__ __forceinline__ uint4 dequant8_bf16_perm(uint32_t word, __nv_bfloat162 scale2) {
  const uint32_t lo = word & 0x0F0F0F0Fu, hi = (word >> 4) & 0x0F0F0F0Fu, magic = 0x43434343u;
  const uint32_t t[4] = {__byte_perm(lo, magic, 0x4140), __byte_perm(lo, magic, 0x4342),
                         __byte_perm(hi, magic, 0x4140), __byte_perm(hi, magic, 0x4342)};
  const uint32_t bias_bits = 0x43074307u;   // bf16 pair (135, 135)
  const __nv_bfloat162 bias2 = *reinterpret_cast<const __nv_bfloat162*>(&bias_bits);
  uint4 r;
  uint32_t* o = &r.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 v = __hmul2(__hsub2(*reinterpret_cast<const __nv_bfloat162*>(&t[i]), bias2), scale2);
    o[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  return r;
}

__device__ __forceinline__ uint4 dequant8_perm(uint32_t word, float scale) {
  float e[8];
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const uint32_t byte = (word >> (8 * b)) & 0xFFu;
    e[2 * b] = static_cast<float>(static_cast<int>(byte & 15u) - 7) * scale;
    e[2 * b + 1] = static_cast<float>(static_cast<int>(byte >> 4) - 7) * scale;
  }
  return make_uint4(pack_bf16x2(e[0], e[2]), pack_bf16x2(e[4], e[6]), pack_bf16x2(e[1], e[3]),
                    pack_bf16x2(e[5], e[7]));
}

// 2^x as the bare exponential-unit instruction (results below 2^-126 flush to zero, which is
// what a softmax weight that small is worth)
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// TMEM column of latent staging slot s (a pair of chunks = 64 columns).  Slots 0 and 1 avoid the
// columns where P of the previous tile may still be read by its PV MMAs (P0 in [0,64), P1 in
// [128,192)), so the next tile's first two pairs can be expanded while those MMAs run; slot 2 is
// P1's place and is first written at pair 2, after a wait for PV_DONE of the second query tile.
__device__ __forceinline__ uint32_t staging_col(int s) { return s == 0 ? 64 : (s == 1 ? 192 : 128); }

// Lap timer of one thread: adds the cycles since the previous lap to a bucket kept in registers;
// flush() adds the buckets to global memory once, at the end.
// The PROF = false specialisation is empty, so the production kernel carries no timers.
template <bool PROF>
struct Laps {
  __device__ __forceinline__ void start(long long*, bool) {}
  __device__ __forceinline__ void lap(int) {}
  __device__ __forceinline__ void flush() {}
};

template <>
struct Laps<true> {
  long long* out;
  unsigned last;
  unsigned acc[13];
  __device__ __forceinline__ void start(long long* dst, bool on) {
    out = on ? dst : nullptr;
#pragma unroll
    for (int i = 0; i < 13; ++i) acc[i] = 0;
    last = static_cast<unsigned>(clock64());
  }
  __device__ __forceinline__ void lap(int bucket) {
    if (out) {
      const unsigned now = static_cast<unsigned>(clock64());
#pragma unroll
      for (int i = 0; i < 13; ++i)
        if (i == bucket) acc[i] += now - last;
      last = now;
    }
  }
  __device__ __forceinline__ void flush() {
    if (out) {
#pragma unroll
      for (int i = 0; i < 13; ++i) out[i] += acc[i];
    }
  }
};

template <int D, bool ROPE, bool CAM, bool PROF>
__global__ void __launch_bounds__(THREADS, 1)
attn_codec_kernel(const __grid_constant__ CUtensorMap map_q,
                  const __grid_constant__ CUtensorMap map_wk,
                  const __grid_constant__ CUtensorMap map_wv,
                  const __grid_constant__ CUtensorMap map_ck,
                  const __grid_constant__ CUtensorMap map_cv, Params p) {
  using L = Layout<D>;
  constexpr int CL = L::CL;
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared window starts at the same offset in every CTA of the cluster, so the
  // aligned base (and every offset from it) names the same location in each peer
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int nw = p.nw;
  uint8_t* meta = smem + L::meta_off(nw, p.rank);
  const int ring_off = L::ring_off(p.rank);
  uint64_t* bars = reinterpret_cast<uint64_t*>(meta + L::BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(meta + L::SLOT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(meta + L::ABORT);
  float* bias = reinterpret_cast<float*>(meta + L::BIAS);            // [64] of this CTA's part
  int* pair_sel = reinterpret_cast<int*>(meta + L::PAIRS);           // [32] (positional restore)
  int* cam_sel = reinterpret_cast<int*>(meta + L::CAMS);             // [8] (camera transform)
  int* crow = reinterpret_cast<int*>(meta + L::CROW);                // [2 buf][128]
  uint16_t* scales = reinterpret_cast<uint16_t*>(meta + L::SCALES);  // [2 buf][128][ngroups]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y;
  const uint32_t rank = cluster_ctarank();
  const int tensor = static_cast<int>(rank) / (CL / 2);   // 0: this CTA rebuilds K columns, 1: V
  const int part = static_cast<int>(rank) % (CL / 2);     // which 64-column part of the head row
  const nkv_history& hist = tensor ? p.hv : p.hk;
  const int q0 = blockIdx.x * (NQ * QT);
  const int nq = q0 >= p.Q ? 0 : ((q0 + QT < p.Q) ? 2 : 1);   // 0: decode duty only
  const int tile0 = blockIdx.z * p.tiles_per_split;       // first history tile of this split
  const int ntiles = max(0, min((p.N + TOK - 1) / TOK - tile0, p.tiles_per_split));
  const int nchunks = p.nchunks;
  const int ng = p.ngroups;

  if (tid == 0) {
    mbar_init(&bars[Q_FULL], 1);
    for (int s = 0; s < MAX_NW; ++s) mbar_init(&bars[W_FULL + s], 1);   // TMA: decoder rows of a pair landed
    for (int s = 0; s < NSTAGE; ++s) mbar_init(&bars[LAT_FULL + s], COMPUTE_WARPS);  // latent pair staged in TMEM
    for (int s = 0; s < NDONE; ++s) mbar_init(&bars[PAIR_DONE + s], 1);  // the pair's MMAs are complete
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[META_FULL + s], 1);
      mbar_init(&bars[META_FREE + s], COMPUTE_WARPS);
      mbar_init(&bars[S_FULL + s], 1);
      mbar_init(&bars[P_READY + s], QT / 32);
      mbar_init(&bars[PV_DONE + s], 1);
    }
    mbar_init(&bars[KV_READY], 1);                    // local arrival + bytes copied in by the peers
    mbar_init(&bars[EPI_LOCAL], COMPUTE_WARPS);     // this CTA's part is in its own shared memory
    mbar_init(&bars[KV_FREE], CL);
    mbar_init(&bars[CODES_FULL], 1);                  // the tile's codes landed (one bulk copy)
    mbar_init(&bars[CODES_FREE], COMPUTE_WARPS);    // every thread is done expanding them                    // one arrival per CTA: its reads are done
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  for (int i = tid; i < PART; i += THREADS)
    bias[i] = (tensor ? p.bias_v : p.bias_k)[head * D + part * PART + i];
  if (CAM) {
    const nkv_camera& cam = tensor ? p.cam_v : p.cam_k;
    for (int i = tid; i < PART / 8; i += THREADS)
      cam_sel[i] = cam.matrices ? (cam.cam_index[head * (D / 8) + part * (PART / 8) + i] & 3) : 0;
  }
  if (ROPE) {
    for (int i = tid; i < PART / 2; i += THREADS) {
      const int local = part * (PART / 2) + i;
      pair_sel[i] = p.rope.pair_index ? p.rope.pair_index[head * (D / 2) + local] : local;
    }
  }
  if (warp == 9) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // every CTA's barriers exist before any peer signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const CUtensorMap* map_w = tensor ? &map_wv : &map_wk;
      const CUtensorMap* map_c = tensor ? &map_cv : &map_ck;
      prefetch_tensormap(map_w);
      prefetch_tensormap(map_c);
      if (nq > 0) {
        prefetch_tensormap(&map_q);
        mbar_arrive_expect_tx(&bars[Q_FULL], nq * L::DCH * TILE_BYTES);
        for (int i = 0; i < nq; ++i)
          for (int c = 0; c < L::DCH; ++c)
            tma_load_3d(smem + L::Q_OFF + (i * L::DCH + c) * TILE_BYTES, &map_q, c * 64, head,
                        q0 + i * QT, &bars[Q_FULL]);
      }
      bool ok = true;
      int slot = 0, use = 0, g = 0;   // g: running pair number over all tiles
      for (int it = 0; it < ntiles && ok; ++it) {
        // the tile's codes: rows are contiguous in the history, so one untiled bulk copy; it is
        // issued as soon as the previous tile's codes are expanded and lands during that tile's
        // epilogue / exchange / attention
        if (it > 0) ok = mbar_wait(&bars[CODES_FREE], (it - 1) & 1, abort_flag, 108);
        if (!ok) break;
        {
          const int npairs = (nchunks + 1) / 2;
          mbar_arrive_expect_tx(&bars[CODES_FULL], npairs * L::CODE_BLOCK);
          for (int pi = 0; pi < npairs; ++pi)   // bytes past the row or the history read as zero
            tma_load_2d(smem + L::CODES_OFF + pi * L::CODE_BLOCK, map_c, pi * 64, (tile0 + it) * TOK,
                        &bars[CODES_FULL]);
        }
        for (int c = 0; c < nchunks && ok; c += 2) {
          const int n = min(2, nchunks - c);     // chunks in this pair
          // the slot's previous tenant was pair g - nw
          if (g >= nw)
            ok = mbar_wait(&bars[PAIR_DONE + ((g - nw) & (NDONE - 1))], ((g - nw) / NDONE) & 1,
                           abort_flag, 110 + slot);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars[W_FULL + slot], n * L::CHUNK_BYTES);
          for (int j = 0; j < n; ++j)
            tma_load_2d(smem + ring_off + slot * L::SLOT_BYTES + j * L::CHUNK_BYTES, map_w,
                        (c + j) * CHUNK, head * D + part * PART, &bars[W_FULL + slot]);
          ++g;
          if (++slot == nw) { slot = 0; ++use; }
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
    // the whole warp runs the (uniform) control flow; one elected lane issues
    {
      const bool leader = elect_one();
      const uint32_t idesc_dec = make_idesc_bf16(128, PART);  // [128 tok] x [64 columns]
      const uint32_t idesc_s = make_idesc_bf16(128, TOK);     // [128 q] x [128 tok]
      const uint32_t idesc_pv = make_idesc_bf16(128, D) | (1u << 16);   // [128 q] x [D], B (V) MN-major
      const uint32_t smem_base = smem_u32(smem);
      const uint16_t all_ctas = static_cast<uint16_t>((1u << CL) - 1);
      Laps<PROF> laps;
      laps.start(p.prof + 16, leader && p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0);
      bool ok = nq > 0 ? mbar_wait(&bars[Q_FULL], 0, abort_flag, 200) : true;
      int slot = 0, use = 0, g = 0;   // decoder-row ring position; running pair number
      uint32_t lat_phase = 0;         // bit s: parity of the next completion of LAT_FULL[s]
      for (int it = 0; it < ntiles && ok; ++it) {
        int st = 0;
        for (int c = 0; c < nchunks && ok; c += 2) {
          const int n = min(2, nchunks - c);
          ok = mbar_wait(&bars[W_FULL + slot], use & 1, abort_flag, 210 + slot);
          laps.lap(0);
          ok = ok && mbar_wait(&bars[LAT_FULL + st], (lat_phase >> st) & 1, abort_flag, 216 + st);
          lat_phase ^= 1u << st;
          laps.lap(1);
          if (!ok) break;
          tc_fence_after();
          // descriptors are built once per chunk; a K = 16 step adds 32 bytes (2 in the address
          // field) to the shared-memory operand and 8 columns to the TMEM operand
          for (int j = 0; j < n; ++j) {
            const uint64_t w_desc = make_smem_desc_sw128(smem_base + ring_off + slot * L::SLOT_BYTES +
                                                         j * L::CHUNK_BYTES);
            const uint32_t lat = tmem_base + staging_col(st) + j * 32;   // chunk staged in TMEM
            if (leader) mma_bf16_ts(tmem_base, lat, w_desc, idesc_dec, c + j > 0);
            if (leader) mma_bf16_ts(tmem_base, lat + 8, w_desc + 2, idesc_dec, true);
            if (leader) mma_bf16_ts(tmem_base, lat + 16, w_desc + 4, idesc_dec, true);
            if (leader) mma_bf16_ts(tmem_base, lat + 24, w_desc + 6, idesc_dec, true);
          }
          // frees the decoder rows and the staging; on the last pair: accumulator done
          if (leader) mma_commit(&bars[PAIR_DONE + (g & (NDONE - 1))]);
          ++g;
          if (++slot == nw) { slot = 0; ++use; }
          if (++st == NSTAGE) st = 0;
          laps.lap(2);
        }
        if (!ok) break;
        // exchange: once this CTA's part is complete locally and every CTA has finished reading
        // the previous tile, copy the part into each peer (asynchronous shared-to-shared copies
        // that report to the peer's KV_READY), then wait for the peers' parts to land here
        ok = mbar_wait(&bars[EPI_LOCAL], it & 1, abort_flag, 218);
        if (ok && it > 0) ok = mbar_wait_cluster(&bars[KV_FREE], (it - 1) & 1, abort_flag, 219);
        laps.lap(7);
        if (!ok) break;
        {
          const uint32_t ready = smem_u32(&bars[KV_READY]);
          for (uint32_t step = 1; step < CL; ++step) {
            const uint32_t peer = (rank + step) % CL;
            const uint32_t peer_ready = map_to_cta(ready, peer);
            // K and V are both stored token-major, one [128 tok x 64 col] tile per part
            const uint32_t src = smem_base + (tensor == 0 ? L::K_OFF : L::VT_OFF) + part * TILE_BYTES;
            if (leader) bulk_copy_to_peer(map_to_cta(src, peer), src, TILE_BYTES, peer_ready);
          }
          if (leader) mbar_arrive_expect_tx(&bars[KV_READY], (CL - 1) * TILE_BYTES);
        }
        ok = mbar_wait_cluster(&bars[KV_READY], it & 1, abort_flag, 220);
        laps.lap(3);
        if (!ok) break;
        tc_fence_after();
        for (int i = 0; i < nq; ++i) {
#pragma unroll
          for (int ch = 0; ch < L::DCH; ++ch) {
            const uint64_t a_desc = make_smem_desc_sw128(smem_base + L::Q_OFF + (i * L::DCH + ch) * TILE_BYTES);
            const uint64_t b_desc = make_smem_desc_sw128(smem_base + L::K_OFF + ch * TILE_BYTES);
            if (leader) mma_bf16(tmem_base + i * 128, a_desc, b_desc, idesc_s, ch > 0);
            if (leader) mma_bf16(tmem_base + i * 128, a_desc + 2, b_desc + 2, idesc_s, true);
            if (leader) mma_bf16(tmem_base + i * 128, a_desc + 4, b_desc + 4, idesc_s, true);
            if (leader) mma_bf16(tmem_base + i * 128, a_desc + 6, b_desc + 6, idesc_s, true);
          }
          if (leader) mma_commit(&bars[S_FULL + i]);
        }
        for (int i = 0; i < nq && ok; ++i) {
          laps.lap(4);
          ok = mbar_wait(&bars[P_READY + i], it & 1, abort_flag, 230 + i);
          laps.lap(5);
          if (!ok) break;
          tc_fence_after();
          // P (bf16 pairs) sits in the first 64 columns of the S region it was computed from
          // V is the B operand in MN-major form: [tokens (K) x d (N)] with d contiguous, 64-column
          // tiles 16 KB apart (leading offset), 8-token groups 1 KB apart (stride offset); a K step
          // of 16 tokens moves the start by 2 KB (128 in the address field)
          {
            const uint64_t b_desc = make_smem_desc_sw128_mn(smem_base + L::VT_OFF, TILE_BYTES);
            const uint32_t p_addr = tmem_base + i * 128;
            const uint32_t o_addr = tmem_base + 256 + i * 128;
#pragma unroll
            for (int ks = 0; ks < TOK / 16; ++ks)
              if (leader) mma_bf16_ts(o_addr, p_addr + 8 * ks, b_desc + 128 * ks, idesc_pv, it > 0 || ks > 0);
          }
          if (leader) mma_commit(&bars[PV_DONE + i]);
        }
        if (!ok) break;
        // tell every CTA of the cluster that this CTA no longer reads the tile's K / V
        if (nq > 0) {
          if (leader) mma_commit_multicast(&bars[KV_FREE], all_ctas);
        } else {
          const uint32_t local = smem_u32(&bars[KV_FREE]);
          for (uint32_t peer = 0; peer < CL; ++peer) if (leader) mbar_arrive_cluster(map_to_cta(local, peer));
        }
        laps.lap(6);
      }
      laps.flush();
    }
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------------------------- per-token metadata, two tiles ahead
    bool ok = true;
    for (int it = 0; it < ntiles && ok; ++it) {
      const int b = it & 1, u = it >> 1;
      if (u >= 1) ok = mbar_wait(&bars[META_FREE + b], (u - 1) & 1, abort_flag, 240 + b);
      if (!ok) break;
      const int t0 = (tile0 + it) * TOK;
      for (int r = lane; r < TOK; r += 32) {
        const int t = t0 + r;
        const bool in = t < p.N;
        crow[b * TOK + r] = in ? center_row_of(hist, t) : 0;
        const uint16_t* src = static_cast<const uint16_t*>(hist.scales) + static_cast<size_t>(t) * ng;
        uint16_t* dst = scales + static_cast<size_t>(b * TOK + r) * ng;
        for (int gi = 0; gi < ng; ++gi) dst[gi] = in ? src[gi] : 0;
      }
      warp_arrive(&bars[META_FULL + b], lane);
    }
  } else {
    // ------------------------------------------------------------ compute warps
    const int wg = tid >> 7;                    // query tile served; also the 32-column half of the part
    const int row = tid & 127;                  // TMEM lane == token row == query row
    const uint32_t lane_sel = static_cast<uint32_t>(32 * (warp & 3)) << 16;
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    int g = 0;   // running pair number over all tiles
    Laps<PROF> laps;
    laps.start(p.prof, p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0);
    for (int it = 0; it < ntiles && ok; ++it) {
      const int t0 = (tile0 + it) * TOK;
      const int valid = min(TOK, p.N - t0);
      const int mb = it & 1;
      if (it > 0) {  // every thread has finished reading S of the previous tile (staging reuses it)
        for (int i = 0; i < nq && ok; ++i)
          ok = mbar_wait(&bars[P_READY + i], (it - 1) & 1, abort_flag, 300 + i);
        if (!ok) break;
      }
      laps.lap(0);
      ok = mbar_wait(&bars[META_FULL + mb], (it >> 1) & 1, abort_flag, 310);
      laps.lap(1);
      if (!ok) break;
      // ---- expand this CTA's codes to bf16 latent chunks in tensor memory (A of the decode MMA)
      ok = mbar_wait(&bars[CODES_FULL], it & 1, abort_flag, 318);
      laps.lap(3);
      if (!ok) break;
      // this thread's 16 bytes of chunk j of pair pi: 16-byte unit 2 j + wg of row `row`, swizzled
      const uint8_t* codes = smem + L::CODES_OFF + row * 64;
      const int unit_xor = (row >> 1) & 3;
      auto code_at = [&](int c) {
        return *reinterpret_cast<const uint4*>(codes + (c >> 1) * L::CODE_BLOCK +
                                               ((((c & 1) * 2 + wg) ^ unit_xor) << 4));
      };
      const uint16_t* my_scales = scales + static_cast<size_t>(mb * TOK + row) * ng;
      // codes of the pair after the one being expanded are fetched ahead of the wait for its slot
      uint4 code_next[2];
      code_next[0] = code_at(0);
      code_next[1] = nchunks > 1 ? code_at(1) : make_uint4(0, 0, 0, 0);
      int st = 0;
      // The pair loop exists twice: FASTQ is the common deployment (one bf16 scale per token,
      // decoder rows in kernel order) with every choice made at compile time; the other copy keeps
      // the run-time choices (grouped or fp16 scales, natural-order rows).  Picking between them
      // inside the loop instead costs 7 % of the kernel.
      auto expand_pairs = [&](auto fast_tag) {
        constexpr bool FASTQ = decltype(fast_tag)::value;
        for (int c0 = 0; c0 < nchunks && ok; c0 += 2) {
          const int n = min(2, nchunks - c0);   // chunks in this pair
          const uint4 code_cur[2] = {code_next[0], code_next[1]};
          if (c0 + 2 < nchunks) code_next[0] = code_at(c0 + 2);
          if (c0 + 3 < nchunks) code_next[1] = code_at(c0 + 3);
          laps.lap(5);
          // The staging slot's previous tenant in this tile is pair g - NSTAGE.  The first NSTAGE pairs
          // of a tile follow pairs of the previous tile, all complete (its epilogue waited for the last
          // one); slot 2 is also where P of the second query tile sat, read by that tile's PV MMAs.
          if (c0 >= 2 * NSTAGE)
            ok = mbar_wait(&bars[PAIR_DONE + ((g - NSTAGE) & (NDONE - 1))], ((g - NSTAGE) / NDONE) & 1,
                           abort_flag, 320 + st);
          else if (c0 == 4 && it > 0 && nq == 2)
            ok = mbar_wait(&bars[PV_DONE + 1], (it - 1) & 1, abort_flag, 323);
          laps.lap(2);
          if (!ok) break;
          tc_fence_after();
  #pragma unroll
          for (int j = 0; j < 2; ++j) {
            if (j < n) {
              const int c = c0 + j;
              const uint4 code = code_cur[j];
              const int col0 = c * CHUNK + wg * 32;   // this thread: token `row`, latent columns col0 .. +32
              const int gi = (FASTQ || ng == 1) ? 0 : (p.group == 32 ? 2 * c + wg : col0 / p.group);
              const uint16_t sbits = my_scales[gi];
              const uint32_t words[4] = {code.x, code.y, code.z, code.w};
              uint32_t packed[16];
              if (FASTQ || p.scale_dtype == NKV_BF16) {
                const uint32_t pair = static_cast<uint32_t>(sbits) * 0x00010001u;
                const __nv_bfloat162 scale2 = *reinterpret_cast<const __nv_bfloat162*>(&pair);
  #pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const uint4 v = (FASTQ || p.w_perm) ? dequant8_bf16_perm(words[k], scale2)
                                                       : dequant8_bf16(words[k], scale2);
                  packed[4 * k] = v.x; packed[4 * k + 1] = v.y; packed[4 * k + 2] = v.z; packed[4 * k + 3] = v.w;
                }
              } else {
                const float sc = scale_to_float(sbits, p.scale_dtype);
  #pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const uint4 v = p.w_perm ? dequant8_perm(words[k], sc) : dequant8(words[k], sc);
                  packed[4 * k] = v.x; packed[4 * k + 1] = v.y; packed[4 * k + 2] = v.z; packed[4 * k + 3] = v.w;
                }
              }
              tmem_st16(tmem_base + lane_sel + staging_col(st) + j * 32 + wg * 16, packed);
            }
          }
          tmem_wait_st();
          tc_fence_before();
          warp_arrive(&bars[LAT_FULL + st], lane);
          laps.lap(4);
          ++g;
          if (++st == NSTAGE) st = 0;
        }
      };
      if (p.w_perm && p.scale_dtype == NKV_BF16 && ng == 1) expand_pairs(std::true_type{});
      else expand_pairs(std::false_type{});
      if (!ok) break;
      // ---- epilogue of this CTA's part: bias, centre, two bf16 roundings, store to every CTA
      {
        const bool in = row < valid;
        // Centre rows of this warp's 32 tokens (32 columns = 64 bytes each), gathered
        // cooperatively: 4 lanes read one row's 16-byte pieces, so a load instruction touches
        // 8 lines instead of 32; the rows are redistributed through a swizzled staging area.
        constexpr int PIECES = 4, RPI = 8;
        const int wrow0 = 32 * (warp & 3);
        const uint16_t* cbase = static_cast<const uint16_t*>(hist.centers) +
                                static_cast<size_t>(head) * D + part * PART + wg * 32;
        uint4 cen[PIECES];
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
          const int rloc = i * RPI + lane / PIECES, piece = lane % PIECES;
          const int crow_i = crow[mb * TOK + wrow0 + rloc];
          cen[i] = __ldg(reinterpret_cast<const uint4*>(
              cbase + static_cast<size_t>(crow_i) * hist.center_width + piece * 8));
        }
        // positional restore (K parts only): this token's frame / row / column
        const bool rotate = ROPE && tensor == 0 && p.rope.cos_sin != nullptr;
        int coord_t = 0, coord_h = 0, coord_w = 0;
        const int band_a = p.rope.table_half - 2 * (p.rope.table_half / 3);
        const int band_b = band_a + p.rope.table_half / 3;
        if (rotate) {
          const int pos = in ? max(__ldg(p.rope.positions + t0 + row), 0) : 0;
          const int last = p.rope.table_rows - 1;
          if (p.rope.frame_seqlen == 0) {   // one table row per token: every band reads row `pos`
            coord_t = coord_h = coord_w = min(pos, last);
          } else {
            const int frame = pos / p.rope.frame_seqlen, spatial = pos - frame * p.rope.frame_seqlen;
            const int prow = spatial / p.rope.width;
            coord_t = min(frame, last);
            coord_h = min(prow, last);
            coord_w = min(spatial - prow * p.rope.width, last);
          }
        }
        // camera transform: this token's frame picks the 4 x 4 matrices
        const nkv_camera& cam = tensor ? p.cam_v : p.cam_k;
        const bool transform = CAM && cam.matrices != nullptr;
        const float* cam_frame = nullptr;
        if (transform)
          cam_frame = cam.matrices +
                      static_cast<size_t>(min((t0 + row) / cam.tokens_per_frame, cam.frames - 1)) * 64;
        // rotation entries of this thread's 16 pairs, requested before the accumulator wait
        float2 rot[16];
        if (ROPE) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            rot[i] = make_float2(1.f, 0.f);
            if (rotate) {
              const int pg = pair_sel[wg * 16 + i];   // native pair this pair retains
              const int coord = pg < band_a ? coord_t : (pg < band_b ? coord_h : coord_w);
              rot[i] = __ldg(reinterpret_cast<const float2*>(p.rope.cos_sin) +
                             static_cast<size_t>(coord) * p.rope.table_half + pg);
            }
          }
        }
        laps.lap(6);
        // accumulator complete: the tile's last pair is pair g - 1
        ok = mbar_wait(&bars[PAIR_DONE + ((g - 1) & (NDONE - 1))], ((g - 1) / NDONE) & 1, abort_flag, 330);
        laps.lap(7);
        if (!ok) break;
        tc_fence_after();
        // the accumulator read stays in flight under the centre staging
        uint32_t acc_raw[32];
        tmem_ld32_issue(tmem_base + lane_sel + wg * 32, acc_raw);
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
          // the staging lived in the code buffer: only now may the next tile's codes overwrite it
          fence_proxy_async();
          warp_arrive(&bars[CODES_FREE], lane);
        }
        tmem_ld32_wait(acc_raw);
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc_raw[i]);
        uint32_t packed[16];
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          const uint32_t cwords[4] = {cen[j4].x, cen[j4].y, cen[j4].z, cen[j4].w};
          float block[8];   // the 8-wide block j4 of this thread's columns (camera transform only)
          if (!ROPE && !CAM) {
            // plain rebuild in packed bf16 arithmetic: bf16x2(acc + bias) then one bf16x2 add of the
            // centre word -- the same two roundings (the sum of two bf16 numbers is exact in fp32
            // unless the smaller one lies below the rounding step of the larger either way)
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const int j = j4 * 8 + w * 2;
              const uint32_t first = pack_bf16x2(v[j] + bias[wg * 32 + j], v[j + 1] + bias[wg * 32 + j + 1]);
              const __nv_bfloat162 sum = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&first),
                                                 *reinterpret_cast<const __nv_bfloat162*>(&cwords[w]));
              packed[j4 * 4 + w] = in ? *reinterpret_cast<const uint32_t*>(&sum) : 0u;
            }
            continue;
          }
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const int j = j4 * 8 + w * 2;
            // the rebuilt pair in packed bf16 arithmetic (as above), then widened for the transforms
            const uint32_t first = pack_bf16x2(v[j] + bias[wg * 32 + j], v[j + 1] + bias[wg * 32 + j + 1]);
            const __nv_bfloat162 sum = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&first),
                                               *reinterpret_cast<const __nv_bfloat162*>(&cwords[w]));
            const uint32_t rebuilt = *reinterpret_cast<const uint32_t*>(&sum);
            float x0 = __uint_as_float(rebuilt << 16), x1 = __uint_as_float(rebuilt & 0xFFFF0000u);
            if (rotate) {   // the pair (x0, x1) of the rebuilt bf16 key is one complex number
              const float2 cs = rot[j >> 1];
              const float k0 = x0, k1 = x1;
              x0 = fmaf(k0, cs.x, -(k1 * cs.y));
              x1 = fmaf(k0, cs.y, k1 * cs.x);
            }
            if (CAM) {
              block[2 * w] = x0;
              block[2 * w + 1] = x1;
            }
            packed[j4 * 4 + w] = in ? pack_bf16x2(x0, x1) : 0u;
          }
          if (transform) {   // slots (w) of the block are mixed by the token's 4 x 4 camera matrix
            const float4* m = reinterpret_cast<const float4*>(cam_frame + cam_sel[wg * 4 + j4] * 16);
#pragma unroll
            for (int k = 0; k < 8; ++k) block[k] = round_to_bf16(block[k]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 mi = __ldg(m + i);
              const float m0 = round_to_bf16(mi.x), m1 = round_to_bf16(mi.y);
              const float m2 = round_to_bf16(mi.z), m3 = round_to_bf16(mi.w);
              const float y0 = fmaf(m3, block[6], fmaf(m2, block[4], fmaf(m1, block[2], m0 * block[0])));
              const float y1 = fmaf(m3, block[7], fmaf(m2, block[5], fmaf(m1, block[3], m0 * block[1])));
              packed[j4 * 4 + i] = in ? pack_bf16x2(y0, y1) : 0u;
            }
          }
        }
        tc_fence_before();
        if (it > 0) {  // every CTA has finished reading the previous tile's K / V
          ok = mbar_wait_cluster(&bars[KV_FREE], (it - 1) & 1, abort_flag, 332);
          if (!ok) break;
        }
        {   // K and V alike: token-major, this thread's 32 columns of its token row
          uint8_t* tile = smem + (tensor == 0 ? L::K_OFF : L::VT_OFF) + part * TILE_BYTES;
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4)
            *reinterpret_cast<uint4*>(tile + sw128_offset(row, wg * 32 + j4 * 8)) =
                make_uint4(packed[j4 * 4], packed[j4 * 4 + 1], packed[j4 * 4 + 2], packed[j4 * 4 + 3]);
        }
      }
      laps.lap(8);
      warp_arrive(&bars[META_FREE + mb], lane);
      fence_proxy_async();
      warp_arrive(&bars[EPI_LOCAL], lane);
      laps.lap(9);
      // ---- online softmax of this thread's query row
      if (wg < nq) {
        ok = mbar_wait(&bars[S_FULL + wg], it & 1, abort_flag, 340 + wg);
        laps.lap(10);
        if (!ok) break;
        tc_fence_after();
        // S of this tile was issued after PV of the previous one, so O is up to date here
        const uint32_t s_addr = tmem_base + lane_sel + wg * 128;
        float mx = -INFINITY;
        {
          uint32_t raw[2][32];
          tmem_ld32_issue(s_addr, raw[0]);
#pragma unroll
          for (int cc = 0; cc < TOK / 32; ++cc) {
            uint32_t (&cur)[32] = raw[cc & 1];
            tmem_ld32_wait(cur);
            if (cc + 1 < TOK / 32) tmem_ld32_issue(s_addr + (cc + 1) * 32, raw[(cc + 1) & 1]);
            if (valid == TOK) {   // four chains instead of one
              float ma = -INFINITY, mb_ = -INFINITY, mc = -INFINITY, md = -INFINITY;
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                ma = fmaxf(ma, __uint_as_float(cur[j]));
                mb_ = fmaxf(mb_, __uint_as_float(cur[j + 1]));
                mc = fmaxf(mc, __uint_as_float(cur[j + 2]));
                md = fmaxf(md, __uint_as_float(cur[j + 3]));
              }
              mx = fmaxf(mx, fmaxf(fmaxf(ma, mb_), fmaxf(mc, md)));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (cc * 32 + j < valid) mx = fmaxf(mx, __uint_as_float(cur[j]));
            }
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
        // P (bf16 pairs) replaces S in place: the 16 cells written per step lie below the 32 read.
        // The load of the next 32 scores stays in flight under the exponentials of the current ones.
        float sum = 0.f, sum_b = 0.f, sum_c = 0.f, sum_d = 0.f;   // four chains instead of one
        uint32_t raw[2][32];
        tmem_ld32_issue(s_addr, raw[0]);
#pragma unroll
        for (int cc = 0; cc < TOK / 32; ++cc) {
          uint32_t (&cur)[32] = raw[cc & 1];
          tmem_ld32_wait(cur);
          if (cc + 1 < TOK / 32) tmem_ld32_issue(s_addr + (cc + 1) * 32, raw[(cc + 1) & 1]);
          uint32_t packed[16];
          if (valid == TOK) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float p0 = exp2_approx(fmaf(__uint_as_float(cur[j]), p.scale_log2, -m_used));
              const float p1 = exp2_approx(fmaf(__uint_as_float(cur[j + 1]), p.scale_log2, -m_used));
              const float p2 = exp2_approx(fmaf(__uint_as_float(cur[j + 2]), p.scale_log2, -m_used));
              const float p3 = exp2_approx(fmaf(__uint_as_float(cur[j + 3]), p.scale_log2, -m_used));
              sum += p0; sum_b += p1; sum_c += p2; sum_d += p3;
              packed[j >> 1] = pack_bf16x2(p0, p1);
              packed[(j >> 1) + 1] = pack_bf16x2(p2, p3);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float p0 = (cc * 32 + j < valid) ? exp2f(fmaf(__uint_as_float(cur[j]), p.scale_log2, -m_used)) : 0.f;
              float p1 = (cc * 32 + j + 1 < valid) ? exp2f(fmaf(__uint_as_float(cur[j + 1]), p.scale_log2, -m_used)) : 0.f;
              sum += p0 + p1;
              packed[j >> 1] = pack_bf16x2(p0, p1);
            }
          }
          tmem_st16(s_addr + cc * 16, packed);
        }
        tmem_wait_st();
        l_run += (sum + sum_b) + (sum_c + sum_d);
        laps.lap(11);
        tc_fence_before();
        warp_arrive(&bars[P_READY + wg], lane);
        laps.lap(12);
      }
    }
    laps.flush();
    // ---- write O / l and the natural-log LSE
    if (ok && wg < nq && ntiles > 0) {
      ok = mbar_wait(&bars[PV_DONE + wg], (ntiles - 1) & 1, abort_flag, 350 + wg);
      if (ok) {
        tc_fence_after();
        const int qrow = q0 + wg * QT + row;
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        const uint32_t o_addr = tmem_base + lane_sel + 256 + wg * 128;
        const size_t split_rows = static_cast<size_t>(blockIdx.z) * p.Q * p.heads;
        uint16_t* dst = p.out + (split_rows + static_cast<size_t>(qrow) * p.heads + head) * D;
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
          p.lse[split_rows + static_cast<size_t>(qrow) * p.heads + head] =
              l_run > 0.f ? (m_used + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  // no CTA may leave while a peer can still store into its shared memory or signal its barriers
  cluster_sync_all();
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

template <int D, bool ROPE, bool CAM, bool PROF>
int launch(const CUtensorMap maps[5], Params& p, cudaStream_t stream) {
  using L = Layout<D>;
  int nw = MAX_NW;   // as many decoder-row slots as fit (at least the two staging slots' worth)
  while (nw > NSTAGE && L::bytes(nw, p.ngroups, p.rank) > SMEM_LIMIT) --nw;
  size_t smem = L::bytes(nw, p.ngroups, p.rank);
  NKV_REQUIRE(smem <= SMEM_LIMIT, NKV_ERR_UNSUPPORTED,
              "codec attention needs %zu bytes of shared memory (rank %d, rank/group %d)", smem,
              p.rank, p.ngroups);
  p.nw = nw;
  p.prof = g_profile;
  auto kernel = attn_codec_kernel<D, ROPE, CAM, PROF>;
  NKV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem)));
  const int qblocks = ceil_div(p.Q, NQ * QT);
  cudaLaunchConfig_t config{};
  const int splits = ceil_div(ceil_div(p.N, TOK), p.tiles_per_split);
  config.gridDim = dim3(ceil_div(qblocks, L::CL) * L::CL, p.heads, splits);   // padded: idle CTAs still decode
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = L::CL;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  config.attrs = &attr;
  config.numAttrs = 1;
  NKV_CUDA(cudaLaunchKernelEx(&config, kernel, maps[0], maps[1], maps[2], maps[3], maps[4], p));
  return NKV_OK;
}

int launch_for(int dk, bool rope, bool cam, const CUtensorMap maps[5], Params& p, cudaStream_t stream) {
  if (g_profile != nullptr && dk == 128 && !rope && !cam)   // the instrumented build exists for this case only
    return launch<128, false, false, true>(maps, p, stream);
  if (cam)   // camera builds always carry the rotation code (a NULL table switches it off at run time)
    return dk == 128 ? launch<128, true, true, false>(maps, p, stream)
                     : launch<64, true, true, false>(maps, p, stream);
  if (dk == 128)
    return rope ? launch<128, true, false, false>(maps, p, stream)
                : launch<128, false, false, false>(maps, p, stream);
  return rope ? launch<64, true, false, false>(maps, p, stream)
              : launch<64, false, false, false>(maps, p, stream);
}

}  // namespace

// out[row][8 g + i] = w[row][8 g + perm[i]], perm = 0 2 4 6 1 3 5 7: the order in which the kernel
// expands a code word (dequant8_bf16_perm).  Thread = one group of 8 columns (16 bytes).
__global__ void __launch_bounds__(256)
prepare_decoder_kernel(const uint4* w, long long groups, uint4* out) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= groups) return;
  const uint4 v = w[idx];   // (e0 e1) (e2 e3) (e4 e5) (e6 e7)
  uint4 r;
  r.x = __byte_perm(v.x, v.y, 0x5410);   // e0 e2
  r.y = __byte_perm(v.z, v.w, 0x5410);   // e4 e6
  r.z = __byte_perm(v.x, v.y, 0x7632);   // e1 e3
  r.w = __byte_perm(v.z, v.w, 0x7632);   // e5 e7
  out[idx] = r;
}

int tc_prepare_decoder(const void* w_bf16, int64_t rows, int rank, void* out_bf16, cudaStream_t stream) {
  NKV_REQUIRE(rank % 8 == 0 && ((reinterpret_cast<uintptr_t>(w_bf16) | reinterpret_cast<uintptr_t>(out_bf16)) & 15) == 0,
              NKV_ERR_INVALID, "prepare_decoder: rank %d must be a multiple of 8, arrays 16-byte aligned", rank);
  const long long groups = rows * (rank / 8);
  if (groups == 0) return NKV_OK;
  prepare_decoder_kernel<<<static_cast<unsigned>((groups + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint4*>(w_bf16), groups, static_cast<uint4*>(out_bf16));
  NKV_LAUNCH_CHECK("prepare_decoder_kernel");
  return NKV_OK;
}

// Development aid: 32 device int64 cycle buckets filled by CTA (0,0) of later launches
// (compute thread 0: buckets 0-12, MMA thread: 16-22); nullptr switches it off.
void tc_attn_set_profile(long long* device_buckets) { g_profile = device_buckets; }

bool tc_attn_supported(int dk, int dv, int rank) {
  return dk == dv && (dk == 64 || dk == 128) && rank % 64 == 0 && rank > 0;
}

int tc_attn_codec(const void* q, int64_t q_stride_token, int64_t q_stride_head, int Q, int heads,
                  int dk, int dv, const nkv_history* hist_k, const nkv_history* hist_v,
                  const void* wk, const float* bias_k, const void* wv, const float* bias_v,
                  float scale, void* out, float* lse, int32_t* status_word, int splits,
                  void* workspace, cudaStream_t stream, const nkv_rope* rope,
                  const nkv_camera* cam_k, const nkv_camera* cam_v, bool prepared_weights) {
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
    int rc = encode_tensor_map(&maps[0], 2, q, 3, dims, strides, box, 128);
    if (rc != NKV_OK) return rc;
  }
  const void* weights[2] = {wk, wv};
  for (int w = 0; w < 2; ++w) {
    uint64_t dims[2] = {static_cast<uint64_t>(rank), static_cast<uint64_t>(heads) * dk};
    uint64_t strides[1] = {static_cast<uint64_t>(rank) * 2};
    uint32_t box[2] = {64, PART};   // one CTA streams 64 rows of the slice
    int rc = encode_tensor_map(&maps[1 + w], 2, weights[w], 2, dims, strides, box, 128);
    if (rc != NKV_OK) return rc;
  }
  NKV_REQUIRE((reinterpret_cast<uintptr_t>(hk.codes) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(hv.codes) & 15) == 0 && (rank / 2) % 16 == 0,
              NKV_ERR_INVALID, "code arrays must be 16-byte aligned with 16-byte multiples per token");
  const void* code_arrays[2] = {hk.codes, hv.codes};
  for (int w = 0; w < 2; ++w) {   // [N tokens x rank/2 bytes]; a box is 64 bytes of 128 tokens
    uint64_t dims[2] = {static_cast<uint64_t>(rank / 2), static_cast<uint64_t>(N)};
    uint64_t strides[1] = {static_cast<uint64_t>(rank / 2)};
    uint32_t box[2] = {64, TOK};
    int rc = encode_tensor_map(&maps[3 + w], 1, code_arrays[w], 2, dims, strides, box, 64);
    if (rc != NKV_OK) return rc;
  }
  Params p{};
  p.Q = Q; p.heads = heads; p.N = N; p.rank = rank; p.nchunks = rank / CHUNK;
  p.group = group; p.ngroups = rank / group; p.scale_dtype = hk.scale_dtype;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.hk = hk; p.hv = hv; p.bias_k = bias_k; p.bias_v = bias_v;
  p.status = status_word;
  p.w_perm = prepared_weights ? 1 : 0;
  if (rope != nullptr) p.rope = *rope;
  if (cam_k != nullptr) p.cam_k = *cam_k;
  if (cam_v != nullptr) p.cam_v = *cam_v;
  // History splits: each grid.z slice attends a contiguous run of tiles and writes a partial
  // (O, lse); the partials are merged by log-sum-exp.  Evens out the rounds of resident clusters.
  const int tiles = ceil_div(N, TOK);
  splits = splits < 1 ? 1 : (splits > tiles ? tiles : splits);
  p.tiles_per_split = ceil_div(tiles, splits);
  splits = ceil_div(tiles, p.tiles_per_split);
  if (splits == 1) {
    p.out = static_cast<uint16_t*>(out); p.lse = lse;
    return launch_for(dk, rope != nullptr, cam_k != nullptr || cam_v != nullptr, maps, p, stream);
  }
  NKV_REQUIRE(workspace != nullptr, NKV_ERR_INVALID, "history splits need a workspace");
  const size_t rows = static_cast<size_t>(Q) * heads;
  uint16_t* part_out = static_cast<uint16_t*>(workspace);
  float* part_lse = reinterpret_cast<float*>(part_out + static_cast<size_t>(splits) * rows * dv);
  p.out = part_out; p.lse = part_lse;
  int rc = launch_for(dk, rope != nullptr, cam_k != nullptr || cam_v != nullptr, maps, p, stream);
  if (rc != NKV_OK) return rc;
  const void* outs[16];
  const float* lses[16];
  for (int z = 0; z < splits; ++z) {
    outs[z] = part_out + static_cast<size_t>(z) * rows * dv;
    lses[z] = part_lse + static_cast<size_t>(z) * rows;
  }
  return lse_merge(outs, lses, splits, static_cast<int64_t>(rows), dv, NKV_BF16, out, lse, stream);
}

}  // namespace nkv
