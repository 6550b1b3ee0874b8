// HBM-bound kernels: INT4 quantise + pack (+ append) and the LSE merge.
#include <atomic>

#include "nkv_internal.h"
#include "nkv_tc.cuh"

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

// Quantiser of bf16 coefficient rows with one scale per token (group == r) or per 32 coefficients.
// LANES threads (8, 16 or 32: the smallest count that covers the row with at most five 16-byte
// pieces each, so no lane idles on a 640-wide row) own one token; every lane keeps its pieces
// (8 coefficients each) in registers, so the row is read once and the codes leave as 4-byte
// stores.  Scale and reciprocal are formed once per token (once per piece in the 32-wide mode,
// where four neighbouring lanes share a group).  `mask` names the token's lanes in the warp.
constexpr int QP_MAXJ = 5;

template <bool IN_BF16, bool GROUP32, int LANES>
__device__ __forceinline__ void quant_pack_row(const uint4 (&v)[QP_MAXJ], int sub, unsigned mask, int r,
                                               float eps, int scale_dtype, long long t, uint8_t* codes,
                                               void* scales) {
  constexpr int MAXJ = QP_MAXJ;
  const int pieces = r >> 3;
  float amax[MAXJ];
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    // |max| of the piece on packed pairs: clear the two sign bits, one paired maximum per word
    const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
    __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t magnitude = w[k] & 0x7FFF7FFFu;
      m2 = __hmax2(m2, *reinterpret_cast<const __nv_bfloat162*>(&magnitude));
    }
    const uint32_t both = *reinterpret_cast<const uint32_t*>(&m2);
    amax[j] = fmaxf(__uint_as_float(both << 16), __uint_as_float(both & 0xFFFF0000u));
  }
  float scale_of[MAXJ], inv_of[MAXJ];
  if (GROUP32) {   // 4 consecutive pieces = 4 consecutive lanes form a group
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      amax[j] = fmaxf(amax[j], __shfl_xor_sync(mask, amax[j], 1));
      amax[j] = fmaxf(amax[j], __shfl_xor_sync(mask, amax[j], 2));
      if (IN_BF16) scale_of[j] = round_to_bf16(__fdiv_rn(fmaxf(amax[j], round_to_bf16(eps)), 7.0f));
      else scale_of[j] = __fdiv_rn(fmaxf(amax[j], eps), 7.0f);
      inv_of[j] = __frcp_rn(scale_of[j]);
    }
  } else {
    float m = amax[0];
#pragma unroll
    for (int j = 1; j < MAXJ; ++j) m = fmaxf(m, amax[j]);
#pragma unroll
    for (int off = LANES / 2; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(mask, m, off));
    float scale;
    if (IN_BF16) scale = round_to_bf16(__fdiv_rn(fmaxf(m, round_to_bf16(eps)), 7.0f));
    else scale = __fdiv_rn(fmaxf(m, eps), 7.0f);
    const float inv = __frcp_rn(scale);
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) { scale_of[j] = scale; inv_of[j] = inv; }
  }
  uint32_t* dst = reinterpret_cast<uint32_t*>(codes + static_cast<size_t>(t) * (r >> 1));
  const int groups = GROUP32 ? (r >> 5) : 1;
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    const int i = sub + LANES * j;
    if (i >= pieces) continue;
    const float scale = scale_of[j], inv = inv_of[j];
    const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
    uint32_t out = 0;
    if (IN_BF16) {
      // The quotient is rounded to bf16 before rint.  z * inv is within 2 ulp of the IEEE quotient,
      // so both round to the same bf16 number unless the product's low 16 bits lie within 4 of the
      // rounding boundary 0x8000; only such values take the division (an exact boundary case cannot
      // occur: a ratio of two 8-bit mantissas is never a 9-bit midpoint).  rint of the bf16 quotient
      // is again the addition of 1.5 * 2^23 (exact on a bf16 number, ties to even as rint has them).
      constexpr float MAGIC = 12582912.0f;
      constexpr uint32_t MAGIC_BITS = 0x4B400000u;
      constexpr uint32_t PACK_BIAS = (MAGIC_BITS - 7u) * 0x11111111u;
      bool ambiguous = false;
      uint32_t acc = 0;
#pragma unroll
      for (int k = 3; k >= 0; --k) {
        const float q1 = __uint_as_float(w[k] & 0xFFFF0000u) * inv;
        const float q0 = __uint_as_float(w[k] << 16) * inv;
        ambiguous |= ((__float_as_uint(q1) + 0x8004u) & 0xFFFFu) <= 8u;
        ambiguous |= ((__float_as_uint(q0) + 0x8004u) & 0xFFFFu) <= 8u;
        const __nv_bfloat162 rounded = __floats2bfloat162_rn(q0, q1);
        const uint32_t both = *reinterpret_cast<const uint32_t*>(&rounded);
        const float t1 = __uint_as_float(both & 0xFFFF0000u) + MAGIC;
        const float t0 = __uint_as_float(both << 16) + MAGIC;
        acc = (acc << 4) + __float_as_uint(t1);
        acc = (acc << 4) + __float_as_uint(t0);
      }
      out = acc - PACK_BIAS;
      if (ambiguous) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t word = w[e >> 1];
          const float z = __uint_as_float((e & 1) ? (word & 0xFFFF0000u) : (word << 16));
          if (((__float_as_uint(z * inv) + 0x8004u) & 0xFFFFu) <= 8u) {
            const uint32_t code = static_cast<uint32_t>(quant_code<true>(z, scale, inv));
            out = (out & ~(0xFu << (4 * e))) | (code << (4 * e));
          }
        }
      }
    } else {
      // whole piece through the reciprocal; a piece holding a value whose scaled form lies within
      // 1e-5 of a half-integer (where the reciprocal and the IEEE quotient could round apart) is
      // redone value by value with the exact rule.  Rounding to the nearest-even integer is the
      // fp32 addition of 1.5 * 2^23 (the integer then sits in the low mantissa bits), which keeps
      // the whole loop on the full-rate floating-point and integer pipes: no conversion
      // instruction per value.  No clamp is needed here: |z| <= the group's maximum and
      // scale = max(that, eps) / 7 bound |z * inv| by 7 (1 + 2^-22) for every finite row, and a row
      // with a non-finite value has no defined codes in the reference either (the 32-bit word of
      // such a piece may then hold arbitrary bits; nothing outside that word is touched).
      constexpr float MAGIC = 12582912.0f;
      constexpr uint32_t MAGIC_BITS = 0x4B400000u;
      // the float bits of (q + MAGIC) are MAGIC_BITS + rint(q): eight of them, each shifted four
      // bits further, add up (mod 2^32) to the packed word plus a constant
      constexpr uint32_t PACK_BIAS = (MAGIC_BITS - 7u) * 0x11111111u;
      float worst = 0.f;
      uint32_t acc = 0;
#pragma unroll
      for (int k = 3; k >= 0; --k) {
        const float q1 = __uint_as_float(w[k] & 0xFFFF0000u) * inv;
        const float q0 = __uint_as_float(w[k] << 16) * inv;
        const float t1 = q1 + MAGIC, t0 = q0 + MAGIC;
        worst = fmaxf(worst, fabsf(q1 - (t1 - MAGIC)));
        worst = fmaxf(worst, fabsf(q0 - (t0 - MAGIC)));
        acc = (acc << 4) + __float_as_uint(t1);
        acc = (acc << 4) + __float_as_uint(t0);
      }
      out = acc - PACK_BIAS;
      const bool near_half = worst > 0.49999f;
      if (near_half) {
        // exact ties are not rare (a row whose maximum has a mantissa divisible by 7 holds many),
        // so only the values that are near a half take the IEEE division; their nibble is replaced
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t word = w[e >> 1];
          const float z = __uint_as_float((e & 1) ? (word & 0xFFFF0000u) : (word << 16));
          const float q = z * inv;
          if (fabsf(q - ((q + MAGIC) - MAGIC)) > 0.49999f) {
            const uint32_t code = static_cast<uint32_t>(quant_code<false>(z, scale, inv));
            out = (out & ~(0xFu << (4 * e))) | (code << (4 * e));
          }
        }
      }
    }
    dst[i] = out;
    if (GROUP32) {
      if ((i & 3) == 0) store_float(scales, scale_dtype, static_cast<size_t>(t) * groups + (i >> 2), scale);
    } else if (i == 0) {
      store_float(scales, scale_dtype, static_cast<size_t>(t), scale);
    }
  }
}

// Small inputs: rows straight from global memory into registers, one pass.
template <bool IN_BF16, bool GROUP32, int LANES>
__global__ void __launch_bounds__(256)
quant_pack_vec_kernel(const uint16_t* coeff, int S, int r, float eps, int scale_dtype,
                      uint8_t* codes, void* scales) {
  const int sub = threadIdx.x % LANES;
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / LANES;
  if (t >= S) return;     // the LANES threads of a token leave together
  const unsigned lane = threadIdx.x & 31;
  const unsigned mask = LANES == 32 ? 0xffffffffu : (((1u << LANES) - 1u) << (lane - sub));
  const int pieces = r >> 3;
  const uint4* src = reinterpret_cast<const uint4*>(coeff + static_cast<size_t>(t) * r);
  uint4 v[QP_MAXJ];
#pragma unroll
  for (int j = 0; j < QP_MAXJ; ++j) {
    const int i = sub + LANES * j;
    v[j] = i < pieces ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
  }
  quant_pack_row<IN_BF16, GROUP32, LANES>(v, sub, mask, r, eps, scale_dtype, t, codes, scales);
}

// Streaming form for large inputs (the HBM-bound case).  Every warp runs its own two-stage ring in
// shared memory: the 32 / LANES consecutive tokens a warp quantises at a time are one contiguous run
// of at most 2,560 bytes, fetched by a bulk asynchronous copy that lane 0 issues and that the
// warp's own mbarrier tracks, so the warp's next rows are in flight for the whole time it works on
// the current ones and no warp ever waits for another (there is no block-wide barrier in the
// loop).  512 threads x 2 blocks per SM keep about 80 KiB of reads outstanding per SM whatever the
// register-limited occupancy.
constexpr int QP_THREADS = 512;
constexpr int QP_STAGES = 2;
constexpr int QP_WARP_BYTES = 2560;       // 32 lanes x 5 pieces x 16 bytes

template <bool IN_BF16, bool GROUP32, int LANES>
__global__ void __launch_bounds__(QP_THREADS, 2)
quant_pack_stream_kernel(const uint16_t* coeff, int S, int r, float eps, int scale_dtype,
                         uint8_t* codes, void* scales, int tiles) {
  extern __shared__ __align__(128) uint8_t qp_smem[];
  constexpr int TILE = 32 / LANES;                         // tokens per warp tile
  constexpr int WARPS = QP_THREADS / 32;
  const int row_bytes = r * 2;
  uint64_t* bars = reinterpret_cast<uint64_t*>(qp_smem + WARPS * QP_STAGES * QP_WARP_BYTES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + WARPS * QP_STAGES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub = lane % LANES, slot = lane / LANES;
  const unsigned mask = LANES == 32 ? 0xffffffffu : (((1u << LANES) - 1u) << (lane - sub));
  const int pieces = r >> 3;
  uint8_t* ring = qp_smem + warp * QP_STAGES * QP_WARP_BYTES;
  uint64_t* my_bars = bars + warp * QP_STAGES;
  const int stride = gridDim.x * WARPS;
  auto issue = [&](int tile, int stage) {
    const long long first = static_cast<long long>(tile) * TILE;
    const int count = static_cast<int>(min(static_cast<long long>(TILE), S - first));
    const uint32_t bytes = static_cast<uint32_t>(count) * row_bytes;
    tc::mbar_arrive_expect_tx(&my_bars[stage], bytes);
    tc::bulk_load_1d(ring + stage * QP_WARP_BYTES, coeff + first * r, bytes, &my_bars[stage]);
  };
  if (tid == 0) *abort_flag = 0;
  if (lane == 0) {
    for (int s = 0; s < QP_STAGES; ++s) tc::mbar_init(&my_bars[s], 1);
    tc::fence_barrier_init();
    tc::fence_proxy_async();
  }
  __syncthreads();
  const int first_tile = blockIdx.x * WARPS + warp;
  if (lane == 0) {
    for (int s = 0; s < QP_STAGES; ++s) {
      const int tile = first_tile + s * stride;
      if (tile < tiles) issue(tile, s);
    }
  }
  __syncwarp();
  int round = 0;
  for (int tile = first_tile; tile < tiles; tile += stride, ++round) {
    const int stage = round % QP_STAGES;
    if (!tc::mbar_wait(&my_bars[stage], (round / QP_STAGES) & 1, abort_flag, 700 + stage)) break;
    const long long t = static_cast<long long>(tile) * TILE + slot;
    uint4 v[QP_MAXJ];
    if (t < S) {
      const uint4* src = reinterpret_cast<const uint4*>(ring + stage * QP_WARP_BYTES + slot * row_bytes);
#pragma unroll
      for (int j = 0; j < QP_MAXJ; ++j) {
        const int i = sub + LANES * j;
        v[j] = i < pieces ? src[i] : make_uint4(0, 0, 0, 0);
      }
    }
    __syncwarp();                          // every lane has its pieces in registers: the stage is free
    const int next = tile + QP_STAGES * stride;
    if (lane == 0 && next < tiles) issue(next, stage);
    if (t < S) quant_pack_row<IN_BF16, GROUP32, LANES>(v, sub, mask, r, eps, scale_dtype, t, codes, scales);
  }
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

// ---- context-parallel merge over peer memory ---------------------------------------------
// Rank r of `world` owns rows [row_begin, row_end) of the merged result: it reads that row range of
// every rank's partial (its own from local memory, the others through peer mappings over NVLink),
// folds them exactly as lse_merge_kernel does, and stores the merged rows into every rank's result
// buffer, so the merge and the all-gather of its result are one kernel.
struct PeerMergeArgs {
  const void* part_out[MAX_PARTS];
  const float* part_lse[MAX_PARTS];
  void* dst_out[MAX_PARTS];
  float* dst_lse[MAX_PARTS];
};

// Ordering of the ranks without a collective: every rank owns a block of flag words that its peers
// can write (NKV_PEER_FLAG_WORDS int32: [0, 16) "rank r's partial of epoch e is complete",
// [16, 32) "rank r has stored its merged slice of epoch e here", [32] a ticket counter of this
// rank's own blocks).  epoch == 0 switches the protocol off (local merges).
struct PeerSync {
  int32_t* flags[MAX_PARTS];   // flag block of every rank, as mapped on this rank
  int rank, epoch;
  long long budget;            // SM cycles a wait may take before the kernel gives up
  int32_t* status;             // receives the wait-site code (980 / 981) when it does
};

__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// bounded: true when the word reached `target`, false (status set) when the budget ran out
__device__ __forceinline__ bool wait_flag_sys(const int32_t* flag, int target, long long budget,
                                              int32_t* status, int code) {
  if (ld_acquire_sys(flag) >= target) return true;
  const long long start = clock64();
  while (ld_acquire_sys(flag) < target) {
    if (clock64() - start > budget) {
      if (status) atomicCAS(status, 0, code);
      return false;
    }
    __nanosleep(100);
  }
  return true;
}

template <typename VEC>  // uint4: 8 two-byte elements; float4 pairs are handled as two uint4 halves
__device__ __forceinline__ VEC peer_load(const void* base, size_t byte_offset) {
  return *reinterpret_cast<const VEC*>(static_cast<const char*>(base) + byte_offset);
}

template <int DTYPE, int MAXP>
__device__ __forceinline__ void cp_merge_rows(const PeerMergeArgs& args, int world, int dests,
                                              long long row_begin, int d, long long idx);

// thread = (row, 8 consecutive columns); MAXP bounds the unrolled part loops (registers)
template <int DTYPE, int MAXP>
__global__ void __launch_bounds__(256)
cp_merge_peer_kernel(PeerMergeArgs args, PeerSync sync, int world, int dests, long long row_begin,
                     long long row_end, int d) {
  __shared__ int gate;
  if (sync.epoch > 0) {
    // this rank's partial is complete (it was written by earlier kernels of this stream): tell every
    // rank, then wait until every rank has said the same here
    if (blockIdx.x == 0 && threadIdx.x < world) st_release_sys(sync.flags[threadIdx.x] + sync.rank, sync.epoch);
    if (threadIdx.x == 0) gate = 1;
    __syncthreads();
    if (threadIdx.x < world &&
        !wait_flag_sys(sync.flags[sync.rank] + threadIdx.x, sync.epoch, sync.budget, sync.status, 980))
      gate = 0;
    __syncthreads();
    if (!gate) return;   // a peer never arrived: nothing is merged, the status word says so
  }
  const int per_row = d >> 3;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx < (row_end - row_begin) * per_row)
    cp_merge_rows<DTYPE, MAXP>(args, world, dests, row_begin, d, idx);
  if (sync.epoch > 0) {
    // every block's stores are out; the last block to get here tells every rank that this rank's
    // slice has landed and waits until all slices have landed here (which also means that every
    // rank is done reading this rank's partial)
    __threadfence_system();
    __syncthreads();
    int32_t* mine = sync.flags[sync.rank];
    if (threadIdx.x == 0) {
      const int ticket = atomicAdd(mine + 32, 1);
      __threadfence();
      gate = ticket == static_cast<int>(gridDim.x) - 1;
    }
    __syncthreads();
    if (!gate) return;
    if (threadIdx.x < world) {
      st_release_sys(sync.flags[threadIdx.x] + 16 + sync.rank, sync.epoch);
      wait_flag_sys(mine + 16 + threadIdx.x, sync.epoch, sync.budget, sync.status, 981);
    }
    if (threadIdx.x == 0) mine[32] = 0;
  }
}

template <int DTYPE, int MAXP>
__device__ __forceinline__ void cp_merge_rows(const PeerMergeArgs& args, int world, int dests,
                                              long long row_begin, int d, long long idx) {
  const int per_row = d >> 3;
  const long long row = row_begin + idx / per_row;
  const int col = static_cast<int>(idx % per_row) * 8;
  const size_t elem = static_cast<size_t>(row) * d + col;

  // every load is issued before the transcendental arithmetic of the fold
  constexpr int VECS = DTYPE == NKV_F32 ? 2 : 1;
  uint4 raw[MAXP][VECS];
  float part_lse[MAXP];
#pragma unroll
  for (int p = 0; p < MAXP; ++p)
    if (p < world) {
      part_lse[p] = args.part_lse[p][row];
#pragma unroll
      for (int v = 0; v < VECS; ++v)
        raw[p][v] = peer_load<uint4>(args.part_out[p], elem * (DTYPE == NKV_F32 ? 4 : 2) + 16 * v);
    }
  float lse = part_lse[0];
#pragma unroll
  for (int p = 1; p < MAXP; ++p)
    if (p < world) lse = logaddexp(lse, part_lse[p]);
  const float origin = isfinite(lse) ? lse : 0.f;

  float acc[8];
#pragma unroll
  for (int p = 0; p < MAXP; ++p)
    if (p < world) {
      const float w = expf(part_lse[p] - origin);
      float v[8];
      if (DTYPE == NKV_F32) {
        const uint32_t words[8] = {raw[p][0].x, raw[p][0].y, raw[p][0].z, raw[p][0].w,
                                   raw[p][VECS - 1].x, raw[p][VECS - 1].y, raw[p][VECS - 1].z, raw[p][VECS - 1].w};
#pragma unroll
        for (int c = 0; c < 8; ++c) v[c] = __uint_as_float(words[c]);
      } else {
        const uint32_t words[4] = {raw[p][0].x, raw[p][0].y, raw[p][0].z, raw[p][0].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (DTYPE == NKV_BF16) {
            v[2 * k] = __uint_as_float(words[k] << 16);
            v[2 * k + 1] = __uint_as_float(words[k] & 0xFFFF0000u);
          } else {
            v[2 * k] = __half2float(__ushort_as_half(static_cast<uint16_t>(words[k] & 0xFFFFu)));
            v[2 * k + 1] = __half2float(__ushort_as_half(static_cast<uint16_t>(words[k] >> 16)));
          }
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float t = __fmul_rn(v[c], w);
        acc[c] = p == 0 ? t : __fadd_rn(acc[c], t);
      }
    }
  if (DTYPE == NKV_F32) {
    const float4 out_lo = make_float4(acc[0], acc[1], acc[2], acc[3]);
    const float4 out_hi = make_float4(acc[4], acc[5], acc[6], acc[7]);
    for (int r = 0; r < dests; ++r) {
      float4* dst = reinterpret_cast<float4*>(static_cast<char*>(args.dst_out[r]) + elem * 4);
      dst[0] = out_lo;
      dst[1] = out_hi;
    }
  } else {
    uint32_t packed[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t lo16, hi16;
      if (DTYPE == NKV_BF16) {
        lo16 = float_to_bf16_bits(acc[2 * k]);
        hi16 = float_to_bf16_bits(acc[2 * k + 1]);
      } else {
        lo16 = __half_as_ushort(__float2half_rn(acc[2 * k]));
        hi16 = __half_as_ushort(__float2half_rn(acc[2 * k + 1]));
      }
      packed[k] = lo16 | (hi16 << 16);
    }
    const uint4 out = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    for (int r = 0; r < dests; ++r)
      *reinterpret_cast<uint4*>(static_cast<char*>(args.dst_out[r]) + elem * 2) = out;
  }
  if (col == 0)
    for (int r = 0; r < dests; ++r) args.dst_lse[r][row] = lse;
}

template <int DTYPE>
void launch_merge(const PeerMergeArgs& args, const PeerSync& sync, int parts, int dests, long long row_begin,
                  long long row_end, int d, cudaStream_t stream) {
  const long long total = (row_end - row_begin) * (d >> 3);
  // with the flag protocol even a rank without rows takes part (one block)
  const unsigned blocks = static_cast<unsigned>(total > 0 ? (total + 255) / 256 : 1);
  if (parts <= 4)
    cp_merge_peer_kernel<DTYPE, 4><<<blocks, 256, 0, stream>>>(args, sync, parts, dests, row_begin, row_end, d);
  else if (parts <= 8)
    cp_merge_peer_kernel<DTYPE, 8><<<blocks, 256, 0, stream>>>(args, sync, parts, dests, row_begin, row_end, d);
  else
    cp_merge_peer_kernel<DTYPE, MAX_PARTS><<<blocks, 256, 0, stream>>>(args, sync, parts, dests, row_begin, row_end, d);
}

// ---- finish of the mixed-dimensional read ------------------------------------------------------
// For query row n and group head g (real head = heads[g]):
//     l      = logaddexp(native_lse, low_lse),  origin = l where finite else 0
//     low    = (lifted + mean[head]) - projected[g]          (only with the value-mean residual)
//     out[n, head, :] = native * exp(native_lse - origin) + low * exp(low_lse - origin)
// in fp32 in exactly this order with one rounding to the output type, scattered to the head's
// place.  thread = (row, group head, 8 columns); every operand is read once, the result written once.
template <int DTYPE>
__device__ __forceinline__ void load8(const void* base, size_t elem, float (&v)[8]) {
  if (DTYPE == NKV_F32) {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const char*>(base) + elem * 4);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const char*>(base) + elem * 4 + 16);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const char*>(base) + elem * 2);
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[2 * k] = __uint_as_float(words[k] << 16);
      v[2 * k + 1] = __uint_as_float(words[k] & 0xFFFF0000u);
    }
  }
}

template <int DTYPE, bool CORRECT>
__global__ void __launch_bounds__(256)
fast_finish_kernel(const void* native, const float* native_lse, const void* lifted, const float* low_lse,
                   const int32_t* heads, const float* mean, const float* projected, long long rows,
                   int total_heads, int group_heads, int d, void* out, float* out_lse) {
  const int per_row = d >> 3;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * group_heads * per_row) return;
  const int col = static_cast<int>(idx % per_row) * 8;
  const long long pair = idx / per_row;              // row * group_heads + g
  const int g = static_cast<int>(pair % group_heads);
  const long long row = pair / group_heads;
  const int head = heads[g];
  const size_t wide = (static_cast<size_t>(row) * total_heads + head);
  float a[8], b[8];
  load8<DTYPE>(native, wide * d + col, a);
  load8<DTYPE>(lifted, static_cast<size_t>(pair) * d + col, b);
  const float x = native_lse[wide], z = low_lse[pair];
  const float l = logaddexp(x, z);
  const float origin = isfinite(l) ? l : 0.f;
  const float wa = expf(x - origin), wb = expf(z - origin);
  if (CORRECT) {
    float m[8], q[8];
    load8<NKV_F32>(mean, static_cast<size_t>(head) * d + col, m);
    load8<NKV_F32>(projected, static_cast<size_t>(g) * d + col, q);
#pragma unroll
    for (int c = 0; c < 8; ++c) b[c] = __fsub_rn(__fadd_rn(b[c], m[c]), q[c]);
  }
  float y[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) y[c] = __fadd_rn(__fmul_rn(a[c], wa), __fmul_rn(b[c], wb));
  if (DTYPE == NKV_F32) {
    float4* dst = reinterpret_cast<float4*>(static_cast<char*>(out) + (wide * d + col) * 4);
    dst[0] = make_float4(y[0], y[1], y[2], y[3]);
    dst[1] = make_float4(y[4], y[5], y[6], y[7]);
  } else {
    uint32_t packed[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      packed[k] = static_cast<uint32_t>(float_to_bf16_bits(y[2 * k])) |
                  (static_cast<uint32_t>(float_to_bf16_bits(y[2 * k + 1])) << 16);
    *reinterpret_cast<uint4*>(static_cast<char*>(out) + (wide * d + col) * 2) =
        make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
  if (out_lse != nullptr && col == 0) out_lse[wide] = l;
}

// ---- INT8 operator storage -> resident bf16 --------------------------------------------------
// out[r][c] = bf16(q[r][c]) * scale[r][c / group] as one bf16 product (|q| <= 127 is exact in
// bf16, so the fp32 product of the two is exact and is rounded once).  Thread = 16 columns.
__global__ void __launch_bounds__(256)
unpack_int8_kernel(const int8_t* q, const uint16_t* scale, long long rows, int cols, int group,
                   uint16_t* out) {
  const int per_row = cols >> 4;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * per_row) return;
  const long long r = idx / per_row;
  const int c0 = static_cast<int>(idx % per_row) * 16;
  const uint4 raw = *reinterpret_cast<const uint4*>(q + r * cols + c0);
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
  const int groups = cols / group;
  uint32_t packed[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int c = c0 + 2 * k;
    const float s0 = bf16_bits_to_float(scale[r * groups + c / group]);
    const float s1 = bf16_bits_to_float(scale[r * groups + (c + 1) / group]);
    const int shift = (2 * k & 3) * 8;
    const float v0 = static_cast<float>(static_cast<int8_t>((words[k >> 1] >> shift) & 0xFFu));
    const float v1 = static_cast<float>(static_cast<int8_t>((words[k >> 1] >> (shift + 8)) & 0xFFu));
    packed[k] = static_cast<uint32_t>(float_to_bf16_bits(v0 * s0)) |
                (static_cast<uint32_t>(float_to_bf16_bits(v1 * s1)) << 16);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + r * cols + c0);
  dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}

// ---- first moments of a compressed history ---------------------------------------------------
// latent_sum[j] = sum_t bf16((code[t][j] - 7) * scale[t][j / group]) and, per centre row, how many
// tokens were assigned to it.  Stage 1: a block sums a slab of MOMENT_SLAB tokens, thread = one
// code byte (two latent columns), and writes its partial row; counts are integer atomics (exact
// in any order).  Stage 2 adds the partial rows in slab order, so the result is deterministic.
constexpr int MOMENT_SLAB = 128;

__global__ void __launch_bounds__(256)
moments_partial_kernel(nkv_history h, float* partial, int* counts) {
  const int slab = blockIdx.x;
  const int t0 = slab * MOMENT_SLAB, t1 = min(h.tokens, t0 + MOMENT_SLAB);
  const int row_bytes = h.rank >> 1, groups = h.rank / h.group;
  for (int b = threadIdx.x; b < row_bytes; b += blockDim.x) {
    float lo = 0.f, hi = 0.f;
    const int g_lo = (2 * b) / h.group, g_hi = (2 * b + 1) / h.group;
#pragma unroll 8
    for (int t = t0; t < t1; ++t) {
      const uint8_t byte = h.codes[static_cast<size_t>(t) * row_bytes + b];
      const float s_lo = load_float(h.scales, h.scale_dtype, static_cast<size_t>(t) * groups + g_lo);
      const float s_hi = g_hi == g_lo ? s_lo
                                      : load_float(h.scales, h.scale_dtype, static_cast<size_t>(t) * groups + g_hi);
      lo += round_to_bf16(static_cast<float>(static_cast<int>(byte & 15u) - 7) * s_lo);
      hi += round_to_bf16(static_cast<float>(static_cast<int>(byte >> 4) - 7) * s_hi);
    }
    partial[static_cast<size_t>(slab) * h.rank + 2 * b] = lo;
    partial[static_cast<size_t>(slab) * h.rank + 2 * b + 1] = hi;
  }
  for (int t = t0 + threadIdx.x; t < t1; t += blockDim.x) atomicAdd(&counts[center_row_of(h, t)], 1);
}

// Vector form for rank % 8 == 0, group % 8 == 0, rank <= 2048: thread = (token sub-lane, one
// 4-byte word of a code row = 8 latent columns sharing one scale); a warp reads 128 contiguous
// bytes of a row.  The sub-lanes' sums are added in sub-lane order, so the result is deterministic.
__global__ void __launch_bounds__(256)
moments_partial_vec_kernel(nkv_history h, float* partial, int* counts) {
  __shared__ float lanes[2048];
  const int slab = blockIdx.x;
  const int t0 = slab * MOMENT_SLAB, t1 = min(h.tokens, t0 + MOMENT_SLAB);
  const int words = h.rank >> 3, groups = h.rank / h.group;
  const int sublanes = blockDim.x / words;
  const int word = threadIdx.x % words, sub = threadIdx.x / words;
  if (sub < sublanes) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const int g = (word * 8) / h.group;
#pragma unroll 4
    for (int t = t0 + sub; t < t1; t += sublanes) {
      const uint32_t packed = reinterpret_cast<const uint32_t*>(h.codes)[static_cast<size_t>(t) * words + word];
      const float scale = load_float(h.scales, h.scale_dtype, static_cast<size_t>(t) * groups + g);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        acc[c] += round_to_bf16(static_cast<float>(static_cast<int>((packed >> (4 * c)) & 15u) - 7) * scale);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) lanes[(sub * words + word) * 8 + c] = acc[c];
  }
  __syncthreads();
  for (int j = threadIdx.x; j < h.rank; j += blockDim.x) {
    float sum = 0.f;
    for (int s = 0; s < sublanes; ++s) sum += lanes[s * h.rank + j];
    partial[static_cast<size_t>(slab) * h.rank + j] = sum;
  }
  for (int t = t0 + threadIdx.x; t < t1; t += blockDim.x) atomicAdd(&counts[center_row_of(h, t)], 1);
}

// block = 8 latent columns; 32 thread groups stride over the slabs, then a fixed-order tree
__global__ void __launch_bounds__(256)
moments_reduce_kernel(const float* partial, int slabs, int rank, float* latent_sum) {
  __shared__ float tree[32][8];
  const int c = threadIdx.x & 7, lane = threadIdx.x >> 3;
  const int j = blockIdx.x * 8 + c;
  float sum = 0.f;
  if (j < rank)
    for (int s = lane; s < slabs; s += 32) sum += partial[static_cast<size_t>(s) * rank + j];
  tree[lane][c] = sum;
  __syncthreads();
  for (int width = 16; width >= 1; width >>= 1) {
    if (lane < width) tree[lane][c] += tree[lane + width][c];
    __syncthreads();
  }
  if (lane == 0 && j < rank) latent_sum[j] = tree[0][c];
}

}  // namespace

int quant_pack(const void* coeff, int coeff_dtype, int S, int r, int group, float eps,
               int quant_mode, int scale_dtype, uint8_t* codes, void* scales,
               cudaStream_t stream) {
  if (S == 0) return NKV_OK;
  const bool aligned = (reinterpret_cast<uintptr_t>(coeff) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(codes) & 3) == 0;
  if (coeff_dtype == NKV_BF16 && r % 8 == 0 && r <= 1280 && aligned && (group == r || group == 32)) {
    const uint16_t* src = static_cast<const uint16_t*>(coeff);
    const int pieces = r / 8;
    const int lanes = pieces <= 40 ? 8 : (pieces <= 80 ? 16 : 32);
    const unsigned blocks = static_cast<unsigned>((static_cast<long long>(S) * lanes + 255) / 256);
    const bool in_bf16 = quant_mode == NKV_QUANT_IN_BF16;
    // large inputs stream through shared memory; small ones (a chunk or two) go straight to registers
    const int tile_tokens = 32 / lanes;                      // per warp
    const int tiles = (S + tile_tokens - 1) / tile_tokens;
    const bool stream_form = S >= 8192 && (r * 2) % 16 == 0;
    static std::atomic<int> sm_count[64];
    int grid = 0;
    size_t smem = 0;
    if (stream_form) {
      int device = 0, sms = 0;
      if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) device = -1;
      if (device >= 0) sms = sm_count[device].load(std::memory_order_relaxed);
      if (sms == 0) {
        if (device < 0 ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
          sms = 148;
        if (device >= 0) sm_count[device].store(sms, std::memory_order_relaxed);
      }
      const int blocks_needed = (tiles + QP_THREADS / 32 - 1) / (QP_THREADS / 32);
      grid = blocks_needed < 2 * sms ? blocks_needed : 2 * sms;
      smem = static_cast<size_t>(QP_THREADS / 32) * QP_STAGES * (QP_WARP_BYTES + 8) + 64;
    }
#define NKV_QP(INB, G32, L)                                                                          \
    do {                                                                                               \
      if (stream_form) {                                                                               \
        auto kernel = quant_pack_stream_kernel<INB, G32, L>;                                           \
        NKV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                                      static_cast<int>(smem)));                                        \
        kernel<<<grid, QP_THREADS, smem, stream>>>(src, S, r, eps, scale_dtype, codes, scales, tiles); \
      } else {                                                                                         \
        quant_pack_vec_kernel<INB, G32, L><<<blocks, 256, 0, stream>>>(src, S, r, eps, scale_dtype,     \
                                                                       codes, scales);                \
      }                                                                                                \
    } while (0)
#define NKV_QP_LANES(INB, G32) \
    do { if (lanes == 8) NKV_QP(INB, G32, 8); else if (lanes == 16) NKV_QP(INB, G32, 16); else NKV_QP(INB, G32, 32); } while (0)
    if (group == 32) { if (in_bf16) NKV_QP_LANES(true, true); else NKV_QP_LANES(false, true); }
    else             { if (in_bf16) NKV_QP_LANES(true, false); else NKV_QP_LANES(false, false); }
#undef NKV_QP_LANES
#undef NKV_QP
    NKV_LAUNCH_CHECK("quant_pack_vec_kernel");
    return NKV_OK;
  }
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
  bool vector = d % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                (dtype == NKV_F32 || dtype == NKV_BF16);
  for (int p = 0; p < parts; ++p) vector = vector && (reinterpret_cast<uintptr_t>(outs[p]) & 15) == 0;
  if (vector) {   // 16-byte loads and stores: the peer-merge kernel with one local destination
    PeerMergeArgs wide{};
    for (int p = 0; p < parts; ++p) { wide.part_out[p] = outs[p]; wide.part_lse[p] = lses[p]; }
    wide.dst_out[0] = out;
    wide.dst_lse[0] = lse_out;
    const PeerSync none{};
    if (dtype == NKV_F32) launch_merge<NKV_F32>(wide, none, parts, 1, 0, rows, d, stream);
    else launch_merge<NKV_BF16>(wide, none, parts, 1, 0, rows, d, stream);
    NKV_LAUNCH_CHECK("cp_merge_peer_kernel");
    return NKV_OK;
  }
  MergeArgs args{};
  for (int p = 0; p < parts; ++p) { args.outs[p] = outs[p]; args.lses[p] = lses[p]; }
  long long total = rows * (d >> 2);
  lse_merge_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      args, parts, rows, d, dtype, out, lse_out);
  NKV_LAUNCH_CHECK("lse_merge_kernel");
  return NKV_OK;
}

int cp_merge_peer(const void* const* part_out, const float* const* part_lse, void* const* dst_out,
                  float* const* dst_lse, int world, int64_t rows, int d, int64_t row_begin,
                  int64_t row_end, int dtype, cudaStream_t stream, int32_t* const* flags, int rank,
                  int epoch, long long budget_cycles, int32_t* status) {
  NKV_REQUIRE(world >= 1 && world <= MAX_PARTS, NKV_ERR_TOO_LARGE,
              "peer merge takes 1..%d ranks, got %d", MAX_PARTS, world);
  NKV_REQUIRE(d % 8 == 0, NKV_ERR_INVALID, "peer merge width %d must be a multiple of 8", d);
  NKV_REQUIRE(0 <= row_begin && row_begin <= row_end && row_end <= rows, NKV_ERR_INVALID,
              "peer merge rows [%lld, %lld) outside [0, %lld)", static_cast<long long>(row_begin),
              static_cast<long long>(row_end), static_cast<long long>(rows));
  PeerMergeArgs args{};
  PeerSync sync{};
  for (int p = 0; p < world; ++p) {
    NKV_REQUIRE(part_out[p] && part_lse[p] && dst_out[p] && dst_lse[p], NKV_ERR_INVALID,
                "peer merge: null buffer of rank %d", p);
    NKV_REQUIRE(((reinterpret_cast<uintptr_t>(part_out[p]) | reinterpret_cast<uintptr_t>(dst_out[p])) & 15) == 0,
                NKV_ERR_INVALID, "peer merge: buffers of rank %d are not 16-byte aligned", p);
    args.part_out[p] = part_out[p];
    args.part_lse[p] = part_lse[p];
    args.dst_out[p] = dst_out[p];
    args.dst_lse[p] = dst_lse[p];
  }
  if (flags != nullptr) {
    NKV_REQUIRE(rank >= 0 && rank < world && epoch > 0 && budget_cycles > 0, NKV_ERR_INVALID,
                "peer exchange: rank=%d of %d, epoch=%d, budget=%lld", rank, world, epoch, budget_cycles);
    for (int p = 0; p < world; ++p) {
      NKV_REQUIRE(flags[p] != nullptr && (reinterpret_cast<uintptr_t>(flags[p]) & 3) == 0, NKV_ERR_INVALID,
                  "peer exchange: flag block of rank %d", p);
      sync.flags[p] = flags[p];
    }
    sync.rank = rank; sync.epoch = epoch; sync.budget = budget_cycles; sync.status = status;
  } else if (row_end == row_begin) {
    return NKV_OK;
  }
  if (dtype == NKV_F32) launch_merge<NKV_F32>(args, sync, world, world, row_begin, row_end, d, stream);
  else if (dtype == NKV_BF16) launch_merge<NKV_BF16>(args, sync, world, world, row_begin, row_end, d, stream);
  else launch_merge<NKV_F16>(args, sync, world, world, row_begin, row_end, d, stream);
  NKV_LAUNCH_CHECK("cp_merge_peer_kernel");
  return NKV_OK;
}

int unpack_int8(const int8_t* q, const void* scale_bf16, int64_t rows, int cols, int group,
                void* out_bf16, cudaStream_t stream) {
  NKV_REQUIRE(cols > 0 && cols % 16 == 0, NKV_ERR_INVALID,
              "unpack_int8: %d columns (need a multiple of 16)", cols);
  NKV_REQUIRE(group > 0 && cols % group == 0, NKV_ERR_INVALID,
              "unpack_int8: group %d must divide %d columns", group, cols);
  NKV_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out_bf16)) & 15) == 0,
              NKV_ERR_INVALID, "unpack_int8: arrays must be 16-byte aligned");
  if (rows == 0) return NKV_OK;
  const long long total = rows * (cols >> 4);
  unpack_int8_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      q, static_cast<const uint16_t*>(scale_bf16), rows, cols, group, static_cast<uint16_t*>(out_bf16));
  NKV_LAUNCH_CHECK("unpack_int8_kernel");
  return NKV_OK;
}

int fast_finish(const void* native, const float* native_lse, const void* lifted, const float* low_lse,
                const int32_t* heads, const float* mean, const float* projected, int64_t rows,
                int total_heads, int group_heads, int d, int dtype, void* out, float* out_lse,
                cudaStream_t stream) {
  NKV_REQUIRE(dtype == NKV_BF16 || dtype == NKV_F32, NKV_ERR_UNSUPPORTED, "fast_finish: dtype %d", dtype);
  NKV_REQUIRE(d > 0 && d % 8 == 0, NKV_ERR_UNSUPPORTED, "fast_finish: width %d (need a multiple of 8)", d);
  NKV_REQUIRE(group_heads > 0 && group_heads <= total_heads, NKV_ERR_INVALID,
              "fast_finish: %d group heads of %d", group_heads, total_heads);
  NKV_REQUIRE((mean == nullptr) == (projected == nullptr), NKV_ERR_INVALID,
              "fast_finish: the value mean and its projected part come together");
  const uintptr_t bits = reinterpret_cast<uintptr_t>(native) | reinterpret_cast<uintptr_t>(lifted) |
                         reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(mean) |
                         reinterpret_cast<uintptr_t>(projected);
  NKV_REQUIRE(bits % 16 == 0, NKV_ERR_INVALID, "fast_finish: arrays must be 16-byte aligned");
  if (rows == 0) return NKV_OK;
  const long long total = rows * group_heads * (d >> 3);
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
#define NKV_FINISH(DT, CORRECT)                                                                     \
  fast_finish_kernel<DT, CORRECT><<<blocks, 256, 0, stream>>>(native, native_lse, lifted, low_lse,  \
      heads, mean, projected, rows, total_heads, group_heads, d, out, out_lse)
  if (dtype == NKV_F32) { if (mean) NKV_FINISH(NKV_F32, true); else NKV_FINISH(NKV_F32, false); }
  else                  { if (mean) NKV_FINISH(NKV_BF16, true); else NKV_FINISH(NKV_BF16, false); }
#undef NKV_FINISH
  NKV_LAUNCH_CHECK("fast_finish_kernel");
  return NKV_OK;
}

// ---- per-head small linear maps of the mixed-dimensional read -----------------------------------
// out[n, g, e] = sum_d x[n, head(g), d] * w[g, d, e]  (fp32 accumulation, one rounding):
// the query reduction q_reduce [h, D, d] and the value lift [h, d, D] of a reader group.
// Block = 32 rows of one group head; the head's matrix sits in shared memory as fp32; a thread owns
// one row and every eighth output column.
template <int DTYPE>
__global__ void __launch_bounds__(256)
head_linear_kernel(const void* x, long long stride_row, long long stride_head, const int32_t* heads,
                   const void* w, long long rows, int din, int dout, int dout_pad, void* out) {
  // Block = 64 rows of one head.  The head's map and the 64 input rows sit in shared memory as
  // fp32; thread (ty, tx) owns rows 4 ty .. 4 ty + 3 and the output columns tx, tx + 16, ...: every
  // value read from shared memory feeds four (a map entry) or dout / 16 (an input) multiply-adds.
  // Each output is one fp32 chain over the input columns in increasing order.
  extern __shared__ float head_linear_smem[];
  constexpr int ROWS = 64, MAXC = 8;            // up to 128 output columns
  float* ws = head_linear_smem;                 // [din][dout]
  float* xs = head_linear_smem + din * dout;    // [din][ROWS + 4]: a column of inputs is contiguous
  const int g = blockIdx.y;
  const int head = heads ? heads[g] : g;
  const long long row0 = static_cast<long long>(blockIdx.x) * ROWS;
  for (int i = threadIdx.x; i < din * dout; i += 256)
    ws[i] = load_float(w, DTYPE, static_cast<size_t>(g) * din * dout + i);
  for (int i = threadIdx.x; i < ROWS * din; i += 256) {
    const int r = i / din, d = i - r * din;
    const long long row = row0 + r;
    xs[d * (ROWS + 4) + r] = row < rows
        ? load_float(x, DTYPE, static_cast<size_t>(row * stride_row + head * stride_head + d)) : 0.f;
  }
  __syncthreads();
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int ncol = (dout + 15) / 16;            // columns tx + 16 k, k < ncol (guarded below)
  float acc[4][MAXC];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int k = 0; k < MAXC; ++k) acc[a][k] = 0.f;
  for (int d = 0; d < din; ++d) {
    const float4 xv = *reinterpret_cast<const float4*>(xs + d * (ROWS + 4) + 4 * ty);
    const float xr[4] = {xv.x, xv.y, xv.z, xv.w};
    const float* wr = ws + d * dout + tx;
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
      if (k < ncol) {
        const float wv = (tx + 16 * k < dout) ? wr[16 * k] : 0.f;
#pragma unroll
        for (int a = 0; a < 4; ++a) acc[a][k] = fmaf(xr[a], wv, acc[a][k]);
      }
    }
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const long long row = row0 + 4 * ty + a;
    if (row >= rows) continue;
    const size_t base = (static_cast<size_t>(row) * gridDim.y + g) * dout_pad;
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
      const int e = tx + 16 * k;
      if (e < dout_pad) store_float(out, DTYPE, base + e, (k < ncol && e < dout) ? acc[a][k] : 0.f);
    }
  }
}

int head_linear(const void* x, int dtype, int64_t stride_row, int64_t stride_head, const int32_t* heads,
                const void* w, int64_t rows, int group_heads, int din, int dout, int dout_pad, void* out,
                cudaStream_t stream) {
  NKV_REQUIRE(dtype == NKV_BF16 || dtype == NKV_F32, NKV_ERR_UNSUPPORTED, "head_linear: dtype %d", dtype);
  NKV_REQUIRE(group_heads > 0 && din > 0 && dout > 0 && dout_pad >= dout, NKV_ERR_INVALID,
              "head_linear: heads=%d din=%d dout=%d pad=%d", group_heads, din, dout, dout_pad);
  const size_t smem = (static_cast<size_t>(din) * dout + static_cast<size_t>(din) * 68) * sizeof(float);
  NKV_REQUIRE(smem <= 200 * 1024 && dout_pad <= 128 && (din * dout) % 4 == 0, NKV_ERR_UNSUPPORTED,
              "head_linear: a %d x %d map (padded to %d) is beyond the built kernel", din, dout, dout_pad);
  if (rows == 0) return NKV_OK;
  dim3 grid(static_cast<unsigned>((rows + 63) / 64), static_cast<unsigned>(group_heads));
  if (dtype == NKV_F32) {
    NKV_CUDA(cudaFuncSetAttribute(head_linear_kernel<NKV_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
    head_linear_kernel<NKV_F32><<<grid, 256, smem, stream>>>(x, stride_row, stride_head, heads, w, rows, din,
                                                             dout, dout_pad, out);
  } else {
    NKV_CUDA(cudaFuncSetAttribute(head_linear_kernel<NKV_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
    head_linear_kernel<NKV_BF16><<<grid, 256, smem, stream>>>(x, stride_row, stride_head, heads, w, rows, din,
                                                              dout, dout_pad, out);
  }
  NKV_LAUNCH_CHECK("head_linear_kernel");
  return NKV_OK;
}

size_t history_moments_workspace_bytes(int tokens, int rank) {
  const size_t slabs = (static_cast<size_t>(tokens > 0 ? tokens : 0) + MOMENT_SLAB - 1) / MOMENT_SLAB;
  return slabs * static_cast<size_t>(rank) * sizeof(float);
}

int history_moments(const nkv_history& h, float* latent_sum, int32_t* center_counts, void* workspace,
                    cudaStream_t stream) {
  NKV_CUDA(cudaMemsetAsync(center_counts, 0, sizeof(int32_t) * static_cast<size_t>(h.center_rows), stream));
  if (h.tokens == 0) {
    NKV_CUDA(cudaMemsetAsync(latent_sum, 0, sizeof(float) * static_cast<size_t>(h.rank), stream));
    return NKV_OK;
  }
  const int slabs = (h.tokens + MOMENT_SLAB - 1) / MOMENT_SLAB;
  const bool vec = h.rank % 8 == 0 && h.group % 8 == 0 && h.rank <= 2048 &&
                   reinterpret_cast<uintptr_t>(h.codes) % 4 == 0;
  if (vec) moments_partial_vec_kernel<<<slabs, 256, 0, stream>>>(h, static_cast<float*>(workspace), center_counts);
  else moments_partial_kernel<<<slabs, 256, 0, stream>>>(h, static_cast<float*>(workspace), center_counts);
  NKV_LAUNCH_CHECK("moments_partial_kernel");
  moments_reduce_kernel<<<(h.rank + 7) / 8, 256, 0, stream>>>(static_cast<const float*>(workspace),
                                                                   slabs, h.rank, latent_sum);
  NKV_LAUNCH_CHECK("moments_reduce_kernel");
  return NKV_OK;
}

}  // namespace nkv
