// Fused codec-attention on tcgen05 tensor cores (bf16 operands, fp32 TMEM accumulators):
// ONE persistent, cooperative launch in which some CTAs rebuild K / V tiles from the
// compressed history and the others attend to them.
//
// The grid is cut into `groups`; a group owns `cons` consumer CTAs and `prod` producer
// CTAs (one CTA per SM) and walks a list of work units (head, history split, block of
// query tiles).  Inside a unit
//   * a producer owns one tensor (K or V) and every (prod/2)-th 128-token tile of it:
//     TMA brings the tile's packed INT4 codes and the head's decoder (or reader) rows
//     into shared memory -- the rows stay resident for the whole unit when they fit --
//     the compute warps expand codes to bf16 latents (code * stored scale, one rounding)
//     straight into tensor memory, tcgen05.mma (A from TMEM) rebuilds the [128 tok x D]
//     tile in TMEM, the epilogue adds bias and the token's centre row with the
//     reference's two bf16 roundings (plus the positional restore) and stores the tile
//     into a slot of the group's tile ring;
//   * a consumer owns up to 256 queries (two 128-row query tiles): TMA brings ring slots
//     into a two-stage K / V buffer, S = Q K^T per query tile in TMEM, online softmax in
//     registers (exp2, lazy rescaling of the O accumulator), P replaces S in TMEM as bf16
//     pairs, O += P V with P from TMEM and V (token-major, read as an MN-major operand)
//     from shared memory.
// The ring is a few MB of device memory (slots of 128 tokens x D for K and for V, `ring`
// slots per group) that is rewritten continuously and stays in the 126 MB L2: every K / V
// tile is rebuilt ONCE per head and read by all of the head's consumers from L2; no K or V
// array of history size exists anywhere and DRAM sees the compressed history only.
// Producers and consumers of a group meet through release / acquire counters in global
// memory (tile published, tile consumed); inside a CTA every hand-off is an mbarrier.
// Every wait, local or global, is bounded: when its cycle budget runs out the CTA raises
// its own abort flag and the launch-wide one, every other wait returns at once, all CTAs
// drain and leave, and the wait-site code lands in the caller's status word.
// No TMA load uses multicast; there are no clusters.
//
// TMEM columns, consumer: [0,128) S / P of query tile 0, [128,256) of tile 1, [256,384) O
// tile 0, [384,512) O tile 1.  Producer: [0,D) the tile accumulator, [256,512) four latent
// staging slots of 64 columns (a pair of 64-column latent chunks each).
#include <mutex>
#include <type_traits>

#include "nkv_internal.h"
#include "nkv_tc.cuh"

namespace nkv {
namespace {

using namespace tc;

constexpr int TOK = 128;          // history tokens per tile
constexpr int QT = 128;           // queries per query tile
constexpr int NQ = 2;             // query tiles per consumer CTA
constexpr int COMPUTE_THREADS = 256;
constexpr int COMPUTE_WARPS = COMPUTE_THREADS / 32;
constexpr int THREADS = COMPUTE_THREADS + 96;
constexpr int CHUNK = 64;         // latent columns per MMA group
constexpr int TILE_BYTES = 128 * 128;  // one [128 rows x 64 bf16] swizzled tile
constexpr int CODE_BLOCK = TOK * 64;   // codes of a pair of chunks: [128 tok x 64 bytes], 64-byte swizzle
constexpr int MAX_NW = 8;         // decoder-row slots (a pair of chunks each) in shared memory
constexpr int NSTAGE = 4;         // latent staging slots in tensor memory
constexpr int NDONE = 8;          // "MMAs of pair g are complete" barriers, indexed by g % 8
constexpr int KVS = 2;            // K / V stages of a consumer
constexpr int META_BYTES = 3072;  // barriers, flags and per-token metadata at the head of shared memory
constexpr int MAX_RING = 56;      // ring slots per group (GF - GF_DONE flag words)
constexpr int NMETA = 4;          // metadata buffers of a producer (it prepares up to four jobs ahead)
constexpr float RESCALE_THRESHOLD = 8.0f;
constexpr float SCORE_WINDOW = 96.0f;   // log2 units a score may exceed the row's reference point by
constexpr int STATUS_SCORE_RANGE = 950;  // status word: a row's scores left that window (its LSE is NaN)
// log2(1 + 2^-9) and 1 / (1 + 2^-9): half a bf16 step above a value, as an exponent offset and back
constexpr float HALF_STEP_LOG2 = 0.0028150156070540f;
constexpr float HALF_STEP_INV = 0.998050682261209f;

enum Bar {
  // consumer
  Q_FULL = 0, Q_FREE = 1, K_FULL = 2, K_FREE = 4, V_FULL = 6, V_FREE = 8, S_FULL = 10, P_READY = 12,
  PV_DONE = 14, O_FREE = 16,
  // producer
  W_FULL = 18, PAIR_DONE = 26, LAT_FULL = 34, META_FULL = 38, META_FREE = 42, CODES_FULL = 46,
  CODES_FREE = 47, OUT_DONE = 48, NUM_BARS = 52
};

// meta block
constexpr int M_SLOT = NUM_BARS * 8;              // TMEM base address
constexpr int M_ABORT = M_SLOT + 4;
constexpr int M_CROW = 512;                       // [NMETA][128] centre row of every token of a tile
static_assert(M_ABORT + 4 <= M_CROW && M_CROW + NMETA * TOK * 4 <= META_BYTES, "meta block layout");

// global flag words
constexpr int F_ABORT = 0;        // launch-wide abort (wait-site code)
constexpr int F_GROUPS = 32;      // then per group GF words:
constexpr int GF = 64;            //   [0, 8): tiles published by producer p of the group (K producers first)
constexpr int GF_DONE = 8;        //   [8, 64): per ring slot, consumers that have taken the slot's tiles
constexpr int MAX_PROD = 8;

struct Params {
  int Q, heads, N, rank, nchunks, npairs, ngroups, group;
  int scale_dtype, nw, w_perm;
  int tiles, tiles_per_split, splits, qchunks;
  int groups, cons, prod, prod_k, ring, units;   // prod producers per group, the first prod_k of them rebuild K tiles
  float scale_log2;
  long long wait_budget;
  nkv_history hk, hv;
  const float* bias_k;
  const float* bias_v;
  uint16_t* out;
  float* lse;
  int32_t* status;
  nkv_rope rope;     // cos_sin == nullptr: keys are used as rebuilt
  nkv_camera cam_k, cam_v;   // matrices == nullptr: no camera transform of that tensor
  uint16_t* ring_k;  // [groups * ring * 128][D]
  uint16_t* ring_v;
  int32_t* flags;
  long long* prof;   // development builds: cycle buckets of group 0's first consumer and first producer
};

struct Unit { int head, z, qc, tile0, nt; };

__device__ __forceinline__ Unit unit_of(const Params& p, int u) {
  Unit r;
  r.z = u % p.splits;
  const int rest = u / p.splits;
  r.head = rest % p.heads;
  r.qc = rest / p.heads;
  r.tile0 = r.z * p.tiles_per_split;
  r.nt = min(p.tiles_per_split, p.tiles - r.tile0);
  return r;
}

// ---- bounded waits ------------------------------------------------------------------------------
struct Ctx {
  volatile int* abort_flag;   // this CTA's (shared memory)
  int32_t* gabort;            // the launch's (global memory)
  long long budget;           // SM cycles per wait
};

__device__ __forceinline__ int ld_relaxed(const int32_t* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// two positive fp32 values -> bf16 pair (lo in the low half) by dropping their low 16 bits
__device__ __forceinline__ uint32_t truncate_bf16x2(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}
__device__ __forceinline__ int ld_acquire(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int4 ld_acquire_v4(const int32_t* p) {
  int4 v;
  asm volatile("ld.acquire.gpu.global.v4.s32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_relaxed_add(int32_t* p, int v) {
  asm volatile("red.relaxed.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release(int32_t* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_add(int32_t* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __noinline__ void raise_abort(const Ctx& c, int code) {
  atomicCAS(const_cast<int*>(c.abort_flag), 0, code);
  atomicCAS(c.gabort, 0, code);
}

// slow path of both waits: true = give up
__device__ __forceinline__ bool wait_expired(const Ctx& c, long long start, int code) {
  if (ld_relaxed(c.gabort) != 0) {   // another CTA gave up: leave too
    atomicCAS(const_cast<int*>(c.abort_flag), 0, 900);
    return true;
  }
  if (clock64() - start > c.budget) {
    raise_abort(c, code);
    return true;
  }
  return false;
}

__device__ __forceinline__ bool mwait(uint64_t* bar, uint32_t parity, const Ctx& c, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  unsigned spins = 0;
  // A waiting warp must not eat the issue slots of the warps that compute on its scheduler (the
  // other query tile's softmax, above all): it parks in the barrier unit and comes back when the
  // phase completes or after a microsecond, whichever is first.
  while (true) {
    if (*c.abort_flag) return false;
    if (mbar_try_wait_parked(bar, parity, 1000u)) return true;
    if ((++spins & 63u) == 0 && wait_expired(c, start, code)) return false;
  }
}

// The same for a whole (converged) warp: every lane waits, and the answer is made uniform so that
// a wait that gives up in some lanes only cannot split the warp in front of a warp-wide barrier.
__device__ __forceinline__ bool mwait_all(uint64_t* bar, uint32_t parity, const Ctx& c, int code) {
  return __all_sync(0xffffffffu, mwait(bar, parity, c, code) ? 1 : 0) != 0;
}

// wait until a global counter (written by other CTAs with release semantics) reaches `target`
__device__ __forceinline__ bool fwait(const int32_t* flag, int target, const Ctx& c, int code) {
  if (ld_acquire(flag) >= target) return true;
  const long long start = clock64();
  unsigned spins = 0;
  while (true) {
    if (*c.abort_flag) return false;
    if (ld_acquire(flag) >= target) return true;
    if ((++spins & 31u) == 0 && wait_expired(c, start, code)) return false;
    __nanosleep(40);
  }
}

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

// Lap timer of one thread (development builds only): adds the cycles since the previous lap to a
// bucket kept in registers; flush() adds the buckets to global memory once, at the end.
#ifdef NKV_DEV
struct Laps {
  long long* out;
  unsigned last;
  unsigned acc[8];
  __device__ __forceinline__ void start(long long* dst, bool on) {
    out = on ? dst : nullptr;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0;
    last = static_cast<unsigned>(clock64());
  }
  __device__ __forceinline__ void lap(int bucket) {
    if (out) {
      const unsigned now = static_cast<unsigned>(clock64());
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i == bucket) acc[i] += now - last;
      last = now;
    }
  }
  __device__ __forceinline__ void flush() {
    if (out) {
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] += acc[i];
    }
  }
};
#else
struct Laps {
  __device__ __forceinline__ void start(long long*, bool) {}
  __device__ __forceinline__ void lap(int) {}
  __device__ __forceinline__ void flush() {}
};
#endif

__device__ __forceinline__ uint32_t bf16x2_max(uint32_t a, uint32_t b) {
  const __nv_bfloat162 m = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                   *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&m);
}

template <int D>
struct Layout {
  static constexpr int DCH = D / 64;                      // 64-column tiles of a head row
  // consumer
  static constexpr int Q_OFF = META_BYTES;                // [NQ][DCH] tiles
  static constexpr int K_OFF = Q_OFF + NQ * DCH * TILE_BYTES;    // [KVS][DCH] tiles [128 tok x 64]
  static constexpr int V_OFF = K_OFF + KVS * DCH * TILE_BYTES;   // [KVS][DCH] tiles, token-major like K
  static constexpr int CONSUMER_BYTES = V_OFF + KVS * DCH * TILE_BYTES;
  // producer: the tile's codes (one block per pair of latent chunks), the centre staging of the
  // epilogue (8 warps x 2 KB), the decoder-row slots, the tokens' scales
  static constexpr int CODES_OFF = META_BYTES;
  static constexpr int SCRATCH_BYTES = COMPUTE_WARPS * 2048;
  __host__ __device__ static int scratch_off(int npairs) { return CODES_OFF + npairs * CODE_BLOCK; }
  static constexpr int SLOT_BYTES = 2 * D * 128;          // a pair of [D rows x 64 latent cols] tiles
  __host__ __device__ static int ring_off(int npairs) { return scratch_off(npairs) + SCRATCH_BYTES; }
  __host__ __device__ static int scales_off(int npairs, int nw) { return ring_off(npairs) + nw * SLOT_BYTES; }
  __host__ __device__ static int producer_bytes(int npairs, int nw, int ngroups) {
    return scales_off(npairs, nw) + NMETA * TOK * ngroups * 2;
  }
};

// ================================================================================ consumer
template <int D>
__device__ __forceinline__ void consumer_role(uint8_t* smem, uint64_t* bars, uint32_t tmem_base,
                                              const CUtensorMap* map_q, const CUtensorMap* map_rk,
                                              const CUtensorMap* map_rv, const Params& p, const Ctx& ctx,
                                              int g, int c) {
  using L = Layout<D>;
  constexpr int DCH = L::DCH;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int R = p.ring;
  int32_t* gflags = p.flags + F_GROUPS + g * GF;
  auto queries_of = [&](const Unit& un, int& q0) {
    q0 = (un.qc * p.cons + c) * (NQ * QT);
    return q0 >= p.Q ? 0 : ((q0 + QT < p.Q) ? 2 : 1);
  };

  if (warp == 8) {
    // ------------------------------------------------------------ TMA: queries, ring -> K / V stages
    if (lane == 0) {
      prefetch_tensormap(map_q);
      prefetch_tensormap(map_rk);
      prefetch_tensormap(map_rv);
      bool ok = true;
      int seq = 0, cseq = 0, ucount = 0;
      int pend_slot = -1, pend_stage = 0, pend_phase = 0;
      int pub[MAX_PROD] = {0, 0, 0, 0, 0, 0, 0, 0};   // cached copy of the producers' counters
      const int PK = p.prod_k, PV = p.prod - p.prod_k;
      Laps laps;
      laps.start(p.prof, p.prof != nullptr && g == 0 && c == 0);
      for (int u = g; u < p.units && ok; u += p.groups) {
        const Unit un = unit_of(p, u);
        int q0;
        const int nq = queries_of(un, q0);
        if (nq > 0) {
          if (ucount > 0) ok = mwait(&bars[Q_FREE], (ucount - 1) & 1, ctx, 101);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars[Q_FULL], nq * DCH * TILE_BYTES);
          for (int i = 0; i < nq; ++i)
            for (int ch = 0; ch < DCH; ++ch)
              tma_load_3d(smem + L::Q_OFF + (i * DCH + ch) * TILE_BYTES, map_q, ch * 64, un.head,
                          q0 + i * QT, &bars[Q_FULL]);
          ++ucount;
        }
        for (int t = 0; t < un.nt && ok; ++t, ++seq) {
          const int slot = seq % R;
          const int stage = cseq % KVS, use = cseq / KVS;
          const int row = (g * R + slot) * TOK;
          laps.lap(7);
          // tile `seq` of K comes from K producer seq % PK as its job number seq / PK, V likewise from
          // V producer PK + seq % PV; the counters are re-read only when the cached copy falls short
          {
            const int who = seq % PK, need = seq / PK + 1;
            const int who_v = PK + seq % PV, need_v = seq / PV + 1;
            if (pub[who] < need || pub[who_v] < need_v) {
              const long long start = clock64();
              unsigned spins = 0;
              while (true) {
                const int4 lo = ld_acquire_v4(gflags);
                pub[0] = lo.x; pub[1] = lo.y; pub[2] = lo.z; pub[3] = lo.w;
                if (p.prod > 4) {
                  const int4 hi = ld_acquire_v4(gflags + 4);
                  pub[4] = hi.x; pub[5] = hi.y; pub[6] = hi.z; pub[7] = hi.w;
                }
                if (pub[who] >= need && pub[who_v] >= need_v) break;
                if (*ctx.abort_flag) { ok = false; break; }
                if ((++spins & 31u) == 0 && wait_expired(ctx, start, 102)) { ok = false; break; }
                __nanosleep(40);
              }
              if (!ok) break;
              fence_proxy_async_all();   // the tiles were written with ordinary stores, TMA reads them
            }
          }
          laps.lap(0);
          if (nq > 0) {
            if (use >= 1) ok = mwait(&bars[K_FREE + stage], (use - 1) & 1, ctx, 103);
            if (!ok) break;
            mbar_arrive_expect_tx(&bars[K_FULL + stage], DCH * TILE_BYTES);
            for (int ch = 0; ch < DCH; ++ch)
              tma_load_2d(smem + L::K_OFF + (stage * DCH + ch) * TILE_BYTES, map_rk, ch * 64, row,
                          &bars[K_FULL + stage]);
            laps.lap(1);
            if (use >= 1) ok = mwait(&bars[V_FREE + stage], (use - 1) & 1, ctx, 105);
            if (!ok) break;
            mbar_arrive_expect_tx(&bars[V_FULL + stage], DCH * TILE_BYTES);
            for (int ch = 0; ch < DCH; ++ch)
              tma_load_2d(smem + L::V_OFF + (stage * DCH + ch) * TILE_BYTES, map_rv, ch * 64, row,
                          &bars[V_FULL + stage]);
          }
          laps.lap(3);
          // the previous tile has landed in shared memory by now: hand its ring slot back.  The
          // slot's data has been read (the copies are complete), so a relaxed add is enough.
          if (pend_slot >= 0) {
            ok = mwait(&bars[K_FULL + pend_stage], pend_phase, ctx, 106) &&
                 mwait(&bars[V_FULL + pend_stage], pend_phase, ctx, 107);
            if (!ok) break;
            laps.lap(4);
            red_relaxed_add(gflags + GF_DONE + pend_slot, 1);
            pend_slot = -1;
            laps.lap(5);
          }
          if (nq > 0) {
            pend_slot = slot; pend_stage = stage; pend_phase = use & 1;
            ++cseq;
          } else {   // nothing to load for this block of queries: the slot is not needed here
            red_relaxed_add(gflags + GF_DONE + slot, 1);
          }
        }
      }
      if (ok && pend_slot >= 0) {
        ok = mwait(&bars[K_FULL + pend_stage], pend_phase, ctx, 106) &&
             mwait(&bars[V_FULL + pend_stage], pend_phase, ctx, 107);
        if (ok) red_relaxed_add(gflags + GF_DONE + pend_slot, 1);
      }
      laps.flush();
      if (!ok) {  // let copies already in flight land before the CTA goes away
        const long long start = clock64();
        while (clock64() - start < (1ll << 21)) {}
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // -------------------------------------------------------------- MMA issuer
    // the whole warp runs the (uniform) control flow; one elected lane issues
    const bool leader = elect_one();
    const uint32_t idesc_s = make_idesc_bf16(128, TOK);                // [128 q] x [128 tok]
    const uint32_t idesc_pv = make_idesc_bf16(128, D) | (1u << 16);    // [128 q] x [D], B (V) MN-major
    const uint32_t smem_base = smem_u32(smem);
    auto issue_s = [&](int i, int stage) {
#pragma unroll
      for (int ch = 0; ch < DCH; ++ch) {
        const uint64_t a_desc = make_smem_desc_sw128(smem_base + L::Q_OFF + (i * DCH + ch) * TILE_BYTES);
        const uint64_t b_desc = make_smem_desc_sw128(smem_base + L::K_OFF + (stage * DCH + ch) * TILE_BYTES);
        if (leader) mma_bf16(tmem_base + i * 128, a_desc, b_desc, idesc_s, ch > 0);
        if (leader) mma_bf16(tmem_base + i * 128, a_desc + 2, b_desc + 2, idesc_s, true);
        if (leader) mma_bf16(tmem_base + i * 128, a_desc + 4, b_desc + 4, idesc_s, true);
        if (leader) mma_bf16(tmem_base + i * 128, a_desc + 6, b_desc + 6, idesc_s, true);
      }
      if (leader) mma_commit(&bars[S_FULL + i]);
    };
    // P (bf16 pairs) sits in the first 64 columns of the S region it was computed from.  V is the B
    // operand in MN-major form: [tokens (K) x d (N)] with d contiguous, 64-column tiles 16 KB apart
    // (leading offset), 8-token groups 1 KB apart (stride offset); a K step of 16 tokens moves the
    // start by 2 KB (128 in the address field)
    auto issue_pv = [&](int i, int stage, bool accumulate) {
      const uint64_t b_desc = make_smem_desc_sw128_mn(smem_base + L::V_OFF + stage * DCH * TILE_BYTES, TILE_BYTES);
      const uint32_t p_addr = tmem_base + i * 128;
      const uint32_t o_addr = tmem_base + 256 + i * 128;
#pragma unroll
      for (int ks = 0; ks < TOK / 16; ++ks)
        if (leader) mma_bf16_ts(o_addr, p_addr + 8 * ks, b_desc + 128 * ks, idesc_pv, accumulate || ks > 0);
      if (leader) mma_commit(&bars[PV_DONE + i]);
    };
    bool ok = true;
    int cseq = 0, ucount = 0;
    int ctile[NQ] = {0, 0}, cunit[NQ] = {0, 0};   // tiles / units each query tile's chain has done
    Laps laps;
    laps.start(p.prof + 8, p.prof != nullptr && g == 0 && c == 0 && leader);
    for (int u = g; u < p.units && ok; u += p.groups) {
      const Unit un = unit_of(p, u);
      int q0;
      const int nq = queries_of(un, q0);
      if (nq == 0) continue;
      ok = mwait_all(&bars[Q_FULL], ucount & 1, ctx, 200);
      if (!ok) break;
      {
        const int stage = cseq % KVS;
        ok = mwait_all(&bars[K_FULL + stage], (cseq / KVS) & 1, ctx, 201);
        if (!ok) break;
        tc_fence_after();
        for (int i = 0; i < nq; ++i) issue_s(i, stage);
        if (leader) mma_commit(&bars[K_FREE + stage]);
      }
      for (int t = 0; t < un.nt && ok; ++t) {
        const int cur = cseq + t, stage = cur % KVS, phase = (cur / KVS) & 1;
        const int nstage = (cur + 1) % KVS;
        for (int i = 0; i < nq && ok; ++i) {
          const int ci = ctile[i] + t;
          laps.lap(7);
          ok = mwait_all(&bars[P_READY + i], ci & 1, ctx, 210 + i);
          laps.lap(i);
          if (ok && i == 0) ok = mwait_all(&bars[V_FULL + stage], phase, ctx, 212);
          laps.lap(2);
          // the first PV of a unit overwrites O: the previous unit's rows must have been read out
          if (ok && t == 0 && cunit[i] > 0) ok = mwait_all(&bars[O_FREE + i], (cunit[i] - 1) & 1, ctx, 214 + i);
          if (!ok) break;
          tc_fence_after();
          issue_pv(i, stage, t > 0);
          if (i == nq - 1 && leader) mma_commit(&bars[V_FREE + stage]);
          laps.lap(3);
          if (t + 1 < un.nt) {
            // S of the next tile overwrites P of this one.  It is issued right behind the PV that
            // reads P: the tensor core executes the MMAs of one issuing thread in order
            if (i == 0) ok = mwait_all(&bars[K_FULL + nstage], ((cur + 1) / KVS) & 1, ctx, 216);
            if (!ok) break;
            laps.lap(4);
            issue_s(i, nstage);
            laps.lap(5);
            if (i == nq - 1 && leader) mma_commit(&bars[K_FREE + nstage]);
          }
        }
      }
      if (!ok) break;
      if (leader) mma_commit(&bars[Q_FREE]);   // every S MMA of the unit is done: Q may be replaced
      cseq += un.nt;
      ++ucount;
      for (int i = 0; i < nq; ++i) { ctile[i] += un.nt; ++cunit[i]; }
    }
    laps.flush();
    __syncwarp();
  } else if (warp < COMPUTE_WARPS) {
    // ------------------------------------------------------------ softmax: one thread per query row
    const int wg = tid >> 7;                    // query tile served
    const int row = tid & 127;                  // TMEM lane == query row
    const uint32_t lane_sel = static_cast<uint32_t>(32 * (warp & 3)) << 16;
    bool ok = true;
    int ci = 0;
    int u = g;
    Laps laps;
    laps.start(p.prof + 16, p.prof != nullptr && g == 0 && c == 0 && tid == 0);
    for (; u < p.units && ok; u += p.groups) {
      const Unit un = unit_of(p, u);
      int q0;
      const int nq = queries_of(un, q0);
      if (wg >= nq) continue;
      float m_used = -INFINITY, l_run = 0.f, m_seen = -INFINITY;
      bool saturated = false;
      for (int t = 0; t < un.nt && ok; ++t, ++ci) {
        const int valid = min(TOK, p.N - (un.tile0 + t) * TOK);
        laps.lap(2);
        ok = mwait_all(&bars[S_FULL + wg], ci & 1, ctx, 300 + wg);
        if (!ok) break;
        tc_fence_after();
        laps.lap(0);
        // S of this tile was issued behind PV of the previous one and its commit covers both, so O is
        // up to date here
        const uint32_t s_addr = tmem_base + lane_sel + wg * 128;
        const uint32_t o_addr = tmem_base + lane_sel + 256 + wg * 128;
        // moves the reference point of the row: O and the running sum are scaled by 2^(old - new)
        auto move_reference = [&](float m_new) {
          const float m_next = fmaxf(m_used, m_new);
          const float alpha = exp2f(m_used - m_next);   // 0 on the first tile (m_used = -inf)
          if (t > 0) {
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
        };
        // The reference point (the exponent every weight of the row is taken against) is exact on
        // the first tile of a unit and on a ragged tile: row maximum first, then the weights.  On
        // every other tile it moves BETWEEN tiles, by the maximum the previous tile saw, so that no
        // exponential ever waits for a maximum; a tile's weights may then exceed 1 by the factor its
        // scores exceed the reference, which fp32 sums and bf16 weights hold up to 2^SCORE_WINDOW.
        if (t == 0 || valid != TOK) {
          float mx = -INFINITY;
          uint32_t raw[2][32];
          tmem_ld32_issue(s_addr, raw[0]);
#pragma unroll
          for (int cc = 0; cc < TOK / 32; ++cc) {
            uint32_t (&cur)[32] = raw[cc & 1];
            tmem_ld32_wait(cur);
            if (cc + 1 < TOK / 32) tmem_ld32_issue(s_addr + (cc + 1) * 32, raw[(cc + 1) & 1]);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (cc * 32 + j < valid) mx = fmaxf(mx, __uint_as_float(cur[j]));
          }
          m_seen = fmaxf(m_seen, mx * p.scale_log2);
        }
        if (__any_sync(0xffffffffu, m_seen > m_used + RESCALE_THRESHOLD)) move_reference(m_seen);
        // One pass over the scores: P (bf16 pairs) replaces S in place -- the 16 cells written per
        // step lie below the 32 read -- and the load of the next 32 scores stays in flight under the
        // exponentials of the current ones.
        // Weights go to bf16 by dropping the low 16 bits (one byte permute per pair) instead of a
        // rounding conversion, which runs on the same quarter-rate unit as the exponentials and
        // would take a third of its time.  So that the dropped bits do not bias the weights, every
        // weight is raised by half a bf16 step first -- for free, as HALF_STEP_LOG2 in the exponent --
        // and the row sum, which then carries the same factor, is divided by it once per unit.
        const float neg_ref = HALF_STEP_LOG2 - m_used;
        float sum = 0.f, sum_b = 0.f, sum_c = 0.f, sum_d = 0.f;   // four chains instead of one
        uint32_t pmax_a = 0u, pmax_b = 0u;
        if (valid == TOK) {
          // The whole row at once: four 32-column loads, ONE wait, and then a single run of
          // instructions without a fence in it, so that the exponential unit's work of one quarter
          // overlaps the arithmetic and the packing of its neighbours (a wait per quarter kept every
          // quarter a closed block: arguments, exponentials, sums, each draining before the next).
          uint32_t raw[4][32];
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) tmem_ld32_issue(s_addr + cc * 32, raw[cc]);
          tmem_ld128_wait(raw[0], raw[1], raw[2], raw[3]);
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t (&cur)[32] = raw[cc];
            uint32_t packed[16];
            float w[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) w[j] = fmaf(__uint_as_float(cur[j]), p.scale_log2, neg_ref);
#pragma unroll
            for (int j = 0; j < 32; ++j) w[j] = exp2_approx(w[j]);
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              sum += w[j]; sum_b += w[j + 1]; sum_c += w[j + 2]; sum_d += w[j + 3];
              packed[j >> 1] = truncate_bf16x2(w[j], w[j + 1]);
              packed[(j >> 1) + 1] = truncate_bf16x2(w[j + 2], w[j + 3]);
            }
            // the largest weight of the quarter, on the packed pairs (weights are positive, so the
            // bf16 bit patterns order like the numbers): half an instruction per score
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              pmax_a = bf16x2_max(pmax_a, packed[j]);
              pmax_b = bf16x2_max(pmax_b, packed[j + 1]);
            }
            tmem_st16(s_addr + cc * 16, packed);
          }
        } else {
          uint32_t raw[2][32];
          tmem_ld32_issue(s_addr, raw[0]);
#pragma unroll
          for (int cc = 0; cc < TOK / 32; ++cc) {
            uint32_t (&cur)[32] = raw[cc & 1];
            tmem_ld32_wait(cur);
            if (cc + 1 < TOK / 32) tmem_ld32_issue(s_addr + (cc + 1) * 32, raw[(cc + 1) & 1]);
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float p0 = (cc * 32 + j < valid) ? exp2f(fmaf(__uint_as_float(cur[j]), p.scale_log2, neg_ref)) : 0.f;
              float p1 = (cc * 32 + j + 1 < valid) ? exp2f(fmaf(__uint_as_float(cur[j + 1]), p.scale_log2, neg_ref)) : 0.f;
              sum += p0 + p1;
              packed[j >> 1] = truncate_bf16x2(p0, p1);
            }
            tmem_st16(s_addr + cc * 16, packed);
          }
        }
        if (valid == TOK) {
          // largest weight 2^(score - reference) -> the largest score the tile saw (to 2^-8)
          const uint32_t pm = bf16x2_max(pmax_a, pmax_b);
          const float wmax = fmaxf(__uint_as_float(pm << 16), __uint_as_float(pm & 0xFFFF0000u));
          m_seen = fmaxf(m_seen, m_used + log2f(wmax));
          // a weight beyond the window has overflowed or lost its meaning: the row cannot be trusted
          saturated = saturated || !(wmax < exp2f(SCORE_WINDOW));
        }
        laps.lap(1);
        tmem_wait_st();
        laps.lap(6);
        l_run += (sum + sum_b) + (sum_c + sum_d);
        tc_fence_before();
        warp_arrive(&bars[P_READY + wg], lane);
      }
      if (!ok) break;
      // ---- the unit's rows: O / l and the natural-log LSE (partial number z when the history is split)
      ok = mwait_all(&bars[PV_DONE + wg], (ci - 1) & 1, ctx, 310 + wg);
      if (!ok) break;
      tc_fence_after();
      const int qrow = q0 + wg * QT + row;
      l_run *= HALF_STEP_INV;    // the weights were summed with the half-step factor on them
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      const uint32_t o_addr = tmem_base + lane_sel + 256 + wg * 128;
      const size_t split_rows = static_cast<size_t>(un.z) * p.Q * p.heads;
      uint16_t* dst = p.out + (split_rows + static_cast<size_t>(qrow) * p.heads + un.head) * D;
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
      if (qrow < p.Q) {
        p.lse[split_rows + static_cast<size_t>(qrow) * p.heads + un.head] =
            saturated ? __int_as_float(0x7fc00000)
                      : (l_run > 0.f ? (m_used + log2f(l_run)) * 0.6931471805599453f : -INFINITY);
        if (saturated && p.status) atomicCAS(p.status, 0, STATUS_SCORE_RANGE);
      }
      tc_fence_before();
      warp_arrive(&bars[O_FREE + wg], lane);
      laps.lap(3);
    }
    laps.flush();
    // a launch that gave up must not hand back rows that look like results: the unit it stopped in
    // and every later one get NaN in their LSE
    if (!ok) {
      for (; u < p.units; u += p.groups) {
        const Unit un = unit_of(p, u);
        int q0;
        const int nq = queries_of(un, q0);
        const int qrow = q0 + wg * QT + row;
        if (wg < nq && qrow < p.Q)
          p.lse[static_cast<size_t>(un.z) * p.Q * p.heads + static_cast<size_t>(qrow) * p.heads + un.head] =
              __int_as_float(0x7fc00000);
      }
    }
  }
}

// ================================================================================ producer
template <int D, bool ROPE, bool CAM>
__device__ __forceinline__ void producer_role(uint8_t* smem, uint64_t* bars, uint32_t tmem_base,
                                              const CUtensorMap* map_w, const CUtensorMap* map_c,
                                              const Params& p, const Ctx& ctx, int g, int pidx) {
  using L = Layout<D>;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int R = p.ring;
  const int tensor = pidx < p.prod_k ? 0 : 1;                   // 0: this CTA rebuilds K tiles, 1: V tiles
  const int PH = tensor ? p.prod - p.prod_k : p.prod_k;         // producers of its kind
  const int mine = tensor ? pidx - p.prod_k : pidx;             // it takes the tiles with seq % PH == mine
  const nkv_history& hist = tensor ? p.hv : p.hk;
  const int nchunks = p.nchunks, npairs = p.npairs, ng = p.ngroups, nw = p.nw;
  const bool resident = npairs <= nw;      // the head's decoder rows stay in shared memory for a whole unit
  const int ring_off = L::ring_off(npairs);
  int32_t* gflags = p.flags + F_GROUPS + g * GF;
  int* crow = reinterpret_cast<int*>(smem + M_CROW);                                        // [NMETA buf][128]
  uint16_t* scales = reinterpret_cast<uint16_t*>(smem + L::scales_off(npairs, nw));         // [NMETA buf][128][ng]
  uint16_t* ring = tensor ? p.ring_v : p.ring_k;

  if (warp == 8) {
    // ------------------------------------------------------------ TMA: codes and decoder rows
    if (lane == 0) {
      prefetch_tensormap(map_w);
      prefetch_tensormap(map_c);
      bool ok = true;
      int seq = 0, jobs = 0, gp = 0;   // gp: running pair number over all jobs of this CTA
      for (int u = g; u < p.units && ok; u += p.groups) {
        const Unit un = unit_of(p, u);
        bool first = true;
        for (int t = 0; t < un.nt && ok; ++t, ++seq) {
          if (seq % PH != mine) continue;
          // the tile's codes: issued as soon as the previous job's codes are expanded, so that they
          // land during that job's epilogue
          if (jobs > 0) ok = mwait(&bars[CODES_FREE], (jobs - 1) & 1, ctx, 401);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars[CODES_FULL], npairs * CODE_BLOCK);
          for (int pi = 0; pi < npairs; ++pi)   // bytes past the row or the history read as zero
            tma_load_2d(smem + L::CODES_OFF + pi * CODE_BLOCK, map_c, pi * 64, (un.tile0 + t) * TOK,
                        &bars[CODES_FULL]);
          for (int pi = 0; pi < npairs && ok; ++pi) {
            const int n = min(2, nchunks - 2 * pi);
            int slot;
            if (resident) {
              if (!first) continue;
              slot = pi;
              // the slot's last reader was pair pi of this CTA's previous job
              if (jobs > 0) {
                const int last = gp - npairs + pi;
                ok = mwait(&bars[PAIR_DONE + (last & (NDONE - 1))], (last / NDONE) & 1, ctx, 402);
              }
            } else {
              const int load = gp + pi;
              slot = load % nw;
              if (load >= nw)
                ok = mwait(&bars[PAIR_DONE + ((load - nw) & (NDONE - 1))], ((load - nw) / NDONE) & 1, ctx, 403);
            }
            if (!ok) break;
            mbar_arrive_expect_tx(&bars[W_FULL + slot], n * D * 128);
            for (int j = 0; j < n; ++j)
              tma_load_2d(smem + ring_off + slot * L::SLOT_BYTES + j * D * 128, map_w, (2 * pi + j) * CHUNK,
                          un.head * D, &bars[W_FULL + slot]);
          }
          gp += npairs;
          ++jobs;
          first = false;
        }
      }
      if (!ok) {
        const long long start = clock64();
        while (clock64() - start < (1ll << 21)) {}
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // -------------------------------------------------------------- MMA issuer
    const bool leader = elect_one();
    const uint32_t idesc_dec = make_idesc_bf16(128, D);   // [128 tok] x [D columns]
    const uint32_t smem_base = smem_u32(smem);
    bool ok = true;
    int seq = 0, gp = 0, wgen = 0, jobs = 0;   // wgen: units whose rows this CTA has loaded (resident form)
    Laps laps;
    laps.start(p.prof + (pidx == 0 ? 32 : 48), p.prof != nullptr && g == 0 && (pidx == 0 || pidx == p.prod_k) && leader);
    for (int u = g; u < p.units && ok; u += p.groups) {
      const Unit un = unit_of(p, u);
      bool first = true;
      for (int t = 0; t < un.nt && ok; ++t, ++seq) {
        if (seq % PH != mine) continue;
        const uint32_t acc = tmem_base + (jobs & 1) * 128;   // two accumulators: the epilogue of a job runs
        ++jobs;                                              // under the MMAs of the next one
        for (int pi = 0; pi < npairs && ok; ++pi, ++gp) {
          const int n = min(2, nchunks - 2 * pi);
          int slot;
          if (resident) {
            slot = pi;
            if (first) ok = mwait_all(&bars[W_FULL + slot], wgen & 1, ctx, 410);
          } else {
            slot = gp % nw;
            ok = mwait_all(&bars[W_FULL + slot], (gp / nw) & 1, ctx, 411);
          }
          const int st = gp % NSTAGE;
          laps.lap(0);
          ok = ok && mwait_all(&bars[LAT_FULL + st], (gp / NSTAGE) & 1, ctx, 412);
          if (!ok) break;
          tc_fence_after();
          laps.lap(1);
          // descriptors are built once per chunk; a K = 16 step adds 32 bytes (2 in the address
          // field) to the shared-memory operand and 8 columns to the TMEM operand
          for (int j = 0; j < n; ++j) {
            const uint64_t w_desc = make_smem_desc_sw128(smem_base + ring_off + slot * L::SLOT_BYTES + j * D * 128);
            const uint32_t lat = tmem_base + 256 + st * 64 + j * 32;   // chunk staged in TMEM
            if (leader) mma_bf16_ts(acc, lat, w_desc, idesc_dec, pi + j > 0);
            if (leader) mma_bf16_ts(acc, lat + 8, w_desc + 2, idesc_dec, true);
            if (leader) mma_bf16_ts(acc, lat + 16, w_desc + 4, idesc_dec, true);
            if (leader) mma_bf16_ts(acc, lat + 24, w_desc + 6, idesc_dec, true);
          }
          // frees the staging slot (and the decoder rows); on the last pair: accumulator done
          if (leader) mma_commit(&bars[PAIR_DONE + (gp & (NDONE - 1))]);
          laps.lap(2);
        }
        if (first && resident) ++wgen;
        first = false;
      }
    }
    laps.flush();
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------------------------- everything that waits on global memory, off the
    // compute warps' path: per-token metadata up to four jobs ahead, the ring slot's release by the
    // consumers (META_FULL also says "the slot is free"), and the publication of finished tiles
    bool ok = true;
    int seq = 0, jobs = 0;
    // Tile of job j: its stores happen before this release by the OUT_DONE barrier, and a release
    // is cumulative, so a consumer that sees the counter sees the tile.
    auto publish = [&](int j) {
      // (job j + NMETA cannot start before job j is published, so the barrier never runs a phase ahead)
      const bool done = mwait_all(&bars[OUT_DONE + j % NMETA], (j / NMETA) & 1, ctx, 505);
      if (done && lane == 0) st_release(gflags + pidx, j + 1);
      return done;
    };
    // This producer's jobs in order: (first token, tile number within the group).
    int it_u = g, it_t = 0, it_seq = 0;
    Unit it_un = unit_of(p, it_u < p.units ? it_u : 0);
    auto next_job = [&](int& t0, int& tile_seq) {
      while (it_u < p.units) {
        if (it_t < it_un.nt) {
          const int t = it_t++, sq = it_seq++;
          if (sq % PH == mine) {
            t0 = (it_un.tile0 + t) * TOK;
            tile_seq = sq;
            return true;
          }
        } else {
          it_u += p.groups;
          it_t = 0;
          if (it_u < p.units) it_un = unit_of(p, it_u);
        }
      }
      return false;
    };
    // A job's per-token metadata (centre row, scale).  The centre row needs the token's segment: a
    // binary search over the segment table, four or five DEPENDENT loads that miss the first-level
    // cache (the centre gathers sweep it) -- several thousand cycles per job when every token
    // searches, more than the compute warps need for the job.  A tile nearly always lies inside one
    // segment, so the segment found last (its token range and centre-row base) is kept in registers
    // and only a tile that leaves it searches again; a tile that straddles segments searches per
    // token.  The id and scale loads of job j + 2 are issued before job j is handled.
    struct Meta { int t0, seq, crow[TOK / 32]; uint16_t scale[TOK / 32]; bool valid; };
    int seg_lo = 0, seg_hi = 0, seg_row = 0;   // tokens [seg_lo, seg_hi) take centre rows from seg_row on
    auto fetch = [&](Meta& m) {
      m.valid = next_job(m.t0, m.seq);
      bool one_segment = false;
      if (m.valid) {
        const int first = m.t0, last = min(m.t0 + TOK, p.N) - 1;
        if (first < seg_lo || first >= seg_hi) {
          const int sg = find_segment(hist.seg_start, hist.segments, first);
          seg_lo = hist.seg_start[sg];
          seg_hi = sg + 1 < hist.segments ? hist.seg_start[sg + 1] : 0x7fffffff;
          seg_row = hist.seg_center_row[sg];
        }
        one_segment = first >= seg_lo && last < seg_hi;
      }
#pragma unroll
      for (int k = 0; k < TOK / 32; ++k) {
        const int tok = m.t0 + lane + 32 * k;
        const bool in = m.valid && tok < p.N;
        m.crow[k] = !in ? 0 : (one_segment ? seg_row + load_id(hist.ids, hist.id_bytes, tok) : center_row_of(hist, tok));
        m.scale[k] = (in && ng == 1) ? __ldg(static_cast<const uint16_t*>(hist.scales) + tok) : uint16_t(0);
      }
    };
    Meta cur{}, ahead1{}, ahead2{};
    fetch(cur);
    fetch(ahead1);
    fetch(ahead2);
    while (cur.valid && ok) {
      {
        const int b = jobs % NMETA, use = jobs / NMETA;
        const int t0 = cur.t0;
        seq = cur.seq;
        if (use >= 1) {   // job jobs - NMETA is finished: its metadata buffer is free, its tile is stored
          ok = mwait_all(&bars[META_FREE + b], (use - 1) & 1, ctx, 420 + b);
          ok = ok && publish(jobs - NMETA);
        }
        if (!ok) break;
        {   // every consumer of the group must have taken the previous tiles of this job's ring slot
          int okf = 1;
          if (lane == 0) okf = fwait(gflags + GF_DONE + seq % R, p.cons * (seq / R), ctx, 504) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, okf, 0) != 0;
        }
        if (!ok) break;
#pragma unroll
        for (int k = 0; k < TOK / 32; ++k) {
          const int r = lane + 32 * k;
          crow[b * TOK + r] = cur.crow[k];
          if (ng == 1) scales[b * TOK + r] = cur.scale[k];
        }
        if (ng > 1) {
          for (int r = lane; r < TOK; r += 32) {
            const int tok = t0 + r;
            const bool in = tok < p.N;
            const uint16_t* src = static_cast<const uint16_t*>(hist.scales) + static_cast<size_t>(tok) * ng;
            uint16_t* dst = scales + static_cast<size_t>(b * TOK + r) * ng;
            for (int gi = 0; gi < ng; ++gi) dst[gi] = in ? src[gi] : 0;
          }
        }
        warp_arrive(&bars[META_FULL + b], lane);
        ++jobs;
      }
      cur = ahead1;
      ahead1 = ahead2;
      fetch(ahead2);
    }
    for (int j = jobs >= NMETA ? jobs - NMETA : 0; j < jobs && ok; ++j) ok = publish(j);
  } else {
    // ------------------------------------------------------------ compute warps: expand, epilogue
    const int wg = tid >> 7;                    // which half of the columns (of a chunk / of the tile)
    const int row = tid & 127;                  // TMEM lane == token row
    const uint32_t lane_sel = static_cast<uint32_t>(32 * (warp & 3)) << 16;
    const nkv_camera& cam = tensor ? p.cam_v : p.cam_k;
    bool ok = true;
    int seq = 0, jobs = 0, gp = 0;
    Laps laps;
    laps.start(p.prof + (pidx == 0 ? 24 : 40), p.prof != nullptr && g == 0 && (pidx == 0 || pidx == p.prod_k) && tid == 0);
    // A job runs in two stages: the codes are expanded (and the MMAs started) right away, its
    // epilogue follows after the NEXT job's expansion, so that the MMAs' tail, the accumulator read
    // and the ring stores of one job hide under the expansion of the following one.
    struct Job { int head, t0, valid, slot, num, last_pair; };
    Job prev{};
    bool have_prev = false;
    auto expand = [&](const Job& job) {
        const int mb = job.num % NMETA;
        laps.lap(7);
        ok = mwait_all(&bars[META_FULL + mb], (job.num / NMETA) & 1, ctx, 500);
        laps.lap(6);
        ok = ok && mwait_all(&bars[CODES_FULL], job.num & 1, ctx, 501);
        if (!ok) return;
        laps.lap(0);
        // ---- expand the tile's codes to bf16 latent chunks in tensor memory (A of the decode MMA)
        // this thread's 16 bytes of chunk j of pair pi: 16-byte unit 2 j + wg of row `row`, swizzled
        const uint8_t* codes = smem + L::CODES_OFF + row * 64;
        const int unit_xor = (row >> 1) & 3;
        auto code_at = [&](int c) {
          return *reinterpret_cast<const uint4*>(codes + (c >> 1) * CODE_BLOCK +
                                                 ((((c & 1) * 2 + wg) ^ unit_xor) << 4));
        };
        const uint16_t* my_scales = scales + static_cast<size_t>(mb * TOK + row) * ng;
        // codes of the pair after the one being expanded are fetched ahead of the wait for its slot
        uint4 code_next[2];
        code_next[0] = code_at(0);
        code_next[1] = nchunks > 1 ? code_at(1) : make_uint4(0, 0, 0, 0);
        // The pair loop exists twice: FASTQ is the common deployment (one bf16 scale per token,
        // decoder rows in kernel order) with every choice made at compile time; the other copy keeps
        // the run-time choices (grouped or fp16 scales, natural-order rows).
        auto expand_pairs = [&](auto fast_tag) {
          constexpr bool FASTQ = decltype(fast_tag)::value;
          for (int c0 = 0; c0 < nchunks && ok; c0 += 2, ++gp) {
            const int n = min(2, nchunks - c0);   // chunks in this pair
            const uint4 code_cur[2] = {code_next[0], code_next[1]};
            if (c0 + 2 < nchunks) code_next[0] = code_at(c0 + 2);
            if (c0 + 3 < nchunks) code_next[1] = code_at(c0 + 3);
            const int st = gp % NSTAGE;
            // the staging slot's previous tenant is pair gp - NSTAGE
            if (gp >= NSTAGE)
              ok = mwait_all(&bars[PAIR_DONE + ((gp - NSTAGE) & (NDONE - 1))], ((gp - NSTAGE) / NDONE) & 1, ctx, 502);
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
                tmem_st16(tmem_base + lane_sel + 256 + st * 64 + j * 32 + wg * 16, packed);
              }
            }
            tmem_wait_st();
            tc_fence_before();
            warp_arrive(&bars[LAT_FULL + st], lane);
          }
        };
        if (p.w_perm && p.scale_dtype == NKV_BF16 && ng == 1) expand_pairs(std::true_type{});
        else expand_pairs(std::false_type{});
        if (!ok) return;
        laps.lap(1);
        fence_proxy_async();   // the codes were read; TMA may overwrite them
        warp_arrive(&bars[CODES_FREE], lane);
    };
    auto epilogue = [&](const Job& job) {
        const int head = job.head, t0 = job.t0, valid = job.valid, mb = job.num % NMETA;
        const int slot = job.slot;   // free: the metadata warp has checked that before META_FULL
        const uint32_t acc = tmem_base + (job.num & 1) * 128;
        // ---- epilogue: bias, centre, two bf16 roundings, positional restore; D / 2 columns per thread
        // in rounds of 32
        const bool in = row < valid;
        constexpr int ROUNDS = D / 64;
        uint16_t* const slot_rows = ring + static_cast<size_t>(g * R + slot) * TOK * D;
        {
          // positional restore (K tiles only): this token's frame / row / column
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
          const bool transform = CAM && cam.matrices != nullptr;
          const float* cam_frame = nullptr;
          if (transform)
            cam_frame = cam.matrices +
                        static_cast<size_t>(min((t0 + row) / cam.tokens_per_frame, cam.frames - 1)) * 64;
          const float* bias_head = (tensor ? p.bias_v : p.bias_k) + head * D;
          // accumulator complete: the tile's last pair is pair gp - 1
          // Centre rows of this warp's 32 tokens (32 columns = 64 bytes per round), gathered
          // cooperatively: 4 lanes read one row's 16-byte pieces, so a load instruction touches
          // 8 lines instead of 32; the rows are redistributed through a swizzled staging area.
          // All rounds are requested here, ahead of the accumulator wait.
          constexpr int PIECES = 4, RPI = 8;
          uint4 cen_all[ROUNDS][PIECES];
          {
            const int wrow0 = 32 * (warp & 3);
#pragma unroll
            for (int sub = 0; sub < ROUNDS; ++sub) {
              const uint16_t* cbase = static_cast<const uint16_t*>(hist.centers) +
                                      static_cast<size_t>(head) * D + wg * (D / 2) + sub * 32;
#pragma unroll
              for (int i = 0; i < PIECES; ++i) {
                const int rloc = i * RPI + lane / PIECES, piece = lane % PIECES;
                const int crow_i = crow[mb * TOK + wrow0 + rloc];
                cen_all[sub][i] = __ldg(reinterpret_cast<const uint4*>(
                    cbase + static_cast<size_t>(crow_i) * hist.center_width + piece * 8));
              }
            }
          }
          bool waited = false;
#pragma unroll
          for (int sub = 0; sub < ROUNDS; ++sub) {
            const int col0 = wg * (D / 2) + sub * 32;   // this thread's columns col0 .. col0 + 32
            uint4 cen[PIECES];
#pragma unroll
            for (int i = 0; i < PIECES; ++i) cen[i] = cen_all[sub][i];
            // rotation entry of pair i of this thread's 16: fetched per block of four pairs, right where
            // it is used (all sixteen held across the accumulator wait cost more in registers than the
            // table's latency does: the table sits in the cache)
            auto rotation_of = [&](int i) {
              const int local = col0 / 2 + i;   // pair of the head row
              const int pg = p.rope.pair_index ? __ldg(p.rope.pair_index + head * (D / 2) + local) : local;
              const int coord = pg < band_a ? coord_t : (pg < band_b ? coord_h : coord_w);
              return __ldg(reinterpret_cast<const float2*>(p.rope.cos_sin) +
                           static_cast<size_t>(coord) * p.rope.table_half + pg);
            };
            float bias[32];
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias_head + col0 + j));
              bias[j] = b4.x; bias[j + 1] = b4.y; bias[j + 2] = b4.z; bias[j + 3] = b4.w;
            }
            if (!waited) {
              ok = mwait_all(&bars[PAIR_DONE + (job.last_pair & (NDONE - 1))], (job.last_pair / NDONE) & 1, ctx, 503);
              waited = true;
              tc_fence_after();
              laps.lap(2);
            }
            // the accumulator read stays in flight under the centre staging
            uint32_t acc_raw[32];
            tmem_ld32_issue(acc + lane_sel + col0, acc_raw);
            {
              uint8_t* stage = smem + L::scratch_off(npairs) + warp * (32 * PIECES * 16);
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
            tmem_ld32_wait(acc_raw);
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc_raw[i]);
            uint32_t packed[16];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const uint32_t cwords[4] = {cen[j4].x, cen[j4].y, cen[j4].z, cen[j4].w};
              float block[8];   // the 8-wide block j4 of this thread's columns (camera transform only)
              float2 rot[4];
              if (ROPE) {
#pragma unroll
                for (int w = 0; w < 4; ++w) rot[w] = rotate ? rotation_of(j4 * 4 + w) : make_float2(1.f, 0.f);
              }
              if (!ROPE && !CAM) {
                // plain rebuild in packed bf16 arithmetic: bf16x2(acc + bias) then one bf16x2 add of the
                // centre word -- the same two roundings (the sum of two bf16 numbers is exact in fp32
                // unless the smaller one lies below the rounding step of the larger either way)
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                  const int j = j4 * 8 + w * 2;
                  const uint32_t first = pack_bf16x2(v[j] + bias[j], v[j + 1] + bias[j + 1]);
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
                const uint32_t first = pack_bf16x2(v[j] + bias[j], v[j + 1] + bias[j + 1]);
                const __nv_bfloat162 sum = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&first),
                                                   *reinterpret_cast<const __nv_bfloat162*>(&cwords[w]));
                const uint32_t rebuilt = *reinterpret_cast<const uint32_t*>(&sum);
                float x0 = __uint_as_float(rebuilt << 16), x1 = __uint_as_float(rebuilt & 0xFFFF0000u);
                if (rotate) {   // the pair (x0, x1) of the rebuilt bf16 key is one complex number
                  const float2 cs = rot[w];
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
                const int which = __ldg(cam.cam_index + head * (D / 8) + col0 / 8 + j4) & 3;
                const float4* m = reinterpret_cast<const float4*>(cam_frame + which * 16);
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
            // Into the ring through the warp's staging area, so that a store instruction writes whole
            // 64-byte row pieces (4 lanes per row, 8 rows) instead of 16 bytes of 32 different rows.
            {
              uint8_t* stage = smem + L::scratch_off(npairs) + warp * (32 * PIECES * 16);
#pragma unroll
              for (int j = 0; j < PIECES; ++j)
                *reinterpret_cast<uint4*>(stage + lane * (PIECES * 16) + ((j ^ (lane & (PIECES - 1))) << 4)) =
                    make_uint4(packed[j * 4], packed[j * 4 + 1], packed[j * 4 + 2], packed[j * 4 + 3]);
              __syncwarp();
              const int wrow0 = 32 * (warp & 3);
#pragma unroll
              for (int i = 0; i < PIECES; ++i) {
                const int rloc = i * RPI + lane / PIECES, piece = lane % PIECES;
                const uint4 v4 = *reinterpret_cast<const uint4*>(stage + rloc * (PIECES * 16) +
                                                                 ((piece ^ (rloc & (PIECES - 1))) << 4));
                *reinterpret_cast<uint4*>(slot_rows + static_cast<size_t>(wrow0 + rloc) * D + col0 + piece * 8) = v4;
              }
              __syncwarp();
            }
          }
        }
        if (!ok) return;
        laps.lap(3);
        // the accumulator has been read, the metadata buffer is free
        warp_arrive(&bars[META_FREE + mb], lane);
        tc_fence_before();
        // ---- the metadata warp publishes the tile once every warp has stored its part
        // (the consumers read the tile with TMA; the fence between the two proxies is on their side,
        // behind the acquire that shows them the tile)
        warp_arrive(&bars[OUT_DONE + job.num % NMETA], lane);
        laps.lap(5);
    };
    for (int u = g; u < p.units && ok; u += p.groups) {
      const Unit un = unit_of(p, u);
      for (int t = 0; t < un.nt && ok; ++t, ++seq) {
        if (seq % PH != mine) continue;
        Job job;
        job.head = un.head;
        job.t0 = (un.tile0 + t) * TOK;
        job.valid = min(TOK, p.N - job.t0);
        job.slot = seq % R;
        job.num = jobs++;
        expand(job);
        job.last_pair = gp - 1;
        if (ok && have_prev) epilogue(prev);
        prev = job;
        have_prev = true;
      }
    }
    if (ok && have_prev) epilogue(prev);
    laps.flush();
  }
}

template <int D, bool ROPE, bool CAM>
__global__ void __launch_bounds__(THREADS, 1)
attn_codec_kernel(const __grid_constant__ CUtensorMap map_q,
                  const __grid_constant__ CUtensorMap map_wk,
                  const __grid_constant__ CUtensorMap map_wv,
                  const __grid_constant__ CUtensorMap map_ck,
                  const __grid_constant__ CUtensorMap map_cv,
                  const __grid_constant__ CUtensorMap map_rk,
                  const __grid_constant__ CUtensorMap map_rv, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + M_SLOT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + M_ABORT);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int per_group = p.cons + p.prod;
  const int g = blockIdx.x / per_group, role = blockIdx.x % per_group;

  if (tid == 0) {
    mbar_init(&bars[Q_FULL], 1);
    mbar_init(&bars[Q_FREE], 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[K_FULL + s], 1);
      mbar_init(&bars[K_FREE + s], 1);
      mbar_init(&bars[V_FULL + s], 1);
      mbar_init(&bars[V_FREE + s], 1);
      mbar_init(&bars[S_FULL + s], 1);
      mbar_init(&bars[P_READY + s], QT / 32);
      mbar_init(&bars[PV_DONE + s], 1);
      mbar_init(&bars[O_FREE + s], QT / 32);
    }
    for (int s = 0; s < NMETA; ++s) {
      mbar_init(&bars[META_FULL + s], 1);
      mbar_init(&bars[META_FREE + s], COMPUTE_WARPS);
    }
    for (int s = 0; s < MAX_NW; ++s) mbar_init(&bars[W_FULL + s], 1);     // TMA: decoder rows of a pair landed
    for (int s = 0; s < NDONE; ++s) mbar_init(&bars[PAIR_DONE + s], 1);   // the pair's MMAs are complete
    for (int s = 0; s < NSTAGE; ++s) mbar_init(&bars[LAT_FULL + s], COMPUTE_WARPS);   // latent pair staged in TMEM
    mbar_init(&bars[CODES_FULL], 1);                 // the tile's codes landed
    mbar_init(&bars[CODES_FREE], COMPUTE_WARPS);     // every warp is done with codes and centre staging
    for (int s = 0; s < NMETA; ++s)
      mbar_init(&bars[OUT_DONE + s], COMPUTE_WARPS);   // every warp's part of the tile is in the ring
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 9) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const Ctx ctx{abort_flag, p.flags + F_ABORT, p.wait_budget};

  if (g < p.groups) {
    if (role < p.cons) {
      consumer_role<D>(smem, bars, tmem_base, &map_q, &map_rk, &map_rv, p, ctx, g, role);
    } else {
      const int pidx = role - p.cons;
      const bool value = pidx >= p.prod_k;
      producer_role<D, ROPE, CAM>(smem, bars, tmem_base, value ? &map_wv : &map_wk,
                                  value ? &map_cv : &map_ck, p, ctx, g, pidx);
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

// ---- the bounded waits on their own: nobody ever arrives, the wait must give up --------------------
__global__ void wait_expiry_kernel(int kind, long long budget, int32_t* gabort, int32_t* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const Ctx ctx{&abort_flag, gabort, budget};
  if (threadIdx.x == 0) {
    const bool ok = kind == 0 ? mwait(&bar, 0, ctx, 990) : fwait(gabort + 1, 1, ctx, 991);
    if (!ok && abort_flag) atomicCAS(status, 0, abort_flag);
  }
}

constexpr size_t SMEM_LIMIT = 232448;  // 227 KB per CTA

// ---- per-device state: the tile ring and the flag words live in the library's own device image ------
constexpr size_t FLAG_BYTES = 65536;
constexpr size_t RING_BYTES = 24u << 20;
static __device__ __align__(1024) unsigned char g_ring[FLAG_BYTES + RING_BYTES];

constexpr int MAX_DEVICES = 64;
struct DeviceState {
  unsigned char* base = nullptr;
  int sms = 0;
  cudaEvent_t last = nullptr;
  cudaStream_t last_stream = nullptr;
  bool used = false;
};
std::mutex g_mutex;
DeviceState g_state[MAX_DEVICES];

int device_state(DeviceState** out) {
  int device = 0;
  NKV_CUDA(cudaGetDevice(&device));
  NKV_REQUIRE(device >= 0 && device < MAX_DEVICES, NKV_ERR_UNSUPPORTED,
              "device ordinal %d beyond the %d the fused read tracks", device, MAX_DEVICES);
  DeviceState& s = g_state[device];
  if (s.base == nullptr) {
    void* resolved = nullptr;
    NKV_CUDA(cudaGetSymbolAddress(&resolved, g_ring));
    NKV_REQUIRE(resolved != nullptr, NKV_ERR_CUDA, "tile ring has no device address");
    NKV_CUDA(cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, device));
    int cooperative = 0;
    NKV_CUDA(cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device));
    NKV_REQUIRE(cooperative != 0, NKV_ERR_UNSUPPORTED, "device %d cannot launch cooperative kernels", device);
    NKV_CUDA(cudaEventCreateWithFlags(&s.last, cudaEventDisableTiming));
    s.base = static_cast<unsigned char*>(resolved);
  }
  *out = &s;
  return NKV_OK;
}

#ifdef NKV_DEV
long long* g_profile = nullptr;
#endif

int tuning(const char* name, int fallback) {
#ifdef NKV_DEV
  const char* env = getenv(name);
  if (env && env[0]) return atoi(env);
#else
  (void)name;
#endif
  return fallback;
}

template <int D, bool ROPE, bool CAM>
int launch(const CUtensorMap maps[7], Params& p, DeviceState& dev, cudaStream_t stream) {
  using L = Layout<D>;
  int nw = MAX_NW;   // as many decoder-row slots as fit
  while (nw > 2 && static_cast<size_t>(L::producer_bytes(p.npairs, nw, p.ngroups)) + 1024 > SMEM_LIMIT) --nw;
  if (nw > p.npairs) nw = p.npairs;
  if (nw < 2 && p.npairs >= 2) nw = 2;
  size_t smem = static_cast<size_t>(L::producer_bytes(p.npairs, nw, p.ngroups));
  if (smem < static_cast<size_t>(L::CONSUMER_BYTES)) smem = L::CONSUMER_BYTES;
  smem += 1024;
  NKV_REQUIRE(smem <= SMEM_LIMIT, NKV_ERR_UNSUPPORTED,
              "codec attention needs %zu bytes of shared memory (rank %d, rank/group %d)", smem,
              p.rank, p.ngroups);
  p.nw = nw;
  auto kernel = attn_codec_kernel<D, ROPE, CAM>;
  NKV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem)));
  // the flag words start every launch at zero
  NKV_CUDA(cudaMemsetAsync(p.flags, 0, static_cast<size_t>(F_GROUPS + p.groups * GF) * 4, stream));
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(p.groups * (p.cons + p.prod));
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeCooperative;   // producers and consumers wait on one another: all CTAs resident
  attr.val.cooperative = 1;
  config.attrs = &attr;
  config.numAttrs = 1;
  NKV_CUDA(cudaLaunchKernelEx(&config, kernel, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5],
                              maps[6], p));
  (void)dev;
  return NKV_OK;
}

int launch_for(int dk, bool rope, bool cam, const CUtensorMap maps[7], Params& p, DeviceState& dev,
               cudaStream_t stream) {
  if (cam)   // camera builds always carry the rotation code (a NULL table switches it off at run time)
    return dk == 128 ? launch<128, true, true>(maps, p, dev, stream)
                     : launch<64, true, true>(maps, p, dev, stream);
  if (dk == 128)
    return rope ? launch<128, true, false>(maps, p, dev, stream)
                : launch<128, false, false>(maps, p, dev, stream);
  return rope ? launch<64, true, false>(maps, p, dev, stream)
              : launch<64, false, false>(maps, p, dev, stream);
}

// Work decomposition of one launch: consumers and producers per group, groups, history splits.
struct Plan { int cons, prod, prod_k, groups, qchunks, splits, tiles_per_split, ring; };

Plan make_plan(int sms, int Q, int heads, int tiles, int rank, int dk, int max_splits) {
  Plan plan{};
  // a producer needs roughly rank-proportional time per tile; one pair of producers (K, V) per
  // tensor keeps up with the consumers at small ranks, two pairs at the codec's ranks.
  int prod_k = rank >= 256 ? 2 : 1, prod_v = prod_k;
  const int qblocks_all = ceil_div(Q, NQ * QT);
  {
    // Producers beyond that are free as long as the SMs still hold the same number of groups: at the
    // codec's ranks the producers set the pace, so the spare SMs of a group's row go to them, K first
    // (a rotated K tile costs its producer nearly twice a V tile).
    const int cons_all = qblocks_all < sms - 2 ? qblocks_all : sms - 2;
    const int groups_now = sms / (cons_all + prod_k + prod_v);
    while (rank >= 256 && groups_now > 0 && prod_k + prod_v < MAX_PROD &&
           sms / (cons_all + prod_k + prod_v + 1) == groups_now) {
      if (prod_k <= prod_v) ++prod_k; else ++prod_v;
    }
  }
  prod_k = tuning("NKV_ATTN_PROD_K", prod_k);
  prod_v = tuning("NKV_ATTN_PROD_V", prod_v);
  if (prod_k < 1) prod_k = 1;
  if (prod_v < 1) prod_v = 1;
  while (prod_k + prod_v > MAX_PROD) { if (prod_k > prod_v) --prod_k; else --prod_v; }
  const int prod = prod_k + prod_v, prod_max = prod_k > prod_v ? prod_k : prod_v;
  const int qblocks = ceil_div(Q, NQ * QT);
  int cons = qblocks < sms - prod ? qblocks : sms - prod;
  const int qchunks = ceil_div(qblocks, cons);
  cons = ceil_div(qblocks, qchunks);
  const int ring_slots = static_cast<int>(RING_BYTES / (2u * TOK * dk * 2u));
  // A producer prepares its jobs up to NMETA ahead and checks the ring slot of a job at that
  // point, with up to NMETA - 1 of its own earlier tiles not yet published; the slot's previous
  // tile must be older than those, which takes more than (NMETA - 1) * (producers of a kind) slots.
  const int min_ring = (NMETA - 1) * prod_max + 1 > 4 ? (NMETA - 1) * prod_max + 1 : 4;
  int wmax = sms / (cons + prod);
  if (wmax > ring_slots / min_ring) wmax = ring_slots / min_ring;
  if (wmax < 1) wmax = 1;
  const int forced = tuning("NKV_ATTN_SPLITS", 0);
  long long best_cost = -1;
  for (int s = 1; s <= max_splits; ++s) {
    if (forced > 0 && s != forced && forced <= max_splits) continue;
    const int tps = ceil_div(tiles, s);
    const int eff = ceil_div(tiles, tps);
    if (eff != s && forced == 0) continue;
    const int units = qchunks * heads * eff;
    const int groups = units < wmax ? units : wmax;
    const int rounds = ceil_div(units, groups);
    // a unit costs its tiles plus a fill / drain of a few tile times; split partials cost a merge
    const long long cost = static_cast<long long>(rounds) * (tps + 6) + (eff > 1 ? 4 + eff : 0);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      plan.splits = eff;
      plan.tiles_per_split = tps;
      plan.groups = groups;
    }
  }
  plan.cons = cons;
  plan.prod = prod;
  plan.prod_k = prod_k;
  plan.qchunks = qchunks;
  int ring = ring_slots / plan.groups;
  plan.ring = ring > MAX_RING ? MAX_RING : ring;
  plan.ring = tuning("NKV_ATTN_RING", plan.ring);
  if (plan.ring > ring) plan.ring = ring;
  if (plan.ring < min_ring) plan.ring = min_ring;
  return plan;
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

#ifdef NKV_DEV
extern "C" void nkv_dev_attn_profile(void* device_buckets) { g_profile = static_cast<long long*>(device_buckets); }
#endif

bool tc_attn_supported(int dk, int dv, int rank) {
  return dk == dv && (dk == 64 || dk == 128) && rank % 64 == 0 && rank > 0;
}

// kind 0: an mbarrier nobody arrives on; kind 1: a global counter nobody advances.  The kernel's
// single waiting thread must give up after `budget_cycles` and report the wait site (990 / 991).
int tc_wait_expiry_selftest(int kind, long long budget_cycles, int32_t* status_word, cudaStream_t stream) {
  NKV_REQUIRE((kind == 0 || kind == 1) && budget_cycles > 0 && budget_cycles <= (1ll << 28) && status_word,
              NKV_ERR_INVALID, "wait self-test: kind=%d budget=%lld", kind, budget_cycles);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* dev = nullptr;
  int rc = device_state(&dev);
  if (rc != NKV_OK) return rc;
  // two private flag words behind the ones the fused read uses
  int32_t* words = reinterpret_cast<int32_t*>(dev->base + FLAG_BYTES - 64);
  NKV_CUDA(cudaMemsetAsync(words, 0, 8, stream));
  wait_expiry_kernel<<<1, 32, 0, stream>>>(kind, budget_cycles, words, status_word);
  NKV_LAUNCH_CHECK("wait_expiry_kernel");
  return NKV_OK;
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
  NKV_REQUIRE(((reinterpret_cast<uintptr_t>(bias_k) | reinterpret_cast<uintptr_t>(bias_v)) & 15) == 0,
              NKV_ERR_INVALID, "bias arrays must be 16-byte aligned");
  if (Q == 0 || heads == 0) return NKV_OK;
  if (N == 0) {
    size_t rows = static_cast<size_t>(Q) * heads;
    fill_empty_kernel<<<static_cast<unsigned>((rows * dv + 255) / 256), 256, 0, stream>>>(
        static_cast<uint16_t*>(out), lse, rows, dv);
    NKV_LAUNCH_CHECK("fill_empty_kernel");
    return NKV_OK;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* dev = nullptr;
  {
    int rc = device_state(&dev);
    if (rc != NKV_OK) return rc;
  }
  const int tiles = ceil_div(N, TOK);
  splits = splits < 1 ? 1 : (splits > tiles ? tiles : splits);
  if (workspace == nullptr) splits = 1;
  const Plan plan = make_plan(dev->sms, Q, heads, tiles, rank, dk, splits);

  CUtensorMap maps[7];
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
    uint32_t box[2] = {64, static_cast<uint32_t>(dk)};   // a producer streams all rows of the head's slice
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
  const size_t ring_rows = static_cast<size_t>(plan.groups) * plan.ring * TOK;
  p.flags = reinterpret_cast<int32_t*>(dev->base);
  p.ring_k = reinterpret_cast<uint16_t*>(dev->base + FLAG_BYTES);
  p.ring_v = p.ring_k + ring_rows * dk;
  const void* rings[2] = {p.ring_k, p.ring_v};
  for (int w = 0; w < 2; ++w) {   // a consumer loads a slot as [128 tok x 64 col] boxes
    uint64_t dims[2] = {static_cast<uint64_t>(dk), static_cast<uint64_t>(ring_rows)};
    uint64_t strides[1] = {static_cast<uint64_t>(dk) * 2};
    uint32_t box[2] = {64, TOK};
    int rc = encode_tensor_map(&maps[5 + w], 2, rings[w], 2, dims, strides, box, 128);
    if (rc != NKV_OK) return rc;
  }
  p.Q = Q; p.heads = heads; p.N = N; p.rank = rank; p.nchunks = rank / CHUNK;
  p.npairs = (p.nchunks + 1) / 2;
  p.group = group; p.ngroups = rank / group; p.scale_dtype = hk.scale_dtype;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.hk = hk; p.hv = hv; p.bias_k = bias_k; p.bias_v = bias_v;
  p.status = status_word;
  p.w_perm = prepared_weights ? 1 : 0;
  if (rope != nullptr) p.rope = *rope;
  if (cam_k != nullptr) p.cam_k = *cam_k;
  if (cam_v != nullptr) p.cam_v = *cam_v;
  p.tiles = tiles;
  p.tiles_per_split = plan.tiles_per_split;
  p.splits = plan.splits;
  p.qchunks = plan.qchunks;
  p.groups = plan.groups; p.cons = plan.cons; p.prod = plan.prod; p.prod_k = plan.prod_k; p.ring = plan.ring;
  p.units = plan.qchunks * heads * plan.splits;
  p.wait_budget = 1ll << 31;   // about a second of SM cycles per wait
#ifdef NKV_DEV
  p.prof = g_profile;
#endif
  // launches of the fused read share the ring: one that is enqueued on another stream than the
  // previous one waits for it
  if (dev->used && dev->last_stream != stream) NKV_CUDA(cudaStreamWaitEvent(stream, dev->last, 0));
  const bool rope_on = rope != nullptr, cam_on = cam_k != nullptr || cam_v != nullptr;
  int rc;
  if (plan.splits == 1) {
    p.out = static_cast<uint16_t*>(out); p.lse = lse;
    rc = launch_for(dk, rope_on, cam_on, maps, p, *dev, stream);
  } else {
    // History splits: each unit attends a contiguous run of tiles and writes a partial (O, lse) in
    // the output dtype; the partials are merged by log-sum-exp.
    const size_t rows = static_cast<size_t>(Q) * heads;
    uint16_t* part_out = static_cast<uint16_t*>(workspace);
    float* part_lse = reinterpret_cast<float*>(part_out + static_cast<size_t>(plan.splits) * rows * dv);
    p.out = part_out; p.lse = part_lse;
    rc = launch_for(dk, rope_on, cam_on, maps, p, *dev, stream);
    if (rc == NKV_OK) {
      const void* outs[16];
      const float* lses[16];
      for (int z = 0; z < plan.splits; ++z) {
        outs[z] = part_out + static_cast<size_t>(z) * rows * dv;
        lses[z] = part_lse + static_cast<size_t>(z) * rows;
      }
      rc = lse_merge(outs, lses, plan.splits, static_cast<int64_t>(rows), dv, NKV_BF16, out, lse, stream);
    }
  }
  if (rc != NKV_OK) return rc;
  NKV_CUDA(cudaEventRecord(dev->last, stream));
  dev->last_stream = stream;
  dev->used = true;
  return NKV_OK;
}

}  // namespace nkv
