// Ragged flash-decode attention for int8 caches, head_dim 128 and up to 8
// grouped query rows on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// The int8 codes never pass through registers: both contractions run as
// integer MMAs that read K, V and the small second operands straight from
// shared memory and accumulate int32 in tensor memory (TMEM).
//
//   S^T[128 tok x 16] = K[128 tok x 128 d] . Ql^T       kind::i8, K-major A and B
//   O^T[128 d  x 16] = V^T[128 d x 128 tok] . Pl^T      kind::i8, MN-major A, K-major B
//
// "Levels" make the small operands 8-bit without losing the precision of the
// bf16 / fp32 values they stand for:
//   * a query row q (bf16) is split as q = s (h + l / 254) with s = amax|q| / 127
//     and h, l signed bytes; rows 0..7 of Ql hold h, rows 8..15 hold l, so the
//     two partial dot products of a token arrive in the same TMEM lane and
//     S = s (S_h + S_l / 254) is exact to 2^-16 of the row's amax;
//   * a probability p in [0, 1] (the running maximum is exact here), times the
//     token's V scale relative to the largest V scale of the tile, becomes a
//     16-bit fixed-point number whose two bytes are the unsigned levels
//     Pl[8 l + r]; O = (O_0 + 2^8 O_1) c / (2^16 - 1): an error of 2^-17 of the
//     tile's largest term per token, far below the bf16 rounding of the result.
// Every int32 sum is exact (|sum| <= 128 * 127 * 255), so the only roundings
// are the two splits above and the fp32 online-softmax arithmetic.
//
// A tile is 128 consecutive valid tokens of one (sequence, KV head) segment;
// tiles are scheduled as in the mma.sync kernel (contiguous shares of one
// global tile list, pieces, last-arriver merge).  K and V rows of a tile land
// in shared memory as 128-byte rows, 16-byte chunks XORed with (row & 7): that
// is the canonical 128-byte-swizzle layout of the tensor core for both operand
// roles (K-major for K, MN-major for V), so nothing is rearranged.  K and V
// have rings of two slots each; where a tensor map describes the cache the
// rows are moved by the copy engine (cp.async.bulk.tensor, one request per
// tile and tensor, one and a half to two tiles ahead, completion counted on an
// mbarrier per slot that only the MMA-issuing threads wait for), else by
// 16-byte cp.async of all threads.  In the softmax phase thread t owns token t
// of the tile (TMEM lane t of S^T); in the output phase thread t owns head-dim
// index t (TMEM lane t of O^T), which also removes the cross-warp merge of the
// accumulators.  The softmax phase is compiled for 8, 4 or 2 query rows.
//
// Fused decode update (jpt_decode_update_attend): the launch also takes the
// step's new K/V token, which becomes the last token of its segment: the
// schedule counts one token more per sequence, and the CTA that processes the
// segment's last tile writes the token's int8 codes into the row behind the
// existing tokens of that tile IN SHARED MEMORY (K tile before the S^T MMA, V
// tile before the O^T MMA), so the token is attended to like any other, with
// no separate softmax term.  CTA b mod grid computes the token's amax over
// this GPU's heads while its first rows are in flight and stores it into the
// exchange slots of every rank (NVLink peer stores when the KV heads are
// sharded); the CTA with the last tile reads the ranks' words (long there by
// then), quantises the token's row of its head with the decode quantiser and
// also writes cache row, scale and stash.  One launch per layer, the
// exchange's round trip hidden under the existing tokens.
//
// Every wait (mbarriers, exchange words) is bounded; a CTA that gives up raises
// the status word of the workspace, frees its tensor memory and returns.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <type_traits>
#include <vector>

#include "attention_tiles.cuh"

namespace jpt {
namespace {

constexpr int kTileU = 128;     // tokens per tile = TMEM lanes = threads per CTA
constexpr int kTmemCols = 32;   // S^T: columns 0..15, O^T: columns 16..31
constexpr int kColO = 16;
constexpr int kCtasPerSm = 3;
#ifndef JPT_PIECE_COST_U
#define JPT_PIECE_COST_U 2
#endif
#ifndef JPT_PIECE_COST_FUSED
#define JPT_PIECE_COST_FUSED 2
#endif
constexpr int kPieceCostU = JPT_PIECE_COST_U;  // overhead slots charged per segment, in 128-token tiles
constexpr long long kWaitCycles = 1000000000ll;  // about half a second: far beyond any wait of a healthy run

struct __align__(1024) SmemU {
  uint8_t k[2][kTileU * kD];             // K ring: [slot][token][128 bytes], swizzled
  uint8_t v[2][kTileU * kD];             // V ring
  uint8_t qlev[16 * kD];                 // query levels: rows 0..7 high bytes, 8..15 low bytes
  uint8_t plev[16 * kTileU];             // probability levels: row 8 l + r, one byte per token
  uint8_t qraw[8 * kD * 2];              // bf16 query rows of the piece that starts with the next tile
  uint8_t ntkv[2][2][kD * 4];            // new token, by tile parity: its K and V rows of this head (bf16 or fp32)
  uint8_t ntv[2][kD];                    // ... and its V codes between the K tile's turn and the V tile's
  float ntsc[2][2];                      // ... and its K and V scales
  unsigned long long ntw[2][2][8];       // ... the ranks' amax words (K, V) as they were when the tile was requested
  int ntpos[2][4];                       // ... and where the token is written
  float xch[4][12];                      // per warp: row maxima of the tile [8], largest V scale [1]
  float red[4][8];                       // per warp: denominators at the end of a piece
  float qsc[8];                          // s_r * sm_scale * log2(e) / 254
  float qsr[8];                          // s_r / 254 (the chain of rounded logits starts from the plain dot product)
  float ntx[4];                          // new token: K amax, V amax
  uint64_t bar[2];                       // MMA completion: S^T, O^T
  uint64_t bar_k[2], bar_v[2];           // rows landed (copy-engine path), per ring slot
  uint32_t tmem_base;
  int start[3];
  int flag;
  TileMeta meta[4];                      // records of the tiles in flight (by tile number mod 4)
};

// 16-byte copy with compile-time offsets on both addresses (one pair of base registers per tensor)
template <int kOff>
__device__ __forceinline__ void cp_async16_at(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0 + %2], [%1 + %2], 16;\n" ::"r"(dst), "l"(src), "n"(kOff));
}
template <int kI>
__device__ __forceinline__ void cp_async_tile_rows(uint32_t dst, const void* src) {
  if constexpr (kI < 8) {  // 8 passes of 16 rows
    cp_async16_at<2048 * kI>(dst, src);
    cp_async_tile_rows<kI + 1>(dst, src);
  }
}
// The two bytes of y into level rows r, 8 + r (kRowOff = 128 r) of the probability levels.
template <int kRowOff>
__device__ __forceinline__ void store_levels(uint32_t addr, uint32_t y) {
  asm volatile("st.shared.u8 [%0 + %2], %1;" ::"r"(addr), "r"(y), "n"(kRowOff) : "memory");
  asm volatile("st.shared.u8 [%0 + %2], %1;" ::"r"(addr), "r"(y >> 8), "n"(kRowOff + 1024) : "memory");
}
constexpr float kNoMax = -1.0e30f;  // "no logit seen yet": finite, far below any logit
__device__ __forceinline__ float ex2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(r) : "f"(x));
  return r;
}
// Rows kRow .. 7 of the thread's token: new running maximum, rescale factor,
// probability, denominator share, and the probability's two level bytes.
// m_run starts at kNoMax (finite), so exp2(old - new) and exp2(-inf - new) need
// no special case.
template <int kRow, int kR>
__device__ __forceinline__ void softmax_rows(float (&m_run)[8], float (&l_run)[8], float (&alpha)[8], const float (&tm)[8],
                                             const float (&xv)[8], float ps, uint32_t p_base) {
  if constexpr (kRow < kR) {
    const float mn = fmaxf(m_run[kRow], tm[kRow]);
    const float al = ex2(m_run[kRow] - mn);
    const float p = ex2(xv[kRow] - mn);
    alpha[kRow] = al;
    m_run[kRow] = mn;
    l_run[kRow] = fmaf(l_run[kRow], al, p);
    // the byte of row r: 16-byte chunk (t / 16) ^ r of that row (the XOR folds into the address)
    store_levels<128 * kRow>(p_base ^ (uint32_t)(kRow << 4), __float2uint_rn(p * ps));
    softmax_rows<kRow + 1, kR>(m_run, l_run, alpha, tm, xv, ps, p_base);
  }
}
// A segment's valid tokens form one run of consecutive rows, or two when the
// ring wraps: [first, first + nA) and [0, n - nA).  Tiles never straddle the
// wrap: run A is cut into tiles of 128 rows (the last one partial), then run B,
// so a tile is always one range of rows (one box for the copy engine).
__device__ __forceinline__ int run_a(const SeqRange& r, int S) { return min(r.n, S - r.first); }
__device__ __forceinline__ int tiles_run(int n) { return (n + kTileU - 1) / kTileU; }
__device__ __forceinline__ int tiles_u(const SeqRange& r, int S) {
  const int na = run_a(r, S);
  return tiles_run(na) + tiles_run(r.n - na);
}
__device__ __forceinline__ int slots_u(const SeqRange& r, int S, int cost) { return r.n > 0 ? tiles_u(r, S) + cost : 0; }
// Tile t of the segment: physical position of its first row and its number of valid rows.
__device__ __forceinline__ void tile_rows(const SeqRange& r, int S, int t, int* pos, int* cnt) {
  const int na = run_a(r, S), ta = tiles_run(na);
  if (t < ta) {
    *pos = r.first + t * kTileU;
    *cnt = min(kTileU, na - t * kTileU);
  } else {
    *pos = (t - ta) * kTileU;
    *cnt = min(kTileU, r.n - na - (t - ta) * kTileU);
  }
}

// Byte offset of (row, byte) in a tile of 128-byte rows with 128-byte swizzle.
__device__ __forceinline__ uint32_t swz(int row, int byte) {
  return (uint32_t)(row * 128 + ((((byte >> 4) ^ (row & 7))) << 4) + (byte & 15));
}

// Shared-memory matrix descriptor: 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);  // start address
  d |= (uint64_t)(1024 >> 4) << 16;       // leading byte offset (one swizzle atom; unused for these shapes)
  d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                 // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
  return d;
}
// Instruction descriptors: int32 accumulators, M = 128.
constexpr uint32_t kIdescS = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);  // s8 x s8, N = 16
constexpr uint32_t kIdescO =
    (2u << 4) | (1u << 7) | (0u << 10) | (1u << 15) | ((16u >> 3) << 17) | ((128u >> 4) << 24);  // s8 (MN-major) x u8, N = 16

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Bounded wait for the phase with the given parity; false when it gave up.
__device__ __forceinline__ bool mbar_probe(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 16; ++i) {
      uint32_t ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}\n"
          : "=r"(ok)
          : "r"(bar), "r"(parity)
          : "memory");
      if (ok) return true;
    }
    if (clock64() - t0 > kWaitCycles) return false;
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  return mbar_probe(bar, parity) || mbar_wait_slow(bar, parity);
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One box of a 4-d tensor map (128 bytes x rows x 1 x 1) into swizzled shared memory of this CTA.
__device__ __forceinline__ void tma_load_rows(uint32_t dst, const CUtensorMap* map, int row, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(row), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
// Tensor maps of the K and V tensors: dense [B, Hkv, S, 128 bytes] with the caller's strides
// (box: the 128 rows of a tile), or the page pool [Hkv, pages, page_size, 128 bytes] (box: a
// page, or 128 rows of a larger one).
struct TmaMaps {
  CUtensorMap k, v;
};
constexpr int kTmaNone = 0, kTmaDense = 1, kTmaPaged = 2;

// maximum over the 32 lanes in one instruction
__device__ __forceinline__ float warp_max(float x) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(x));
  return r;
}

#ifdef JPT_UMMA_SPANS
// Debug builds only: per CTA, nanosecond stamps of the phases of its life.
__device__ unsigned long long g_umma_spans[1024 * 8];
__device__ __forceinline__ unsigned long long gtimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define JPT_SPAN(k)                                                                    \
  do {                                                                                 \
    if (threadIdx.x == 0 && blockIdx.x < 1024) g_umma_spans[8 * blockIdx.x + (k)] = gtimer_ns(); \
  } while (0)
#else
#define JPT_SPAN(k) do {} while (0)
#endif


// kFused = the launch carries the decode step's new token, kRound = dense_attention's rounded
// logit chain, kTma = the copy engine moves the K/V rows (tensor maps) instead of the threads, kR = query
// rows the softmax phase works on (8; 4 for groups of up to four query heads; 2 for multi-head attention
// with its single row per KV head; the level rows of the others hold zeros, their results are never
// looked at).
template <bool kFused, bool kRound, bool kTma, int kR>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
    flash_decode_i8_umma_kernel(const __grid_constant__ AttnArgs a, const __grid_constant__ MmaScratch x, int* status,
                                const __grid_constant__ NewTokenArgs nt, const __grid_constant__ TmaMaps maps, int tma_mode,
                                int box_rows) {
  // The swizzled tiles need a 1024-byte aligned base.  The array is declared
  // with that alignment (and used in place, so that every access compiles to a
  // shared-memory instruction); a base that is not aligned after all is reported.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  SmemU& sm = *reinterpret_cast<SmemU*>(smem_raw);
  if ((smem_u32(smem_raw) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicExch(status, 2);
    return;
  }

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // slots charged per segment on top of its tiles (with the new token: one more for its quantisation)
  constexpr int kPieceCost = kFused ? JPT_PIECE_COST_FUSED : kPieceCostU;
  const int R = a.R;
  const bool quant = a.k_scale != nullptr;
  const int cta = blockIdx.x;
#ifdef JPT_UMMA_SPANS
  if (threadIdx.x == 0 && blockIdx.x < 1024)
    for (int z = 0; z < 8; ++z) g_umma_spans[8 * blockIdx.x + z] = 0;
#endif
  JPT_SPAN(2);  // entry

  // ------------------------------------------------------------------ barriers and tensor memory
  // (warp 1; warp 0 is busy with the scan below, the barriers of the schedule publish the result)
  if (tid == 32) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sm.bar[0])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sm.bar[1])));
    if constexpr (kTma) {
      for (int z = 0; z < 2; ++z) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sm.bar_k[z])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sm.bar_v[z])));
      }
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.k)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.v)) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  // Up to here nothing of global memory was touched: with a programmatic launch all of
  // it ran under the kernel before this one (the append of the new token).
  grid_dependency_wait();
  grid_dependency_trigger();
  JPT_SPAN(0);  // the kernel before this one is complete

  // ------------------------------------------------------------------ new token: amax to every rank
  unsigned nt_epoch = 0;
  if constexpr (kFused) nt_epoch = *reinterpret_cast<volatile unsigned*>(&nt.px_state[0]) + 1u;
  // Called once by every CTA, after its first rows have been requested (the reduction runs under their latency).
  auto post_amax = [&]() {
    const int HD = a.Hkv * kD;
    for (int b = cta; b < a.B; b += gridDim.x) {
      float am[2];
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        // 16 bytes per load, the loads of a pass in flight together (rows are kD elements: 16-byte multiples)
        const int chunks = HD * (nt.in_f32 ? 4 : 2) / 16;
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(nt.x[which]) +
                                                          (int64_t)b * HD * (nt.in_f32 ? 4 : 2));
        float v = 0.f;
        for (int c0 = 0; c0 < chunks; c0 += 4 * kThreads) {
          uint4 u[4];
#pragma unroll
          for (int z = 0; z < 4; ++z) {
            const int c = c0 + z * kThreads + tid;
            u[z] = c < chunks ? src[c] : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int z = 0; z < 4; ++z) {
            const uint32_t w[4] = {u[z].x, u[z].y, u[z].z, u[z].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (nt.in_f32) {
                v = fmaxf(v, fabsf(__uint_as_float(w[e])));
              } else {  // two bf16 values: their magnitudes as floats
                v = fmaxf(v, fmaxf(fabsf(__uint_as_float(w[e] << 16)), fabsf(__uint_as_float(w[e] & 0xffff0000u))));
              }
            }
          }
        }
        am[which] = warp_max(v);
      }
      __syncthreads();  // the scratch may still be read for the slot before
      if (lane == 0) {
        sm.xch[warp][0] = am[0];
        sm.xch[warp][1] = am[1];
      }
      __syncthreads();
      if (tid < 2) {
        const float m4 = fmaxf(fmaxf(sm.xch[0][tid], sm.xch[1][tid]), fmaxf(sm.xch[2][tid], sm.xch[3][tid]));
        const size_t row = (size_t)(nt_epoch & 1u) * nt.px_world + nt.px_rank;
        const unsigned long long word = ((unsigned long long)nt_epoch << 32) | __float_as_uint(m4);
        for (int r = 0; r < nt.px_world; ++r)
          asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(nt.px_slots[r] + row * (2 * a.B) + tid * a.B + b), "l"(word)
                       : "memory");
      }
    }
    __syncthreads();
  };
  // Counts this CTA as done with the exchange of this launch; the last one advances the launch number.
  auto exchange_done = [&]() {
    if constexpr (kFused) {
      if (tid == 0) {
        __threadfence();
        const unsigned done = atomicAdd(&nt.px_state[1], 1u);
        if (done == gridDim.x - 1) {
          nt.px_state[1] = 0;
          __threadfence();
          atomicAdd(&nt.px_state[0], 1u);
        }
      }
    }
  };

  // Valid range of sequence b as the schedule sees it: with the fused update the step's new token
  // counts as the segment's last token (a full cache has no row for it: reported, the token is dropped).
  auto seg_range = [&](int b, int* use_add, bool* extended = nullptr) {
    SeqRange r = seq_range_x(a, x, b, use_add);
    if constexpr (kFused) {
      const bool room = r.n < a.S;
      if (room) {
        r.n += 1;
      } else {
        atomicExch(status, 3);
      }
      if (extended) *extended = room;
    }
    return r;
  };

  // ------------------------------------------------------------------ schedule
  // Slots per sequence (tiles + overhead) -> exclusive prefix over sequences;
  // each thread owns a slice of ceil(B/128) sequences.  The scan scratch
  // aliases the probability levels, which are not in use yet.
  int* scan = reinterpret_cast<int*>(&sm.plev[0]);  // 129 ints
  const int per = (a.B + kThreads - 1) / kThreads;
  const int b_lo = min(a.B, tid * per), b_hi = min(a.B, b_lo + per);
  int mine = 0;
  for (int b = b_lo; b < b_hi; ++b) {
    int ua;
    mine += slots_u(seg_range(b, &ua), a.S, kPieceCost);
  }
  scan[tid] = mine;
  __syncthreads();
  if (warp == 0) {
    int v4[4], s = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v4[i] = scan[4 * lane + i];
      s += v4[i];
    }
    int incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    int run = incl - s;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      scan[4 * lane + i] = run;
      run += v4[i];
    }
    if (lane == 31) scan[kThreads] = incl;
  }
  __syncthreads();
  const int total = scan[kThreads] * a.Hkv;  // the host checked that this fits in 31 bits
  // CTA c takes slots [G0, G1): the first `rem` CTAs one slot more than the others
  const int share_lo = total / x.num_ctas, rem = total - share_lo * x.num_ctas;
  const int G0 = cta * share_lo + min(cta, rem);
  const int G1 = G0 + share_lo + (cta < rem ? 1 : 0);
  auto cta_of_slot = [&](int slot) {
    const int big = rem * (share_lo + 1);
    return slot < big ? slot / (share_lo + 1) : rem + (slot - big) / max(share_lo, 1);
  };
  {
    // the thread whose slice holds slot G0 walks it and publishes (b, h, slot in segment)
    const int lo = scan[tid] * a.Hkv, hi = scan[tid + 1] * a.Hkv;
    if (G0 < G1 && G0 >= lo && G0 < hi) {
      int run = lo;
      for (int b = b_lo; b < b_hi; ++b) {
        int ua;
        const int sl = slots_u(seg_range(b, &ua), a.S, kPieceCost);
        const int nxt = run + sl * a.Hkv;
        if (G0 < nxt) {
          const int rem = G0 - run;
          sm.start[0] = b;
          sm.start[1] = rem / sl;
          sm.start[2] = rem % sl;
          break;
        }
        run = nxt;
      }
    }
  }
  __syncthreads();  // sm.start and the tensor-memory address visible; last reads of `scan` done
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  JPT_SPAN(1);

  const __nv_bfloat16* qbase = static_cast<const __nv_bfloat16*>(a.q);
  // The new token of segment (b, h), whose last tile has number `seq` in this CTA: the copies of its K and V
  // rows start when the tile's K rows are requested (two iterations before they are needed) ...
  const int nt_row_bytes = nt.in_f32 ? kD * 4 : kD * 2;
  auto stage_new_token = [&](int seq, int b, int h) {
    const int64_t row = ((int64_t)b * a.Hkv + h) * nt_row_bytes;
    const int chunks = nt_row_bytes / 16;
    if (tid < 2 * chunks) {
      const int which = tid / chunks, ch = tid - which * chunks;
      cp_async16(smem_u32(&sm.ntkv[seq & 1][which][0]) + ch * 16, static_cast<const uint8_t*>(nt.x[which]) + row + ch * 16, true);
    }
    // the exchange words of this sequence (normally posted long ago; looked at again if not) and the position
    if (tid >= 64 && tid < 64 + 2 * nt.px_world) {
      const int which = (tid - 64) / nt.px_world, r = (tid - 64) - which * nt.px_world;
      const unsigned long long* p =
          nt.px_slots[nt.px_rank] + ((size_t)(nt_epoch & 1u) * nt.px_world + r) * (2 * a.B) + which * a.B + b;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(smem_u32(&sm.ntw[seq & 1][which][r])), "l"(p));
    }
    if (tid == 96) {
      if (nt.pos) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(&sm.ntpos[seq & 1][0])),
                     "l"(nt.pos + (nt.pos_count == 1 ? 0 : b)));
      } else {
        sm.ntpos[seq & 1][0] = nt.pos_host;
      }
    }
  };
  // ... and once the tile's K rows are in shared memory, the whole CTA (thread tid: head-dim index tid)
  // turns the token into codes: all-ranks amax -> scales -> codes of this head's row -> the K code into
  // row `row` of the K tile, the V code aside for the V tile's turn, cache row, scales and stash to
  // global memory.  The caller's barrier publishes the shared-memory writes.
  auto quantise_new_token = [&](int seq, int b, int h, int row) {
    if (tid < 2) {  // K amax, V amax: largest partial over the ranks
      const size_t xrow = (size_t)(nt_epoch & 1u) * nt.px_world;
      float m = 0.f;
      const long long t0 = clock64();
      for (int r = 0; r < nt.px_world; ++r) {
        const unsigned long long* p = nt.px_slots[nt.px_rank] + (xrow + r) * (2 * a.B) + tid * a.B + b;
        unsigned long long w = sm.ntw[seq & 1][tid][r];
        while ((unsigned)(w >> 32) != nt_epoch) {
          asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
          if ((unsigned)(w >> 32) == nt_epoch) break;
          if (clock64() - t0 > nt.px_wait_cycles) {  // a rank never came: report, go on with what is there
            atomicExch(&nt.px_state[2], 1u);
            w = 0;
            break;
          }
        }
        m = fmaxf(m, __uint_as_float((unsigned)w));
      }
      sm.ntx[tid] = m;
    }
    __syncthreads();
    const float amax_k = sm.ntx[0], amax_v = sm.ntx[1];
    const float sc_k = nt.in_f32 ? decode_scale<float>(amax_k) : decode_scale<__nv_bfloat16>(amax_k);
    const float sc_v = nt.in_f32 ? decode_scale<float>(amax_v) : decode_scale<__nv_bfloat16>(amax_v);
    const int64_t xi = ((int64_t)b * a.Hkv + h) * kD + tid;
    float xk, xv;
    if (nt.in_f32) {
      xk = reinterpret_cast<const float*>(&sm.ntkv[seq & 1][0][0])[tid];
      xv = reinterpret_cast<const float*>(&sm.ntkv[seq & 1][1][0])[tid];
    } else {
      xk = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(&sm.ntkv[seq & 1][0][0])[tid]);
      xv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(&sm.ntkv[seq & 1][1][0])[tid]);
    }
    const int8_t ck = nt.in_f32 ? decode_code<float>(xk, sc_k) : decode_code<__nv_bfloat16>(xk, sc_k);
    const int8_t cv = nt.in_f32 ? decode_code<float>(xv, sc_v) : decode_code<__nv_bfloat16>(xv, sc_v);
    sm.k[seq & 1][swz(row, tid)] = (uint8_t)ck;
    sm.ntv[seq & 1][tid] = (uint8_t)cv;
    if (tid < 2) sm.ntsc[seq & 1][tid] = tid == 0 ? sc_k : sc_v;
    if (nt.quant[0]) nt.quant[0][xi] = ck;
    if (nt.quant[1]) nt.quant[1][xi] = cv;
    int pos = sm.ntpos[seq & 1][0];
    if (pos < 0) pos += a.S;
    const bool write = nt.write_cache && pos >= 0 && pos < a.S;
    if (write) {
      const int64_t off = (int64_t)b * a.kv_b + (int64_t)h * a.kv_h + (int64_t)pos * a.kv_s + tid;
      static_cast<int8_t*>(const_cast<void*>(a.k))[off] = ck;
      static_cast<int8_t*>(const_cast<void*>(a.v))[off] = cv;
    }
    if (tid < 2) {  // every head's CTA writes the same scale: harmless, and no CTA has to wait for another
      const float sc = tid == 0 ? sc_k : sc_v;
      void* out = nt.scale_out[tid];
      void* cache = const_cast<void*>(tid == 0 ? a.k_scale : a.v_scale);
      const int64_t sidx = (int64_t)b * a.sc_b + (int64_t)pos * a.sc_s;
      if (nt.in_f32) {
        if (out) static_cast<float*>(out)[b] = sc;
        if (write) static_cast<float*>(cache)[sidx] = sc;
      } else {
        if (out) static_cast<__nv_bfloat16*>(out)[b] = __float2bfloat16_rn(sc);
        if (write) static_cast<__nv_bfloat16*>(cache)[sidx] = __float2bfloat16_rn(sc);
      }
    }
  };
  // Rows of empty sequences are nobody's tile: sequence b is cleared by CTA b mod grid (at the end of
  // the CTA's life, off the path to its first tile).  (With the fused update no sequence is empty.)
  auto clear_empty_rows = [&]() {
    for (int b = cta; b < a.B; b += gridDim.x) {
      int ua;
      if (seg_range(b, &ua).n == 0) {
        const int64_t r0 = (int64_t)b * a.Hkv * R;
        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.o);
        for (int i = tid; i < a.Hkv * R * kD; i += kThreads) o[r0 * kD + i] = __float2bfloat16_rn(0.f);
        for (int i = tid; i < a.Hkv * R; i += kThreads) {
          if (a.m) a.m[r0 + i] = -INFINITY;
          if (a.l) a.l[r0 + i] = 0.f;
        }
      }
    }
  };
  if (G0 >= G1) {  // no tile for this CTA
    if constexpr (kFused) post_amax();
    clear_empty_rows();
    exchange_done();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kTmemCols) : "memory");
    }
    return;
  }
  const uint32_t tmem_lane = tmem + ((uint32_t)(warp * 32) << 16);  // this warp's 32 lanes

  const int8_t* kbase = static_cast<const int8_t*>(a.k);
  const int8_t* vbase = static_cast<const int8_t*>(a.v);
  const __nv_bfloat16* mask = static_cast<const __nv_bfloat16*>(a.mask);

  // ------------------------------------------------------------------ producer
  // K and V rows travel in rings of their own (two slots of 16 KB each; tile j uses slot j % 2 of
  // both).  A K slot is free as soon as the S^T MMA of its tile is complete, a V slot when the O^T
  // MMA is: in iteration i the K rows of tile i + 2 and the V rows of tile i + 1 are requested, so
  // every row has one and a half to two iterations to land.
  // Position of the next tile whose K rows are to be fetched (uniform across the CTA) ...
  int pb = sm.start[0], ph = sm.start[1], pt, pslot = G0;  // pslot: global slot index of tile pt
  int pT, pn, pfirst, puse_add;
  bool pext = false;  // the sequence's last token is the step's new one
  // ... and what follows from it for this thread: 16-byte column tid % 8 of
  // rows tid / 8 + 16 i of a tile.  The swizzled shared-memory offset of row
  // + 16 i is that of row plus 2048 i.
  const int prow = tid >> 3, pcol = tid & 7;
  const uint32_t pdst = (uint32_t)(prow * kD + ((pcol ^ (prow & 7)) << 4));
  // pages that hold whole 16-row copy passes: one table entry per pass
  const bool pass_pages = a.paged && (a.page_size % 16) == 0 &&
                          ((kTileU % a.page_size) == 0 || (a.page_size % kTileU) == 0);
  const int passes_per_page = pass_pages ? a.page_size / 16 : 1;
  const bool rows_packed = !a.paged && a.kv_s == kD;  // rows of a tile kD bytes apart
  const int kv_s32 = (int)a.kv_s, sc_s32 = (int)a.sc_s;
  int pfirst_cta, pparts;

  auto load_seq = [&]() {
    const SeqRange r = seg_range(pb, &puse_add, &pext);
    pn = r.n;
    pfirst = r.first;
    pT = tiles_u(r, a.S);
  };
  auto seg_setup = [&]() {  // pt, pslot are set
    const int t0slot = pslot - pt;  // slot of tile 0 of this segment
    pfirst_cta = cta_of_slot(t0slot);
    pparts = cta_of_slot(t0slot + pT - 1) - pfirst_cta + 1;
  };
  auto advance = [&]() {
    ++pslot;
    if (++pt < pT) return;
    pt = 0;
    pslot += kPieceCost;  // the overhead slots of the next segment
    if (++ph == a.Hkv) {
      ph = 0;
      do {
        if (++pb >= a.B) {  // past the end of the list
          pb = a.B - 1;
          pslot = INT_MAX / 2;
          return;
        }
        load_seq();
      } while (pT == 0);
    }
    seg_setup();
  };
  {
    load_seq();
    const int v0 = sm.start[2];  // slot inside the segment: overhead slots come first
    if (v0 < kPieceCost) {
      pslot += kPieceCost - v0;
      pt = 0;
    } else {
      pt = v0 - kPieceCost;
    }
    seg_setup();
  }

  // Rows [pos, pos + cnt) of segment (b, h) of one tensor (a tile: cnt <= 128, no ring wrap inside)
  // into the 16 KB at `dst`, by all threads; paged caches: pos is the token index.
  auto copy_rows = [&](uint32_t dst, const int8_t* base, int b, int h, int pos, int cnt) {
    const int8_t* seg = base + (a.paged ? (int64_t)h * a.kv_h : (int64_t)b * a.kv_b + (int64_t)h * a.kv_h) + pcol * 16;
    dst += pdst;
    if (rows_packed && cnt == kTileU) {
      // whole tile valid, rows kD bytes apart: one address
      cp_async_tile_rows<0>(dst, seg + (int64_t)(pos + prow) * kD);
    } else if (pass_pages) {
      // pass i (rows 16 i ..) lies inside one page (tiles of paged caches start at multiples of 128)
      int pi = pos / a.page_size, within = (pos % a.page_size) / 16;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const bool valid = 16 * i + prow < cnt;
        const int page = 16 * i < cnt ? a.page_table[(int64_t)b * a.max_pages + pi] : 0;
        const int64_t off = (int64_t)page * a.kv_page + (int64_t)(within * 16 + prow) * kD;
        cp_async16(dst + 2048 * i, seg + off, valid);
        if (++within == passes_per_page) {
          within = 0;
          ++pi;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = prow + 16 * i;
        const bool valid = r < cnt;
        const int tok = valid ? pos + r : pos;
        int64_t off;
        if (a.paged) {
          const int pg = a.page_table[(int64_t)b * a.max_pages + tok / a.page_size];
          off = (int64_t)pg * a.kv_page + (int64_t)(tok % a.page_size) * kD;
        } else {
          off = (int64_t)tok * kv_s32;
        }
        cp_async16(dst + 2048 * i, seg + off, valid);
      }
    }
  };
  // The same by the copy engine, requested by the calling thread alone: whole boxes (rows past cnt
  // hold other tokens or the zero fill of the tensor's edge; their logits are masked and their
  // probabilities zero), 16 KB in all, counted on `bar`.
  auto request_rows = [&](uint32_t dst, const CUtensorMap* map, uint32_t bar, int b, int h, int pos, int cnt) {
    fence_async_smem();  // earlier accesses of the threads to this slot (the merge scratch) come first
    mbar_arrive_expect_tx(bar, (uint32_t)(kTileU * kD));
    if (tma_mode == kTmaDense) {
      tma_load_rows(dst, map, pos, h, b, bar);
    } else if (box_rows == kTileU) {  // pages of 128 rows or more: the tile lies inside one
      const int page = a.page_table[(int64_t)b * a.max_pages + pos / a.page_size];
      tma_load_rows(dst, map, pos % a.page_size, page, h, bar);
    } else {  // one box per page
      int pi = pos / a.page_size;
      for (int r = 0; r < kTileU; r += box_rows, ++pi) {
        const int page = r < cnt ? a.page_table[(int64_t)b * a.max_pages + pi] : 0;
        tma_load_rows(dst + r * kD, map, 0, page, h, bar);
      }
    }
  };

  // K rows of the next tile of the share (with its record) into ring position `seq`; a record
  // with t = -1 when the share is exhausted.
  // Without the new token's staging (which every thread takes part in) the per-tile bookkeeping of the
  // CTA is spread over its warps: warp 0 issues the S^T MMAs, warp 1 walks the tile list, writes the
  // records and requests the K rows, warp 2 requests the V rows, warp 3 issues the O^T MMAs
  // (44.1 us per launch on the bench workload against 45.2 with everything in thread 0).
  constexpr bool kSpread = kTma && !kFused;
  constexpr int kWalkerWarp = kSpread ? 1 : 0, kWalkerThread = 32 * kWalkerWarp;
  constexpr int kVRequestThread = kSpread ? 64 : 0, kPvThread = kSpread ? 96 : 0;
  auto issue_k = [&](int seq) {
    if constexpr (kSpread) {
      if (warp != kWalkerWarp) {  // (the others keep their count of copy groups in step)
        cp_async_commit();
        return;
      }
    }
    if (pslot < G1) {
      SeqRange rg;
      rg.n = pn;
      rg.first = pfirst;
      int pos, cnt;
      tile_rows(rg, a.S, pt, &pos, &cnt);
      if (tid == kWalkerThread) {
        TileMeta mt;
        mt.b = pb; mt.h = ph; mt.t = pt; mt.T = pT; mt.n = pn; mt.first = pfirst; mt.use_add = puse_add;
        mt.first_cta = pfirst_cta; mt.parts = pparts;
        mt.pad[0] = cnt;  // valid rows of the tile
        mt.pad[1] = pos;  // position of its first row (paged: token index)
        mt.pad[2] = (pslot + 1 >= G1 ? 1 : 0)              // no tile follows in this CTA's share
                    | (pext && pt == pT - 1 ? 2 : 0);      // the tile's last row is the step's new token
        sm.meta[seq & 3] = mt;
        if constexpr (kTma) request_rows(smem_u32(&sm.k[seq & 1][0]), &maps.k, smem_u32(&sm.bar_k[seq & 1]), pb, ph, pos, cnt);
      }
      if constexpr (!kTma) copy_rows(smem_u32(&sm.k[seq & 1][0]), kbase, pb, ph, pos, cnt);
      if constexpr (kFused) {
        if (pext && pt == pT - 1) stage_new_token(seq, pb, ph);  // the segment's last tile takes the new token
      }
      advance();
    } else if (tid == kWalkerThread) {
      sm.meta[seq & 3].t = -1;
    }
    cp_async_commit();
  };
  // V rows of the tile at ring position `seq` (its record is in shared memory), its query rows when
  // it starts a piece (converted at the end of this iteration), and the scales of this thread's
  // token in it, consumed by this same thread an iteration later:
  // they stay raw bits until then, so that nothing here waits for the loads.
  const bool sc_f32 = a.scale_is_f32 != 0;
  const uint32_t raw_one = sc_f32 ? 0x3f800000u : 0x3f80u;
  auto scale_of = [&](uint32_t raw) { return __uint_as_float(sc_f32 ? raw : raw << 16); };
  uint32_t nks = raw_one, nvs = 0u;
  auto issue_v = [&](int seq) {
    const int mb = sm.meta[seq & 3].b, mh = sm.meta[seq & 3].h, mtile = sm.meta[seq & 3].t;
    const int cnt = sm.meta[seq & 3].pad[0], pos = sm.meta[seq & 3].pad[1];
    if (mtile >= 0) {
      if constexpr (kTma) {
        if (tid == kVRequestThread) request_rows(smem_u32(&sm.v[seq & 1][0]), &maps.v, smem_u32(&sm.bar_v[seq & 1]), mb, mh, pos, cnt);
      } else {
        copy_rows(smem_u32(&sm.v[seq & 1][0]), vbase, mb, mh, pos, cnt);
      }
      if (seq == 0 || mtile == 0) {  // a piece starts with this tile
        const __nv_bfloat16* q = qbase + ((int64_t)mb * a.Hkv + mh) * R * kD;
        for (int ch = tid; ch < R * 16; ch += kThreads) cp_async16(smem_u32(&sm.qraw[0]) + ch * 16, q + ch * 8, true);
      }
      nks = raw_one;
      nvs = 0u;
      if (tid < cnt) {
        nvs = raw_one;
        if (quant) {
          const int tok = pos + tid;
          int64_t sidx;
          if (a.paged) {
            const int pg = a.page_table[(int64_t)mb * a.max_pages + tok / a.page_size];
            sidx = (int64_t)pg * a.page_size + tok % a.page_size;
          } else {
            sidx = (int64_t)mb * a.sc_b + (int64_t)tok * sc_s32;
          }
          if (sc_f32) {
            nks = static_cast<const uint32_t*>(a.k_scale)[sidx];
            nvs = static_cast<const uint32_t*>(a.v_scale)[sidx];
          } else {
            nks = static_cast<const uint16_t*>(a.k_scale)[sidx];
            nvs = static_cast<const uint16_t*>(a.v_scale)[sidx];
          }
        }
      }
    }
    cp_async_commit();
  };

  // ------------------------------------------------------------------ consumer state
  float m_run[8], l_run[8], o[8];  // l_run: this thread's token share of the denominators; o: head-dim index tid
  int piece_t0 = 0;
  bool dead = false;  // a wait ran out
  const float unit2 = a.sm_scale * kLog2e;
  const uint32_t bar_s = smem_u32(&sm.bar[0]), bar_o = smem_u32(&sm.bar[1]);
  const uint32_t q_desc_addr = smem_u32(&sm.qlev[0]), p_desc_addr = smem_u32(&sm.plev[0]);
  // this thread's byte of row r of the probability levels: ((tid / 16) ^ r) * 16 + tid % 16.
  // plev is 1024-byte aligned, so the XOR with r << 4 can be applied to the whole address.
  const uint32_t p_base = smem_u32(&sm.plev[0]) + (tid & 15) + ((uint32_t)(tid >> 4) << 4);

  // Query levels of the piece that starts with tile number `seq` of this CTA (when it
  // starts one), then S^T of that tile on the tensor core.  Called by the whole
  // CTA once the tile's K rows have landed and a barrier has made them (and the
  // record) visible; the logits of the tile before are out of tensor memory.
  auto prepare = [&](int seq, const TileMeta& mt, bool first) {
    if (first || mt.t == 0) {
      // thread (row = tid / 16, chunk = tid % 16) converts 8 values of one query row
      const int row = tid >> 4, ch = tid & 15;
      float f[8];
      if (row < R) {
        const uint4 raw = *reinterpret_cast<const uint4*>(&sm.qraw[row * (kD * 2) + ch * 16]);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t = __bfloat1622float2(p2[e]);
          f[2 * e] = t.x;
          f[2 * e + 1] = t.y;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = 0.f;
      }
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
#pragma unroll
      for (int sh = 1; sh <= 8; sh <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sh));
      const float inv = amax > 0.f ? 127.f / amax : 0.f;
      uint32_t hi[2] = {0u, 0u}, lo[2] = {0u, 0u};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float t = f[e] * inv;
        const float h = rintf(t);
        const float l = rintf((t - h) * 254.f);
        hi[e >> 2] |= ((uint32_t)(int)h & 0xffu) << (8 * (e & 3));
        lo[e >> 2] |= ((uint32_t)(int)l & 0xffu) << (8 * (e & 3));
      }
      *reinterpret_cast<uint2*>(&sm.qlev[swz(row, 8 * ch)]) = make_uint2(hi[0], hi[1]);
      *reinterpret_cast<uint2*>(&sm.qlev[swz(8 + row, 8 * ch)]) = make_uint2(lo[0], lo[1]);
      if (ch == 0) {
        sm.qsc[row] = amax * (1.f / 127.f) * unit2 * (1.f / 254.f);
        if constexpr (kRound) sm.qsr[row] = amax * (1.f / 127.f) * (1.f / 254.f);
      }
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
    }
    if constexpr (kFused) {
      if (mt.pad[2] & 2) {  // the new token becomes the row behind the tile's existing tokens
        if constexpr (kTma) {
          if (!mbar_wait(smem_u32(&sm.bar_k[seq & 1]), (uint32_t)(seq >> 1) & 1u)) dead = true;  // the rows must be there first
        }
        quantise_new_token(seq, mt.b, mt.h, mt.pad[0] - 1);
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
      }
    }
    if (tid == 0) {
      if constexpr (kTma) {
        if (!mbar_wait(smem_u32(&sm.bar_k[seq & 1]), (uint32_t)(seq >> 1) & 1u)) dead = true;
      }
      tc_fence_after();
      const uint32_t k_addr = smem_u32(&sm.k[seq & 1][0]);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_i8(tmem, umma_desc(k_addr + 32 * ks), umma_desc(q_desc_addr + 32 * ks), kIdescS, ks > 0);
      umma_commit(bar_s);
    }
  };
  // O^T of the tile with the given parity into the accumulators (alpha and cmax are that tile's)
  auto add_output = [&](uint32_t parity, const float (&alpha)[8], float cmax) {
    if (!mbar_wait(bar_o, parity)) dead = true;
    tc_fence_after();
    uint32_t o01[16];
    tmem_ld16(tmem_lane + kColO, o01);
    tmem_ld_wait();
    tc_fence_before();
    const float oscale = cmax * (1.f / 65535.f);
#pragma unroll
    for (int r = 0; r < kR; ++r)  // the two levels combine exactly in int32
      o[r] = fmaf(o[r], alpha[r], (float)((int)o01[r] + ((int)o01[8 + r] << 8)) * oscale);
  };

  // The tensor core works one step ahead of the threads: S^T of tile i+1 is
  // issued at the end of iteration i, and O^T of tile i is collected in
  // iteration i+1 (at once only when tile i ends a piece), so neither MMA is
  // waited for right after it was issued.
  // Copy groups are committed in the order K0, V0, K1, then V(i+1), K(i+2) in iteration i.
  issue_k(0);
  __syncthreads();  // the record of tile 0
  issue_v(0);
  issue_k(1);
  if constexpr (kFused) post_amax();
  cp_async_wait<1>();  // K0 and V0 (with the query rows)
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  TileMeta mt = sm.meta[0];
  JPT_SPAN(3);
  if (mt.t >= 0) prepare(0, mt, true);

  float alpha_prev[8], cmax_prev = 0.f;
  bool pending = false;  // O^T of the tile before has not been added yet
  for (int i = 0; mt.t >= 0; ++i) {
    float cks = scale_of(nks), cvs = scale_of(nvs);  // scales of this thread's token in tile i
    if constexpr (kFused) {
      if ((mt.pad[2] & 2) && tid == mt.pad[0] - 1) {  // the new token: its scales were just computed
        cks = sm.ntsc[i & 1][0];
        cvs = sm.ntsc[i & 1][1];
      }
    }
    const bool last_of_share = (mt.pad[2] & 1) != 0;
    const uint32_t par = (uint32_t)i & 1u;
    if (i == 0 || mt.t == 0) {  // a piece starts (the one before was flushed when it ended)
      piece_t0 = mt.t;
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        m_run[r] = kNoMax;
        l_run[r] = 0.f;
        o[r] = 0.f;
      }
    }

    // ---------------- the output of the tile before and the logits of this one leave
    // tensor memory in one round trip; the K slot of this tile and the V slot of the tile
    // before are free after that
    if (!mbar_wait(bar_s, par)) dead = true;
    if (pending && !mbar_wait(bar_o, par ^ 1u)) dead = true;
    tc_fence_after();
    float xv[8];
    {
      uint32_t s[16];
      if (pending) {
        uint32_t o01[16];
        tmem_ld16(tmem_lane + kColO, o01);
        tmem_ld16(tmem_lane, s);
        tmem_ld_wait();
        const float oscale = cmax_prev * (1.f / 65535.f);
#pragma unroll
        for (int r = 0; r < kR; ++r)  // the two levels combine exactly in int32 (|O_0 + 256 O_1| < 2^31)
          o[r] = fmaf(o[r], alpha_prev[r], (float)((int)o01[r] + ((int)o01[8 + r] << 8)) * oscale);
        pending = false;
      } else {
        tmem_ld16(tmem_lane, s);
        tmem_ld_wait();
      }
      issue_v(i + 1);
      issue_k(i + 2);
      const bool valid = tid < mt.pad[0];
      float mk = valid ? 0.f : -INFINITY;  // a row past the tile's tokens: finite dot product + (-inf)
      if (mt.use_add && valid)             // additive mask that is not a plain 0 / -inf range (rare)
        mk = __bfloat162float(mask[(int64_t)mt.b * a.mk_b + mt.pad[1] + tid]);
      if constexpr (!kRound) {
        const float4 q0 = *reinterpret_cast<const float4*>(&sm.qsc[0]), q1 = *reinterpret_cast<const float4*>(&sm.qsc[4]);
        const float qc[8] = {q0.x * cks, q0.y * cks, q0.z * cks, q0.w * cks, q1.x * cks, q1.y * cks, q1.z * cks, q1.w * cks};
        const float ml = mk * kLog2e;
#pragma unroll
        for (int r = 0; r < kR; ++r) xv[r] = fmaf((float)((int)s[r] * 254 + (int)s[8 + r]), qc[r], ml);
      } else {
        // dense_attention on bf16 tensors: the reference rounds the logit to bf16 after every step
        const float sqrt_d = __frcp_rn(a.sm_scale);
#pragma unroll
        for (int r = 0; r < kR; ++r)
          xv[r] = kLog2e * rounded_logit((float)((int)s[r] * 254 + (int)s[8 + r]) * sm.qsr[r], sqrt_d, cks, quant, mk);
      }
    }
    // tile maxima per row (and the largest V scale) across the 128 tokens
    {
      float wm[9] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kR; ++r) wm[r] = warp_max(xv[r]);
      wm[8] = warp_max(cvs);
      if (lane == 0) {
        *reinterpret_cast<float4*>(&sm.xch[warp][0]) = make_float4(wm[0], wm[1], wm[2], wm[3]);
        *reinterpret_cast<float4*>(&sm.xch[warp][4]) = make_float4(wm[4], wm[5], wm[6], wm[7]);
        sm.xch[warp][8] = wm[8];
      }
    }
    tc_fence_before();
    __syncthreads();

    float alpha[8];
    float cmax;
    {
      float4 t0[4], t1[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        t0[w] = *reinterpret_cast<const float4*>(&sm.xch[w][0]);
        t1[w] = *reinterpret_cast<const float4*>(&sm.xch[w][4]);
      }
      cmax = fmaxf(fmaxf(sm.xch[0][8], sm.xch[1][8]), fmaxf(sm.xch[2][8], sm.xch[3][8]));
      float tm[8];
      tm[0] = fmaxf(fmaxf(t0[0].x, t0[1].x), fmaxf(t0[2].x, t0[3].x));
      tm[1] = fmaxf(fmaxf(t0[0].y, t0[1].y), fmaxf(t0[2].y, t0[3].y));
      tm[2] = fmaxf(fmaxf(t0[0].z, t0[1].z), fmaxf(t0[2].z, t0[3].z));
      tm[3] = fmaxf(fmaxf(t0[0].w, t0[1].w), fmaxf(t0[2].w, t0[3].w));
      tm[4] = fmaxf(fmaxf(t1[0].x, t1[1].x), fmaxf(t1[2].x, t1[3].x));
      tm[5] = fmaxf(fmaxf(t1[0].y, t1[1].y), fmaxf(t1[2].y, t1[3].y));
      tm[6] = fmaxf(fmaxf(t1[0].z, t1[1].z), fmaxf(t1[2].z, t1[3].z));
      tm[7] = fmaxf(fmaxf(t1[0].w, t1[1].w), fmaxf(t1[2].w, t1[3].w));
      // p <= 1 and the product is held at 2^16 - 1 (the fast division may land one ulp above)
      const float rc = cmax > 0.f ? __fdividef(65535.f, cmax) : 0.f;
      const float ps = fminf(cvs * rc, 65535.f);
      softmax_rows<0, kR>(m_run, l_run, alpha, tm, xv, ps, p_base);
    }
    if constexpr (kFused) {
      if (mt.pad[2] & 2) {  // the new token's V codes into the row behind the tile's existing tokens
        if constexpr (kTma) {
          if (!mbar_wait(smem_u32(&sm.bar_v[i & 1]), (uint32_t)(i >> 1) & 1u)) dead = true;
        } else {
          cp_async_wait<3>();
          __syncthreads();  // every thread's copies into this tile have landed
        }
        sm.v[i & 1][swz(mt.pad[0] - 1, tid)] = sm.ntv[i & 1][tid];
      }
    }
    cp_async_wait<3>();  // V rows of this tile (younger groups: K(i+1), V(i+1), K(i+2))
    fence_async_smem();
    __syncthreads();

    // ---------------- O^T = V^T Pl^T on the tensor core
    if (tid == kPvThread) {
      if constexpr (kTma) {
        if (!mbar_wait(smem_u32(&sm.bar_v[i & 1]), (uint32_t)(i >> 1) & 1u)) dead = true;
      }
      tc_fence_after();
      const uint32_t v_addr = smem_u32(&sm.v[i & 1][0]);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_i8(tmem + kColO, umma_desc(v_addr + 4096 * ks), umma_desc(p_desc_addr + 32 * ks), kIdescO, ks > 0);
      umma_commit(bar_o);
    }

    // The tile that ends a piece leaves through the epilogue below, after the next tile's S^T has been
    // issued (the tensor core and the copies keep going while the rows are written or merged).
    const bool piece_ends = last_of_share || mt.t == mt.T - 1;
    const int cb = mt.b, chd = mt.h, ct = mt.t, cT = mt.T, cfirst_cta = mt.first_cta, cparts = mt.parts;
    if (!piece_ends) {
#pragma unroll
      for (int r = 0; r < kR; ++r) alpha_prev[r] = alpha[r];
      cmax_prev = cmax;
      pending = true;
    }

    // ---------------- the next tile: its K rows were requested an iteration ago
    if (sm.meta[(i + 1) & 3].t == 0) {
      cp_async_wait<1>();  // it starts a piece: its query rows travel with V(i+1) (younger group: K(i+2))
    } else {
      cp_async_wait<2>();  // (younger groups: V(i+1), K(i+2))
    }
    fence_async_smem();
    tc_fence_before();
    if (__syncthreads_or(dead)) {
      if (tid == 0) {
        atomicExch(status, 1);
        if constexpr (kTma) {  // requests of the copy engine that may still be in flight get their (bounded) time
          if (sm.meta[(i + 1) & 3].t >= 0) {
            mbar_wait(smem_u32(&sm.bar_k[(i + 1) & 1]), (uint32_t)((i + 1) >> 1) & 1u);
            mbar_wait(smem_u32(&sm.bar_v[(i + 1) & 1]), (uint32_t)((i + 1) >> 1) & 1u);
            if (sm.meta[(i + 2) & 3].t >= 0) mbar_wait(smem_u32(&sm.bar_k[i & 1]), (uint32_t)((i + 2) >> 1) & 1u);
          }
        }
      }
      break;
    }
    mt = sm.meta[(i + 1) & 3];
    if (mt.t >= 0) prepare(i + 1, mt, false);
    if (piece_ends) {
      // ---------------- end of a piece: write the rows, or a partial for the merge
      const bool is_final = piece_t0 == 0 && ct == cT - 1;
      const int slot = piece_t0 > 0 ? 0 : 1;
      const int64_t row_base = ((int64_t)cb * a.Hkv + chd) * R;
      // denominators: sum the token shares of the 128 threads (while the last O^T MMA runs)
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        float l = l_run[r];
#pragma unroll
        for (int sh = 1; sh <= 16; sh <<= 1) l += __shfl_xor_sync(0xffffffffu, l, sh);
        if (lane == r) sm.red[warp][r] = l;
      }
      __syncthreads();
      add_output(par, alpha, cmax);
      float L8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, M8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        L8[r] = (sm.red[0][r] + sm.red[1][r]) + (sm.red[2][r] + sm.red[3][r]);
        M8[r] = m_run[r] > 0.5f * kNoMax ? m_run[r] : -INFINITY;  // every logit of the row was masked
      }
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        if (r < R) {
          const float L = L8[r], M = M8[r];
          if (is_final) {
            const int64_t row = row_base + r;
            static_cast<__nv_bfloat16*>(a.o)[row * kD + tid] = __float2bfloat16_rn(L > 0.f ? o[r] / L : 0.f);
            if (tid == 0) {
              if (a.m) a.m[row] = M * kLn2;
              if (a.l) a.l[row] = L > 0.f ? L : 0.f;
            }
          } else {
            const int64_t pr = ((int64_t)cta * 2 + slot) * kMaxRows + r;
            __stcg(&x.part_o[pr * kD + tid], o[r]);
            if (tid == 0) {
              __stcg(&x.part_m[pr], M);
              __stcg(&x.part_l[pr], L);
              __stcg(&x.part_t[pr], M);
            }
          }
        }
      }
      if (!is_final) {
        // Whoever delivers the last piece of the segment combines all of them.
        // The counter wraps back to zero on that arrival, ready for the next launch.
        // (the barrier orders the CTA's stores before thread 0's fence, which publishes them with the arrival)
        __syncthreads();
        if (tid == 0) {
          __threadfence();
          const unsigned old = atomicInc(&x.counters[cb * a.Hkv + chd], (unsigned)(cparts - 1));
          sm.flag = old == (unsigned)(cparts - 1);
        }
        __syncthreads();
        if (sm.flag) {
          __threadfence();
          merge_segment(a, x, cfirst_cta, cparts, row_base);
        }
      }
    
    }
    if (i == 0) JPT_SPAN(4);
#ifdef JPT_UMMA_SPANS
    if (threadIdx.x == 0 && blockIdx.x < 1024) {
      g_umma_spans[8 * blockIdx.x + 6] += 1;                                  // tiles
    }
#endif
  }
  JPT_SPAN(5);
  clear_empty_rows();
  exchange_done();
  cp_async_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kTmemCols) : "memory");
  }
  JPT_SPAN(7);  // end
}

int umma_num_ctas() { return sm_count() * kCtasPerSm; }

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// [dims[3]][dims[2]][dims[1]][128] bytes with byte strides str[0..2] between rows / dims[2] / dims[3].
bool encode_rows_map(CUtensorMap* map, const void* base, const cuuint64_t (&dims)[4], const cuuint64_t (&str)[3], int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint32_t box[4] = {(cuuint32_t)kD, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, str, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapKey {
  const void *k, *v;
  int64_t d1, d2, d3, s0, s1, s2;
  int mode, box_rows, device;
  bool operator==(const MapKey& o) const {
    return k == o.k && v == o.v && d1 == o.d1 && d2 == o.d2 && d3 == o.d3 && s0 == o.s0 && s1 == o.s1 && s2 == o.s2 &&
           mode == o.mode && box_rows == o.box_rows && device == o.device;
  }
};
struct MapEntry {
  MapKey key;
  TmaMaps maps;
};

// Tensor maps for this call (cached per tensor pair and geometry); kTmaNone when
// the layout cannot be described (the kernel then copies the rows with its threads).
// JPT_NO_TMA=1 in the environment forces that path.
int tensor_maps_for(const jpt_attn_params& p, TmaMaps* out, int* box_rows) {
  static const bool off = [] {
    const char* e = getenv("JPT_NO_TMA");
    return e && e[0] == '1';
  }();
  if (off) return kTmaNone;
  MapKey key{};
  key.k = p.k;
  key.v = p.v;
  key.device = current_device();
  if (p.paged) {
    if (p.page_size % 16 != 0 || p.kv_page != (int64_t)p.page_size * kD || p.kv_h <= 0 || p.kv_h % p.kv_page != 0) return kTmaNone;
    if ((kTileU % p.page_size) != 0 && (p.page_size % kTileU) != 0) return kTmaNone;
    key.mode = kTmaPaged;
    key.box_rows = p.page_size < kTileU ? p.page_size : kTileU;
    key.d1 = p.page_size; key.d2 = p.kv_h / p.kv_page; key.d3 = p.Hkv;
    key.s0 = kD; key.s1 = p.kv_page; key.s2 = p.kv_h;
  } else {
    key.mode = kTmaDense;
    key.box_rows = kTileU;
    key.d1 = p.S; key.d2 = p.Hkv; key.d3 = p.B;
    key.s0 = p.kv_s; key.s1 = p.kv_h; key.s2 = p.kv_b;
    if (p.Hkv == 1 && key.s1 <= 0) key.s1 = key.s0 * p.S;  // a single head: its stride is never used
    if (p.B == 1 && key.s2 <= 0) key.s2 = key.s1 * p.Hkv;
  }
  if (key.s0 % 16 || key.s1 % 16 || key.s2 % 16 || key.s0 < kD || key.s1 <= 0 || key.s2 <= 0) return kTmaNone;
  if (!aligned(p.k, 16) || !aligned(p.v, 16)) return kTmaNone;
  *box_rows = key.box_rows;
  static std::mutex mu;
  static std::vector<MapEntry> cache;
  std::lock_guard<std::mutex> lock(mu);
  for (const MapEntry& e : cache) {
    if (e.key == key) {
      *out = e.maps;
      return key.mode;
    }
  }
  const cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)key.d1, (cuuint64_t)key.d2, (cuuint64_t)key.d3};
  const cuuint64_t str[3] = {(cuuint64_t)key.s0, (cuuint64_t)key.s1, (cuuint64_t)key.s2};
  MapEntry e;
  e.key = key;
  if (!encode_rows_map(&e.maps.k, p.k, dims, str, key.box_rows) || !encode_rows_map(&e.maps.v, p.v, dims, str, key.box_rows))
    return kTmaNone;
  if (cache.size() >= 4096) cache.clear();
  cache.push_back(e);
  *out = e.maps;
  return key.mode;
}

}  // namespace

bool attention_umma_eligible(const jpt_attn_params& p) {
  const int R = (p.Hq / p.Hkv) * p.Tq;
  return attention_mma_eligible(p) && p.kv_dtype == JPT_INT8 && R <= 8;
}

int launch_attention_umma(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st, const NewTokenArgs* nt_in) {
  const ScratchLayout lay = scratch_layout(p, umma_num_ctas());
  JPT_REQUIRE(p.workspace && p.workspace_bytes >= lay.total, JPT_EWORKSPACE,
              "flash_decode: workspace of %zu bytes needed, %zu given", lay.total, p.workspace_bytes);
  JPT_REQUIRE(aligned(p.workspace, 256), JPT_EALIGN, "flash_decode: workspace must be 256-byte aligned");
  char* ws = static_cast<char*>(p.workspace);
  MmaScratch x;
  x.counters = reinterpret_cast<unsigned*>(ws + lay.counters);
  x.seqinfo = reinterpret_cast<int32_t*>(ws + lay.seqinfo);
  x.part_m = reinterpret_cast<float*>(ws + lay.part_m);
  x.part_l = reinterpret_cast<float*>(ws + lay.part_l);
  x.part_t = reinterpret_cast<float*>(ws + lay.part_t);
  x.part_o = reinterpret_cast<float*>(ws + lay.part_o);
  x.num_ctas = lay.num_ctas;
  int* status = reinterpret_cast<int*>(ws + kWorkspaceStatusOffset);

  constexpr int smem_bytes = (int)sizeof(SmemU);
  static_assert(kCtasPerSm * (smem_bytes + 1024) <= 228 * 1024, "shared memory of the resident CTAs exceeds the SM");
  static std::atomic<bool> configured[kMaxDevices];
  if (int rc = configure_once_per_device(configured, "flash_decode_i8_umma_kernel", [] {
        cudaError_t e = cudaSuccess;
        auto set = [&e](auto kernel) {  // three CTAs of 73 KB per SM
          if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
          if (e == cudaSuccess)
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        };
        set(flash_decode_i8_umma_kernel<false, false, false, 8>);
        set(flash_decode_i8_umma_kernel<false, false, true, 8>);
        set(flash_decode_i8_umma_kernel<false, true, false, 8>);
        set(flash_decode_i8_umma_kernel<false, true, true, 8>);
        set(flash_decode_i8_umma_kernel<true, false, false, 8>);
        set(flash_decode_i8_umma_kernel<true, false, true, 8>);
        set(flash_decode_i8_umma_kernel<true, true, false, 8>);
        set(flash_decode_i8_umma_kernel<true, true, true, 8>);
        set(flash_decode_i8_umma_kernel<false, false, false, 4>);
        set(flash_decode_i8_umma_kernel<false, false, true, 4>);
        set(flash_decode_i8_umma_kernel<false, true, false, 4>);
        set(flash_decode_i8_umma_kernel<false, true, true, 4>);
        set(flash_decode_i8_umma_kernel<true, false, false, 4>);
        set(flash_decode_i8_umma_kernel<true, false, true, 4>);
        set(flash_decode_i8_umma_kernel<true, true, false, 4>);
        set(flash_decode_i8_umma_kernel<true, true, true, 4>);
        set(flash_decode_i8_umma_kernel<false, false, false, 2>);
        set(flash_decode_i8_umma_kernel<false, false, true, 2>);
        set(flash_decode_i8_umma_kernel<false, true, false, 2>);
        set(flash_decode_i8_umma_kernel<false, true, true, 2>);
        set(flash_decode_i8_umma_kernel<true, false, false, 2>);
        set(flash_decode_i8_umma_kernel<true, false, true, 2>);
        set(flash_decode_i8_umma_kernel<true, true, false, 2>);
        set(flash_decode_i8_umma_kernel<true, true, true, 2>);
        return e;
      }))
    return rc;
  if (a.mask_mode == JPT_MASK_ADD) {
    if (int rc = launch_mask_ranges(a, x, st)) return rc;
  }
  NewTokenArgs nt;
  memset(&nt, 0, sizeof(nt));
  if (nt_in) {
    nt = *nt_in;
    if (nt.px_state == nullptr) {  // one GPU: the exchange slots live in the workspace
      nt.px_state = reinterpret_cast<unsigned*>(ws + lay.exchange);
      nt.px_slots[0] = reinterpret_cast<unsigned long long*>(ws + lay.exchange + kExchangeStateBytes);
      nt.px_rank = 0;
      nt.px_world = 1;
    }
    if (nt.px_wait_cycles <= 0) nt.px_wait_cycles = kWaitCycles;
    nt.enabled = 1;
  }
  TmaMaps maps;
  memset(&maps, 0, sizeof(maps));
  int box_rows = kTileU;
  const int tma_mode = tensor_maps_for(p, &maps, &box_rows);
  const bool fused = nt.enabled != 0, round = a.round_logits != 0, tma = tma_mode != kTmaNone;
  const dim3 grid(lay.num_ctas), block(kThreads);
#define JPT_UMMA_LAUNCH2(F, Rd, T)                                                                                       \
  do {                                                                                                                   \
    if (a.R <= 2)                                                                                                        \
      launch_after_previous(flash_decode_i8_umma_kernel<F, Rd, T, 2>, grid, block, smem_bytes, st, a, x, status, nt, maps, \
                            tma_mode, box_rows);                                                                         \
    else if (a.R <= 4)                                                                                                   \
      launch_after_previous(flash_decode_i8_umma_kernel<F, Rd, T, 4>, grid, block, smem_bytes, st, a, x, status, nt, maps, \
                            tma_mode, box_rows);                                                                         \
    else                                                                                                                 \
      launch_after_previous(flash_decode_i8_umma_kernel<F, Rd, T, 8>, grid, block, smem_bytes, st, a, x, status, nt, maps, \
                            tma_mode, box_rows);                                                                         \
  } while (0)
#define JPT_UMMA_LAUNCH(F, Rd, T) JPT_UMMA_LAUNCH2(F, Rd, T)
  if (fused) {
    if (round) { if (tma) JPT_UMMA_LAUNCH(true, true, true); else JPT_UMMA_LAUNCH(true, true, false); }
    else       { if (tma) JPT_UMMA_LAUNCH(true, false, true); else JPT_UMMA_LAUNCH(true, false, false); }
  } else {
    if (round) { if (tma) JPT_UMMA_LAUNCH(false, true, true); else JPT_UMMA_LAUNCH(false, true, false); }
    else       { if (tma) JPT_UMMA_LAUNCH(false, false, true); else JPT_UMMA_LAUNCH(false, false, false); }
  }
#undef JPT_UMMA_LAUNCH2
#undef JPT_UMMA_LAUNCH
  return check_launch("flash_decode_i8_umma_kernel");
}

}  // namespace jpt

#ifdef JPT_UMMA_SPANS
extern "C" int jpt_debug_umma_spans(unsigned long long* out_host, int n_ctas) {
  return (int)cudaMemcpyFromSymbol(out_host, jpt::g_umma_spans, sizeof(unsigned long long) * 8 * n_ctas);
}
#endif
