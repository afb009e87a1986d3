// Ragged flash-decode attention for int8 caches, head_dim 128 and up to 8
// grouped query rows on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// The int8 codes never pass through registers: both contractions run as
// integer MMAs that read K, V and the small second operands straight from
// shared memory and accumulate int32 in tensor memory (TMEM).  A round handles
// a tile of 256 consecutive valid tokens of one (sequence, KV head) segment as
// two halves of 128 tokens (128 = the M extent of one MMA = the TMEM lanes):
//
//   S^T_h[128 tok x 16] = K_h[128 tok x 128 d] . Ql^T     kind::i8, K-major A and B   (h = 0, 1)
//   O^T[128 d x 16]    += V_h^T[128 d x 128 tok] . Pl_h^T kind::i8, MN-major A, K-major B
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
//     Pl[8 l + r]; O = (O_0 + 2^8 O_1) c / (2^16 - 1).  The rounding error of a
//     probability is at most 2^-17 of the row's largest one.
// Every int32 sum is exact (|O_0 + 2^8 O_1| <= 256 * 127 * 65535 < 2^31), so
// the only roundings are the two splits above and the fp32 online-softmax
// arithmetic.
//
// A CTA has 256 threads, one per token of the tile: thread (g, t) of group g
// (warps 4 g .. 4 g + 3) owns token 128 g + t in the softmax phase (TMEM lane t
// of S^T_g) and head-dim index t of rows 4 g .. 4 g + 3 in the output phase
// (TMEM lane t of O^T), which also removes the cross-warp merge of the
// accumulators.  One exchange of row maxima, one MMA issue and one rescale of
// the accumulators serve 256 tokens; two CTAs of 8 warps share an SM.
//
// Tiles are scheduled as in the mma.sync kernel (equal contiguous shares of one
// global tile list, pieces, last-arriver merge).  K and V rows land in shared
// memory as 128-byte rows, 16-byte chunks XORed with (row & 7): the canonical
// 128-byte-swizzle layout of the tensor core for both operand roles (K-major
// for K, MN-major for V), so nothing is rearranged.  K has ONE buffer (the
// S^T MMAs of a round are issued a round ahead and are long finished when the
// next K rows are requested), V has two.  The rows are moved by the copy engine
// where the cache can be described by a tensor map (cp.async.bulk.tensor boxes
// of 256 or 32 rows with the 128-byte swizzle, issued by one thread, completion
// counted in bytes on an mbarrier); caches that cannot (row strides that are not
// multiples of 16 bytes, page sizes that are not multiples of 32) are copied 16
// bytes at a time by all threads.  A segment whose valid range wraps around the
// ring is cut into tiles run by run, so a tile is always one range of rows.
//
// Fused decode update (jpt_decode_update_attend): the launch also takes the
// step's new K/V token.  CTA b mod grid computes the token's amax over this
// GPU's heads first thing and stores it into the exchange slots of every rank
// (NVLink peer stores when the KV heads are sharded); the tiles of the existing
// tokens stream as usual; the CTA that writes a segment's final rows reads the
// ranks' words (long there by then), quantises the token's row for its head
// with the decode quantiser, writes cache row, scale and stash, and folds the
// token into the result as one more softmax term.  One launch per layer, the
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

constexpr int kHalfU = 128;           // tokens per MMA = TMEM lanes
constexpr int kTileU = 2 * kHalfU;    // tokens per round
constexpr int kThreadsU = kTileU;     // one thread per token of a round
constexpr int kTmemCols = 64;         // S^T_0: columns 0..15, S^T_1: 16..31, O^T: 32..47
constexpr int kColS1 = 16, kColO = 32;
constexpr int kCtasPerSm = 2;
#ifndef JPT_PIECE_COST_U
#define JPT_PIECE_COST_U 1
#endif
constexpr int kPieceCostU = JPT_PIECE_COST_U;  // overhead slots charged per segment, in 256-token tiles
constexpr long long kWaitCycles = 1000000000ll;  // about half a second: far beyond any wait of a healthy run

struct __align__(1024) SmemU {
  uint8_t k[kTileU * kD];        // [token][128 bytes], swizzled; halves 16 KB apart
  uint8_t v[2][kTileU * kD];     // [stage][token][128 bytes], swizzled
  uint8_t qlev[16 * kD];         // query levels: rows 0..7 high bytes, 8..15 low bytes
  uint8_t plev[2][16 * kHalfU];  // probability levels per half: row 8 l + r, one byte per token
  uint8_t qraw[8 * kD * 2];      // bf16 query rows of the piece whose first tile is in flight
  float xch[8][12];              // per warp: row maxima of the tile [8], largest V scale [1]
  float red[8][8];               // per warp: denominators at the end of a piece
  float ntx[2][4];               // new token, per 128-thread group: K amax, V amax
  float dot[2][4][8];            // new token, per group and warp: partial logits of up to 8 rows
  float qsc[8];                  // s_r * sm_scale * log2(e) / 254
  float qsr[8];                  // s_r / 254 (the chain of rounded logits starts from the plain dot product)
  uint64_t bar[2];               // MMA completion: S^T (both halves), O^T
  uint64_t bar_in[3];            // rows landed (copy-engine path): K, V stage 0, V stage 1
  uint32_t tmem_base;
  int start[3];
  int flag;
  TileMeta meta[2];
};

// 16-byte copy with compile-time offsets on both addresses (one pair of base registers per tensor)
template <int kOff>
__device__ __forceinline__ void cp_async16_at(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0 + %2], [%1 + %2], 16;\n" ::"r"(dst), "l"(src), "n"(kOff));
}
template <int kI>
__device__ __forceinline__ void cp_async_tile_rows(uint32_t kdst, uint32_t vdst, const void* kp, const void* vp) {
  if constexpr (kI < 8) {  // 8 passes of 32 rows
    cp_async16_at<4096 * kI>(kdst, kp);
    cp_async16_at<4096 * kI>(vdst, vp);
    cp_async_tile_rows<kI + 1>(kdst, vdst, kp, vp);
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
template <int kRow>
__device__ __forceinline__ void softmax_rows(float (&m_run)[8], float (&l_run)[8], float (&alpha)[8], const float (&tm)[8],
                                             const float (&x)[8], float ps, uint32_t p_base) {
  if constexpr (kRow < 8) {
    const float mn = fmaxf(m_run[kRow], tm[kRow]);
    const float al = ex2(m_run[kRow] - mn);
    const float p = ex2(x[kRow] - mn);
    alpha[kRow] = al;
    m_run[kRow] = mn;
    l_run[kRow] = fmaf(l_run[kRow], al, p);
    // the byte of row r: 16-byte chunk (t / 16) ^ r of that row (the XOR folds into the address)
    store_levels<128 * kRow>(p_base ^ (uint32_t)(kRow << 4), __float2uint_rn(p * ps));
    softmax_rows<kRow + 1>(m_run, l_run, alpha, tm, x, ps, p_base);
  }
}
// A segment's valid tokens form one run of consecutive rows, or two when the
// ring wraps: [first, first + nA) and [0, n - nA).  Tiles never straddle the
// wrap: run A is cut into tiles of 256 rows (the last one partial), then run B.
__device__ __forceinline__ int run_a(const SeqRange& r, int S) { return min(r.n, S - r.first); }
__device__ __forceinline__ int tiles_run(int n) { return (n + kTileU - 1) / kTileU; }
__device__ __forceinline__ int tiles_u(const SeqRange& r, int S) {
  const int na = run_a(r, S);
  return tiles_run(na) + tiles_run(r.n - na);
}
__device__ __forceinline__ int slots_u(const SeqRange& r, int S) { return r.n > 0 ? tiles_u(r, S) + kPieceCostU : 0; }
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
// Instruction descriptors: int32 accumulators, M = 128, N = 16.
constexpr uint32_t kIdescS = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);  // s8 x s8
constexpr uint32_t kIdescO =
    (2u << 4) | (1u << 7) | (0u << 10) | (1u << 15) | ((16u >> 3) << 17) | ((128u >> 4) << 24);  // s8 (MN-major) x u8

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
      if (mbar_probe(bar, parity)) return true;
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
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// barrier of one 128-thread group of the CTA (ids 3 and 4; 0 is __syncthreads, 2 the merge's)
__device__ __forceinline__ void group_barrier(int g) {
  if (g == 0) {
    asm volatile("bar.sync 3, 128;" ::: "memory");
  } else {
    asm volatile("bar.sync 4, 128;" ::: "memory");
  }
}
// maximum over the 32 lanes in one instruction
__device__ __forceinline__ float warp_max(float x) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(x));
  return r;
}

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

// Tensor maps of the K and V tensors: dense [B, Hkv, S, 128 bytes] with the
// caller's strides, or the page pool [Hkv, pages, page_size, 128 bytes]; one
// map per box height (big: a whole tile of a dense cache or a whole page,
// 32 rows: tails).
struct TmaMaps {
  CUtensorMap k_big, v_big, k_rows32, v_rows32;
};
constexpr int kTmaNone = 0, kTmaDense = 1, kTmaPaged = 2;

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

__global__ void __launch_bounds__(kThreadsU, kCtasPerSm)
    flash_decode_i8_umma_kernel(AttnArgs a, MmaScratch x, int* status, const __grid_constant__ TmaMaps maps, int tma_mode,
                                int big_rows, const __grid_constant__ NewTokenArgs nt) {
  // The swizzled tiles need a 1024-byte aligned base.  The array is declared
  // with that alignment (and used in place, so that every access compiles to a
  // shared-memory instruction); a base that is not aligned after all is reported.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  SmemU& sm = *reinterpret_cast<SmemU*>(smem_raw);
  if ((smem_u32(smem_raw) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicExch(status, 2);
    return;
  }

  // Thread tid owns token tid of the tile in the softmax phase.  The two groups of 128
  // threads (warps 0..3, warps 4..7) own the two halves, i.e. S^T_0 and S^T_1, whose TMEM
  // lane is t = tid mod 128.  In the output phase thread (g, t) owns head-dim index t of
  // rows 4 g .. 4 g + 3.
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = tid >> 7, t = tid & (kHalfU - 1);
  const int R = a.R;
  const bool quant = a.k_scale != nullptr;
  const int cta = blockIdx.x;
#ifdef JPT_UMMA_SPANS
  if (threadIdx.x == 0 && blockIdx.x < 1024)
    for (int z = 0; z < 8; ++z) g_umma_spans[8 * blockIdx.x + z] = 0;
#endif
  JPT_SPAN(0);

  // ------------------------------------------------------------------ barriers and tensor memory
  // (warp 1; warp 0 is busy with the scan below, the barriers of the schedule publish the result)
  if (tid == 32) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sm.bar[0])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sm.bar[1])));
    for (int z = 0; z < 3; ++z) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sm.bar_in[z])));
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
  // it ran under the kernel before this one.
  grid_dependency_wait();
  grid_dependency_trigger();

  // ------------------------------------------------------------------ new token: amax to every rank
  unsigned nt_epoch = 0;
  if (nt.enabled) {
    nt_epoch = *reinterpret_cast<volatile unsigned*>(&nt.px_state[0]) + 1u;
    const int HD = a.Hkv * kD;
    for (int b = cta; b < a.B; b += gridDim.x) {
      float am[2];
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        float v = 0.f;
        for (int e = tid; e < HD; e += kThreadsU) {
          const int64_t idx = (int64_t)b * HD + e;
          const float xv = nt.in_f32 ? static_cast<const float*>(nt.x[which])[idx]
                                     : __bfloat162float(static_cast<const __nv_bfloat16*>(nt.x[which])[idx]);
          v = fmaxf(v, fabsf(xv));
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
        float m8 = sm.xch[0][tid];
#pragma unroll
        for (int w = 1; w < 8; ++w) m8 = fmaxf(m8, sm.xch[w][tid]);
        const size_t row = (size_t)(nt_epoch & 1u) * nt.px_world + nt.px_rank;
        const unsigned long long word = ((unsigned long long)nt_epoch << 32) | __float_as_uint(m8);
        for (int r = 0; r < nt.px_world; ++r)
          asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(nt.px_slots[r] + row * (2 * a.B) + tid * a.B + b), "l"(word)
                       : "memory");
      }
    }
    __syncthreads();
  }
  // Counts this CTA as done with the exchange of this launch; the last one advances the launch number.
  auto exchange_done = [&]() {
    if (nt.enabled && tid == 0) {
      __threadfence();
      const unsigned done = atomicAdd(&nt.px_state[1], 1u);
      if (done == gridDim.x - 1) {
        nt.px_state[1] = 0;
        __threadfence();
        atomicAdd(&nt.px_state[0], 1u);
      }
    }
  };

  // ------------------------------------------------------------------ schedule
  // Slots per sequence (tiles + overhead) -> exclusive prefix over sequences;
  // each of the first 128 threads owns a slice of ceil(B/128) sequences.  The scan
  // scratch aliases the probability levels, which are not in use yet.
  int* scan = reinterpret_cast<int*>(&sm.plev[0][0]);  // 129 ints
  const int per = (a.B + kThreads - 1) / kThreads;
  const int b_lo = min(a.B, t * per), b_hi = min(a.B, b_lo + per);
  if (g == 0) {
    int mine = 0;
    for (int b = b_lo; b < b_hi; ++b) {
      int ua;
      mine += slots_u(seq_range_x(a, x, b, &ua), a.S);
    }
    scan[tid] = mine;
  }
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
  const int share = (total + x.num_ctas - 1) / x.num_ctas;
  const int G0 = cta * share;
  const int G1 = min(total, G0 + share);
  if (g == 0) {
    // the thread whose slice holds slot G0 walks it and publishes (b, h, slot in segment)
    const int lo = scan[tid] * a.Hkv, hi = scan[tid + 1] * a.Hkv;
    if (G0 < G1 && G0 >= lo && G0 < hi) {
      int run = lo;
      for (int b = b_lo; b < b_hi; ++b) {
        int ua;
        const int sl = slots_u(seq_range_x(a, x, b, &ua), a.S);
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
  bool dead = false;  // a wait ran out
  // The decode step's new token of slot b, KV head h, folded into rows r0 .. r0 + kRows - 1 by
  // the 128-thread group `grp` (thread t: head-dim index t): all-ranks amax -> scale -> codes of
  // this head's row -> (group 0) cache row, scale, stash -> one more softmax term on top of
  // (M, L, acc): M[j] maximum in the log2 domain (-inf: no token yet), L[j] denominator, acc[j]
  // this thread's component of the unnormalised output.  Every thread of the group calls it.
  auto add_new_token = [&](auto rows_tag, int grp, int b, int h, int r0, float* M, float* L, float* acc) {
    constexpr int kRows = decltype(rows_tag)::value;
    group_barrier(grp);  // the group's scratch is free
    if (t < 2) {         // K amax, V amax: largest partial over the ranks
      const size_t row = (size_t)(nt_epoch & 1u) * nt.px_world;
      float m = 0.f;
      const long long t0 = clock64();
      for (int r = 0; r < nt.px_world; ++r) {
        const unsigned long long* p = nt.px_slots[nt.px_rank] + (row + r) * (2 * a.B) + t * a.B + b;
        unsigned long long w;
        for (;;) {
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
      sm.ntx[grp][t] = m;
    }
    group_barrier(grp);
    const float amax_k = sm.ntx[grp][0], amax_v = sm.ntx[grp][1];
    const float sc_k = nt.in_f32 ? decode_scale<float>(amax_k) : decode_scale<__nv_bfloat16>(amax_k);
    const float sc_v = nt.in_f32 ? decode_scale<float>(amax_v) : decode_scale<__nv_bfloat16>(amax_v);
    const int64_t xi = ((int64_t)b * a.Hkv + h) * kD + t;
    float xk, xv;
    if (nt.in_f32) {
      xk = static_cast<const float*>(nt.x[0])[xi];
      xv = static_cast<const float*>(nt.x[1])[xi];
    } else {
      xk = __bfloat162float(static_cast<const __nv_bfloat16*>(nt.x[0])[xi]);
      xv = __bfloat162float(static_cast<const __nv_bfloat16*>(nt.x[1])[xi]);
    }
    const int8_t ck = nt.in_f32 ? decode_code<float>(xk, sc_k) : decode_code<__nv_bfloat16>(xk, sc_k);
    const int8_t cv = nt.in_f32 ? decode_code<float>(xv, sc_v) : decode_code<__nv_bfloat16>(xv, sc_v);
    if (grp == 0) {
      if (nt.quant[0]) nt.quant[0][xi] = ck;
      if (nt.quant[1]) nt.quant[1][xi] = cv;
      int pos = nt.pos ? nt.pos[nt.pos_count == 1 ? 0 : b] : nt.pos_host;
      if (pos < 0) pos += a.S;
      const bool write = nt.write_cache && pos >= 0 && pos < a.S;
      if (write) {
        const int64_t off = (int64_t)b * a.kv_b + (int64_t)h * a.kv_h + (int64_t)pos * a.kv_s + t;
        static_cast<int8_t*>(const_cast<void*>(a.k))[off] = ck;
        static_cast<int8_t*>(const_cast<void*>(a.v))[off] = cv;
      }
      if (t < 2) {  // every head's CTA writes the same scale: harmless, and no CTA has to wait for another
        const float sc = t == 0 ? sc_k : sc_v;
        void* out = nt.scale_out[t];
        void* cache = const_cast<void*>(t == 0 ? a.k_scale : a.v_scale);
        const int64_t sidx = (int64_t)b * a.sc_b + (int64_t)pos * a.sc_s;
        if (nt.in_f32) {
          if (out) static_cast<float*>(out)[b] = sc;
          if (write) static_cast<float*>(cache)[sidx] = sc;
        } else {
          if (out) static_cast<__nv_bfloat16*>(out)[b] = __float2bfloat16_rn(sc);
          if (write) static_cast<__nv_bfloat16*>(cache)[sidx] = __float2bfloat16_rn(sc);
        }
      }
    }
    // logits of the query rows against the new key: sum over the 128 head-dim indices of the group
    const __nv_bfloat16* q = qbase + ((int64_t)b * a.Hkv + h) * R * kD;
    const float kf = (float)ck;
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      float d = r0 + j < R ? __bfloat162float(q[(r0 + j) * kD + t]) * kf : 0.f;
#pragma unroll
      for (int sh = 1; sh <= 16; sh <<= 1) d += __shfl_xor_sync(0xffffffffu, d, sh);
      if (lane == j) sm.dot[grp][warp & 3][j] = d;
    }
    group_barrier(grp);
    const float unit = sc_k * a.sm_scale * kLog2e;
    const float vf = (float)cv * sc_v;
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      if (r0 + j < R) {
        const float xn = ((sm.dot[grp][0][j] + sm.dot[grp][1][j]) + (sm.dot[grp][2][j] + sm.dot[grp][3][j])) * unit;
        const float mn = fmaxf(M[j], xn);
        const float al = M[j] == -INFINITY ? 0.f : ex2(M[j] - mn);
        const float pn = ex2(xn - mn);
        acc[j] = fmaf(acc[j], al, pn * vf);
        L[j] = fmaf(L[j], al, pn);
        M[j] = mn;
      }
    }
  };
  // Rows of empty sequences are nobody's tile: sequence b is handled by CTA b mod grid (at the end of
  // the CTA's life, off the path to its first tile): zero rows, or the new token alone.
  auto clear_empty_rows = [&]() {
    for (int b = cta; b < a.B; b += gridDim.x) {
      int ua;
      if (seq_range_x(a, x, b, &ua).n == 0) {
        const int64_t r0 = (int64_t)b * a.Hkv * R;
        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.o);
        if (nt.enabled) {
          for (int h = 0; h < a.Hkv; ++h) {
            float M[4], L[4], acc[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              M[j] = -INFINITY;
              L[j] = 0.f;
              acc[j] = 0.f;
            }
            add_new_token(std::integral_constant<int, 4>(), g, b, h, 4 * g, M, L, acc);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (4 * g + j < R) {
                const int64_t row = r0 + (int64_t)h * R + 4 * g + j;
                o[row * kD + t] = __float2bfloat16_rn(acc[j] / L[j]);
                if (t == 0) {
                  if (a.m) a.m[row] = M[j] * kLn2;
                  if (a.l) a.l[row] = L[j];
                }
              }
            }
          }
          continue;
        }
        for (int i = tid; i < a.Hkv * R * kD; i += kThreadsU) o[r0 * kD + i] = __float2bfloat16_rn(0.f);
        for (int i = tid; i < a.Hkv * R; i += kThreadsU) {
          if (a.m) a.m[r0 + i] = -INFINITY;
          if (a.l) a.l[r0 + i] = 0.f;
        }
      }
    }
  };
  if (G0 >= G1) {  // no tile for this CTA
    clear_empty_rows();
    exchange_done();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kTmemCols) : "memory");
    }
    return;
  }
  JPT_SPAN(2);
  // this warp's 32 lanes; the group's logits are in S^T_g
  const uint32_t tmem_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  const uint32_t tmem_s = tmem_lane + (uint32_t)(g * kColS1);
  const uint32_t tmem_o = tmem_lane + (uint32_t)(kColO + 4 * g);  // level 0 of rows 4 g ..; level 1 is 8 columns on

  const int8_t* kbase = static_cast<const int8_t*>(a.k);
  const int8_t* vbase = static_cast<const int8_t*>(a.v);
  const __nv_bfloat16* mask = static_cast<const __nv_bfloat16*>(a.mask);

  // ------------------------------------------------------------------ producer
  // Position of the next tile to fetch (uniform across the CTA) ...
  int pb = sm.start[0], ph = sm.start[1], pt, pslot = G0;  // pslot: global slot index of tile pt
  int pT, pn, pfirst, puse_add;
  // ... and what follows from it for this thread when the threads copy the rows themselves:
  // 16-byte column tid % 8 of rows tid / 8 + 32 i of a tile.  The swizzled shared-memory offset
  // of row + 32 i is that of row plus 4096 i.
  const int prow = tid >> 3, pcol = tid & 7;
  const uint32_t pdst = (uint32_t)(prow * kD + ((pcol ^ (prow & 7)) << 4));
  const bool rows_packed = !a.paged && a.kv_s == kD;  // rows of a tile kD bytes apart
  const int kv_s32 = (int)a.kv_s, sc_s32 = (int)a.sc_s;
  const int8_t *kseg, *vseg;  // segment base + this thread's column
  int64_t scseg;
  int ppos, pcnt;             // physical position of row 0 of tile pt, its valid rows
  int pfirst_cta, pparts;
  SeqRange prange;

  auto load_seq = [&]() {
    prange = seq_range_x(a, x, pb, &puse_add);
    pn = prange.n;
    pfirst = prange.first;
    pT = tiles_u(prange, a.S);
  };
  auto seg_setup = [&]() {  // pt, pslot are set
    const int64_t seg = a.paged ? (int64_t)ph * a.kv_h : (int64_t)pb * a.kv_b + (int64_t)ph * a.kv_h;
    kseg = kbase + seg + pcol * 16;
    vseg = vbase + seg + pcol * 16;
    scseg = a.paged ? 0 : (int64_t)pb * a.sc_b;
    tile_rows(prange, a.S, pt, &ppos, &pcnt);
    const int t0slot = pslot - pt;  // slot of tile 0 of this segment
    pfirst_cta = t0slot / share;
    pparts = (t0slot + pT - 1) / share - pfirst_cta + 1;
  };
  auto advance = [&]() {
    ++pslot;
    if (++pt < pT) {
      tile_rows(prange, a.S, pt, &ppos, &pcnt);
      return;
    }
    pt = 0;
    pslot += kPieceCostU;  // the overhead slots of the next segment
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
    if (v0 < kPieceCostU) {
      pslot += kPieceCostU - v0;
      pt = 0;
    } else {
      pt = v0 - kPieceCostU;
    }
    seg_setup();
  }

  float nks = 1.f, nvs = 0.f;  // scales of this thread's token in the tile fetched last
  bool first_issue = true;

  // K rows of tile pt into the K buffer, V rows into V stage `vstage`, the record into meta[mslot].
  auto issue_tile = [&](int vstage, int mslot) {
    const bool piece_start = first_issue || pt == 0;
    first_issue = false;
    if (tid == 0) {
      TileMeta mt;
      mt.b = pb; mt.h = ph; mt.t = pt; mt.T = pT; mt.n = pn; mt.first = pfirst; mt.use_add = puse_add;
      mt.first_cta = pfirst_cta; mt.parts = pparts;
      mt.pad[0] = pcnt;             // valid rows of the tile
      mt.pad[1] = ppos;             // physical position of its first row
      mt.pad[2] = pslot + 1 >= G1;  // no tile follows in this CTA's share
      sm.meta[mslot] = mt;
    }
    if (tma_mode != kTmaNone) {
      // One thread hands the rows to the copy engine: boxes of `big_rows` rows while that many
      // valid rows remain (a whole dense tile, a whole page), boxes of 32 rows for the rest.  Rows
      // of the last box past the valid ones are whatever follows in the cache (or zeros past its
      // end); their logits are masked and their probabilities are zero.
      if (tid == 0) {
        const uint32_t kbar = smem_u32(&sm.bar_in[0]), vbar = smem_u32(&sm.bar_in[1 + vstage]);
        const uint32_t k0 = smem_u32(&sm.k[0]), v0 = smem_u32(&sm.v[vstage][0]);
        const int n_big = pcnt / big_rows;
        const int n_32 = (pcnt - n_big * big_rows + 31) >> 5;
        const uint32_t bytes = (uint32_t)(n_big * big_rows + n_32 * 32) * kD;
        mbar_arrive_expect_tx(kbar, bytes);
        mbar_arrive_expect_tx(vbar, bytes);
        int r = 0;
        for (int bx = 0; bx < n_big + n_32; ++bx) {
          const bool big = bx < n_big;
          int row = ppos + r, c2 = ph, c3 = pb;
          if (tma_mode == kTmaPaged) {
            c2 = a.page_table[(int64_t)pb * a.max_pages + row / a.page_size];
            c3 = ph;
            row = row % a.page_size;
          }
          tma_load_rows(k0 + r * kD, big ? &maps.k_big : &maps.k_rows32, row, c2, c3, kbar);
          tma_load_rows(v0 + r * kD, big ? &maps.v_big : &maps.v_rows32, row, c2, c3, vbar);
          r += big ? big_rows : 32;
        }
      }
    } else {
      const uint32_t kdst = smem_u32(&sm.k[0]) + pdst;
      const uint32_t vdst = smem_u32(&sm.v[vstage][0]) + pdst;
      if (rows_packed && pcnt == kTileU) {
        // whole tile valid, rows kD bytes apart: one address per tensor
        const int64_t off = (int64_t)(ppos + prow) * kD;
        cp_async_tile_rows<0>(kdst, vdst, kseg + off, vseg + off);
      } else {
        const int passes = (pcnt + 31) >> 5;  // 32-row passes that hold a valid row
#pragma unroll 2
        for (int i = 0; i < passes; ++i) {
          const int r = prow + 32 * i;
          const bool valid = r < pcnt;
          const int pos = valid ? ppos + r : ppos;
          int64_t off;
          if (a.paged) {
            const int pg = a.page_table[(int64_t)pb * a.max_pages + pos / a.page_size];
            off = (int64_t)pg * a.kv_page + (int64_t)(pos % a.page_size) * kD;
          } else {
            off = (int64_t)pos * kv_s32;
          }
          cp_async16(kdst + 4096 * i, kseg + off, valid);
          cp_async16(vdst + 4096 * i, vseg + off, valid);
        }
      }
    }
    if (piece_start) {
      const __nv_bfloat16* q = qbase + ((int64_t)pb * a.Hkv + ph) * R * kD;
      for (int ch = tid; ch < R * 16; ch += kThreadsU) cp_async16(smem_u32(&sm.qraw[0]) + ch * 16, q + ch * 8, true);
    }
    // scales of token `tid` of the tile, consumed by this same thread
    nks = 1.f;
    nvs = 0.f;
    if (tid < pcnt) {
      nvs = 1.f;
      if (quant) {
        const int pos = ppos + tid;
        int64_t sidx;
        if (a.paged) {
          const int pg = a.page_table[(int64_t)pb * a.max_pages + pos / a.page_size];
          sidx = (int64_t)pg * a.page_size + pos % a.page_size;
        } else {
          sidx = scseg + (int64_t)pos * sc_s32;
        }
        nks = load_scale(a.k_scale, sidx, a.scale_is_f32);
        nvs = load_scale(a.v_scale, sidx, a.scale_is_f32);
      }
    }
  };
  // Fetch the next tile of the share, or mark the record as empty.
  auto produce = [&](int vstage, int mslot) {
    const bool more = pslot < G1;
    if (more) {
      issue_tile(vstage, mslot);
      advance();
    } else if (tid == 0) {
      sm.meta[mslot].t = -1;
    }
    cp_async_commit();
    return more;
  };
  // The K rows of round `round` (and everything else requested with them by the
  // threads themselves) have landed.
  auto rows_landed = [&](int round) {
    if (tma_mode != kTmaNone && !mbar_wait(smem_u32(&sm.bar_in[0]), (uint32_t)round & 1u)) dead = true;
    cp_async_wait<0>();
  };

  // ------------------------------------------------------------------ consumer state
  float m_run[8], l_run[8];  // l_run: this thread's token share of the denominators
  float o[4];                // rows 4 g .. 4 g + 3, head-dim index t
  int piece_t0 = 0;
  const float unit2 = a.sm_scale * kLog2e;
  const uint32_t bar_s = smem_u32(&sm.bar[0]), bar_o = smem_u32(&sm.bar[1]);
  const uint32_t q_desc_addr = smem_u32(&sm.qlev[0]), p_desc_addr = smem_u32(&sm.plev[0][0]);
  const uint32_t k_addr = smem_u32(&sm.k[0]);
  // this thread's byte of row 0 of its half's probability levels: chunk t / 16, byte t % 16.  Each
  // half is 1024-byte aligned, so row r's XOR with r << 4 can be applied to the whole address.
  const uint32_t p_base = smem_u32(&sm.plev[g][0]) + (t & 15) + ((uint32_t)(t >> 4) << 4);

  // Query levels of the piece that starts with the tile of record `mt` (when it
  // starts one), then S^T of that tile (one MMA group per half that holds a
  // token) on the tensor core.  Called by the whole CTA once the tile's K rows
  // have landed and a barrier has made them (and the record) visible; the
  // logits of the tile before are out of tensor memory.
  auto prepare = [&](const TileMeta& mt, bool first) {
    if (first || mt.t == 0) {
      if (g == 0) {
        // thread (row = t / 16, chunk = t % 16) converts 8 values of one query row
        const int row = t >> 4, ch = t & 15;
        float f[8];
        if (row < R) {
          const uint4 raw = *reinterpret_cast<const uint4*>(&sm.qraw[row * (kD * 2) + ch * 16]);
          const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 tt = __bfloat1622float2(p2[e]);
            f[2 * e] = tt.x;
            f[2 * e + 1] = tt.y;
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
          const float tt = f[e] * inv;
          const float h = rintf(tt);
          const float l = rintf((tt - h) * 254.f);
          hi[e >> 2] |= ((uint32_t)(int)h & 0xffu) << (8 * (e & 3));
          lo[e >> 2] |= ((uint32_t)(int)l & 0xffu) << (8 * (e & 3));
        }
        *reinterpret_cast<uint2*>(&sm.qlev[swz(row, 8 * ch)]) = make_uint2(hi[0], hi[1]);
        *reinterpret_cast<uint2*>(&sm.qlev[swz(8 + row, 8 * ch)]) = make_uint2(lo[0], lo[1]);
        if (ch == 0) {
          sm.qsc[row] = amax * (1.f / 127.f) * unit2 * (1.f / 254.f);
          sm.qsr[row] = amax * (1.f / 127.f) * (1.f / 254.f);
        }
        fence_async_smem();
      }
      tc_fence_before();
      __syncthreads();
    }
    if (tid == 0) {
      tc_fence_after();
      const bool two = mt.pad[0] > kHalfU;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_i8(tmem, umma_desc(k_addr + 32 * ks), umma_desc(q_desc_addr + 32 * ks), kIdescS, ks > 0);
      if (two) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_i8(tmem + kColS1, umma_desc(k_addr + kHalfU * kD + 32 * ks), umma_desc(q_desc_addr + 32 * ks), kIdescS,
                  ks > 0);
      }
      umma_commit(bar_s);
    }
  };
  // O^T of the tile with the given parity into the accumulators (alpha and cmax are that tile's)
  auto add_output = [&](uint32_t parity, const float (&al4)[4], float cmax) {
    if (!mbar_wait(bar_o, parity)) dead = true;
    tc_fence_after();
    uint32_t o0[4], o1[4];
    tmem_ld4(tmem_o, o0);
    tmem_ld4(tmem_o + 8, o1);
    tmem_ld_wait();
    tc_fence_before();
    const float oscale = cmax * (1.f / 65535.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = fmaf(o[j], al4[j], (float)((int)o0[j] + ((int)o1[j] << 8)) * oscale);
  };

  // The tensor core works one step ahead of the threads: S^T of tile i+1 is
  // issued at the end of iteration i, and O^T of tile i is collected in
  // iteration i+1 (at once only when tile i ends a piece), so neither MMA is
  // waited for right after it was issued.
  bool more = produce(0, 0);
  if (more) rows_landed(0);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  TileMeta mt = sm.meta[0];
  JPT_SPAN(3);
  if (mt.t >= 0) prepare(mt, true);

  float alpha_prev[4], cmax_prev = 0.f;
  bool pending = false;  // O^T of the tile before has not been added yet
  for (int i = 0; mt.t >= 0; ++i) {
    const float cks = nks, cvs = nvs;  // scales of this thread's token in this tile
    const int vstage = i & 1;
    const bool last_of_share = mt.pad[2] != 0;
    const uint32_t par = (uint32_t)i & 1u;
    const int left = mt.pad[0];            // valid rows of this tile
    const bool two = left > kHalfU;        // the second half holds a token
    const bool mine = g == 0 || two;       // this thread's half does
    if (i == 0 || mt.t == 0) {  // a piece starts (the one before was flushed when it ended)
      piece_t0 = mt.t;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        m_run[r] = kNoMax;
        l_run[r] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = 0.f;
    }

    // ---------------- the output of the tile before and the logits of this one leave
    // tensor memory in one round trip; the K buffer and the V stage of the tile before
    // are free after that
    if (!mbar_wait(bar_s, par)) dead = true;
    if (pending && !mbar_wait(bar_o, par ^ 1u)) dead = true;
    tc_fence_after();
    float xr[8];
    {
      uint32_t s[16];
      if (pending) {
        uint32_t o0[4], o1[4];
        tmem_ld4(tmem_o, o0);
        tmem_ld4(tmem_o + 8, o1);
        if (mine) tmem_ld16(tmem_s, s);
        tmem_ld_wait();
        const float oscale = cmax_prev * (1.f / 65535.f);
#pragma unroll
        for (int j = 0; j < 4; ++j)  // the two levels combine exactly in int32
          o[j] = fmaf(o[j], alpha_prev[j], (float)((int)o0[j] + ((int)o1[j] << 8)) * oscale);
        pending = false;
      } else {
        if (mine) tmem_ld16(tmem_s, s);
        tmem_ld_wait();
      }
      more = produce(vstage ^ 1, (i + 1) & 1);
      const bool valid = tid < left;
      float mk = valid ? 0.f : -INFINITY;  // a token past the end: finite dot product + (-inf)
      if (mt.use_add && valid)            // additive mask that is not a plain 0 / -inf range (rare)
        mk = __bfloat162float(mask[(int64_t)mt.b * a.mk_b + mt.pad[1] + tid]);
      if (!mine) {
#pragma unroll
        for (int r = 0; r < 8; ++r) xr[r] = -INFINITY;
      } else if (!a.round_logits) {
        const float4 q0 = *reinterpret_cast<const float4*>(&sm.qsc[0]), q1 = *reinterpret_cast<const float4*>(&sm.qsc[4]);
        const float qs[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const float ml = mk * kLog2e;
#pragma unroll
        for (int r = 0; r < 8; ++r) xr[r] = fmaf((float)((int)s[r] * 254 + (int)s[8 + r]), qs[r] * cks, ml);
      } else {
        // dense_attention on bf16 tensors: the reference rounds the logit to bf16 after every step
        const float sqrt_d = __frcp_rn(a.sm_scale);
#pragma unroll
        for (int r = 0; r < 8; ++r)
          xr[r] = kLog2e * rounded_logit((float)((int)s[r] * 254 + (int)s[8 + r]) * sm.qsr[r], sqrt_d, cks, quant, mk);
      }
    }
    // tile maxima per row (and the largest V scale) across the 256 tokens: per warp first ...
    {
      float wm[9];
#pragma unroll
      for (int r = 0; r < 8; ++r) wm[r] = warp_max(xr[r]);
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
      // ... then lane c of every warp folds column c of the 8 warps, and the lanes hand the
      // 9 results round
      const int col = lane < 9 ? lane : 8;
      float v = sm.xch[0][col];
#pragma unroll
      for (int w = 1; w < 8; ++w) v = fmaxf(v, sm.xch[w][col]);
      float tm[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) tm[r] = __shfl_sync(0xffffffffu, v, r);
      cmax = __shfl_sync(0xffffffffu, v, 8);
      // p <= 1 and the product is held at 2^16 - 1 (the fast division may land one ulp above)
      const float rc = cmax > 0.f ? __fdividef(65535.f, cmax) : 0.f;
      const float ps = fminf(cvs * rc, 65535.f);
      softmax_rows<0>(m_run, l_run, alpha, tm, xr, ps, p_base);
    }
    fence_async_smem();
    __syncthreads();

    // ---------------- O^T = V^T Pl^T on the tensor core
    if (tid == 0) {
      // V rows of this tile were requested a round ago (stage `vstage` takes rounds vstage, vstage + 2, ...)
      if (tma_mode != kTmaNone && !mbar_wait(smem_u32(&sm.bar_in[1 + vstage]), (uint32_t)(i >> 1) & 1u)) dead = true;
      tc_fence_after();
      const uint32_t v_addr = smem_u32(&sm.v[vstage][0]);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_i8(tmem + kColO, umma_desc(v_addr + 4096 * ks), umma_desc(p_desc_addr + 32 * ks), kIdescO, ks > 0);
      if (two) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_i8(tmem + kColO, umma_desc(v_addr + kHalfU * kD + 4096 * ks), umma_desc(p_desc_addr + 2048 + 32 * ks),
                  kIdescO, 1u);
      }
      umma_commit(bar_o);
    }

    float al4[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) al4[j] = g == 0 ? alpha[j] : alpha[4 + j];
    if (!(last_of_share || mt.t == mt.T - 1)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) alpha_prev[j] = al4[j];
      cmax_prev = cmax;
      pending = true;
    } else {
      // ---------------- end of a piece: write the rows, or a partial for the merge
      const bool is_final = piece_t0 == 0 && mt.t == mt.T - 1;
      const int slot = piece_t0 > 0 ? 0 : 1;
      const int64_t row_base = ((int64_t)mt.b * a.Hkv + mt.h) * R;
      // denominators: sum the token shares of the 256 threads (while the last O^T MMA runs)
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        float l = l_run[r];
#pragma unroll
        for (int sh = 1; sh <= 16; sh <<= 1) l += __shfl_xor_sync(0xffffffffu, l, sh);
        if (lane == r) sm.red[warp][r] = l;
      }
      __syncthreads();
      add_output(par, al4, cmax);
      float L4[4], M4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = 4 * g + j;
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) L += sm.red[w][r];
        L4[j] = L;
        const float mr = g == 0 ? m_run[j] : m_run[4 + j];
        M4[j] = mr > 0.5f * kNoMax ? mr : -INFINITY;  // every logit of the row was masked
      }
      if (is_final && nt.enabled) add_new_token(std::integral_constant<int, 4>(), g, mt.b, mt.h, 4 * g, M4, L4, o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = 4 * g + j;
        if (r < R) {
          const float L = L4[j], M = M4[j];
          if (is_final) {
            const int64_t row = row_base + r;
            static_cast<__nv_bfloat16*>(a.o)[row * kD + t] = __float2bfloat16_rn(L > 0.f ? o[j] / L : 0.f);
            if (t == 0) {
              if (a.m) a.m[row] = M * kLn2;
              if (a.l) a.l[row] = L > 0.f ? L : 0.f;
            }
          } else {
            const int64_t pr = ((int64_t)cta * 2 + slot) * kMaxRows + r;
            __stcg(&x.part_o[pr * kD + t], o[j]);
            if (t == 0) {
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
        __threadfence();
        __syncthreads();
        if (tid == 0) {
          const unsigned old = atomicInc(&x.counters[mt.b * a.Hkv + mt.h], (unsigned)(mt.parts - 1));
          sm.flag = old == (unsigned)(mt.parts - 1);
        }
        __syncthreads();
        if (sm.flag && g == 0) {  // the first 128 threads merge (thread t: head-dim index t of all rows)
          __threadfence();
          // the O^T MMA of this tile is complete, so its V stage (32 KB) is free; the next
          // tile's V rows go to the other stage
          float* scratch = reinterpret_cast<float*>(&sm.v[vstage][0]);
          if (nt.enabled) {
            const int hb = mt.b, hh = mt.h;
            merge_segment<true>(a, x, mt.first_cta, mt.parts, row_base, scratch,
                                [&](float* sM, float* sL, float (&acc)[kMaxRows]) {
                                  float M8[8], L8[8], a8[8];
#pragma unroll
                                  for (int r = 0; r < 8; ++r) {
                                    M8[r] = sM[r];
                                    L8[r] = sL[r];
                                    a8[r] = acc[r];
                                  }
                                  add_new_token(std::integral_constant<int, 8>(), 0, hb, hh, 0, M8, L8, a8);
#pragma unroll
                                  for (int r = 0; r < 8; ++r) acc[r] = a8[r];
                                  group_sync<true>();  // every thread has read sM / sL
                                  if (t < 8) {
                                    sM[t] = M8[t];
                                    sL[t] = L8[t];
                                  }
                                  group_sync<true>();
                                });
          } else {
            merge_segment<true>(a, x, mt.first_cta, mt.parts, row_base, scratch);
          }
        }
      }
    }

    // ---------------- the next tile: its rows have had the iteration to land
    if (more) rows_landed(i + 1);
    fence_async_smem();
    tc_fence_before();
    if (__syncthreads_or(dead)) {
      if (tid == 0) atomicExch(status, 1);
      // give a copy-engine request that may still be in flight its (bounded) time to finish
      if (more && tma_mode != kTmaNone) {
        mbar_wait(smem_u32(&sm.bar_in[0]), (uint32_t)(i + 1) & 1u);
        mbar_wait(smem_u32(&sm.bar_in[1 + ((i + 1) & 1)]), (uint32_t)((i + 1) >> 1) & 1u);
      }
      break;
    }
    mt = sm.meta[(i + 1) & 1];
    if (mt.t >= 0) prepare(mt, false);
    if (i == 0) JPT_SPAN(4);
#ifdef JPT_UMMA_SPANS
    if (threadIdx.x == 0 && blockIdx.x < 1024) g_umma_spans[8 * blockIdx.x + 6] += 1;  // tiles
#endif
  }
  JPT_SPAN(5);
  clear_empty_rows();
  exchange_done();
  cp_async_wait<0>();  // (a copy-engine request is never left in flight: every issued tile was waited for)
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kTmemCols) : "memory");
  }
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
  int mode, big_rows, device;
  bool operator==(const MapKey& o) const {
    return k == o.k && v == o.v && d1 == o.d1 && d2 == o.d2 && d3 == o.d3 && s0 == o.s0 && s1 == o.s1 && s2 == o.s2 &&
           mode == o.mode && big_rows == o.big_rows && device == o.device;
  }
};
struct MapEntry {
  MapKey key;
  TmaMaps maps;
};

// Tensor maps for this call (cached per tensor pair and geometry); kTmaNone when
// the layout cannot be described (the kernel then copies the rows with its threads).
int tensor_maps_for(const jpt_attn_params& p, TmaMaps* out, int* big_rows) {
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
    if (p.page_size % 32 != 0 || p.kv_page != (int64_t)p.page_size * kD || p.kv_h <= 0 || p.kv_h % p.kv_page != 0) return kTmaNone;
    if ((kTileU % p.page_size) != 0 && (p.page_size % kTileU) != 0) return kTmaNone;
    key.mode = kTmaPaged;
    key.big_rows = p.page_size < kTileU ? p.page_size : kTileU;
    key.d1 = p.page_size; key.d2 = p.kv_h / p.kv_page; key.d3 = p.Hkv;
    key.s0 = kD; key.s1 = p.kv_page; key.s2 = p.kv_h;
  } else {
    key.mode = kTmaDense;
    key.big_rows = kTileU;
    key.d1 = p.S; key.d2 = p.Hkv; key.d3 = p.B;
    key.s0 = p.kv_s; key.s1 = p.kv_h; key.s2 = p.kv_b;
    if (p.Hkv == 1 && key.s1 <= 0) key.s1 = key.s0 * p.S;  // a single head: its stride is never used
    if (p.B == 1 && key.s2 <= 0) key.s2 = key.s1 * p.Hkv;
  }
  if (key.s0 % 16 || key.s1 % 16 || key.s2 % 16 || key.s0 < kD || key.s1 <= 0 || key.s2 <= 0) return kTmaNone;
  if (!aligned(p.k, 16) || !aligned(p.v, 16)) return kTmaNone;
  *big_rows = key.big_rows;
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
  if (!encode_rows_map(&e.maps.k_big, p.k, dims, str, key.big_rows) || !encode_rows_map(&e.maps.v_big, p.v, dims, str, key.big_rows) ||
      !encode_rows_map(&e.maps.k_rows32, p.k, dims, str, 32) || !encode_rows_map(&e.maps.v_rows32, p.v, dims, str, 32))
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
  static std::atomic<bool> configured[kMaxDevices];
  if (int rc = configure_once_per_device(configured, "flash_decode_i8_umma_kernel", [] {
        cudaError_t e = cudaFuncSetAttribute(flash_decode_i8_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             smem_bytes);
        if (e == cudaSuccess)  // two CTAs of 105 KB per SM
          e = cudaFuncSetAttribute(flash_decode_i8_umma_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   (int)cudaSharedmemCarveoutMaxShared);
        return e;
      }))
    return rc;
  if (a.mask_mode == JPT_MASK_ADD) {
    if (int rc = launch_mask_ranges(a, x, st)) return rc;
  }
  TmaMaps maps;
  memset(&maps, 0, sizeof(maps));
  int big_rows = kTileU;
  const int tma_mode = tensor_maps_for(p, &maps, &big_rows);
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
  launch_after_previous(flash_decode_i8_umma_kernel, dim3(lay.num_ctas), dim3(kThreadsU), smem_bytes, st, a, x, status, maps,
                        tma_mode, big_rows, nt);
  return check_launch("flash_decode_i8_umma_kernel");
}

}  // namespace jpt

#ifdef JPT_UMMA_SPANS
extern "C" int jpt_debug_umma_spans(unsigned long long* out_host, int n_ctas) {
  return (int)cudaMemcpyFromSymbol(out_host, jpt::g_umma_spans, sizeof(unsigned long long) * 8 * n_ctas);
}
#endif
