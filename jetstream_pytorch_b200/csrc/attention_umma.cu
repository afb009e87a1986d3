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
// tiles are scheduled exactly as in the mma.sync kernel (equal contiguous
// shares of one global tile list, pieces, last-arriver merge).  K and V rows
// of a tile land in shared memory as 128-byte rows, 16-byte chunks XORed with
// (row & 7): that is the canonical 128-byte-swizzle layout of the tensor core
// for both operand roles (K-major for K, MN-major for V), so nothing is
// rearranged.  In the softmax phase thread t owns token t of the tile (TMEM
// lane t of S^T); in the output phase thread t owns head-dim index t (TMEM
// lane t of O^T), which also removes the cross-warp merge of the accumulators.
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
#include <string.h>

#include <type_traits>

#include "attention_tiles.cuh"

namespace jpt {
namespace {

constexpr int kTileU = 128;     // tokens per tile = TMEM lanes = threads per CTA
constexpr int kStagesU = 2;     // K/V ring depth
constexpr int kTmemCols = 32;   // S^T: columns 0..15, O^T: columns 16..31
constexpr int kColO = 16;
constexpr int kCtasPerSm = 3;
#ifndef JPT_PIECE_COST_U
#define JPT_PIECE_COST_U 1
#endif
constexpr int kPieceCostU = JPT_PIECE_COST_U;  // overhead slots charged per segment, in 128-token tiles
constexpr long long kWaitCycles = 1000000000ll;  // about half a second: far beyond any wait of a healthy run
constexpr int kMaxPartsU = 250;  // pieces of one segment the in-kernel merge can hold in its 16 KB of scratch

struct __align__(1024) SmemU {
  uint8_t kv[kStagesU][2][kTileU * kD];  // [stage][K, V][token][128 bytes], swizzled
  uint8_t qlev[16 * kD];                 // query levels: rows 0..7 high bytes, 8..15 low bytes
  uint8_t plev[16 * kTileU];             // probability levels: row 8 l + r, one byte per token
  uint8_t qraw[8 * kD * 2];              // bf16 query rows of the piece whose first tile is in flight
  float xch[4][12];                      // per warp: row maxima of the tile [8], largest V scale [1]
  float red[4][8];                       // per warp: denominators at the end of a piece
  float qsc[8];                          // s_r * sm_scale * log2(e) / 254
  float qsr[8];                          // s_r / 254 (the chain of rounded logits starts from the plain dot product)
  float ntx[4];                          // new token: K amax, V amax
  float dot[4][8];                       // new token, per warp: partial logits of the 8 rows
  uint64_t bar[2];                       // MMA completion: S^T, O^T
  uint32_t tmem_base;
  int start[3];
  int flag;
  TileMeta meta[kStagesU];
};

// 16-byte copy with compile-time offsets on both addresses (one pair of base registers per tensor)
template <int kOff>
__device__ __forceinline__ void cp_async16_at(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0 + %2], [%1 + %2], 16;\n" ::"r"(dst), "l"(src), "n"(kOff));
}
template <int kI>
__device__ __forceinline__ void cp_async_tile_rows(uint32_t kdst, uint32_t vdst, const void* kp, const void* vp) {
  if constexpr (kI < 8) {
    cp_async16_at<2048 * kI>(kdst, kp);
    cp_async16_at<2048 * kI>(vdst, vp);
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
                                             const float (&xv)[8], float ps, uint32_t p_base) {
  if constexpr (kRow < 8) {
    const float mn = fmaxf(m_run[kRow], tm[kRow]);
    const float al = ex2(m_run[kRow] - mn);
    const float p = ex2(xv[kRow] - mn);
    alpha[kRow] = al;
    m_run[kRow] = mn;
    l_run[kRow] = fmaf(l_run[kRow], al, p);
    // the byte of row r: 16-byte chunk (t / 16) ^ r of that row (the XOR folds into the address)
    store_levels<128 * kRow>(p_base ^ (uint32_t)(kRow << 4), __float2uint_rn(p * ps));
    softmax_rows<kRow + 1>(m_run, l_run, alpha, tm, xv, ps, p_base);
  }
}
__device__ __forceinline__ int tiles_u(int n) { return (n + kTileU - 1) / kTileU; }
__device__ __forceinline__ int slots_u(int n) { return n > 0 ? tiles_u(n) + kPieceCostU : 0; }

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

// kFused = the launch carries the decode step's new token, kRound = dense_attention's rounded logit chain.
template <bool kFused, bool kRound>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
    flash_decode_i8_umma_kernel(const __grid_constant__ AttnArgs a, const __grid_constant__ MmaScratch x, int* status,
                                const __grid_constant__ NewTokenArgs nt) {
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

  // ------------------------------------------------------------------ new token: amax to every rank
  unsigned nt_epoch = 0;
  if constexpr (kFused) {
    nt_epoch = *reinterpret_cast<volatile unsigned*>(&nt.px_state[0]) + 1u;
    const int HD = a.Hkv * kD;
    for (int b = cta; b < a.B; b += gridDim.x) {
      float am[2];
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        float v = 0.f;
        for (int e = tid; e < HD; e += kThreads) {
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
        const float m4 = fmaxf(fmaxf(sm.xch[0][tid], sm.xch[1][tid]), fmaxf(sm.xch[2][tid], sm.xch[3][tid]));
        const size_t row = (size_t)(nt_epoch & 1u) * nt.px_world + nt.px_rank;
        const unsigned long long word = ((unsigned long long)nt_epoch << 32) | __float_as_uint(m4);
        for (int r = 0; r < nt.px_world; ++r)
          asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(nt.px_slots[r] + row * (2 * a.B) + tid * a.B + b), "l"(word)
                       : "memory");
      }
    }
    __syncthreads();
  }
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
    mine += slots_u(seq_range_x(a, x, b, &ua).n);
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
  const int share = (total + x.num_ctas - 1) / x.num_ctas;
  const int G0 = cta * share;
  const int G1 = min(total, G0 + share);
  {
    // the thread whose slice holds slot G0 walks it and publishes (b, h, slot in segment)
    const int lo = scan[tid] * a.Hkv, hi = scan[tid + 1] * a.Hkv;
    if (G0 < G1 && G0 >= lo && G0 < hi) {
      int run = lo;
      for (int b = b_lo; b < b_hi; ++b) {
        int ua;
        const int sl = slots_u(seq_range_x(a, x, b, &ua).n);
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
  // The decode step's new token of slot b, KV head h, folded into the 8 rows of the segment by the
  // whole CTA (thread tid: head-dim index tid): all-ranks amax -> scale -> codes of this head's row
  // -> cache row, scale, stash -> one more softmax term on top of (M, L, acc): M[r] maximum in the
  // log2 domain (-inf: no token yet), L[r] denominator, acc[r] this thread's component of the
  // unnormalised output.  Every thread of the CTA calls it.
  auto add_new_token = [&](int b, int h, float* M, float* L, float* acc) {
    __syncthreads();  // the scratch is free
    if (tid < 2) {    // K amax, V amax: largest partial over the ranks
      const size_t row = (size_t)(nt_epoch & 1u) * nt.px_world;
      float m = 0.f;
      const long long t0 = clock64();
      for (int r = 0; r < nt.px_world; ++r) {
        const unsigned long long* p = nt.px_slots[nt.px_rank] + (row + r) * (2 * a.B) + tid * a.B + b;
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
      sm.ntx[tid] = m;
    }
    __syncthreads();
    const float amax_k = sm.ntx[0], amax_v = sm.ntx[1];
    const float sc_k = nt.in_f32 ? decode_scale<float>(amax_k) : decode_scale<__nv_bfloat16>(amax_k);
    const float sc_v = nt.in_f32 ? decode_scale<float>(amax_v) : decode_scale<__nv_bfloat16>(amax_v);
    const int64_t xi = ((int64_t)b * a.Hkv + h) * kD + tid;
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
    {
      if (nt.quant[0]) nt.quant[0][xi] = ck;
      if (nt.quant[1]) nt.quant[1][xi] = cv;
      int pos = nt.pos ? nt.pos[nt.pos_count == 1 ? 0 : b] : nt.pos_host;
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
    }
    // logits of the query rows against the new key: sum over the 128 head-dim indices
    const __nv_bfloat16* q = qbase + ((int64_t)b * a.Hkv + h) * R * kD;
    const float kf = (float)ck;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float d = j < R ? __bfloat162float(q[j * kD + tid]) * kf : 0.f;
#pragma unroll
      for (int sh = 1; sh <= 16; sh <<= 1) d += __shfl_xor_sync(0xffffffffu, d, sh);
      if (lane == j) sm.dot[warp][j] = d;
    }
    __syncthreads();
    const float unit = sc_k * a.sm_scale * kLog2e;
    const float vf = (float)cv * sc_v;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < R) {
        const float xn = ((sm.dot[0][j] + sm.dot[1][j]) + (sm.dot[2][j] + sm.dot[3][j])) * unit;
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
        if constexpr (kFused) {
          for (int h = 0; h < a.Hkv; ++h) {
            float M[8], L[8], acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              M[j] = -INFINITY;
              L[j] = 0.f;
              acc[j] = 0.f;
            }
            add_new_token(b, h, M, L, acc);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (j < R) {
                const int64_t row = r0 + (int64_t)h * R + j;
                o[row * kD + tid] = __float2bfloat16_rn(acc[j] / L[j]);
                if (tid == 0) {
                  if (a.m) a.m[row] = M[j] * kLn2;
                  if (a.l) a.l[row] = L[j];
                }
              }
            }
          }
        } else {
          for (int i = tid; i < a.Hkv * R * kD; i += kThreads) o[r0 * kD + i] = __float2bfloat16_rn(0.f);
          for (int i = tid; i < a.Hkv * R; i += kThreads) {
            if (a.m) a.m[r0 + i] = -INFINITY;
            if (a.l) a.l[r0 + i] = 0.f;
          }
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
  const uint32_t tmem_lane = tmem + ((uint32_t)(warp * 32) << 16);  // this warp's 32 lanes

  const int8_t* kbase = static_cast<const int8_t*>(a.k);
  const int8_t* vbase = static_cast<const int8_t*>(a.v);
  const __nv_bfloat16* mask = static_cast<const __nv_bfloat16*>(a.mask);

  // ------------------------------------------------------------------ producer
  // Position of the next tile to fetch (uniform across the CTA) ...
  int pb = sm.start[0], ph = sm.start[1], pt, pslot = G0;  // pslot: global slot index of tile pt
  int pT, pn, pfirst, puse_add;
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
  const int8_t *kseg, *vseg;  // segment base + this thread's column
  int64_t scseg;
  int ppos;                   // physical position of row 0 of tile pt
  int pfirst_cta, pparts;

  auto load_seq = [&]() {
    const SeqRange r = seq_range_x(a, x, pb, &puse_add);
    pn = r.n;
    pfirst = r.first;
    pT = tiles_u(r.n);
  };
  auto seg_setup = [&]() {  // pt, pslot are set
    const int64_t seg = a.paged ? (int64_t)ph * a.kv_h : (int64_t)pb * a.kv_b + (int64_t)ph * a.kv_h;
    kseg = kbase + seg + pcol * 16;
    vseg = vbase + seg + pcol * 16;
    scseg = a.paged ? 0 : (int64_t)pb * a.sc_b;
    ppos = pfirst + pt * kTileU;
    if (ppos >= a.S) ppos -= a.S;
    const int t0slot = pslot - pt;  // slot of tile 0 of this segment
    pfirst_cta = t0slot / share;
    pparts = (t0slot + pT - 1) / share - pfirst_cta + 1;
  };
  auto advance = [&]() {
    ++pslot;
    ppos += kTileU;
    if (ppos >= a.S) ppos -= a.S;
    if (++pt < pT) return;
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

  auto issue_tile = [&](int stage) {
    const int j0 = pt * kTileU;
    const bool piece_start = first_issue || pt == 0;
    first_issue = false;
    if (tid == 0) {
      TileMeta mt;
      mt.b = pb; mt.h = ph; mt.t = pt; mt.T = pT; mt.n = pn; mt.first = pfirst; mt.use_add = puse_add;
      mt.first_cta = pfirst_cta; mt.parts = pparts;
      mt.pad[0] = mt.pad[1] = 0;
      mt.pad[2] = pslot + 1 >= G1;  // no tile follows in this CTA's share
      sm.meta[stage] = mt;
    }
    const uint32_t kdst = smem_u32(&sm.kv[stage][0][0]) + pdst;
    const uint32_t vdst = smem_u32(&sm.kv[stage][1][0]) + pdst;
    if (rows_packed && j0 + kTileU <= pn && ppos + kTileU <= a.S) {
      // whole tile valid, no ring wrap, rows kD bytes apart: one address per tensor
      const int64_t off = (int64_t)(ppos + prow) * kD;
      const int8_t* kp = kseg + off;
      const int8_t* vp = vseg + off;
      cp_async_tile_rows<0>(kdst, vdst, kp, vp);
    } else if (pass_pages) {
      // paged caches start at position 0: pass i (rows 16 i ..) lies inside one page
      int pi = j0 / a.page_size, within = (j0 % a.page_size) / 16;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const bool valid = j0 + 16 * i + prow < pn;
        const int page = (j0 + 16 * i) < pn ? a.page_table[(int64_t)pb * a.max_pages + pi] : 0;
        const int64_t off = (int64_t)page * a.kv_page + (int64_t)(within * 16 + prow) * kD;
        cp_async16(kdst + 2048 * i, kseg + off, valid);
        cp_async16(vdst + 2048 * i, vseg + off, valid);
        if (++within == passes_per_page) {
          within = 0;
          ++pi;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = prow + 16 * i;
        const bool valid = j0 + r < pn;
        int pos = valid ? ppos + r : ppos;
        if (pos >= a.S) pos -= a.S;
        int64_t off;
        if (a.paged) {
          const int pg = a.page_table[(int64_t)pb * a.max_pages + pos / a.page_size];
          off = (int64_t)pg * a.kv_page + (int64_t)(pos % a.page_size) * kD;
        } else {
          off = (int64_t)pos * kv_s32;
        }
        cp_async16(kdst + 2048 * i, kseg + off, valid);
        cp_async16(vdst + 2048 * i, vseg + off, valid);
      }
    }
    if (piece_start) {
      const __nv_bfloat16* q = qbase + ((int64_t)pb * a.Hkv + ph) * R * kD;
      for (int ch = tid; ch < R * 16; ch += kThreads) cp_async16(smem_u32(&sm.qraw[0]) + ch * 16, q + ch * 8, true);
    }
    // scales of token `tid` of the tile, consumed by this same thread
    nks = 1.f;
    nvs = 0.f;
    if (j0 + tid < pn) {
      nvs = 1.f;
      if (quant) {
        int pos = ppos + tid;
        if (pos >= a.S) pos -= a.S;
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
  // Fetch the next tile of the share into `stage`, or mark the stage as empty.
  auto produce = [&](int stage) {
    if (pslot < G1) {
      issue_tile(stage);
      advance();
    } else if (tid == 0) {
      sm.meta[stage].t = -1;
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

  // Query levels of the piece that starts with the tile in `st` (when it
  // starts one), then S^T of that tile on the tensor core.  Called by the whole
  // CTA once the tile's rows have landed and a barrier has made them (and the
  // record) visible; the logits of the tile before are out of tensor memory.
  auto prepare = [&](int st, const TileMeta& mt, bool first) {
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
    if (tid == 0) {
      tc_fence_after();
      const uint32_t k_addr = smem_u32(&sm.kv[st][0][0]);
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
    for (int r = 0; r < 8; ++r)  // the two levels combine exactly in int32
      o[r] = fmaf(o[r], alpha[r], (float)((int)o01[r] + ((int)o01[8 + r] << 8)) * oscale);
  };

  // The tensor core works one step ahead of the threads: S^T of tile i+1 is
  // issued at the end of iteration i, and O^T of tile i is collected in
  // iteration i+1 (at once only when tile i ends a piece), so neither MMA is
  // waited for right after it was issued.
  produce(0);
  cp_async_wait<0>();
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  TileMeta mt = sm.meta[0];
  JPT_SPAN(3);
  if (mt.t >= 0) prepare(0, mt, true);

  float alpha_prev[8], cmax_prev = 0.f;
  bool pending = false;  // O^T of the tile before has not been added yet
  int stage = 0;
  for (int i = 0; mt.t >= 0; ++i) {
    const float cks = nks, cvs = nvs;  // scales of this thread's token in the tile of `stage`
    const int next_stage = stage ^ 1;
    const bool last_of_share = mt.pad[2] != 0;
    const uint32_t par = (uint32_t)i & 1u;
    if (i == 0 || mt.t == 0) {  // a piece starts (the one before was flushed when it ended)
      piece_t0 = mt.t;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        m_run[r] = kNoMax;
        l_run[r] = 0.f;
        o[r] = 0.f;
      }
    }

    // ---------------- the output of the tile before and the logits of this one leave
    // tensor memory in one round trip; the stage of the tile before is free after that
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
        for (int r = 0; r < 8; ++r)  // the two levels combine exactly in int32 (|O_0 + 256 O_1| < 2^31)
          o[r] = fmaf(o[r], alpha_prev[r], (float)((int)o01[r] + ((int)o01[8 + r] << 8)) * oscale);
        pending = false;
      } else {
        tmem_ld16(tmem_lane, s);
        tmem_ld_wait();
      }
      produce(next_stage);
      const bool valid = mt.t * kTileU + tid < mt.n;
      float mk = valid ? 0.f : -INFINITY;  // a token past the end: finite dot product + (-inf)
      if (mt.use_add && valid) {  // additive mask that is not a plain 0 / -inf range (rare)
        SeqRange rg;
        rg.n = mt.n;
        rg.first = mt.first;
        mk = __bfloat162float(mask[(int64_t)mt.b * a.mk_b + physical_pos(a, rg, mt.t * kTileU + tid)]);
      }
      if constexpr (!kRound) {
        const float4 q0 = *reinterpret_cast<const float4*>(&sm.qsc[0]), q1 = *reinterpret_cast<const float4*>(&sm.qsc[4]);
        const float qc[8] = {q0.x * cks, q0.y * cks, q0.z * cks, q0.w * cks, q1.x * cks, q1.y * cks, q1.z * cks, q1.w * cks};
        const float ml = mk * kLog2e;
#pragma unroll
        for (int r = 0; r < 8; ++r) xv[r] = fmaf((float)((int)s[r] * 254 + (int)s[8 + r]), qc[r], ml);
      } else {
        // dense_attention on bf16 tensors: the reference rounds the logit to bf16 after every step
        const float sqrt_d = __frcp_rn(a.sm_scale);
#pragma unroll
        for (int r = 0; r < 8; ++r)
          xv[r] = kLog2e * rounded_logit((float)((int)s[r] * 254 + (int)s[8 + r]) * sm.qsr[r], sqrt_d, cks, quant, mk);
      }
    }
    // tile maxima per row (and the largest V scale) across the 128 tokens
    {
      float wm[9];
#pragma unroll
      for (int r = 0; r < 8; ++r) wm[r] = warp_max(xv[r]);
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
      softmax_rows<0>(m_run, l_run, alpha, tm, xv, ps, p_base);
    }
    fence_async_smem();
    __syncthreads();

    // ---------------- O^T = V^T Pl^T on the tensor core
    if (tid == 0) {
      tc_fence_after();
      const uint32_t v_addr = smem_u32(&sm.kv[stage][1][0]);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_i8(tmem + kColO, umma_desc(v_addr + 4096 * ks), umma_desc(p_desc_addr + 32 * ks), kIdescO, ks > 0);
      umma_commit(bar_o);
    }

    if (!(last_of_share || mt.t == mt.T - 1)) {
#pragma unroll
      for (int r = 0; r < 8; ++r) alpha_prev[r] = alpha[r];
      cmax_prev = cmax;
      pending = true;
    } else {
      // ---------------- end of a piece: write the rows, or a partial for the merge
      const bool is_final = piece_t0 == 0 && mt.t == mt.T - 1;
      const int slot = piece_t0 > 0 ? 0 : 1;
      const int64_t row_base = ((int64_t)mt.b * a.Hkv + mt.h) * R;
      // denominators: sum the token shares of the 128 threads (while the last O^T MMA runs)
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        float l = l_run[r];
#pragma unroll
        for (int sh = 1; sh <= 16; sh <<= 1) l += __shfl_xor_sync(0xffffffffu, l, sh);
        if (lane == r) sm.red[warp][r] = l;
      }
      __syncthreads();
      add_output(par, alpha, cmax);
      float L8[8], M8[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        L8[r] = (sm.red[0][r] + sm.red[1][r]) + (sm.red[2][r] + sm.red[3][r]);
        M8[r] = m_run[r] > 0.5f * kNoMax ? m_run[r] : -INFINITY;  // every logit of the row was masked
      }
      if constexpr (kFused) {
        if (is_final) add_new_token(mt.b, mt.h, M8, L8, o);
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
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
        __threadfence();
        __syncthreads();
        if (tid == 0) {
          const unsigned old = atomicInc(&x.counters[mt.b * a.Hkv + mt.h], (unsigned)(mt.parts - 1));
          sm.flag = old == (unsigned)(mt.parts - 1);
        }
        __syncthreads();
        if (sm.flag) {
          __threadfence();
          // both MMAs of this stage are complete, so its K rows (16 KB) are free
          float* scratch = reinterpret_cast<float*>(&sm.kv[stage][0][0]);
          if constexpr (kFused) {
            const int hb = mt.b, hh = mt.h;
            merge_segment<false>(a, x, mt.first_cta, mt.parts, row_base, scratch,
                                 [&](float* sM, float* sL, float (&acc)[kMaxRows]) {
                                   float Mh[8], Lh[8], ah[8];
#pragma unroll
                                   for (int r = 0; r < 8; ++r) {
                                     Mh[r] = sM[r];
                                     Lh[r] = sL[r];
                                     ah[r] = acc[r];
                                   }
                                   add_new_token(hb, hh, Mh, Lh, ah);  // (its first barrier: every thread has read sM / sL)
#pragma unroll
                                   for (int r = 0; r < 8; ++r) acc[r] = ah[r];
                                   if (tid < 8) {
                                     sM[tid] = Mh[tid];
                                     sL[tid] = Lh[tid];
                                   }
                                   __syncthreads();
                                 });
          } else {
            merge_segment<false>(a, x, mt.first_cta, mt.parts, row_base, scratch);
          }
        }
      }
    }

    // ---------------- the next tile: its rows have had the iteration to land
    cp_async_wait<0>();
    fence_async_smem();
    tc_fence_before();
    if (__syncthreads_or(dead)) {
      if (tid == 0) atomicExch(status, 1);
      break;
    }
    mt = sm.meta[next_stage];
    if (mt.t >= 0) prepare(next_stage, mt, false);
    stage = next_stage;
    if (i == 0) JPT_SPAN(4);
#ifdef JPT_UMMA_SPANS
    if (threadIdx.x == 0 && blockIdx.x < 1024) {
      g_umma_spans[8 * blockIdx.x + 6] += 1;                                  // tiles
      if (i == 0 || sm.meta[stage ^ 1].t >= 0) g_umma_spans[8 * blockIdx.x + 7] += (mt.t == 0);  // pieces started after the first
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
}

int umma_num_ctas() { return sm_count() * kCtasPerSm; }

}  // namespace

bool attention_umma_eligible(const jpt_attn_params& p) {
  const int R = (p.Hq / p.Hkv) * p.Tq;
  // the merge of a segment's pieces keeps (pieces + 4) * 16 floats in its scratch; a segment spans at most
  // its tiles + 1 CTAs
  const int max_tiles = (p.S + kTileU - 1) / kTileU;
  return attention_mma_eligible(p) && p.kv_dtype == JPT_INT8 && R <= 8 && max_tiles + 1 <= kMaxPartsU;
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
        cudaError_t e = cudaSuccess;
        auto set = [&e](auto kernel) {  // three CTAs of 73 KB per SM
          if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
          if (e == cudaSuccess)
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        };
        set(flash_decode_i8_umma_kernel<false, false>);
        set(flash_decode_i8_umma_kernel<false, true>);
        set(flash_decode_i8_umma_kernel<true, false>);
        set(flash_decode_i8_umma_kernel<true, true>);
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
  const bool fused = nt.enabled != 0, round = a.round_logits != 0;
  const dim3 grid(lay.num_ctas), block(kThreads);
  if (fused && round) launch_after_previous(flash_decode_i8_umma_kernel<true, true>, grid, block, smem_bytes, st, a, x, status, nt);
  else if (fused) launch_after_previous(flash_decode_i8_umma_kernel<true, false>, grid, block, smem_bytes, st, a, x, status, nt);
  else if (round) launch_after_previous(flash_decode_i8_umma_kernel<false, true>, grid, block, smem_bytes, st, a, x, status, nt);
  else launch_after_previous(flash_decode_i8_umma_kernel<false, false>, grid, block, smem_bytes, st, a, x, status, nt);
  return check_launch("flash_decode_i8_umma_kernel");
}

}  // namespace jpt

#ifdef JPT_UMMA_SPANS
extern "C" int jpt_debug_umma_spans(unsigned long long* out_host, int n_ctas) {
  return (int)cudaMemcpyFromSymbol(out_host, jpt::g_umma_spans, sizeof(unsigned long long) * 8 * n_ctas);
}
#endif
