// Ragged flash-decode attention for head_dim 128 and int8 caches on tensor
// cores (sm_100a): a persistent, work-balanced kernel plus a small merge kernel.
//
// Work model.  A "tile" is 64 consecutive valid tokens of one (sequence, KV
// head) segment.  All tiles of all segments form one global list ordered by
// (sequence, head, tile); every CTA of the persistent grid takes an equal,
// contiguous share of that list, so ragged lengths cost nothing in balance.
// A CTA therefore works on a run of "pieces" (its share cut at segment
// borders).  A piece that covers its whole segment is written out as final
// rows; the at most two pieces per CTA that do not (the first and the last
// one) go to a per-CTA scratch slot and are combined by the merge kernel,
// which also writes the rows of empty sequences.
//
// Data path.  K and V tiles travel global -> shared memory as 16-byte cp.async
// copies through a 3-stage ring that keeps running across piece borders; the
// query rows of a piece ride in the stage of its first tile.  Each of the four
// warps owns 16 tokens of a tile and keeps a private online-softmax state for
// the query rows of the KV group (rep * Tq <= 16).  Tokens are the M dimension
// of mma.sync.m16n8k16 and the grouped query rows the N dimension:
//   S^T[16 tok x 8 rows] = K[16 tok x 16 d] . Q^T        (8 k-steps over d)
//   O^T[16 d  x 8 rows] += V^T[16 d x 16 tok] . P^T      (8 m-tiles over d)
// so 8 grouped rows fill N exactly.  P^T moves from the accumulator layout to
// the B-operand layout with two movmatrix transposes.
//
// int8 -> fp16 without convert instructions: (x ^ 0x80) is x + 128 as an
// unsigned byte and 0x6400 | byte is the fp16 number 1024 + byte, so one PRMT
// yields two halves worth x + 1152.  For K the offset is taken out after the
// dot product (S - 1152 * sum_d q_d, exact enough in fp32); for V one HSUB2
// removes it so the accumulators only ever hold the signal.  Contraction and
// output indices are free to permute, so head_dim is assigned to MMA slots
// such that every thread reads whole 16-byte chunks of token rows:
//   QK^T: k-step j, slots {2c,2c+1,2c+8,2c+9}   <-> d = 32c + 4j + {0,1,2,3}
//   PV  : m-tile x, rows {g, g+8}               <-> d = 16g + x, 16g + 8 + x
// (g = lane / 4, c = lane % 4).  Shared-memory rows are 128 bytes with their
// 16-byte chunks XOR-swizzled by (row & 7), which makes both access patterns
// bank-conflict free.
#include <limits.h>
#include <math.h>

#include "attention_common.cuh"

namespace jpt {
namespace {

constexpr int kTile = 64;
constexpr int kStages = 3;
constexpr int kThreads = 128;
constexpr int kD = 128;
constexpr int kMaxRows = 16;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Scratch handed to the kernels (all inside the caller's workspace).
struct MmaScratch {
  int32_t* prefix;    // [B + 1] tiles before each sequence (per head); [B] = total per head
  int32_t* seqinfo;   // [B][4] (first, n, use_add, -) for additive masks
  float* part_o;      // [num_ctas][2][16][128] unnormalised partial outputs
  float* part_m;      // [num_ctas][2][16] (log2 domain)
  float* part_l;      // [num_ctas][2][16]
  int num_ctas;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.f16x2 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(a));
  return r;
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(r) : "f"(x));
  return r;
}

template <bool kRows16>
struct __align__(128) Smem {
  struct Stage {
    uint8_t k[kTile * kD];  // K rows, then V rows: 16 KB that double as the warp-merge buffer
    uint8_t v[kTile * kD];
  } kv[kStages];
  uint8_t q[kStages][(kRows16 ? 16 : 8) * kD * 2];  // bf16 query rows of the piece starting in this stage
  float ks2[kStages][kTile];                        // k_scale * sm_scale * log2(e)
  float vs[kStages][kTile];                         // v_scale
};

// Valid range of a sequence for every mask mode (additive masks have been
// reduced to ranges by mask_ranges_kernel).
__device__ __forceinline__ SeqRange seq_range_x(const AttnArgs& a, const MmaScratch& x, int b, int* use_add) {
  *use_add = 0;
  if (a.mask_mode == JPT_MASK_ADD) {
    SeqRange r;
    r.first = x.seqinfo[4 * b];
    r.n = x.seqinfo[4 * b + 1];
    *use_add = x.seqinfo[4 * b + 2];
    return r;
  }
  return seq_range(a, b);
}

// Position in the global tile list.
struct Cursor {
  int b, h, t, T;  // sequence, head, tile inside the segment, tiles per segment of b
  SeqRange rg;
  int use_add;
};

__device__ __forceinline__ void cursor_load_seq(const AttnArgs& a, const MmaScratch& x, Cursor& cu) {
  cu.rg = seq_range_x(a, x, cu.b, &cu.use_add);
  cu.T = (cu.rg.n + kTile - 1) / kTile;
}

__device__ __forceinline__ void cursor_advance(const AttnArgs& a, const MmaScratch& x, Cursor& cu) {
  if (++cu.t < cu.T) return;
  cu.t = 0;
  if (++cu.h < a.Hkv) return;
  cu.h = 0;
  do {
    ++cu.b;
    if (cu.b >= a.B) {  // past the end: only reached after the CTA's last tile
      cu.b = a.B - 1;
      cu.T = 1;
      cu.rg.n = 0;
      cu.rg.first = 0;
      return;
    }
    cursor_load_seq(a, x, cu);
  } while (cu.T == 0);
}

template <bool kRows16>
__global__ void __launch_bounds__(kThreads, kRows16 ? 2 : 4) flash_decode_i8_kernel(AttnArgs a, MmaScratch x) {
  constexpr int NT = kRows16 ? 2 : 1;  // n-tiles of 8 query rows
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Smem<kRows16>& sm = *reinterpret_cast<Smem<kRows16>*>(smem_raw);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int R = a.R;
  const bool quant = a.k_scale != nullptr;
  const int cta = blockIdx.x;

  // ------------------------------------------------------------------ schedule
  // Tiles per sequence -> exclusive prefix over sequences (each thread owns a
  // slice of ceil(B/128) sequences); scratch aliases the scale arrays.
  int* scan = reinterpret_cast<int*>(&sm.ks2[0][0]);  // 129 ints <= 3 * 64 floats
  __shared__ int s_start[4];
  const int per = (a.B + kThreads - 1) / kThreads;
  const int b_lo = min(a.B, tid * per), b_hi = min(a.B, b_lo + per);
  int mine = 0;
  for (int b = b_lo; b < b_hi; ++b) {
    int ua;
    const SeqRange r = seq_range_x(a, x, b, &ua);
    mine += (r.n + kTile - 1) / kTile;
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
  const int total_per_head = scan[kThreads];
  const long long total = (long long)total_per_head * a.Hkv;
  if (cta == 0) {  // publish the prefix for the merge kernel
    int run = scan[tid];
    for (int b = b_lo; b < b_hi; ++b) {
      x.prefix[b] = run;
      int ua;
      const SeqRange r = seq_range_x(a, x, b, &ua);
      run += (r.n + kTile - 1) / kTile;
    }
    if (tid == 0) x.prefix[a.B] = total_per_head;
  }
  const long long share = (total + x.num_ctas - 1) / x.num_ctas;
  const long long G0 = (long long)cta * share;
  const long long G1 = min(total, G0 + share);
  if (share == 0 || G0 >= G1) return;
  const int count = (int)(G1 - G0);
  {
    // the thread whose slice holds tile G0 walks it and publishes (b, h, t)
    const long long lo = (long long)scan[tid] * a.Hkv;
    const long long hi = (long long)scan[tid + 1] * a.Hkv;
    if (G0 >= lo && G0 < hi) {
      long long run = lo;
      for (int b = b_lo; b < b_hi; ++b) {
        int ua;
        const SeqRange r = seq_range_x(a, x, b, &ua);
        const int T = (r.n + kTile - 1) / kTile;
        const long long nxt = run + (long long)T * a.Hkv;
        if (G0 < nxt) {
          const int rem = (int)(G0 - run);
          s_start[0] = b;
          s_start[1] = rem / T;
          s_start[2] = rem % T;
          break;
        }
        run = nxt;
      }
    }
  }
  __syncthreads();  // also orders the last reads of `scan` before the ring is filled
  Cursor icur;      // producer position
  icur.b = s_start[0];
  icur.h = s_start[1];
  icur.t = s_start[2];
  cursor_load_seq(a, x, icur);
  Cursor ccur = icur;  // consumer position

  const int8_t* kbase = static_cast<const int8_t*>(a.k);
  const int8_t* vbase = static_cast<const int8_t*>(a.v);
  const __nv_bfloat16* qbase = static_cast<const __nv_bfloat16*>(a.q);
  const __nv_bfloat16* mask = static_cast<const __nv_bfloat16*>(a.mask);

  // ------------------------------------------------------------------ producer
  float pend = 0.f;  // this thread's scale of the tile issued last, stored one iteration later
  int pend_stage = -1;

  auto issue_tile = [&](int stage, bool piece_start) {
    const int col = tid & 7;
    const int j0 = icur.t * kTile;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = (tid >> 3) + 16 * i;
      const int j = j0 + row;
      const bool valid = j < icur.rg.n;
      int64_t sidx;
      const int64_t off = kv_row_offset(a, icur.b, icur.h, physical_pos(a, icur.rg, valid ? j : 0), &sidx);
      const uint32_t dst = (uint32_t)(row * kD + ((col ^ (row & 7)) << 4));
      cp_async16(smem_u32(&sm.kv[stage].k[0]) + dst, kbase + off + col * 16, valid);
      cp_async16(smem_u32(&sm.kv[stage].v[0]) + dst, vbase + off + col * 16, valid);
    }
    if (piece_start) {
      const __nv_bfloat16* q = qbase + ((int64_t)icur.b * a.Hkv + icur.h) * R * kD;
      for (int ch = tid; ch < R * 16; ch += kThreads) {
        cp_async16(smem_u32(&sm.q[stage][0]) + ch * 16, q + ch * 8, true);
      }
    }
    if (quant) {
      const int tok = tid & 63;
      const int j = j0 + tok;
      pend = 1.f;
      if (j < icur.rg.n) {
        int64_t sidx;
        (void)kv_row_offset(a, icur.b, icur.h, physical_pos(a, icur.rg, j), &sidx);
        pend = load_scale(tid < 64 ? a.k_scale : a.v_scale, sidx, a.scale_is_f32);
      }
      pend_stage = stage;
    }
  };
  auto flush_side = [&]() {
    if (pend_stage >= 0) {
      const int tok = tid & 63;
      if (tid < 64) sm.ks2[pend_stage][tok] = pend * a.sm_scale * kLog2e;
      else sm.vs[pend_stage][tok] = pend;
      pend_stage = -1;
    }
  };

  // ------------------------------------------------------------------ consumer state
  uint32_t qb[NT][8][2];
  float bias[NT][2];
  float o[NT][8][4];
  float m_run[NT][2], l_run[NT][2];
  int piece_t0 = 0;
  const float unit2 = a.sm_scale * kLog2e;

  for (int s = 0; s < kStages - 1; ++s) {
    if (s < count) {
      flush_side();
      issue_tile(s, s == 0 || icur.t == 0);
      cursor_advance(a, x, icur);
    }
    cp_async_commit();
  }

  for (int i = 0; i < count; ++i) {
    const int stage = i % kStages;
    cp_async_wait<kStages - 2>();
    flush_side();
    __syncthreads();
    if (i + kStages - 1 < count) {
      issue_tile((i + kStages - 1) % kStages, icur.t == 0);
      cursor_advance(a, x, icur);
    }
    cp_async_commit();

    // ---------------- start of a piece: query fragments and fresh state
    if (i == 0 || ccur.t == 0) {
      piece_t0 = ccur.t;
      const uint32_t q_addr = smem_u32(&sm.q[stage][0]);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int row = 8 * nt + g;
        float sum = 0.f;
        if (row < R) {
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {  // 8 bf16 per 16-byte load = k-steps 2*k4, 2*k4+1
            const uint4 raw = lds128(q_addr + row * (kD * 2) + 64 * c + 16 * k4);
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(p2[e]);
              const __half2 hh = __floats2half2_rn(f.x, f.y);
              qb[nt][2 * k4 + (e >> 1)][e & 1] = *reinterpret_cast<const uint32_t*>(&hh);
              const float2 rr = __half22float2(hh);
              sum += rr.x + rr.y;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) qb[nt][j][0] = qb[nt][j][1] = 0u;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        // the row sums live in lanes by g; this thread needs rows 2c and 2c+1
        bias[nt][0] = 1152.f * __shfl_sync(0xffffffffu, sum, 8 * c);
        bias[nt][1] = 1152.f * __shfl_sync(0xffffffffu, sum, 8 * c + 4);
        m_run[nt][0] = m_run[nt][1] = -INFINITY;
        l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
        for (int xx = 0; xx < 8; ++xx) o[nt][xx][0] = o[nt][xx][1] = o[nt][xx][2] = o[nt][xx][3] = 0.f;
      }
    }

    // ---------------- S^T = K Q^T for this warp's 16 tokens
    const uint32_t ks_addr = smem_u32(&sm.kv[stage].k[0]);
    const uint32_t vs_addr = smem_u32(&sm.kv[stage].v[0]);
    const int tok0 = warp * 16;
    float sc[NT][2][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int u = 0; u < 2; ++u) sc[nt][u][0] = sc[nt][u][1] = sc[nt][u][2] = sc[nt][u][3] = 0.f;
    {
      uint32_t kw[2][8];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int row = tok0 + 8 * hh + g;
        const uint32_t rbase = ks_addr + row * kD;
        const uint4 k0 = lds128(rbase + (((2 * c) ^ (row & 7)) << 4));
        const uint4 k1 = lds128(rbase + (((2 * c + 1) ^ (row & 7)) << 4));
        kw[hh][0] = k0.x; kw[hh][1] = k0.y; kw[hh][2] = k0.z; kw[hh][3] = k0.w;
        kw[hh][4] = k1.x; kw[hh][5] = k1.y; kw[hh][6] = k1.z; kw[hh][7] = k1.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t xl = kw[0][j] ^ 0x80808080u, xh = kw[1][j] ^ 0x80808080u;
        uint32_t af[4];
        af[0] = prmt(xl, 0x64646464u, 0x5140u);
        af[1] = prmt(xh, 0x64646464u, 0x5140u);
        af[2] = prmt(xl, 0x64646464u, 0x5342u);
        af[3] = prmt(xh, 0x64646464u, 0x5342u);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_f16(sc[nt][j & 1], af, qb[nt][j][0], qb[nt][j][1]);
      }
    }

    // ---------------- logits (log2 domain), masking, online softmax
    const int jlo = ccur.t * kTile + tok0 + g;  // logical index of token g; token g+8 is jlo + 8
    const bool valid_lo = jlo < ccur.rg.n, valid_hi = (jlo + 8) < ccur.rg.n;
    const float sk_lo = quant ? sm.ks2[stage][tok0 + g] : unit2;
    const float sk_hi = quant ? sm.ks2[stage][tok0 + 8 + g] : unit2;
    const float vs_lo = quant ? sm.vs[stage][tok0 + g] : 1.f;
    const float vs_hi = quant ? sm.vs[stage][tok0 + 8 + g] : 1.f;
    float mk_lo = 0.f, mk_hi = 0.f;
    if (ccur.use_add) {  // additive mask that is not a plain 0 / -inf range (rare)
      if (valid_lo) mk_lo = kLog2e * __bfloat162float(mask[(int64_t)ccur.b * a.mk_b + physical_pos(a, ccur.rg, jlo)]);
      if (valid_hi) mk_hi = kLog2e * __bfloat162float(mask[(int64_t)ccur.b * a.mk_b + physical_pos(a, ccur.rg, jlo + 8)]);
    }
    uint32_t pb[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float xv[4];  // (tok g,row 2c) (tok g,row 2c+1) (tok g+8,row 2c) (tok g+8,row 2c+1)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float s = sc[nt][0][e] + sc[nt][1][e];
        const bool hi = e >= 2;
        const float v = (s - bias[nt][e & 1]) * (hi ? sk_hi : sk_lo) + (hi ? mk_hi : mk_lo);
        xv[e] = (hi ? valid_hi : valid_lo) ? v : -INFINITY;
      }
      float mx0 = fmaxf(xv[0], xv[2]), mx1 = fmaxf(xv[1], xv[3]);
#pragma unroll
      for (int sh = 4; sh <= 16; sh <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
      }
      const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
      const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
      const float al0 = fast_exp2(m_run[nt][0] - mu0), al1 = fast_exp2(m_run[nt][1] - mu1);
      m_run[nt][0] = mn0;
      m_run[nt][1] = mn1;
      const float p00 = fast_exp2(xv[0] - mu0), p01 = fast_exp2(xv[1] - mu1);
      const float p10 = fast_exp2(xv[2] - mu0), p11 = fast_exp2(xv[3] - mu1);
      l_run[nt][0] = l_run[nt][0] * al0 + (p00 + p10);
      l_run[nt][1] = l_run[nt][1] * al1 + (p01 + p11);
      if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
        for (int xx = 0; xx < 8; ++xx) {
          o[nt][xx][0] *= al0;
          o[nt][xx][1] *= al1;
          o[nt][xx][2] *= al0;
          o[nt][xx][3] *= al1;
        }
      }
      // P^T as the B operand: transpose the two 8x8 (token x row) blocks
      pb[nt][0] = movmatrix_trans(pack_half2(p00 * vs_lo, p01 * vs_lo));
      pb[nt][1] = movmatrix_trans(pack_half2(p10 * vs_hi, p11 * vs_hi));
    }

    // ---------------- O^T += V^T P^T: this thread converts the 16-byte chunk g
    // of token rows 2c, 2c+1, 2c+8, 2c+9
    {
      uint32_t vw[4][4];
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const int row = tok0 + 2 * c + (r4 & 1) + 8 * (r4 >> 1);
        const uint4 q4 = lds128(vs_addr + row * kD + ((g ^ (row & 7)) << 4));
        vw[r4][0] = q4.x ^ 0x80808080u; vw[r4][1] = q4.y ^ 0x80808080u;
        vw[r4][2] = q4.z ^ 0x80808080u; vw[r4][3] = q4.w ^ 0x80808080u;
      }
#pragma unroll
      for (int wd = 0; wd < 2; ++wd) {
        // bytes 4wd..4wd+3 (rows g of the m-tiles 4wd..4wd+3) and bytes 8+4wd.. (rows g+8)
        const uint32_t a01 = prmt(vw[0][wd], vw[1][wd], 0x5140u), a23 = prmt(vw[0][wd], vw[1][wd], 0x7362u);
        const uint32_t b01 = prmt(vw[0][wd + 2], vw[1][wd + 2], 0x5140u), b23 = prmt(vw[0][wd + 2], vw[1][wd + 2], 0x7362u);
        const uint32_t c01 = prmt(vw[2][wd], vw[3][wd], 0x5140u), c23 = prmt(vw[2][wd], vw[3][wd], 0x7362u);
        const uint32_t d01 = prmt(vw[2][wd + 2], vw[3][wd + 2], 0x5140u), d23 = prmt(vw[2][wd + 2], vw[3][wd + 2], 0x7362u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t sel = (e & 1) ? 0x5342u : 0x5140u;
          uint32_t af[4];
          af[0] = hsub2_u32(prmt(e < 2 ? a01 : a23, 0x64646464u, sel), 0x64806480u);
          af[1] = hsub2_u32(prmt(e < 2 ? b01 : b23, 0x64646464u, sel), 0x64806480u);
          af[2] = hsub2_u32(prmt(e < 2 ? c01 : c23, 0x64646464u, sel), 0x64806480u);
          af[3] = hsub2_u32(prmt(e < 2 ? d01 : d23, 0x64646464u, sel), 0x64806480u);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_f16(o[nt][4 * wd + e], af, pb[nt][0], pb[nt][1]);
        }
      }
    }

    // ---------------- end of a piece: merge the four warps and write out
    if (i == count - 1 || ccur.t == ccur.T - 1) {
      const bool is_final = piece_t0 == 0 && ccur.t == ccur.T - 1;
      const int slot = piece_t0 > 0 ? 0 : 1;
      const int64_t row_base = ((int64_t)ccur.b * a.Hkv + ccur.h) * R;
      float* obuf = reinterpret_cast<float*>(&sm.kv[stage]);  // [4 warps][8 rows][128] = K and V of the stage
      float* msm = &sm.ks2[stage][0];                            // [4][8]
      float* lsm = &sm.vs[stage][0];                             // [4][8]
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float l0 = l_run[nt][0], l1 = l_run[nt][1];
#pragma unroll
        for (int sh = 4; sh <= 16; sh <<= 1) {
          l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
          l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
        }
        __syncthreads();  // every warp is done with the tile (and with the previous pass)
        {
          float4* d0 = reinterpret_cast<float4*>(obuf + ((warp * 8 + 2 * c) * kD) + 16 * g);
          float4* d1 = reinterpret_cast<float4*>(obuf + ((warp * 8 + 2 * c + 1) * kD) + 16 * g);
          d0[0] = make_float4(o[nt][0][0], o[nt][1][0], o[nt][2][0], o[nt][3][0]);
          d0[1] = make_float4(o[nt][4][0], o[nt][5][0], o[nt][6][0], o[nt][7][0]);
          d0[2] = make_float4(o[nt][0][2], o[nt][1][2], o[nt][2][2], o[nt][3][2]);
          d0[3] = make_float4(o[nt][4][2], o[nt][5][2], o[nt][6][2], o[nt][7][2]);
          d1[0] = make_float4(o[nt][0][1], o[nt][1][1], o[nt][2][1], o[nt][3][1]);
          d1[1] = make_float4(o[nt][4][1], o[nt][5][1], o[nt][6][1], o[nt][7][1]);
          d1[2] = make_float4(o[nt][0][3], o[nt][1][3], o[nt][2][3], o[nt][3][3]);
          d1[3] = make_float4(o[nt][4][3], o[nt][5][3], o[nt][6][3], o[nt][7][3]);
          if (g == 0) {
            msm[warp * 8 + 2 * c] = m_run[nt][0];
            msm[warp * 8 + 2 * c + 1] = m_run[nt][1];
            lsm[warp * 8 + 2 * c] = l0;
            lsm[warp * 8 + 2 * c + 1] = l1;
          }
        }
        __syncthreads();
        const int rows_here = min(8, R - 8 * nt);
        for (int r = 0; r < rows_here; ++r) {
          float M = msm[r];
#pragma unroll
          for (int w = 1; w < 4; ++w) M = fmaxf(M, msm[w * 8 + r]);
          float L = 0.f, acc = 0.f;
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const float mw = msm[w * 8 + r];
            const float wg = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
            L += wg * lsm[w * 8 + r];
            acc += wg * obuf[(w * 8 + r) * kD + tid];
          }
          const int rr = 8 * nt + r;
          if (is_final) {
            const int64_t row = row_base + rr;
            static_cast<__nv_bfloat16*>(a.o)[row * kD + tid] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
            if (tid == 0) {
              if (a.m) a.m[row] = M * kLn2;
              if (a.l) a.l[row] = L;
            }
          } else {
            const int64_t pr = ((int64_t)cta * 2 + slot) * kMaxRows + rr;
            x.part_o[pr * kD + tid] = acc;
            if (tid == 0) {
              x.part_m[pr] = M;
              x.part_l[pr] = L;
            }
          }
        }
      }
      // The next iteration's barrier orders these reads before the stage is refilled.
    }
    cursor_advance(a, x, ccur);
  }
  cp_async_wait<0>();
}

// One block per (sequence, head) segment: combine the partials of segments that
// were cut by CTA borders and write the rows of empty sequences.
__global__ void __launch_bounds__(kThreads) flash_decode_merge_kernel(AttnArgs a, MmaScratch x) {
  const int seg = blockIdx.x;
  const int b = seg / a.Hkv, h = seg % a.Hkv;
  const int R = a.R, tid = threadIdx.x;
  const int T = x.prefix[b + 1] - x.prefix[b];
  const int64_t row_base = (int64_t)seg * R;
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.o);
  if (T == 0) {
    for (int r = 0; r < R; ++r) {
      o[(row_base + r) * kD + tid] = __float2bfloat16_rn(0.f);
      if (tid == 0) {
        if (a.m) a.m[row_base + r] = -INFINITY;
        if (a.l) a.l[row_base + r] = 0.f;
      }
    }
    return;
  }
  const long long total = (long long)x.prefix[a.B] * a.Hkv;
  const long long share = (total + x.num_ctas - 1) / x.num_ctas;
  const long long gs = (long long)x.prefix[b] * a.Hkv + (long long)h * T;
  const int first = (int)(gs / share), last = (int)((gs + T - 1) / share);
  if (first == last) return;  // written as final rows by the main kernel
  for (int r = 0; r < R; ++r) {
    float M = -INFINITY;
    for (int cta = first; cta <= last; ++cta) {
      const int slot = cta == first ? 1 : 0;
      M = fmaxf(M, x.part_m[((int64_t)cta * 2 + slot) * kMaxRows + r]);
    }
    float L = 0.f, acc = 0.f;
    for (int cta = first; cta <= last; ++cta) {
      const int slot = cta == first ? 1 : 0;
      const int64_t pr = ((int64_t)cta * 2 + slot) * kMaxRows + r;
      const float mw = x.part_m[pr];
      const float wg = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
      L += wg * x.part_l[pr];
      acc += wg * x.part_o[pr * kD + tid];
    }
    o[(row_base + r) * kD + tid] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    if (tid == 0) {
      if (a.m) a.m[row_base + r] = M * kLn2;
      if (a.l) a.l[row_base + r] = L;
    }
  }
}

// Additive masks -> valid ranges.  A mask row whose finite entries form one run
// (possibly wrapping around the end of the cache) becomes (first, n); if all
// finite entries are zero the mask itself is not needed any more.  Any other
// row keeps the whole cache length and the additive term.
__global__ void __launch_bounds__(kThreads) mask_ranges_kernel(AttnArgs a, MmaScratch x) {
  const int b = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* mask = static_cast<const __nv_bfloat16*>(a.mask) + (int64_t)b * a.mk_b;
  int cnt = 0, lo = INT_MAX, hi = -1, bad_lo = INT_MAX, bad_hi = -1, nonzero = 0;
  for (int s = tid; s < a.S; s += kThreads) {
    const float v = __bfloat162float(mask[s]);
    if (v == -INFINITY) {
      bad_lo = min(bad_lo, s);
      bad_hi = max(bad_hi, s);
    } else {
      ++cnt;
      lo = min(lo, s);
      hi = max(hi, s);
      if (v != 0.f) nonzero = 1;
    }
  }
  __shared__ int sh[6];
  if (tid == 0) {
    sh[0] = 0; sh[1] = INT_MAX; sh[2] = -1; sh[3] = INT_MAX; sh[4] = -1; sh[5] = 0;
  }
  __syncthreads();
  atomicAdd(&sh[0], cnt);
  atomicMin(&sh[1], lo);
  atomicMax(&sh[2], hi);
  atomicMin(&sh[3], bad_lo);
  atomicMax(&sh[4], bad_hi);
  atomicOr(&sh[5], nonzero);
  __syncthreads();
  if (tid == 0) {
    int first = 0, n = a.S, use_add = 1;
    cnt = sh[0];
    if (cnt == 0) {
      n = 0;
      use_add = 0;
    } else if (cnt == sh[2] - sh[1] + 1) {  // one run [lo, hi]
      first = sh[1];
      n = cnt;
      use_add = sh[5];
    } else if (cnt == sh[3] + (a.S - 1 - sh[4])) {  // a run that wraps: [bad_hi+1, S) U [0, bad_lo)
      first = sh[4] + 1;
      n = cnt;
      use_add = sh[5];
    }
    x.seqinfo[4 * b] = first;
    x.seqinfo[4 * b + 1] = n;
    x.seqinfo[4 * b + 2] = use_add;
    x.seqinfo[4 * b + 3] = 0;
  }
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct ScratchLayout {
  size_t prefix, seqinfo, part_m, part_l, part_o, total;
  int num_ctas;
};

ScratchLayout scratch_layout(const jpt_attn_params& p) {
  const int R = (p.Hq / p.Hkv) * p.Tq;
  ScratchLayout s;
  s.num_ctas = sm_count() * (R > 8 ? 2 : 4);
  size_t off = 0;
  s.prefix = off;
  off = align_up(off + sizeof(int32_t) * (p.B + 1), 256);
  s.seqinfo = off;
  off = align_up(off + sizeof(int32_t) * 4 * p.B, 256);
  s.part_m = off;
  off = align_up(off + sizeof(float) * s.num_ctas * 2 * kMaxRows, 256);
  s.part_l = off;
  off = align_up(off + sizeof(float) * s.num_ctas * 2 * kMaxRows, 256);
  s.part_o = off;
  off = align_up(off + sizeof(float) * s.num_ctas * 2 * kMaxRows * kD, 256);
  s.total = off;
  return s;
}

}  // namespace

bool attention_mma_eligible(const jpt_attn_params& p) {
  const int R = (p.Hq / p.Hkv) * p.Tq;
  if (p.D != kD || R > kMaxRows || p.q_dtype != JPT_BF16 || p.kv_dtype != JPT_INT8) return false;
  if (p.mask_mode == JPT_MASK_ADD && p.mk_r != 0) return false;  // per-row masks: scalar kernel
  if (!aligned(p.q, 16) || !aligned(p.k, 16) || !aligned(p.v, 16)) return false;
  if (p.paged) {
    if (p.kv_h % 16 || p.kv_page % 16) return false;
  } else if (p.kv_b % 16 || p.kv_h % 16 || p.kv_s % 16) {
    return false;
  }
  return true;
}

size_t attention_mma_workspace_bytes(const jpt_attn_params& p) { return scratch_layout(p).total; }

int launch_attention_mma(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st) {
  const ScratchLayout lay = scratch_layout(p);
  JPT_REQUIRE(p.workspace && p.workspace_bytes >= lay.total, JPT_EWORKSPACE,
              "flash_decode: workspace of %zu bytes needed, %zu given", lay.total, p.workspace_bytes);
  JPT_REQUIRE(aligned(p.workspace, 256), JPT_EALIGN, "flash_decode: workspace must be 256-byte aligned");
  char* ws = static_cast<char*>(p.workspace);
  MmaScratch x;
  x.prefix = reinterpret_cast<int32_t*>(ws + lay.prefix);
  x.seqinfo = reinterpret_cast<int32_t*>(ws + lay.seqinfo);
  x.part_m = reinterpret_cast<float*>(ws + lay.part_m);
  x.part_l = reinterpret_cast<float*>(ws + lay.part_l);
  x.part_o = reinterpret_cast<float*>(ws + lay.part_o);
  x.num_ctas = lay.num_ctas;

  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(flash_decode_i8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)sizeof(Smem<false>));
    cudaFuncSetAttribute(flash_decode_i8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)sizeof(Smem<true>));
    configured = true;
  }
  if (a.mask_mode == JPT_MASK_ADD) {
    mask_ranges_kernel<<<a.B, kThreads, 0, st>>>(a, x);
    if (int rc = check_launch("mask_ranges_kernel")) return rc;
  }
  if (a.R > 8) {
    flash_decode_i8_kernel<true><<<lay.num_ctas, kThreads, sizeof(Smem<true>), st>>>(a, x);
  } else {
    flash_decode_i8_kernel<false><<<lay.num_ctas, kThreads, sizeof(Smem<false>), st>>>(a, x);
  }
  if (int rc = check_launch("flash_decode_i8_kernel")) return rc;
  flash_decode_merge_kernel<<<a.B * a.Hkv, kThreads, 0, st>>>(a, x);
  return check_launch("flash_decode_merge_kernel");
}

}  // namespace jpt
