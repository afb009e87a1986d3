// Ragged flash-decode attention for head_dim 128 and int8 caches on tensor
// cores (sm_100a): one persistent, work-balanced kernel.
//
// Work model.  A "tile" is 64 consecutive valid tokens of one (sequence, KV
// head) segment.  All tiles of all segments form one global list ordered by
// (sequence, head, tile), each segment preceded by kPieceCost "overhead" slots
// that stand for the fixed cost of starting and finishing a segment; every CTA
// of the persistent grid takes an equal, contiguous share of that list, so
// ragged lengths cost nothing in balance.  A CTA therefore works on a run of
// "pieces" (its share cut at segment borders).  A piece that covers its whole
// segment is written out as final rows.  A piece that does not goes to a
// per-CTA scratch slot (there are at most two per CTA: its first and its last
// piece); the CTA that delivers the last missing piece of a segment (found with
// one wrapping atomic counter per segment) combines them and writes the rows.
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
// dot product (S - 1152 * sum_d q_d); for V an all-ones m-tile accumulates
// sum_t P^T next to O^T and 1152 times that sum is subtracted when a piece is
// written (both corrections are far below the fp32 accumulation noise that the
// 2e-2 output tolerance allows).  Contraction and output indices are free to
// permute, so head_dim is assigned to MMA slots such that every thread reads
// whole 16-byte chunks of token rows:
//   QK^T: k-step j, slots {2c,2c+1,2c+8,2c+9}   <-> d = 32c + 4j + {0,1,2,3}
//   PV  : m-tile x, rows {g, g+8}               <-> d = 16g + x, 16g + 8 + x
// (g = lane / 4, c = lane % 4).  Shared-memory rows are 128 bytes with their
// 16-byte chunks XOR-swizzled by (row & 7), which makes both access patterns
// bank-conflict free.
//
// The running maximum of the online softmax is only raised when a new logit
// exceeds it by more than kLazy (log2 units), so the accumulators are rarely
// rescaled; probabilities then stay below 2^kLazy, well inside fp16.  The true
// maximum is tracked on the side for the (m, l) outputs.
#include <limits.h>
#include <math.h>

#include "attention_tiles.cuh"

namespace jpt {
namespace {

constexpr int kTile = 64;
constexpr int kStages = 3;
constexpr float kLazy = 8.f;

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
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Four 8x8 b16 matrices; lane l gives the address of row l % 8 of matrix l / 8,
// and receives elements (l / 4, 2 (l % 4) .. +1) of each (transposed with .trans).
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf162(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
#ifdef JPT_ATTN_TIMING
__device__ unsigned long long g_attn_timing[4096 * 4];
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned smid() {
  unsigned r;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(r));
  return r;
}
#endif

// int8 caches: 3 stages of 16 KB; bf16 caches: 2 stages of 32 KB.
template <bool kBf16>
struct Geometry {
  static constexpr int kES = kBf16 ? 2 : 1;           // bytes per cache element
  static constexpr int kRowBytes = kD * kES;          // one token row
  static constexpr int kNS = kBf16 ? 2 : kStages;     // ring depth
  static constexpr int kCpr = kRowBytes / 16;         // 16-byte chunks per row
  static constexpr int kRpp = kThreads / kCpr;        // rows covered by one copy pass of the CTA
  static constexpr int kPasses = kTile / kRpp;        // copy passes per tile (each moves 2048 bytes per tensor)
};

template <bool kBf16>
struct __align__(16) Stage {
  uint8_t k[kTile * Geometry<kBf16>::kRowBytes];  // K rows, then V rows; the first 16 KB double as the merge buffer of a piece
  uint8_t v[kTile * Geometry<kBf16>::kRowBytes];
};

template <bool kRows16, bool kBf16>
struct __align__(128) Smem {
  Stage<kBf16> kv[Geometry<kBf16>::kNS];
  uint8_t q[Geometry<kBf16>::kNS][(kRows16 ? 16 : 8) * kD * 2];  // bf16 query rows of the piece starting in this stage
  float ks2[Geometry<kBf16>::kNS][kTile];                        // k_scale * sm_scale * log2(e)
  float vs[Geometry<kBf16>::kNS][kTile];                         // v_scale
};

__device__ __forceinline__ int tiles_of(int n) { return (n + kTile - 1) / kTile; }
__device__ __forceinline__ int slots_of(int n) { return n > 0 ? tiles_of(n) + kPieceCost : 0; }

template <bool kRows16, bool kBf16>
__global__ void __launch_bounds__(kThreads, kRows16 ? 2 : (kBf16 ? 3 : 4))
    flash_decode_kernel(AttnArgs a, MmaScratch x) {
  constexpr int NT = kRows16 ? 2 : 1;  // n-tiles of 8 query rows
  using Geo = Geometry<kBf16>;
  constexpr int kNS = Geo::kNS, kES = Geo::kES, kRowBytes = Geo::kRowBytes;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Smem<kRows16, kBf16>& sm = *reinterpret_cast<Smem<kRows16, kBf16>*>(smem_raw);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int R = a.R;
  const bool quant = a.k_scale != nullptr;
  const int cta = blockIdx.x;
#ifdef JPT_ATTN_TIMING
  if (tid == 0 && cta < 4096) {
    g_attn_timing[4 * cta] = globaltimer_ns();
    g_attn_timing[4 * cta + 2] = smid();
    g_attn_timing[4 * cta + 1] = 0;
    g_attn_timing[4 * cta + 3] = 0;
  }
  int dbg_pieces = 0, dbg_tiles = 0;
#endif

  // ------------------------------------------------------------------ schedule
  // Slots per sequence (tiles + overhead) -> exclusive prefix over sequences;
  // each thread owns a slice of ceil(B/128) sequences.  The scan scratch
  // aliases the scale arrays, which are not in use yet.
  int* scan = reinterpret_cast<int*>(&sm.ks2[0][0]);  // 129 ints <= 3 * 64 floats
  __shared__ int s_start[4];
  __shared__ int s_flag;
  __shared__ TileMeta s_meta[kNS];
  const int per = (a.B + kThreads - 1) / kThreads;
  const int b_lo = min(a.B, tid * per), b_hi = min(a.B, b_lo + per);
  int mine = 0;
  for (int b = b_lo; b < b_hi; ++b) {
    int ua;
    mine += slots_of(seq_range_x(a, x, b, &ua).n);
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
        const int sl = slots_of(seq_range_x(a, x, b, &ua).n);
        const int nxt = run + sl * a.Hkv;
        if (G0 < nxt) {
          const int rem = G0 - run;
          s_start[0] = b;
          s_start[1] = rem / sl;
          s_start[2] = rem % sl;
          break;
        }
        run = nxt;
      }
    }
  }
  // Rows of empty sequences are nobody's tile: sequence b is cleared by CTA b mod grid.
  for (int b = cta; b < a.B; b += gridDim.x) {
    int ua;
    if (seq_range_x(a, x, b, &ua).n == 0) {
      const int64_t r0 = (int64_t)b * a.Hkv * R;
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.o);
      for (int i = tid; i < a.Hkv * R * kD; i += kThreads) o[r0 * kD + i] = __float2bfloat16_rn(0.f);
      for (int i = tid; i < a.Hkv * R; i += kThreads) {
        if (a.m) a.m[r0 + i] = -INFINITY;
        if (a.l) a.l[r0 + i] = 0.f;
      }
    }
  }
  __syncthreads();  // s_start visible; last reads of `scan` done before the ring is filled
  if (G0 >= G1) return;

  const int8_t* kbase = static_cast<const int8_t*>(a.k);
  const int8_t* vbase = static_cast<const int8_t*>(a.v);
  const __nv_bfloat16* qbase = static_cast<const __nv_bfloat16*>(a.q);
  const __nv_bfloat16* mask = static_cast<const __nv_bfloat16*>(a.mask);

  // ------------------------------------------------------------------ producer
  // Position of the next tile to fetch (uniform across the CTA) ...
  int pb = s_start[0], ph = s_start[1], pt, pslot = G0;  // pslot: global slot index of tile pt
  int pT, pn, pfirst, puse_add;
  // ... and what follows from it for this thread: 16-byte column tid % kCpr of
  // rows (tid / kCpr) + kRpp i of a tile.  kRpp is a multiple of 8, so the
  // swizzled shared-memory offset of row + kRpp i is that of row plus 2048 i.
  const int prow = tid / Geo::kCpr, pcol = tid % Geo::kCpr;
  const uint32_t pdst = (uint32_t)(prow * kRowBytes + ((pcol ^ (prow & 7)) << 4));
  const bool tile_pages = a.paged && (a.page_size % kTile) == 0;
  const bool rows_packed = a.paged ? tile_pages : (a.kv_s == kD);  // rows of a tile kD bytes apart
  const int kv_s32 = (int)a.kv_s, sc_s32 = (int)a.sc_s;
  const int8_t *kseg, *vseg;  // segment base + this thread's column
  int64_t scseg;
  int ppos;                   // physical position of row 0 of tile pt
  int pfirst_cta, pparts;

  auto load_seq = [&]() {
    const SeqRange r = seq_range_x(a, x, pb, &puse_add);
    pn = r.n;
    pfirst = r.first;
    pT = tiles_of(r.n);
  };
  auto seg_setup = [&]() {  // pt, pslot are set
    const int64_t seg = a.paged ? (int64_t)ph * a.kv_h : (int64_t)pb * a.kv_b + (int64_t)ph * a.kv_h;
    kseg = kbase + seg * kES + pcol * 16;
    vseg = vbase + seg * kES + pcol * 16;
    scseg = a.paged ? 0 : (int64_t)pb * a.sc_b;
    ppos = pfirst + pt * kTile;
    if (ppos >= a.S) ppos -= a.S;
    const int t0slot = pslot - pt;  // slot of tile 0 of this segment
    pfirst_cta = t0slot / share;
    pparts = (t0slot + pT - 1) / share - pfirst_cta + 1;
  };
  auto advance = [&]() {
    ++pslot;
    ppos += kTile;
    if (ppos >= a.S) ppos -= a.S;
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
    const int v0 = s_start[2];  // slot inside the segment: overhead slots come first
    if (v0 < kPieceCost) {
      pslot += kPieceCost - v0;
      pt = 0;
    } else {
      pt = v0 - kPieceCost;
    }
    seg_setup();
  }

  float pend = 0.f;  // this thread's scale of the tile issued last, stored one iteration later
  int pend_stage = -1;
  bool first_issue = true;

  auto issue_tile = [&](int stage) {
    const int j0 = pt * kTile;
    const bool piece_start = first_issue || pt == 0;
    first_issue = false;
    if (tid == 0) {
      TileMeta mt;
      mt.b = pb; mt.h = ph; mt.t = pt; mt.T = pT; mt.n = pn; mt.first = pfirst; mt.use_add = puse_add;
      mt.first_cta = pfirst_cta; mt.parts = pparts;
      mt.pad[0] = mt.pad[1] = 0;
      mt.pad[2] = pslot + 1 >= G1;  // no tile follows in this CTA's share
      s_meta[stage] = mt;
    }
    const uint32_t kdst = smem_u32(&sm.kv[stage].k[0]) + pdst;
    const uint32_t vdst = smem_u32(&sm.kv[stage].v[0]) + pdst;
    int page = -1, page_pos0 = 0;
    if (tile_pages) {
      const int pi = j0 / a.page_size;
      page = a.page_table[(int64_t)pb * a.max_pages + pi];
      page_pos0 = pi * a.page_size;
    }
    if (rows_packed && j0 + kTile <= pn && ppos + kTile <= a.S) {
      // whole tile valid, no ring wrap, rows kD bytes apart: one address per tensor
      const int64_t off = a.paged ? (int64_t)page * a.kv_page + (int64_t)(j0 - page_pos0 + prow) * kD
                                  : (int64_t)(ppos + prow) * kD;
      const int8_t* kp = kseg + off * kES;
      const int8_t* vp = vseg + off * kES;
#pragma unroll
      for (int i = 0; i < Geo::kPasses; ++i) {
        cp_async16(kdst + 2048 * i, kp + 2048 * i, true);
        cp_async16(vdst + 2048 * i, vp + 2048 * i, true);
      }
    } else {
#pragma unroll
      for (int i = 0; i < Geo::kPasses; ++i) {
        const int r = prow + Geo::kRpp * i;
        const bool valid = j0 + r < pn;
        int pos = valid ? ppos + r : ppos;
        if (pos >= a.S) pos -= a.S;
        int64_t off;
        if (a.paged) {
          int pg = page, tok = pos - page_pos0;
          if (!tile_pages) {
            pg = a.page_table[(int64_t)pb * a.max_pages + pos / a.page_size];
            tok = pos % a.page_size;
          }
          off = (int64_t)pg * a.kv_page + (int64_t)tok * kD;
        } else {
          off = (int64_t)pos * kv_s32;
        }
        cp_async16(kdst + 2048 * i, kseg + off * kES, valid);
        cp_async16(vdst + 2048 * i, vseg + off * kES, valid);
      }
    }
    if (piece_start) {
      const __nv_bfloat16* q = qbase + ((int64_t)pb * a.Hkv + ph) * R * kD;
      for (int ch = tid; ch < R * 16; ch += kThreads) {
        cp_async16(smem_u32(&sm.q[stage][0]) + ch * 16, q + ch * 8, true);
      }
    }
    if (quant) {
      const int r = tid & 63;
      pend = 1.f;
      if (j0 + r < pn) {
        int pos = ppos + r;
        if (pos >= a.S) pos -= a.S;
        int64_t sidx;
        if (a.paged) {
          int pg = page, tok = pos - page_pos0;
          if (!tile_pages) {
            pg = a.page_table[(int64_t)pb * a.max_pages + pos / a.page_size];
            tok = pos % a.page_size;
          }
          sidx = (int64_t)pg * a.page_size + tok;
        } else {
          sidx = scseg + (int64_t)pos * sc_s32;
        }
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
  // Fetch the next tile of the share into `stage`, or mark the stage as empty.
  auto produce = [&](int stage) {
    if (pslot < G1) {
      flush_side();
      issue_tile(stage);
      advance();
    } else if (tid == 0) {
      s_meta[stage].t = -1;
    }
    cp_async_commit();
  };

  // ------------------------------------------------------------------ consumer state
  uint32_t qb[NT][8][2];
  float bias[NT][2];
  float o[NT][8][4];
  float wsum[NT][4];  // sum_t P^T[t][row] from an all-ones m-tile: carries the V offset
  float m_run[NT][2], m_true[NT][2], l_run[NT][2];
  int piece_t0 = 0;
  const float unit2 = a.sm_scale * kLog2e;
  const float inv_unit2 = 1.f / unit2, sqrt_d = __frcp_rn(a.sm_scale);  // used when the logit chain is rounded
  // shared-memory offsets of this thread's operands inside a stage
  const int tok0 = warp * 16;
  uint32_t koff[2][2], voff[4];
  if constexpr (!kBf16) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int row = tok0 + 8 * hh + g;
      koff[hh][0] = row * kD + (((2 * c) ^ (row & 7)) << 4);
      koff[hh][1] = row * kD + (((2 * c + 1) ^ (row & 7)) << 4);
    }
#pragma unroll
    for (int r4 = 0; r4 < 4; ++r4) {
      const int row = tok0 + 2 * c + (r4 & 1) + 8 * (r4 >> 1);
      voff[r4] = kTile * kD + row * kD + ((g ^ (row & 7)) << 4);
    }
  } else {
    // ldmatrix row addresses of this lane: matrix mi = lane / 8, row lane % 8.
    // K (A operand, tokens on M): token tok0 + 8 (mi & 1) + row, 16-byte chunk 2 j + (mi >> 1).
    // V (A operand through .trans, d on M): token tok0 + 8 (mi >> 1) + row, chunk 2 x + (mi & 1).
    // The chunk of k-step j / m-tile x differs from chunk 0's only in bits 1..3,
    // which the swizzle leaves alone or flips by a constant: offset ^ (2 j << 4).
    const int mi = lane >> 3, r8 = lane & 7;
    const int ktok = tok0 + 8 * (mi & 1) + r8, vtok = tok0 + 8 * (mi >> 1) + r8;
    koff[0][0] = ktok * kRowBytes + (((mi >> 1) ^ (ktok & 7)) << 4);
    voff[0] = kTile * kRowBytes + vtok * kRowBytes + (((mi & 1) ^ (vtok & 7)) << 4);
    koff[0][1] = koff[1][0] = koff[1][1] = 0;
    voff[1] = voff[2] = voff[3] = 0;
  }

#pragma unroll
  for (int s0 = 0; s0 < kNS - 1; ++s0) produce(s0);

  int stage = 0;
  for (int i = 0;; ++i) {
    cp_async_wait<kNS - 2>();
    flush_side();
    __syncthreads();
    {
      int ps = stage + kNS - 1;
      if (ps >= kNS) ps -= kNS;
      produce(ps);
    }
    const TileMeta mt = s_meta[stage];
    if (mt.t < 0) break;
    const int next_stage = stage + 1 == kNS ? 0 : stage + 1;
    const bool last_of_share = mt.pad[2] != 0;
#ifdef JPT_ATTN_TIMING
    ++dbg_tiles;
#endif

    // ---------------- start of a piece: query fragments and fresh state
    if (i == 0 || mt.t == 0) {
      piece_t0 = mt.t;
#ifdef JPT_ATTN_TIMING
      ++dbg_pieces;
#endif
      const uint32_t q_addr = smem_u32(&sm.q[stage][0]);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int row = 8 * nt + g;
        float sum = 0.f;
        if constexpr (kBf16) {
          // B operand of k-step j: d = 16 j + 2 c, +1 and 16 j + 8 + 2 c, +1 of row g,
          // which is what ldmatrix hands out for the chunks 2 j and 2 j + 1 of the 8 rows.
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4(q_addr + (8 * nt + (lane & 7)) * (kD * 2) + (4 * k4 + (lane >> 3)) * 16, r0, r1, r2, r3);
            const bool ok = row < R;
            qb[nt][2 * k4][0] = ok ? r0 : 0u;
            qb[nt][2 * k4][1] = ok ? r1 : 0u;
            qb[nt][2 * k4 + 1][0] = ok ? r2 : 0u;
            qb[nt][2 * k4 + 1][1] = ok ? r3 : 0u;
          }
        } else if (row < R) {
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
        m_true[nt][0] = m_true[nt][1] = -INFINITY;
        l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
        for (int xx = 0; xx < 8; ++xx) o[nt][xx][0] = o[nt][xx][1] = o[nt][xx][2] = o[nt][xx][3] = 0.f;
        wsum[nt][0] = wsum[nt][1] = wsum[nt][2] = wsum[nt][3] = 0.f;
      }
    }

    // ---------------- S^T = K Q^T for this warp's 16 tokens
    const uint32_t st_addr = smem_u32(&sm.kv[stage]);
    float sc[NT][2][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int u = 0; u < 2; ++u) sc[nt][u][0] = sc[nt][u][1] = sc[nt][u][2] = sc[nt][u][3] = 0.f;
    if constexpr (kBf16) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t af[4];
        ldmatrix_x4(st_addr + (koff[0][0] ^ (uint32_t)(2 * j << 4)), af[0], af[1], af[2], af[3]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_bf16(sc[nt][j & 1], af, qb[nt][j][0], qb[nt][j][1]);
      }
    } else {
      uint32_t kw[2][8];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const uint4 k0 = lds128(st_addr + koff[hh][0]);
        const uint4 k1 = lds128(st_addr + koff[hh][1]);
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
    const int jlo = mt.t * kTile + tok0 + g;  // logical index of token g; token g+8 is jlo + 8
    const bool valid_lo = jlo < mt.n, valid_hi = (jlo + 8) < mt.n;
    const float sk_lo = quant ? sm.ks2[stage][tok0 + g] : unit2;
    const float sk_hi = quant ? sm.ks2[stage][tok0 + 8 + g] : unit2;
    const float vs_lo = quant ? sm.vs[stage][tok0 + g] : 1.f;
    const float vs_hi = quant ? sm.vs[stage][tok0 + 8 + g] : 1.f;
    float mk_lo = 0.f, mk_hi = 0.f;
    if (mt.use_add) {  // additive mask that is not a plain 0 / -inf range (rare)
      SeqRange rg;
      rg.n = mt.n;
      rg.first = mt.first;
      if (valid_lo) mk_lo = kLog2e * __bfloat162float(mask[(int64_t)mt.b * a.mk_b + physical_pos(a, rg, jlo)]);
      if (valid_hi) mk_hi = kLog2e * __bfloat162float(mask[(int64_t)mt.b * a.mk_b + physical_pos(a, rg, jlo + 8)]);
    }
    uint32_t pb2[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float xv[4];  // (tok g,row 2c) (tok g,row 2c+1) (tok g+8,row 2c) (tok g+8,row 2c+1)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float s = sc[nt][0][e] + sc[nt][1][e];
        const bool hi = e >= 2;
        float v = (s - bias[nt][e & 1]) * (hi ? sk_hi : sk_lo) + (hi ? mk_hi : mk_lo);
        if (a.round_logits) {
          // the K scale is a bf16 value: rounding undoes the error of dividing it back out
          const float ks = quant ? bf16_round((hi ? sk_hi : sk_lo) * inv_unit2) : 1.f;
          v = kLog2e * rounded_logit(s - bias[nt][e & 1], sqrt_d, ks, quant, (hi ? mk_hi : mk_lo) * kLn2);
        }
        xv[e] = (hi ? valid_hi : valid_lo) ? v : -INFINITY;
      }
      float mx0 = fmaxf(xv[0], xv[2]), mx1 = fmaxf(xv[1], xv[3]);
#pragma unroll
      for (int sh = 4; sh <= 16; sh <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
      }
      m_true[nt][0] = fmaxf(m_true[nt][0], mx0);
      m_true[nt][1] = fmaxf(m_true[nt][1], mx1);
      // raise the reference maximum only when it is exceeded by more than kLazy
      const bool up0 = mx0 > m_run[nt][0] + kLazy, up1 = mx1 > m_run[nt][1] + kLazy;
      if (__any_sync(0xffffffffu, up0 || up1)) {
        const float mn0 = up0 ? mx0 : m_run[nt][0], mn1 = up1 ? mx1 : m_run[nt][1];
        const float al0 = up0 ? fast_exp2(m_run[nt][0] - mn0) : 1.f;  // exp2(-inf) = 0 on the first tokens
        const float al1 = up1 ? fast_exp2(m_run[nt][1] - mn1) : 1.f;
        m_run[nt][0] = mn0;
        m_run[nt][1] = mn1;
        l_run[nt][0] *= al0;
        l_run[nt][1] *= al1;
#pragma unroll
        for (int xx = 0; xx < 8; ++xx) {
          o[nt][xx][0] *= al0;
          o[nt][xx][1] *= al1;
          o[nt][xx][2] *= al0;
          o[nt][xx][3] *= al1;
        }
        wsum[nt][0] *= al0;
        wsum[nt][1] *= al1;
      }
      // m_run is -inf only while every logit of the row so far was masked
      const float mu0 = m_run[nt][0] == -INFINITY ? 0.f : m_run[nt][0];
      const float mu1 = m_run[nt][1] == -INFINITY ? 0.f : m_run[nt][1];
      const float p00 = fast_exp2(xv[0] - mu0), p01 = fast_exp2(xv[1] - mu1);
      const float p10 = fast_exp2(xv[2] - mu0), p11 = fast_exp2(xv[3] - mu1);
      l_run[nt][0] += p00 + p10;
      l_run[nt][1] += p01 + p11;
      // P^T as the B operand: transpose the two 8x8 (token x row) blocks
      if constexpr (kBf16) {
        pb2[nt][0] = movmatrix_trans(pack_bf162(p00 * vs_lo, p01 * vs_lo));
        pb2[nt][1] = movmatrix_trans(pack_bf162(p10 * vs_hi, p11 * vs_hi));
      } else {
        pb2[nt][0] = movmatrix_trans(pack_half2(p00 * vs_lo, p01 * vs_lo));
        pb2[nt][1] = movmatrix_trans(pack_half2(p10 * vs_hi, p11 * vs_hi));
      }
    }

    // ---------------- O^T += V^T P^T: this thread converts the 16-byte chunk g
    // of token rows 2c, 2c+1, 2c+8, 2c+9 (int8); bf16 rows come transposed out of ldmatrix
    if constexpr (kBf16) {
#pragma unroll
      for (int xx = 0; xx < 8; ++xx) {
        uint32_t af[4];
        ldmatrix_x4_trans(st_addr + (voff[0] ^ (uint32_t)(2 * xx << 4)), af[0], af[1], af[2], af[3]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_bf16(o[nt][xx], af, pb2[nt][0], pb2[nt][1]);
      }
    } else {
      uint32_t vw[4][4];
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const uint4 q4 = lds128(st_addr + voff[r4]);
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
          af[0] = prmt(e < 2 ? a01 : a23, 0x64646464u, sel);
          af[1] = prmt(e < 2 ? b01 : b23, 0x64646464u, sel);
          af[2] = prmt(e < 2 ? c01 : c23, 0x64646464u, sel);
          af[3] = prmt(e < 2 ? d01 : d23, 0x64646464u, sel);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_f16(o[nt][4 * wd + e], af, pb2[nt][0], pb2[nt][1]);
        }
      }
      // V entered as code + 1152; the all-ones tile accumulates sum_t P^T so the
      // offset can be taken out when the piece is written.
      const uint32_t ones[4] = {0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) mma_f16(wsum[nt], ones, pb2[nt][0], pb2[nt][1]);
    }

    // ---------------- end of a piece: merge the four warps and write out
    if (last_of_share || mt.t == mt.T - 1) {
      const bool is_final = piece_t0 == 0 && mt.t == mt.T - 1;
      const int slot = piece_t0 > 0 ? 0 : 1;
      const int64_t row_base = ((int64_t)mt.b * a.Hkv + mt.h) * R;
      float* obuf = reinterpret_cast<float*>(&sm.kv[stage]);  // [4 warps][8 rows][128] = K and V of the stage
      float* msm = &sm.ks2[stage][0];                          // [4][8] reference maxima of the warps
      float* wsm = &sm.ks2[stage][32];                         // [4][8] weights of the warps
      float* lsm = &sm.vs[stage][0];                           // [4][8] denominators of the warps
      float* tsm = &sm.vs[stage][32];                          // [4][8] true maxima; then [8] M, [8] L, [8] Mtrue
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float l0 = l_run[nt][0], l1 = l_run[nt][1];
#pragma unroll
        for (int sh = 4; sh <= 16; sh <<= 1) {
          l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
          l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
        }
        __syncthreads();  // every warp is done with the tile (and with the previous pass)
        if constexpr (kBf16) {
          // accumulator x holds d = 16 x + g and 16 x + 8 + g of rows 2c, 2c+1; the
          // column is XORed with 8 c so that the 32 lanes of a store hit 32 banks
          float* d0 = obuf + (warp * 8 + 2 * c) * kD;
          float* d1 = d0 + kD;
#pragma unroll
          for (int xx = 0; xx < 8; ++xx) {
            const int col = (16 * xx + g) ^ (8 * c);
            d0[col] = o[nt][xx][0];
            d1[col] = o[nt][xx][1];
            d0[col ^ 8] = o[nt][xx][2];
            d1[col ^ 8] = o[nt][xx][3];
          }
        } else {
          const float w0 = 1152.f * wsum[nt][0], w1 = 1152.f * wsum[nt][1];
          float4* d0 = reinterpret_cast<float4*>(obuf + ((warp * 8 + 2 * c) * kD) + 16 * g);
          float4* d1 = reinterpret_cast<float4*>(obuf + ((warp * 8 + 2 * c + 1) * kD) + 16 * g);
          d0[0] = make_float4(o[nt][0][0] - w0, o[nt][1][0] - w0, o[nt][2][0] - w0, o[nt][3][0] - w0);
          d0[1] = make_float4(o[nt][4][0] - w0, o[nt][5][0] - w0, o[nt][6][0] - w0, o[nt][7][0] - w0);
          d0[2] = make_float4(o[nt][0][2] - w0, o[nt][1][2] - w0, o[nt][2][2] - w0, o[nt][3][2] - w0);
          d0[3] = make_float4(o[nt][4][2] - w0, o[nt][5][2] - w0, o[nt][6][2] - w0, o[nt][7][2] - w0);
          d1[0] = make_float4(o[nt][0][1] - w1, o[nt][1][1] - w1, o[nt][2][1] - w1, o[nt][3][1] - w1);
          d1[1] = make_float4(o[nt][4][1] - w1, o[nt][5][1] - w1, o[nt][6][1] - w1, o[nt][7][1] - w1);
          d1[2] = make_float4(o[nt][0][3] - w1, o[nt][1][3] - w1, o[nt][2][3] - w1, o[nt][3][3] - w1);
          d1[3] = make_float4(o[nt][4][3] - w1, o[nt][5][3] - w1, o[nt][6][3] - w1, o[nt][7][3] - w1);
        }
        {
          if (g == 0) {
            msm[warp * 8 + 2 * c] = m_run[nt][0];
            msm[warp * 8 + 2 * c + 1] = m_run[nt][1];
            lsm[warp * 8 + 2 * c] = l0;
            lsm[warp * 8 + 2 * c + 1] = l1;
            tsm[warp * 8 + 2 * c] = m_true[nt][0];
            tsm[warp * 8 + 2 * c + 1] = m_true[nt][1];
          }
        }
        __syncthreads();
        float rM = 0.f, rL = 0.f, rT = 0.f;
        if (tid < 32) {  // thread (w, r): weight of warp w for row r; w == 0 also reduces the row
          const int w = tid >> 3, r = tid & 7;
          const float M = fmaxf(fmaxf(msm[r], msm[8 + r]), fmaxf(msm[16 + r], msm[24 + r]));
          const float mw = msm[w * 8 + r];
          wsm[w * 8 + r] = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
          if (w == 0) {
            float L = 0.f;
#pragma unroll
            for (int ww = 0; ww < 4; ++ww) {
              const float m2 = msm[ww * 8 + r];
              L += (m2 == -INFINITY ? 0.f : fast_exp2(m2 - M)) * lsm[ww * 8 + r];
            }
            rM = M;
            rL = L;
            rT = fmaxf(fmaxf(tsm[r], tsm[8 + r]), fmaxf(tsm[16 + r], tsm[24 + r]));
          }
        }
        __syncthreads();
        if (tid < 8) {  // after the barrier: the reduced rows replace the per-warp true maxima
          tsm[tid] = rM;
          tsm[8 + tid] = rL;
          tsm[16 + tid] = rT;
        }
        __syncthreads();
        const int rows_here = min(8, R - 8 * nt);
        for (int r = 0; r < rows_here; ++r) {
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < 4; ++w) acc += wsm[w * 8 + r] * obuf[(w * 8 + r) * kD + (kBf16 ? tid ^ (8 * (r >> 1)) : tid)];
          const int rr = 8 * nt + r;
          const float M = tsm[r], L = tsm[8 + r], Mt = tsm[16 + r];
          if (is_final) {
            const int64_t row = row_base + rr;
            static_cast<__nv_bfloat16*>(a.o)[row * kD + tid] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
            if (tid == 0) {
              if (a.m) a.m[row] = Mt * kLn2;
              if (a.l) a.l[row] = L > 0.f ? L * fast_exp2(M - Mt) : 0.f;
            }
          } else {
            const int64_t pr = ((int64_t)cta * 2 + slot) * kMaxRows + rr;
            __stcg(&x.part_o[pr * kD + tid], acc);
            if (tid == 0) {
              __stcg(&x.part_m[pr], M);
              __stcg(&x.part_l[pr], L);
              __stcg(&x.part_t[pr], Mt);
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
          s_flag = old == (unsigned)(mt.parts - 1);
        }
        __syncthreads();
        if (s_flag) {
          __threadfence();
          merge_segment(a, x, mt.first_cta, mt.parts, row_base);
        }
      }
      // The next iteration's barrier orders these reads before the stage is refilled.
    }
    stage = next_stage;
  }
  cp_async_wait<0>();
#ifdef JPT_ATTN_TIMING
  if (tid == 0 && cta < 4096) {
    g_attn_timing[4 * cta + 1] = globaltimer_ns();
    g_attn_timing[4 * cta + 3] = (unsigned long long)dbg_tiles | ((unsigned long long)dbg_pieces << 32);
  }
#endif
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

}  // namespace

int launch_mask_ranges(const AttnArgs& a, const MmaScratch& x, cudaStream_t st) {
  mask_ranges_kernel<<<a.B, kThreads, 0, st>>>(a, x);
  return check_launch("mask_ranges_kernel");
}

bool attention_mma_eligible(const jpt_attn_params& p) {
  const int R = (p.Hq / p.Hkv) * p.Tq;
  if (p.D != kD || R > kMaxRows || p.q_dtype != JPT_BF16) return false;
  if (p.kv_dtype != JPT_INT8 && p.kv_dtype != JPT_BF16) return false;
  if (p.mask_mode == JPT_MASK_ADD && p.mk_r != 0) return false;  // per-row masks: scalar kernel
  if (!aligned(p.q, 16) || !aligned(p.k, 16) || !aligned(p.v, 16)) return false;
  if (p.paged) {
    if (p.kv_h % 16 || p.kv_page % 16) return false;
  } else if (p.kv_b % 16 || p.kv_h % 16 || p.kv_s % 16) {
    return false;
  }
  // the merge of a segment's pieces keeps (pieces + 3) * 16 floats in a 16 KB buffer
  if (p.S > 16000) return false;
  if ((size_t)p.B * p.Hkv > kWorkspaceMaxSegments) return false;
  // slot indices are 32-bit
  if ((double)p.B * p.Hkv * ((double)p.S / kTile + 1 + kPieceCost) > 1.0e9) return false;
  return true;
}

// Persistent CTAs per launch: as many as fit on the device at once.
static int mma_num_ctas(const jpt_attn_params& p) {
  const int R = (p.Hq / p.Hkv) * p.Tq;
  return sm_count() * (R > 8 ? 2 : (p.kv_dtype == JPT_BF16 ? 3 : 4));
}

size_t attention_mma_workspace_bytes(const jpt_attn_params& p) { return scratch_layout(p, mma_num_ctas(p)).total; }

int launch_attention_mma(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st) {
  const ScratchLayout lay = scratch_layout(p, mma_num_ctas(p));
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

  static std::atomic<bool> configured[kMaxDevices];
  if (int rc = configure_once_per_device(configured, "flash_decode_kernel", [] {
        cudaError_t e = cudaFuncSetAttribute(flash_decode_kernel<false, false>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem<false, false>));
        if (e == cudaSuccess)
          e = cudaFuncSetAttribute(flash_decode_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)sizeof(Smem<true, false>));
        if (e == cudaSuccess)
          e = cudaFuncSetAttribute(flash_decode_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)sizeof(Smem<false, true>));
        if (e == cudaSuccess)
          e = cudaFuncSetAttribute(flash_decode_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)sizeof(Smem<true, true>));
        return e;
      }))
    return rc;
  if (a.mask_mode == JPT_MASK_ADD) {
    if (int rc = launch_mask_ranges(a, x, st)) return rc;
  }
  const bool bf16 = p.kv_dtype == JPT_BF16;
  if (a.R > 8) {
    if (bf16) flash_decode_kernel<true, true><<<lay.num_ctas, kThreads, sizeof(Smem<true, true>), st>>>(a, x);
    else flash_decode_kernel<true, false><<<lay.num_ctas, kThreads, sizeof(Smem<true, false>), st>>>(a, x);
  } else {
    if (bf16) flash_decode_kernel<false, true><<<lay.num_ctas, kThreads, sizeof(Smem<false, true>), st>>>(a, x);
    else flash_decode_kernel<false, false><<<lay.num_ctas, kThreads, sizeof(Smem<false, false>), st>>>(a, x);
  }
  return check_launch("flash_decode_kernel");
}

}  // namespace jpt

#ifdef JPT_ATTN_TIMING
// Debug builds only: per-CTA (start ns, end ns, SM id, tiles | pieces << 32) of the last launch.
extern "C" int jpt_debug_attn_timing(unsigned long long* out_host, int n_ctas) {
  return (int)cudaMemcpyFromSymbol(out_host, jpt::g_attn_timing, sizeof(unsigned long long) * 4 * n_ctas);
}
#endif
