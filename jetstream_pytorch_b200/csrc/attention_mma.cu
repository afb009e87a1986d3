// Ragged flash-decode attention for head_dim 128 on tensor cores (sm_100a).
//
// One CTA (4 warps) walks a contiguous range of 64-token tiles of one
// (sequence, KV head) pair.  K and V tiles travel global -> shared memory with
// 16-byte cp.async copies through a 4-stage ring; each warp owns 16 tokens of
// a tile and keeps its own online-softmax state for the up to 16 query rows of
// the KV group (rep * Tq), which are the M dimension of mma.sync.m16n8k16:
//   S[rows x 8 tokens]  = Q[rows x 16 d] . K^T      (8 k-steps over d)
//   O[rows x 8 d]      += P[rows x 16 tokens] . V   (16 n-tiles over d)
// The C-fragment layout of S is the A-fragment layout of P, so probabilities
// never leave registers.  Warps are merged through shared memory at the end and
// the CTA writes either the final rows or a split-K partial.
//
// int8 caches: a code x is turned into fp16 without a convert instruction:
// (x ^ 0x80) is x + 128 as an unsigned byte and 0x6400 | byte is the fp16 number
// 1024 + byte, so one PRMT builds two halves worth x + 1152.  For K the offset
// is removed after the dot product (S - 1152 * sum_d q_d); for V it is removed
// with one HSUB2 so that the accumulators only ever hold the signal.  Because
// the contraction index may be permuted freely, head_dim is assigned to MMA
// slots so that every thread reads whole 16-byte chunks of a token row (see
// the d(...) comments below); outputs are un-permuted when they are written.
#include <limits.h>
#include <math.h>

#include "attention_common.cuh"

namespace jpt {
namespace {

constexpr int kTile = 64;     // tokens per pipeline stage
constexpr int kStages = 4;
constexpr int kThreads = 128;
constexpr int kD = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

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

// Shared memory of one CTA.
struct __align__(128) SmemI8 {
  uint8_t k[kStages][kTile * kD];  // rows of 128 bytes, 16-byte chunks XOR-swizzled by (row & 7)
  uint8_t v[kStages][kTile * kD];
  float ks2[kStages][kTile];       // k_scale * sm_scale * log2(e)
  float vs[kStages][kTile];        // v_scale
  float mk2[kStages][kTile];       // additive mask * log2(e)
};

// Row address pieces of one logical token.
struct TokAddr {
  int64_t off;   // element offset of the K/V row
  int64_t sidx;  // scale index
  int pos;       // physical position (mask index)
  bool valid;
};

__device__ __forceinline__ TokAddr tok_addr(const AttnArgs& a, const SeqRange& rg, int b, int h, int j) {
  TokAddr t;
  t.valid = j < rg.n;
  const int jj = t.valid ? j : 0;
  t.pos = physical_pos(a, rg, jj);
  t.off = kv_row_offset(a, b, h, t.pos, &t.sidx);
  return t;
}

template <bool kRows16>
__global__ void __launch_bounds__(kThreads, 3) flash_decode_i8_kernel(AttnArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  SmemI8& sm = *reinterpret_cast<SmemI8*>(smem_raw);

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int R = a.R;
  const bool quant = a.k_scale != nullptr;
  const bool add_mask = a.mask_mode == JPT_MASK_ADD;

  const SeqRange rg = seq_range(a, b);
  const int ntiles = (rg.n + kTile - 1) / kTile;
  int t0 = (int)(((long long)split * ntiles) / a.nsplit);
  int t1 = (int)(((long long)(split + 1) * ntiles) / a.nsplit);

  const int64_t row_base = ((int64_t)b * a.Hkv + h) * R;  // first output row of this KV group
  const __nv_bfloat16* mask = static_cast<const __nv_bfloat16*>(a.mask);

  // ---- query fragments (fp16) with the K-side head_dim assignment:
  // k-step j, slots {2c, 2c+1, 2c+8, 2c+9}  <->  d = 32c + 4j + {0, 1, 2, 3}
  uint32_t qa[8][4];
  float bias_lo = 0.f, bias_hi = 0.f;  // 1152 * sum_d q[row][d] for rows g and g+8
  {
    const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(a.q) + row_base * kD;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = g + 8 * half;
      float sum = 0.f;
      if ((half == 0 || kRows16) && row < R) {
        const uint4* src = reinterpret_cast<const uint4*>(q + (int64_t)row * kD + 32 * c);
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // 8 bf16 per 16-byte load = k-steps 2i and 2i+1
          const uint4 raw = src[i];
          const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
          float2 f0 = __bfloat1622float2(p2[0]), f1 = __bfloat1622float2(p2[1]);
          float2 f2 = __bfloat1622float2(p2[2]), f3 = __bfloat1622float2(p2[3]);
          const __half2 h0 = __floats2half2_rn(f0.x, f0.y), h1 = __floats2half2_rn(f1.x, f1.y);
          const __half2 h2 = __floats2half2_rn(f2.x, f2.y), h3 = __floats2half2_rn(f3.x, f3.y);
          qa[2 * i][half] = *reinterpret_cast<const uint32_t*>(&h0);
          qa[2 * i][2 + half] = *reinterpret_cast<const uint32_t*>(&h1);
          qa[2 * i + 1][half] = *reinterpret_cast<const uint32_t*>(&h2);
          qa[2 * i + 1][2 + half] = *reinterpret_cast<const uint32_t*>(&h3);
          const float2 r0 = __half22float2(h0), r1 = __half22float2(h1), r2 = __half22float2(h2),
                       r3 = __half22float2(h3);
          sum += (r0.x + r0.y) + (r1.x + r1.y) + (r2.x + r2.y) + (r3.x + r3.y);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          qa[j][half] = 0u;
          qa[j][2 + half] = 0u;
        }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      // int8 codes enter the MMA as x + 1152: remove 1152 * sum_d q_d afterwards
      if (half == 0) bias_lo = 1152.f * sum;
      else bias_hi = 1152.f * sum;
    }
  }
  (void)bias_hi;

  // ---- additive masks: shrink the tile range to the span that holds any
  // finite mask value (causal and ring masks are one or two runs of zeros)
  if (add_mask && t1 > t0) {
    int lo = INT_MAX, hi = -1;
    for (int j = t0 * kTile + tid; j < min(t1 * kTile, rg.n); j += kThreads) {
      const float mv = __bfloat162float(mask[(int64_t)b * a.mk_b + j]);
      if (mv != -INFINITY) {
        lo = min(lo, j);
        hi = max(hi, j);
      }
    }
    __shared__ int s_lo, s_hi;
    if (tid == 0) {
      s_lo = INT_MAX;
      s_hi = -1;
    }
    __syncthreads();
    atomicMin(&s_lo, lo);
    atomicMax(&s_hi, hi);
    __syncthreads();
    if (s_hi < 0) {
      t1 = t0;
    } else {
      t0 = s_lo / kTile;
      t1 = s_hi / kTile + 1;
    }
  }

  // ---- producer: one tile = 512 + 512 16-byte chunks, 4 + 4 per thread
  const int8_t* kbase = static_cast<const int8_t*>(a.k);
  const int8_t* vbase = static_cast<const int8_t*>(a.v);
  float pend_a = 0.f, pend_b = 0.f;  // side data loaded one iteration ahead
  int pend_stage = -1;

  auto issue_tile = [&](int t, int stage) {
    const int col = tid & 7;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = (tid >> 3) + 16 * i;
      const TokAddr ta = tok_addr(a, rg, b, h, t * kTile + row);
      const uint32_t dst = (uint32_t)(row * kD + ((col ^ (row & 7)) << 4));
      cp_async16(smem_u32(&sm.k[stage][0]) + dst, kbase + ta.off + col * 16, ta.valid);
      cp_async16(smem_u32(&sm.v[stage][0]) + dst, vbase + ta.off + col * 16, ta.valid);
    }
    if (quant || add_mask) {
      const int tok = tid & 63;
      const TokAddr ta = tok_addr(a, rg, b, h, t * kTile + tok);
      pend_a = 1.f;
      pend_b = 0.f;
      if (ta.valid) {
        if (quant) pend_a = load_scale(tid < 64 ? a.k_scale : a.v_scale, ta.sidx, a.scale_is_f32);
        if (add_mask && tid < 64) pend_b = __bfloat162float(mask[(int64_t)b * a.mk_b + ta.pos]);
      }
      pend_stage = stage;
    }
  };
  auto flush_side = [&]() {
    if (pend_stage >= 0) {
      const int tok = tid & 63;
      if (tid < 64) {
        sm.ks2[pend_stage][tok] = pend_a * a.sm_scale * kLog2e;
        sm.mk2[pend_stage][tok] = pend_b * kLog2e;
      } else {
        sm.vs[pend_stage][tok] = pend_a;
      }
      pend_stage = -1;
    }
  };

  // ---- per-warp online softmax state
  float o[16][4];
#pragma unroll
  for (int x = 0; x < 16; ++x) o[x][0] = o[x][1] = o[x][2] = o[x][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  const float unit2 = a.sm_scale * kLog2e;

  for (int s = 0; s < kStages - 1; ++s) {
    if (t0 + s < t1) {
      flush_side();
      issue_tile(t0 + s, s);
    }
    cp_async_commit();
  }

  for (int t = t0; t < t1; ++t) {
    const int stage = (t - t0) % kStages;
    cp_async_wait<kStages - 2>();
    flush_side();
    __syncthreads();
    {
      const int tn = t + kStages - 1;
      if (tn < t1) issue_tile(tn, (tn - t0) % kStages);
      cp_async_commit();
    }
    // The side data of the tile consumed now was flushed at least one barrier
    // ago unless the range is shorter than the ring; the barrier above covers
    // that case because flush_side() runs before it.

    const uint32_t ks_addr = smem_u32(&sm.k[stage][0]);
    const uint32_t vs_addr = smem_u32(&sm.v[stage][0]);
    const int tok0 = warp * 16;  // first token of this warp inside the tile

    // ---- S = Q K^T for 16 tokens (two n-tiles of 8)
    float sc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
      const int row = tok0 + 8 * nt + g;
      const uint32_t rbase = ks_addr + row * kD;
      const uint4 k0 = lds128(rbase + (((2 * c) ^ (row & 7)) << 4));
      const uint4 k1 = lds128(rbase + (((2 * c + 1) ^ (row & 7)) << 4));
      const uint32_t w[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t x = w[j] ^ 0x80808080u;
        const uint32_t b0 = prmt(x, 0x64646464u, 0x5140u);
        const uint32_t b1 = prmt(x, 0x64646464u, 0x5342u);
        mma_f16(sc[nt], qa[j], b0, b1);
      }
    }

    // ---- logits (log2 domain), masking, online softmax
    float x_lo[4], x_hi[4];
    const int jbase = t * kTile + tok0;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tok = tok0 + 8 * nt + 2 * c + e;
        const bool valid = (jbase + 8 * nt + 2 * c + e) < rg.n;
        const float sk = (quant || add_mask) ? sm.ks2[stage][tok] : unit2;
        const float mk = add_mask ? sm.mk2[stage][tok] : 0.f;
        x_lo[2 * nt + e] = valid ? (sc[nt][e] - bias_lo) * sk + mk : -INFINITY;
        if (kRows16) x_hi[2 * nt + e] = valid ? (sc[nt][2 + e] - bias_hi) * sk + mk : -INFINITY;
      }
    }
    float mx_lo = fmaxf(fmaxf(x_lo[0], x_lo[1]), fmaxf(x_lo[2], x_lo[3]));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo);
    const float mu_lo = mn_lo == -INFINITY ? 0.f : mn_lo;
    const float al_lo = fast_exp2(m_lo - mu_lo);
    m_lo = mn_lo;
    float al_hi = 1.f, mu_hi = 0.f;
    if (kRows16) {
      float mx_hi = fmaxf(fmaxf(x_hi[0], x_hi[1]), fmaxf(x_hi[2], x_hi[3]));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_hi = fmaxf(m_hi, mx_hi);
      mu_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      al_hi = fast_exp2(m_hi - mu_hi);
      m_hi = mn_hi;
    }
    float p_lo[4], p_hi[4];
    float ps_lo = 0.f, ps_hi = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      p_lo[i] = fast_exp2(x_lo[i] - mu_lo);
      ps_lo += p_lo[i];
      if (kRows16) {
        p_hi[i] = fast_exp2(x_hi[i] - mu_hi);
        ps_hi += p_hi[i];
      } else {
        p_hi[i] = 0.f;
      }
    }
    l_lo = l_lo * al_lo + ps_lo;
    if (kRows16) l_hi = l_hi * al_hi + ps_hi;
    if (__any_sync(0xffffffffu, al_lo != 1.f || al_hi != 1.f)) {
#pragma unroll
      for (int x = 0; x < 16; ++x) {
        o[x][0] *= al_lo;
        o[x][1] *= al_lo;
        if (kRows16) {
          o[x][2] *= al_hi;
          o[x][3] *= al_hi;
        }
      }
    }
    uint32_t pa[4];
    {
      float vsc[4] = {1.f, 1.f, 1.f, 1.f};
      if (quant) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          vsc[2 * nt] = sm.vs[stage][tok0 + 8 * nt + 2 * c];
          vsc[2 * nt + 1] = sm.vs[stage][tok0 + 8 * nt + 2 * c + 1];
        }
      }
      pa[0] = pack_half2(p_lo[0] * vsc[0], p_lo[1] * vsc[1]);
      pa[1] = pack_half2(p_hi[0] * vsc[0], p_hi[1] * vsc[1]);
      pa[2] = pack_half2(p_lo[2] * vsc[2], p_lo[3] * vsc[3]);
      pa[3] = pack_half2(p_hi[2] * vsc[2], p_hi[3] * vsc[3]);
    }

    // ---- O += P V.  n-tile x, column n  <->  d = 16 n + x, so the thread that
    // supplies column g reads the 16-byte chunk g of its four token rows
    // (tokens 2c, 2c+1, 2c+8, 2c+9 of the warp's 16).
    {
      uint32_t vw[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = tok0 + 2 * c + (i & 1) + 8 * (i >> 1);
        const uint4 r4 = lds128(vs_addr + row * kD + ((g ^ (row & 7)) << 4));
        vw[i][0] = r4.x; vw[i][1] = r4.y; vw[i][2] = r4.z; vw[i][3] = r4.w;
      }
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        const uint32_t A = vw[0][wd] ^ 0x80808080u, Bw = vw[1][wd] ^ 0x80808080u;
        const uint32_t C = vw[2][wd] ^ 0x80808080u, Dw = vw[3][wd] ^ 0x80808080u;
        const uint32_t p01 = prmt(A, Bw, 0x5140u), p23 = prmt(A, Bw, 0x7362u);
        const uint32_t q01 = prmt(C, Dw, 0x5140u), q23 = prmt(C, Dw, 0x7362u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t sel = (e & 1) ? 0x5342u : 0x5140u;
          const uint32_t b0 = hsub2_u32(prmt(e < 2 ? p01 : p23, 0x64646464u, sel), 0x64806480u);
          const uint32_t b1 = hsub2_u32(prmt(e < 2 ? q01 : q23, 0x64646464u, sel), 0x64806480u);
          mma_f16(o[4 * wd + e], pa, b0, b1);
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the four warps through shared memory (the pipeline buffers are free now)
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  if (kRows16) {
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  }
  constexpr int kRowsMax = kRows16 ? 16 : 8;
  float* osm = reinterpret_cast<float*>(smem_raw);             // [4 warps][kRowsMax][128]
  float* msm = osm + 4 * kRowsMax * kD;                         // [4][kRowsMax]
  float* lsm = msm + 4 * kRowsMax;                              // [4][kRowsMax]
  {
    float* dst = osm + ((int64_t)warp * kRowsMax + g) * kD + 32 * c;
#pragma unroll
    for (int x = 0; x < 16; ++x) {
      dst[x] = o[x][0];
      dst[16 + x] = o[x][1];
      if (kRows16) {
        dst[8 * kD + x] = o[x][2];
        dst[8 * kD + 16 + x] = o[x][3];
      }
    }
    if (c == 0) {
      msm[warp * kRowsMax + g] = m_lo;
      lsm[warp * kRowsMax + g] = l_lo;
      if (kRows16) {
        msm[warp * kRowsMax + g + 8] = m_hi;
        lsm[warp * kRowsMax + g + 8] = l_hi;
      }
    }
  }
  __syncthreads();
  const int d = tid;  // 128 threads <-> 128 head_dim columns
  for (int r = 0; r < R; ++r) {
    float M = msm[r];
#pragma unroll
    for (int w = 1; w < 4; ++w) M = fmaxf(M, msm[w * kRowsMax + r]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = msm[w * kRowsMax + r];
      const float wg = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
      L += wg * lsm[w * kRowsMax + r];
      acc += wg * osm[((int64_t)w * kRowsMax + r) * kD + d];
    }
    const int64_t row = row_base + r;
    if (a.nsplit == 1) {
      static_cast<__nv_bfloat16*>(a.o)[row * kD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
      if (d == 0) {
        if (a.m) a.m[row] = M * kLn2;
        if (a.l) a.l[row] = L;
      }
    } else {
      a.ws_o[(row * a.nsplit + split) * kD + d] = acc;
      if (d == 0) {
        a.ws_m[row * a.nsplit + split] = M * kLn2;
        a.ws_l[row * a.nsplit + split] = L;
      }
    }
  }
}

}  // namespace

bool attention_mma_eligible(const jpt_attn_params& p) {
  const int R = (p.Hq / p.Hkv) * p.Tq;
  if (p.D != kD || R > 16 || p.q_dtype != JPT_BF16 || p.kv_dtype != JPT_INT8) return false;
  if (p.mask_mode == JPT_MASK_ADD && p.mk_r != 0) return false;  // per-row masks: scalar kernel
  if (!aligned(p.q, 16) || !aligned(p.k, 16) || !aligned(p.v, 16)) return false;
  if (p.paged) {
    if (p.kv_h % 16 || p.kv_page % 16) return false;
  } else if (p.kv_b % 16 || p.kv_h % 16 || p.kv_s % 16) {
    return false;
  }
  return true;
}

int attention_mma_pick_splits(const jpt_attn_params& p) {
  // Enough CTAs for a few waves over 148 SMs x 3 resident CTAs, at most one
  // split per 256 tokens of cache length.
  const long base = (long)p.B * p.Hkv;
  int want = (int)((4L * 148 * 3 + base - 1) / base);
  int maxs = (p.S + 255) / 256;
  if (want > maxs) want = maxs;
  if (want > 32) want = 32;
  return want < 1 ? 1 : want;
}

int launch_attention_mma(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st) {
  (void)p;
  dim3 grid(a.nsplit, a.Hkv, a.B);
  const size_t smem = sizeof(SmemI8);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(flash_decode_i8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(flash_decode_i8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  if (a.R > 8) {
    flash_decode_i8_kernel<true><<<grid, kThreads, smem, st>>>(a);
  } else {
    flash_decode_i8_kernel<false><<<grid, kThreads, smem, st>>>(a);
  }
  return check_launch("flash_decode_i8_kernel");
}

}  // namespace jpt
