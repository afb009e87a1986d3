// Pieces shared by the persistent tensor-core decode-attention kernels: the
// scratch handed to a launch, the record a producer publishes per tile, the
// merge of a segment's partial results, and the host-side scratch layout.
#pragma once

#include <limits.h>
#include <math.h>

#include <atomic>

#include "attention_common.cuh"

namespace jpt {

constexpr int kThreads = 128;
constexpr int kD = 128;
constexpr int kMaxRows = 16;
constexpr int kPieceCost = 1;  // overhead slots charged per segment, in tiles
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Scratch handed to the kernel (all inside the caller's workspace).
struct MmaScratch {
  unsigned* counters;  // [B * Hkv] wrapping arrival counters, zero between launches
  int32_t* seqinfo;    // [B][4] (first, n, use_add, -) for additive masks
  float* part_o;       // [num_ctas][2][16][128] unnormalised partial outputs
  float* part_m;       // [num_ctas][2][16] reference maximum (log2 domain)
  float* part_l;       // [num_ctas][2][16] sum of exp2(x - reference)
  float* part_t;       // [num_ctas][2][16] true maximum (log2 domain)
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
__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(r) : "f"(x));
  return r;
}


// What the producer publishes about the tile it put into a stage.
struct TileMeta {
  int b, h;        // sequence, KV head
  int t, T;        // tile inside the segment (-1: no tile, the CTA's share is exhausted), tiles of the segment
  int n, first;    // valid tokens of the sequence and position of its first one
  int use_add;     // additive mask values must be applied
  int first_cta;   // CTA that holds tile 0 of the segment
  int parts;       // number of CTAs the segment is spread over
  int pad[3];
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

// Combine the `parts` partials of one segment (CTAs first .. first+parts-1) and
// write its R final rows.  Called by 128 threads (threadIdx.x 0..127): thread t
// owns head-dim index t of every row
// and the rows' statistics travel by warp shuffles, so there is no staging in
// shared memory and no barrier; two pieces are combined per step with all of
// their loads in flight at once (one L2 round trip for the usual two pieces).
struct NoMergeHook {
  template <typename A>
  __device__ __forceinline__ void operator()(A&, A&, A&) const {}
};

// `hook(M, L, acc)` runs after the pieces are combined and before the rows are
// written: M[r] the maximum (log2 domain) and L[r] the denominator of row r
// (equal in every thread), acc[r] this thread's head-dim component of the
// unnormalised output.  It may change all three, the same way in every thread
// (the tcgen05 kernel adds the decode step's new token there), and is called by
// all 128 threads.
template <int kR, typename Hook>
static __device__ __forceinline__ void merge_rows(const AttnArgs& a, const MmaScratch& x, int first, int parts, int64_t row_base,
                                                  Hook& hook) {
  const int tid = threadIdx.x, lane = tid & 31, R = a.R;
  // Lane r of every warp keeps row r's statistics (reference maximum, denominator relative to
  // it, true maximum) and hands the weights to the other lanes by shuffles.
  const bool mine = lane < R;
  float Mr = -INFINITY, Lr = 0.f, Tr = -INFINITY;
  float acc[kR];
#pragma unroll
  for (int r = 0; r < kR; ++r) acc[r] = 0.f;
  for (int pi = 0; pi < parts; pi += 2) {
    const bool two = pi + 1 < parts;
    const int64_t i0 = ((int64_t)(first + pi) * 2 + (pi == 0 ? 1 : 0)) * kMaxRows;
    const int64_t i1 = ((int64_t)(first + pi + 1) * 2) * kMaxRows;
    const float m0 = mine ? __ldcg(x.part_m + i0 + lane) : -INFINITY;
    const float l0 = mine ? __ldcg(x.part_l + i0 + lane) : 0.f;
    const float t0 = mine ? __ldcg(x.part_t + i0 + lane) : -INFINITY;
    const float m1 = (mine && two) ? __ldcg(x.part_m + i1 + lane) : -INFINITY;
    const float l1 = (mine && two) ? __ldcg(x.part_l + i1 + lane) : 0.f;
    const float t1 = (mine && two) ? __ldcg(x.part_t + i1 + lane) : -INFINITY;
    float v0[kR], v1[kR];
#pragma unroll
    for (int r = 0; r < kR; ++r) {
      v0[r] = r < R ? __ldcg(x.part_o + (i0 + r) * kD + tid) : 0.f;
      v1[r] = (two && r < R) ? __ldcg(x.part_o + (i1 + r) * kD + tid) : 0.f;
    }
    const float mn = fmaxf(Mr, fmaxf(m0, m1));
    const float s = Mr == -INFINITY ? 0.f : fast_exp2(Mr - mn);
    const float w0 = m0 == -INFINITY ? 0.f : fast_exp2(m0 - mn);
    const float w1 = m1 == -INFINITY ? 0.f : fast_exp2(m1 - mn);
    Lr = Lr * s + w0 * l0 + w1 * l1;
    Mr = mn;
    Tr = fmaxf(Tr, fmaxf(t0, t1));
#pragma unroll
    for (int r = 0; r < kR; ++r) {
      const float S = __shfl_sync(0xffffffffu, s, r), W0 = __shfl_sync(0xffffffffu, w0, r), W1 = __shfl_sync(0xffffffffu, w1, r);
      acc[r] = acc[r] * S + W0 * v0[r] + W1 * v1[r];
    }
  }
  // the denominator and the output relative to the true maximum, which is what gets reported
  const float c = Lr > 0.f ? fast_exp2(Mr - Tr) : 0.f;
  Lr *= c;
  Mr = Tr;
  float M[kR], L[kR];
#pragma unroll
  for (int r = 0; r < kR; ++r) {
    acc[r] *= __shfl_sync(0xffffffffu, c, r);
    M[r] = __shfl_sync(0xffffffffu, Mr, r);
    L[r] = __shfl_sync(0xffffffffu, Lr, r);
  }
  hook(M, L, acc);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.o);
#pragma unroll
  for (int r = 0; r < kR; ++r) {
    if (r < R) {
      if (tid == r) {
        if (a.m) a.m[row_base + r] = M[r] * kLn2;
        if (a.l) a.l[row_base + r] = L[r];
      }
      o[(row_base + r) * kD + tid] = __float2bfloat16_rn(L[r] > 0.f ? acc[r] / L[r] : 0.f);
    }
  }
}

template <typename Hook = NoMergeHook>
static __device__ void merge_segment(const AttnArgs& a, const MmaScratch& x, int first, int parts, int64_t row_base,
                                     Hook hook = Hook()) {
  if (a.R <= 8) {
    merge_rows<8>(a, x, first, parts, row_base, hook);
  } else {
    merge_rows<kMaxRows>(a, x, first, parts, row_base, hook);
  }
}

// Per-device facts are kept per device ordinal: a process may drive several GPUs.
constexpr int kMaxDevices = 64;

inline int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  return dev;
}

inline int sm_count() {
  static std::atomic<int> n[kMaxDevices];
  const int dev = current_device();
  int v = n[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

// Runs `configure` (which returns a cudaError_t) once per device, with that
// device current; cudaFuncSetAttribute applies to the current device only.
// Returns 0 or the positive CUDA error of a failed configuration (not cached,
// so the next call tries again).
template <typename F>
inline int configure_once_per_device(std::atomic<bool> (&done)[kMaxDevices], const char* what, F configure) {
  const int dev = current_device();
  if (done[dev].load(std::memory_order_acquire)) return 0;
  const cudaError_t e = configure();
  if (e != cudaSuccess) return fail((int)e, "%s: configuring the kernel on device %d: %s", what, dev, cudaGetErrorString(e));
  done[dev].store(true, std::memory_order_release);
  return 0;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct ScratchLayout {
  size_t counters, seqinfo, exchange, part_m, part_l, part_t, part_o, total;
  int num_ctas;
};

// Exchange area of one rank for the per-token amax of a decode step: 64 bytes of
// state {launches done, CTAs done, gave up}, then slots[parity][writer rank][2 B]
// of 64-bit words.  The same layout serves jpt_peer_exchange buffers.
constexpr size_t kExchangeStateBytes = 64;
inline size_t exchange_bytes(int B, int world) {
  return kExchangeStateBytes + (size_t)2 * world * 2 * B * sizeof(unsigned long long);
}

// Layout of the scratch of a persistent launch of `num_ctas` CTAs.
inline ScratchLayout scratch_layout(const jpt_attn_params& p, int num_ctas) {
  ScratchLayout s;
  s.num_ctas = num_ctas;
  size_t off = 0;
  s.counters = off;  // fixed-size header shared by every shape that uses the workspace
  off = kWorkspaceCounterBytes;
  s.seqinfo = off;
  off = align_up(off + sizeof(int32_t) * 4 * p.B, 256);
  s.exchange = kWorkspaceExchangeOffset;  // one-GPU exchange slots of the fused update, inside the header
  s.part_m = off;
  off = align_up(off + sizeof(float) * s.num_ctas * 2 * kMaxRows, 256);
  s.part_l = off;
  off = align_up(off + sizeof(float) * s.num_ctas * 2 * kMaxRows, 256);
  s.part_t = off;
  off = align_up(off + sizeof(float) * s.num_ctas * 2 * kMaxRows, 256);
  s.part_o = off;
  off = align_up(off + sizeof(float) * s.num_ctas * 2 * kMaxRows * kD, 256);
  s.total = off;
  return s;
}

// Additive masks -> valid ranges in x.seqinfo (one CTA per sequence).
int launch_mask_ranges(const AttnArgs& a, const MmaScratch& x, cudaStream_t st);

}  // namespace jpt
