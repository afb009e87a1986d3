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

// Barrier of the 128 threads that run merge_segment: the whole CTA, or (in a
// CTA with more warps) threads 0..127 through named barrier 2.
template <bool kWorkerGroup>
__device__ __forceinline__ void group_sync() {
  if constexpr (kWorkerGroup) {
    asm volatile("bar.sync 2, 128;" ::: "memory");
  } else {
    __syncthreads();
  }
}

// Combine the `parts` partials of one segment (CTAs first .. first+parts-1) and
// write its R final rows.  `scratch` is at least (parts + 4) * 16 floats of
// shared memory.  Called by 128 threads (threadIdx.x 0..127).
struct NoMergeHook {
  __device__ __forceinline__ void operator()(float*, float*, float (&)[kMaxRows]) const {}
};

// `hook(M, L, acc)` runs after the pieces are combined and before the rows are
// written: M[r] the maximum (log2 domain) and L[r] the denominator of row r (in
// shared memory, read by every thread), acc[r] this thread's head-dim component
// of the unnormalised output.  It may change all three (the tcgen05 kernel adds
// the decode step's new token there) and is called by all 128 threads.
template <bool kWorkerGroup = false, typename Hook = NoMergeHook>
static __device__ void merge_segment(const AttnArgs& a, const MmaScratch& x, int first, int parts, int64_t row_base,
                                     float* scratch, Hook hook = Hook()) {
  const int tid = threadIdx.x, R = a.R;
  float* s_w = scratch;                     // [parts][16] weights
  float* s_M = scratch + parts * kMaxRows;  // [16] reference maximum
  float* s_L = s_M + kMaxRows;              // [16] denominator relative to s_M
  for (int i = tid; i < parts * R; i += kThreads) {
    const int pi = i / R, r = i - pi * R;
    s_w[pi * kMaxRows + r] = __ldcg(&x.part_m[((int64_t)(first + pi) * 2 + (pi == 0 ? 1 : 0)) * kMaxRows + r]);
  }
  group_sync<kWorkerGroup>();
  if (tid < R) {
    float M = -INFINITY;
    for (int pi = 0; pi < parts; ++pi) M = fmaxf(M, s_w[pi * kMaxRows + tid]);
    s_M[tid] = M;
  }
  group_sync<kWorkerGroup>();
  for (int i = tid; i < parts * R; i += kThreads) {
    const int pi = i / R, r = i - pi * R;
    const float mw = s_w[pi * kMaxRows + r];
    s_w[pi * kMaxRows + r] = mw == -INFINITY ? 0.f : fast_exp2(mw - s_M[r]);
  }
  group_sync<kWorkerGroup>();
  if (tid < R) {
    float L = 0.f, mt = -INFINITY;
    for (int pi = 0; pi < parts; ++pi) {
      const int64_t pr = ((int64_t)(first + pi) * 2 + (pi == 0 ? 1 : 0)) * kMaxRows + tid;
      L += s_w[pi * kMaxRows + tid] * __ldcg(&x.part_l[pr]);
      mt = fmaxf(mt, __ldcg(&x.part_t[pr]));
    }
    // keep the denominator relative to the true maximum, which is what gets reported
    s_L[tid] = L > 0.f ? L * fast_exp2(s_M[tid] - mt) : 0.f;
    s_w[parts * kMaxRows + 2 * kMaxRows + tid] = L > 0.f ? fast_exp2(s_M[tid] - mt) : 0.f;  // rescale of acc
    s_M[tid] = mt;
  }
  group_sync<kWorkerGroup>();
  float acc[kMaxRows];
#pragma unroll
  for (int r = 0; r < kMaxRows; ++r) acc[r] = 0.f;
  if (R <= 8) {
    // two pieces per step: 16 independent loads in flight instead of one L2 round trip per piece
    for (int pi = 0; pi < parts; pi += 2) {
      const bool two = pi + 1 < parts;
      const float* s0 = x.part_o + (((int64_t)(first + pi) * 2 + (pi == 0 ? 1 : 0)) * kMaxRows) * kD + tid;
      const float* s1 = x.part_o + (((int64_t)(first + pi + 1) * 2) * kMaxRows) * kD + tid;
      float v0[8], v1[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        v0[r] = r < R ? __ldcg(s0 + r * kD) : 0.f;
        v1[r] = (two && r < R) ? __ldcg(s1 + r * kD) : 0.f;
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        acc[r] += s_w[pi * kMaxRows + r] * v0[r];
        if (two) acc[r] += s_w[(pi + 1) * kMaxRows + r] * v1[r];
      }
    }
  } else {
    for (int pi = 0; pi < parts; ++pi) {
      const float* src = x.part_o + (((int64_t)(first + pi) * 2 + (pi == 0 ? 1 : 0)) * kMaxRows) * kD + tid;
#pragma unroll
      for (int r = 0; r < kMaxRows; ++r) {
        if (r < R) acc[r] += s_w[pi * kMaxRows + r] * __ldcg(src + r * kD);
      }
    }
  }
  float* s_c = s_L + kMaxRows;  // [16] factor that brings acc to the true maximum
#pragma unroll
  for (int r = 0; r < kMaxRows; ++r) {
    if (r < R) acc[r] *= s_c[r];
  }
  hook(s_M, s_L, acc);
  if (tid < R) {
    if (a.m) a.m[row_base + tid] = s_M[tid] * kLn2;
    if (a.l) a.l[row_base + tid] = s_L[tid];
  }
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.o);
#pragma unroll
  for (int r = 0; r < kMaxRows; ++r) {
    if (r < R) {
      const float L = s_L[r];
      o[(row_base + r) * kD + tid] = __float2bfloat16_rn(L > 0.f ? acc[r] / L : 0.f);
    }
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
  s.exchange = off;  // one-GPU exchange slots of the fused update (zero after workspace init, kept consistent by the kernel)
  off = align_up(off + exchange_bytes(p.B, 1), 256);
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
