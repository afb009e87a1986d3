// Weight-only int8 linear layer for decode batches: y[m, n] = (sum_k x[m, k] W[n, k]) * scale[n]
// with x bf16 [M <= 128, K], W int8 [N, K] (one scale per output channel), y bf16 [M, N]
// (WeightOnlyPerChannelQuantizedLinear.forward, symmetric weights, no activation quantisation:
// jetstream_pt/layers.py:141-166).
//
// A decode step streams every weight byte once, so the kernel is bound by the HBM read of W.  The
// int8 weights go from HBM to shared memory by the copy engine and from there straight into the
// tensor core: the contraction runs as tcgen05 integer MMAs with the weights as the M = 128 operand
// and the activations as the N operand.  The bf16 activations become 8-bit without losing their
// precision by the same two-level split the attention kernel uses for its queries: a row x of the
// batch is s (h + l / 254) with s = amax|x| / 127 and h, l signed bytes (error 2^-16 of the row's
// amax), so the N operand holds 2 M rows (all h rows, then all l rows) and
//   y[m, n] = scale[n] * s_m * (S_h[n, m] + S_l[n, m] / 254)
// with exact int32 sums S_h, S_l in tensor memory.  Nothing is converted in registers.
//
// Launches: (1) split of the activations into levels (one CTA per row of x), (2) the GEMM: one CTA
// per 256 output channels and K split; the CTAs of a tile's K splits form a thread-block cluster.
// 128 threads: thread 0 requests the tiles of a 3-stage ring of 128-byte-swizzled [256 x 128 B] weight
// and [2 M x 128 B] activation tiles, thread 32 issues the MMAs, two per K step of 32 bytes, one for
// each half of the channels, so that an activation tile read from L2 serves 256 channels, and frees
// the stages through tcgen05.commit.  Epilogue: all four warps read the accumulators out of tensor
// memory; the rows of the batch are dealt out to the CTAs of the cluster in groups of eight, every
// CTA stores its partial sums of a group into the shared memory of the group's owner (the ring is
// free by then), and the owner adds the partials in the order of the splits, rounds to bf16,
// multiplies by the channel's scale and rounds again, as the reference's two bf16 operations do.
// No partial result goes through global memory.  Every wait on data is bounded; a CTA that gives up
// raises the status word, still meets its cluster at the two cluster barriers, and returns.
//
// Also here, because they write the same level matrix: RMSNorm and the feed-forward gate (SiLU-mul) as
// kernels that can leave the level split of their result behind, so that the layers after them start
// at their GEMM; and the row-parallel form of the layer over the GPUs of one box, in which the owner
// of a group of rows adds the partial sums of all ranks (fetched over NVLink) before it rounds.
#include <cuda.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <type_traits>
#include <vector>

#include "common.cuh"

namespace jpt {
namespace {

constexpr int kTileN = 256;      // output channels per CTA: two accumulators of 128 TMEM lanes
constexpr int kTileK = 128;      // int8 elements per stage and row: one 128-byte swizzle atom
constexpr int kStages = 3;
constexpr int kMaxM = 128;       // rows of x: the N operand holds 2 * M rows (<= 256)
constexpr int kTmemColsL = 512;  // two accumulators [128 lanes x 2 M columns]
constexpr int kThreadsL = 128;
constexpr int kMaxSplit = 8;     // K splits of a tile = CTAs of a cluster (the portable limit)
constexpr long long kWaitCyclesL = 1000000000ll;

struct __align__(1024) SmemL {
  uint8_t w[kStages][kTileN * kTileK];        // weight tiles, swizzled
  uint8_t x[kStages][2 * kMaxM * kTileK];     // activation level tiles (only 2 M rows are filled)
  uint64_t full[kStages], empty[kStages], done;
  float xs[kMaxM];  // s_m / 254 of the rows of x
  uint32_t tmem_base;
};

struct LinearMaps {
  CUtensorMap w, x;
};

// Row-parallel layer over the GPUs of one box (the input features are sharded: every rank holds x[:, K_r] and
// W[:, K_r], the result is the sum over the ranks).  buffers[r] is rank r's receive buffer (own or an IPC
// mapping): a status word and the launch counter, launch numbers [2 (launch parity)][8 (source rank)][1024 (tile)]
// [8 (K split)] u32, then the rank's OWN fp32 partial sums [2][128][N].  A rank writes its sums into its own buffer,
// tells the others with the launch number (one small peer store per CTA and rank, behind a system-scope fence) and
// reads theirs with 16-byte peer loads, twelve of a thread in flight at a time: loads cross NVLink at about
// twice the rate of narrow peer stores.  world = 1: a layer of one GPU.
struct TpArgs {
  int world, rank;
  // number of this launch (the same on every rank): counted on the device by the level kernel in front of the GEMM,
  // so that a captured graph can be replayed
  unsigned* launch_counter;
  long long wait_cycles;
  char* buffers[8];
  int* status;  // in the rank's own buffer: raised when a wait for a peer ran out
};
constexpr int kTpMaxTiles = 1024;
constexpr size_t kTpFlagOffset = 256;
constexpr size_t kTpFlagBytes = (size_t)2 * 8 * kTpMaxTiles * 8 * sizeof(unsigned);
constexpr size_t kTpDataOffset = kTpFlagOffset + kTpFlagBytes;
__device__ __forceinline__ void st_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// (no memory clobber: the loads of a batch must be free to go out together; the flag's wait, fence and barrier
// stand before them)
__device__ __forceinline__ float4 ld_sys_f32x4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait for the phase with the given parity; false when it gave up.
__device__ __noinline__ bool mbar_wait_l(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 16; ++i) {
      if (mbar_try(bar, parity)) return true;
    }
    if (clock64() - t0 > kWaitCyclesL) return false;
  }
}
__device__ __forceinline__ uint64_t desc_k_major_128b(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);  // start address
  d |= (uint64_t)(1024 >> 4) << 16;       // leading byte offset (one swizzle atom)
  d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                 // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// Thread-block cluster: barrier over all its threads (with release / acquire of shared-memory stores),
// the address of a shared-memory location in the CTA of another rank, a store there.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t remote_smem(uint32_t local_addr, int rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  // (no memory clobber: the cluster barriers order these stores, and the loads around them must stay free to move)
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v));
}

// 32 consecutive accumulator columns of this thread's lane
__device__ __forceinline__ void tmem_ld_32(uint32_t addr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
        "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(addr));
}

// ---------------------------------------------------------------- (1) activation levels
// x [M, K] bf16 -> levels [2 Mp, K] int8 (rows 0 .. M-1: h, rows Mp .. Mp+M-1: l, the others zero)
// and xs[m] = s_m / 254.
__global__ void __launch_bounds__(256) x_levels_kernel(const __nv_bfloat16* x, int8_t* lev, float* xs, int* status, int M,
                                                       int Mp, int K, int clear_status, unsigned* launch_counter) {
  __shared__ float red[33];
  const int m = blockIdx.x, tid = threadIdx.x;  // one CTA per row of the padded batch
  grid_dependency_trigger();
  if (m == 0 && tid == 0 && clear_status) *status = 0;
  if (m == 0 && tid == 0 && launch_counter) *launch_counter += 1u;  // (one thread, launches in stream order)
  uint2* hrow = reinterpret_cast<uint2*>(lev + (int64_t)m * K);
  uint2* lrow = reinterpret_cast<uint2*>(lev + (int64_t)(Mp + m) * K);
  const int nvec = K / 8;  // eight elements per step: 16 bytes in, 8 + 8 bytes out
  if (m >= M) {  // padding rows of the level matrix
    for (int v = tid; v < nvec; v += 256) hrow[v] = lrow[v] = make_uint2(0u, 0u);
    return;
  }
  const uint4* row = reinterpret_cast<const uint4*>(x + (int64_t)m * K);
  constexpr int kHeld = 8;  // steps of a thread kept in registers between the two passes (rows of up to 16384 elements)
  uint4 held[kHeld];
  __nv_bfloat162 mx = __float2bfloat162_rn(0.f);
  auto fold = [&](const uint4& r) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int j = 0; j < 4; ++j) mx = __hmax2(mx, __habs2(h2[j]));
  };
#pragma unroll
  for (int i = 0; i < kHeld; ++i) {
    const int v = tid + 256 * i;
    held[i] = v < nvec ? __ldg(row + v) : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int i = 0; i < kHeld; ++i) fold(held[i]);
  for (int v = tid + 256 * kHeld; v < nvec; v += 256) fold(__ldg(row + v));
  const float amax = block_max(fmaxf(__low2float(mx), __high2float(mx)), red);
  const float inv = amax > 0.f ? 127.f / amax : 0.f;
  auto split_levels = [&](const uint4& r, int v) {
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&r);
    uint32_t hb[2] = {0u, 0u}, lb[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float t = __bfloat162float(e[j]) * inv;
      const float h = rintf(t);
      const float l = rintf((t - h) * 254.f);
      hb[j >> 2] |= ((uint32_t)(int)h & 0xffu) << (8 * (j & 3));
      lb[j >> 2] |= ((uint32_t)(int)l & 0xffu) << (8 * (j & 3));
    }
    hrow[v] = make_uint2(hb[0], hb[1]);
    lrow[v] = make_uint2(lb[0], lb[1]);
  };
#pragma unroll
  for (int i = 0; i < kHeld; ++i) {
    const int v = tid + 256 * i;
    if (v < nvec) split_levels(held[i], v);
  }
  for (int v = tid + 256 * kHeld; v < nvec; v += 256) split_levels(__ldg(row + v), v);
  if (tid == 0) xs[m] = amax * (1.f / 127.f) * (1.f / 254.f);
}

// ---------------------------------------------------------------- producers of the activations that split on the way
// Eight bf16 values of a row -> their two level bytes each, stored at step v of the row's h and l rows.
__device__ __forceinline__ void split_levels8(const __nv_bfloat16 (&e)[8], float inv, uint2* hrow, uint2* lrow, int v) {
  uint32_t hb[2] = {0u, 0u}, lb[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float t = __bfloat162float(e[j]) * inv;
    const float h = rintf(t);
    const float l = rintf((t - h) * 254.f);
    hb[j >> 2] |= ((uint32_t)(int)h & 0xffu) << (8 * (j & 3));
    lb[j >> 2] |= ((uint32_t)(int)l & 0xffu) << (8 * (j & 3));
  }
  hrow[v] = make_uint2(hb[0], hb[1]);
  lrow[v] = make_uint2(lb[0], lb[1]);
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int sh = 16; sh > 0; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float x = lane < (int)((blockDim.x + 31) >> 5) ? red[lane] : 0.f;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) x += __shfl_xor_sync(0xffffffffu, x, sh);
    if (lane == 0) red[32] = x;
  }
  __syncthreads();
  return red[32];
}

constexpr int kRowThreads = 1024;  // threads of a CTA of the element-wise producers
// The CTAs of a cluster (gridDim.x of them, rank blockIdx.x) share a row: a value of every CTA combined in the
// order of the ranks.  Every CTA stores its value into slot `rank` of every CTA's `slots`; one cluster barrier later
// all slots are there.  (`slots` must not be reused for another reduction: a fast CTA could overwrite a slot
// that a slow one has not read yet.)
template <typename Op>
__device__ __forceinline__ float cluster_combine(float v, float* slots, Op op) {
  const int csize = (int)gridDim.x, rank = (int)blockIdx.x;
  if (csize == 1) return v;
  if ((int)threadIdx.x < csize) st_cluster_f32(remote_smem(smem_addr(&slots[rank]), (int)threadIdx.x), v);
  cluster_sync();
  float r = slots[0];
  for (int c = 1; c < csize; ++c) r = op(r, slots[c]);
  return r;
}

// A row of results, eight at a time from `compute(step, out)`: written to `dst`, and with `levels` split into the
// row's level bytes once the row's amax is known.  The first steps of a thread stay in registers between the two
// passes (1024 threads x 4 steps x 8: rows of up to 32768 elements); longer rows compute their tail twice.
template <typename Compute>
__device__ __forceinline__ void write_row_and_levels(Compute& compute, uint4* dst, int v_lo, int nvec, bool levels, uint2* hrow,
                                                     uint2* lrow, float* xs, int m, float* red, float* slots) {
  constexpr int kHeldOut = 4;
  const int tid = threadIdx.x + v_lo;  // (this CTA's steps are v_lo .. nvec - 1)
  uint4 held[kHeldOut];
  float amax = 0.f;
  auto fold = [&](const __nv_bfloat16 (&o)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(__bfloat162float(o[j])));
  };
#pragma unroll
  for (int i = 0; i < kHeldOut; ++i) {
    const int v = tid + kRowThreads * i;
    if (v < nvec) {
      __nv_bfloat16 o[8];
      compute(v, o);
      fold(o);
      held[i] = *reinterpret_cast<const uint4*>(o);
      dst[v] = held[i];
    }
  }
  for (int v = tid + kRowThreads * kHeldOut; v < nvec; v += kRowThreads) {
    __nv_bfloat16 o[8];
    compute(v, o);
    fold(o);
    dst[v] = *reinterpret_cast<const uint4*>(o);
  }
  if (!levels) return;
  amax = cluster_combine(block_max(amax, red), slots, [](float p, float q) { return fmaxf(p, q); });
  const float inv = amax > 0.f ? 127.f / amax : 0.f;
#pragma unroll
  for (int i = 0; i < kHeldOut; ++i) {
    const int v = tid + kRowThreads * i;
    if (v < nvec) split_levels8(*reinterpret_cast<const __nv_bfloat16(*)[8]>(&held[i]), inv, hrow, lrow, v);
  }
  for (int v = tid + kRowThreads * kHeldOut; v < nvec; v += kRowThreads) {
    __nv_bfloat16 o[8];
    compute(v, o);
    split_levels8(o, inv, hrow, lrow, v);
  }
  if (threadIdx.x == 0 && blockIdx.x == 0) xs[m] = amax * (1.f / 127.f) * (1.f / 254.f);
}

// RMSNorm (jetstream_pt/layers.py:337-350 with a bf16 weight): n = bf16(x * rsqrt(mean(x^2) + eps)) in fp32,
// y = bf16(n * weight).  With `lev` the row's levels are written too (the rows M .. Mp-1 of the level matrix as zeros),
// so that the linear layers that read y start at their GEMM.  One CTA per row.
__global__ void __launch_bounds__(kRowThreads) rmsnorm_levels_kernel(const __nv_bfloat16* x, const __nv_bfloat16* weight, float eps,
                                                             __nv_bfloat16* y, int8_t* lev, float* xs, int* status, int M, int Mp,
                                                             int K) {
  __shared__ float red[33], slots_ss[8], slots_amax[8];
  // row m = blockIdx.y; the CTAs of the row's cluster (blockIdx.x) take equal parts of its steps of eight elements
  const int m = blockIdx.y, tid = threadIdx.x, per = K / 8 / (int)gridDim.x;
  const int v_lo = (int)blockIdx.x * per, nvec = v_lo + per;
  grid_dependency_wait();
  grid_dependency_trigger();
  if (m == 0 && blockIdx.x == 0 && tid == 0 && status) *status = 0;
  uint2* hrow = lev ? reinterpret_cast<uint2*>(lev + (int64_t)m * K) : nullptr;
  uint2* lrow = lev ? reinterpret_cast<uint2*>(lev + (int64_t)(Mp + m) * K) : nullptr;
  if (m >= M) {  // (a padding row: the whole cluster is here, nobody waits for it)
    for (int v = v_lo + tid; v < nvec; v += kRowThreads) hrow[v] = lrow[v] = make_uint2(0u, 0u);
    return;
  }
  const uint4* row = reinterpret_cast<const uint4*>(x + (int64_t)m * K);
  const uint4* wrow = reinterpret_cast<const uint4*>(weight);
  float ss = 0.f;
  for (int v = v_lo + tid; v < nvec; v += kRowThreads) {
    const uint4 r = __ldg(row + v);
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&r);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = __bfloat162float(e[j]);
      ss = fmaf(f, f, ss);
    }
  }
  ss = cluster_combine(block_sum(ss, red), slots_ss, [](float p, float q) { return p + q; });
  const float rs = 1.f / sqrtf(ss / (float)K + eps);
  auto normed = [&](int v, __nv_bfloat16 (&o)[8]) {
    const uint4 r = __ldg(row + v), wv = __ldg(wrow + v);
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&r);
    const __nv_bfloat16* we = reinterpret_cast<const __nv_bfloat16*>(&wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float n = __bfloat162float(__float2bfloat16_rn(__bfloat162float(e[j]) * rs));
      o[j] = __float2bfloat16_rn(n * __bfloat162float(we[j]));
    }
  };
  write_row_and_levels(normed, reinterpret_cast<uint4*>(y + (int64_t)m * K), v_lo, nvec, lev != nullptr, hrow, lrow, xs, m, red,
                       slots_amax);
  if (gridDim.x > 1) cluster_sync();  // (no CTA leaves while a peer may still store into its slots)
}

// The feed-forward block's gate (third_party/llama/model_exportable.py:84-86): h = bf16(bf16(silu(a)) * b), and with
// `lev` the levels of h for the down projection.
__global__ void __launch_bounds__(kRowThreads) silu_mul_levels_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* h,
                                                              int8_t* lev, float* xs, int* status, int M, int Mp, int K) {
  __shared__ float red[33], slots_amax[8];
  const int m = blockIdx.y, tid = threadIdx.x, per = K / 8 / (int)gridDim.x;
  const int v_lo = (int)blockIdx.x * per, nvec = v_lo + per;
  grid_dependency_wait();
  grid_dependency_trigger();
  if (m == 0 && blockIdx.x == 0 && tid == 0 && status) *status = 0;
  uint2* hrow = lev ? reinterpret_cast<uint2*>(lev + (int64_t)m * K) : nullptr;
  uint2* lrow = lev ? reinterpret_cast<uint2*>(lev + (int64_t)(Mp + m) * K) : nullptr;
  if (m >= M) {
    for (int v = v_lo + tid; v < nvec; v += kRowThreads) hrow[v] = lrow[v] = make_uint2(0u, 0u);
    return;
  }
  const uint4* arow = reinterpret_cast<const uint4*>(a + (int64_t)m * K);
  const uint4* brow = reinterpret_cast<const uint4*>(b + (int64_t)m * K);
  auto gated = [&](int v, __nv_bfloat16 (&o)[8]) {
    const uint4 ra = __ldg(arow + v), rb = __ldg(brow + v);
    const __nv_bfloat16* ea = reinterpret_cast<const __nv_bfloat16*>(&ra);
    const __nv_bfloat16* eb = reinterpret_cast<const __nv_bfloat16*>(&rb);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = __bfloat162float(ea[j]);
      // (fast exponential and division: the quotient is rounded to bf16, and the exact forms are subroutines)
      const float s = __bfloat162float(__float2bfloat16_rn(__fdividef(f, 1.f + __expf(-f))));
      o[j] = __float2bfloat16_rn(s * __bfloat162float(eb[j]));
    }
  };
  write_row_and_levels(gated, reinterpret_cast<uint4*>(h + (int64_t)m * K), v_lo, nvec, lev != nullptr, hrow, lrow, xs, m, red,
                       slots_amax);
  if (gridDim.x > 1) cluster_sync();  // (no CTA leaves while a peer may still store into its slots)
}

// ---------------------------------------------------------------- (2) the GEMM
// grid (ceil(N / 256), ksplit), clusters of (1, ksplit): the rank of a CTA in its cluster is its K split.
__global__ void __launch_bounds__(kThreadsL, 1)
    w8a16_gemm_kernel(const __grid_constant__ LinearMaps maps, const float* xs, const __nv_bfloat16* scale, __nv_bfloat16* y,
                      int M, int Mp, int N, int K, int k_tiles, int* status, const __grid_constant__ TpArgs tp) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  SmemL& sm = *reinterpret_cast<SmemL*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5;
  if ((smem_addr(smem_raw) & 1023u) != 0u) {
    grid_dependency_wait();  // (the launch before this one clears the status word)
    if (tid == 0) atomicExch(status, 2);
    return;
  }
  const int n0 = blockIdx.x * kTileN, split = blockIdx.y;
  // K steps of this split: the k_tiles steps dealt out as evenly as whole steps allow (the first splits one more)
  const int nsplit = (int)gridDim.y, k_lo = split * (k_tiles / nsplit) + min(split, k_tiles % nsplit);
  const int iters = k_tiles / nsplit + (split < k_tiles % nsplit ? 1 : 0), k_begin = k_lo * kTileK;
  const int n_mma = 2 * Mp;  // columns of the accumulator (a multiple of 16)

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&sm.full[s])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&sm.empty[s])));
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&sm.done)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.x)) : "memory");
    // The weights do not depend on the launch before this one (only the activation levels do): the weight
    // tiles of the first stages are requested before the wait on that launch.  Their bytes are announced to
    // the stage's barrier without an arrival; the arrival comes with the activation tile's request.
    const int rot0 = (int)(blockIdx.x % (unsigned)iters);
    for (int it = 0; it < kStages && it < iters; ++it) {
      const int kt = it + rot0 < iters ? it + rot0 : it + rot0 - iters;
      const uint32_t bar = smem_addr(&sm.full[it]);
      asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"((uint32_t)(kTileN * kTileK)) : "memory");
      tma_load_2d(smem_addr(&sm.w[it][0]), &maps.w, k_begin + kt * kTileK, n0, bar);
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&sm.tmem_base)),
                 "r"((uint32_t)kTmemColsL)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  grid_dependency_wait();
  grid_dependency_trigger();
  const unsigned tp_epoch = tp.world > 1 ? *reinterpret_cast<volatile unsigned*>(tp.launch_counter) : 0u;
  sm.xs[tid] = tid < M ? xs[tid] : 0.f;
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sm.tmem_base;
  bool dead = false;

  if (tid == 0) {
    // ---- producer: tiles of stage s are requested when the MMAs that read its previous contents are done
    // Every CTA of a K split reads the same activation tiles: each starts at another K step (the sums are
    // exact integers, their order is free), so that the CTAs do not ask the same L2 lines at the same time.
    const int rot = (int)(blockIdx.x % (unsigned)iters);
    const uint32_t w_bytes = (uint32_t)(kTileN * kTileK), x_bytes = (uint32_t)(n_mma * kTileK);
    for (int it = 0; it < iters && !dead; ++it) {
      const int s = it % kStages;
      if (it >= kStages && !mbar_wait_l(smem_addr(&sm.empty[s]), (uint32_t)((it / kStages) - 1) & 1u)) dead = true;
      if (dead) break;
      const uint32_t bar = smem_addr(&sm.full[s]);
      const int kt = it + rot < iters ? it + rot : it + rot - iters;
      if (it >= kStages) {  // (the weight tiles of the first stages are on their way already)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(w_bytes + x_bytes) : "memory");
        tma_load_2d(smem_addr(&sm.w[s][0]), &maps.w, k_begin + kt * kTileK, n0, bar);
      } else {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(x_bytes) : "memory");
      }
      tma_load_2d(smem_addr(&sm.x[s][0]), &maps.x, k_begin + kt * kTileK, 0, bar);
    }
  } else if (tid == 32) {
    // ---- MMA issue: D_half[128 n x 2 Mp] += W_tile[half][128 x 128 B] . Xl_tile^T, four K steps of 32 bytes per stage
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (((uint32_t)n_mma >> 3) << 17) | ((128u >> 4) << 24);
    for (int it = 0; it < iters && !dead; ++it) {
      const int s = it % kStages;
      if (!mbar_wait_l(smem_addr(&sm.full[s]), (uint32_t)(it / kStages) & 1u)) {
        dead = true;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t wa = smem_addr(&sm.w[s][0]), xa = smem_addr(&sm.x[s][0]);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t bd = desc_k_major_128b(xa + 32 * ks);
        const uint32_t acc = (it > 0 || ks > 0) ? 1u : 0u;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint64_t ad = desc_k_major_128b(wa + half * (128 * kTileK) + 32 * ks);
          asm volatile(
              "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem + (uint32_t)(half * n_mma)),
              "l"(ad), "l"(bd), "r"(idesc), "r"(acc)
              : "memory");
        }
      }
      // the stage is free again when these MMAs have read it
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&sm.empty[s]))
                   : "memory");
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&sm.done))
                 : "memory");
  }
  __syncwarp();
  // ---- epilogue: lane n of accumulator `half` belongs to thread n (output channel n0 + 128 half + n)
  const int csize = (int)gridDim.y;  // CTAs in the cluster = K splits
  const int groups = Mp / 8;         // groups of eight rows of the batch; group j belongs to rank j % csize
  const int owned = (groups + csize - 1) / csize;
  // landing area in the ring: [source rank][owned group][half][row of the group][thread] fp32
  float* land = reinterpret_cast<float*>(smem_raw);
  const bool ok = mbar_wait_l(smem_addr(&sm.done), 0u);
  const bool bad = __syncthreads_or(dead || !ok) != 0;
  if (bad && tid == 0) atomicExch(status, 1);  // (only if the copy engine or the tensor core stopped answering)
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  cluster_sync();  // every ring of the cluster has been read to the end: the landing areas are free
  if (!bad) {
    for (int m0 = 0; m0 < Mp; m0 += 32) {
      uint32_t h[2][32], l[2][32];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(half * n_mma);
        tmem_ld_32(lane_addr + (uint32_t)m0, h[half]);
        tmem_ld_32(lane_addr + (uint32_t)(Mp + m0), l[half]);
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      float xr[32];  // (all loads before the stores: the compiler cannot move them across)
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) xr[jj] = sm.xs[(m0 + jj) & (kMaxM - 1)];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = m0 / 8 + c;
        if (j < groups) {
          const int owner = j % csize, q = j / csize;
          const uint32_t base = remote_smem(smem_addr(land + ((((int64_t)split * owned + q) * 2) * 8) * kThreadsL + tid), owner);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              const int jj = 8 * c + r;
              const float v = fmaf((float)(int)h[half][jj], 254.f, (float)(int)l[half][jj]) * xr[jj];
              st_cluster_f32(base + (uint32_t)((half * 8 + r) * kThreadsL * 4), v);
            }
          }
        }
      }
    }
  }
  float sc[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int n = n0 + half * 128 + tid;
    sc[half] = n < N ? __bfloat162float(scale[n]) : 0.f;
  }
  cluster_sync();  // all partial sums have landed
  if (!bad) {
    auto reduce = [&](auto cs_tag) {
      constexpr int kCs = decltype(cs_tag)::value;
      for (int q = 0; q < owned; ++q) {
        const int j = q * kCs + split;
        if (j >= groups) break;
        float acc[2][8];  // (sixteen independent chains; all loads before the stores)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int r = 0; r < 8; ++r) acc[half][r] = land[(((0 * owned + q) * 2 + half) * 8 + r) * kThreadsL + tid];
        }
#pragma unroll
        for (int src = 1; src < kCs; ++src) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int r = 0; r < 8; ++r) acc[half][r] += land[(((src * owned + q) * 2 + half) * 8 + r) * kThreadsL + tid];
          }
        }
        if (tp.world > 1) {
          // this rank's sums of the group go into its own buffer, where the other ranks read them; the roundings
          // follow below, on the sum over the ranks
          float* dst = reinterpret_cast<float*>(tp.buffers[tp.rank] + kTpDataOffset) + (int64_t)(tp_epoch & 1u) * kMaxM * N;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int n = n0 + half * 128 + tid;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              const int m = 8 * j + r;
              if (m < M && n < N) __stcg(&dst[(int64_t)m * N + n], acc[half][r]);
            }
          }
          continue;
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int n = n0 + half * 128 + tid;
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const int m = 8 * j + r;
            const float dot = __bfloat162float(__float2bfloat16_rn(acc[half][r]));            // F.linear's bf16 result
            if (m < M && n < N) y[(int64_t)m * N + n] = __float2bfloat16_rn(dot * sc[half]);  // * weight_scaler
          }
        }
      }
    };
    switch (csize) {
      case 1: reduce(std::integral_constant<int, 1>{}); break;
      case 2: reduce(std::integral_constant<int, 2>{}); break;
      case 3: reduce(std::integral_constant<int, 3>{}); break;
      case 4: reduce(std::integral_constant<int, 4>{}); break;
      case 5: reduce(std::integral_constant<int, 5>{}); break;
      case 6: reduce(std::integral_constant<int, 6>{}); break;
      case 7: reduce(std::integral_constant<int, 7>{}); break;
      default: reduce(std::integral_constant<int, 8>{}); break;
    }
    if (tp.world > 1 && split < groups) {  // (a CTA without a group of rows has nothing to send or to wait for)
      // ---- sum over the ranks: tell every rank that this CTA's groups are in this rank's buffer, wait (bounded) for
      // the same CTA of every rank, read their sums and add them in the order of the ranks
      const int par = (int)(tp_epoch & 1u);
      auto flag_of = [&](int buffer_of, int src) {  // the sums of rank `src` are ready, as told to rank `buffer_of`
        return reinterpret_cast<unsigned*>(tp.buffers[buffer_of] + kTpFlagOffset) +
               (((size_t)par * 8 + src) * kTpMaxTiles + blockIdx.x) * 8 + split;
      };
      __syncthreads();  // every thread's stores are issued ...
      if (tid < tp.world && tid != tp.rank) {
        __threadfence_system();  // ... and ordered before the launch number that announces them
        st_sys_u32(flag_of(tid, tp.rank), tp_epoch);
        const long long t0c = clock64();
        while (ld_sys_u32(flag_of(tp.rank, tid)) != tp_epoch) {
          if (clock64() - t0c > tp.wait_cycles) {  // a rank never came: report, go on with what is there
            atomicExch(tp.status, 1);
            break;
          }
        }
        __threadfence_system();
      }
      __syncthreads();
      asm volatile("" ::: "memory");  // (the peer loads below carry no memory clobber of their own)
      const size_t part_off = kTpDataOffset + (size_t)par * kMaxM * N * sizeof(float);
      // A group is eight rows x 256 channels: 512 pieces of four channels (16 bytes), four per thread.  A thread
      // has the pieces of up to three groups (twelve loads per rank) in flight at a time.
      constexpr int kBatch = 12;
      const int my_groups = (groups - split + csize - 1) / csize;
      for (int base = 0; base < 4 * my_groups; base += kBatch) {
        float4 sum[kBatch];
        int64_t at[kBatch];  // element offset of the piece, -1: none
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          const int idx = base + b, item = (idx & 3) * kThreadsL + tid;
          const int m = 8 * ((idx >> 2) * csize + split) + (item >> 6), n = n0 + 4 * (item & 63);
          at[b] = (idx < 4 * my_groups && m < M && n < N) ? (int64_t)m * N + n : -1;
          sum[b] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int src = 0; src < tp.world; ++src) {
          const float* part = reinterpret_cast<const float*>(tp.buffers[src] + part_off);
          float4 v[kBatch];
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            v[b] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (at[b] >= 0) v[b] = src == tp.rank ? __ldcg(reinterpret_cast<const float4*>(part + at[b])) : ld_sys_f32x4(part + at[b]);
          }
#pragma unroll
          for (int b = 0; b < kBatch; ++b) sum[b].x += v[b].x, sum[b].y += v[b].y, sum[b].z += v[b].z, sum[b].w += v[b].w;
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          if (at[b] < 0) continue;
          const int n = (int)(at[b] % N);
          const uint2 sraw = __ldg(reinterpret_cast<const uint2*>(scale + n));
          const __nv_bfloat16* sb = reinterpret_cast<const __nv_bfloat16*>(&sraw);
          const float a4[4] = {sum[b].x, sum[b].y, sum[b].z, sum[b].w};
          uint2 o;
          __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            ob[e] = __float2bfloat16_rn(__bfloat162float(__float2bfloat16_rn(a4[e])) * __bfloat162float(sb[e]));
          *reinterpret_cast<uint2*>(y + at[b]) = o;
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kTmemColsL) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
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
// rows x K bytes, row-major; boxes of box_rows x 128 bytes with the 128-byte swizzle
bool encode_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t str[1] = {(cuuint64_t)K};
  const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, str, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int split_for(int N, int K) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  const int tiles = (N + kTileN - 1) / kTileN, k_tiles = K / kTileK;
  // The K splits of a tile are the CTAs of one cluster (1 .. 8; the K steps are dealt out evenly).  The split with
  // the shortest estimated run is taken: CTAs run in waves of one per SM; a CTA costs about 8 us of set-up, first
  // fetch and epilogue plus 0.6 us per K step (measured on B200 for 96 rows).
  int split = 1;
  float best = 0.f;
  for (int c = 1; c <= kMaxSplit && c <= k_tiles; ++c) {
    const int waves = (tiles * c + sms - 1) / sms;
    const float cost = (float)waves * (8.f + 0.6f * (float)((k_tiles + c - 1) / c));
    if (c == 1 || cost < best) best = cost, split = c;
  }
  return split;
}

}  // namespace
}  // namespace jpt

using namespace jpt;

extern "C" size_t jpt_w8a16_linear_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int Mp = (std::min(M, kMaxM) + 7) / 8 * 8;  // (more rows are taken in blocks of 128, one after the other)
  const size_t levels = ((size_t)2 * Mp * K + 255) / 256 * 256;
  const size_t xs = 1024;
  (void)N;
  return 256 + levels + xs;
}

namespace jpt {
namespace {
// The workspace of up to 128 rows: status word, level matrix [2 Mp, K], row scales.
struct LevelsView {
  int* status;  // 0, or the code of a CTA that gave up
  int8_t* lev;
  float* xs;
  int Mp;
};
LevelsView levels_view(void* workspace, int M, int K) {
  LevelsView v;
  v.Mp = (M + 7) / 8 * 8;
  char* ws = static_cast<char*>(workspace);
  v.status = reinterpret_cast<int*>(ws);
  v.lev = reinterpret_cast<int8_t*>(ws + 256);
  const size_t levels = ((size_t)2 * v.Mp * K + 255) / 256 * 256;
  v.xs = reinterpret_cast<float*>(ws + 256 + levels);
  return v;
}

// The GEMM on levels that a launch before this one in the stream wrote.  The launch may start while that one
// drains (it requests its first weight tiles at once) and waits for its results on the device.
int launch_gemm(const LevelsView& lv, const void* w, const void* w_scale, void* y, int M, int N, int K, cudaStream_t st,
                const TpArgs* tp_in = nullptr) {
  const int ksplit = split_for(N, K);
  TpArgs tp;
  memset(&tp, 0, sizeof(tp));
  tp.world = 1;
  if (tp_in) tp = *tp_in;
  static std::mutex mu;
  LinearMaps maps;
  memset(&maps, 0, sizeof(maps));
  {
    std::lock_guard<std::mutex> lock(mu);
    JPT_REQUIRE(encode_2d(&maps.w, w, N, K, kTileN) && encode_2d(&maps.x, lv.lev, 2 * lv.Mp, K, 2 * lv.Mp), JPT_EINVAL,
                "w8a16_linear: the tensors cannot be described by a tensor map");
  }
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(w8a16_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmemL));
    if (e != cudaSuccess) return fail((int)e, "w8a16_linear: configuring the kernel: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((N + kTileN - 1) / kTileN, ksplit);
  cfg.blockDim = dim3(kThreadsL);
  cfg.dynamicSmemBytes = sizeof(SmemL);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = ksplit;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;  // (also inside a graph capture: the weight tiles stream in under the level kernel)
  const cudaError_t e = cudaLaunchKernelEx(&cfg, w8a16_gemm_kernel, maps, static_cast<const float*>(lv.xs),
                                           static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(y), M, lv.Mp, N, K,
                                           K / kTileK, lv.status, tp);
  if (e != cudaSuccess) return fail((int)e, "w8a16_gemm_kernel: %s", cudaGetErrorString(e));
  return 0;
}

// (the level kernel also clears the status word and the padding rows of the level matrix)
int launch_levels(const void* x, const LevelsView& lv, int M, int K, cudaStream_t st, bool clear_status,
                  unsigned* launch_counter = nullptr) {
  x_levels_kernel<<<lv.Mp, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), lv.lev, lv.xs, lv.status, M, lv.Mp, K,
                                         clear_status ? 1 : 0, launch_counter);
  return check_launch("x_levels_kernel");
}

// CTAs per row of the element-wise producers (a cluster along x): enough of them to fill the GPU
int row_parts(int rows, int K) {
  const int steps = K / 8;
  int c = 1;
  // (one CTA of 1024 threads per row measured faster than a row split over a cluster: 3.7 against 9.8 us for
  // RMSNorm of [96, 8192]; the split stays available for single rows of long vectors)
  while (c < 8 && rows * c < 8 && steps % (c * 2) == 0 && steps / (c * 2) >= kRowThreads) c *= 2;
  return c;
}
template <typename... KArgs, typename... Args>
int launch_rows(const char* name, void (*kernel)(KArgs...), int rows, int parts, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(parts, rows);
  cfg.blockDim = dim3(kRowThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = parts;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  if (e != cudaSuccess) return fail((int)e, "%s: %s", name, cudaGetErrorString(e));
  return 0;
}

int check_levels_args(const char* who, int M, int K, const void* workspace, size_t workspace_bytes) {
  JPT_REQUIRE(M >= 1 && M <= kMaxM, JPT_EINVAL, "%s: M = %d rows, activation levels are kept for 1 .. %d rows", who, M, kMaxM);
  JPT_REQUIRE(K >= kTileK && K % kTileK == 0, JPT_EINVAL, "%s: K = %d must be a multiple of %d", who, K, kTileK);
  const size_t need = jpt_w8a16_linear_workspace_bytes(M, 1, K);
  JPT_REQUIRE(workspace && workspace_bytes >= need, JPT_EWORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who, need,
              workspace_bytes);
  JPT_REQUIRE(aligned(workspace, 256), JPT_EALIGN, "%s: workspace must be 256-byte aligned", who);
  return 0;
}
}  // namespace
}  // namespace jpt

extern "C" int jpt_w8a16_linear(const void* x, const void* w, const void* w_scale, void* y, int M, int N, int K,
                                void* workspace, size_t workspace_bytes, void* stream) {
  JPT_REQUIRE(x && w && w_scale && y, JPT_EINVAL, "w8a16_linear: null tensor");
  JPT_REQUIRE(M >= 1, JPT_EINVAL, "w8a16_linear: M = %d rows", M);
  JPT_REQUIRE(N >= 1 && K >= kTileK && K % kTileK == 0, JPT_EINVAL, "w8a16_linear: K = %d must be a multiple of %d", K, kTileK);
  JPT_REQUIRE(aligned(x, 16) && aligned(w, 16) && aligned(y, 2), JPT_EALIGN, "w8a16_linear: x and w must be 16-byte aligned");
  const size_t need = jpt_w8a16_linear_workspace_bytes(M, N, K);
  JPT_REQUIRE(workspace && workspace_bytes >= need, JPT_EWORKSPACE, "w8a16_linear: workspace of %zu bytes needed, %zu given", need,
              workspace_bytes);
  JPT_REQUIRE(aligned(workspace, 256), JPT_EALIGN, "w8a16_linear: workspace must be 256-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // More than 128 rows (prefill shapes) go through in blocks of 128 that reuse the workspace in stream order;
  // every block streams the weights again, which is the wrong trade for a compute-bound shape but a correct one.
  for (int m0 = 0; m0 < M; m0 += kMaxM) {
    const int rows = std::min(kMaxM, M - m0);
    const LevelsView lv = levels_view(workspace, rows, K);
    if (int rc = launch_levels(static_cast<const char*>(x) + (size_t)m0 * K * 2, lv, rows, K, st, m0 == 0)) return rc;
    if (int rc = launch_gemm(lv, w, w_scale, static_cast<char*>(y) + (size_t)m0 * N * 2, rows, N, K, st)) return rc;
  }
  return 0;
}

extern "C" int jpt_w8a16_split_levels(const void* x, int M, int K, void* workspace, size_t workspace_bytes, void* stream) {
  JPT_REQUIRE(x && aligned(x, 16), JPT_EALIGN, "w8a16_split_levels: x must be 16-byte aligned");
  if (int rc = check_levels_args("w8a16_split_levels", M, K, workspace, workspace_bytes)) return rc;
  return launch_levels(x, levels_view(workspace, M, K), M, K, static_cast<cudaStream_t>(stream), true);
}

extern "C" int jpt_w8a16_linear_from_levels(void* workspace, size_t workspace_bytes, const void* w, const void* w_scale, void* y,
                                            int M, int N, int K, void* stream) {
  JPT_REQUIRE(w && w_scale && y && N >= 1, JPT_EINVAL, "w8a16_linear_from_levels: null tensor");
  JPT_REQUIRE(aligned(w, 16), JPT_EALIGN, "w8a16_linear_from_levels: w must be 16-byte aligned");
  if (int rc = check_levels_args("w8a16_linear_from_levels", M, K, workspace, workspace_bytes)) return rc;
  return launch_gemm(levels_view(workspace, M, K), w, w_scale, y, M, N, K, static_cast<cudaStream_t>(stream));
}

extern "C" int jpt_rmsnorm(const void* x, const void* weight, float eps, void* y, int M, int K, void* levels_workspace,
                           size_t workspace_bytes, void* stream) {
  JPT_REQUIRE(x && weight && y && M >= 1 && K >= 8 && K % 8 == 0, JPT_EINVAL, "rmsnorm: M = %d, K = %d (K must be a multiple of 8)", M, K);
  JPT_REQUIRE(aligned(x, 16) && aligned(weight, 16) && aligned(y, 16), JPT_EALIGN, "rmsnorm: tensors must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(weight);
  if (!levels_workspace) {
    return launch_rows("rmsnorm_levels_kernel", rmsnorm_levels_kernel, M, row_parts(M, K), st, xp, wp, eps, static_cast<__nv_bfloat16*>(y),
                       nullptr, nullptr, nullptr, M, M, K);
  }
  if (int rc = check_levels_args("rmsnorm", M, K, levels_workspace, workspace_bytes)) return rc;
  const LevelsView lv = levels_view(levels_workspace, M, K);
  return launch_rows("rmsnorm_levels_kernel", rmsnorm_levels_kernel, lv.Mp, row_parts(lv.Mp, K), st, xp, wp, eps,
                     static_cast<__nv_bfloat16*>(y), lv.lev, lv.xs, lv.status, M, lv.Mp, K);
}

extern "C" int jpt_silu_mul(const void* a, const void* b, void* h, int M, int K, void* levels_workspace, size_t workspace_bytes,
                            void* stream) {
  JPT_REQUIRE(a && b && h && M >= 1 && K >= 8 && K % 8 == 0, JPT_EINVAL, "silu_mul: M = %d, K = %d (K must be a multiple of 8)", M, K);
  JPT_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(h, 16), JPT_EALIGN, "silu_mul: tensors must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* ap = static_cast<const __nv_bfloat16*>(a);
  const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(b);
  if (!levels_workspace) {
    return launch_rows("silu_mul_levels_kernel", silu_mul_levels_kernel, M, row_parts(M, K), st, ap, bp, static_cast<__nv_bfloat16*>(h),
                       nullptr, nullptr, nullptr, M, M, K);
  }
  if (int rc = check_levels_args("silu_mul", M, K, levels_workspace, workspace_bytes)) return rc;
  const LevelsView lv = levels_view(levels_workspace, M, K);
  return launch_rows("silu_mul_levels_kernel", silu_mul_levels_kernel, lv.Mp, row_parts(lv.Mp, K), st, ap, bp,
                     static_cast<__nv_bfloat16*>(h), lv.lev, lv.xs, lv.status, M, lv.Mp, K);
}

extern "C" size_t jpt_w8a16_tp_buffer_bytes(int N, int world) {
  if (N < 4 || N % 4 || world < 1 || world > 8 || (N + kTileN - 1) / kTileN > kTpMaxTiles) return 0;
  return kTpDataOffset + (size_t)2 * kMaxM * N * sizeof(float);
}

extern "C" int jpt_w8a16_linear_tp(const void* x, const void* w, const void* w_scale, void* y, int M, int N, int K, void* workspace,
                                   size_t workspace_bytes, const jpt_tp_sum* tp, void* stream) {
  JPT_REQUIRE(x && w && w_scale && y && tp, JPT_EINVAL, "w8a16_linear_tp: null argument");
  JPT_REQUIRE(N >= 4 && N % 4 == 0, JPT_EINVAL, "w8a16_linear_tp: N = %d must be a multiple of 4", N);
  JPT_REQUIRE(aligned(x, 16) && aligned(w, 16) && aligned(y, 8) && aligned(w_scale, 8), JPT_EALIGN,
              "w8a16_linear_tp: x and w must be 16-byte aligned, y and the scales 8-byte aligned");
  JPT_REQUIRE(tp->world >= 1 && tp->world <= 8 && tp->rank >= 0 && tp->rank < tp->world, JPT_EINVAL,
              "w8a16_linear_tp: rank %d of %d", tp->rank, tp->world);
  JPT_REQUIRE(tp->buffer_bytes >= jpt_w8a16_tp_buffer_bytes(N, tp->world) && jpt_w8a16_tp_buffer_bytes(N, tp->world) > 0, JPT_EWORKSPACE,
              "w8a16_linear_tp: receive buffers of %zu bytes are too small for N = %d on %d ranks", tp->buffer_bytes, N, tp->world);
  if (int rc = check_levels_args("w8a16_linear_tp", M, K, workspace, workspace_bytes)) return rc;
  TpArgs t;
  memset(&t, 0, sizeof(t));
  t.world = tp->world;
  t.rank = tp->rank;
  t.wait_cycles = tp->wait_cycles > 0 ? tp->wait_cycles : kWaitCyclesL;
  for (int r = 0; r < tp->world; ++r) {
    JPT_REQUIRE(tp->buffers[r], JPT_EINVAL, "w8a16_linear_tp: no buffer for rank %d", r);
    t.buffers[r] = static_cast<char*>(tp->buffers[r]);
  }
  t.status = reinterpret_cast<int*>(t.buffers[t.rank]);
  t.launch_counter = reinterpret_cast<unsigned*>(t.buffers[t.rank] + 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const LevelsView lv = levels_view(workspace, M, K);
  if (int rc = launch_levels(x, lv, M, K, st, true, t.launch_counter)) return rc;
  return launch_gemm(lv, w, w_scale, y, M, N, K, st, &t);
}

extern "C" int jpt_w8a16_tp_status(const jpt_tp_sum* tp, void* stream) {
  JPT_REQUIRE(tp && tp->buffers[tp->rank], JPT_EINVAL, "w8a16_tp_status: null buffer");
  int v = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(&v, static_cast<const char*>(tp->buffers[tp->rank]), sizeof(v), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail((int)e, "w8a16_tp_status: %s", cudaGetErrorString(e));
  return v;
}
