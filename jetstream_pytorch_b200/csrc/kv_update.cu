// Decode-time KV cache update kernels: fused int8 quantise + append (dense and
// paged), plain row scatter (bf16 / fp32 append and lazy finalize), and the
// device-side page/token index walk.
#include <stdarg.h>
#include <stdlib.h>

#include <atomic>

#include "common.cuh"

namespace jpt {

char* last_error_buffer() {
  static thread_local char buf[512] = "";
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

static std::atomic<long long> g_launches{0};
long long launch_count() { return g_launches.load(); }

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("JPT_NO_PDL");
    return !(e && e[0] == '1');
  }();
  return on;
}

int check_launch(const char* what) {
  g_launches.fetch_add(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(last_error_buffer(), 512, "%s: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

namespace {

// ---------------------------------------------------------------------------
// Fused quantise + append.  One block per (item, K|V).  An item is a batch slot
// (dense) or an active entry of page_token_indices (paged).  The token's H*D
// values are held in registers between the amax pass and the quantise pass
// (NV vectors of VEC elements per thread).
// ---------------------------------------------------------------------------
constexpr int kMaxPeers = 8;

struct QuantAppendArgs {
  const void* x[2];     // xk, xv
  int8_t* cache[2];     // may be null
  void* scaler[2];      // may be null
  int8_t* quant[2];     // may be null (paged)
  void* scale_out[2];   // may be null (paged)
  const float* amax_in; // [2,B] amax to use instead of the local one, or null
  float* amax_out;      // [2,B]: write the local amax and stop, or null
  const int32_t* pos;   // dense
  int pos_count, pos_host;
  const int32_t* pti;   // paged: rows of pti_stride entries
  const int32_t* n_active_dev;  // optional device-side count
  int n_active;
  int64_t pti_stride;
  int paged;
  int B, H, S, D, ps;
  int64_t cs_b, cs_h, cs_s, ss_b, ss_s;  // dense; paged uses cs_h = P*ps*D, cs_s = D
  // Head-sharded caches: the partial amax of every rank travels through peer memory inside this launch.
  unsigned long long* px_slots[kMaxPeers];  // slot area of each rank's exchange buffer (index = rank); null: off
  unsigned* px_state;                       // this rank's {launches done, CTAs done, gave up}
  int px_rank, px_world;
  long long px_wait_cycles;                 // how long a rank waits for a peer's word
};

// Exchange buffer of one rank: kPeerStateBytes of state, then slots[parity][writer rank][2 B],
// each slot one 64-bit word (launch number << 32 | amax bits) written with a single store,
// so a reader sees either an older launch's word or the complete new one.
constexpr size_t kPeerStateBytes = 64;
constexpr long long kPeerWaitCycles = 1000000000ll;  // about half a second

__device__ __forceinline__ void st_peer(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_peer(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

template <typename T, int VEC>
struct VecIO;

template <int VEC>
struct VecIO<__nv_bfloat16, VEC> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[VEC]) {
    if constexpr (VEC == 1) {
      v[0] = __bfloat162float(p[0]);
    } else {
      static_assert(VEC % 8 == 0, "");
#pragma unroll
      for (int i = 0; i < VEC / 8; ++i) {
        uint4 raw = reinterpret_cast<const uint4*>(p)[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(h[j]);
          v[i * 8 + 2 * j] = f.x;
          v[i * 8 + 2 * j + 1] = f.y;
        }
      }
    }
  }
};

template <int VEC>
struct VecIO<float, VEC> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[VEC]) {
    if constexpr (VEC == 1) {
      v[0] = p[0];
    } else {
#pragma unroll
      for (int i = 0; i < VEC / 4; ++i) {
        float4 raw = reinterpret_cast<const float4*>(p)[i];
        v[i * 4] = raw.x; v[i * 4 + 1] = raw.y; v[i * 4 + 2] = raw.z; v[i * 4 + 3] = raw.w;
      }
    }
  }
};

template <int VEC>
__device__ __forceinline__ void store_codes(int8_t* p, const int8_t (&c)[VEC]) {
  if constexpr (VEC == 16) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(c);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = c[i];
  }
}

// NV = vectors per thread (token elements = NV * VEC * blockDim at most).
template <typename T, int VEC, int NV>
__global__ void __launch_bounds__(256) quant_append_kernel(QuantAppendArgs a) {
  __shared__ float red[33];
  grid_dependency_wait();     // the new token may come from the kernel before this one
  grid_dependency_trigger();  // the attention launch that follows may set itself up meanwhile
  const int item = blockIdx.x, which = blockIdx.y;
  const int HD = a.H * a.D;
  int slot, page = 0, tok = 0;
  if (a.paged) {
    const int n_act = a.n_active_dev ? *a.n_active_dev : a.n_active;
    if (item >= n_act) return;
    page = a.pti[item];
    tok = a.pti[a.pti_stride + item] - item * a.ps;
    slot = a.pti[2 * a.pti_stride + item];
    if (slot < 0 || slot >= a.B) return;
  } else {
    slot = item;
  }
  const T* x = static_cast<const T*>(a.x[which]) + (int64_t)slot * HD;

  float v[NV][VEC];
  float amax = 0.f;
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    const int e = (n * blockDim.x + threadIdx.x) * VEC;
    if (e < HD) {
      VecIO<T, VEC>::load(x + e, v[n]);
#pragma unroll
      for (int i = 0; i < VEC; ++i) amax = fmaxf(amax, fabsf(v[n][i]));
    }
  }
  amax = block_max(amax, red);
  if (a.px_state) {
    // All-ranks maximum over NVLink: thread 0 stores (launch number, partial amax) into every
    // rank's buffer and then reads the words the other ranks stored into this rank's buffer.
    __shared__ float s_amax;
    if (threadIdx.x == 0) {
      const unsigned epoch = *reinterpret_cast<volatile unsigned*>(&a.px_state[0]) + 1u;
      const int idx = which * a.B + slot;
      const size_t row = (size_t)(epoch & 1u) * a.px_world;
      const unsigned long long word = ((unsigned long long)epoch << 32) | __float_as_uint(amax);
      for (int r = 0; r < a.px_world; ++r) st_peer(a.px_slots[r] + (row + a.px_rank) * (2 * a.B) + idx, word);
      float m = amax;
      const long long t0 = clock64();
      for (int r = 0; r < a.px_world; ++r) {
        if (r == a.px_rank) continue;
        const unsigned long long* p = a.px_slots[a.px_rank] + (row + r) * (2 * a.B) + idx;
        unsigned long long v = ld_peer(p);
        while ((unsigned)(v >> 32) != epoch) {
          if (clock64() - t0 > a.px_wait_cycles) {  // the peer never came: report, go on with what is there
            atomicExch(&a.px_state[2], 1u);
            v = 0;
            break;
          }
          v = ld_peer(p);
        }
        m = fmaxf(m, __uint_as_float((unsigned)v));
      }
      s_amax = m;
    }
    __syncthreads();
    amax = s_amax;
  }
  if (a.amax_out) {  // phase one of a sharded update: publish the partial amax
    if (threadIdx.x == 0) a.amax_out[which * a.B + slot] = amax;
    return;
  }
  if (a.amax_in) amax = a.amax_in[which * a.B + slot];
  const float scale = decode_scale<T>(amax);

  // destination row
  bool write_cache = a.cache[which] != nullptr;
  int64_t row_base = 0, scaler_idx = 0;
  if (a.paged) {
    if (page < 0 || page >= a.S || tok < 0 || tok >= a.ps) write_cache = false;  // a.S holds P
    row_base = (int64_t)page * a.ps * a.D + (int64_t)tok * a.D;
    scaler_idx = (int64_t)page * a.ps + tok;
  } else {
    int p = a.pos ? a.pos[a.pos_count == 1 ? 0 : slot] : a.pos_host;
    if (p < 0) p += a.S;
    if (p < 0 || p >= a.S) write_cache = false;
    row_base = (int64_t)slot * a.cs_b + (int64_t)p * a.cs_s;
    scaler_idx = (int64_t)slot * a.ss_b + (int64_t)p * a.ss_s;
  }

#pragma unroll
  for (int n = 0; n < NV; ++n) {
    const int e = (n * blockDim.x + threadIdx.x) * VEC;
    if (e < HD) {
      int8_t c[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) c[i] = decode_code<T>(v[n][i], scale);
      if (a.quant[which]) store_codes<VEC>(a.quant[which] + (int64_t)slot * HD + e, c);
      if (write_cache) {
        const int h = e / a.D, d = e - h * a.D;  // VEC divides D: a vector never straddles heads
        store_codes<VEC>(a.cache[which] + row_base + (int64_t)h * a.cs_h + d, c);
      }
    }
  }
  if (threadIdx.x == 0) {
    if (a.scale_out[which]) static_cast<T*>(a.scale_out[which])[slot] = from_f32<T>(scale);
    if (write_cache && a.scaler[which]) static_cast<T*>(a.scaler[which])[scaler_idx] = from_f32<T>(scale);
    if (a.px_state) {  // the last CTA of the launch advances the launch number for the next one
      __threadfence();
      const unsigned done = atomicAdd(&a.px_state[1], 1u);
      if (done == gridDim.x * gridDim.y - 1) {
        a.px_state[1] = 0;
        __threadfence();
        atomicAdd(&a.px_state[0], 1u);
      }
    }
  }
}

template <typename T>
int launch_quant_append(const QuantAppendArgs& a, int items, cudaStream_t st) {
  const int HD = a.H * a.D;
  bool vec_ok = (a.D % 16 == 0) && (a.cs_h % 16 == 0) && (a.cs_s % 16 == 0) && (a.cs_b % 16 == 0);
  for (int w = 0; w < 2; ++w) {
    vec_ok = vec_ok && aligned(a.x[w], 16) && aligned(a.cache[w], 16) && aligned(a.quant[w], 16);
  }
  dim3 grid(items, 2);
  if (vec_ok && HD <= 16 * 256 * 2) {
    const int nvec = HD / 16;
    if (nvec <= 256) {
      int threads = ((nvec + 31) / 32) * 32;
      launch_after_previous(quant_append_kernel<T, 16, 1>, grid, dim3(threads), 0, st, a);
    } else {
      launch_after_previous(quant_append_kernel<T, 16, 2>, grid, dim3(256), 0, st, a);
    }
  } else {
    JPT_REQUIRE(HD <= 256 * 32, JPT_ERANGE, "quant_append: H*D = %d too large for the scalar path", HD);
    int threads = HD < 256 ? ((HD + 31) / 32) * 32 : 256;
    launch_after_previous(quant_append_kernel<T, 1, 32>, grid, dim3(threads), 0, st, a);
  }
  return check_launch("quant_append_kernel");
}

// ---------------------------------------------------------------------------
// Row scatter.  One thread per 16-byte chunk (or per element when unaligned).
// ---------------------------------------------------------------------------
struct ScatterArgs {
  const char* src[2];
  char* dst[2];
  const int32_t* pos;
  int pos_count, pos_host, clamp;
  int NL, B, H, S;
  int row_bytes, chunk;             // chunk = 16 or elem_bytes
  int64_t ds_l, ds_b, ds_h, ds_s;   // bytes
};

__global__ void scatter_rows_kernel(ScatterArgs a) {
  const int chunks_per_row = a.row_bytes / a.chunk;
  const int64_t total = (int64_t)a.NL * a.B * a.H * chunks_per_row;
  const int which = blockIdx.y;
  if (a.src[which] == nullptr) return;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % chunks_per_row);
    int64_t r = i / chunks_per_row;
    const int h = (int)(r % a.H);
    r /= a.H;
    const int b = (int)(r % a.B);
    const int l = (int)(r / a.B);
    int p = a.pos ? a.pos[a.pos_count == 1 ? 0 : b] : a.pos_host;
    if (a.clamp) {
      p = p < 0 ? 0 : (p > a.S - 1 ? a.S - 1 : p);
    } else {
      if (p < 0) p += a.S;
      if (p < 0 || p >= a.S) continue;
    }
    const char* s = a.src[which] + (((int64_t)l * a.B + b) * a.H + h) * a.row_bytes + (int64_t)c * a.chunk;
    char* d = a.dst[which] + l * a.ds_l + b * a.ds_b + h * a.ds_h + p * a.ds_s + (int64_t)c * a.chunk;
    if (a.chunk == 16) {
      *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(s);
    } else if (a.chunk == 4) {
      *reinterpret_cast<uint32_t*>(d) = *reinterpret_cast<const uint32_t*>(s);
    } else if (a.chunk == 2) {
      *reinterpret_cast<uint16_t*>(d) = *reinterpret_cast<const uint16_t*>(s);
    } else {
      *d = *s;
    }
  }
}

// ---------------------------------------------------------------------------
// Paged append without quantisation.
// ---------------------------------------------------------------------------
struct PagedCopyArgs {
  const char* x[2];
  char* cache[2];
  const int32_t* pti;
  const int32_t* n_active_dev;
  int64_t pti_stride;
  int n_active, B, H, P, ps;
  int row_bytes, chunk;
};

__global__ void paged_append_copy_kernel(PagedCopyArgs a) {
  const int chunks_per_row = a.row_bytes / a.chunk;
  const int n_act = a.n_active_dev ? *a.n_active_dev : a.n_active;
  const int64_t total = (int64_t)n_act * a.H * chunks_per_row;
  const int which = blockIdx.y;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % chunks_per_row);
    int64_t r = i / chunks_per_row;
    const int h = (int)(r % a.H);
    const int j = (int)(r / a.H);
    const int page = a.pti[j];
    const int tok = a.pti[a.pti_stride + j] - j * a.ps;
    const int slot = a.pti[2 * a.pti_stride + j];
    if (page < 0 || page >= a.P || tok < 0 || tok >= a.ps || slot < 0 || slot >= a.B) continue;
    const char* s = a.x[which] + ((int64_t)slot * a.H + h) * a.row_bytes + (int64_t)c * a.chunk;
    char* d = a.cache[which] + (((int64_t)h * a.P + page) * a.ps + tok) * a.row_bytes + (int64_t)c * a.chunk;
    if (a.chunk == 16) {
      *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(s);
    } else if (a.chunk == 4) {
      *reinterpret_cast<uint32_t*>(d) = *reinterpret_cast<const uint32_t*>(s);
    } else if (a.chunk == 2) {
      *reinterpret_cast<uint16_t*>(d) = *reinterpret_cast<const uint16_t*>(s);
    } else {
      *d = *s;
    }
  }
}

// ---------------------------------------------------------------------------
// get_page_token_indices on the device (single block, ordered compaction).
// ---------------------------------------------------------------------------
__global__ void page_token_indices_kernel(const int32_t* lens, const int32_t* page_indices, int B,
                                          int max_pages, int ps, int32_t* pti, int32_t* n_active,
                                          int32_t* new_lengths) {
  __shared__ int s_warp[33];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int len = tid < B ? lens[tid] : 0;
  const int active = len > 0;
  const unsigned ballot = __ballot_sync(0xffffffffu, active);
  const int in_warp = __popc(ballot & ((1u << lane) - 1));
  if (lane == 0) s_warp[warp] = __popc(ballot);
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
      int c = s_warp[w];
      s_warp[w] = acc;
      acc += c;
    }
    s_warp[32] = acc;
  }
  __syncthreads();
  const int total = s_warp[32];
  if (tid < B) {
    new_lengths[tid] = active ? len + 1 : 0;
    if (active) {
      const int j = s_warp[warp] + in_warp;
      int col = len / ps;
      if (col >= max_pages) col = max_pages - 1;
      // Rows of the compacted table are B wide so the layout does not depend
      // on the (device-side) count; entries past n_active are left untouched.
      pti[j] = page_indices[(int64_t)tid * max_pages + col];
      pti[B + j] = j * ps + len % ps;
      pti[2 * B + j] = tid;
    }
  }
  if (tid == 0) *n_active = total;
}

}  // namespace
}  // namespace jpt

using namespace jpt;

extern "C" const char* jpt_last_error_string(void) { return last_error_buffer(); }
extern "C" int jpt_version(void) { return 100; }
extern "C" long long jpt_launch_count(void) { return launch_count(); }

// Shared body of the dense entry points; px may be null.
static int quant_append_dense(const void* xk, const void* xv, int in_dtype, int8_t* cache_k, int8_t* cache_v,
                              void* k_scaler, void* v_scaler, int8_t* k_quant, int8_t* v_quant, void* k_scale,
                              void* v_scale, const int32_t* pos, int pos_count, int pos_host, int B, int H, int S,
                              int D, int64_t cs_b, int64_t cs_h, int64_t cs_s, int64_t ss_b, int64_t ss_s,
                              const float* amax_in, float* amax_out, const jpt_peer_exchange* px, void* stream);

extern "C" int jpt_kv_quant_append_dense(const void* xk, const void* xv, int in_dtype, int8_t* cache_k,
                                         int8_t* cache_v, void* k_scaler, void* v_scaler, int8_t* k_quant,
                                         int8_t* v_quant, void* k_scale, void* v_scale, const int32_t* pos,
                                         int pos_count, int pos_host, int B, int H, int S, int D,
                                         int64_t cs_b, int64_t cs_h, int64_t cs_s, int64_t ss_b,
                                         int64_t ss_s, const float* amax_in, float* amax_out,
                                         void* stream) {
  return quant_append_dense(xk, xv, in_dtype, cache_k, cache_v, k_scaler, v_scaler, k_quant, v_quant, k_scale, v_scale,
                            pos, pos_count, pos_host, B, H, S, D, cs_b, cs_h, cs_s, ss_b, ss_s, amax_in, amax_out,
                            nullptr, stream);
}

extern "C" int jpt_kv_quant_append_dense_peers(const void* xk, const void* xv, int in_dtype, int8_t* cache_k,
                                               int8_t* cache_v, void* k_scaler, void* v_scaler, int8_t* k_quant,
                                               int8_t* v_quant, void* k_scale, void* v_scale, const int32_t* pos,
                                               int pos_count, int pos_host, int B, int H, int S, int D,
                                               int64_t cs_b, int64_t cs_h, int64_t cs_s, int64_t ss_b,
                                               int64_t ss_s, const jpt_peer_exchange* px, void* stream) {
  JPT_REQUIRE(px, JPT_EINVAL, "kv_quant_append_dense_peers: null exchange");
  JPT_REQUIRE(px->world >= 1 && px->world <= kMaxPeers && px->rank >= 0 && px->rank < px->world, JPT_EINVAL,
              "kv_quant_append_dense_peers: rank %d of %d", px->rank, px->world);
  JPT_REQUIRE(px->batch == B, JPT_EINVAL, "kv_quant_append_dense_peers: buffers are sized for batch %d, not %d",
              px->batch, B);
  JPT_REQUIRE(px->wait_cycles >= 0, JPT_EINVAL, "kv_quant_append_dense_peers: negative wait limit");
  for (int r = 0; r < px->world; ++r)
    JPT_REQUIRE(px->buffers[r] && aligned(px->buffers[r], 8), JPT_EINVAL,
                "kv_quant_append_dense_peers: buffer of rank %d missing or unaligned", r);
  return quant_append_dense(xk, xv, in_dtype, cache_k, cache_v, k_scaler, v_scaler, k_quant, v_quant, k_scale, v_scale,
                            pos, pos_count, pos_host, B, H, S, D, cs_b, cs_h, cs_s, ss_b, ss_s, nullptr, nullptr, px,
                            stream);
}

extern "C" size_t jpt_peer_exchange_bytes(int B, int world) {
  if (B <= 0 || world <= 0 || world > kMaxPeers) return 0;
  return kPeerStateBytes + (size_t)2 * world * 2 * B * sizeof(unsigned long long);
}

extern "C" int jpt_peer_exchange_alloc(size_t bytes, void** ptr) {
  JPT_REQUIRE(ptr && bytes >= kPeerStateBytes, JPT_EINVAL, "peer_exchange_alloc: bad arguments");
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e == cudaSuccess) e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return fail((int)e, "peer_exchange_alloc: %s", cudaGetErrorString(e));
  return 0;
}

extern "C" int jpt_peer_exchange_free(void* ptr) {
  const cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail((int)e, "peer_exchange_free: %s", cudaGetErrorString(e));
  return 0;
}

extern "C" int jpt_peer_exchange_export(void* ptr, void* handle64) {
  JPT_REQUIRE(ptr && handle64, JPT_EINVAL, "peer_exchange_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  const cudaError_t e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), ptr);
  if (e != cudaSuccess) return fail((int)e, "peer_exchange_export: %s", cudaGetErrorString(e));
  return 0;
}

extern "C" int jpt_peer_exchange_import(const void* handle64, void** peer_ptr) {
  JPT_REQUIRE(handle64 && peer_ptr, JPT_EINVAL, "peer_exchange_import: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  const cudaError_t e = cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail((int)e, "peer_exchange_import: %s", cudaGetErrorString(e));
  return 0;
}

extern "C" int jpt_peer_exchange_release(void* peer_ptr) {
  const cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
  if (e != cudaSuccess) return fail((int)e, "peer_exchange_release: %s", cudaGetErrorString(e));
  return 0;
}

extern "C" int jpt_peer_exchange_status(const void* own_buffer, void* stream) {
  JPT_REQUIRE(own_buffer, JPT_EINVAL, "peer_exchange_status: null buffer");
  unsigned st3[3] = {0, 0, 0};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(st3, own_buffer, sizeof(st3), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail((int)e, "peer_exchange_status: %s", cudaGetErrorString(e));
  return (int)st3[2];
}

extern "C" int jpt_kv_scatter_rows(const void* src_k, const void* src_v, void* dst_k, void* dst_v,
                                   int elem_bytes, const int32_t* pos, int pos_count, int pos_host,
                                   int clamp, int NL, int B, int H, int S, int D, int64_t ds_l,
                                   int64_t ds_b, int64_t ds_h, int64_t ds_s, void* stream) {
  JPT_REQUIRE(src_k && dst_k, JPT_EINVAL, "kv_scatter_rows: null tensor");
  JPT_REQUIRE((src_v == nullptr) == (dst_v == nullptr), JPT_EINVAL, "kv_scatter_rows: src_v/dst_v mismatch");
  JPT_REQUIRE(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4, JPT_EINVAL,
              "kv_scatter_rows: elem_bytes must be 1, 2 or 4");
  JPT_REQUIRE(NL > 0 && B > 0 && H > 0 && D > 0 && S > 0, JPT_EINVAL, "kv_scatter_rows: bad shape");
  JPT_REQUIRE(pos == nullptr || pos_count == 1 || pos_count == B, JPT_EINVAL,
              "kv_scatter_rows: pos_count must be 1 or B");
  ScatterArgs a{};
  a.src[0] = static_cast<const char*>(src_k); a.src[1] = static_cast<const char*>(src_v);
  a.dst[0] = static_cast<char*>(dst_k); a.dst[1] = static_cast<char*>(dst_v);
  a.pos = pos; a.pos_count = pos_count; a.pos_host = pos_host; a.clamp = clamp;
  a.NL = NL; a.B = B; a.H = H; a.S = S;
  a.row_bytes = D * elem_bytes;
  a.ds_l = ds_l * elem_bytes; a.ds_b = ds_b * elem_bytes; a.ds_h = ds_h * elem_bytes; a.ds_s = ds_s * elem_bytes;
  bool v16 = a.row_bytes % 16 == 0 && a.ds_l % 16 == 0 && a.ds_b % 16 == 0 && a.ds_h % 16 == 0 &&
             a.ds_s % 16 == 0 && aligned(src_k, 16) && aligned(dst_k, 16) && aligned(src_v, 16) &&
             aligned(dst_v, 16);
  a.chunk = v16 ? 16 : elem_bytes;
  const int64_t total = (int64_t)NL * B * H * (a.row_bytes / a.chunk);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  dim3 grid(blocks, src_v ? 2 : 1);
  scatter_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("scatter_rows_kernel");
}

extern "C" int jpt_kv_append_paged(const void* xk, const void* xv, int in_dtype, void* cache_k,
                                   void* cache_v, int cache_dtype, void* k_scale_pool, void* v_scale_pool,
                                   const int32_t* pti, int64_t pti_stride, int n_active,
                                   const int32_t* n_active_dev, int B, int H, int P, int ps, int D,
                                   void* stream) {
  JPT_REQUIRE(xk && xv && cache_k && cache_v && pti, JPT_EINVAL, "kv_append_paged: null tensor");
  JPT_REQUIRE(B > 0 && H > 0 && P > 0 && ps > 0 && D > 0 && n_active >= 0 && n_active <= B, JPT_EINVAL,
              "kv_append_paged: bad shape");
  JPT_REQUIRE(pti_stride >= n_active, JPT_EINVAL, "kv_append_paged: pti_stride < n_active");
  if (n_active == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cache_dtype == in_dtype) {
    PagedCopyArgs a{};
    a.x[0] = static_cast<const char*>(xk); a.x[1] = static_cast<const char*>(xv);
    a.cache[0] = static_cast<char*>(cache_k); a.cache[1] = static_cast<char*>(cache_v);
    a.pti = pti; a.n_active = n_active; a.n_active_dev = n_active_dev; a.pti_stride = pti_stride;
    a.B = B; a.H = H; a.P = P; a.ps = ps;
    const int eb = dtype_bytes(in_dtype);
    JPT_REQUIRE(eb > 0, JPT_EINVAL, "kv_append_paged: bad dtype");
    a.row_bytes = D * eb;
    bool v16 = a.row_bytes % 16 == 0 && aligned(xk, 16) && aligned(xv, 16) && aligned(cache_k, 16) &&
               aligned(cache_v, 16);
    a.chunk = v16 ? 16 : eb;
    const int64_t total = (int64_t)n_active * H * (a.row_bytes / a.chunk);
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    paged_append_copy_kernel<<<dim3(blocks, 2), 256, 0, st>>>(a);
    return check_launch("paged_append_copy_kernel");
  }
  JPT_REQUIRE(cache_dtype == JPT_INT8 && (in_dtype == JPT_BF16 || in_dtype == JPT_F32), JPT_EINVAL,
              "kv_append_paged: unsupported dtype pair");
  JPT_REQUIRE(k_scale_pool && v_scale_pool, JPT_EINVAL, "kv_append_paged: int8 pools need scale pools");
  QuantAppendArgs a{};
  a.x[0] = xk; a.x[1] = xv;
  a.cache[0] = static_cast<int8_t*>(cache_k); a.cache[1] = static_cast<int8_t*>(cache_v);
  a.scaler[0] = k_scale_pool; a.scaler[1] = v_scale_pool;
  a.pti = pti; a.n_active = n_active; a.n_active_dev = n_active_dev; a.pti_stride = pti_stride; a.paged = 1;
  a.B = B; a.H = H; a.S = P; a.D = D; a.ps = ps;
  a.cs_b = 0; a.cs_h = (int64_t)P * ps * D; a.cs_s = D; a.ss_b = 0; a.ss_s = 1;
  return in_dtype == JPT_BF16 ? launch_quant_append<__nv_bfloat16>(a, n_active, st)
                              : launch_quant_append<float>(a, n_active, st);
}

extern "C" int jpt_page_token_indices(const int32_t* lens, const int32_t* page_indices, int B, int max_pages,
                                      int ps, int32_t* pti, int32_t* n_active, int32_t* new_lengths,
                                      void* stream) {
  JPT_REQUIRE(lens && page_indices && pti && n_active && new_lengths, JPT_EINVAL,
              "page_token_indices: null tensor");
  JPT_REQUIRE(B > 0 && B <= 1024 && max_pages > 0 && ps > 0, JPT_ERANGE,
              "page_token_indices: need 0 < B <= 1024");
  const int threads = ((B + 31) / 32) * 32;
  page_token_indices_kernel<<<1, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      lens, page_indices, B, max_pages, ps, pti, n_active, new_lengths);
  return check_launch("page_token_indices_kernel");
}

static int quant_append_dense(const void* xk, const void* xv, int in_dtype, int8_t* cache_k, int8_t* cache_v,
                              void* k_scaler, void* v_scaler, int8_t* k_quant, int8_t* v_quant, void* k_scale,
                              void* v_scale, const int32_t* pos, int pos_count, int pos_host, int B, int H, int S,
                              int D, int64_t cs_b, int64_t cs_h, int64_t cs_s, int64_t ss_b, int64_t ss_s,
                              const float* amax_in, float* amax_out, const jpt_peer_exchange* px, void* stream) {
  JPT_REQUIRE(xk && xv, JPT_EINVAL, "kv_quant_append_dense: null input");
  JPT_REQUIRE(in_dtype == JPT_BF16 || in_dtype == JPT_F32, JPT_EINVAL,
              "kv_quant_append_dense: input dtype must be bf16 or f32");
  JPT_REQUIRE(B > 0 && H > 0 && D > 0 && S > 0, JPT_EINVAL, "kv_quant_append_dense: bad shape");
  JPT_REQUIRE((cache_k == nullptr) == (cache_v == nullptr), JPT_EINVAL,
              "kv_quant_append_dense: cache_k and cache_v must both be given or both be null");
  JPT_REQUIRE(pos == nullptr || pos_count == 1 || pos_count == B, JPT_EINVAL,
              "kv_quant_append_dense: pos_count must be 1 or B");
  QuantAppendArgs a{};
  a.x[0] = xk; a.x[1] = xv;
  a.cache[0] = cache_k; a.cache[1] = cache_v;
  a.scaler[0] = k_scaler; a.scaler[1] = v_scaler;
  a.quant[0] = k_quant; a.quant[1] = v_quant;
  a.scale_out[0] = k_scale; a.scale_out[1] = v_scale;
  a.pos = pos; a.pos_count = pos_count; a.pos_host = pos_host;
  a.amax_in = amax_in; a.amax_out = amax_out;
  if (px) {
    for (int r = 0; r < px->world; ++r)
      a.px_slots[r] = reinterpret_cast<unsigned long long*>(static_cast<char*>(px->buffers[r]) + kPeerStateBytes);
    a.px_state = static_cast<unsigned*>(px->buffers[px->rank]);
    a.px_rank = px->rank;
    a.px_world = px->world;
    a.px_wait_cycles = px->wait_cycles > 0 ? px->wait_cycles : kPeerWaitCycles;
  }
  a.paged = 0;
  a.B = B; a.H = H; a.S = S; a.D = D; a.ps = 0;
  a.cs_b = cs_b; a.cs_h = cs_h; a.cs_s = cs_s; a.ss_b = ss_b; a.ss_s = ss_s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return in_dtype == JPT_BF16 ? launch_quant_append<__nv_bfloat16>(a, B, st)
                              : launch_quant_append<float>(a, B, st);
}

