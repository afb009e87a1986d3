// Prefill -> decode-slot insert: scatter a prefix's K/V rows into a dense cache
// slot (clamped or modular positions) or into pages (zero-filled tail), with
// optional per-token int8 quantisation (round half even, EPS-clamped scale).
#include "common.cuh"

namespace jpt {
namespace {

struct InsertArgs {
  const void* prefix[2];
  void* cache[2];
  void* scaler[2];  // may be null
  const int32_t* upd;  // paged: page ids
  int paged, wrap;
  int ntensors;  // 2 = K and V, 1 = a single tensor
  int slot, pos;
  int NL, H, L, Ltot, S, D, P, ps;
  int64_t ps_l, ps_h, ps_t;        // prefix strides (elements)
  int64_t cs_l, cs_b, cs_h, cs_s;  // cache strides (elements)
  int64_t ss_l, ss_b, ss_s;        // scaler strides (elements)
};

struct Dest {
  int64_t row0;   // element offset of (h = 0, d = 0) for this token
  int64_t sidx;   // scaler element offset
  int64_t hstep;  // elements between heads
  bool ok;
};

__device__ __forceinline__ Dest resolve(const InsertArgs& a, int l, int t) {
  Dest d;
  d.ok = true;
  if (a.paged) {
    const int page = a.upd[t / a.ps], tok = t % a.ps;
    if (page < 0 || page >= a.P) d.ok = false;
    d.row0 = l * a.cs_l + ((int64_t)page * a.ps + tok) * a.D;
    d.hstep = (int64_t)a.P * a.ps * a.D;
    d.sidx = l * a.ss_l + (int64_t)page * a.ps + tok;
  } else {
    int s;
    if (a.wrap) {
      s = (a.pos + t) % a.S;
      if (s < 0) s += a.S;
    } else {
      s = a.pos + t;  // pos already clamped on the host
      if (s < 0 || s >= a.S) d.ok = false;
    }
    d.row0 = l * a.cs_l + (int64_t)a.slot * a.cs_b + (int64_t)s * a.cs_s;
    d.hstep = a.cs_h;
    d.sidx = l * a.ss_l + (int64_t)a.slot * a.ss_b + (int64_t)s * a.ss_s;
  }
  return d;
}

template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T* p, float (&v)[VEC]) {
  if constexpr (VEC == 1) {
    v[0] = to_f32<T>(p[0]);
  } else if constexpr (sizeof(T) == 2) {
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
  } else {
#pragma unroll
    for (int i = 0; i < VEC / 4; ++i) {
      float4 raw = reinterpret_cast<const float4*>(p)[i];
      v[i * 4] = raw.x; v[i * 4 + 1] = raw.y; v[i * 4 + 2] = raw.z; v[i * 4 + 3] = raw.w;
    }
  }
}

// grid (Ltot, 2, NL); one block per token of one tensor of one layer.
template <typename T, int VEC, int NV>
__global__ void __launch_bounds__(256) insert_quant_kernel(InsertArgs a) {
  __shared__ float red[33];
  const int t = blockIdx.x, which = blockIdx.y, l = blockIdx.z;
  const int HD = a.H * a.D;
  const Dest dst = resolve(a, l, t);
  int8_t* cache = static_cast<int8_t*>(a.cache[which]);
  T* scaler = static_cast<T*>(a.scaler[which]);
  if (t >= a.L) {  // page tail: code 0, scale 0
    if (!dst.ok) return;
    for (int n = 0; n < NV; ++n) {
      const int e = (n * blockDim.x + threadIdx.x) * VEC;
      if (e < HD) {
        const int h = e / a.D, d = e - h * a.D;
        int8_t* p = cache + dst.row0 + h * dst.hstep + d;
        if constexpr (VEC == 16) {
          *reinterpret_cast<uint4*>(p) = make_uint4(0, 0, 0, 0);
        } else {
          for (int i = 0; i < VEC; ++i) p[i] = 0;
        }
      }
    }
    if (threadIdx.x == 0 && scaler) scaler[dst.sidx] = from_f32<T>(0.f);
    return;
  }
  const T* src = static_cast<const T*>(a.prefix[which]) + l * a.ps_l + (int64_t)t * a.ps_t;
  float v[NV][VEC];
  float amax = 0.f;
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    const int e = (n * blockDim.x + threadIdx.x) * VEC;
    if (e < HD) {
      const int h = e / a.D, d = e - h * a.D;
      load_vec<T, VEC>(src + h * a.ps_h + d, v[n]);
#pragma unroll
      for (int i = 0; i < VEC; ++i) amax = fmaxf(amax, fabsf(v[n][i]));
    }
  }
  amax = block_max(amax, red);
  const float scale = insert_scale<T>(amax);
  const float recip = insert_recip<T>(scale);
  if (!dst.ok) return;
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    const int e = (n * blockDim.x + threadIdx.x) * VEC;
    if (e < HD) {
      const int h = e / a.D, d = e - h * a.D;
      int8_t c[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) c[i] = insert_code<T>(v[n][i], recip);
      int8_t* p = cache + dst.row0 + h * dst.hstep + d;
      if constexpr (VEC == 16) {
        *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(c);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) p[i] = c[i];
      }
    }
  }
  if (threadIdx.x == 0 && scaler) scaler[dst.sidx] = from_f32<T>(scale);
}

// The same work with one warp per token (8 tokens per CTA) and NVW 16-element
// vectors per lane: the maximum stays inside the warp (no shared memory, no
// block barrier) and every lane has NVW independent loads in flight.  Used
// when H*D is a multiple of 512.
template <typename T, int NVW>
__global__ void __launch_bounds__(256) insert_quant_warp_kernel(InsertArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp, which = blockIdx.y, l = blockIdx.z;
  if (t >= a.Ltot) return;
  const Dest dst = resolve(a, l, t);
  int8_t* cache = static_cast<int8_t*>(a.cache[which]);
  T* scaler = static_cast<T*>(a.scaler[which]);
  if (t >= a.L) {  // page tail: code 0, scale 0
    if (!dst.ok) return;
#pragma unroll
    for (int n = 0; n < NVW; ++n) {
      const int e = (n * 32 + lane) * 16;
      const int h = e / a.D, d = e - h * a.D;
      *reinterpret_cast<uint4*>(cache + dst.row0 + h * dst.hstep + d) = make_uint4(0, 0, 0, 0);
    }
    if (lane == 0 && scaler) scaler[dst.sidx] = from_f32<T>(0.f);
    return;
  }
  const T* src = static_cast<const T*>(a.prefix[which]) + l * a.ps_l + (int64_t)t * a.ps_t;
  if constexpr (sizeof(T) == 2) {
    // bf16 tokens: the reference's chain is a chain of bf16 operations, which the packed bf16
    // instructions perform exactly (|x| and max are exact; the product of two bf16 values rounded
    // once to bf16 is what `bf16(w * r)` is), two elements per instruction.
    uint4 raw[NVW][2];
#pragma unroll
    for (int n = 0; n < NVW; ++n) {
      const int e = (n * 32 + lane) * 16;
      const int h = e / a.D, d = e - h * a.D;
      const uint4* p = reinterpret_cast<const uint4*>(src + h * a.ps_h + d);
      raw[n][0] = p[0];
      raw[n][1] = p[1];
    }
    __nv_bfloat162 m2 = __float2bfloat162_rn(0.f);
#pragma unroll
    for (int n = 0; n < NVW; ++n)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[n][j]);
#pragma unroll
        for (int i = 0; i < 4; ++i) m2 = __hmax2(m2, __habs2(h2[i]));
      }
    const float2 mf = __bfloat1622float2(m2);
    float amax = fmaxf(mf.x, mf.y);
#pragma unroll
    for (int sh = 16; sh >= 1; sh >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sh));
    const float scale = insert_scale<T>(amax);
    const float recip = insert_recip<T>(scale);
    if (!dst.ok) return;
    const __nv_bfloat162 r2 = __float2bfloat162_rn(recip);  // (exact: recip is a bf16 value)
#pragma unroll
    for (int n = 0; n < NVW; ++n) {
      const int e = (n * 32 + lane) * 16;
      const int h = e / a.D, d = e - h * a.D;
      uint32_t packed[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[n][j]);
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // four elements -> four bytes
          const float2 lo = __bfloat1622float2(__hmul2(h2[2 * i], r2)), hi = __bfloat1622float2(__hmul2(h2[2 * i + 1], r2));
          // round half to even, then saturate to int8 while packing (element 0 in the lowest byte)
          const int q0 = __float2int_rn(lo.x), q1 = __float2int_rn(lo.y), q2 = __float2int_rn(hi.x), q3 = __float2int_rn(hi.y);
          uint32_t top, all;
          asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(top) : "r"(q3), "r"(q2), "r"(0));
          asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(all) : "r"(q1), "r"(q0), "r"(top));
          packed[2 * j + i] = all;
        }
      }
      *reinterpret_cast<uint4*>(cache + dst.row0 + h * dst.hstep + d) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    if (lane == 0 && scaler) scaler[dst.sidx] = from_f32<T>(scale);
    return;
  }
  float v[NVW][16];
  float amax = 0.f;
#pragma unroll
  for (int n = 0; n < NVW; ++n) {
    const int e = (n * 32 + lane) * 16;
    const int h = e / a.D, d = e - h * a.D;
    load_vec<T, 16>(src + h * a.ps_h + d, v[n]);
  }
#pragma unroll
  for (int n = 0; n < NVW; ++n)
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[n][i]));
#pragma unroll
  for (int sh = 16; sh >= 1; sh >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sh));
  const float scale = insert_scale<T>(amax);
  const float recip = insert_recip<T>(scale);
  if (!dst.ok) return;
#pragma unroll
  for (int n = 0; n < NVW; ++n) {
    const int e = (n * 32 + lane) * 16;
    const int h = e / a.D, d = e - h * a.D;
    int8_t c[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) c[i] = insert_code<T>(v[n][i], recip);
    *reinterpret_cast<uint4*>(cache + dst.row0 + h * dst.hstep + d) = *reinterpret_cast<const uint4*>(c);
  }
  if (lane == 0 && scaler) scaler[dst.sidx] = from_f32<T>(scale);
}

// Same-dtype copy: one thread per chunk of `chunk` bytes.
__global__ void insert_copy_kernel(InsertArgs a, int elem_bytes, int chunk) {
  const int which = blockIdx.y, l = blockIdx.z;
  const int row_bytes = a.D * elem_bytes;
  const int cpr = row_bytes / chunk;
  const int64_t total = (int64_t)a.Ltot * a.H * cpr;
  const char* src = static_cast<const char*>(a.prefix[which]);
  char* cache = static_cast<char*>(a.cache[which]);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    // chunk fastest, then token, then head: consecutive threads walk one
    // (head, token-range) stripe of the prefix, which is contiguous in memory.
    const int c = (int)(i % cpr);
    int64_t r = i / cpr;
    const int t = (int)(r % a.Ltot);
    const int h = (int)(r / a.Ltot);
    const Dest dst = resolve(a, l, t);
    if (!dst.ok) continue;
    char* d = cache + (dst.row0 + h * dst.hstep) * elem_bytes + (int64_t)c * chunk;
    const char* s = src + (l * a.ps_l + h * a.ps_h + (int64_t)t * a.ps_t) * elem_bytes + (int64_t)c * chunk;
    const bool pad = t >= a.L;
    if (chunk == 16) {
      *reinterpret_cast<uint4*>(d) = pad ? make_uint4(0, 0, 0, 0) : *reinterpret_cast<const uint4*>(s);
    } else if (chunk == 4) {
      *reinterpret_cast<uint32_t*>(d) = pad ? 0u : *reinterpret_cast<const uint32_t*>(s);
    } else if (chunk == 2) {
      *reinterpret_cast<uint16_t*>(d) = pad ? (uint16_t)0 : *reinterpret_cast<const uint16_t*>(s);
    } else {
      *d = pad ? (char)0 : *s;
    }
  }
}

template <typename T>
int launch_quant(const InsertArgs& a, cudaStream_t st) {
  const int HD = a.H * a.D;
  bool vec_ok = a.D % 16 == 0 && a.ps_l % 8 == 0 && a.ps_h % 8 == 0 && a.ps_t % 8 == 0 &&
                a.cs_l % 16 == 0 && a.cs_b % 16 == 0 && a.cs_h % 16 == 0 && a.cs_s % 16 == 0;
  for (int w = 0; w < a.ntensors; ++w) vec_ok = vec_ok && aligned(a.prefix[w], 16) && aligned(a.cache[w], 16);
  dim3 grid(a.Ltot, a.ntensors, a.NL);
  if (vec_ok && (HD == 512 || HD == 1024 || HD == 2048)) {
    const dim3 wgrid((a.Ltot + 7) / 8, a.ntensors, a.NL);
    if (HD == 512) insert_quant_warp_kernel<T, 1><<<wgrid, 256, 0, st>>>(a);
    else if (HD == 1024) insert_quant_warp_kernel<T, 2><<<wgrid, 256, 0, st>>>(a);
    else insert_quant_warp_kernel<T, 4><<<wgrid, 256, 0, st>>>(a);
    return check_launch("insert_quant_warp_kernel");
  }
  if (vec_ok && HD <= 16 * 256 * 2) {
    const int nvec = HD / 16;
    if (nvec <= 256) {
      insert_quant_kernel<T, 16, 1><<<grid, ((nvec + 31) / 32) * 32, 0, st>>>(a);
    } else {
      insert_quant_kernel<T, 16, 2><<<grid, 256, 0, st>>>(a);
    }
  } else {
    JPT_REQUIRE(HD <= 256 * 32, JPT_ERANGE, "prefill_insert: H*D = %d too large for the scalar path", HD);
    const int threads = HD < 256 ? ((HD + 31) / 32) * 32 : 256;
    insert_quant_kernel<T, 1, 32><<<grid, threads, 0, st>>>(a);
  }
  return check_launch("insert_quant_kernel");
}

int launch_insert(InsertArgs& a, int in_dtype, int cache_dtype, cudaStream_t st) {
  JPT_REQUIRE(a.prefix[0] && a.cache[0] && (a.ntensors == 1 || (a.prefix[1] && a.cache[1])), JPT_EINVAL, "prefill_insert: null tensor");
  JPT_REQUIRE(a.NL > 0 && a.H > 0 && a.L >= 0 && a.D > 0, JPT_EINVAL, "prefill_insert: bad shape");
  if (a.Ltot == 0) return 0;
  if (cache_dtype == JPT_INT8 && in_dtype != JPT_INT8) {
    JPT_REQUIRE(in_dtype == JPT_BF16 || in_dtype == JPT_F32, JPT_EINVAL, "prefill_insert: bad input dtype");
    return in_dtype == JPT_BF16 ? launch_quant<__nv_bfloat16>(a, st) : launch_quant<float>(a, st);
  }
  JPT_REQUIRE(cache_dtype == in_dtype, JPT_EINVAL,
              "prefill_insert: cache dtype must equal the input dtype or be int8");
  const int eb = dtype_bytes(in_dtype);
  JPT_REQUIRE(eb > 0, JPT_EINVAL, "prefill_insert: bad dtype");
  const int row_bytes = a.D * eb;
  bool v16 = row_bytes % 16 == 0;
  const int64_t strides[] = {a.ps_l, a.ps_h, a.ps_t, a.cs_l, a.cs_b, a.cs_h, a.cs_s};
  for (int64_t s : strides) v16 = v16 && (s * eb) % 16 == 0;
  for (int w = 0; w < a.ntensors; ++w) v16 = v16 && aligned(a.prefix[w], 16) && aligned(a.cache[w], 16);
  const int chunk = v16 ? 16 : eb;
  const int64_t total = (int64_t)a.Ltot * a.H * (row_bytes / chunk);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  insert_copy_kernel<<<dim3(blocks, a.ntensors, a.NL), 256, 0, st>>>(a, eb, chunk);
  return check_launch("insert_copy_kernel");
}

}  // namespace
}  // namespace jpt

using namespace jpt;

extern "C" int jpt_prefill_insert_dense(const void* prefix_k, const void* prefix_v, int in_dtype,
                                        void* cache_k, void* cache_v, int cache_dtype, void* k_scaler,
                                        void* v_scaler, int slot, int pos, int wrap, int NL, int H, int L,
                                        int S, int D, int64_t ps_l, int64_t ps_h, int64_t ps_t,
                                        int64_t cs_l, int64_t cs_b, int64_t cs_h, int64_t cs_s,
                                        int64_t ss_l, int64_t ss_b, int64_t ss_s, void* stream) {
  JPT_REQUIRE(S > 0 && slot >= 0, JPT_EINVAL, "prefill_insert_dense: bad slot or cache length");
  JPT_REQUIRE(wrap || L <= S, JPT_ERANGE, "prefill_insert_dense: prefix longer than the cache (L=%d, S=%d)", L, S);
  InsertArgs a{};
  a.prefix[0] = prefix_k; a.prefix[1] = prefix_v;
  a.cache[0] = cache_k; a.cache[1] = cache_v;
  a.scaler[0] = k_scaler; a.scaler[1] = v_scaler;
  a.paged = 0; a.wrap = wrap; a.slot = slot; a.ntensors = 2;
  if (!wrap) pos = pos < 0 ? 0 : (pos > S - L ? S - L : pos);  // dynamic_update_slice clamps
  a.pos = pos;
  a.NL = NL; a.H = H; a.L = L; a.Ltot = L; a.S = S; a.D = D;
  a.ps_l = ps_l; a.ps_h = ps_h; a.ps_t = ps_t;
  a.cs_l = cs_l; a.cs_b = cs_b; a.cs_h = cs_h; a.cs_s = cs_s;
  a.ss_l = ss_l; a.ss_b = ss_b; a.ss_s = ss_s;
  return launch_insert(a, in_dtype, cache_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int jpt_prefill_insert_paged(const void* prefix_k, const void* prefix_v, int in_dtype,
                                        void* cache_k, void* cache_v, int cache_dtype, void* k_scale_pool,
                                        void* v_scale_pool, const int32_t* update_indexes, int n_pages,
                                        int NL, int H, int L, int P, int ps, int D, int64_t ps_l,
                                        int64_t ps_h, int64_t ps_t, int64_t cs_l, int64_t ss_l,
                                        void* stream) {
  JPT_REQUIRE(update_indexes != nullptr || n_pages == 0, JPT_EINVAL, "prefill_insert_paged: null page list");
  JPT_REQUIRE(P > 0 && ps > 0 && n_pages >= 0, JPT_EINVAL, "prefill_insert_paged: bad pool shape");
  JPT_REQUIRE((int64_t)n_pages * ps >= L, JPT_ERANGE,
              "prefill_insert_paged: %d pages of %d tokens cannot hold a prefix of %d", n_pages, ps, L);
  InsertArgs a{};
  a.prefix[0] = prefix_k; a.prefix[1] = prefix_v;
  a.cache[0] = cache_k; a.cache[1] = cache_v;
  a.scaler[0] = k_scale_pool; a.scaler[1] = v_scale_pool;
  a.upd = update_indexes;
  a.paged = 1; a.ntensors = 2;
  a.NL = NL; a.H = H; a.L = L; a.Ltot = n_pages * ps; a.D = D; a.P = P; a.ps = ps;
  a.ps_l = ps_l; a.ps_h = ps_h; a.ps_t = ps_t;
  a.cs_l = cs_l; a.ss_l = ss_l;
  return launch_insert(a, in_dtype, cache_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int jpt_quantize_tokens(const void* w, int in_dtype, int token_major, int H, int L, int D,
                                   int8_t* codes, void* scales, void* stream) {
  JPT_REQUIRE(w && codes && scales, JPT_EINVAL, "quantize_tokens: null tensor");
  JPT_REQUIRE(in_dtype == JPT_BF16 || in_dtype == JPT_F32, JPT_EINVAL, "quantize_tokens: bad dtype");
  InsertArgs a{};
  a.ntensors = 1;
  a.prefix[0] = w;
  a.cache[0] = codes;
  a.scaler[0] = scales;
  a.paged = 0; a.wrap = 0; a.slot = 0; a.pos = 0;
  a.NL = 1; a.H = H; a.L = L; a.Ltot = L; a.S = L; a.D = D;
  if (token_major) {
    a.ps_h = D; a.ps_t = (int64_t)H * D; a.cs_h = D; a.cs_s = (int64_t)H * D;
  } else {
    a.ps_h = (int64_t)L * D; a.ps_t = D; a.cs_h = (int64_t)L * D; a.cs_s = D;
  }
  a.ss_s = 1;
  return launch_insert(a, in_dtype, JPT_INT8, static_cast<cudaStream_t>(stream));
}

// Lets kernels launched on `device` read the memory of `peer` (NVLink peer loads): what a decode GPU needs
// to insert a prefix that still lies in the prefill GPU's memory.  Idempotent; the current device is kept.
extern "C" int jpt_enable_peer_access(int device, int peer) {
  JPT_REQUIRE(device >= 0 && peer >= 0, JPT_EINVAL, "enable_peer_access: negative device");
  if (device == peer) return 0;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, device, peer);
  if (e != cudaSuccess) return fail((int)e, "enable_peer_access: %s", cudaGetErrorString(e));
  JPT_REQUIRE(can, JPT_EINVAL, "enable_peer_access: device %d cannot access the memory of device %d", device, peer);
  int cur = 0;
  cudaGetDevice(&cur);
  e = cudaSetDevice(device);
  if (e == cudaSuccess) {
    e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      cudaGetLastError();  // (not an error: clear it)
      e = cudaSuccess;
    }
  }
  cudaSetDevice(cur);
  if (e != cudaSuccess) return fail((int)e, "enable_peer_access: %s", cudaGetErrorString(e));
  return 0;
}
