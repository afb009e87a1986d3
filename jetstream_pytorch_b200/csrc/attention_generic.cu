// Decode attention, scalar kernel for any head_dim <= 256, any row count and
// any of bf16 / fp32 / int8 caches, plus the split-K merge, the two-partial
// merge and the jpt_flash_decode dispatcher.  The tensor-core kernel for
// head_dim 128 lives in attention_mma.cu; this one covers every other shape.
#include <math.h>

#include <atomic>

#include "attention_tiles.cuh"

namespace jpt {
namespace {

constexpr int kWarps = 4;
constexpr int kRowTile = 4;   // query rows per block
constexpr int kMaxDPL = 8;    // head_dim <= 32 * kMaxDPL

template <typename TQ, typename TKV>
__global__ void __launch_bounds__(kWarps * 32) flash_decode_generic_kernel(AttnArgs a) {
  extern __shared__ float smem[];
  const int split = blockIdx.x;
  const int rc = blockIdx.y % ((a.R + kRowTile - 1) / kRowTile);
  const int h = blockIdx.y / ((a.R + kRowTile - 1) / kRowTile);
  const int b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r0 = rc * kRowTile;
  const int nrows = min(kRowTile, a.R - r0);
  const int D = a.D;

  float* q_s = smem;                         // [kRowTile][D], pre-scaled by sm_scale
  float* red = smem + kRowTile * D;          // [kWarps][kRowTile][D + 2]

  const int64_t row_base = ((int64_t)b * a.Hkv + h) * a.R + r0;
  const TQ* q = static_cast<const TQ*>(a.q) + row_base * D;
  for (int i = threadIdx.x; i < kRowTile * D; i += blockDim.x) {
    const int r = i / D;
    q_s[i] = r < nrows ? to_f32<TQ>(q[i]) * (a.round_logits ? 1.f : a.sm_scale) : 0.f;
  }
  __syncthreads();

  const SeqRange rg = seq_range(a, b);
  const int chunk = (rg.n + a.nsplit - 1) / a.nsplit;
  const int j0 = split * chunk;
  const int j1 = min(rg.n, j0 + chunk);

  float m[kRowTile], l[kRowTile], o[kRowTile][kMaxDPL];
#pragma unroll
  for (int r = 0; r < kRowTile; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxDPL; ++i) o[r][i] = 0.f;
  }

  const TKV* kbase = static_cast<const TKV*>(a.k);
  const TKV* vbase = static_cast<const TKV*>(a.v);
  const TQ* mask = static_cast<const TQ*>(a.mask);

  for (int j = j0 + warp; j < j1; j += kWarps) {
    const int p = physical_pos(a, rg, j);
    int64_t sidx;
    const int64_t off = kv_row_offset(a, b, h, p, &sidx);
    float kk[kMaxDPL], vv[kMaxDPL];
#pragma unroll
    for (int i = 0; i < kMaxDPL; ++i) {
      const int d = lane + 32 * i;
      kk[i] = d < D ? to_f32<TKV>(kbase[off + d]) : 0.f;
      vv[i] = d < D ? to_f32<TKV>(vbase[off + d]) : 0.f;
    }
    float ks = 1.f, vs = 1.f;
    if (a.k_scale) {
      ks = load_scale(a.k_scale, sidx, a.scale_is_f32);
      vs = load_scale(a.v_scale, sidx, a.scale_is_f32);
    }
#pragma unroll
    for (int r = 0; r < kRowTile; ++r) {
      if (r >= nrows) break;
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxDPL; ++i) {
        const int d = lane + 32 * i;
        if (d < D) s += q_s[r * D + d] * kk[i];
      }
      s = warp_sum(s);
      const float mask_value =
          a.mask_mode == JPT_MASK_ADD ? to_f32<TQ>(mask[(int64_t)b * a.mk_b + (int64_t)(r0 + r) * a.mk_r + p]) : 0.f;
      if (a.round_logits) {
        s = rounded_logit(s, __frcp_rn(a.sm_scale), ks, a.k_scale != nullptr, mask_value);
      } else {
        s = s * ks + mask_value;
      }
      if (s == -INFINITY) continue;  // fully masked position
      const float mn = fmaxf(m[r], s);
      const float corr = expf(m[r] - mn);  // exp(-inf) = 0 on the first token
      const float pr = expf(s - mn);
      l[r] = l[r] * corr + pr;
      const float pv = pr * vs;
#pragma unroll
      for (int i = 0; i < kMaxDPL; ++i) o[r][i] = o[r][i] * corr + pv * vv[i];
      m[r] = mn;
    }
  }

  // combine the warps of the block
  const int stride = D + 2;
  for (int r = 0; r < nrows; ++r) {
    float* dst = red + ((int64_t)warp * kRowTile + r) * stride;
#pragma unroll
    for (int i = 0; i < kMaxDPL; ++i) {
      const int d = lane + 32 * i;
      if (d < D) dst[d] = o[r][i];
    }
    if (lane == 0) {
      dst[D] = m[r];
      dst[D + 1] = l[r];
    }
  }
  __syncthreads();
  for (int r = 0; r < nrows; ++r) {
    float M = -INFINITY;
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, red[((int64_t)w * kRowTile + r) * stride + D]);
    float L = 0.f;
    float wgt[kWarps];
    for (int w = 0; w < kWarps; ++w) {
      const float mw = red[((int64_t)w * kRowTile + r) * stride + D];
      wgt[w] = mw == -INFINITY ? 0.f : expf(mw - M);
      L += wgt[w] * red[((int64_t)w * kRowTile + r) * stride + D + 1];
    }
    const int64_t row = row_base + r;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float acc = 0.f;
      for (int w = 0; w < kWarps; ++w) acc += wgt[w] * red[((int64_t)w * kRowTile + r) * stride + d];
      if (a.nsplit == 1) {
        const float out = L > 0.f ? acc / L : 0.f;
        static_cast<TQ*>(a.o)[row * D + d] = from_f32<TQ>(out);
      } else {
        a.ws_o[(row * a.nsplit + split) * D + d] = acc;
      }
    }
    if (threadIdx.x == 0) {
      if (a.nsplit == 1) {
        if (a.m) a.m[row] = M;
        if (a.l) a.l[row] = L;
      } else {
        a.ws_m[row * a.nsplit + split] = M;
        a.ws_l[row * a.nsplit + split] = L;
      }
    }
  }
}

// One block per output row: combine the nsplit partials.
template <typename TQ>
__global__ void splitk_merge_kernel(AttnArgs a) {
  const int64_t row = blockIdx.x;
  const int D = a.D;
  float M = -INFINITY;
  for (int s = 0; s < a.nsplit; ++s) M = fmaxf(M, a.ws_m[row * a.nsplit + s]);
  float L = 0.f;
  for (int s = 0; s < a.nsplit; ++s) {
    const float ms = a.ws_m[row * a.nsplit + s];
    if (ms != -INFINITY) L += expf(ms - M) * a.ws_l[row * a.nsplit + s];
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < a.nsplit; ++s) {
      const float ms = a.ws_m[row * a.nsplit + s];
      if (ms != -INFINITY) acc += expf(ms - M) * a.ws_o[(row * a.nsplit + s) * D + d];
    }
    static_cast<TQ*>(a.o)[row * D + d] = from_f32<TQ>(L > 0.f ? acc / L : 0.f);
  }
  if (threadIdx.x == 0) {
    if (a.m) a.m[row] = M;
    if (a.l) a.l[row] = L;
  }
}

template <typename TI, typename TO>
__global__ void merge_partials_kernel(const TI* o1, const float* m1, const float* l1, const TI* o2,
                                      const float* m2, const float* l2, TO* o, int64_t rows, int D) {
  const int64_t total = rows * D;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / D;
    const float a1 = m1[r], a2 = m2[r];
    const float g = fmaxf(a1, a2);
    // An empty side has m = -inf and l = 0; its weight is zero (the reference
    // formula would produce exp(-inf - -inf) only when both sides are empty).
    const float alpha = a1 == -INFINITY ? 0.f : expf(a1 - g);
    const float beta = a2 == -INFINITY ? 0.f : expf(a2 - g);
    const float denom = alpha * l1[r] + beta * l2[r];
    const float num = l1[r] * alpha * to_f32<TI>(o1[i]) + beta * to_f32<TI>(o2[i]) * l2[r];
    o[i] = from_f32<TO>(num / denom);
  }
}

template <typename TQ>
int launch_generic_kv(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st) {
  const int rcs = (a.R + kRowTile - 1) / kRowTile;
  dim3 grid(a.nsplit, a.Hkv * rcs, a.B);
  const size_t smem = sizeof(float) * (kRowTile * a.D + kWarps * kRowTile * (a.D + 2));
  switch (p.kv_dtype) {
    case JPT_BF16:
      flash_decode_generic_kernel<TQ, __nv_bfloat16><<<grid, kWarps * 32, smem, st>>>(a);
      break;
    case JPT_F32:
      flash_decode_generic_kernel<TQ, float><<<grid, kWarps * 32, smem, st>>>(a);
      break;
    case JPT_INT8:
      flash_decode_generic_kernel<TQ, int8_t><<<grid, kWarps * 32, smem, st>>>(a);
      break;
    default:
      return fail(JPT_EINVAL, "flash_decode: bad kv dtype %d", p.kv_dtype);
  }
  return check_launch("flash_decode_generic_kernel");
}

}  // namespace

int launch_attention_generic(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st) {
  JPT_REQUIRE(a.D <= 32 * kMaxDPL, JPT_ERANGE, "flash_decode: head_dim %d > %d unsupported", a.D, 32 * kMaxDPL);
  return p.q_dtype == JPT_BF16 ? launch_generic_kv<__nv_bfloat16>(p, a, st) : launch_generic_kv<float>(p, a, st);
}

int launch_splitk_merge(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st) {
  const int64_t rows = (int64_t)a.B * a.Hkv * a.R;
  const int threads = a.D >= 128 ? 128 : (a.D > 32 ? 64 : 32);
  if (p.q_dtype == JPT_BF16) {
    splitk_merge_kernel<__nv_bfloat16><<<(unsigned)rows, threads, 0, st>>>(a);
  } else {
    splitk_merge_kernel<float><<<(unsigned)rows, threads, 0, st>>>(a);
  }
  return check_launch("splitk_merge_kernel");
}

static int auto_splits_generic(const jpt_attn_params& p, int R) {
  const int rcs = (R + kRowTile - 1) / kRowTile;
  const long base = (long)p.B * p.Hkv * rcs;
  int want = (int)((2L * 148 + base - 1) / base);
  int maxs = (p.S + 127) / 128;
  if (want > maxs) want = maxs;
  if (want > 64) want = 64;
  return want < 1 ? 1 : want;
}

static int resolve_splits(const jpt_attn_params& p, int R) {
  if (p.num_splits > 0) return p.num_splits;
  return auto_splits_generic(p, R);
}

static int validate(const jpt_attn_params& p) {
  JPT_REQUIRE(p.q && p.k && p.v && p.o, JPT_EINVAL, "flash_decode: null tensor");
  JPT_REQUIRE(p.q_dtype == JPT_BF16 || p.q_dtype == JPT_F32, JPT_EINVAL, "flash_decode: q dtype must be bf16 or f32");
  JPT_REQUIRE(p.B > 0 && p.Hq > 0 && p.Hkv > 0 && p.Tq > 0 && p.D > 0 && p.S > 0, JPT_EINVAL,
              "flash_decode: bad shape");
  JPT_REQUIRE(p.Hq % p.Hkv == 0, JPT_EINVAL, "flash_decode: Hq (%d) not a multiple of Hkv (%d)", p.Hq, p.Hkv);
  JPT_REQUIRE((p.k_scale == nullptr) == (p.v_scale == nullptr), JPT_EINVAL, "flash_decode: need both scales or none");
  if (p.mask_mode == JPT_MASK_LENGTH) JPT_REQUIRE(p.end, JPT_EINVAL, "flash_decode: JPT_MASK_LENGTH needs end");
  if (p.mask_mode == JPT_MASK_RING) JPT_REQUIRE(p.start && p.end, JPT_EINVAL, "flash_decode: JPT_MASK_RING needs start and end");
  if (p.mask_mode == JPT_MASK_ADD) JPT_REQUIRE(p.mask, JPT_EINVAL, "flash_decode: JPT_MASK_ADD needs mask");
  JPT_REQUIRE(p.mask_mode >= 0 && p.mask_mode <= 3, JPT_EINVAL, "flash_decode: bad mask mode");
  if (p.paged) {
    JPT_REQUIRE(p.page_table && p.page_size > 0 && p.max_pages > 0, JPT_EINVAL, "flash_decode: paged needs a page table");
    JPT_REQUIRE(p.S == p.page_size * p.max_pages, JPT_EINVAL, "flash_decode: paged S must be max_pages*page_size");
    JPT_REQUIRE(p.mask_mode == JPT_MASK_LENGTH, JPT_EINVAL, "flash_decode: paged caches use JPT_MASK_LENGTH");
  }
  return 0;
}

}  // namespace jpt

using namespace jpt;

extern "C" size_t jpt_flash_decode_workspace_bytes(const jpt_attn_params* p) {
  if (!p || validate(*p) != 0) return 0;
  const int R = (p->Hq / p->Hkv) * p->Tq;
  if (p->force_generic != 1 && attention_mma_eligible(*p)) return attention_mma_workspace_bytes(*p);
  const int ns = resolve_splits(*p, R);
  if (ns <= 1) return 0;
  const size_t rows = (size_t)p->B * p->Hkv * R;
  return kWorkspaceCounterBytes + rows * ns * (p->D + 2) * sizeof(float);
}

static AttnArgs attn_args_of(const jpt_attn_params& p) {
  AttnArgs a{};
  a.q = p.q; a.k = p.k; a.v = p.v; a.k_scale = p.k_scale; a.v_scale = p.v_scale;
  a.page_table = p.page_table; a.start = p.start; a.end = p.end; a.mask = p.mask;
  a.o = p.o; a.m = p.m; a.l = p.l;
  a.B = p.B; a.Hq = p.Hq; a.Hkv = p.Hkv; a.Tq = p.Tq; a.D = p.D; a.R = (p.Hq / p.Hkv) * p.Tq;
  a.S = p.S; a.paged = p.paged; a.page_size = p.page_size; a.max_pages = p.max_pages;
  a.kv_b = p.kv_b; a.kv_h = p.kv_h; a.kv_s = p.kv_s; a.kv_page = p.kv_page;
  a.sc_b = p.sc_b; a.sc_s = p.sc_s; a.mk_b = p.mk_b; a.mk_r = p.mk_r;
  a.mask_mode = p.mask_mode; a.scale_is_f32 = p.scale_dtype == JPT_F32;
  a.sm_scale = p.sm_scale;
  a.round_logits = p.logit_rounding != 0 && p.q_dtype == JPT_BF16;
  return a;
}

extern "C" int jpt_decode_update_attend(const jpt_attn_params* pp, const jpt_new_token* nt, void* stream) {
  JPT_REQUIRE(pp && nt, JPT_EINVAL, "decode_update_attend: null argument");
  const jpt_attn_params& p = *pp;
  if (int rc = validate(p)) return rc;
  JPT_REQUIRE(p.force_generic == 0 && attention_umma_eligible(p) && !p.paged, JPT_EINVAL,
              "decode_update_attend: needs a dense int8 cache with head_dim 128 and at most 8 grouped query rows");
  JPT_REQUIRE(p.mask_mode == JPT_MASK_LENGTH || p.mask_mode == JPT_MASK_RING, JPT_EINVAL,
              "decode_update_attend: the existing tokens are a length or a ring range");
  JPT_REQUIRE(p.k_scale && p.v_scale, JPT_EINVAL, "decode_update_attend: an int8 cache needs its scales");
  JPT_REQUIRE(nt->xk && nt->xv, JPT_EINVAL, "decode_update_attend: null new token");
  JPT_REQUIRE(aligned(nt->xk, 16) && aligned(nt->xv, 16), JPT_EALIGN, "decode_update_attend: the new token must be 16-byte aligned");
  JPT_REQUIRE(nt->in_dtype == JPT_BF16 || nt->in_dtype == JPT_F32, JPT_EINVAL,
              "decode_update_attend: the new token must be bf16 or f32");
  JPT_REQUIRE(p.scale_dtype == nt->in_dtype || !nt->write_cache, JPT_EINVAL,
              "decode_update_attend: the scale caches must have the new token's dtype");
  JPT_REQUIRE(nt->px != nullptr || exchange_bytes(p.B, 1) <= kWorkspaceExchangeBytes, JPT_EINVAL,
              "decode_update_attend: batch %d is more than the workspace's exchange area holds", p.B);
  JPT_REQUIRE(nt->pos == nullptr || nt->pos_count == 1 || nt->pos_count == p.B, JPT_EINVAL,
              "decode_update_attend: pos_count must be 1 or B");
  NewTokenArgs n{};
  n.x[0] = nt->xk; n.x[1] = nt->xv;
  n.quant[0] = nt->k_quant; n.quant[1] = nt->v_quant;
  n.scale_out[0] = nt->k_scale; n.scale_out[1] = nt->v_scale;
  n.pos = nt->pos; n.pos_count = nt->pos_count; n.pos_host = nt->pos_host;
  n.in_f32 = nt->in_dtype == JPT_F32;
  n.write_cache = nt->write_cache != 0;
  if (const jpt_peer_exchange* px = nt->px) {
    JPT_REQUIRE(px->world >= 1 && px->world <= 8 && px->rank >= 0 && px->rank < px->world, JPT_EINVAL,
                "decode_update_attend: rank %d of %d", px->rank, px->world);
    JPT_REQUIRE(px->batch == p.B, JPT_EINVAL, "decode_update_attend: exchange buffers are sized for batch %d, not %d",
                px->batch, p.B);
    JPT_REQUIRE(px->wait_cycles >= 0, JPT_EINVAL, "decode_update_attend: negative wait limit");
    for (int r = 0; r < px->world; ++r) {
      JPT_REQUIRE(px->buffers[r] && aligned(px->buffers[r], 8), JPT_EINVAL,
                  "decode_update_attend: buffer of rank %d missing or unaligned", r);
      n.px_slots[r] = reinterpret_cast<unsigned long long*>(static_cast<char*>(px->buffers[r]) + kExchangeStateBytes);
    }
    n.px_state = static_cast<unsigned*>(px->buffers[px->rank]);
    n.px_rank = px->rank;
    n.px_world = px->world;
    n.px_wait_cycles = px->wait_cycles;
  }
  AttnArgs a = attn_args_of(p);
  a.nsplit = 1;
  return launch_attention_umma(p, a, static_cast<cudaStream_t>(stream), &n);
}

extern "C" int jpt_flash_decode(const jpt_attn_params* pp, void* stream) {
  JPT_REQUIRE(pp, JPT_EINVAL, "flash_decode: null params");
  const jpt_attn_params& p = *pp;
  if (int rc = validate(p)) return rc;
  const int R = (p.Hq / p.Hkv) * p.Tq;
  const bool use_mma = p.force_generic != 1 && attention_mma_eligible(p);
  AttnArgs a = attn_args_of(p);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (use_mma) {
    a.nsplit = 1;
    if (p.force_generic != 2 && attention_umma_eligible(p)) return launch_attention_umma(p, a, st);
    return launch_attention_mma(p, a, st);
  }
  a.nsplit = resolve_splits(p, R);
  if (a.nsplit > 1) {
    const size_t rows = (size_t)p.B * p.Hkv * R;
    const size_t need = kWorkspaceCounterBytes + rows * a.nsplit * (p.D + 2) * sizeof(float);
    JPT_REQUIRE(p.workspace && p.workspace_bytes >= need, JPT_EWORKSPACE,
                "flash_decode: workspace of %zu bytes needed, %zu given", need, p.workspace_bytes);
    JPT_REQUIRE(aligned(p.workspace, 16), JPT_EALIGN, "flash_decode: workspace must be 16-byte aligned");
    // the split-K partials live behind the counter header, which stays untouched
    a.ws_o = reinterpret_cast<float*>(static_cast<char*>(p.workspace) + kWorkspaceCounterBytes);
    a.ws_m = a.ws_o + rows * a.nsplit * p.D;
    a.ws_l = a.ws_m + rows * a.nsplit;
  }
  if (int rc = launch_attention_generic(p, a, st)) return rc;
  if (a.nsplit > 1) return launch_splitk_merge(p, a, st);
  return 0;
}

extern "C" int jpt_flash_decode_workspace_init(void* workspace, size_t bytes, void* stream) {
  JPT_REQUIRE(workspace || bytes == 0, JPT_EINVAL, "flash_decode_workspace_init: null workspace");
  if (bytes == 0) return 0;
  cudaError_t e = cudaMemsetAsync(workspace, 0, bytes, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail((int)e, "flash_decode_workspace_init: %s", cudaGetErrorString(e));
  return 0;
}

// ---------------------------------------------------------------------------
// Attention without a caller-provided workspace.
//
// The scratch lives in this file-scope device array.  Every GPU whose context
// loads the library carries its own 16 MiB copy until the process exits; all
// calls on one GPU share it.
// ---------------------------------------------------------------------------
namespace {
constexpr size_t kStaticScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
constexpr int kMaxStaticDevices = 64;
std::atomic<void*> g_static_scratch_addr[kMaxStaticDevices];  // device address of the array, per device ordinal

// Address of the built-in scratch on the current device (looked up once per device).
int static_scratch_address(const char* who, void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail((int)e, "%s: cudaGetDevice: %s", who, cudaGetErrorString(e));
  JPT_REQUIRE(dev >= 0 && dev < kMaxStaticDevices, JPT_ERANGE, "%s: device ordinal %d unsupported", who, dev);
  void* ptr = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    // One-time set-up for the current device: `g_static_scratch` as written in
    // host code is only a handle, the address the kernels need comes from here.
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      return fail(e != cudaSuccess ? (int)e : JPT_EINVAL, "%s: cudaGetSymbolAddress: %s", who, cudaGetErrorString(e));
    }
    g_static_scratch_addr[dev].store(ptr, std::memory_order_release);  // every thread would store the same value
  }
  *out = ptr;
  return 0;
}
}  // namespace

extern "C" int jpt_flash_decode_static(const jpt_attn_params* pp, void* stream) {
  JPT_REQUIRE(pp, JPT_EINVAL, "flash_decode_static: null params");
  void* scratch = nullptr;
  if (int rc = static_scratch_address("flash_decode_static", &scratch)) return rc;
  jpt_attn_params p = *pp;
  p.workspace = scratch;
  p.workspace_bytes = kStaticScratchBytes;
  if (int rc = validate(p)) return rc;
  const size_t need = jpt_flash_decode_workspace_bytes(&p);
  JPT_REQUIRE(need <= kStaticScratchBytes, JPT_EWORKSPACE,
              "flash_decode_static: this shape needs %zu bytes of scratch, the built-in scratch holds %zu; "
              "use jpt_flash_decode with a workspace of your own",
              need, kStaticScratchBytes);
  if (need) {
    // The array keeps whatever the previous call left behind.  The arrival
    // counters at its start must read zero on entry; the status word behind
    // them is left alone so that a wait that gave up stays visible to
    // jpt_flash_decode_status(NULL, ...).
    const cudaError_t e = cudaMemsetAsync(p.workspace, 0, kWorkspaceStatusOffset, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail((int)e, "flash_decode_static: clearing the scratch header: %s", cudaGetErrorString(e));
  }
  return jpt_flash_decode(&p, stream);
}

extern "C" int jpt_flash_decode_status(const void* workspace, void* stream) {
  if (workspace == nullptr) {  // the scratch built into the library (jpt_flash_decode_static), current device
    void* scratch = nullptr;
    if (int rc = static_scratch_address("flash_decode_status", &scratch)) return rc;
    workspace = scratch;
  }
  int status = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(&status, static_cast<const char*>(workspace) + kWorkspaceStatusOffset, sizeof(int),
                                  cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail((int)e, "flash_decode_status: %s", cudaGetErrorString(e));
  return status;
}

extern "C" int jpt_merge_partials(const void* o1, const float* m1, const float* l1, const void* o2,
                                  const float* m2, const float* l2, int in_dtype, void* o, int out_dtype,
                                  int64_t rows, int D, void* stream) {
  JPT_REQUIRE(o1 && m1 && l1 && o2 && m2 && l2 && o, JPT_EINVAL, "merge_partials: null tensor");
  JPT_REQUIRE(rows >= 0 && D > 0, JPT_EINVAL, "merge_partials: bad shape");
  if (rows == 0) return 0;
  const int64_t total = rows * D;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define JPT_MERGE(TI, TO)                                                                     \
  merge_partials_kernel<TI, TO><<<blocks, 256, 0, st>>>(static_cast<const TI*>(o1), m1, l1,   \
                                                        static_cast<const TI*>(o2), m2, l2,   \
                                                        static_cast<TO*>(o), rows, D)
  if (in_dtype == JPT_BF16 && out_dtype == JPT_BF16) JPT_MERGE(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == JPT_BF16 && out_dtype == JPT_F32) JPT_MERGE(__nv_bfloat16, float);
  else if (in_dtype == JPT_F32 && out_dtype == JPT_F32) JPT_MERGE(float, float);
  else if (in_dtype == JPT_F32 && out_dtype == JPT_BF16) JPT_MERGE(float, __nv_bfloat16);
  else return fail(JPT_EINVAL, "merge_partials: bad dtypes");
#undef JPT_MERGE
  return check_launch("merge_partials_kernel");
}
