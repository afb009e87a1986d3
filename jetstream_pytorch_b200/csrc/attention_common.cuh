// Pieces shared by the decode-attention kernels: the per-sequence valid range,
// token addressing for dense and paged caches, and the split-K scratch layout.
#pragma once

#include "common.cuh"

namespace jpt {

// Device-side view of jpt_attn_params with the derived sizes added.
struct AttnArgs {
  const void* q;
  const void* k;
  const void* v;
  const void* k_scale;
  const void* v_scale;
  const int32_t* page_table;
  const int32_t* start;
  const int32_t* end;
  const void* mask;
  void* o;
  float* m;
  float* l;
  float* ws_o;  // [rows_total, nsplit, D] unnormalised partial outputs
  float* ws_m;  // [rows_total, nsplit]
  float* ws_l;  // [rows_total, nsplit]
  int B, Hq, Hkv, Tq, D, R;  // R = (Hq/Hkv)*Tq rows per KV head
  int S, paged, page_size, max_pages;
  int64_t kv_b, kv_h, kv_s, kv_page;
  int64_t sc_b, sc_s;
  int64_t mk_b, mk_r;
  int mask_mode, scale_is_f32;
  int nsplit;
  float sm_scale;
  int round_logits;  // dense_attention with bf16 tensors: every step of the logit chain is rounded to bf16
};

// dense_attention's logit chain on bf16 tensors (jetstream_pt/attention_kernel.py:611-616): the dot
// product, the division by sqrt(D), the product with the K scale and the sum with the mask are
// separate bf16 tensor operations there, each rounding its result.  `dot` is the fp32 dot product of
// the unscaled query row and the K row, `ks` the K scale (1 when unquantised), `mask_value` the
// additive mask entry (0 when there is none).
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float rounded_logit(float dot, float sqrt_d, float ks, bool quantised, float mask_value) {
  float s = bf16_round(dot);
  s = bf16_round(__fdiv_rn(s, sqrt_d));
  if (quantised) s = bf16_round(s * ks);
  return bf16_round(s + mask_value);
}

// Valid range of one sequence in "logical" token order: logical token j
// (0 <= j < n) lives at physical position (first + j) mod S.
struct SeqRange {
  int n, first;
};

__device__ __forceinline__ SeqRange seq_range(const AttnArgs& a, int b) {
  SeqRange r;
  r.first = 0;
  if (a.mask_mode == JPT_MASK_LENGTH) {
    int e = a.end[b];
    r.n = e < 0 ? 0 : (e > a.S ? a.S : e);
  } else if (a.mask_mode == JPT_MASK_RING) {
    int st = a.start[b], en = a.end[b];
    st = st < 0 ? 0 : (st >= a.S ? a.S - 1 : st);
    en = en < 0 ? 0 : (en > a.S ? a.S : en);
    r.first = st;
    r.n = st == en ? 0 : (st < en ? en - st : a.S - st + en);
  } else {
    r.n = a.S;
  }
  return r;
}

__device__ __forceinline__ int physical_pos(const AttnArgs& a, const SeqRange& r, int j) {
  int p = r.first + j;
  return p >= a.S ? p - a.S : p;
}

// Element offset of the K/V row of (b, kv head h, physical position p), and
// the index of its scale.  Returns false when the page id is out of range.
__device__ __forceinline__ int64_t kv_row_offset(const AttnArgs& a, int b, int h, int p, int64_t* scale_idx) {
  if (a.paged) {
    const int page = a.page_table[(int64_t)b * a.max_pages + p / a.page_size];
    const int tok = p % a.page_size;
    *scale_idx = (int64_t)page * a.page_size + tok;
    return (int64_t)h * a.kv_h + (int64_t)page * a.kv_page + (int64_t)tok * a.D;
  }
  *scale_idx = (int64_t)b * a.sc_b + (int64_t)p * a.sc_s;
  return (int64_t)b * a.kv_b + (int64_t)h * a.kv_h + (int64_t)p * a.kv_s;
}

__device__ __forceinline__ float load_scale(const void* base, int64_t idx, int is_f32) {
  return is_f32 ? static_cast<const float*>(base)[idx]
                : __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
}

// Every workspace starts with this many bytes of per-segment arrival counters
// that must stay zero between launches; no kernel puts anything else there.
// header: 192 KiB of counters, then the one-GPU exchange area of the fused decode step, then one status
// word in the last 256 bytes.  Everything whose meaning outlives a launch lives here, at offsets that do
// not depend on the shape, because one workspace serves calls of any shape (whose partials would
// otherwise land on another shape's state).
constexpr size_t kWorkspaceCounterBytes = 256 * 1024;
constexpr size_t kWorkspaceStatusOffset = kWorkspaceCounterBytes - 256;
constexpr size_t kWorkspaceExchangeOffset = 192 * 1024;
constexpr size_t kWorkspaceExchangeBytes = kWorkspaceStatusOffset - kWorkspaceExchangeOffset;
constexpr size_t kWorkspaceMaxSegments = kWorkspaceExchangeOffset / sizeof(unsigned);  // (sequence, head) pairs

// The new token of a decode step, handed to the attention launch itself
// (jpt_decode_update_attend): quantised with the decode quantiser, written to
// the cache row and / or the stash outputs, and attended to together with the
// existing tokens.  The per-token amax over all heads travels through exchange
// slots: one 64-bit word (launch number << 32 | amax bits) per (K|V, slot) and
// writer rank, in the buffers of a jpt_peer_exchange or (one GPU) in the
// workspace.
struct NewTokenArgs {
  const void* x[2];        // xk, xv [B,Hkv,1,D]
  int8_t* quant[2];        // [B,Hkv,1,D] out, may be null
  void* scale_out[2];      // [B] out (input dtype), may be null
  const int32_t* pos;      // where the token is written
  int pos_count, pos_host;
  unsigned long long* px_slots[8];  // slot area of each rank's exchange buffer (index = rank)
  unsigned* px_state;               // this rank's {launches done, CTAs done, gave up}
  int px_rank, px_world;
  long long px_wait_cycles;
  int enabled, in_f32, write_cache;
};

// Host-side launchers implemented by the individual kernels.
int launch_attention_generic(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st);
bool attention_mma_eligible(const jpt_attn_params& p);
size_t attention_mma_workspace_bytes(const jpt_attn_params& p);
// Launches the persistent kernel and its merge (and the mask pre-pass when the
// mask is additive); uses p.workspace for its scratch.
int launch_attention_mma(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st);
// int8 caches with up to 8 grouped query rows: the tcgen05 kernel.  Its scratch
// fits in attention_mma_workspace_bytes().
bool attention_umma_eligible(const jpt_attn_params& p);
int launch_attention_umma(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st, const NewTokenArgs* nt = nullptr);
int launch_splitk_merge(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st);

}  // namespace jpt
