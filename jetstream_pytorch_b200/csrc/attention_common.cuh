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
};

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
constexpr size_t kWorkspaceCounterBytes = 256 * 1024;  // header: counters, then one status word in its last 256 bytes
constexpr size_t kWorkspaceStatusOffset = kWorkspaceCounterBytes - 256;
constexpr size_t kWorkspaceMaxSegments = kWorkspaceStatusOffset / sizeof(unsigned);  // (sequence, head) pairs

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
int launch_attention_umma(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st);
int launch_splitk_merge(const jpt_attn_params& p, const AttnArgs& a, cudaStream_t st);

}  // namespace jpt
