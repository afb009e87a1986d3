/*
 * C ABI of libjpt_b200.so: the KV-cache hot path of jetstream-pytorch as
 * hand-written CUDA for sm_100a.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host;
 *   - strides are in ELEMENTS of the tensor they belong to, the innermost
 *     (head_dim) axis is always contiguous;
 *   - `stream` is a cudaStream_t passed as void*;
 *   - every function returns 0 on success, a negative JPT_E* code for an
 *     argument error detected before anything is launched, or a positive
 *     cudaError_t; jpt_last_error_string() describes the last failure of the
 *     calling thread;
 *   - no function allocates device memory, synchronises the device or touches
 *     the host page cache: all of them are stream-ordered and may be captured
 *     in a CUDA graph, unless its comment says otherwise;
 *   - caches are updated IN PLACE (the reference's functional updates run with
 *     buffer donation, jetstream_pt/engine.py:112-121, so the two are
 *     observationally equal).
 *
 * Each entry point names the reference code it stands in for (paths relative to
 * the reference project root).
 */
#ifndef JPT_B200_H_
#define JPT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define JPT_BF16 0
#define JPT_F32 1
#define JPT_INT8 2

/* error codes (negative) */
#define JPT_EINVAL (-1)     /* bad size / null pointer / unsupported combination */
#define JPT_EALIGN (-2)     /* pointer or stride not aligned as the kernel needs */
#define JPT_EWORKSPACE (-3) /* workspace too small */
#define JPT_ERANGE (-4)     /* value outside the supported range */

const char* jpt_last_error_string(void);
int jpt_version(void);
/* Number of kernels this library has launched in this process so far. */
long long jpt_launch_count(void);

/* ------------------------------------------------------------------------- */
/* Decode-time update                                                        */
/* ------------------------------------------------------------------------- */

/*
 * Fused int8 quantise + append of one new token per slot, K and V in one
 * launch.  Replaces Int8KVCacheGenerate.quantize + .update,
 * jetstream_pt/cache_manager.py:532-582 (ring write 561-565, per-slot write
 * 566-571, lazy stash 544-560 when cache_k == NULL).
 *
 *   xk, xv        [B,H,1,D] contiguous, in_dtype (JPT_BF16 or JPT_F32)
 *   cache_k/v     int8, addressed cache[b*cs_b + h*cs_h + pos*cs_s + d]; NULL =
 *                 do not write the cache (lazy mode: only the stash outputs)
 *   k/v_scaler    scale cache in in_dtype, scaler[b*ss_b + pos*ss_s]; may be NULL
 *   k/v_quant     int8 [B,H,1,D] contiguous out (the quantised new token)
 *   k/v_scale     in_dtype [B] out (the new token's scale, shape [B,1,1,1])
 *   pos           int32 device array with pos_count entries (1 = one shared
 *                 position, B = one per slot) or NULL to use pos_host for all.
 *                 Negative positions count from the end; a position outside
 *                 [-S, S) writes nothing for that slot.
 * scale = amax(|x|) over (H,D) / 127; code = trunc(x / scale); every operation
 * is rounded to in_dtype as eager torch does.  An all-zero token gets scale 0
 * and codes 0.
 *
 * Sharded caches (KV heads split across GPUs): the scale spans ALL heads of a
 * token, so the update runs in two phases around a max-reduction over ranks.
 * amax_out != NULL: only write this rank's partial amax, float [2,B] (K row
 * then V row), and return.  amax_in != NULL: use amax_in[2,B] (the reduced
 * values) instead of the local maximum.  Both NULL: single-GPU behaviour.
 */
int jpt_kv_quant_append_dense(const void* xk, const void* xv, int in_dtype,
                              int8_t* cache_k, int8_t* cache_v, void* k_scaler,
                              void* v_scaler, int8_t* k_quant, int8_t* v_quant,
                              void* k_scale, void* v_scale, const int32_t* pos,
                              int pos_count, int pos_host, int B, int H, int S,
                              int D, int64_t cs_b, int64_t cs_h, int64_t cs_s,
                              int64_t ss_b, int64_t ss_s, const float* amax_in,
                              float* amax_out, void* stream);

/*
 * The same update for caches whose KV heads are split across the GPUs of one
 * node, with the max-reduction of the per-token amax done INSIDE the launch
 * over NVLink peer memory: every rank stores (launch number, partial amax) as
 * one 64-bit word per (K|V, slot) into every rank's exchange buffer and reads
 * what the others stored into its own; no collective call, no second kernel.
 * Replaces the reduction that GSPMD inserts for the sharded head axis of
 * jetstream_pt/cache_manager.py:532-535 (environment.py:225-242 gives the
 * sharding).  Codes and scales are bit-identical to the single-GPU ones (max
 * is order-independent).
 *
 * All ranks must call this the same number of times, in the same order, with
 * the same B.  A rank whose peer does not arrive within the wait limit (about
 * half a second unless px->wait_cycles says otherwise) goes on with the values
 * it has and raises the status of its buffer (jpt_peer_exchange_status);
 * nothing waits without a limit.
 *
 * Setting up (once per process, any host-side transport for the handles):
 *   bytes = jpt_peer_exchange_bytes(B, world);
 *   jpt_peer_exchange_alloc(bytes, &own);            zero-filled device memory
 *   jpt_peer_exchange_export(own, handle);           64 bytes, send to the peers
 *   jpt_peer_exchange_import(handle_of_r, &buf[r]);  for every other rank r
 *   px = { rank, world, B, { buf[0..world-1] }, 0 } with buf[rank] = own.
 * jpt_peer_exchange_release(buf[r]) and jpt_peer_exchange_free(own) undo it.
 */
typedef struct jpt_peer_exchange {
  int rank, world; /* 1 <= world <= 8 */
  int batch;       /* the B the buffers were sized for */
  void* buffers[8];
  /* How long a rank waits for a peer's word, in GPU clock cycles; 0 = the
   * default (about half a second).  After a rank gave up, its status stays 1
   * and the launch numbers of the ranks keep advancing together, so later
   * launches pair up again. */
  long long wait_cycles;
} jpt_peer_exchange;

size_t jpt_peer_exchange_bytes(int B, int world);
int jpt_peer_exchange_alloc(size_t bytes, void** ptr);
int jpt_peer_exchange_free(void* ptr);
int jpt_peer_exchange_export(void* ptr, void* handle64);
int jpt_peer_exchange_import(const void* handle64, void** peer_ptr);
int jpt_peer_exchange_release(void* peer_ptr);
/* 0: every wait of every launch so far was satisfied; 1: some launch gave up. */
int jpt_peer_exchange_status(const void* own_buffer, void* stream);

int jpt_kv_quant_append_dense_peers(const void* xk, const void* xv, int in_dtype,
                                    int8_t* cache_k, int8_t* cache_v, void* k_scaler,
                                    void* v_scaler, int8_t* k_quant, int8_t* v_quant,
                                    void* k_scale, void* v_scale, const int32_t* pos,
                                    int pos_count, int pos_host, int B, int H, int S,
                                    int D, int64_t cs_b, int64_t cs_h, int64_t cs_s,
                                    int64_t ss_b, int64_t ss_s,
                                    const jpt_peer_exchange* px, void* stream);

/*
 * Row scatter without quantisation, K and V in one launch:
 *   dst[l*ds_l + b*ds_b + h*ds_h + pos_b*ds_s + d] = src[((l*B + b)*H + h)*D + d]
 * Replaces KVCacheGenerate.update (jetstream_pt/cache_manager.py:227-293; NL=1)
 * and the lazy finalize of both cache classes (update_single_cache_line,
 * cache_manager.py:154-225, 422-503, 584-657; NL = stacked layers, and the
 * scalers with H = D = 1).  elem_bytes is 1, 2 or 4.  `clamp` = 1 clamps the
 * position to [0,S-1] (dynamic_update_slice semantics of finalize); 0 drops
 * out-of-range positions (scatter semantics of update).  src_v/dst_v may be
 * NULL to move a single tensor.
 */
int jpt_kv_scatter_rows(const void* src_k, const void* src_v, void* dst_k,
                        void* dst_v, int elem_bytes, const int32_t* pos,
                        int pos_count, int pos_host, int clamp, int NL, int B,
                        int H, int S, int D, int64_t ds_l, int64_t ds_b,
                        int64_t ds_h, int64_t ds_s, void* stream);

/*
 * Paged append: cache[h, page_j, tok_j, :] = x[slot_j, h, 0, :] for the n_active
 * entries of page_token_indices.  Replaces PageKVCacheGenerate.update,
 * jetstream_pt/cache_manager.py:681-706 (which gathers and re-scatters whole
 * pages to the same effect).
 *   pti           int32, three rows of pti_stride entries = (page ids, j*ps +
 *                 token offset, slots), as PageAttentionManager.
 *                 get_page_token_indices returns it (pti_stride = n_active) or as
 *                 jpt_page_token_indices writes it (pti_stride = B)
 *   n_active      entries to process; when n_active_dev is not NULL the count is
 *                 read from the device instead and n_active is only the upper
 *                 bound used to size the launch
 *   cache_k/v     [H,P,ps,D] contiguous, cache_dtype
 *   xk, xv        [B,H,1,D] contiguous, in_dtype
 * cache_dtype == in_dtype copies.  cache_dtype == JPT_INT8 with a bf16/f32
 * input quantises like jpt_kv_quant_append_dense and also writes the scale
 * pools [1,P,ps,1] (in_dtype); the reference has no int8 paged cache
 * (cache_manager.py:660-661) -- this mode is an extension.
 */
int jpt_kv_append_paged(const void* xk, const void* xv, int in_dtype,
                        void* cache_k, void* cache_v, int cache_dtype,
                        void* k_scale_pool, void* v_scale_pool,
                        const int32_t* pti, int64_t pti_stride, int n_active,
                        const int32_t* n_active_dev, int B, int H, int P,
                        int ps, int D, void* stream);

/*
 * Device-side page/token index computation for one decode step: the table walk
 * of PageAttentionManager.get_page_token_indices,
 * jetstream_pt/page_attention_manager.py:145-177, without the host round trip
 * of jetstream_pt/engine.py:739-744.  lens int32 [B] are the lengths BEFORE the
 * step; page_indices int32 [B,max_pages].  Writes pti int32 [3,B] compacted
 * over active slots (len > 0), n_active (int32 [1]) and new_lengths
 * (len + 1 for active slots, else 0).  Single block; B <= 1024.
 */
int jpt_page_token_indices(const int32_t* lens, const int32_t* page_indices,
                           int B, int max_pages, int ps, int32_t* pti,
                           int32_t* n_active, int32_t* new_lengths,
                           void* stream);

/* ------------------------------------------------------------------------- */
/* Prefill insert                                                            */
/* ------------------------------------------------------------------------- */

/*
 * Scatter a prefix's K and V into one decode slot of a dense cache, optionally
 * quantising on the way.  Replaces the cache part of PyTorchEngine._insert_no_wrap
 * and _insert_wrap, jetstream_pt/engine.py:371-488, 491-581, including
 * quantize_tensor(prefix, (-3,-1)) (jetstream_pt/quantize.py:24-75) for int8
 * caches.
 *   prefix_k/v    [NL][1,H,L,D]: element (l,h,t,d) at l*ps_l + h*ps_h + t*ps_t + d
 *   cache_k/v     element (l,slot,h,s,d) at l*cs_l + slot*cs_b + h*cs_h + s*cs_s + d
 *   k/v_scaler    (int8 caches) element (l,slot,s) at l*ss_l + slot*ss_b + s*ss_s
 *   wrap = 0      rows go to pos .. pos+L-1 with pos clamped to [0, S-L]
 *                 (dynamic_update_slice); wrap = 1: rows go to (pos + t) mod S.
 * cache_dtype JPT_INT8 with in_dtype bf16/f32 quantises per token over (H,D):
 * max = clamp(amax|x|, 1e-5); scale = max/127; code = clamp(round_half_even(
 * x * (1/scale)), -128, 127), every operation rounded to in_dtype.
 */
int jpt_prefill_insert_dense(const void* prefix_k, const void* prefix_v,
                             int in_dtype, void* cache_k, void* cache_v,
                             int cache_dtype, void* k_scaler, void* v_scaler,
                             int slot, int pos, int wrap, int NL, int H, int L,
                             int S, int D, int64_t ps_l, int64_t ps_h,
                             int64_t ps_t, int64_t cs_l, int64_t cs_b,
                             int64_t cs_h, int64_t cs_s, int64_t ss_l,
                             int64_t ss_b, int64_t ss_s, void* stream);

/*
 * Disaggregated serving: the prefix produced on a prefill GPU may be handed to
 * jpt_prefill_insert_dense / jpt_prefill_insert_paged of the decode GPU while it
 * still lies in the prefill GPU's memory (prefix_k / prefix_v are then peer
 * pointers; everything else belongs to the device the call is launched on).
 * The insert kernels read it over NVLink and write rows, codes and scales in
 * the cache's own format, so the transfer and the insert are one pass.
 * Replaces the prefill -> decode hand-over through host memory of
 * jetstream_pt/ray_worker.py:501-551 and jetstream_pt/ray_engine.py:119-127.
 * This call makes the peer's memory readable from `device` (idempotent).
 */
int jpt_enable_peer_access(int device, int peer);

/*
 * Scatter a prefix into pages: page i of the prefix goes to page
 * update_indexes[i]; the tail of the last page is written with zeros.
 * Replaces PageAttentionManager.insert_prefill_cache,
 * jetstream_pt/page_attention_manager.py:83-142 (driven by
 * jetstream_pt/engine.py:583-672).
 *   prefix_k/v    as above ([NL][1,H,L,D])
 *   cache_k/v     [NL][H,P,ps,D], layer stride cs_l, otherwise contiguous
 *   update_indexes int32 [n_pages], n_pages >= ceil(L/ps)
 * cache_dtype JPT_INT8 with bf16/f32 input (extension, see
 * jpt_kv_append_paged) quantises the L real tokens with the insert quantiser
 * and writes codes and scales (scale pools [NL][1,P,ps,1], layer stride ss_l);
 * padded tokens get code 0 and scale 0.
 */
int jpt_prefill_insert_paged(const void* prefix_k, const void* prefix_v,
                             int in_dtype, void* cache_k, void* cache_v,
                             int cache_dtype, void* k_scale_pool,
                             void* v_scale_pool, const int32_t* update_indexes,
                             int n_pages, int NL, int H, int L, int P, int ps,
                             int D, int64_t ps_l, int64_t ps_h, int64_t ps_t,
                             int64_t cs_l, int64_t ss_l, void* stream);

/*
 * The KV insert quantiser on its own: quantize_tensor(w, reduce_axis, 8,
 * symmetric=True, block_size=-1), jetstream_pt/quantize.py:24-75, for the two
 * layouts the insert path uses: w [1,H,L,D] reduced over (-3,-1) (token_major=0;
 * element (h,t,d) at h*L*D + t*D + d) and w [L,H,D] reduced over (1,2)
 * (token_major=1).  codes int8 in w's layout; scales in_dtype [L].
 */
int jpt_quantize_tokens(const void* w, int in_dtype, int token_major, int H,
                        int L, int D, int8_t* codes, void* scales,
                        void* stream);

/* ------------------------------------------------------------------------- */
/* Decode attention                                                          */
/* ------------------------------------------------------------------------- */

#define JPT_MASK_NONE 0   /* every position of the cache row is valid        */
#define JPT_MASK_LENGTH 1 /* valid = [0, end_b)            (ragged_mqa_reference) */
#define JPT_MASK_RING 2   /* valid = [start_b, end_b) or wrapped; start==end empty (ragged_mqa) */
#define JPT_MASK_ADD 3    /* additive mask values, -inf = masked (dense/flash_attention) */

typedef struct jpt_attn_params {
  /* query [B,Hq,Tq,D] contiguous; rows of one KV group (rep*Tq) are processed together */
  const void* q;
  int q_dtype; /* JPT_BF16 or JPT_F32; also the dtype of o */
  int B, Hq, Hkv, Tq, D;
  /* keys / values */
  const void* k;
  const void* v;
  int kv_dtype;              /* JPT_BF16, JPT_F32 or JPT_INT8 */
  int paged;                 /* 0: dense rows, 1: page pool */
  int S;                     /* dense: cache length; paged: max_pages*page_size */
  int64_t kv_b, kv_h, kv_s;  /* dense strides (elements) */
  int page_size;             /* paged: tokens per page */
  int64_t kv_page;           /* paged: elements between pages (ps*D), kv_h = P*ps*D */
  const int32_t* page_table; /* paged: [B,max_pages] */
  int max_pages;
  /* per-token scales (int8 caches), NULL = unquantised */
  const void* k_scale;
  const void* v_scale;
  int scale_dtype;       /* JPT_BF16 or JPT_F32 */
  int64_t sc_b, sc_s;    /* dense: scale[b*sc_b + s*sc_s]; paged: pool index page*ps + tok */
  /* validity */
  int mask_mode;
  const int32_t* start; /* [B], JPT_MASK_RING */
  const int32_t* end;   /* [B], JPT_MASK_LENGTH / RING; paged: lengths */
  const void* mask;     /* JPT_MASK_ADD: mask[b*mk_b + row*mk_r + s], q_dtype */
  int64_t mk_b, mk_r;
  float sm_scale;       /* logits = q.k * sm_scale (* k_scale) */
  /* outputs */
  void* o;              /* [B,Hq,Tq,D] q_dtype */
  float* m;             /* [B,Hq,Tq] running max of the logits, or NULL */
  float* l;             /* [B,Hq,Tq] softmax denominator (v scale not included), or NULL */
  /* scratch for split sequences: at least jpt_flash_decode_workspace_bytes(p) bytes,
   * 256-byte aligned, cleared once with jpt_flash_decode_workspace_init() */
  void* workspace;
  size_t workspace_bytes;
  int num_splits;       /* split-K factor; 0 = choose automatically */
  int force_generic;    /* testing: 1 = always the scalar kernel, 2 = the mma.sync kernel instead of the tcgen05 one */
  /* 1: round every logit to bf16 after each step of dense_attention's chain
   * (q.k, / sqrt(D), * k_scale, + mask), as the reference's bf16 tensors do
   * (jetstream_pt/attention_kernel.py:611-616); the softmax stays in fp32.
   * 0: fp32 logits (flash_attention, the ragged kernels, paged attention). */
  int logit_rounding;
} jpt_attn_params;

/*
 * Ragged flash-decode attention over a dense ring / left-aligned cache or a
 * page pool, with split-K and an in-kernel merge.  One entry point for
 *   ragged_mha / ragged_mqa_reference / ragged_mqa
 *     (jetstream_pt/attention_kernel.py:480-580, 255-466, 22-252),
 *   dense_attention and flash_attention at decode shapes (605-633, 636-710),
 *   call_paged_attention (789-808).
 * o = sum_s softmax(logits)_s * v_scale_s * V_s, m = max logit, l = sum
 * exp(logit - m); an empty row gives o = 0, m = -inf, l = 0.
 */
int jpt_flash_decode(const jpt_attn_params* p, void* stream);
size_t jpt_flash_decode_workspace_bytes(const jpt_attn_params* p);
/*
 * Zero-fills a workspace (stream-ordered memset).  Call it once after
 * allocating the buffer, and again after a launch that returned an error: the
 * kernel keeps per-sequence arrival counters at the start of the workspace that
 * it leaves at zero after every completed launch and expects at zero on entry.
 * One workspace may serve calls of any shape, but never two calls that can
 * overlap on the GPU.  (No counterpart in the reference.)
 */
int jpt_flash_decode_workspace_init(void* workspace, size_t bytes, void* stream);
/*
 * Health word of the attention kernels that used this workspace: 0, or a
 * positive code: 1 if a bounded wait inside a kernel ever gave up (the kernel
 * then returns early and its outputs are invalid), 2 for a misaligned shared
 * memory base, 3 if jpt_decode_update_attend met a sequence whose cache had no
 * row left for the new token.  Copies one int to the host and
 * SYNCHRONISES the stream: a diagnostic for tests, not for the step path.
 * workspace == NULL reads the word of the scratch built into the library (the
 * one jpt_flash_decode_static uses) on the current device.  The word is sticky:
 * it is only cleared by jpt_flash_decode_workspace_init (never, for the
 * built-in scratch).  (No counterpart in the reference.)
 */
int jpt_flash_decode_status(const void* workspace, void* stream);

/*
 * jpt_flash_decode for callers that cannot hand over a workspace because they
 * cannot allocate device memory at the point of the call: code running inside a
 * serving loop whose memory pool is fixed and fully handed out, a plugin host
 * that forbids allocation after start-up, a callback on a path where cudaMalloc
 * (which synchronises the device) must not run.  p->workspace and
 * p->workspace_bytes are ignored; the scratch is a 16 MiB array built into the
 * library, one per GPU that loads the library, held until the process exits.
 * This entry point has no counterpart in the reference.
 *
 *   - Shapes whose jpt_flash_decode_workspace_bytes() exceeds 16 MiB are rejected
 *     with JPT_EWORKSPACE; nothing is launched.
 *   - The first call on each device looks up the array's device address; make
 *     that first call outside any stream capture.
 *   - No cudaMalloc / cudaFree / allocating library routine is called, here or
 *     in anything this function calls.
 *   - All calls on a GPU share the one array and each call clears the arrival
 *     counters it relies on, so two calls that can overlap on the GPU (different
 *     streams without ordering, concurrent host threads) race.  Calls ordered on
 *     one stream are safe.
 */
int jpt_flash_decode_static(const jpt_attn_params* p, void* stream);

/*
 * One launch for a decode step's cache update AND attention: the new token of
 * every slot is quantised with the decode quantiser (as
 * jpt_kv_quant_append_dense does), written to the cache row / scale cache and
 * the stash outputs, and attended to together with the tokens already in the
 * cache.  Replaces the pair Int8KVCacheGenerate.update + ragged attention that
 * Int8KVAttentionKernel issues per layer (jetstream_pt/layers.py:676-706), and
 * with write_cache = 0 the lazy form of it (stash only, existing + new merged,
 * layers.py:708-718).
 *
 *   p        as for jpt_flash_decode; int8 dense cache, head_dim 128, at most 8
 *            grouped query rows, JPT_MASK_LENGTH or JPT_MASK_RING, scales
 *            given.  start / end describe the tokens ALREADY in the cache (the
 *            new token is not part of that range).  p->k, p->v, p->k_scale,
 *            p->v_scale are written at `pos` when write_cache is set.
 *   nt       the new token.  px = NULL: unsharded cache (the amax passes through
 *            the workspace); px != NULL: KV heads sharded over px->world GPUs,
 *            the amax is max-reduced over NVLink inside the launch exactly as
 *            jpt_kv_quant_append_dense_peers does, but the round trip is hidden
 *            under the attention over the existing tokens.  A launch of this
 *            function and a launch of jpt_kv_quant_append_dense_peers on the same
 *            exchange buffers both count as one step of the exchange.
 *            xk, xv must be 16-byte aligned.
 * The token is attended to as the LAST token of its sequence (the kernel
 * writes its codes into the last tile's rows in shared memory), so the
 * range must leave room for it: end - start < S (ring) / end < S (length).
 * A sequence that does not is attended to without the token and the
 * workspace's status word reads 3 (jpt_flash_decode_status).
 * Returns JPT_EINVAL for shapes the fused kernel does not take (use the two
 * separate calls then).  Codes, scales and cache contents are bit-identical to
 * the separate update; attention rows agree within rounding.
 */
typedef struct jpt_new_token {
  const void* xk;   /* [B,Hkv,1,D] contiguous, in_dtype */
  const void* xv;
  int in_dtype;     /* JPT_BF16 or JPT_F32: also the dtype of the scale caches and scale outputs */
  int write_cache;  /* 1: write codes and scale at pos; 0: only the stash outputs */
  int8_t* k_quant;  /* [B,Hkv,1,D] out, may be NULL */
  int8_t* v_quant;
  void* k_scale;    /* [B] out (in_dtype), may be NULL */
  void* v_scale;
  const int32_t* pos; /* as in jpt_kv_quant_append_dense */
  int pos_count;
  int pos_host;
  const jpt_peer_exchange* px;
} jpt_new_token;

int jpt_decode_update_attend(const jpt_attn_params* p, const jpt_new_token* nt, void* stream);

/*
 * Merge two softmax partials: g = max(m1,m2); o = (l1 e^{m1-g} o1 + l2 e^{m2-g}
 * o2) / (l1 e^{m1-g} + l2 e^{m2-g}).  Replaces the "attn_global" block of
 * AttentionKernel / Int8KVAttentionKernel, jetstream_pt/layers.py:539-550,
 * 708-718.  o1,o2 [rows,D] in_dtype; o [rows,D] out_dtype; m,l float [rows].
 */
int jpt_merge_partials(const void* o1, const float* m1, const float* l1,
                       const void* o2, const float* m2, const float* l2,
                       int in_dtype, void* o, int out_dtype, int64_t rows, int D,
                       void* stream);

/*
 * Weight-only int8 linear layer for decode batches (next to the KV path in a
 * decode step: the weights are the other stream of bytes).  Replaces
 * WeightOnlyPerChannelQuantizedLinear.forward with symmetric weights and
 * without activation quantisation, jetstream_pt/layers.py:141-166:
 *   y = bf16(bf16(x @ W^T) * w_scale)
 *   x        [M, K] bf16, K a multiple of 128, 16-byte aligned; made for decode
 *            batches: up to 128 rows stream the weights once, more rows are
 *            taken in blocks of 128 (each block streams the weights again)
 *   w        [N, K] int8 (one row per output channel), 16-byte aligned
 *   w_scale  [N] bf16
 *   y        [M, N] bf16 out
 *   workspace  jpt_w8a16_linear_workspace_bytes(M, N, K) bytes, 256-byte
 *            aligned; its first int is 0 after the call, or 1 if a bounded wait
 *            inside the kernel gave up (the output is then invalid)
 * The int8 weights go to the tensor core as they are (tcgen05 integer MMAs);
 * the bf16 activations are split into two int8 levels (exact to 2^-16 of a
 * row's amax), so the sums are exact integers.
 */
size_t jpt_w8a16_linear_workspace_bytes(int M, int N, int K);
int jpt_w8a16_linear(const void* x, const void* w, const void* w_scale, void* y,
                     int M, int N, int K, void* workspace,
                     size_t workspace_bytes, void* stream);

/*
 * The same layer in two steps, for activations that feed several layers (wq /
 * wk / wv after the attention norm, w1 / w3 after the ffn norm): the level
 * split once into a workspace (M <= 128 rows), then one GEMM per layer on the
 * levels it holds.  jpt_w8a16_linear(x, ...) equals jpt_w8a16_split_levels(x)
 * followed by jpt_w8a16_linear_from_levels(...), bit for bit.
 */
int jpt_w8a16_split_levels(const void* x, int M, int K, void* workspace,
                           size_t workspace_bytes, void* stream);
int jpt_w8a16_linear_from_levels(void* workspace, size_t workspace_bytes,
                                 const void* w, const void* w_scale, void* y,
                                 int M, int N, int K, void* stream);

/*
 * The two element-wise producers of a linear layer's activations in a decoder
 * block, each of which can leave the level split of its result in a workspace
 * (levels_workspace non-NULL, M <= 128) so that the layers behind it start at
 * their GEMM.  All tensors bf16, 16-byte aligned, K a multiple of 8 (of 128 with
 * levels).
 *   jpt_rmsnorm   RMSNorm.forward, jetstream_pt/layers.py:337-350, with a bf16
 *                 weight: y = bf16(bf16(x * rsqrt(mean(x^2) + eps)) * weight),
 *                 x, y [M, K], weight [K]; the mean and the product in fp32
 *   jpt_silu_mul  the gate of FeedForward.forward,
 *                 third_party/llama/model_exportable.py:84-86:
 *                 h = bf16(bf16(silu(a)) * b), a, b, h [M, K]
 */
int jpt_rmsnorm(const void* x, const void* weight, float eps, void* y, int M,
                int K, void* levels_workspace, size_t workspace_bytes,
                void* stream);
int jpt_silu_mul(const void* a, const void* b, void* h, int M, int K,
                 void* levels_workspace, size_t workspace_bytes, void* stream);

/*
 * The row-parallel form of the layer over the GPUs of one box: the input
 * features are sharded (rank r holds x[:, K_r] and w[:, K_r], as `wo` and `w2`
 * are in jetstream_pt/default_shardings/llama.yaml:10,20), and what GSPMD
 * inserts behind the reference's matmul, an all-reduce of the partial results,
 * happens inside the GEMM's epilogue: every CTA stores the fp32 sums of its
 * rows into its rank's own buffer, tells the other ranks with the number of
 * the launch (a small peer store behind a system-scope fence), waits (bounded)
 * for the same CTA of the other ranks, fetches their sums over NVLink (plain
 * 16-byte peer loads) and adds the partials in the order of the ranks; then the
 * two bf16 roundings and the channel scale, as on one GPU.  N must be a
 * multiple of 4.  Every rank gets the
 * whole y.  M <= 128.  All ranks make the same sequence of calls with the same
 * shapes; the calls are numbered on the device (a captured graph of them can be
 * replayed), and two consecutive calls use the two halves of the buffers.
 * Setting up: every rank allocates jpt_w8a16_tp_buffer_bytes(N_max, world)
 * zero-filled bytes (jpt_peer_exchange_alloc), exports the handle and imports
 * the others' (jpt_peer_exchange_export / _import), as for jpt_peer_exchange.
 * jpt_w8a16_tp_status: 0, or 1 after a launch gave up on a peer (its y is then
 * the sum of what had arrived).
 */
typedef struct jpt_tp_sum {
  int rank, world;       /* 1 <= world <= 8 */
  void* buffers[8];      /* buffers[rank] = own */
  size_t buffer_bytes;   /* size of each */
  long long wait_cycles; /* 0 = the default (about half a second) */
} jpt_tp_sum;
size_t jpt_w8a16_tp_buffer_bytes(int N, int world);
int jpt_w8a16_linear_tp(const void* x, const void* w, const void* w_scale, void* y,
                        int M, int N, int K, void* workspace, size_t workspace_bytes,
                        const jpt_tp_sum* tp, void* stream);
int jpt_w8a16_tp_status(const jpt_tp_sum* tp, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* JPT_B200_H_ */
