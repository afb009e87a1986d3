"""Prefill -> decode-slot insert: the cache part of the reference engine's
`_insert_no_wrap`, `_insert_wrap`, `insert` and
`insert_page_attention_with_reservation` (jetstream_pt/engine.py:371-672),
plus the per-slot bookkeeping rows (mask, start, input_pos, lens) those
functions write.  Caches are written in place.
"""

import torch

from jetstream_pytorch_b200 import _lib


_peer_enabled = set()


def prefix_on_peer(prefix, cache_device):
  """Disaggregated serving (the reference hands the prefix from the prefill engine to the decode
  engine through host memory, ray_worker.py:501-551): a prefix that lies on ANOTHER GPU of the box
  is inserted as it is.  The insert kernels of the cache's GPU read it over NVLink and write rows,
  codes and scales in the cache's format, so transfer and insert are one pass.  This makes the
  prefix's memory readable from `cache_device` (once per pair of devices) and orders the cache
  device's stream after the work queued so far on the prefix's device."""
  src, dst = prefix.device, torch.device(cache_device)
  if src == dst:
    return
  if src.type != "cuda" or dst.type != "cuda":
    raise ValueError(f"prefix on {src}, cache on {dst}: both must be GPUs of one box")
  if (dst.index, src.index) not in _peer_enabled:
    _lib.check(_lib.lib().jpt_enable_peer_access(dst.index, src.index))
    _peer_enabled.add((dst.index, src.index))
  done = torch.cuda.Event()
  done.record(torch.cuda.current_stream(src))
  torch.cuda.current_stream(dst).wait_event(done)


def _prefix_strides(pk, pv):
  if pk.stride(-1) != 1 or pv.stride() != pk.stride():
    pk, pv = pk.contiguous(), pv.contiguous()
  return pk, pv


def insert_dense(prefix_k, prefix_v, cache_k, cache_v, slot, pos, *, wrap=False, layer=None, k_scaler=None,
                 v_scaler=None):
  """Write one layer's prefix [1,H,L,D] into slot `slot` of a dense cache
  [B,H,S,D] (or layer `layer` of a stacked one).  No wrap: rows pos..pos+L-1
  with the start clamped like dynamic_update_slice (engine.py:397-405, 434-450);
  wrap: rows (pos + t) mod S (engine.py:534-539, 554-557).  An int8 cache with
  a bf16/fp32 prefix quantises per token over (heads, dim) on the way and
  writes the scales [.,1,S,1] (engine.py:427-432, 545-553)."""
  if layer is not None:
    cache_k, cache_v = cache_k[layer], cache_v[layer]
    if k_scaler is not None:
      k_scaler, v_scaler = k_scaler[layer], v_scaler[layer]
  pk, pv = _prefix_strides(prefix_k, prefix_v)
  if pk.device != cache_k.device:  # a prefix still on the prefill GPU: read over NVLink by this GPU's kernel
    prefix_on_peer(pk, cache_k.device)
  _, h, l, d = pk.shape
  b, hc, s, dc = cache_k.shape
  if (hc, dc) != (h, d):
    raise ValueError(f"prefix heads/dim {(h, d)} do not match the cache {(hc, dc)}")
  if not 0 <= slot < b:
    raise ValueError(f"slot {slot} outside [0, {b})")
  quant = cache_k.dtype == torch.int8 and pk.dtype != torch.int8
  if quant and k_scaler is None:
    raise ValueError("an int8 cache needs its scalers")
  ss = (0, 0)
  if k_scaler is not None:
    ss = (k_scaler.stride(0), k_scaler.stride(2))
  with torch.cuda.device(cache_k.device):  # the launch belongs to the cache's GPU
    _lib.check(_lib.lib().jpt_prefill_insert_dense(
        _lib.ptr(pk), _lib.ptr(pv), _lib.dt(pk), _lib.ptr(cache_k), _lib.ptr(cache_v), _lib.dt(cache_k),
        _lib.ptr(k_scaler), _lib.ptr(v_scaler), slot, int(pos), int(wrap), 1, h, l, s, d, 0, pk.stride(1),
        pk.stride(2), 0, cache_k.stride(0), cache_k.stride(1), cache_k.stride(2), 0, ss[0], ss[1], _lib.stream()))


def insert_mask_row(cache_len, pos, current_pos, wrap, device, dtype=torch.float32):
  """The mask row of the slot: 0 on valid positions, -inf elsewhere
  (engine.py:386-389 no wrap; 506-521 wrap)."""
  x = torch.arange(cache_len, device=device)
  if not wrap:
    cond = (x < current_pos) & (x >= pos)
  elif current_pos > pos:
    cond = (x >= pos) & (x < current_pos)
  else:
    cond = (x >= pos) | (x < current_pos)
  return torch.where(cond, 0.0, float("-inf")).to(dtype)


def insert(env, prefix_caches, seq_len, caches, cache_scales, slot, current_position, *, mask=None, start=None,
           input_pos=None, lens=None):
  """`PyTorchEngine.insert`, engine.py:627-648, for the dense layouts.

  prefix_caches: [(k, v)] per layer, each [1,H,Lpad,D]; caches: [(k, v)] per
  layer ([B,H,S,D]) or one stacked pair ([NL,B,H,S,D]); cache_scales likewise
  for int8.  Ring buffer: no wrap when 0 <= cur - seq_len and cur - seq_len +
  Lpad < S, else modular positions; left aligned: always position 0.
  Updates (in place, when given) mask[slot], start[slot], input_pos[slot],
  lens[slot] exactly as engine.py:386-395 / 506-524 do."""
  s = env.cache_len
  lpad = prefix_caches[0][0].shape[2]
  if env.ring_buffer:
    start_insert = current_position - seq_len
    wrap = not (start_insert >= 0 and start_insert + lpad < s)
    pos = start_insert % s if wrap else start_insert
    cur = current_position
  else:
    wrap, pos, cur = False, 0, seq_len
  stacked = env.generate_cache_stacked
  for i, (pk, pv) in enumerate(prefix_caches):
    ck, cv = caches[0] if stacked else caches[i]
    ks = vs = None
    if cache_scales:
      ks, vs = cache_scales[0] if stacked else cache_scales[i]
    insert_dense(pk, pv, ck, cv, slot, pos, wrap=wrap, layer=i if stacked else None, k_scaler=ks, v_scaler=vs)
  if mask is not None:
    mask[slot] = insert_mask_row(s, pos, cur, wrap, mask.device, mask.dtype)
  if start is not None:
    start[slot] = pos % s
  if input_pos is not None:
    input_pos[slot] = seq_len
  if lens is not None:
    lens[slot] = 1
  return caches, cache_scales


def insert_page_attention_with_reservation(page_attention_manager, prefix_caches, seq_len, caches, slot,
                                           cache_scales=None):
  """engine.py:650-672 -> 583-625: reserve ceil(seq_len/ps) pages for the slot
  on the host, then scatter the prefix into them (zero tail on the last page).
  Raises queue.Empty when the pool has too few free pages."""
  num_pages, update_indexes = page_attention_manager.reserve_pages_insert(slot, seq_len)
  page_attention_manager.insert_prefill_cache(prefix_caches, caches, update_indexes, None, None,
                                              decode_scales=cache_scales)
  return caches
