"""Oracle (test infrastructure): prefill -> decode-slot insert of the
reference engine (cache part and the per-slot bookkeeping rows), functional.

Follows jetstream_pt/engine.py:371-488 (`_insert_no_wrap`), 491-581
(`_insert_wrap`), 583-672 (paged insert).
"""

import numpy as np
import torch

from oracle.pages import insert_prefill_pages
from oracle.quant import quantize_insert


def insert_no_wrap(cache, prefix, slot, pos, layer=None, scaler=None, quantize=False):
  """engine.py:397-477: dynamic_update_slice of the prefix [1,H,L,D] at
  [slot, 0, pos, 0] (stacked: [layer, slot, 0, pos, 0]).  With `quantize` the
  prefix is first quantised per token over (heads, dim) -- reduce axes (-3,-1),
  engine.py:428-432 -- and the scales [1,1,L,1] are written the same way.
  Start indices are clamped like dynamic_update_slice does.
  Returns cache, or (cache, scaler) when quantising."""
  out = cache.clone()
  tgt = out if layer is None else out[layer]
  s = tgt.shape[2]
  length = prefix.shape[2]
  p = max(0, min(int(pos), s - length))
  if not quantize:
    tgt[slot, :, p:p + length, :] = prefix[0].to(tgt.dtype)
    return out
  codes, scales = quantize_insert(prefix, (-3, -1))
  tgt[slot, :, p:p + length, :] = codes[0]
  sout = scaler.clone()
  stgt = sout if layer is None else sout[layer]
  stgt[slot, :, p:p + length, :] = scales[0].to(stgt.dtype)
  return out, sout


def insert_wrap(cache, prefix, slot, start_insert, scaler=None, quantize=False):
  """engine.py:491-560: rows go to (arange(L) + start_insert) mod S of the
  slot.  The int8 variant transposes to [L,H,D] and quantises over axes (1,2),
  the same per-token groups as the no-wrap path."""
  out = cache.clone()
  s = cache.shape[2]
  length = prefix.shape[2]
  idx = (torch.arange(length) + int(start_insert) % s) % s
  if not quantize:
    out[slot][:, idx, :] = prefix[0].to(out.dtype)
    return out
  entry = prefix[0].permute(1, 0, 2)
  codes, scales = quantize_insert(entry, (1, 2))  # [L,H,D], [L,1,1]
  out[slot][:, idx, :] = codes.permute(1, 0, 2)
  sout = scaler.clone()
  sout[slot][:, idx, :] = scales.permute(1, 0, 2).to(sout.dtype)
  return out, sout


def insert_mask_row(cache_len, pos, current_pos, wrap):
  """The slot's mask row, engine.py:386-389 (no wrap: 0 on [pos, current_pos))
  and 506-521 (wrap: [start, cur) if cur > start else [start, S) U [0, cur))."""
  x = torch.arange(cache_len)
  if not wrap:
    cond = (x < current_pos) & (x >= pos)
  elif current_pos > pos:
    cond = (x >= pos) & (x < current_pos)
  else:
    cond = (x >= pos) | (x < current_pos)
  return torch.where(cond, 0.0, float("-inf"))


def engine_insert(ring_buffer, stacked, quantized, cache_len, current_position, seq_len, prefix_caches, caches,
                  scales, slot):
  """`PyTorchEngine.insert`, engine.py:627-648, with the two functions it
  dispatches to.  Ring buffer: the no-wrap path when 0 <= cur - seq_len and
  cur - seq_len + Lpad < S, else the modular one; left aligned: position 0.
  prefix_caches [(k, v)] per layer ([1,H,Lpad,D]); caches [(k, v)] per layer or
  one stacked pair; scales likewise (int8).  Returns (caches, scales, mask_row
  fp32 [S], start, input_pos, lens) for the slot."""
  lpad = prefix_caches[0][0].shape[2]
  if ring_buffer:
    start_insert = current_position - seq_len
    wrap = not (start_insert >= 0 and start_insert + lpad < cache_len)
    cur = current_position
  else:
    start_insert, wrap, cur = 0, False, seq_len
  pos = start_insert % cache_len if wrap else start_insert
  caches = [tuple(t.clone() for t in pair) for pair in caches]
  scales = [tuple(t.clone() for t in pair) for pair in (scales or [])]
  for i, new in enumerate(prefix_caches):
    j = 0 if stacked else i
    out_pair, out_scale = [], []
    for t in range(2):
      sc = scales[j][t] if quantized else None
      if wrap:
        r = insert_wrap(caches[j][t], new[t], slot, pos, scaler=sc, quantize=quantized)
      else:
        r = insert_no_wrap(caches[j][t], new[t], slot, pos, layer=i if stacked else None, scaler=sc,
                           quantize=quantized)
      if quantized:
        out_pair.append(r[0])
        out_scale.append(r[1])
      else:
        out_pair.append(r)
    caches[j] = tuple(out_pair)
    if quantized:
      scales[j] = tuple(out_scale)
  mask_row = insert_mask_row(cache_len, pos, cur, wrap)
  return caches, scales, mask_row, pos % cache_len, seq_len, 1


def insert_paged(cache, prefix, update_indexes, page_size):
  """engine.py:583-625 -> page_attention_manager.py:83-142."""
  return insert_prefill_pages(cache, prefix, update_indexes, page_size)


def insert_paged_int8(cache, scale_pool, prefix, update_indexes, page_size):
  """EXTENSION (the reference has no int8 paged cache, cache_manager.py:660-661,
  engine.py:614): quantise the L real tokens per token over (heads, dim) with
  the insert quantiser, then page-pad codes and scales separately with zeros, so
  page tails hold code 0 and scale 0.  cache int8 [H,P,ps,D]; scale_pool
  [1,P,ps,1]."""
  codes, scales = quantize_insert(prefix, (-3, -1))  # [1,H,L,D], [1,1,L,1]
  cache = insert_prefill_pages(cache, codes, update_indexes, page_size)
  scale_pool = insert_prefill_pages(scale_pool, scales, update_indexes, page_size)
  return cache, scale_pool
