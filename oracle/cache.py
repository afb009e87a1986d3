"""Oracle (test infrastructure): decode-time cache updates of the reference,
restated functionally (inputs are never modified; new tensors are returned).

Layouts: unstacked cache [B, H, S, D], stacked [NL, B, H, S, D]; int8 scalers
[B, 1, S, 1] / [NL, B, 1, S, 1]; paged pool [H, P, ps, D].
"""

import numpy as np
import torch

from oracle.quant import quantize_decode


def _pos_list(input_pos, batch):
  pos = torch.as_tensor(np.asarray(input_pos)).reshape(-1).to(torch.int64)
  if pos.numel() == 1:
    pos = pos.expand(batch)
  return pos


def append_ring(cache, new, pos):
  """`cache[..., pos, :] = new` with one shared position:
  jetstream_pt/cache_manager.py:254-262 (bf16) and 562-565 (int8 + scalers).
  cache [B,H,S,D], new [B,H,1,D] (or scalers [B,1,S,1] / [B,1,1,1])."""
  out = cache.clone()
  out[:, :, int(pos), :] = new[:, :, 0, :]
  return out


def append_per_slot(cache, new, pos, layer=None):
  """`cache[layer?, arange(B), :, pos_b, :] = new.squeeze(2)`:
  jetstream_pt/cache_manager.py:265-293 (bf16), 566-571 (int8)."""
  out = cache.clone()
  tgt = out if layer is None else out[layer]
  b = tgt.shape[0]
  pos = _pos_list(pos, b)
  tgt[torch.arange(b), :, pos, :] = new[:, :, 0, :]
  return out


def int8_update(cache_k, cache_v, k_scaler, v_scaler, xk, xv, input_pos, *,
                ring_buffer, lazy, layer=None):
  """`Int8KVCacheGenerate.update`, jetstream_pt/cache_manager.py:539-582.
  Returns the 8-tuple (cache_k, cache_v, k_quant, v_quant, k_scaler, v_scaler,
  kscale, vscale).  With `lazy` the caches come back unchanged (the rows are
  written later by `finalize_*`)."""
  kq, ks = quantize_decode(xk)
  vq, vs = quantize_decode(xv)
  if lazy:
    pass
  elif ring_buffer:
    p = int(np.asarray(input_pos).reshape(-1)[0])
    cache_k = append_ring(cache_k, kq, p)
    cache_v = append_ring(cache_v, vq, p)
    k_scaler = append_ring(k_scaler, ks, p)
    v_scaler = append_ring(v_scaler, vs, p)
  else:
    cache_k = append_per_slot(cache_k, kq, input_pos, layer)
    cache_v = append_per_slot(cache_v, vq, input_pos, layer)
    k_scaler = append_per_slot(k_scaler, ks, input_pos, layer)
    v_scaler = append_per_slot(v_scaler, vs, input_pos, layer)
  return cache_k, cache_v, kq, vq, k_scaler, v_scaler, ks, vs


def finalize_rows(cache, new_rows, input_pos):
  """Lazy finalize: `update_single_cache_line`,
  jetstream_pt/cache_manager.py:154-173 and 422-503: for every slot b one
  dynamic_update_slice of that slot's stashed row at position pos_b.
  cache [B,H,S,D] with new_rows [B,H,1,D], or stacked cache [NL,B,H,S,D] with
  new_rows [NL,B,H,1,D] (all layers written at the same pos_b).  Scalers use
  the same call with H == D == 1."""
  out = cache.clone()
  b = cache.shape[-4]
  pos = _pos_list(input_pos, b)
  s = cache.shape[-2]
  for bb in range(b):
    pp = int(pos[bb])
    pp = max(0, min(pp, s - 1))  # dynamic_update_slice clamps the start index
    if cache.ndim == 5:
      out[:, bb, :, pp, :] = new_rows[:, bb, :, 0, :]
    else:
      out[bb, :, pp, :] = new_rows[bb, :, 0, :]
  return out


def finalize_ring(cache, new_rows, pos):
  """Ring + lazy finalize, jetstream_pt/cache_manager.py:180-189 / 588-597
  (K and V only; the int8 variant leaves the scalers untouched)."""
  return append_ring(cache, new_rows, int(np.asarray(pos).reshape(-1)[0]))


def paged_append(cache, new, page_token_indices, page_size):
  """`PageKVCacheGenerate.update`, jetstream_pt/cache_manager.py:681-706.
  cache [H,P,ps,D]; new [B,H,1,D]; page_token_indices int [3, n_active] =
  (page ids, j*ps + token offset, batch slots).  The reference gathers the
  selected pages, writes one row in each and scatters the pages back; the net
  effect is one row write per active slot."""
  out = cache.clone()
  pti = np.asarray(page_token_indices)
  for j in range(pti.shape[1]):
    page, tok, slot = int(pti[0, j]), int(pti[1, j]) - j * page_size, int(pti[2, j])
    out[:, page, tok, :] = new[slot, :, 0, :]
  return out
