"""Page manager with the reference's API (jetstream_pt/page_attention_manager.py):
a host-side FIFO free list and page table, and the device-side prefill insert
and page-table gather.

Host state keeps the reference's observable conventions: the free list starts
as 0..P-1 in order, `page_indices` is int32 [B, max_pages] filled with the
sentinel P-1, `lengths` is int32 [B].
"""

import queue
from typing import List, Tuple

import numpy as np
import torch

from jetstream_pytorch_b200 import _lib


def _layer_strides(prefill_caches, decode_caches, decode_scales):
  """(prefix, pool, scale-pool) layer strides in elements when every layer's
  tensors are same-shaped views at a constant address step (so that one launch
  can serve all layers), else None."""
  n = len(prefill_caches)
  if n < 2 or len(decode_caches) != n or (decode_scales is not None and len(decode_scales) != n):
    return None

  def step(tensors):
    t0 = tensors[0]
    if not t0.is_cuda:
      return None
    for t in tensors:
      if t.shape != t0.shape or t.dtype != t0.dtype or t.stride() != t0.stride():
        return None
    d = tensors[1].data_ptr() - t0.data_ptr()
    if d <= 0 or d % t0.element_size():
      return None
    for i, t in enumerate(tensors):
      if t.data_ptr() - t0.data_ptr() != i * d:
        return None
    return d // t0.element_size()

  pk = [c[0] for c in prefill_caches]
  pv = [c[1] for c in prefill_caches]
  ck = [c[0] for c in decode_caches]
  cv = [c[1] for c in decode_caches]
  if pk[0].stride(-1) != 1 or pv[0].stride() != pk[0].stride() or not ck[0].is_contiguous() or not cv[0].is_contiguous():
    return None
  sp, sv, sc, scv = step(pk), step(pv), step(ck), step(cv)
  if sp is None or sp != sv or sc is None or sc != scv:
    return None
  ss = 0
  if decode_scales is not None:
    ks = [c[0] for c in decode_scales]
    vs = [c[1] for c in decode_scales]
    if ks[0] is None:
      return None
    ss, ssv = step(ks), step(vs)
    if ss is None or ss != ssv:
      return None
  return sp, sc, ss


class PageAttentionManager:
  """Manages page blocks: reserve pages for prefill insert and decode, hand the
  page/token indices of a decode step to the cache, move prefill caches into
  pages, free a finished slot's pages."""

  def __init__(self, batch_size: int, paged_attention_total_num_pages: int, paged_attention_page_size: int,
               max_pages_per_sequence: int, free_page_order=None):
    """page_attention_manager.py:21-39.  `free_page_order` (an iterable of page
    ids) replaces the default 0..P-1 initial order of the free list."""
    self.unused_pages = queue.Queue()
    self.batch_size = batch_size
    self.total_num_pages = paged_attention_total_num_pages
    self.page_indices = np.full((batch_size, max_pages_per_sequence), paged_attention_total_num_pages - 1,
                                dtype=np.int32)
    self.lengths = np.zeros(batch_size, dtype=np.int32)
    self.paged_attention_page_size = paged_attention_page_size
    self.max_pages_per_sequence = max_pages_per_sequence
    order = range(paged_attention_total_num_pages) if free_page_order is None else free_page_order
    for i in order:
      self.unused_pages.put(int(i), block=False)

  # -- host bookkeeping -----------------------------------------------------

  def reserve_pages_insert(self, slot: int, seq_len: int):
    """page_attention_manager.py:42-52.  Raises queue.Empty when the pool runs
    dry (pages popped before the failure stay popped, as in the reference)."""
    self.lengths[slot] = seq_len
    ps = self.paged_attention_page_size
    num_pages = (seq_len + ps - 1) // ps
    if num_pages > self.max_pages_per_sequence:
      raise ValueError(f"{seq_len} tokens need {num_pages} pages, more than max_pages_per_sequence")
    indices = [self.unused_pages.get(block=False) for _ in range(num_pages)]
    self.page_indices[slot, :num_pages] = indices
    return num_pages, self.page_indices[slot, :num_pages]

  def reserve_pages_decode(self, slot: int, seq_len: int):
    """page_attention_manager.py:55-59."""
    ps = self.paged_attention_page_size
    if seq_len > 0 and seq_len % ps == 0:
      index = self.unused_pages.get(block=False)
      self.page_indices[slot, seq_len // ps] = index

  def fill_new_pages(self, lens):
    """page_attention_manager.py:62-64."""
    for slot in range(self.batch_size):
      self.reserve_pages_decode(slot, int(lens[slot]))

  def get_page_token_indices(self, lens):
    """page_attention_manager.py:145-177: int array [3, n_active] of (page id,
    j*ps + token offset, slot) for every slot with len > 0; `lens` are the
    lengths before this step, `self.lengths` becomes len + 1 for those slots."""
    lens = np.asarray(lens)
    ps = self.paged_attention_page_size
    active = np.nonzero(lens > 0)[0]
    l_act = lens[active]
    pages = self.page_indices[active, l_act // ps]
    toks = np.arange(active.size) * ps + l_act % ps
    self.lengths = np.where(lens == 0, 0, lens + 1).astype(np.int32)
    return np.stack((pages.astype(np.int64), toks.astype(np.int64), active.astype(np.int64)))

  def free_pages_resource(self, slot):
    """Return a slot's pages to the tail of the free list in table order,
    reset its table row to the sentinel and its length to zero.

    The reference's method of this name (page_attention_manager.py:214-222) is
    never called and cannot run (it uses a jax-only `.at` on a numpy array and
    looks for negative ids in a table whose sentinel is P-1); these semantics
    are this package's own."""
    ps = self.paged_attention_page_size
    n = (int(self.lengths[slot]) + ps - 1) // ps
    for i in range(n):
      self.unused_pages.put(int(self.page_indices[slot, i]), block=False)
    self.page_indices[slot, :] = self.total_num_pages - 1
    self.lengths[slot] = 0

  # -- device side ------------------------------------------------------------

  def device_tables(self, device):
    """(page_indices int32 [B,max_pages], lengths int32 [B]) copied to `device`
    (pinned staging, asynchronous on the current stream)."""
    pi = torch.from_numpy(np.ascontiguousarray(self.page_indices)).pin_memory().to(device, non_blocking=True)
    ln = torch.from_numpy(np.ascontiguousarray(self.lengths.astype(np.int32))).pin_memory().to(
        device, non_blocking=True)
    return pi, ln

  def get_page_token_indices_device(self, lens_dev, page_indices_dev):
    """The table walk of get_page_token_indices on the device, without the host
    round trip of jetstream_pt/engine.py:739-744.  Returns (pti int32 [3,B] with
    rows compacted over active slots, n_active int32 [1], new_lengths int32
    [B]).  The caller remains responsible for page reservation
    (`fill_new_pages`) on the host."""
    b = self.batch_size
    dev = lens_dev.device
    pti = torch.zeros((3, b), dtype=torch.int32, device=dev)
    n_active = torch.zeros((1,), dtype=torch.int32, device=dev)
    new_lengths = torch.empty((b,), dtype=torch.int32, device=dev)
    _lib.check(_lib.lib().jpt_page_token_indices(
        _lib.ptr(lens_dev), _lib.ptr(page_indices_dev), b, self.max_pages_per_sequence,
        self.paged_attention_page_size, _lib.ptr(pti), _lib.ptr(n_active), _lib.ptr(new_lengths), _lib.stream()))
    return pti, n_active, new_lengths

  def prefill_cache_padding(self, caches, seq_len: int, num_pages: int):
    """page_attention_manager.py:67-81 (zero-pad the sequence axis to whole pages)."""
    pad_width = num_pages * self.paged_attention_page_size - seq_len
    if pad_width == 0:
      return caches
    return [(self.pad_sequences(k, pad_width), self.pad_sequences(v, pad_width)) for k, v in caches]

  def pad_sequences(self, array, pad_width=10):
    """page_attention_manager.py:203-211."""
    return torch.nn.functional.pad(array, (0, 0, 0, pad_width))

  def insert_prefill_cache(self, prefill_caches: List[Tuple[torch.Tensor, torch.Tensor]],
                           decode_caches: List[Tuple[torch.Tensor, torch.Tensor]], update_indexes, tep_kv=None,
                           sharding=None, decode_scales=None):
    """Scatter each layer's prefix [1,H,L,D] into the pages `update_indexes` of
    that layer's pools [H,P,ps,D]; the tail of the last page is zero-filled
    (page_attention_manager.py:83-142).  `tep_kv` (the reference's zero staging
    buffer) and `sharding` are accepted and unused.  Pools are written in place
    and returned.  With int8 pools, `decode_scales` [(k_scale_pool,
    v_scale_pool)] per layer receives the per-token scales (extension)."""
    dev = decode_caches[0][0].device
    upd = _lib.as_i32(update_indexes, dev).contiguous()
    n_pages = upd.numel()
    if prefill_caches[0][0].device != dev:
      # a prefix still on the prefill GPU (disaggregated serving): this GPU's kernel reads it over NVLink
      from jetstream_pytorch_b200.insert import prefix_on_peer
      prefix_on_peer(prefill_caches[0][0], dev)  # (one device pair, one ordering point for all layers)
      with torch.cuda.device(dev):
        return self._insert_prefill_cache_here(prefill_caches, decode_caches, upd, n_pages, decode_scales)
    return self._insert_prefill_cache_here(prefill_caches, decode_caches, upd, n_pages, decode_scales)

  def _insert_prefill_cache_here(self, prefill_caches, decode_caches, upd, n_pages, decode_scales):
    stacked = _layer_strides(prefill_caches, decode_caches, decode_scales)
    if stacked is not None:
      # the layers lie at a constant stride (views of stacked tensors): one launch for all of them
      ps_l, cs_l, ss_l = stacked
      (pk, pv), (ck, cv) = prefill_caches[0], decode_caches[0]
      h, p, ps, d = ck.shape
      ks, vs = decode_scales[0] if decode_scales is not None else (None, None)
      _lib.check(_lib.lib().jpt_prefill_insert_paged(
          _lib.ptr(pk), _lib.ptr(pv), _lib.dt(pk), _lib.ptr(ck), _lib.ptr(cv), _lib.dt(ck), _lib.ptr(ks),
          _lib.ptr(vs), _lib.ptr(upd), n_pages, len(prefill_caches), h, pk.shape[2], p, ps, d, ps_l, pk.stride(1),
          pk.stride(2), cs_l, ss_l, _lib.stream()))
      return decode_caches
    for i, ((pk, pv), (ck, cv)) in enumerate(zip(prefill_caches, decode_caches)):
      h, p, ps, d = ck.shape
      _, hp, l, dp = pk.shape
      if (hp, dp) != (h, d):
        raise ValueError(f"prefix heads/dim {(hp, dp)} do not match the pool {(h, d)}")
      if pk.stride(-1) != 1 or pv.stride() != pk.stride():
        pk, pv = pk.contiguous(), pv.contiguous()
      ks = vs = None
      if decode_scales is not None:
        ks, vs = decode_scales[i]
      _lib.check(_lib.lib().jpt_prefill_insert_paged(
          _lib.ptr(pk), _lib.ptr(pv), _lib.dt(pk), _lib.ptr(ck), _lib.ptr(cv), _lib.dt(ck), _lib.ptr(ks),
          _lib.ptr(vs), _lib.ptr(upd), n_pages, 1, h, l, p, ps, d, 0, pk.stride(1), pk.stride(2), 0, 0,
          _lib.stream()))
    return decode_caches

  def get_compress_kv_cache(self, decode_caches, slot: int):
    """page_attention_manager.py:180-192."""
    lens = int(self.lengths[slot])
    indices = self.page_indices[slot]
    return [(self._compress_cache(k, lens, indices), self._compress_cache(v, lens, indices))
            for k, v in decode_caches]

  def _compress_cache(self, cache, lens: int, indices):
    """page_attention_manager.py:194-200 (not on the step path: torch gather)."""
    head, _, _, dim = cache.shape
    idx = torch.as_tensor(np.asarray(indices), device=cache.device).long()
    return cache[:, idx, :, :].reshape(head, -1, dim)[:, :lens, :]
