"""Oracle (test infrastructure): the page manager of the reference, restated
with a plain Python list as the FIFO free list and numpy tables.

Follows jetstream_pt/page_attention_manager.py.  `free_pages` is NOT a
restatement: the reference's `free_pages_resource` (lines 214-222) is dead code
that cannot run (it calls `.at` on a numpy array and tests `index < 0` against a
table whose sentinel is the last page id); the recycling order defined here is
this project's extension and is marked as such.
"""

import numpy as np
import torch


class PageTableOracle:
  """`PageAttentionManager.__init__`, page_attention_manager.py:21-39: FIFO
  free list 0..P-1, `page_indices` [B, max_pages] filled with the sentinel
  P-1, `lengths` zeros."""

  def __init__(self, batch_size, total_num_pages, page_size, max_pages_per_sequence,
               free_order=None):
    self.batch_size = batch_size
    self.total = total_num_pages
    self.ps = page_size
    self.max_pages = max_pages_per_sequence
    self.free = list(range(total_num_pages) if free_order is None else free_order)
    self.page_indices = np.full((batch_size, max_pages_per_sequence),
                                total_num_pages - 1, dtype=np.int32)
    self.lengths = np.zeros(batch_size, dtype=np.int32)

  def _pop(self):
    if not self.free:
      raise IndexError("no free page")  # reference: queue.Empty
    return self.free.pop(0)

  def reserve_pages_insert(self, slot, seq_len):
    """page_attention_manager.py:42-52."""
    self.lengths[slot] = seq_len
    n = -(-seq_len // self.ps)
    pages = [self._pop() for _ in range(n)]
    self.page_indices[slot, :n] = pages
    return n, self.page_indices[slot, :n].copy()

  def fill_new_pages(self, lens):
    """`reserve_pages_decode` for every slot, page_attention_manager.py:55-64:
    a slot whose current length is a positive multiple of the page size gets
    one fresh page at column len // ps."""
    for slot in range(self.batch_size):
      n = int(lens[slot])
      if n > 0 and n % self.ps == 0:
        self.page_indices[slot, n // self.ps] = self._pop()

  def get_page_token_indices(self, lens):
    """page_attention_manager.py:145-177.  `lens` are the lengths BEFORE this
    step's token; afterwards `lengths = lens + 1` for active slots."""
    lens = np.asarray(lens)
    pages, toks, slots = [], [], []
    offset = 0
    for slot in range(self.batch_size):
      n = int(lens[slot])
      if n == 0:
        continue
      pages.append(int(self.page_indices[slot, n // self.ps]))
      toks.append(offset + n % self.ps)
      slots.append(slot)
      offset += self.ps
    self.lengths = np.where(lens == 0, 0, lens + 1).astype(self.lengths.dtype)
    return np.stack((np.asarray(pages, dtype=np.int64),
                     np.asarray(toks, dtype=np.int64),
                     np.asarray(slots, dtype=np.int64)))

  def free_pages(self, slot):
    """EXTENSION (no working counterpart in the reference): return the slot's
    pages to the tail of the FIFO in table order, reset its row to the sentinel
    and its length to zero."""
    n = -(-int(self.lengths[slot]) // self.ps)
    self.free.extend(int(p) for p in self.page_indices[slot, :n])
    self.page_indices[slot, :] = self.total - 1
    self.lengths[slot] = 0


def insert_prefill_pages(cache, prefix, update_indexes, page_size):
  """`insert_prefill_cache` for one tensor, page_attention_manager.py:83-142.
  cache [H,P,ps,D]; prefix [1,H,L,D]; the prefix is copied into a zero buffer
  of n*ps tokens, cut into pages and scattered, so the tail of the last page is
  overwritten with zeros."""
  idx = torch.as_tensor(np.asarray(update_indexes)).to(torch.int64)
  h, _, ps, d = cache.shape
  assert ps == page_size
  n = idx.numel()
  length = prefix.shape[2]
  assert length <= n * ps
  tep = torch.zeros((h, n * ps, d), dtype=cache.dtype)
  tep[:, :length, :] = prefix[0].to(cache.dtype)
  out = cache.clone()
  out[:, idx, :, :] = tep.reshape(h, n, ps, d)
  return out


def compress_cache(cache, page_row, length):
  """`_compress_cache`, page_attention_manager.py:194-200: gather a slot's
  pages through its page-table row and keep the first `length` tokens."""
  h, _, _, d = cache.shape
  idx = torch.as_tensor(np.asarray(page_row)).to(torch.int64)
  return cache[:, idx, :, :].reshape(h, -1, d)[:, :int(length), :]
