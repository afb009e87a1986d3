"""Oracle (test infrastructure): the bookkeeping of the reference engine's
decode step, restated with plain Python loops over numpy arrays.

Follows jetstream_pt/engine.py:751-848 (`generate_impl`: mask, input_pos, lens,
current_position, the result-token block) and 674-729
(`precompute_ragged_block_indices`).
"""

import numpy as np


def ragged_block_indices(start, input_pos, cache_len, block_size):
  """engine.py:674-729, one (slot, block) at a time.  Returns int arrays
  [B, S // bk]: the slot and the block the grid point should fetch."""
  b_count = len(start)
  num_bk = cache_len // block_size
  out_b = np.zeros((b_count, num_bk), dtype=np.int64)
  out_i = np.zeros((b_count, num_bk), dtype=np.int64)
  for b in range(b_count):
    st = int(start[b])
    en = (st + int(input_pos[b])) % cache_len
    last = b == b_count - 1
    last_good = (en - 1) // block_size if st < en else (cache_len - 1) // block_size
    next_b = b if last else b + 1
    next_i = last_good if last else 0
    for i in range(num_bk):
      if st < en:
        nb, ni = (next_b, next_i) if i * block_size >= en else (b, i)
        if (i + 1) * block_size <= st:
          ni = st // block_size
      elif st == en:
        nb, ni = next_b, next_i
      else:
        nb = b
        ni = st // block_size if (i * block_size >= en and (i + 1) * block_size <= st) else i
      out_b[b, i], out_i[b, i] = nb, ni
  return out_b, out_i


def decode_step_bookkeeping(ring_buffer, lazy_cache_update, cache_len, tokens, lens, input_pos, mask,
                            current_position, next_token):
  """engine.py:774-846 around the model call.  tokens, lens [B,1]; input_pos
  [B]; mask [B,S] float.  Returns (mask given to the model, mask afterwards,
  input_pos, lens, current_position, result data [B,3])."""
  mask = mask.copy()

  def opened(m):
    m = m.copy()
    if ring_buffer:
      m[:, current_position] = 0
    else:
      for b in range(m.shape[0]):
        m[b, int(input_pos[b])] = 0
    return m

  model_mask = mask if lazy_cache_update else opened(mask)
  new_mask = opened(mask)
  if ring_buffer:
    new_pos, new_lens = input_pos + 1, lens + 1
  else:
    new_pos = np.where(input_pos == 0, 0, input_pos + 1)  # `x + 1 % cache_len` is x + 1
    new_lens = np.where(lens == 0, 0, lens + 1)
  data = np.concatenate([tokens, np.ones_like(next_token), new_lens], axis=-1)
  return model_mask, new_mask, new_pos, new_lens, (current_position + 1) % cache_len, data
