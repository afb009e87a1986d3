"""The KV-cache side of the reference's serving engine step
(jetstream_pt/engine.py): `DecodeState`, `init_decode_state`, `insert`, the
bookkeeping of `generate_impl` (mask, input_pos, lens, current_position, the
result-token block), `precompute_ragged_block_indices`, greedy sampling, and the
paged driver `generate_page_attention` without its per-step device-to-host
round trip.

The model itself is not part of this package: `KVCacheEngine` takes the model
as a callable with the argument list the reference passes to its PyTorch model
(tokens, input_pos, caches, mask, start, ragged_batch_index,
ragged_block_index) and expects logits [B, T, vocab] back.  State tensors live
on the GPU and are updated in place where the reference updates donated
buffers.
"""

import dataclasses
from typing import Any, Callable, List, Optional, Tuple

import numpy as np
import torch

from jetstream_pytorch_b200 import _lib
from jetstream_pytorch_b200 import cache_manager
from jetstream_pytorch_b200 import insert as insert_ops
from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager


@dataclasses.dataclass
class Prefix:
  """engine.py:58-63."""
  token: torch.Tensor  # [1, 1] the first generated token
  caches: List[Tuple[torch.Tensor, torch.Tensor]]  # per layer [1,H,Lpad,D]
  seq_len: int  # true length of the prompt


@dataclasses.dataclass
class DecodeState:
  """engine.py:66-78."""
  tokens: torch.Tensor  # [B, 1] int32
  caches: List[Tuple[torch.Tensor, torch.Tensor]]
  cache_scales: List[Tuple[torch.Tensor, torch.Tensor]]  # int8 caches only
  current_position: int
  lens: torch.Tensor  # [B, 1] int32, generated tokens per slot
  start: torch.Tensor  # [B] int32, first valid position per slot
  input_pos: torch.Tensor  # [B] int32, tokens in the cache per slot
  mask: torch.Tensor  # [B, S]: 0 valid, -inf invalid


def greedy_sampling(logits):
  """The greedy branch of the reference's sampling (engine.py:283-297 with
  sampling_algorithm "greedy"): argmax over the vocabulary of the last
  position, as int32 [B, 1]."""
  if logits.ndim == 2:
    logits = logits.unsqueeze(0)
  last = logits[:, -1]
  return torch.argmax(last, dim=-1).reshape(last.shape[0], -1).to(torch.int32)


def update_mask(env, mask, current_position, input_pos):
  """engine.py:774-779: open this step's position in the mask, in place."""
  if env.ring_buffer:
    mask[:, current_position] = 0
  else:
    batch = torch.arange(mask.shape[0], device=mask.device)
    mask[batch, input_pos.long()] = 0
  return mask


def advance_positions(env, input_pos, lens):
  """engine.py:807-818.  Ring buffer: every slot advances.  Left aligned: idle
  slots (0) stay idle; the reference writes `x + 1 % cache_len`, which is
  `x + 1` by operator precedence, and so does this."""
  if env.ring_buffer:
    return input_pos + 1, lens + 1
  return (torch.where(input_pos == 0, torch.zeros_like(input_pos), input_pos + 1),
          torch.where(lens == 0, torch.zeros_like(lens), lens + 1))


def precompute_ragged_block_indices(env, start, input_pos):
  """engine.py:674-729: for every (slot, block) of the (batch, S // bk) grid, the
  (slot, block) whose K/V block the TPU kernel should fetch next, so that blocks
  outside [start, end) are skipped.  The CUDA kernels skip by their loop bounds
  and ignore these tables; they are produced for callers that pass them on."""
  s, bk = env.cache_len, env.block_size
  b_count = start.shape[0]
  end = ((start + input_pos) % s).reshape(b_count, 1)
  start = start.reshape(b_count, 1)
  dev = start.device
  b = torch.arange(b_count, device=dev, dtype=start.dtype).reshape(b_count, 1)
  num_bk = s // bk
  i = torch.arange(num_bk, device=dev, dtype=start.dtype).reshape(1, num_bk).expand(b_count, num_bk)
  am_last = b == b_count - 1
  last_good = torch.where(start < end, torch.div(end - 1, bk, rounding_mode="trunc"),
                          torch.full_like(end, (s - 1) // bk))
  next_b = torch.where(am_last, b, b + 1)
  next_i = torch.where(am_last, last_good, torch.zeros_like(last_good))
  past_end = i * bk >= end
  t_b = torch.where(past_end, next_b, b)
  t_i = torch.where(past_end, next_i, i)
  t_i = torch.where((i + 1) * bk <= start, torch.div(start, bk, rounding_mode="trunc"), t_i)
  f_b = b.expand(b_count, num_bk)
  f_i = torch.where(past_end & ((i + 1) * bk <= start), torch.div(start, bk, rounding_mode="trunc").expand_as(i), i)
  lt, eq = start < end, start == end
  b_next = torch.where(lt, t_b, torch.where(eq, next_b.expand(b_count, num_bk), f_b))
  i_next = torch.where(lt, t_i, torch.where(eq, next_i.expand(b_count, num_bk), f_i))
  return b_next, i_next


class KVCacheEngine:
  """`PyTorchEngine` reduced to what touches the KV cache."""

  def __init__(self, env, model_fn: Optional[Callable] = None):
    self.env = env
    self.model_fn = model_fn
    self.default_dtype = torch.bfloat16 if env.bf16_enable else torch.float32
    self.page_attention_manager = None
    self._pam_device = None
    if env.page_attention:
      ps = env.paged_attention_page_size
      assert env.cache_len % ps == 0, "cache_sequence_length should be a multiple of the page size"
      self.page_attention_manager = PageAttentionManager(
          batch_size=env.batch_size, paged_attention_total_num_pages=env.paged_attention_total_num_pages,
          paged_attention_page_size=ps, max_pages_per_sequence=env.cache_len // ps)
      self._host_pos = np.zeros(env.batch_size, dtype=np.int64)  # host mirror of input_pos (no device read per step)

  # ------------------------------------------------------------------ state
  def init_decode_state(self) -> DecodeState:
    """engine.py:163-186."""
    env, dev = self.env, self.env.device
    objs = env.make_caches_generate()
    caches = [c.state() for c in objs]
    scalers = [c.scalers() for c in objs] if env.quant_config.enable_kv_quantization else []
    b = env.batch_size
    return DecodeState(
        torch.zeros((b, 1), dtype=torch.int32, device=dev), caches, scalers, env.starting_position,
        torch.zeros((b, 1), dtype=torch.int32, device=dev), torch.zeros((b,), dtype=torch.int32, device=dev),
        torch.zeros((b,), dtype=torch.int32, device=dev),
        torch.full((b, env.cache_len), float("-inf"), dtype=self.default_dtype, device=dev))

  # ------------------------------------------------------------------ insert
  def insert(self, prefix: Prefix, decode_state: DecodeState, slot: int) -> DecodeState:
    """engine.py:627-672: scatter the prefix into the slot (dense: no-wrap /
    wrap; paged: reserve pages, then scatter) and write the slot's rows of
    tokens, mask, start, input_pos and lens."""
    env = self.env
    decode_state.tokens[slot] = prefix.token.reshape(-1).to(decode_state.tokens.dtype)
    if env.page_attention:
      insert_ops.insert_page_attention_with_reservation(
          self.page_attention_manager, prefix.caches, prefix.seq_len, decode_state.caches, slot,
          cache_scales=decode_state.cache_scales or None)
      decode_state.mask[slot] = insert_ops.insert_mask_row(env.cache_len, 0, prefix.seq_len, False,
                                                           decode_state.mask.device, decode_state.mask.dtype)
      decode_state.start[slot] = 0
      decode_state.input_pos[slot] = prefix.seq_len
      decode_state.lens[slot] = 1
      self._host_pos[slot] = prefix.seq_len
      self._pam_device = None
      self.page_attention_manager.lengths_device = None
      self.page_attention_manager.page_indices_device = None
      return decode_state
    insert_ops.insert(env, prefix.caches, prefix.seq_len, decode_state.caches, decode_state.cache_scales or None, slot,
                      decode_state.current_position, mask=decode_state.mask, start=decode_state.start,
                      input_pos=decode_state.input_pos, lens=decode_state.lens)
    return decode_state

  # ------------------------------------------------------------------ one decode step
  def precompute_ragged_block_indices(self, decode_state: DecodeState):
    return precompute_ragged_block_indices(self.env, decode_state.start, decode_state.input_pos)

  def make_caches(self, decode_state: DecodeState, input_indexes, page_token_indices=None, n_active_dev=None):
    """The cache objects `_call_model_generate` builds for the model's layers
    (engine.py:201-236)."""
    env = self.env
    if env.quant_config.enable_kv_quantization and not env.page_attention:
      return [cache_manager.Int8KVCacheGenerate(k, v, ks, vs, input_indexes, env=env)
              for (k, v), (ks, vs) in zip(decode_state.caches, decode_state.cache_scales)]
    if env.page_attention:
      scales = decode_state.cache_scales or [(None, None)] * len(decode_state.caches)
      return [cache_manager.PageKVCacheGenerate(k, v, self.page_attention_manager, page_token_indices, None, env=env,
                                                k_scaler=ks, v_scaler=vs, n_active_dev=n_active_dev)
              for (k, v), (ks, vs) in zip(decode_state.caches, scales)]
    return [cache_manager.KVCacheGenerate(k, v, input_indexes, None, env=env) for k, v in decode_state.caches]

  def generate_impl(self, params: Any, decode_state: DecodeState, sampler=None, page_token_indices=None,
                    n_active_dev=None):
    """engine.py:751-848.  Returns (new DecodeState, result data [B, 3]:
    previous tokens | ones | lens, the layout of the reference's ResultTokens)."""
    env = self.env
    pos = decode_state.current_position
    input_indexes = [pos] if env.ring_buffer else decode_state.input_pos
    rbi, rbk = self.precompute_ragged_block_indices(decode_state)
    rbi, rbk = rbi.reshape(-1), rbk.reshape(-1)
    mask = decode_state.mask
    if not env.lazy_cache_update:
      mask = update_mask(env, mask, pos, decode_state.input_pos)
    caches_obj = self.make_caches(decode_state, input_indexes, page_token_indices, n_active_dev)
    logits = self.model_fn(params, decode_state.tokens, decode_state.input_pos, caches_obj,
                           mask.unsqueeze(1).unsqueeze(2), decode_state.start, rbi, rbk)
    new_caches, new_scales = [], []
    for c in caches_obj:
      c.finalize()
      new_caches.append(c.state())
    if env.quant_config.enable_kv_quantization and not env.page_attention:
      new_scales = [c.scalers() for c in caches_obj]
    elif decode_state.cache_scales:
      new_scales = decode_state.cache_scales
    if env.lazy_cache_update:
      mask = update_mask(env, mask, pos, decode_state.input_pos)  # after the model: it used flash attention
    next_token = sampler(logits[:, -1]) if sampler else greedy_sampling(logits)
    input_pos, lens = advance_positions(env, decode_state.input_pos, decode_state.lens)
    data = torch.cat([decode_state.tokens, torch.ones_like(next_token), lens], dim=-1)
    new_state = DecodeState(next_token, new_caches, new_scales, (pos + 1) % env.cache_len, lens, decode_state.start,
                            input_pos, mask)
    return new_state, data

  def generate_page_attention(self, params: Any, decode_state: DecodeState, sampler=None):
    """engine.py:736-749 without the device read: the host keeps a mirror of
    input_pos (it changes by +1 per step for active slots and by `insert`), so
    page reservation (the FIFO free list, exactly the reference's order) runs on
    the host without waiting for the GPU; the page table goes to the device only
    after it changed, and the (page, offset, slot) triples of the step are
    computed there by `jpt_page_token_indices`."""
    pam, dev = self.page_attention_manager, self.env.device
    before = pam.page_indices.copy()
    pam.fill_new_pages(self._host_pos)
    if self._pam_device is None or not np.array_equal(before, pam.page_indices):
      self._pam_device = torch.as_tensor(pam.page_indices, dtype=torch.int32).to(dev, non_blocking=True)
    pti, n_active, new_lengths = pam.get_page_token_indices_device(decode_state.input_pos, self._pam_device)
    pam.lengths_device, pam.page_indices_device = new_lengths, self._pam_device  # read by the attention caller
    new_state, data = self.generate_impl(params, decode_state, sampler=sampler, page_token_indices=pti,
                                         n_active_dev=n_active)
    self._host_pos = np.where(self._host_pos == 0, 0, self._host_pos + 1)
    pam.lengths = self._host_pos.astype(np.asarray(pam.lengths).dtype)  # what get_page_token_indices would have stored
    return new_state, data

  def generate(self, params: Any, decode_state: DecodeState, sampler=None):
    if self.env.page_attention:
      return self.generate_page_attention(params, decode_state, sampler)
    return self.generate_impl(params, decode_state, sampler)
