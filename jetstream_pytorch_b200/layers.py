"""The two attention callers that sit directly above the KV-cache path, with
the branch structure, call order and return shapes of the reference's
`AttentionKernel` and `Int8KVAttentionKernel` (jetstream_pt/layers.py:382-550,
553-718).  They exist so the cache objects and attention entry points can be
exercised exactly the way the reference's model code drives them; projections,
RoPE and the rest of `layers.Attention` stay outside this package.
"""

import torch

from jetstream_pytorch_b200 import attention_kernel as ak


class _AttentionKernelBase:
  quantized = False

  def __init__(self, env, layer_id):
    self.env = env
    self.layer_id = layer_id
    self.q_shard_axis = 0 if env.shard_on_batch else 1
    self.kv_shard_axis = 0 if env.shard_on_batch else 2 if env.generate_cache_stacked else 1
    self.dense_attention = ak.dense_attention
    self.flash_attention = ak.flash_attention
    self.page_attention = ak.call_paged_attention
    self.ragged_attention_orig = ak.RaggedAttentionKernel(env, q_shard_axis=self.q_shard_axis,
                                                          kv_shard_axis=self.kv_shard_axis)
    self.ragged_attention_new = ak.RaggedAttentionKernel(env, q_shard_axis=self.q_shard_axis,
                                                         kv_shard_axis=self.q_shard_axis)

  def _attend(self, xq, keys, values, k_scaler, v_scaler, local_mask, cache, start, end, ragged_batch_index,
              ragged_block_index, seqlen, n_rep):
    """`attend`, layers.py:440-516 / 610-674."""
    env = self.env
    bsz, num_heads, _, head_dim = xq.shape
    impl = self.ragged_attention_new if keys.ndim == 4 else self.ragged_attention_orig
    true_len = seqlen
    paged = (not self.quantized) and env.page_attention
    # q is padded to two rows unless grouped ragged attention takes it
    # (layers.py:449-457, 619-623); the padded row is dropped again below.
    if not (env.ragged_mha and n_rep > 1) and seqlen == 1 and not paged:
      true_len = 2
      xq = torch.nn.functional.pad(xq, (0, 0, 0, true_len - seqlen), "constant", 0)
    local_max = local_denom = None
    if env.ragged_mha and seqlen == 1 and keys.shape[-2] > 1:
      local_output, (local_max, local_denom) = impl(xq, keys, values, self.layer_id, start, end,
                                                    ragged_batch_index, ragged_block_index, k_scaler, v_scaler)
    elif env.flash_attention and seqlen == 1:
      local_output, (local_max, local_denom) = self.flash_attention(
          xq=xq, keys=keys, values=values, layer=self.layer_id, k_scaler=k_scaler, v_scaler=v_scaler,
          mask=local_mask)
    elif paged and seqlen == 1:
      # the engine's paged driver leaves device copies of the tables behind (no host copy per layer)
      pam = cache.page_attention_manager
      lengths = getattr(pam, "lengths_device", None)
      table = getattr(pam, "page_indices_device", None)
      local_output = self.page_attention(env, torch.squeeze(xq, 2), keys, values,
                                         pam.lengths if lengths is None else lengths,
                                         pam.page_indices if table is None else table)
    else:
      local_output = self.dense_attention(xq=xq, keys=keys, values=values, k_scaler=k_scaler,
                                          v_scaler=v_scaler, mask=local_mask)
    local_output = local_output.reshape(bsz, num_heads, true_len, head_dim)
    if local_max is not None:
      local_max = local_max.reshape(bsz, num_heads, true_len, 1)
      local_denom = local_denom.reshape(bsz, num_heads, true_len, 1)
    if true_len != seqlen:
      local_output = local_output[:, :, 0:seqlen, :]
      if local_max is not None:
        local_max = local_max[:, :, 0:seqlen, :]
        local_denom = local_denom[:, :, 0:seqlen, :]
    return local_output, (local_max, local_denom)

  @staticmethod
  def _merge(existing_output, existing_max, existing_denom, new_output, new_max, new_denom):
    """"attn_global", layers.py:539-550 / 708-718 (result in float32, as the
    float32 denominators promote it in the reference)."""
    return ak.merge_partials(existing_output, existing_max, existing_denom, new_output, new_max, new_denom)


class AttentionKernel(_AttentionKernelBase):
  """layers.py:382-550."""

  def __call__(self, xq, xk, xv, mask, cache, start=None, end=None, ragged_batch_index=None,
               ragged_block_index=None):
    _, num_heads, seqlen, _ = xq.shape
    n_rep = num_heads // xk.shape[-3]
    args = (cache, start, end, ragged_batch_index, ragged_block_index, seqlen, n_rep)
    orig_keys, orig_values = cache.update(xk, xv, self.layer_id)
    existing_output, (existing_max, existing_denom) = self._attend(xq, orig_keys, orig_values, None, None, mask,
                                                                   *args)
    if not self.env.lazy_cache_update or seqlen > 1:
      return existing_output
    new_output, (new_max, new_denom) = self._attend(xq, xk, xv, None, None, None, *args)
    return self._merge(existing_output, existing_max, existing_denom, new_output, new_max, new_denom)


class Int8KVAttentionKernel(_AttentionKernelBase):
  """layers.py:553-718."""

  quantized = True
  fused_step = True  # the lazy ragged decode step of a GQA model runs as one launch where the shape allows

  def __call__(self, xq, xk, xv, mask, cache, start=None, end=None, ragged_batch_index=None,
               ragged_block_index=None):
    bsz, num_heads, seqlen, head_dim = xq.shape
    n_rep = num_heads // xk.shape[-3]
    args = (cache, start, end, ragged_batch_index, ragged_block_index, seqlen, n_rep)
    if (self.fused_step and self.env.ragged_mha and self.env.lazy_cache_update and n_rep > 1 and seqlen == 1
        and hasattr(cache, "update_and_attend") and cache.fused_step_supported(xq, xk)):
      # One launch instead of update + ragged attention over the cache + flash attention over the
      # new token + merge (the four steps below): the same softmax over the same tokens.
      _, (out, _, _) = cache.update_and_attend(xq, xk, xv, self.layer_id, start, end)
      return out.reshape(bsz, num_heads, seqlen, head_dim).float()  # the merge of the four-step form yields float32
    (orig_keys, orig_values, new_key, new_value, k_scaler, v_scaler, new_k_scaler,
     new_v_scaler) = cache.update(xk, xv, self.layer_id)
    existing_output, (existing_max, existing_denom) = self._attend(xq, orig_keys, orig_values, k_scaler,
                                                                   v_scaler, mask, *args)
    if not self.env.lazy_cache_update or seqlen > 1:
      return existing_output
    new_output, (new_max, new_denom) = self._attend(xq, new_key, new_value, new_k_scaler, new_v_scaler, None,
                                                    *args)
    return self._merge(existing_output, existing_max, existing_denom, new_output, new_max, new_denom)
