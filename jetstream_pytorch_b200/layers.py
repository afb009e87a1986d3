"""The two attention callers that sit directly above the KV-cache path, with
the branch structure, call order and return shapes of the reference's
`AttentionKernel` and `Int8KVAttentionKernel` (jetstream_pt/layers.py:382-550,
553-718).  They exist so the cache objects and attention entry points can be
exercised exactly the way the reference's model code drives them; RoPE and the
rest of `layers.Attention` stay outside this package.

`WeightOnlyPerChannelQuantizedLinear` (jetstream_pt/layers.py:69-166) is the
other byte stream of a decode step: the int8 weights of the projections.
`RMSNorm` (layers.py:337-350) and `FeedForward`
(third_party/llama/model_exportable.py:32-86) are the producers and consumers of
its activations in a decoder block; for decode batches they hand the int8 level
split of their results (`ActivationLevels`) to the linear layers behind them.
"""

import ctypes

import torch

from jetstream_pytorch_b200 import _lib
from jetstream_pytorch_b200 import attention_kernel as ak
from jetstream_pytorch_b200.environment import QuantizationConfig


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


class WeightOnlyPerChannelQuantizedLinear(torch.nn.Module):
  """layers.py:69-166 for decode batches: int8 weights [out, in] with one bf16
  scale per output channel, bf16 activations, result
  bf16(bf16(inputs @ weight^T) * weight_scaler).

  Built: 8-bit symmetric weights, no activation quantisation, `in_features` a
  multiple of 128.  The kernel is made for decode batches (up to 128 rows of
  activations stream the weights once); more rows go through in blocks of 128.
  Anything else raises; there is no eager path."""

  def __init__(self, in_features, out_features, bias=False, device=None, quant_config=None):
    super().__init__()
    quant_config = QuantizationConfig() if quant_config is None else quant_config
    assert not bias, "Quantized Linear doesn't support bias."
    if not getattr(quant_config, "is_symmetric_weight", True):
      raise NotImplementedError("asymmetric weights are not provided")
    if getattr(quant_config, "enable_activation_quantization", False):
      raise NotImplementedError("activation quantisation is not provided")
    if getattr(quant_config, "num_bits_weight", 8) != 8:
      raise NotImplementedError("only 8-bit weights are provided")
    if in_features % 128:
      raise NotImplementedError(f"in_features = {in_features} must be a multiple of 128")
    self.in_features = in_features
    self.out_features = out_features
    self.register_buffer("weight", torch.ones((out_features, in_features), dtype=torch.int8, device=device))
    self.register_buffer("weight_scaler", torch.ones((out_features,), dtype=torch.bfloat16, device=device))
    self.register_buffer("zero_point", None)
    self.is_symmetric_weight = True
    self.n_bit = 8
    self.quantize_activation = False
    self._workspace = None

  def _load_quantized_weights(self, w_q, scale, zp=None):
    """layers.py:114-120 with `load_q_weight_helper` (quantize.py:86-93)."""
    if zp is not None:
      raise NotImplementedError("asymmetric weights are not provided")
    dev = self.weight.device
    self.weight = w_q.to(torch.int8).to(dev).contiguous()
    self.weight_scaler = scale.reshape(self.out_features).to(torch.bfloat16).to(dev).contiguous()

  def quantize_weight_from_nn_linear(self, weight):
    """layers.py:122-133: per-channel symmetric quantisation of a float weight
    (quantize.py:58-76).  Offline work, plain torch."""
    assert weight.dim() == 2, "Expect 2D weight from torch.nn.Linear."
    assert weight.shape == (self.out_features, self.in_features), (
        f"Got unexpected weight of shape {weight.shape}, expected weight shape "
        f"({self.out_features}, {self.in_features}).")
    max_val = weight.abs().amax(dim=1, keepdim=True).clamp(min=1e-5)
    scales = max_val / 127
    w_q = torch.clamp(torch.round(weight * (1.0 / scales)), -128, 127).to(torch.int8)
    self._load_quantized_weights(w_q, scales.squeeze(-1))

  def kernel_status(self):
    """0, or 1 if a bounded wait inside the last launch gave up (synchronises)."""
    return 0 if self._workspace is None else int(self._workspace[:4].view(torch.int32).item())

  def forward(self, inputs, levels=None, tp=None):
    """`levels` (an `ActivationLevels` of `inputs`, from `RMSNorm`, `FeedForward`
    or `ActivationLevels.of`): the layer starts at its GEMM.
    `tp` (a `TensorParallelSum`): this rank holds a slice of the input features
    (`weight` [out, in / world], `inputs` [..., in / world]); the partial results
    of the ranks are added inside the kernel and every rank gets the whole
    output (the all-reduce behind `wo` and `w2` of the reference's sharding,
    default_shardings/llama.yaml:10,20)."""
    if inputs.dtype != torch.bfloat16:
      raise NotImplementedError(f"activations must be bfloat16, got {inputs.dtype}")
    k, n = self.in_features, self.out_features
    x = inputs.reshape(-1, k)
    m = x.shape[0]
    if m < 1:
      return inputs.new_empty((*inputs.shape[:-1], n))
    if tp is not None:
      if levels is not None or m > ActivationLevels.MAX_ROWS:
        raise NotImplementedError("the row-parallel form takes up to 128 rows of bf16 activations")
      x = x.contiguous()
      lib = _lib.lib()
      need = lib.jpt_w8a16_linear_workspace_bytes(m, n, k)
      if self._workspace is None or self._workspace.numel() < need or self._workspace.device != x.device:
        self._workspace = torch.empty((need,), dtype=torch.uint8, device=x.device)
      y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
      _lib.check(lib.jpt_w8a16_linear_tp(_lib.ptr(x), _lib.ptr(self.weight), _lib.ptr(self.weight_scaler), _lib.ptr(y), m, n, k,
                                         _lib.ptr(self._workspace), self._workspace.numel(), ctypes.byref(tp.struct),
                                         _lib.stream()))
      return y.reshape(*inputs.shape[:-1], n)
    if levels is not None:
      if (levels.rows, levels.features) != (m, k):
        raise ValueError(f"levels of a [{levels.rows}, {levels.features}] activation given for [{m}, {k}]")
      y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
      ws = levels.workspace
      _lib.check(_lib.lib().jpt_w8a16_linear_from_levels(_lib.ptr(ws), ws.numel(), _lib.ptr(self.weight),
                                                         _lib.ptr(self.weight_scaler), _lib.ptr(y), m, n, k, _lib.stream()))
      self._workspace = ws  # (kernel_status reads the status word of the workspace last used)
      return y.reshape(*inputs.shape[:-1], n)
    if not x.is_contiguous():
      x = x.contiguous()
    lib = _lib.lib()
    need = lib.jpt_w8a16_linear_workspace_bytes(m, n, k)
    if self._workspace is None or self._workspace.numel() < need or self._workspace.device != x.device:
      self._workspace = torch.empty((need,), dtype=torch.uint8, device=x.device)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    _lib.check(lib.jpt_w8a16_linear(_lib.ptr(x), _lib.ptr(self.weight), _lib.ptr(self.weight_scaler), _lib.ptr(y), m, n,
                                    k, _lib.ptr(self._workspace), self._workspace.numel(), _lib.stream()))
    return y.reshape(*inputs.shape[:-1], n)


class ActivationLevels:
  """The int8 level split of a [rows, features] bf16 activation (rows <= 128), as
  the weight-only linear layers' GEMM reads it: x = s (h + l / 254) per row with
  signed bytes h, l.  One split serves every layer that reads the activation."""

  MAX_ROWS = 128

  def __init__(self, rows, features, device):
    if not 1 <= rows <= self.MAX_ROWS or features % 128:
      raise NotImplementedError(f"levels are kept for 1 .. {self.MAX_ROWS} rows of a multiple of 128 features, "
                                f"got [{rows}, {features}]")
    self.rows, self.features = rows, features
    need = _lib.lib().jpt_w8a16_linear_workspace_bytes(rows, 1, features)
    self.workspace = torch.empty((need,), dtype=torch.uint8, device=device)

  @classmethod
  def fits(cls, x):
    return x.is_cuda and x.dtype == torch.bfloat16 and 1 <= x.numel() // x.shape[-1] <= cls.MAX_ROWS and x.shape[-1] % 128 == 0

  @classmethod
  def of(cls, x):
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    lv = cls(x2.shape[0], x2.shape[1], x.device)
    _lib.check(_lib.lib().jpt_w8a16_split_levels(_lib.ptr(x2), lv.rows, lv.features, _lib.ptr(lv.workspace),
                                                 lv.workspace.numel(), _lib.stream()))
    return lv


class RMSNorm(torch.nn.Module):
  """layers.py:337-350 with a bf16 weight:
  bf16(bf16(x * rsqrt(mean(x^2) + eps)) * weight), the mean in fp32."""

  def __init__(self, dim: int, eps: float = 1e-6, device=None):
    super().__init__()
    self.eps = eps
    self.weight = torch.nn.Parameter(torch.ones(dim, dtype=torch.bfloat16, device=device), requires_grad=False)

  def forward(self, x, with_levels=False):
    """Returns y, or (y, ActivationLevels of y) with `with_levels`."""
    if x.dtype != torch.bfloat16 or self.weight.dtype != torch.bfloat16:
      raise NotImplementedError("RMSNorm is provided for bfloat16 activations and weights")
    k = x.shape[-1]
    x2 = x.reshape(-1, k).contiguous()
    m = x2.shape[0]
    y = torch.empty_like(x2)
    lv = ActivationLevels(m, k, x.device) if with_levels else None
    _lib.check(_lib.lib().jpt_rmsnorm(_lib.ptr(x2), _lib.ptr(self.weight), float(self.eps), _lib.ptr(y), m, k,
                                      _lib.ptr(lv.workspace) if lv else None, lv.workspace.numel() if lv else 0,
                                      _lib.stream()))
    y = y.reshape(x.shape)
    return (y, lv) if with_levels else y


def silu_mul(a, b, with_levels=False):
  """bf16(bf16(silu(a)) * b); with `with_levels` also the level split of the result."""
  if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.shape != b.shape:
    raise NotImplementedError("silu_mul takes two bfloat16 tensors of one shape")
  k = a.shape[-1]
  a2, b2 = a.reshape(-1, k).contiguous(), b.reshape(-1, k).contiguous()
  m = a2.shape[0]
  h = torch.empty_like(a2)
  lv = ActivationLevels(m, k, a.device) if with_levels else None
  _lib.check(_lib.lib().jpt_silu_mul(_lib.ptr(a2), _lib.ptr(b2), _lib.ptr(h), m, k, _lib.ptr(lv.workspace) if lv else None,
                                     lv.workspace.numel() if lv else 0, _lib.stream()))
  h = h.reshape(a.shape)
  return (h, lv) if with_levels else h


class FeedForward(torch.nn.Module):
  """third_party/llama/model_exportable.py:32-86 with weight-only int8 linear
  layers: w2(silu(w1(x)) * w3(x)).  For a decode batch the level split of x is
  made once for w1 and w3 (or taken from the norm in front: `levels`), and the
  gate writes the split of its result for w2: five launches in all."""

  def __init__(self, dim, hidden_dim, device=None, quant_config=None):
    super().__init__()
    self.w1 = WeightOnlyPerChannelQuantizedLinear(dim, hidden_dim, device=device, quant_config=quant_config)
    self.w2 = WeightOnlyPerChannelQuantizedLinear(hidden_dim, dim, device=device, quant_config=quant_config)
    self.w3 = WeightOnlyPerChannelQuantizedLinear(dim, hidden_dim, device=device, quant_config=quant_config)

  def forward(self, x, levels=None):
    if not ActivationLevels.fits(x):
      return self.w2(silu_mul(self.w1(x), self.w3(x)))
    if levels is None:
      levels = ActivationLevels.of(x)
    h, h_levels = silu_mul(self.w1(x, levels=levels), self.w3(x, levels=levels), with_levels=True)
    return self.w2(h, levels=h_levels)


class TensorParallelSum:
  """Receive buffers for the sum of the row-parallel linear layers' partial
  results over the GPUs of one box (`WeightOnlyPerChannelQuantizedLinear.forward(
  ..., tp=...)`): every rank allocates one buffer, exports its CUDA IPC handle and
  opens the others'.  `handles_all_gather(handle) -> [handle of rank 0, ...]` is
  any host-side all-gather of 64-byte strings.  All ranks must then make the same
  sequence of calls with the same shapes; one object serves every layer whose
  output has at most `max_out_features` channels."""

  def __init__(self, max_out_features, rank, world_size, handles_all_gather, wait_cycles=0):
    lib = _lib.lib()
    nbytes = lib.jpt_w8a16_tp_buffer_bytes(max_out_features, world_size)
    if nbytes == 0:
      raise ValueError(f"no row-parallel sum for {max_out_features} channels on {world_size} ranks (1..8 ranks)")
    own = ctypes.c_void_p()
    _lib.check(lib.jpt_peer_exchange_alloc(nbytes, ctypes.byref(own)))
    self._own = own
    handle = ctypes.create_string_buffer(64)
    _lib.check(lib.jpt_peer_exchange_export(own, handle))
    handles = handles_all_gather(handle.raw)
    self.struct = _lib.TpSumStruct()
    self.struct.rank, self.struct.world = rank, world_size
    self.struct.buffer_bytes = nbytes
    self.struct.wait_cycles = int(wait_cycles)
    self._opened = []
    for r in range(world_size):
      if r == rank:
        self.struct.buffers[r] = own.value
      else:
        peer = ctypes.c_void_p()
        _lib.check(lib.jpt_peer_exchange_import(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(peer)))
        self._opened.append(peer)
        self.struct.buffers[r] = peer.value

  @classmethod
  def with_torch_distributed(cls, max_out_features, wait_cycles=0):
    import torch.distributed as dist

    rank, world = dist.get_rank(), dist.get_world_size()

    def gather(h):
      out = [None] * world
      dist.all_gather_object(out, h)
      return out

    tp = cls(max_out_features, rank, world, gather, wait_cycles)
    dist.barrier()  # every rank has opened every buffer before anybody launches
    return tp

  def status(self):
    """0 while every wait of every launch was satisfied; 1 after a launch gave up on a peer."""
    return _lib.lib().jpt_w8a16_tp_status(ctypes.byref(self.struct), _lib.stream())

  def close(self):
    lib = _lib.lib()
    for p in self._opened:
      lib.jpt_peer_exchange_release(p)
    self._opened = []
    if self._own is not None:
      lib.jpt_peer_exchange_free(self._own)
      self._own = None
