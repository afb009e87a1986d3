"""The slice of the reference's engine environment that the KV-cache path reads.

Mirrors the field names and the mode derivation of
jetstream_pt/environment.py:31-139 (data) and 143-246 (derived flags).  The
JAX mesh / PartitionSpec helpers of the reference become a (rank, world_size)
pair: KV heads are split evenly across ranks, everything else is replicated.
"""

import dataclasses
from typing import Tuple

import torch


@dataclasses.dataclass
class QuantizationConfig:
  """jetstream_pt/environment.py:31-40."""

  enable_weight_quantization: bool = False
  num_bits_weight: int = 8
  is_blockwise_weight: bool = False
  block_size_weight: int = 128
  is_symmetric_weight: bool = True

  enable_activation_quantization: bool = False
  enable_kv_quantization: bool = False
  exclude_layers: object = None


@dataclasses.dataclass
class JetEngineEnvironmentData:
  """jetstream_pt/environment.py:43-139, fields used by the cache path."""

  batch_size: int = 32
  cache_sequence_length: int = 2048
  max_input_sequence_length: int = 1024
  quant_config: QuantizationConfig = dataclasses.field(default_factory=QuantizationConfig)
  cache_shape: Tuple[int, ...] = ()
  num_layers: int = 0
  bf16_enable: bool = True
  shard_on_batch: bool = False
  ragged_mha: bool = False
  block_size: int = 512
  starting_position: int = 0
  ring_buffer: bool = True
  flash_attention: bool = False
  paged_attention_total_num_pages: int = 0
  paged_attention_page_size: int = 64
  generate_cache_stacked: bool = False
  new_cache_stacked: bool = False
  lazy_cache_update: bool = False
  testing: bool = False
  testing_seed: int = 0
  n_reps: int = 0


class JetEngineEnvironment:
  """Derived mode flags, jetstream_pt/environment.py:143-246."""

  def __init__(self, data: JetEngineEnvironmentData, device=None, rank=0, world_size=1):
    self._data = data
    self.device = torch.device(device if device is not None else "cuda")
    self.rank, self.world_size = rank, world_size
    self.batch_size = data.batch_size
    self.seq_len = data.max_input_sequence_length
    self.cache_len = data.cache_sequence_length
    self.block_size = data.block_size
    self.starting_position = data.starting_position
    self.num_layers = data.num_layers
    self.testing = data.testing
    self.testing_seed = data.testing_seed
    self.ring_buffer = data.ring_buffer
    self.page_attention = data.paged_attention_total_num_pages > 0
    on = not self.ring_buffer
    self.lazy_cache_update = on
    self.ragged_mha = on
    self.flash_attention = on
    self.generate_cache_stacked = on
    self.new_cache_stacked = on
    if self.testing:
      self.lazy_cache_update = data.lazy_cache_update
      self.ragged_mha = data.ragged_mha
      self.flash_attention = data.flash_attention
      self.generate_cache_stacked = data.generate_cache_stacked
      self.new_cache_stacked = data.new_cache_stacked
    if self.page_attention:
      self.lazy_cache_update = False
      self.ragged_mha = False
      self.flash_attention = False
      self.generate_cache_stacked = False
      self.new_cache_stacked = False
    self.default_type = torch.bfloat16 if data.bf16_enable else torch.float32
    if self.generate_cache_stacked:
      self.cache_shape = (self.num_layers, *data.cache_shape)
      self.cache_sharding_axis = 0 if data.shard_on_batch else 2
    else:
      self.cache_shape = tuple(data.cache_shape)
      self.cache_sharding_axis = 0 if (data.shard_on_batch or self.page_attention) else 1
    self.cache_sharding = None

  def __getattr__(self, name):
    return getattr(self._data, name)

  def apply_sharding(self, tensor, *, axis):
    """Sharding constraints are a no-op: each rank already holds its shard."""
    return None

  def make_caches_generate(self):
    """jetstream_pt/environment.py:288-313."""
    from jetstream_pytorch_b200 import cache_manager

    count = 1 if self.generate_cache_stacked else self.num_layers
    if self._data.quant_config.enable_kv_quantization:
      cls = cache_manager.Int8KVCacheGenerate
    elif self.page_attention:
      cls = cache_manager.PageKVCacheGenerate
    else:
      cls = cache_manager.KVCacheGenerate
    return [cls.empty(self.cache_shape, self.device, env=self) for _ in range(count)]

  def make_caches_prefill(self):
    """jetstream_pt/environment.py:281-286."""
    from jetstream_pytorch_b200 import cache_manager

    return [cache_manager.KVCachePrefill() for _ in range(self.num_layers)]
