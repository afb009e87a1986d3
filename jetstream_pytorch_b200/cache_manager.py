"""KV cache objects with the reference's names, constructor arguments, attribute
names and return shapes (jetstream_pt/cache_manager.py), backed by the CUDA
library.  Caches are CUDA tensors updated in place; `update` returns the same
tensor objects it was constructed with.

Cache layouts (unchanged from the reference): dense [B,H,S,D] or stacked
[NL,B,H,S,D]; int8 scalers [B,1,S,1] / [NL,B,1,S,1]; page pools [H,P,ps,D].
"""

import numpy as np
import ctypes

import torch

from jetstream_pytorch_b200 import _lib
from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager


class CacheInterface:
  """Kv cache interface, jetstream_pt/cache_manager.py:26-39 (one layer's
  cache: `update(key, value)` with [B,H,T,D] tensors returns the full cache)."""

  def update(self, key, value):
    raise NotImplementedError


class KVCachePrefill:
  """jetstream_pt/cache_manager.py:42-69: remembers K/V as given.  With
  `kv_quantize` it returns the int8-style 8-tuple with unit scalers
  [B,1,T,1] and no "new" entries, so prefill attention runs unquantised."""

  def __init__(self, kv_quantize=False, stacked=False):
    self.kv_quantize = kv_quantize
    self.cache_k = None
    self.cache_v = None
    self.stacked = stacked

  def update(self, key, value, layer_id):
    self.cache_k = key
    self.cache_v = value
    if self.kv_quantize:
      bsz, _, seq, _ = key.shape
      ones = torch.ones((bsz, 1, seq, 1), dtype=torch.bfloat16, device=key.device)
      return key, value, None, None, ones, ones, None, None
    return key, value

  def state(self):
    return self.cache_k, self.cache_v

  def finalize(self):
    return


def _pos_args(input_pos, device, batch):
  """(device int32 tensor or None, count, host value) for the C ABI."""
  if isinstance(input_pos, torch.Tensor):
    t = _lib.as_i32(input_pos.reshape(-1), device).contiguous()
    n = t.numel()
  elif isinstance(input_pos, (int, np.integer)):
    return None, 1, int(input_pos), None
  else:
    arr = np.asarray(input_pos).reshape(-1)
    if arr.size == 1:
      return None, 1, int(arr[0]), None
    t = _lib.as_i32(arr, device)
    n = t.numel()
  if n not in (1, batch):
    raise ValueError(f"input_pos has {n} entries, expected 1 or {batch}")
  return _lib.ptr(t), n, 0, t  # keep `t` alive until the launch is enqueued


def _scatter_rows(src_k, src_v, dst_k, dst_v, input_pos, clamp, nl, b, h, s, d, strides):
  """dst[l, b, h, pos_b, :] = src[l, b, h, :] for K and V (C ABI jpt_kv_scatter_rows)."""
  p, n, host, keep = _pos_args(input_pos, dst_k.device, b)
  ds_l, ds_b, ds_h, ds_s = strides
  _lib.check(_lib.lib().jpt_kv_scatter_rows(
      _lib.ptr(src_k), _lib.ptr(src_v), _lib.ptr(dst_k), _lib.ptr(dst_v), dst_k.element_size(),
      p, n, host, int(clamp), nl, b, h, s, d, ds_l, ds_b, ds_h, ds_s, _lib.stream()))
  del keep


def _dense_strides(cache):
  if cache.stride(-1) != 1:
    raise ValueError("cache head_dim axis must be contiguous")
  if cache.ndim == 5:
    return cache.stride(0), cache.stride(1), cache.stride(2), cache.stride(3)
  return 0, cache.stride(0), cache.stride(1), cache.stride(2)


class KVCacheGenerate:
  """Unquantised decode cache, jetstream_pt/cache_manager.py:93-313."""

  # pylint: disable=too-many-instance-attributes
  def __init__(self, cache_k, cache_v, position, sharding=None, env=None):
    self.cache_k = cache_k
    self.cache_v = cache_v
    self.input_pos = position
    self.sharding = sharding
    self.env = env
    self.new_ks = None
    self.new_vs = None
    self.stacked = env.generate_cache_stacked
    if env.lazy_cache_update:
      if env.generate_cache_stacked:
        if env.new_cache_stacked:
          layer, batch, heads, _, dim = cache_k.shape
          shape = (layer, batch, heads, 1, dim)
          self.new_ks = torch.zeros(shape, dtype=cache_k.dtype, device=cache_k.device)
          self.new_vs = torch.zeros(shape, dtype=cache_k.dtype, device=cache_k.device)
        else:
          self.new_ks, self.new_vs = [], []
      else:
        assert not env.new_cache_stacked

  def _write(self, cache_k, cache_v, key, value, clamp=False):
    """One row per (slot, head) into an unstacked [B,H,S,D] view."""
    b, h, s, d = cache_k.shape
    _scatter_rows(key.contiguous(), value.contiguous(), cache_k, cache_v, self.input_pos, clamp, 1, b, h, s, d,
                  _dense_strides(cache_k))

  def update(self, key, value, layer_id: int):
    """cache_manager.py:227-293."""
    env = self.env
    if env.lazy_cache_update:
      if env.new_cache_stacked:
        assert env.generate_cache_stacked, "When new cache stacked, must have generate_cache_stacked!"
        self.new_ks[layer_id].copy_(key)
        self.new_vs[layer_id].copy_(value)
        return self.cache_k[layer_id], self.cache_v[layer_id]
      if env.generate_cache_stacked:
        self.new_ks.append(key)
        self.new_vs.append(value)
        return self.cache_k[layer_id], self.cache_v[layer_id]
      self.new_ks, self.new_vs = key, value
      return self.cache_k, self.cache_v
    if env.ring_buffer:
      assert not env.new_cache_stacked and not env.generate_cache_stacked, (
          "Ring buffer doesn't support stacked cache.")
      self._write(self.cache_k, self.cache_v, key, value)
      return self.cache_k, self.cache_v
    if env.generate_cache_stacked:
      self._write(self.cache_k[layer_id], self.cache_v[layer_id], key, value)
      return self.cache_k[layer_id], self.cache_v[layer_id]
    self._write(self.cache_k, self.cache_v, key, value)
    return self.cache_k, self.cache_v

  def finalize(self):
    """cache_manager.py:175-225."""
    env = self.env
    if not env.lazy_cache_update:
      return
    if env.ring_buffer:
      self._write(self.cache_k, self.cache_v, self.new_ks, self.new_vs)
      return
    if env.generate_cache_stacked:
      nl, b, h, s, d = self.cache_k.shape
      if env.new_cache_stacked:
        _scatter_rows(self.new_ks, self.new_vs, self.cache_k, self.cache_v, self.input_pos, True, nl, b, h, s, d,
                      _dense_strides(self.cache_k))
      else:
        for i in range(env.num_layers):
          self._write(self.cache_k[i], self.cache_v[i], self.new_ks[i], self.new_vs[i])
    else:
      self._write(self.cache_k, self.cache_v, self.new_ks, self.new_vs, clamp=True)

  def state(self):
    return self.cache_k, self.cache_v

  @classmethod
  def empty(cls, shape, device, env):
    """cache_manager.py:299-313: zeros, or uniform [0,1) when env.testing."""
    dtype = torch.bfloat16 if env.bf16_enable else torch.float32
    device = _device(device, env)
    if env.testing:
      g = torch.Generator(device="cpu").manual_seed(env.testing_seed)
      k = torch.rand(tuple(shape), generator=g).to(dtype).to(device)
      v = torch.rand(tuple(shape), generator=g).to(dtype).to(device)
    else:
      k = torch.zeros(tuple(shape), dtype=dtype, device=device)
      v = torch.zeros(tuple(shape), dtype=dtype, device=device)
    return cls(k, v, 0, None, env=env)


def _device(device, env):
  if isinstance(device, (torch.device, str)):
    return torch.device(device)
  return getattr(env, "device", torch.device("cuda"))


class Int8KVCacheGenerate:
  """Int8 decode cache with per-token scalers,
  jetstream_pt/cache_manager.py:337-657."""

  # pylint: disable=too-many-instance-attributes
  def __init__(self, cache_k, cache_v, cache_k_scaler, cache_v_scaler, input_pos, sharding=None, env=None):
    self.cache_k = cache_k
    self.cache_v = cache_v
    self.k_scaler = cache_k_scaler
    self.v_scaler = cache_v_scaler
    self.new_ks = None
    self.new_vs = None
    self.new_k_scaler = None
    self.new_v_scaler = None
    self.input_pos = input_pos
    self.sharding = sharding
    self.env = env
    self.stacked = env.generate_cache_stacked
    if env.lazy_cache_update:
      if env.generate_cache_stacked:
        layer, batch, heads, _, dim = cache_k.shape
        dev = cache_k.device
        if env.new_cache_stacked:
          self.new_ks = torch.zeros((layer, batch, heads, 1, dim), dtype=torch.int8, device=dev)
          self.new_vs = torch.zeros((layer, batch, heads, 1, dim), dtype=torch.int8, device=dev)
          self.new_k_scaler = torch.zeros((layer, batch, 1, 1, 1), dtype=env.default_type, device=dev)
          self.new_v_scaler = torch.zeros((layer, batch, 1, 1, 1), dtype=env.default_type, device=dev)
        else:
          self.new_ks, self.new_vs, self.new_k_scaler, self.new_v_scaler = [], [], [], []
      else:
        assert not env.new_cache_stacked

  def state(self):
    return self.cache_k, self.cache_v

  def scalers(self):
    return self.k_scaler, self.v_scaler

  @classmethod
  def empty(cls, shape, device, env):
    """cache_manager.py:513-530: zero codes, unit bf16 scalers."""
    device = _device(device, env)
    cache_k = torch.zeros(tuple(shape), dtype=torch.int8, device=device)
    cache_v = torch.zeros(tuple(shape), dtype=torch.int8, device=device)
    if env.generate_cache_stacked:
      s_shape = (shape[0], shape[1], 1, shape[3], 1)
    else:
      s_shape = (shape[0], 1, shape[2], 1)
    kscaler = torch.ones(s_shape, dtype=torch.bfloat16, device=device)
    vscaler = torch.ones(s_shape, dtype=torch.bfloat16, device=device)
    return cls(cache_k, cache_v, kscaler, vscaler, 0, None, env=env)

  def _quant_append(self, xk, xv, cache_k, cache_v, k_scaler, v_scaler, outs=None, amax_in=None, peers=None):
    """Quantise the new token of every slot and (when a cache view is given)
    write codes and scale at this step's position: one launch for K and V."""
    b, h, t, d = xk.shape
    if t != 1:
      raise ValueError("the decode cache takes one new token per step")
    xk, xv = xk.contiguous(), xv.contiguous()
    if outs is None:
      kq = torch.empty((b, h, 1, d), dtype=torch.int8, device=xk.device)
      vq = torch.empty((b, h, 1, d), dtype=torch.int8, device=xk.device)
      ks = torch.empty((b, 1, 1, 1), dtype=xk.dtype, device=xk.device)
      vs = torch.empty((b, 1, 1, 1), dtype=xk.dtype, device=xk.device)
    else:
      kq, vq, ks, vs = outs
      if ks.dtype != xk.dtype or vs.dtype != xk.dtype:  # the kernel writes the scale in the input's dtype
        raise ValueError(f"scale buffers of dtype {ks.dtype} cannot take the scales of {xk.dtype} inputs")
      if kq.dtype != torch.int8 or vq.dtype != torch.int8:
        raise ValueError("the buffers for the quantised new token must be int8")
    p, n, host, keep = (None, 1, 0, None)
    s = 1
    cs = (0, 0, 0)
    ss = (0, 0)
    if cache_k is not None:
      if k_scaler.dtype != xk.dtype:
        raise ValueError(f"scaler dtype {k_scaler.dtype} differs from the input dtype {xk.dtype}")
      s = cache_k.shape[2]
      _, cs_b, cs_h, cs_s = _dense_strides(cache_k)
      cs = (cs_b, cs_h, cs_s)
      ss = (k_scaler.stride(0), k_scaler.stride(2))
      p, n, host, keep = _pos_args(self.input_pos, xk.device, b)
    if peers is not None:
      if amax_in is not None:
        raise ValueError("give either the reduced amax or the peer exchange, not both")
      _lib.check(_lib.lib().jpt_kv_quant_append_dense_peers(
          _lib.ptr(xk), _lib.ptr(xv), _lib.dt(xk), _lib.ptr(cache_k), _lib.ptr(cache_v), _lib.ptr(k_scaler),
          _lib.ptr(v_scaler), _lib.ptr(kq), _lib.ptr(vq), _lib.ptr(ks), _lib.ptr(vs), p, n, host, b, h, s, d,
          cs[0], cs[1], cs[2], ss[0], ss[1], ctypes.byref(peers.struct), _lib.stream()))
    else:
      _lib.check(_lib.lib().jpt_kv_quant_append_dense(
          _lib.ptr(xk), _lib.ptr(xv), _lib.dt(xk), _lib.ptr(cache_k), _lib.ptr(cache_v), _lib.ptr(k_scaler),
          _lib.ptr(v_scaler), _lib.ptr(kq), _lib.ptr(vq), _lib.ptr(ks), _lib.ptr(vs), p, n, host, b, h, s, d,
          cs[0], cs[1], cs[2], ss[0], ss[1], _lib.ptr(amax_in), None, _lib.stream()))
    del keep
    return kq, vq, ks, vs

  def local_amax(self, xk, xv):
    """Phase one of a head-sharded update: this rank's max |x| per slot over
    its own heads, float32 [2,B] (K row, V row).  Reduce it with MAX over the
    ranks and pass the result to `update(..., amax=...)`."""
    b, h, _, d = xk.shape
    out = torch.empty((2, b), dtype=torch.float32, device=xk.device)
    xk, xv = xk.contiguous(), xv.contiguous()
    _lib.check(_lib.lib().jpt_kv_quant_append_dense(
        _lib.ptr(xk), _lib.ptr(xv), _lib.dt(xk), None, None, None, None, None, None, None, None, None, 1, 0,
        b, h, 1, d, 0, 0, 0, 0, 0, None, _lib.ptr(out), _lib.stream()))
    return out

  def quantize(self, val):
    """cache_manager.py:532-537: (codes, scale [B,1,T,1]); truncating cast."""
    b, h, t, d = val.shape
    if t == 1:
      kq, _, ks, _ = self._quant_append(val, val, None, None, None, None)
      return kq, ks
    # several tokens: one token per "slot" of the kernel
    x = val.permute(0, 2, 1, 3).reshape(b * t, h, 1, d)
    kq, _, ks, _ = self._quant_append(x, x, None, None, None, None)
    return (kq.reshape(b, t, h, d).permute(0, 2, 1, 3).contiguous(), ks.reshape(b, t, 1, 1).permute(0, 2, 1, 3))

  def update(self, xk, xv, layer_id: int, amax=None, peers=None):
    """cache_manager.py:539-582.  `amax` (float32 [2,B], optional) replaces the
    local per-token maxima when the KV heads are sharded across GPUs and the
    caller has max-reduced `local_amax` over the ranks (the reference gets the
    same effect from GSPMD's all-reduce of the amax over the sharded head axis).
    `peers` (a `PeerAmaxExchange`, optional) does that reduction inside the
    launch over NVLink peer memory instead: no `local_amax`, no collective."""
    env = self.env
    if env.lazy_cache_update:
      if env.new_cache_stacked:
        outs = (self.new_ks[layer_id], self.new_vs[layer_id], self.new_k_scaler[layer_id],
                self.new_v_scaler[layer_id])
        k_quant, v_quant, kscale, vscale = self._quant_append(xk, xv, None, None, None, None, outs, amax, peers)
      else:
        k_quant, v_quant, kscale, vscale = self._quant_append(xk, xv, None, None, None, None, None, amax, peers)
        if env.generate_cache_stacked:
          self.new_ks.append(k_quant)
          self.new_vs.append(v_quant)
          self.new_k_scaler.append(kscale)
          self.new_v_scaler.append(vscale)
        else:
          self.new_ks, self.new_vs = k_quant, v_quant
          self.new_k_scaler, self.new_v_scaler = kscale, vscale
    elif self.cache_k.ndim == 5:
      # Eager write into a stacked cache: the reference leaves this
      # combination unhandled (cache_manager.py:567); the layer's slice is
      # written here.
      k_quant, v_quant, kscale, vscale = self._quant_append(
          xk, xv, self.cache_k[layer_id], self.cache_v[layer_id], self.k_scaler[layer_id],
          self.v_scaler[layer_id], None, amax, peers)
    else:
      # ring buffer (one shared position) and left aligned (one per slot) differ
      # only in how many positions `input_pos` holds
      k_quant, v_quant, kscale, vscale = self._quant_append(
          xk, xv, self.cache_k, self.cache_v, self.k_scaler, self.v_scaler, None, amax, peers)
    return (self.cache_k, self.cache_v, k_quant, v_quant, self.k_scaler, self.v_scaler, kscale, vscale)

  def fused_step_supported(self, xq, xk):
    """True when `update_and_attend` can run as ONE launch: dense int8 cache
    (not the lazily finalised stacked stash of several layers at once), head_dim
    128, one new token, at most 8 query rows per KV head."""
    b, hq, tq, d = xq.shape
    h = xk.shape[1]
    return (d == 128 and tq == 1 and xk.shape[2] == 1 and hq % h == 0 and hq // h <= 8
            and xk.dtype in (torch.bfloat16, torch.float32) and xq.dtype == torch.bfloat16
            and self.k_scaler is not None and self.k_scaler.dtype == xk.dtype)

  def update_and_attend(self, xq, xk, xv, layer_id: int, start, end, ring=False, peers=None, out=None):
    """`update(xk, xv, layer_id)` and ragged attention of `xq` over the cache
    INCLUDING the new token, as one kernel launch.

    start, end: the valid range of the tokens already in the cache (the new
    token is not part of it): [0, end) when `ring` is false, the ring range
    [start, end) otherwise.  The new token is written at `input_pos` exactly as
    `update` does (ring buffer: the shared position; left aligned: one position
    per slot); with `env.lazy_cache_update` only the stash (`new_ks`, ...) is
    written and `finalize` moves it into the cache later, as in the reference.
    `peers` (a `PeerAmaxExchange`) shards the KV heads over GPUs; the amax
    exchange then runs inside the same launch, hidden under the attention over
    the existing tokens.  The token is attended to as the sequence's last one,
    so the range must leave room for it (end - start < cache length); a sequence
    that does not is attended to without it and `kernel_status()` reads 3.

    Returns (the 8-tuple `update` returns, (o [B,Hkv,rep,D], m, l [B,Hkv,rep])).
    Codes, scales and cache contents equal those of `update` bit for bit; the
    attention rows equal those of `update` followed by `ragged_mha` over the
    extended range within rounding (the reference pair is
    jetstream_pt/layers.py:676-718).  Falls back to those two calls for shapes
    the fused kernel does not take."""
    from jetstream_pytorch_b200 import attention_kernel as ak

    env = self.env
    if not self.fused_step_supported(xq, xk):
      r = self.update(xk, xv, layer_id, peers=peers)
      if env.lazy_cache_update:
        raise ValueError("the unfused lazy step is the caller's: attend to the cache and to the new token, then merge")
      end_all = torch.as_tensor(end).to(xq.device) + 1
      o, ml = ak.ragged_mha(xq, r[0], r[1], layer_id, start, end_all, None, None, r[4], r[5], ring=ring, out=out)
      return r, (o, ml[0], ml[1])
    b, h, _, d = xk.shape
    xk, xv = xk.contiguous(), xv.contiguous()
    lazy = env.lazy_cache_update
    stash = None
    if lazy and env.new_cache_stacked:
      stash = (self.new_ks[layer_id], self.new_vs[layer_id], self.new_k_scaler[layer_id], self.new_v_scaler[layer_id])
      if stash[2].dtype != xk.dtype:
        raise ValueError(f"scale buffers of dtype {stash[2].dtype} cannot take the scales of {xk.dtype} inputs")
    if stash is None:
      stash = (torch.empty((b, h, 1, d), dtype=torch.int8, device=xk.device),
               torch.empty((b, h, 1, d), dtype=torch.int8, device=xk.device),
               torch.empty((b, 1, 1, 1), dtype=xk.dtype, device=xk.device),
               torch.empty((b, 1, 1, 1), dtype=xk.dtype, device=xk.device))
    kq, vq, ks, vs = stash
    cache_k, cache_v, k_scaler, v_scaler = self.cache_k, self.cache_v, self.k_scaler, self.v_scaler
    if cache_k.ndim == 5:
      cache_k, cache_v, k_scaler, v_scaler = cache_k[layer_id], cache_v[layer_id], k_scaler[layer_id], v_scaler[layer_id]
    nt = _lib.NewTokenStruct()
    nt.xk, nt.xv, nt.in_dtype = _lib.ptr(xk), _lib.ptr(xv), _lib.dt(xk)
    nt.write_cache = 0 if lazy else 1
    nt.k_quant, nt.v_quant, nt.k_scale, nt.v_scale = _lib.ptr(kq), _lib.ptr(vq), _lib.ptr(ks), _lib.ptr(vs)
    p, n, host, keep = _pos_args(self.input_pos, xk.device, b)
    nt.pos, nt.pos_count, nt.pos_host = p, n, host
    if peers is not None:
      nt.px = ctypes.pointer(peers.struct)
    o, (m, l) = ak.ragged_mha(xq, cache_k, cache_v, 0, start, end, None, None, k_scaler, v_scaler, ring=ring, out=out,
                              new_token=nt)
    del keep
    if lazy:
      if not env.new_cache_stacked:
        if env.generate_cache_stacked:
          self.new_ks.append(kq)
          self.new_vs.append(vq)
          self.new_k_scaler.append(ks)
          self.new_v_scaler.append(vs)
        else:
          self.new_ks, self.new_vs, self.new_k_scaler, self.new_v_scaler = kq, vq, ks, vs
    return (self.cache_k, self.cache_v, kq, vq, self.k_scaler, self.v_scaler, ks, vs), (o, m, l)

  def finalize(self):
    """cache_manager.py:584-657."""
    env = self.env
    if not env.lazy_cache_update:
      return
    if env.ring_buffer:
      # K and V only: the reference does not write the scalers here
      # (cache_manager.py:588-597)
      b, h, s, d = self.cache_k.shape
      _scatter_rows(self.new_ks, self.new_vs, self.cache_k, self.cache_v, self.input_pos, False, 1, b, h, s, d,
                    _dense_strides(self.cache_k))
      return
    if env.generate_cache_stacked:
      nl, b, h, s, d = self.cache_k.shape
      if env.new_cache_stacked:
        new = (self.new_ks, self.new_vs, self.new_k_scaler, self.new_v_scaler)
      else:
        new = tuple(torch.stack(x) for x in (self.new_ks, self.new_vs, self.new_k_scaler, self.new_v_scaler))
    else:
      nl = 1
      b, h, s, d = self.cache_k.shape
      new = (self.new_ks, self.new_vs, self.new_k_scaler, self.new_v_scaler)
    _scatter_rows(new[0], new[1], self.cache_k, self.cache_v, self.input_pos, True, nl, b, h, s, d,
                  _dense_strides(self.cache_k))
    _scatter_rows(new[2], new[3], self.k_scaler, self.v_scaler, self.input_pos, True, nl, b, 1, s, 1,
                  _dense_strides(self.k_scaler))


class PageKVCacheGenerate:
  """Paged decode cache, jetstream_pt/cache_manager.py:660-724.  The reference
  class is bf16/fp32 only; int8 pools with scale pools [1,P,ps,1] are accepted
  here as an extension (quantise-on-append like Int8KVCacheGenerate)."""

  def __init__(self, cache_k, cache_v, page_attention_manager: PageAttentionManager, page_token_indices,
               sharding=None, env=None, k_scaler=None, v_scaler=None, n_active_dev=None):
    """`n_active_dev` (int32 device tensor [1], optional): the number of valid
    columns of `page_token_indices` when the table was computed on the device
    (`PageAttentionManager.get_page_token_indices_device`) and is B columns wide."""
    self.n_active_dev = n_active_dev
    self.cache_k = cache_k
    self.cache_v = cache_v
    self.page_attention_manager = page_attention_manager
    self.page_token_indices = page_token_indices
    self.sharding = sharding
    self.env = env
    self.stacked = False
    self.k_scaler = k_scaler
    self.v_scaler = v_scaler

  def update(self, key, value, layer_id=0):
    """cache[h, page_j, tok_j, :] = key[slot_j, h, 0, :] for every active slot
    (cache_manager.py:681-706); `layer_id` is ignored as in the reference."""
    h, p, ps, d = self.cache_k.shape
    b = key.shape[0]
    pti = _lib.as_i32(self.page_token_indices, key.device).contiguous()
    n = pti.shape[1]
    _lib.check(_lib.lib().jpt_kv_append_paged(
        _lib.ptr(key.contiguous()), _lib.ptr(value.contiguous()), _lib.dt(key), _lib.ptr(self.cache_k),
        _lib.ptr(self.cache_v), _lib.dt(self.cache_k), _lib.ptr(self.k_scaler), _lib.ptr(self.v_scaler),
        _lib.ptr(pti), n, n, _lib.ptr(self.n_active_dev), b, h, p, ps, d, _lib.stream()))
    return self.cache_k, self.cache_v

  def state(self):
    return self.cache_k, self.cache_v

  def scalers(self):
    return self.k_scaler, self.v_scaler

  def finalize(self):
    return

  @classmethod
  def empty(cls, shape, device, env):
    """cache_manager.py:717-724."""
    dtype = torch.bfloat16 if env.bf16_enable else torch.float32
    device = _device(device, env)
    k = torch.zeros(tuple(shape), dtype=dtype, device=device)
    v = torch.zeros(tuple(shape), dtype=dtype, device=device)
    return cls(k, v, None, None, None, env=env)


class PeerAmaxExchange:
  """Exchange buffers for the in-kernel max-reduction of the per-token amax
  between the GPUs of one node that hold the KV heads of a cache
  (`Int8KVCacheGenerate.update(..., peers=...)`).

  Every rank allocates one small buffer, exports its CUDA IPC handle and opens
  the handles of the others; `handles_all_gather(handle) -> [handle of rank 0,
  ...]` is any host-side all-gather of 64-byte strings
  (`PeerAmaxExchange.with_torch_distributed` uses the default process group).
  All ranks must then make the same sequence of `update` calls."""

  def __init__(self, batch_size, rank, world_size, handles_all_gather, wait_cycles=0):
    """`wait_cycles`: how long a rank waits for a peer's word, in GPU clock
    cycles (0 = the library default, about half a second)."""
    lib = _lib.lib()
    self.rank, self.world = rank, world_size
    nbytes = lib.jpt_peer_exchange_bytes(batch_size, world_size)
    if nbytes == 0:
      raise ValueError(f"peer exchange for batch {batch_size} on {world_size} ranks is not possible (1..8 ranks)")
    own = ctypes.c_void_p()
    _lib.check(lib.jpt_peer_exchange_alloc(nbytes, ctypes.byref(own)))
    self._own = own
    handle = ctypes.create_string_buffer(64)
    _lib.check(lib.jpt_peer_exchange_export(own, handle))
    handles = handles_all_gather(handle.raw)
    self.struct = _lib.PeerExchangeStruct()
    self.struct.rank, self.struct.world, self.struct.batch = rank, world_size, batch_size
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
  def with_torch_distributed(cls, batch_size):
    import torch.distributed as dist

    rank, world = dist.get_rank(), dist.get_world_size()

    def gather(h):
      out = [None] * world
      dist.all_gather_object(out, h)
      return out

    px = cls(batch_size, rank, world, gather)
    dist.barrier()  # every rank has opened every buffer before anybody launches
    return px

  def status(self):
    """0 while every wait of every launch was satisfied; 1 after a launch gave up on a peer."""
    return _lib.lib().jpt_peer_exchange_status(self._own, _lib.stream())

  def close(self):
    lib = _lib.lib()
    for p in self._opened:
      lib.jpt_peer_exchange_release(p)
    self._opened = []
    if self._own is not None:
      lib.jpt_peer_exchange_free(self._own)
      self._own = None
