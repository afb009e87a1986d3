"""Decode attention entry points with the reference's names and signatures
(jetstream_pt/attention_kernel.py), all routed to the one CUDA flash-decode
kernel family behind `jpt_flash_decode`.

Shapes follow the reference: queries [B,Hq,T,D]; dense caches [B,Hkv,S,D] or
stacked [NL,B,Hkv,S,D]; int8 scalers [B,1,S,1]; page pools [Hkv,P,ps,D].
The block-skipping tables `ragged_batch_index` / `ragged_block_index`
(jetstream_pt/engine.py:674-729) are accepted and ignored: the kernel's loop
bounds skip invalid blocks by themselves.
"""

import ctypes
import math

import numpy as np
import torch

from jetstream_pytorch_b200 import _lib

DEFAULT_MASK_VALUE = -0.7 * float(np.finfo(np.dtype("float32")).max)

_workspaces = {}  # (device, stream handle or None) -> grow-only scratch tensor


def _workspace(device, nbytes):
  """Grow-only attention scratch, allocated by torch and owned here, cleared
  once when it is created as the kernel's arrival counters require.

  Two launches that share a workspace must not overlap on the GPU, so every
  stream gets its own.  CUDA graph captures run on a stream of their own and
  must not allocate: they use one more workspace per device (key `None`) that
  every eager call keeps at least as large as its own, so a shape that ran once
  eagerly can be captured.  Graphs captured on one device share that
  workspace: replay them on one stream, or on streams ordered by events."""
  capturing = torch.cuda.is_current_stream_capturing()
  stream = torch.cuda.current_stream(device)
  keys = [(device, None)] if capturing else [(device, stream.cuda_stream), (device, None)]
  for key in keys:
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
      if capturing:
        raise RuntimeError("the attention workspace for CUDA graphs is too small and cannot grow during capture; "
                           "call the same shape once before capturing")
      ws = torch.empty(max(nbytes, 8 << 20), dtype=torch.uint8, device=device)
      _lib.check(_lib.lib().jpt_flash_decode_workspace_init(_lib.ptr(ws), ws.numel(), stream.cuda_stream))
      _workspaces[key] = ws
  return _workspaces[keys[0]]


def kernel_status(device=None):
  """0 if no attention kernel on `device` ever gave up on a bounded wait, else
  the code it recorded.  Covers every workspace this module handed out and the
  scratch built into the library (`static_scratch=True`).  A workspace whose
  status is raised is cleared again (its arrival counters may be left non-zero
  by the launch that gave up).  Synchronises (diagnostic only)."""
  lib = _lib.lib()
  worst = 0
  devices = set()
  for (dev, stream), ws in _workspaces.items():
    if device is not None and torch.device(device) != dev:
      continue
    devices.add(dev)
    with torch.cuda.device(dev):
      torch.cuda.synchronize(dev)  # launches of any stream (and graph replays) have finished
      on = stream if stream is not None else _lib.stream()
      rc = lib.jpt_flash_decode_status(_lib.ptr(ws), on)
      if rc < 0:
        _lib.check(rc)
      if rc:
        worst = worst or rc
        _lib.check(lib.jpt_flash_decode_workspace_init(_lib.ptr(ws), ws.numel(), on))
  if device is not None:
    devices.add(torch.device(device))
  elif not devices and torch.cuda.is_available():
    devices.add(torch.device("cuda", torch.cuda.current_device()))
  for dev in devices:
    with torch.cuda.device(dev):
      rc = lib.jpt_flash_decode_status(None, _lib.stream())
      if rc < 0:
        _lib.check(rc)
      worst = worst or rc
  return worst


def _flash_decode(q, k, v, *, paged=False, page_table=None, page_size=0, k_scale=None, v_scale=None,
                  scale_strides=(0, 0), mask_mode=_lib.MASK_NONE, start=None, end=None, mask=None,
                  mask_strides=(0, 0), sm_scale=1.0, kv_strides=(0, 0, 0), n_kv_heads=None, seq=None,
                  want_ml=True, num_splits=0, force_generic=False, static_scratch=False, out=None,
                  logit_rounding=False, new_token=None):
  """q [B,Hq,Tq,D] contiguous.  Returns o (q's shape and dtype), m, l float32
  [B,Hq,Tq] (or None, None).

  `new_token` (a `_lib.NewTokenStruct`, optional) routes the call through
  `jpt_decode_update_attend`: the step's new K/V token is quantised, written
  and attended to in the same launch (see `Int8KVCacheGenerate.update_and_attend`).

  `out=(o, m, l)` (m, l may be None) makes the call write into tensors the
  caller already owns instead of creating new ones: a step loop that keeps its
  buffers, or a CUDA graph whose outputs must stay at fixed addresses.

  `static_scratch=True` routes the call through `jpt_flash_decode_static`: no
  workspace tensor is created or passed, the kernels use the scratch array
  built into the library (for callers that must not allocate at this point;
  shapes needing more than its 16 MiB raise ValueError)."""
  q = q.contiguous()
  b, hq, tq, d = q.shape
  dev = q.device
  if dev.index is not None and dev.index != torch.cuda.current_device():
    # launches go to the current device's stream and kernel attributes are per device
    with torch.cuda.device(dev):
      return _flash_decode(q, k, v, paged=paged, page_table=page_table, page_size=page_size, k_scale=k_scale,
                           v_scale=v_scale, scale_strides=scale_strides, mask_mode=mask_mode, start=start, end=end,
                           mask=mask, mask_strides=mask_strides, sm_scale=sm_scale, kv_strides=kv_strides,
                           n_kv_heads=n_kv_heads, seq=seq, want_ml=want_ml, num_splits=num_splits,
                           force_generic=force_generic, static_scratch=static_scratch, out=out,
                           logit_rounding=logit_rounding, new_token=new_token)
  for t in (k, v, k_scale, v_scale, mask):
    if t is not None and t.device != dev:
      raise ValueError(f"attention operands live on {t.device} and {dev}")
  p = _lib.AttnParams()
  p.q, p.q_dtype = _lib.ptr(q), _lib.dt(q)
  p.B, p.Hq, p.Hkv, p.Tq, p.D = b, hq, n_kv_heads, tq, d
  p.k, p.v, p.kv_dtype = _lib.ptr(k), _lib.ptr(v), _lib.dt(k)
  p.paged = int(paged)
  keep = [q, k, v]
  if paged:
    page_table = _lib.as_i32(page_table, dev).contiguous()
    keep.append(page_table)
    p.page_table, p.max_pages, p.page_size = _lib.ptr(page_table), page_table.shape[1], page_size
    p.S = page_table.shape[1] * page_size
    p.kv_h, p.kv_page = k.stride(0), k.stride(1)
  else:
    p.S = seq
    p.kv_b, p.kv_h, p.kv_s = kv_strides
  if k_scale is not None:
    if k_scale.dtype != v_scale.dtype:
      raise ValueError("k and v scales must share a dtype")
    p.k_scale, p.v_scale, p.scale_dtype = _lib.ptr(k_scale), _lib.ptr(v_scale), _lib.dt(k_scale)
    p.sc_b, p.sc_s = scale_strides
    keep += [k_scale, v_scale]
  p.mask_mode = mask_mode
  if start is not None:
    start = _lib.as_i32(start, dev).contiguous()
    p.start = _lib.ptr(start)
    keep.append(start)
  if end is not None:
    end = _lib.as_i32(end, dev).contiguous()
    p.end = _lib.ptr(end)
    keep.append(end)
  if mask is not None:
    p.mask = _lib.ptr(mask)
    p.mk_b, p.mk_r = mask_strides
    keep.append(mask)
  p.sm_scale = sm_scale
  m = l = None
  if out is not None:
    o, m, l = out
    if o.shape != q.shape or o.dtype != q.dtype or o.device != dev or not o.is_contiguous():
      raise ValueError("out[0] must be a contiguous tensor of the query's shape, dtype and device")
    for t in (m, l):
      if t is not None and (t.numel() != b * hq * tq or t.dtype != torch.float32 or t.device != dev
                            or not t.is_contiguous()):
        raise ValueError("out[1], out[2] must be contiguous float32 tensors of B*Hq*Tq elements")
  else:
    o = torch.empty_like(q)
    if want_ml:
      m = torch.empty((b, hq, tq), dtype=torch.float32, device=dev)
      l = torch.empty((b, hq, tq), dtype=torch.float32, device=dev)
  p.o = _lib.ptr(o)
  if m is not None and l is not None:
    p.m, p.l = _lib.ptr(m), _lib.ptr(l)
  p.num_splits, p.force_generic = num_splits, int(force_generic)
  p.logit_rounding = int(logit_rounding)
  lib = _lib.lib()
  if static_scratch:
    if new_token is not None:
      raise ValueError("the fused update needs a workspace that keeps its contents between calls")
    _lib.check(lib.jpt_flash_decode_static(ctypes.byref(p), _lib.stream()))
  else:
    need = lib.jpt_flash_decode_workspace_bytes(ctypes.byref(p))
    if need:
      ws = _workspace(dev, need)
      p.workspace, p.workspace_bytes = _lib.ptr(ws), ws.numel()
    if new_token is not None:
      _lib.check(lib.jpt_decode_update_attend(ctypes.byref(p), ctypes.byref(new_token), _lib.stream()))
    else:
      _lib.check(lib.jpt_flash_decode(ctypes.byref(p), _lib.stream()))
  del keep
  return o, m, l


def _dense_kv(keys, values, layer):
  """Select the layer of a stacked cache; returns (k, v, strides, Hkv, S)."""
  if keys.ndim == 5:
    keys, values = keys[layer], values[layer]
  if keys.stride(-1) != 1 or values.stride() != keys.stride():
    keys, values = keys.contiguous(), values.contiguous()
  return keys, values, (keys.stride(0), keys.stride(1), keys.stride(2)), keys.shape[1], keys.shape[2]


def _dense_scales(k_scaler, v_scaler, layer):
  """Scalers [B,1,S,1] or [B,1,S] (stacked: leading NL) -> tensors + (b, s) strides."""
  if k_scaler is None:
    return None, None, (0, 0)
  if k_scaler.ndim == 5 or (k_scaler.ndim == 4 and k_scaler.shape[-1] != 1):
    k_scaler, v_scaler = k_scaler[layer], v_scaler[layer]
  if v_scaler.stride() != k_scaler.stride():
    k_scaler, v_scaler = k_scaler.contiguous(), v_scaler.contiguous()
  return k_scaler, v_scaler, (k_scaler.stride(0), k_scaler.stride(2))


def reshape_heads(xq, keys):
  """attention_kernel.py:583-590: group the query heads of each KV head."""
  bq, hq, tq, dq = xq.shape
  hkv = keys.shape[-3]
  rep = hq // hkv
  if rep > 1:
    xq = xq.reshape(bq, hkv, rep * tq, dq)
  return xq, rep


def reshape_outputs(rep, o, m=None, d=None):
  """attention_kernel.py:593-602."""
  bq, hqo, tqo, dq = o.shape
  tq = tqo // rep
  hq = hqo * rep
  o = o.reshape(bq, hq, tq, dq)
  if m is not None and d is not None:
    m = m.reshape(bq, hq, tq, 1)
    d = d.reshape(bq, hq, tq, 1)
  return o, (m, d)


def _mask_args(mask, q, s, n_kv_heads):
  """Additive mask -> (mode, tensor, (batch stride, row stride)).  The kernels
  read mask[b * mk_b + row * mk_r + s] for row in [0, rep * Tq): the batch
  extent must be 1 or B and the row extent 1 or rep * Tq, exactly what
  broadcasts against the grouped scores [B,Hkv,rep*Tq,S] in the reference
  (attention_kernel.py:611-615), which raises for anything else."""
  if mask is None:
    return _lib.MASK_NONE, None, (0, 0)
  b, hq, tq, _ = q.shape
  rows = (hq // n_kv_heads) * tq
  if mask.ndim != 4 or mask.shape[1] != 1 or mask.shape[3] != s:
    raise ValueError(f"mask must be [B|1, 1, R|1, S]; got {tuple(mask.shape)}")
  if mask.shape[0] not in (1, b) or mask.shape[2] not in (1, rows):
    raise ValueError(f"mask {tuple(mask.shape)} does not broadcast against scores [{b}, {n_kv_heads}, {rows}, {s}]")
  if mask.dtype != q.dtype:
    mask = mask.to(q.dtype)
  if mask.stride(3) != 1:
    mask = mask.contiguous()
  mk_b = mask.stride(0) if mask.shape[0] > 1 else 0
  mk_r = mask.stride(2) if mask.shape[2] > 1 else 0
  return _lib.MASK_ADD, mask, (mk_b, mk_r)


def dense_attention(xq, keys, values, k_scaler=None, v_scaler=None, mask=None, **kw):
  """attention_kernel.py:605-633: masked softmax attention over the whole cache
  row; `mask` holds 0 / -inf (or any additive values).  Returns [B,Hq,T,D]."""
  k, v, strides, hkv, s = _dense_kv(keys, values, 0)
  ks, vs, sst = _dense_scales(k_scaler, v_scaler, 0)
  mode, mask, mst = _mask_args(mask, xq, s, hkv)
  # The reference computes the logits of this function as bf16 tensor operations when its
  # inputs are bf16 (matmul, / sqrt(D), * k_scaler, + mask: four roundings); the kernels
  # reproduce those roundings so that the softmax sees the same numbers.
  o, _, _ = _flash_decode(xq, k, v, k_scale=ks, v_scale=vs, scale_strides=sst, mask_mode=mode, mask=mask,
                          mask_strides=mst, sm_scale=1.0 / math.sqrt(xq.shape[-1]), kv_strides=strides,
                          n_kv_heads=hkv, seq=s, want_ml=False, logit_rounding=xq.dtype == torch.bfloat16,
                          **kw)
  return o


def flash_attention(xq, keys, values, layer, k_scaler=None, v_scaler=None, mask=None, normalize_var=True):
  """attention_kernel.py:636-710.  Returns o [B,Hq,T,D], (m, l) [B,Hq,T,1]
  float32: the row max of the logits and the softmax denominator (the v scale
  is applied to the numerator only)."""
  k, v, strides, hkv, s = _dense_kv(keys, values, layer)
  ks, vs, sst = _dense_scales(k_scaler, v_scaler, layer)
  mode, mask, mst = _mask_args(mask, xq, s, hkv)
  sm = 1.0 / math.sqrt(k.shape[-1]) if normalize_var else 1.0
  o, m, l = _flash_decode(xq, k, v, k_scale=ks, v_scale=vs, scale_strides=sst, mask_mode=mode, mask=mask,
                          mask_strides=mst, sm_scale=sm, kv_strides=strides, n_kv_heads=hkv, seq=s)
  return o, (m.unsqueeze(-1), l.unsqueeze(-1))


def _ragged_per_head(q, k, v, layer, start, end, k_scaler, v_scaler, normalize_var, mode, **kw):
  """q [B,T,D]; k,v [B,S,D] or stacked [NL,B,S,D]; scalers [B,1,S]."""
  if k.ndim == 4:
    k, v = k[layer], v[layer]
    if k_scaler is not None and k_scaler.ndim == 4:
      k_scaler, v_scaler = k_scaler[layer], v_scaler[layer]
  if k.stride(-1) != 1 or v.stride() != k.stride():
    k, v = k.contiguous(), v.contiguous()
  sst = (0, 0)
  if k_scaler is not None:
    if v_scaler.stride() != k_scaler.stride():
      k_scaler, v_scaler = k_scaler.contiguous(), v_scaler.contiguous()
    sst = (k_scaler.stride(0), k_scaler.stride(2))
  sm = 1.0 / math.sqrt(k.shape[-1]) if normalize_var else 1.0
  o, m, l = _flash_decode(q.unsqueeze(1), k, v, k_scale=k_scaler, v_scale=v_scaler, scale_strides=sst,
                          mask_mode=mode, start=start, end=end, sm_scale=sm,
                          kv_strides=(k.stride(0), 0, k.stride(1)), n_kv_heads=1, seq=k.shape[1], **kw)
  return o.squeeze(1), (m.squeeze(1), l.squeeze(1))


def ragged_mqa(q, k, v, layer, start, end, ragged_batch_index=None, ragged_block_index=None, k_scaler=None,
               v_scaler=None, bk=512, mask_value=DEFAULT_MASK_VALUE, normalize_var=True, testing=False,
               quantized=False, **kw):
  """Ragged multi query attention over a ring-buffer cache,
  attention_kernel.py:122-252 with the kernel body at 22-109: valid positions
  are [start, end), or [start, S) U [0, end) when start > end; start == end
  means an empty row.  q [B,T,D]; k,v [B,S,D]; scalers [B,1,S].
  Returns out [B,T,D], (m, l) [B,T]."""
  del ragged_batch_index, ragged_block_index, bk, mask_value, testing, quantized
  return _ragged_per_head(q, k, v, layer, start, end, k_scaler, v_scaler, normalize_var, _lib.MASK_RING, **kw)


def ragged_mqa_reference(q, k, v, layer, start, end, ragged_batch_index=None, ragged_block_index=None,
                         k_scaler=None, v_scaler=None, bk=512, mask_value=DEFAULT_MASK_VALUE,
                         normalize_var=True, testing=False, quantized=False, **kw):
  """Left-aligned ragged multi query attention, attention_kernel.py:342-466
  with the kernel body at 255-329: valid positions are [0, end); `start` is
  ignored."""
  del start, ragged_batch_index, ragged_block_index, bk, mask_value, testing, quantized
  return _ragged_per_head(q, k, v, layer, None, end, k_scaler, v_scaler, normalize_var, _lib.MASK_LENGTH, **kw)


def ragged_mha(q, k, v, layer, start, end, ragged_batch_index=None, ragged_block_index=None, k_scaler=None,
               v_scaler=None, bk=512, mask_value=DEFAULT_MASK_VALUE, normalize_var=True, q_shard_axis=0,
               kv_shard_axis=0, testing=False, ring=False, **kw):
  """Ragged multi head attention, attention_kernel.py:480-580.

  q [B,Hq,T,D]; k,v [B,Hkv,S,D] or stacked [NL,B,Hkv,S,D]; scalers [B,1,S,1]
  (stacked: [NL,B,1,S,1]) or None.  Returns out [B,Hkv,rep*T,D] and (m, l)
  [B,Hkv,rep*T].  Like the reference (which maps `ragged_mqa_reference` over
  the heads, attention_kernel.py:561-579) the valid range is [0, end);
  `ring=True` selects the [start, end) ring semantics of `ragged_mqa` instead.
  """
  del ragged_batch_index, ragged_block_index, bk, mask_value, q_shard_axis, kv_shard_axis, testing
  assert k.shape[-1] == q.shape[-1]
  assert k.shape[-4] == q.shape[-4]
  kk, vv, strides, hkv, s = _dense_kv(k, v, layer)
  ks, vs, sst = _dense_scales(k_scaler, v_scaler, layer)
  if ks is not None:
    assert ks.shape[0] == q.shape[0] and ks.shape[2] == s
  bq, hq, tq, dq = q.shape
  sm = 1.0 / math.sqrt(dq) if normalize_var else 1.0
  mode = _lib.MASK_RING if ring else _lib.MASK_LENGTH
  o, m, l = _flash_decode(q, kk, vv, k_scale=ks, v_scale=vs, scale_strides=sst, mask_mode=mode,
                          start=start if ring else None, end=end, sm_scale=sm, kv_strides=strides,
                          n_kv_heads=hkv, seq=s, **kw)
  rt = (hq // hkv) * tq
  if m is None:  # out=(o, None, None): the caller does not want the softmax statistics
    return o.reshape(bq, hkv, rt, dq), (None, None)
  return o.reshape(bq, hkv, rt, dq), (m.reshape(bq, hkv, rt), l.reshape(bq, hkv, rt))


class RaggedAttentionKernel:
  """attention_kernel.py:713-759.  The shard_map / jit wrapping of the
  reference disappears: each rank calls the kernel on its own KV heads."""

  def __init__(self, env, input_specs=None, output_specs=None, q_shard_axis=0, kv_shard_axis=0):
    self.env = env
    self.bk = env.block_size

  def __call__(self, xq, keys, values, layer, start, end, ragged_batch_index=None, ragged_block_index=None,
               k_scaler=None, v_scaler=None):
    return ragged_mha(xq, keys, values, layer, start, end, ragged_batch_index, ragged_block_index, k_scaler,
                      v_scaler, bk=self.bk)


def shard_kv_heads(paged_attention_impl, mesh=None, kv_head_mesh_axis_name="x"):
  """attention_kernel.py:762-786: with one process per GPU each rank already
  holds its own KV heads, so the wrapper is the identity."""
  return paged_attention_impl


def call_paged_attention(env, xq, keys, values, seq_lens, page_indices, sm_scale=None, k_scaler=None,
                         v_scaler=None, **kw):
  """Paged decode attention, attention_kernel.py:789-808.  xq [B,Hq,D]; page
  pools [Hkv,P,ps,D]; seq_lens int [B]; page_indices int [B,max_pages] (numpy
  or tensor).  Returns [B,Hq,D].

  The reference delegates to JAX's Pallas paged-attention kernel and passes q
  unscaled; whether that kernel divides by sqrt(D) cannot be read from the
  reference, whose own dense equivalent (tests/test_attention_kernal.py:
  101-113) does.  `sm_scale` therefore defaults to 1/sqrt(D) and can be set to
  1.0.  int8 pools take scale pools [1,P,ps,1] (extension)."""
  del env
  hkv, _, ps, d = keys.shape
  if sm_scale is None:
    sm_scale = 1.0 / math.sqrt(d)
  o, _, _ = _flash_decode(xq.unsqueeze(2), keys, values, paged=True, page_table=page_indices, page_size=ps,
                          k_scale=k_scaler, v_scale=v_scaler, mask_mode=_lib.MASK_LENGTH, end=seq_lens,
                          sm_scale=sm_scale, n_kv_heads=hkv, want_ml=False, **kw)
  return o.squeeze(2)


def merge_partials(o1, m1, l1, o2, m2, l2, out_dtype=None):
  """The "attn_global" merge of jetstream_pt/layers.py:539-550 / 708-718 for
  two softmax partials.  o [..,D]; m, l [..,1] float32."""
  o1, o2 = o1.contiguous(), o2.contiguous()
  m1, l1, m2, l2 = (t.contiguous().float() for t in (m1, l1, m2, l2))
  d = o1.shape[-1]
  rows = o1.numel() // d
  out_dtype = out_dtype or torch.float32
  out = torch.empty(o1.shape, dtype=out_dtype, device=o1.device)
  _lib.check(_lib.lib().jpt_merge_partials(_lib.ptr(o1), _lib.ptr(m1), _lib.ptr(l1), _lib.ptr(o2), _lib.ptr(m2),
                                          _lib.ptr(l2), _lib.dt(o1), _lib.ptr(out), _lib.dt(out_dtype), rows, d,
                                          _lib.stream()))
  return out
