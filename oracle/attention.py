"""Oracle (test infrastructure): decode attention of the reference on torch CPU.

`dense_attention` / `flash_attention` repeat the torch op sequence of
jetstream_pt/attention_kernel.py:583-710 (pinned by golden vectors).  The two
ragged functions restate the bodies of the Pallas-TPU kernels
(attention_kernel.py:22-109 and 255-329) block by block, including the
per-block re-normalisation and rounding of `o` to the query dtype (unpinned: the
kernels cannot be executed without JAX).  `paged_attention` is the dense
equivalent that tests/test_attention_kernal.py:101-113,159-189 builds for the
third-party paged kernel (unpinned).
"""

import math

import numpy as np
import torch

DEFAULT_MASK_VALUE = -0.7 * float(np.finfo(np.float32).max)


def group_heads(xq, n_kv_heads):
  """`reshape_heads`, attention_kernel.py:583-590: [B,Hq,T,D] ->
  [B,Hkv,rep*T,D] (query heads of one KV group become rows)."""
  b, hq, t, d = xq.shape
  rep = hq // n_kv_heads
  return xq.reshape(b, n_kv_heads, rep * t, d), rep


def ungroup_heads(rep, o, m=None, l=None):
  """`reshape_outputs`, attention_kernel.py:593-602."""
  b, hkv, rt, d = o.shape
  t = rt // rep
  o = o.reshape(b, hkv * rep, t, d)
  if m is not None:
    m = m.reshape(b, hkv * rep, t, 1)
    l = l.reshape(b, hkv * rep, t, 1)
  return o, (m, l)


def dense_attention(xq, keys, values, k_scaler=None, v_scaler=None, mask=None):
  """attention_kernel.py:605-633.  Every intermediate lives in xq's dtype
  except the softmax, which is fp32 and cast back.  int8 keys/values are
  converted to xq's dtype first (exact)."""
  hkv = keys.shape[-3]
  q, rep = group_heads(xq, hkv)
  bsz, _, _, d = q.shape
  s = keys.shape[2]
  kf, vf = keys.to(q.dtype), values.to(q.dtype)
  scores = torch.matmul(q, kf.transpose(-1, -2)) / math.sqrt(d)
  if k_scaler is not None:
    scores = scores * k_scaler.reshape(bsz, 1, 1, s)
  if mask is not None:
    scores = scores + mask
  scores = torch.softmax(scores.float(), dim=-1).to(q.dtype)
  if v_scaler is not None:
    scores = scores * v_scaler.reshape(bsz, 1, 1, s)
  out = torch.matmul(scores, vf)
  return ungroup_heads(rep, out)[0]


def flash_attention(xq, keys, values, layer=0, k_scaler=None, v_scaler=None,
                    mask=None, normalize_var=True):
  """attention_kernel.py:636-710: fp32 logits, the v scale applied after the
  denominator is taken, (u * v_scale) rounded to xq's dtype before the PV
  product.  Returns o [B,Hq,T,D], (m, l) [B,Hq,T,1]."""
  if keys.ndim == 5:
    keys, values = keys[layer], values[layer]
    k_scaler = k_scaler[layer] if k_scaler is not None else None
    v_scaler = v_scaler[layer] if v_scaler is not None else None
  hkv = keys.shape[-3]
  q, rep = group_heads(xq, hkv)
  logits = torch.matmul(q.float(), keys.float().transpose(-1, -2))
  if normalize_var:
    logits = logits / math.sqrt(keys.shape[-1])
  if k_scaler is not None:
    logits = logits * k_scaler.reshape(k_scaler.shape[-4], 1, 1, k_scaler.shape[-2])
  if mask is not None:
    logits = logits + mask
  m = logits.max(dim=-1, keepdim=True).values
  u = torch.exp(logits - m)
  l = u.sum(dim=-1, keepdim=True)
  if v_scaler is not None:
    u = u * v_scaler.reshape(v_scaler.shape[-4], 1, 1, v_scaler.shape[-2])
  o = torch.matmul(u.to(q.dtype), values.to(q.dtype)) / l
  return ungroup_heads(rep, o, m, l)


def _ragged_blocks(q, k, v, start, end, k_scale, v_scale, bk, wrap,
                   mask_value=DEFAULT_MASK_VALUE, normalize_var=True):
  """One (batch-vectorised) KV head.  q [B,R,D]; k,v [B,S,D]; k_scale,
  v_scale [B,S] or None; start,end int [B].  Returns o [B,R,D] (q dtype),
  m,l [B,R] fp32."""
  b, r, d = q.shape
  s = k.shape[1]
  o = torch.zeros_like(q)
  m = torch.full((b, r), -float("inf"), dtype=torch.float32)
  l = torch.zeros((b, r), dtype=torch.float32)
  qf = q.float()
  quantized = k_scale is not None
  iota = torch.arange(bk)
  for bb in range(b):
    st, en = int(start[bb]), int(end[bb])
    if wrap:
      length = en if st < en else s - 1  # line_end, attention_kernel.py:189
    else:
      length = en  # left aligned, attention_kernel.py:287
    for i in range(s // bk):
      if not i * bk < length:
        continue
      if wrap and st == en:  # attention_kernel.py:57
        continue
      kb = k[bb, i * bk:(i + 1) * bk].float()
      vb = v[bb, i * bk:(i + 1) * bk].float()
      qk = qf[bb] @ kb.T
      if normalize_var:
        qk = qk / math.sqrt(d)
      if quantized:
        qk = qk * k_scale[bb, i * bk:(i + 1) * bk].float()[None, :]
      pos = i * bk + iota
      if wrap:
        if st <= en:
          valid = (pos >= st) & (pos < en)
        else:
          valid = (pos >= st) | (pos < en)
      else:
        valid = pos < length
      qk = qk + torch.where(valid, 0.0, mask_value)[None, :]
      m_curr = qk.max(dim=-1).values
      s_curr = torch.exp(qk - m_curr[:, None])
      l_curr = s_curr.sum(dim=-1)
      if quantized:
        s_curr = s_curr * v_scale[bb, i * bk:(i + 1) * bk].float()[None, :]
      o_curr = s_curr @ vb
      m_prev, l_prev = m[bb].clone(), l[bb].clone()
      m_next = torch.maximum(m_prev, m_curr)
      alpha = torch.exp(m_prev - m_next)
      beta = torch.exp(m_curr - m_next)
      l_next = alpha * l_prev + beta * l_curr
      l_safe = torch.where(l_next == 0.0, torch.ones_like(l_next), l_next)
      m[bb], l[bb] = m_next, l_safe
      o[bb] = (((l_prev * alpha)[:, None] * o[bb].float() + beta[:, None] * o_curr)
               / l_safe[:, None]).to(q.dtype)
  return o, m, l


def ragged_mha(q, k, v, layer, start, end, k_scaler=None, v_scaler=None, bk=512,
               wrap=False, normalize_var=True):
  """`ragged_mha`, attention_kernel.py:480-580: group the query heads, use unit
  scales when unquantised, run the per-head kernel over the KV-head axis.
  `wrap=False` is the live left-aligned kernel (`ragged_mqa_reference`, valid
  positions [0, end)); `wrap=True` is the ring kernel body of `ragged_mqa`
  (valid [start,end), or [start,S) U [0,end) when start > end; start == end is
  empty).  q [B,Hq,T,D]; k,v [B,Hkv,S,D] or stacked [NL,B,Hkv,S,D];
  scalers [B,1,S,1] (or stacked).  Returns o [B,Hkv,rep*T,D], (m,l)
  [B,Hkv,rep*T]."""
  if k.ndim == 5:
    k, v = k[layer], v[layer]
    if k_scaler is not None:
      k_scaler, v_scaler = k_scaler[layer], v_scaler[layer]
  bk = min(bk, k.shape[-2])
  hkv = k.shape[-3]
  qg, _ = group_heads(q, hkv)
  ks = vs = None
  if k_scaler is not None:
    ks = k_scaler.reshape(k_scaler.shape[0], -1)
    vs = v_scaler.reshape(v_scaler.shape[0], -1)
  outs, ms, ls = [], [], []
  for h in range(hkv):
    o, m, l = _ragged_blocks(qg[:, h], k[:, h], v[:, h], start, end, ks, vs, bk,
                             wrap, normalize_var=normalize_var)
    outs.append(o)
    ms.append(m)
    ls.append(l)
  return torch.stack(outs, 1), (torch.stack(ms, 1), torch.stack(ls, 1))


def paged_attention(xq, k_pages, v_pages, lengths, page_indices, sm_scale=None,
                    k_scale_pages=None, v_scale_pages=None):
  """Dense equivalent of the paged decode kernel
  (tests/test_attention_kernal.py:101-113,159-189): gather each sequence's
  pages, mask positions >= length, softmax in fp32.  xq [B,Hq,D]; pages
  [Hkv,P,ps,D]; lengths int [B]; page_indices int [B,max_pages].  The int8
  scale pools [1,P,ps,1] are this project's extension (the reference has no
  int8 paged cache).  Returns [B,Hq,D] in xq's dtype; a length of 0 gives 0."""
  b, hq, d = xq.shape
  hkv, _, ps, _ = k_pages.shape
  rep = hq // hkv
  if sm_scale is None:
    sm_scale = 1.0 / math.sqrt(d)
  out = torch.zeros_like(xq)
  for bb in range(b):
    n = int(lengths[bb])
    if n == 0:
      continue
    npg = -(-n // ps)
    idx = torch.as_tensor(np.asarray(page_indices[bb][:npg])).to(torch.int64)
    kk = k_pages[:, idx].reshape(hkv, npg * ps, d)[:, :n].float()
    vv = v_pages[:, idx].reshape(hkv, npg * ps, d)[:, :n].float()
    q = xq[bb].reshape(hkv, rep, d).float()
    logits = torch.matmul(q, kk.transpose(-1, -2)) * sm_scale
    if k_scale_pages is not None:
      ksc = k_scale_pages[0, idx].reshape(npg * ps)[:n].float()
      logits = logits * ksc[None, None, :]
    p = torch.softmax(logits, dim=-1)
    if v_scale_pages is not None:
      vsc = v_scale_pages[0, idx].reshape(npg * ps)[:n].float()
      p = p * vsc[None, None, :]
    out[bb] = torch.matmul(p, vv).reshape(hq, d).to(xq.dtype)
  return out


def merge_partials(o1, m1, l1, o2, m2, l2):
  """The two-partial merge of `AttentionKernel.__call__` /
  `Int8KVAttentionKernel.__call__`, jetstream_pt/layers.py:539-550, 708-718."""
  g = torch.max(m1, m2)
  alpha = torch.exp(m1 - g)
  beta = torch.exp(m2 - g)
  denom = alpha * l1 + beta * l2
  return (l1 * alpha * o1 + beta * o2 * l2) / denom
