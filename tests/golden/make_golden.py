"""Generates the golden fixtures in this directory by EXECUTING THE REFERENCE'S
OWN MODULES (cache_manager.py, page_attention_manager.py, attention_kernel.py,
quantize.py), imported unmodified from a reference checkout.

    python tests/golden/make_golden.py /path/to/jetstream-pytorch

The reference needs jax and torch_xla2 only for array plumbing on this path
(the arithmetic is torch / numpy), so `_refshim.py` supplies torch-backed
stand-ins for those packages, including a sequential grid interpreter for
`pallas_call` on which the reference's ragged-attention kernel bodies run as
written, and placeholder modules that let `engine.py` import so that its insert
functions can run.  The third-party JAX paged-attention kernel is not in the
reference checkout and has no fixture.
Inputs are drawn from torch generators with fixed seeds and stored with the
outputs, so the tests never need the reference.
"""

import os
import sys
import types

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import _refshim  # noqa: E402
import golden_inputs  # noqa: E402
from golden_io import save  # noqa: E402


def make_env(**kw):
  base = dict(
      batch_size=4, num_layers=3, cache_len=16, block_size=8,
      ring_buffer=True, lazy_cache_update=False, ragged_mha=False,
      flash_attention=False, generate_cache_stacked=False,
      new_cache_stacked=False, page_attention=False, testing=False,
      bf16_enable=True, default_type=torch.bfloat16, shard_on_batch=False,
      cache_sharding_axis=1, mesh=None, cache_sharding=None,
      partition_by_axis=lambda *a: None,
  )
  base.update(kw)
  return types.SimpleNamespace(**base)


def randn(gen, *shape, dtype=torch.bfloat16, scale=1.0):
  return (torch.randn(*shape, generator=gen) * scale).to(dtype)


def plain(t):
  return t.detach().as_subclass(torch.Tensor).clone()


def gen_quantizers(cm, q):
  g = torch.Generator().manual_seed(1)
  out = {}
  for tag, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
    w = randn(g, 1, 4, 24, 32, dtype=dt)
    w[0, :, 3, :] = 0  # all-zero token: EPS clamp on insert, 0/0 on decode
    w[0, :, 5, :] = (torch.randint(-5, 6, (4, 32), generator=g) * 0.5).to(dt)
    w[0, :, 7, :] *= 1e-6
    w[0, :, 9, :] *= 300.0
    codes, scale, _ = q.quantize_tensor(w, (-3, -1))
    wt = w[0].permute(1, 0, 2).contiguous()
    codes_t, scale_t, _ = q.quantize_tensor(wt, (1, 2))
    out[f"insert_in_{tag}"] = w
    out[f"insert_codes_{tag}"] = plain(codes)
    out[f"insert_scale_{tag}"] = plain(scale)
    out[f"insert_codes_t_{tag}"] = plain(codes_t)
    out[f"insert_scale_t_{tag}"] = plain(scale_t)
    x = w[0].permute(1, 0, 2).reshape(24, 4, 1, 32).contiguous()  # 24 "slots"
    dc, ds = cm.Int8KVCacheGenerate.quantize(None, x)
    out[f"decode_in_{tag}"] = x
    out[f"decode_codes_{tag}"] = plain(dc)
    out[f"decode_scale_{tag}"] = plain(ds)
  save("quantizers", out)


def gen_int8_cache(cm):
  g = torch.Generator().manual_seed(2)
  out = {}
  b, h, s, d, nl = 4, 2, 16, 8, 3
  xk = randn(g, b, h, 1, d)
  xv = randn(g, b, h, 1, d)
  out["xk"], out["xv"] = xk, xv

  def start_state(stacked):
    shape = (nl, b, h, s, d) if stacked else (b, h, s, d)
    sshape = (nl, b, 1, s, 1) if stacked else (b, 1, s, 1)
    ck = torch.randint(-127, 128, shape, generator=g).to(torch.int8)
    cv = torch.randint(-127, 128, shape, generator=g).to(torch.int8)
    ks = (torch.rand(sshape, generator=g) + 0.01).to(torch.bfloat16)
    vs = (torch.rand(sshape, generator=g) + 0.01).to(torch.bfloat16)
    return ck, cv, ks, vs

  # ring buffer, one shared position (cache_manager.py:561-565)
  ck, cv, ks, vs = start_state(False)
  for n, t in zip(("ck", "cv", "ks", "vs"), (ck, cv, ks, vs)):
    out[f"ring_in_{n}"] = t.clone()
  env = make_env(batch_size=b, ring_buffer=True)
  c = cm.Int8KVCacheGenerate(ck.clone(), cv.clone(), ks.clone(), vs.clone(), [5], env=env)
  r = c.update(xk, xv, 1)
  for n, t in zip(("ck", "cv", "kq", "vq", "ks", "vs", "kscale", "vscale"), r):
    out[f"ring_out_{n}"] = plain(t)

  # left aligned, eager per-slot write (cache_manager.py:566-571)
  pos = torch.tensor([3, 0, 15, 7])
  out["slot_pos"] = pos
  env = make_env(batch_size=b, ring_buffer=False)
  c = cm.Int8KVCacheGenerate(ck.clone(), cv.clone(), ks.clone(), vs.clone(), pos, env=env)
  r = c.update(xk, xv, 1)
  for n, t in zip(("ck", "cv", "kq", "vq", "ks", "vs", "kscale", "vscale"), r):
    out[f"slot_out_{n}"] = plain(t)

  # left aligned, lazy, stacked cache and stacked new entries, then finalize
  # (cache_manager.py:544-549, 584-620, 422-503)
  ck, cv, ks, vs = start_state(True)
  for n, t in zip(("ck", "cv", "ks", "vs"), (ck, cv, ks, vs)):
    out[f"lazy_in_{n}"] = t.clone()
  env = make_env(batch_size=b, ring_buffer=False, lazy_cache_update=True,
                 generate_cache_stacked=True, new_cache_stacked=True, num_layers=nl)
  c = cm.Int8KVCacheGenerate(ck.clone(), cv.clone(), ks.clone(), vs.clone(), pos, env=env)
  xs = []
  for layer in range(nl):
    lk, lv = randn(g, b, h, 1, d), randn(g, b, h, 1, d)
    xs.append((lk, lv))
    c.update(lk, lv, layer)
  out["lazy_xk"] = torch.stack([a for a, _ in xs])
  out["lazy_xv"] = torch.stack([a for _, a in xs])
  c.finalize()
  for n, t in zip(("ck", "cv", "ks", "vs"), (c.cache_k, c.cache_v, c.k_scaler, c.v_scaler)):
    out[f"lazy_out_{n}"] = plain(t)
  out["lazy_new_ks"] = plain(c.new_ks)
  out["lazy_new_k_scaler"] = plain(c.new_k_scaler)
  save("int8_cache", out)


def gen_float_cache(cm):
  g = torch.Generator().manual_seed(3)
  out = {}
  b, h, s, d, nl = 4, 2, 16, 8, 3
  xk, xv = randn(g, b, h, 1, d), randn(g, b, h, 1, d)
  out["xk"], out["xv"] = xk, xv
  ck, cv = randn(g, b, h, s, d), randn(g, b, h, s, d)
  out["in_ck"], out["in_cv"] = ck.clone(), cv.clone()
  pos = torch.tensor([3, 0, 15, 7])
  out["slot_pos"] = pos
  W = _refshim.JTensor.wrap

  env = make_env(batch_size=b, ring_buffer=True)
  c = cm.KVCacheGenerate(W(ck.clone()), W(cv.clone()), [5], None, env=env)
  rk, rv = c.update(W(xk), W(xv), 0)
  out["ring_out_ck"], out["ring_out_cv"] = plain(rk), plain(rv)

  env = make_env(batch_size=b, ring_buffer=False)
  c = cm.KVCacheGenerate(W(ck.clone()), W(cv.clone()), W(pos), None, env=env)
  rk, rv = c.update(W(xk), W(xv), 0)
  out["slot_out_ck"], out["slot_out_cv"] = plain(rk), plain(rv)

  sk, sv = randn(g, nl, b, h, s, d), randn(g, nl, b, h, s, d)
  out["stk_in_ck"], out["stk_in_cv"] = sk.clone(), sv.clone()
  env = make_env(batch_size=b, ring_buffer=False, generate_cache_stacked=True, num_layers=nl)
  c = cm.KVCacheGenerate(W(sk.clone()), W(sv.clone()), W(pos), None, env=env)
  c.update(W(xk), W(xv), 2)
  out["stk_out_ck"], out["stk_out_cv"] = plain(c.cache_k), plain(c.cache_v)

  env = make_env(batch_size=b, ring_buffer=False, lazy_cache_update=True,
                 generate_cache_stacked=True, new_cache_stacked=True, num_layers=nl)
  c = cm.KVCacheGenerate(W(sk.clone()), W(sv.clone()), W(pos), None, env=env)
  xs = [(randn(g, b, h, 1, d), randn(g, b, h, 1, d)) for _ in range(nl)]
  for layer, (lk, lv) in enumerate(xs):
    c.update(W(lk), W(lv), layer)
  c.finalize()
  out["lazy_xk"] = torch.stack([a for a, _ in xs])
  out["lazy_xv"] = torch.stack([a for _, a in xs])
  out["lazy_out_ck"], out["lazy_out_cv"] = plain(c.cache_k), plain(c.cache_v)
  save("float_cache", out)


def gen_pages(cm, pam_mod):
  g = torch.Generator().manual_seed(4)
  out = {}
  b, p, ps, maxp, h, d = 6, 40, 4, 6, 2, 8
  pam = pam_mod.PageAttentionManager(b, p, ps, maxp)
  ck = randn(g, h, p, ps, d)
  cv = randn(g, h, p, ps, d)
  out["in_ck"], out["in_cv"] = ck.clone(), cv.clone()
  W = _refshim.JTensor.wrap
  caches = [(W(ck.clone()), W(cv.clone()))]
  inserts = [(2, 5), (0, 8), (5, 13), (3, 1)]  # (slot, prefix length)
  out["inserts"] = np.asarray(inserts)
  for i, (slot, length) in enumerate(inserts):
    pk, pv = randn(g, 1, h, length, d), randn(g, 1, h, length, d)
    out[f"prefix_k{i}"], out[f"prefix_v{i}"] = pk, pv
    n, idx = pam.reserve_pages_insert(slot, length)
    out[f"insert_pages{i}"] = np.asarray(idx).copy()
    tep = W(torch.zeros((h, n * ps, d), dtype=torch.bfloat16))
    caches = pam.insert_prefill_cache([(W(pk), W(pv))], caches, W(torch.as_tensor(np.asarray(idx)).long()), tep, None)
  out["after_insert_ck"], out["after_insert_cv"] = plain(caches[0][0]), plain(caches[0][1])
  out["after_insert_page_indices"] = pam.page_indices.copy()
  lens = np.asarray([8, 0, 5, 1, 0, 13])
  # three decode steps: table growth on page boundaries, row appends
  env = make_env(batch_size=b, page_attention=True)
  k, v = caches[0]
  for step in range(3):
    pam.fill_new_pages(lens)
    pti = pam.get_page_token_indices(lens)
    out[f"step{step}_lens"] = lens.copy()
    out[f"step{step}_pti"] = pti.copy()
    out[f"step{step}_page_indices"] = pam.page_indices.copy()
    out[f"step{step}_lengths"] = np.asarray(pam.lengths).copy()
    xk, xv = randn(g, b, h, 1, d), randn(g, b, h, 1, d)
    out[f"step{step}_xk"], out[f"step{step}_xv"] = xk, xv
    c = cm.PageKVCacheGenerate(k, v, pam, W(torch.as_tensor(pti)), None, env=env)
    k, v = c.update(W(xk), W(xv))
    out[f"step{step}_ck"], out[f"step{step}_cv"] = plain(k), plain(v)
    lens = np.where(lens == 0, 0, lens + 1)
  comp = pam.get_compress_kv_cache([(k, v)], 5)
  out["compress_slot5_k"] = plain(comp[0][0])
  save("pages", out)


def gen_attention(ak, q):
  g = torch.Generator().manual_seed(5)
  out = {}
  b, hq, hkv, s, d = 3, 8, 2, 40, 16
  for tag, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
    for tq in (1, 2):
      xq = randn(g, b, hq, tq, d, dtype=dt)
      kf, vf = randn(g, b, hkv, s, d, dtype=dt), randn(g, b, hkv, s, d, dtype=dt)
      lens = [40, 17, 1]
      mask = torch.full((b, 1, 1, s), float("-inf"))
      for i, n in enumerate(lens):
        mask[i, :, :, :n] = 0
      mask = mask.to(dt)
      kq, ks, _ = q.quantize_tensor(kf, (-3, -1))
      vq, vs, _ = q.quantize_tensor(vf, (-3, -1))
      kq, vq, ks, vs = plain(kq), plain(vq), plain(ks), plain(vs)
      pre = f"{tag}_t{tq}_"
      out[pre + "xq"], out[pre + "k"], out[pre + "v"] = xq, kf, vf
      out[pre + "mask"] = mask
      out[pre + "kq"], out[pre + "vq"], out[pre + "ks"], out[pre + "vs"] = kq, vq, ks, vs
      out[pre + "dense_float"] = plain(ak.dense_attention(xq, kf, vf, None, None, mask))
      # int8 codes enter the einsum converted to the query dtype (exact);
      # torch_xla2 promotes the same way, plain torch CPU refuses mixed dtypes.
      out[pre + "dense_int8"] = plain(
          ak.dense_attention(xq, kq.to(dt), vq.to(dt), ks, vs, mask))
      o, (m, l) = ak.flash_attention(xq, kf, vf, 0, None, None, mask)
      out[pre + "flash_float_o"], out[pre + "flash_float_m"], out[pre + "flash_float_l"] = (
          plain(o), plain(m), plain(l))
      o, (m, l) = ak.flash_attention(xq, kq.to(dt), vq.to(dt), 0, ks, vs, mask)
      out[pre + "flash_int8_o"], out[pre + "flash_int8_m"], out[pre + "flash_int8_l"] = (
          plain(o), plain(m), plain(l))
  save("attention", out)


def gen_ragged(ak):
  """`ragged_mha` (which maps `ragged_mqa_reference` over the KV heads with
  jax.vmap and runs the kernel body of attention_kernel.py:255-329 through
  pallas_call) for the left-aligned cases; the ring-buffer kernel body
  `ragged_flash_attention_kernel` (attention_kernel.py:22-109) for the ring
  cases.  The ring wrapper `ragged_mqa` passes its kernel one operand too few
  in this snapshot (attention_kernel.py:207-218 omits `layer`), so the body is
  driven here by a pallas_call over the same (batch, S // bk) grid with plain
  block index maps, one KV head at a time as `ragged_mha` would."""
  import functools
  from jax.experimental import pallas as pl
  from jax.experimental.pallas import tpu as pltpu
  W = _refshim.JTensor.wrap
  out = {}
  for name in golden_inputs.RAGGED_CASES:
    x = golden_inputs.ragged_inputs(name)
    out[name + "_checksum"] = np.int64(golden_inputs.checksum(x))
    q, k, v, ks, vs = x["q"], x["k"], x["v"], x["ks"], x["vs"]
    stacked = k.ndim == 5
    if not x["ring"]:
      o, (m, l) = ak.ragged_mha(
          W(q), W(k), W(v), x["layer"], W(x["start"]), W(x["end"]), None, None,
          None if ks is None else W(ks), None if vs is None else W(vs), bk=x["bk"],
          q_shard_axis=1, kv_shard_axis=2 if stacked else 1, testing=True)
    else:
      b, hq, t, d = q.shape
      hkv, s = k.shape[1], k.shape[2]
      rep = hq // hkv
      qg = q.reshape(b, hkv, rep * t, d)
      bk = min(x["bk"], s)
      quantized = ks is not None
      ksq = (ks if quantized else torch.ones(b, 1, s, 1, dtype=torch.bfloat16)).squeeze(-1)
      vsq = (vs if quantized else torch.ones(b, 1, s, 1, dtype=torch.bfloat16)).squeeze(-1)
      start, end = x["start"], x["end"]
      line_end = torch.where(start < end, end, torch.full_like(end, s - 1))  # attention_kernel.py:189
      body = functools.partial(ak.ragged_flash_attention_kernel, bk=bk, mask_value=ak.DEFAULT_MASK_VALUE,
                               normalize_var=True, quantized=quantized)
      row = pl.BlockSpec(index_map=lambda bb, i, *_: (bb, 0, 0), block_shape=(None, rep * t, d))
      blk = pl.BlockSpec(index_map=lambda bb, i, *_: (bb, i, 0), block_shape=(None, bk, d))
      sc = pl.BlockSpec(index_map=lambda bb, i, *_: (bb, 0, i), block_shape=(None, 1, bk))
      os_, ms_, ls_ = [], [], []
      for h in range(hkv):
        qh = qg[:, h].contiguous()
        res = pl.pallas_call(
            body,
            grid_spec=pltpu.PrefetchScalarGridSpec(
                num_scalar_prefetch=6, in_specs=[row, blk, blk, sc, sc], out_specs=[row, row, row],
                grid=(b, s // bk)),
            out_shape=[qh, _refshim.ShapeDtypeStruct((b, rep * t, d), torch.float32),
                       _refshim.ShapeDtypeStruct((b, rep * t, d), torch.float32)],
        )(torch.tensor([0]), start, end, line_end, None, None, qh, k[:, h].contiguous(), v[:, h].contiguous(),
          ksq, vsq)
        os_.append(plain(res[0]))
        ms_.append(plain(res[1])[..., 0])
        ls_.append(plain(res[2])[..., 0])
      o, m, l = torch.stack(os_, 1), torch.stack(ms_, 1), torch.stack(ls_, 1)
    out[name + "_o"], out[name + "_m"], out[name + "_l"] = plain(o), plain(m), plain(l)
  save("ragged", out)


def gen_engine_insert(eng, pam_mod):
  """`PyTorchEngine.insert` / `_insert_no_wrap` / `_insert_wrap`
  (engine.py:371-648) and `insert_page_attention_with_reservation` (650-672),
  called as unbound functions on a stand-in `self` that carries the fields they
  read (env, shardings, the page manager)."""
  W = _refshim.JTensor.wrap
  out = {}
  b, h, s, d, nl, lpad, seq_len = 4, 2, 32, 8, 2, 12, 10
  cases = {  # name -> (ring_buffer, stacked, quantized, current_position)
      "ring_nowrap_i8": (True, False, True, 20),
      "ring_wrap_i8": (True, False, True, 5),
      "ring_edge_i8": (True, False, True, 30),  # start 20, 20 + 12 == S: takes the wrap path without wrapping
      "ring_nowrap_bf16": (True, False, False, 20),
      "ring_wrap_bf16": (True, False, False, 5),
      "left_i8": (False, False, True, 0),
      "left_i8_stacked": (False, True, True, 0),
      "left_bf16_stacked": (False, True, False, 0),
  }
  out["geometry"] = np.asarray([b, h, s, d, nl, lpad, seq_len])
  for ci, (name, (ring, stacked, quant, cur)) in enumerate(cases.items()):
    g = torch.Generator().manual_seed(200 + ci)
    env = types.SimpleNamespace(
        ring_buffer=ring, cache_sequence_length=s, generate_cache_stacked=stacked,
        quant_config=types.SimpleNamespace(enable_kv_quantization=quant))
    me = types.SimpleNamespace(env=env, cache_sharding=None, replicated=None)
    me._insert_no_wrap = functools_partial(eng.PyTorchEngine._insert_no_wrap, me)
    me._insert_wrap = functools_partial(eng.PyTorchEngine._insert_wrap, me)
    shape = (nl, b, h, s, d) if stacked else (b, h, s, d)
    sshape = (nl, b, 1, s, 1) if stacked else (b, 1, s, 1)
    n_caches = 1 if stacked else nl
    caches, scales = [], []
    for _ in range(n_caches):
      if quant:
        caches.append((torch.randint(-127, 128, shape, generator=g).to(torch.int8),
                       torch.randint(-127, 128, shape, generator=g).to(torch.int8)))
        scales.append(((torch.rand(sshape, generator=g) + 0.01).to(torch.bfloat16),
                       (torch.rand(sshape, generator=g) + 0.01).to(torch.bfloat16)))
      else:
        caches.append((randn(g, *shape), randn(g, *shape)))
    prefix = [(randn(g, 1, h, lpad, d), randn(g, 1, h, lpad, d)) for _ in range(nl)]
    prefix[0][0][0, :, 3, :] = 0  # an all-zero token
    slot = 2
    for i, (ck, cv) in enumerate(caches):
      out[f"{name}_in_ck{i}"], out[f"{name}_in_cv{i}"] = ck.clone(), cv.clone()
    for i, (a, c) in enumerate(scales):
      out[f"{name}_in_ks{i}"], out[f"{name}_in_vs{i}"] = a.clone(), c.clone()
    for i, (pk, pv) in enumerate(prefix):
      out[f"{name}_prefix_k{i}"], out[f"{name}_prefix_v{i}"] = pk.clone(), pv.clone()
    out[f"{name}_args"] = np.asarray([int(ring), int(stacked), int(quant), cur, slot])
    state = eng.DecodeState(
        W(torch.zeros(b, 1, dtype=torch.int32)), [(W(a.clone()), W(c.clone())) for a, c in caches],
        [(W(a.clone()), W(c.clone())) for a, c in scales], cur, W(torch.full((b, 1), 9, dtype=torch.int32)),
        W(torch.full((b, 1), 3, dtype=torch.int32)), W(torch.full((b, 1), 4, dtype=torch.int32)),
        W(torch.full((b, s), float("-inf"))))
    pre = eng.Prefix(W(torch.tensor([[7]], dtype=torch.int32)), [(W(a), W(c)) for a, c in prefix], seq_len)
    res = eng.PyTorchEngine.insert(me, pre, state, slot)
    for i, (ck, cv) in enumerate(res.caches):
      out[f"{name}_out_ck{i}"], out[f"{name}_out_cv{i}"] = plain(ck), plain(cv)
    for i, (a, c) in enumerate(res.cache_scales or []):
      out[f"{name}_out_ks{i}"], out[f"{name}_out_vs{i}"] = plain(a), plain(c)
    out[f"{name}_out_mask"] = plain(res.mask)
    out[f"{name}_out_start"], out[f"{name}_out_input_pos"] = plain(res.start), plain(res.input_pos)
    out[f"{name}_out_lens"], out[f"{name}_out_tokens"] = plain(res.lens), plain(res.tokens)

  # paged insert with reservation (bf16 pools; the reference has no int8 paged cache)
  g = torch.Generator().manual_seed(260)
  p, ps, maxp = 24, 4, 6
  pam = pam_mod.PageAttentionManager(b, p, ps, maxp)
  pam.reserve_pages_insert(0, 6)  # pages 0, 1 are taken before the insert under test
  env = types.SimpleNamespace(ring_buffer=False, cache_sequence_length=s, generate_cache_stacked=False,
                              quant_config=types.SimpleNamespace(enable_kv_quantization=False))
  me = types.SimpleNamespace(env=env, cache_sharding=None, replicated=None, page_attention_manager=pam,
                             default_dtype=torch.bfloat16, prefill_cache_sharding=None)
  me._insert_page_attention_jit = functools_partial(eng.PyTorchEngine._insert_page_attention, me)
  pools = [(randn(g, h, p, ps, d), randn(g, h, p, ps, d)) for _ in range(nl)]
  prefix = [(randn(g, 1, h, lpad, d), randn(g, 1, h, lpad, d)) for _ in range(nl)]
  for i in range(nl):
    out[f"paged_in_ck{i}"], out[f"paged_in_cv{i}"] = pools[i][0].clone(), pools[i][1].clone()
    out[f"paged_prefix_k{i}"], out[f"paged_prefix_v{i}"] = prefix[i][0].clone(), prefix[i][1].clone()
  state = eng.DecodeState(
      W(torch.zeros(b, 1, dtype=torch.int32)), [(W(a.clone()), W(c.clone())) for a, c in pools], [], 0,
      W(torch.full((b, 1), 9, dtype=torch.int32)), W(torch.full((b, 1), 3, dtype=torch.int32)),
      W(torch.full((b, 1), 4, dtype=torch.int32)), W(torch.full((b, s), float("-inf"))))
  pre = eng.Prefix(W(torch.tensor([[7]], dtype=torch.int32)), [(W(a), W(c)) for a, c in prefix], seq_len)
  res = eng.PyTorchEngine.insert_page_attention_with_reservation(me, pre, state, 3)
  for i, (ck, cv) in enumerate(res.caches):
    out[f"paged_out_ck{i}"], out[f"paged_out_cv{i}"] = plain(ck), plain(cv)
  out["paged_geometry"] = np.asarray([p, ps, maxp, 3, seq_len])
  out["paged_out_page_indices"] = pam.page_indices.copy()
  out["paged_out_lengths"] = np.asarray(pam.lengths).copy()
  out["paged_out_mask"], out["paged_out_start"] = plain(res.mask), plain(res.start)
  out["paged_out_input_pos"], out["paged_out_lens"] = plain(res.input_pos), plain(res.lens)
  save("engine_insert", out)


def gen_engine_step(eng):
  """`PyTorchEngine.generate_impl` (engine.py:751-848) and
  `precompute_ragged_block_indices` (674-729) for three consecutive steps, with
  the model call replaced by a stand-in that returns fixed logits: what is
  recorded is the bookkeeping around the model (mask, positions, lengths, the
  result-token block, the block-skipping tables) and what the model was given."""
  W = _refshim.JTensor.wrap
  out = {}
  b, s, bk, vocab, steps = 4, 32, 8, 10, 3
  eng.engine_api.ResultTokens = lambda **kw: types.SimpleNamespace(**kw)
  out["geometry"] = np.asarray([b, s, bk, vocab, steps])
  for name, ring in (("ring", True), ("left", False)):
    env = types.SimpleNamespace(
        ring_buffer=ring, cache_sequence_length=s, cache_len=s, block_size=bk, batch_size=b,
        lazy_cache_update=not ring, page_attention=False, generate_cache_stacked=False,
        quant_config=types.SimpleNamespace(enable_kv_quantization=False))
    me = types.SimpleNamespace(env=env)
    me.precompute_ragged_block_indices = functools_partial(eng.PyTorchEngine.precompute_ragged_block_indices, me)
    seen = []

    def call_model(params, tokens, input_indexes, caches, scales, mask, start, input_pos, rbi, rbk, pti):
      seen.append((plain(torch.as_tensor(input_indexes)), plain(mask), plain(rbi), plain(rbk)))
      logits = torch.zeros(b, 1, vocab)
      logits[torch.arange(b), 0, (tokens[:, 0].long() * 3 + 1) % vocab] = 1
      return W(logits), caches, scales

    me._call_model_generate = call_model
    state = eng.DecodeState(
        W(torch.tensor([[1], [2], [3], [4]], dtype=torch.int32)), [], [], 30,
        W(torch.tensor([[1], [0], [3], [2]], dtype=torch.int32)), W(torch.tensor([30, 0, 3, 7], dtype=torch.int32)),
        W(torch.tensor([6, 0, 29, 9], dtype=torch.int32)), W(torch.full((b, s), float("-inf"))))
    for n, t in (("tokens", state.tokens), ("lens", state.lens), ("start", state.start),
                 ("input_pos", state.input_pos), ("mask", state.mask)):
      out[f"{name}_in_{n}"] = plain(t)
    out[f"{name}_in_current_position"] = np.int64(state.current_position)
    sampler = lambda logits: W(logits.argmax(-1).reshape(b, 1).to(torch.int32))
    for step in range(steps):
      state, res = eng.PyTorchEngine.generate_impl(me, None, state, sampler=sampler)
      pre = f"{name}_step{step}_"
      out[pre + "tokens"], out[pre + "lens"] = plain(state.tokens), plain(state.lens)
      out[pre + "input_pos"], out[pre + "mask"] = plain(state.input_pos), plain(state.mask)
      out[pre + "current_position"] = np.int64(state.current_position)
      out[pre + "data"] = plain(res.data)
      out[pre + "model_input_indexes"], out[pre + "model_mask"] = seen[-1][0], seen[-1][1]
      out[pre + "ragged_batch_index"], out[pre + "ragged_block_index"] = seen[-1][2], seen[-1][3]
  save("engine_step", out)


def gen_linear(layers):
  """`WeightOnlyPerChannelQuantizedLinear` (layers.py:69-166): the reference's
  own weight quantiser and forward.  Its `F.linear(bf16, int8)` exists only under
  torch_xla2, where the int8 weight is promoted to bfloat16 (jax type promotion);
  on CPU torch that one call is given the promoted weight, everything else runs
  as written."""
  real_linear = layers.F.linear

  def promoted_linear(inputs, weight, bias=None):
    return real_linear(inputs, weight.to(inputs.dtype) if weight.dtype == torch.int8 else weight, bias)

  g = torch.Generator().manual_seed(11)
  out = {}
  for tag, (m, k, n) in (("small", (5, 256, 192)), ("batch", (96, 1024, 320))):
    lin = layers.WeightOnlyPerChannelQuantizedLinear(k, n)
    w = torch.randn(n, k, generator=g) * 0.05
    w[3] = 0  # an all-zero channel: the EPS clamp of the scale
    w[7] *= 1e-4
    lin.quantize_weight_from_nn_linear(w)
    x = randn(g, 1, m, k)
    x[0, 1] = 0
    x[0, 2] *= 37.0
    layers.F.linear = promoted_linear
    try:
      y = lin(x)
    finally:
      layers.F.linear = real_linear
    assert y.dtype == torch.bfloat16 and lin.weight.dtype == torch.int8 and lin.weight_scaler.dtype == torch.bfloat16
    if tag == "small":
      out[f"{tag}_w"] = w  # (the float weight only where the quantiser is pinned: it is the bulk of the file)
    out.update({f"{tag}_x": x, f"{tag}_weight": lin.weight, f"{tag}_weight_scaler": lin.weight_scaler,
                f"{tag}_y": y})
  # RMSNorm (layers.py:337-350) as the model runs it in bf16: the weight converted like the other parameters
  norm = layers.RMSNorm(512, eps=1e-5, device="cpu")
  norm.weight = torch.nn.Parameter((1 + 0.1 * torch.randn(512, generator=g)).to(torch.bfloat16), requires_grad=False)
  xn = randn(g, 2, 9, 512)
  xn[0, 1] = 0
  xn[0, 2] *= 50.0
  yn = norm(xn)
  assert yn.dtype == torch.bfloat16
  out.update({"norm_x": xn, "norm_weight": norm.weight.data, "norm_eps": np.float32(1e-5), "norm_y": yn})
  save("linear", out)


def functools_partial(fn, first):
  return lambda *a: fn(first, *a)


def main():
  if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py <path of a jetstream-pytorch checkout>")
  ref = sys.argv[1]
  cm, pam, ak, q = _refshim.import_reference(ref)
  gen_quantizers(cm, q)
  gen_int8_cache(cm)
  gen_float_cache(cm)
  gen_pages(cm, pam)
  gen_attention(ak, q)
  gen_ragged(ak)
  eng = _refshim.import_reference_engine(ref)
  gen_engine_insert(eng, pam)
  gen_engine_step(eng)
  gen_linear(_refshim.import_reference_layers(ref))
  print("golden fixtures written")


if __name__ == "__main__":
  main()
