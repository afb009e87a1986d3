"""Generates the golden fixtures in this directory by EXECUTING THE REFERENCE'S
OWN MODULES (cache_manager.py, page_attention_manager.py, attention_kernel.py,
quantize.py), imported unmodified from a reference checkout.

    python tests/golden/make_golden.py /path/to/jetstream-pytorch

The reference needs jax and torch_xla2 only for array plumbing on this path
(the arithmetic is torch / numpy), so `_refshim.py` supplies torch-backed
stand-ins for those packages.  The Pallas-TPU ragged kernels and the JAX
paged-attention kernel cannot be executed this way and have no fixture.
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
  print("golden fixtures written")


if __name__ == "__main__":
  main()
