"""KV-head sharding on CPU ranks (gloo, world_size 2): the per-token int8 scale
spans all heads, so each rank contributes the amax of its own heads, the ranks
max-reduce it, and every rank quantises with the reduced value.  The result must
equal the unsharded oracle bit for bit, and attention over a rank's heads must
equal the matching slice of unsharded attention (no communication)."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention as oa
from oracle.quant import local_amax, quantize_decode, quantize_insert


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _worker(rank, world, port, out):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    g = torch.Generator().manual_seed(5)
    b, hq, hkv, s, d = 6, 16, 4, 48, 32
    xk = torch.randn(b, hkv, 1, d, generator=g).to(torch.bfloat16)
    xk[2] = 0
    q = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
    k = torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16)
    v = torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16)
    kq, ks = quantize_insert(k, (-3, -1))
    vq, vs = quantize_insert(v, (-3, -1))
    end = torch.randint(1, s + 1, (b,), generator=g)
    hs = slice(rank * hkv // world, (rank + 1) * hkv // world)
    qs = slice(rank * hq // world, (rank + 1) * hq // world)
    # sharded decode quantiser
    amax = local_amax(xk[:, hs])
    dist.all_reduce(amax, op=dist.ReduceOp.MAX)
    codes, scale = quantize_decode(xk[:, hs], amax=amax)
    full_codes, full_scale = quantize_decode(xk)
    ok = torch.equal(codes, full_codes[:, hs]) and torch.equal(scale, full_scale)
    # attention over this rank's heads, no exchange
    o, (m, l) = oa.ragged_mha(q[:, qs], kq[:, hs], vq[:, hs], 0, torch.zeros(b), end, ks, vs, bk=16)
    fo, (fm, fl) = oa.ragged_mha(q, kq, vq, 0, torch.zeros(b), end, ks, vs, bk=16)
    ok = ok and torch.equal(o, fo[:, hs]) and torch.equal(m, fm[:, hs]) and torch.equal(l, fl[:, hs])
    out[rank] = bool(ok)
  finally:
    dist.destroy_process_group()


def test_head_sharded_quantise_and_attention_match_unsharded():
  world = 2
  port = _free_port()
  with mp.Manager() as mgr:
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def _linear_worker(rank, world, port, out):
  """Row-parallel weight-only int8 layer: each rank multiplies its slice of the input features; the fp32 partial
  results are summed over the ranks (what the device kernel does over NVLink, here a gloo all-reduce), then come
  the two bf16 roundings and the channel scale."""
  from oracle import linear as ol

  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    g = torch.Generator().manual_seed(9)
    m, k, n = 24, 512, 96
    wq, sc = ol.quantize_weight(torch.randn(n, k, generator=g) * 0.05)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    ks = slice(rank * k // world, (rank + 1) * k // world)
    partial = (x[:, ks].double() @ wq[:, ks].double().t()).float()  # this rank's sums, as the GEMM leaves them
    dist.all_reduce(partial, op=dist.ReduceOp.SUM)
    y = (partial.to(torch.bfloat16).float() * sc.float()).to(torch.bfloat16)
    want = ol.w8a16_linear(x, wq, sc)
    err = (y.float() - want.float()).abs().double()
    same = (y.view(torch.int16) == want.view(torch.int16)).float().mean().item()
    out[rank] = bool((err <= ol.w8a16_tolerance(x, wq, sc)).all()) and same > 0.99
  finally:
    dist.destroy_process_group()


def test_row_parallel_linear_sums_to_the_unsharded_layer():
  world = 2
  port = _free_port()
  with mp.Manager() as mgr:
    out = mgr.dict()
    mp.spawn(_linear_worker, args=(world, port, out), nprocs=world, join=True)
    assert all(out[r] for r in range(world)), dict(out)
