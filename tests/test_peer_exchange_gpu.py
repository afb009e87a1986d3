"""The in-kernel NVLink max-reduction of the per-token amax (head-sharded int8 caches).

One rank: the exchange machinery (launch numbers, parity, completion counter)
against the plain update.  Two ranks (run when the box has two GPUs): each
process owns half of the KV heads; codes and scales must equal the unsharded
update bit for bit.  Nothing here waits without a limit: a rank that loses
its peer goes on after about half a second and reports it through status().
"""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

pytestmark = pytest.mark.gpu

B, H, S, D, STEPS = 12, 8, 64, 128, 5


def _inputs(step):
  g = torch.Generator().manual_seed(500 + step)
  xk = torch.randn(B, H, 1, D, generator=g).to(torch.bfloat16)
  xv = (torch.randn(B, H, 1, D, generator=g) * 3).to(torch.bfloat16)
  if step == 2:
    xk[3] = 0  # an all-zero token: scale 0, codes 0
  return xk, xv


def _make_cache(heads, dev):
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData

  data = JetEngineEnvironmentData(batch_size=B, cache_sequence_length=S, num_layers=1, ring_buffer=False, testing=True,
                                  cache_shape=(B, heads, S, D))
  data.quant_config.enable_kv_quantization = True
  env = JetEngineEnvironment(data, device=dev)
  ck = torch.zeros((B, heads, S, D), dtype=torch.int8, device=dev)
  cv = torch.zeros((B, heads, S, D), dtype=torch.int8, device=dev)
  ks = torch.zeros((B, 1, S, 1), dtype=torch.bfloat16, device=dev)
  vs = torch.zeros((B, 1, S, 1), dtype=torch.bfloat16, device=dev)
  pos = torch.arange(B, dtype=torch.int32, device=dev) % S
  return Int8KVCacheGenerate(ck, cv, ks, vs, pos, env=env), (ck, cv, ks, vs)


def _run_steps(cache, lo, hi, dev, peers):
  for step in range(STEPS):
    xk, xv = _inputs(step)
    cache.input_pos = ((torch.arange(B, dtype=torch.int32) + step) % S).to(dev)
    cache.update(xk[:, lo:hi].contiguous().to(dev), xv[:, lo:hi].contiguous().to(dev), 0, peers=peers)
  torch.cuda.synchronize(dev)


def test_single_rank_exchange_equals_plain_update():
  from jetstream_pytorch_b200.cache_manager import PeerAmaxExchange

  dev = torch.device("cuda", 0)
  plain, ref = _make_cache(H, dev)
  _run_steps(plain, 0, H, dev, None)
  fused, got = _make_cache(H, dev)
  px = PeerAmaxExchange(B, 0, 1, lambda h: [h])
  try:
    _run_steps(fused, 0, H, dev, px)
    assert px.status() == 0
  finally:
    px.close()
  for a, b in zip(ref, got):
    assert torch.equal(a, b)


def _worker(rank, world, port, out_path):
  import torch.distributed as dist

  os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
  os.environ["NCCL_NVLS_ENABLE"] = "0"
  torch.cuda.set_device(rank)
  dev = torch.device("cuda", rank)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  from jetstream_pytorch_b200.cache_manager import PeerAmaxExchange

  hs = H // world
  cache, got = _make_cache(hs, dev)
  px = PeerAmaxExchange.with_torch_distributed(B)
  _run_steps(cache, rank * hs, (rank + 1) * hs, dev, px)
  status = px.status()
  dist.barrier()  # nobody frees a buffer that a peer may still write to
  px.close()
  torch.save({"status": status, "tensors": [t.cpu() for t in got]}, f"{out_path}.{rank}")
  dist.barrier()
  dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_equal_the_unsharded_update(tmp_path):
  import torch.multiprocessing as mp

  world = 2
  out = str(tmp_path / "rank")
  mp.spawn(_worker, args=(world, 29600 + os.getpid() % 300, out), nprocs=world, join=True)
  dev = torch.device("cuda", 0)
  plain, ref = _make_cache(H, dev)
  _run_steps(plain, 0, H, dev, None)
  ref = [t.cpu() for t in ref]
  hs = H // world
  for rank in range(world):
    res = torch.load(f"{out}.{rank}")
    assert res["status"] == 0
    ck, cv, ks, vs = res["tensors"]
    assert torch.equal(ck, ref[0][:, rank * hs:(rank + 1) * hs])
    assert torch.equal(cv, ref[1][:, rank * hs:(rank + 1) * hs])
    assert torch.equal(ks, ref[2]) and torch.equal(vs, ref[3])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_drives_two_gpus():
  """Kernel attributes (the dynamic shared-memory opt-in) and the SM count are
  per device: the tensor-core attention kernels must work on cuda:1 after their
  first use on cuda:0, from one process."""
  from jetstream_pytorch_b200 import attention_kernel as ak
  from oracle import attention as oa
  from oracle.quant import quantize_insert
  from parity_tools import attention_close, describe

  g = torch.Generator().manual_seed(77)
  b, hq, hkv, s, d = 4, 32, 4, 512, 128
  q = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
  kf = torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16)
  vf = torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16)
  k, ks = quantize_insert(kf, (-3, -1))
  v, vs = quantize_insert(vf, (-3, -1))
  end = torch.tensor([512, 1, 300, 77])
  start = torch.zeros(b, dtype=torch.int64)
  eo_i8, _ = oa.ragged_mha(q, k, v, 0, start, end, ks, vs, bk=512)
  eo_bf, _ = oa.ragged_mha(q, kf, vf, 0, start, end, None, None, bk=512)
  for index in (0, 1):  # the current device stays cuda:0 throughout
    dev = torch.device("cuda", index)
    o, _ = ak.ragged_mha(q.to(dev), k.to(dev), v.to(dev), 0, start.to(dev), end.to(dev), None, None, ks.to(dev),
                         vs.to(dev))
    assert o.device == dev and attention_close(o, eo_i8), describe(o, eo_i8)
    o, _ = ak.ragged_mha(q.to(dev), kf.to(dev), vf.to(dev), 0, start.to(dev), end.to(dev), None, None, None, None)
    assert attention_close(o, eo_bf), describe(o, eo_bf)
  assert ak.kernel_status() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_prefix_inserted_from_the_other_gpu():
  """Disaggregated prefill -> decode: the prefix lies on cuda:1, the caches on cuda:0; the insert
  kernels of cuda:0 read it over NVLink.  Dense (int8, quantising, wrap and no wrap) and paged
  (stacked int8 pools in one launch) results must equal those of a prefix on the same GPU."""
  from jetstream_pytorch_b200.insert import insert_dense
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  d0, d1 = torch.device("cuda", 0), torch.device("cuda", 1)
  g = torch.Generator().manual_seed(901)
  h, l, d, s, b = 8, 300, 128, 512, 4
  pk = torch.randn(1, h, l, d, generator=g).to(torch.bfloat16)
  pv = torch.randn(1, h, l, d, generator=g).to(torch.bfloat16)
  for wrap, pos in ((False, 17), (True, 400)):
    out = []
    for src in (d0, d1):
      ck = torch.zeros(b, h, s, d, dtype=torch.int8, device=d0)
      cv = torch.zeros(b, h, s, d, dtype=torch.int8, device=d0)
      ks = torch.ones(b, 1, s, 1, dtype=torch.bfloat16, device=d0)
      vs = torch.ones(b, 1, s, 1, dtype=torch.bfloat16, device=d0)
      insert_dense(pk.to(src), pv.to(src), ck, cv, 2, pos, wrap=wrap, k_scaler=ks, v_scaler=vs)
      torch.cuda.synchronize(d0)
      out.append((ck.cpu(), cv.cpu(), ks.cpu(), vs.cpu()))
    for a, c in zip(out[0], out[1]):
      assert torch.equal(a, c), f"wrap={wrap}: a prefix on the other GPU gave a different cache"
    assert out[0][0][2].any()

  nl, p, ps, maxp = 3, 32, 64, 8
  spk = torch.randn(nl, 1, h, l, d, generator=g).to(torch.bfloat16)
  spv = torch.randn(nl, 1, h, l, d, generator=g).to(torch.bfloat16)
  out = []
  for src in (d0, d1):
    pam = PageAttentionManager(b, p, ps, maxp)
    _, upd = pam.reserve_pages_insert(1, l)
    kp = torch.zeros(nl, h, p, ps, d, dtype=torch.int8, device=d0)
    vp = torch.zeros(nl, h, p, ps, d, dtype=torch.int8, device=d0)
    ksp = torch.zeros(nl, 1, p, ps, 1, dtype=torch.bfloat16, device=d0)
    vsp = torch.zeros(nl, 1, p, ps, 1, dtype=torch.bfloat16, device=d0)
    a_k, a_v = spk.to(src), spv.to(src)
    pam.insert_prefill_cache([(a_k[i], a_v[i]) for i in range(nl)], [(kp[i], vp[i]) for i in range(nl)], upd, None, None,
                             decode_scales=[(ksp[i], vsp[i]) for i in range(nl)])
    torch.cuda.synchronize(d0)
    out.append((kp.cpu(), vp.cpu(), ksp.cpu(), vsp.cpu()))
  for a, c in zip(out[0], out[1]):
    assert torch.equal(a, c), "paged: a prefix on the other GPU gave different pools"
  assert out[0][0].any()
