"""The row-parallel weight-only int8 linear layer: the input features sharded
over the GPUs of one box, the partial results added inside the GEMM's epilogue
over NVLink peer memory.  Two ranks run as two processes when the box has two
GPUs; nothing waits without a limit (a rank that loses its peer goes on after
its wait ran out and reports it through status())."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import linear as ol  # noqa: E402

pytestmark = pytest.mark.gpu

CASES = [(96, 2048, 1000), (7, 1024, 256), (128, 4096, 8192)]  # (rows, in features, out features)
CALLS = 3


def _case(i, call):
  m, k, n = CASES[i]
  g = torch.Generator().manual_seed(900 + 10 * i)
  wq, sc = ol.quantize_weight(torch.randn(n, k, generator=g) * 0.03)
  gx = torch.Generator().manual_seed(950 + 10 * i + call)
  x = (torch.randn(m, k, generator=gx) * torch.rand(m, 1, generator=gx) * 3).to(torch.bfloat16)
  return x, wq, sc


def _run(rank, world, dev, tp):
  """Every case CALLS times (different activations each time): the launch parity alternates, shapes change
  between cases."""
  from jetstream_pytorch_b200.layers import WeightOnlyPerChannelQuantizedLinear

  outs = []
  for i, (m, k, n) in enumerate(CASES):
    ks = k // world
    lin = WeightOnlyPerChannelQuantizedLinear(ks, n, device=dev)
    _, wq, sc = _case(i, 0)
    lin._load_quantized_weights(wq[:, rank * ks:(rank + 1) * ks].contiguous(), sc)
    for call in range(CALLS):
      x, _, _ = _case(i, call)
      outs.append(lin(x[:, rank * ks:(rank + 1) * ks].contiguous().to(dev), tp=tp).cpu())
    torch.cuda.synchronize(dev)
    assert lin.kernel_status() == 0
  return outs


def _check(outs):
  it = iter(outs)
  for i in range(len(CASES)):
    for call in range(CALLS):
      x, wq, sc = _case(i, call)
      y = next(it)
      err = (y.float() - ol.w8a16_linear(x, wq, sc).float()).abs().double()
      assert (err <= ol.w8a16_tolerance(x, wq, sc)).all(), (i, call)
      same = (y.view(torch.int16) == ol.w8a16_linear(x, wq, sc).view(torch.int16)).float().mean().item()
      assert same > 0.95, same


def test_one_rank_goes_through_the_same_entry_point():
  from jetstream_pytorch_b200.layers import TensorParallelSum

  dev = torch.device("cuda", 0)
  tp = TensorParallelSum(8192, 0, 1, lambda h: [h])
  try:
    outs = _run(0, 1, dev, tp)
    assert tp.status() == 0
  finally:
    tp.close()
  _check(outs)


def _worker(rank, world, port, out_path):
  import torch.distributed as dist

  os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
  os.environ["NCCL_NVLS_ENABLE"] = "0"
  torch.cuda.set_device(rank)
  dev = torch.device("cuda", rank)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  from jetstream_pytorch_b200.layers import TensorParallelSum

  tp = TensorParallelSum.with_torch_distributed(8192)
  outs = _run(rank, world, dev, tp)
  status = tp.status()
  dist.barrier()  # nobody frees a buffer that a peer may still write to
  tp.close()
  torch.save({"status": status, "outs": outs}, f"{out_path}.{rank}")
  dist.barrier()
  dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_sum_inside_the_kernel(tmp_path, world):
  """Two ranks exchange their partial sums; with four a tile's owner adds them and returns the result."""
  import torch.multiprocessing as mp

  if torch.cuda.device_count() < world:
    pytest.skip(f"needs {world} GPUs")
  out = str(tmp_path / "rank")
  mp.spawn(_worker, args=(world, 29900 + os.getpid() % 300, out), nprocs=world, join=True)
  res = [torch.load(f"{out}.{rank}") for rank in range(world)]
  for r in res:
    assert r["status"] == 0
    _check(r["outs"])
  # every rank adds the same partial sums in the same order: the same bits everywhere
  for other in res[1:]:
    for a, b in zip(res[0]["outs"], other["outs"]):
      assert torch.equal(a, b)


def test_a_peer_that_never_comes_is_reported():
  """World of two with only this rank launching (the other buffer is a second local allocation that nobody
  writes): the wait runs out after the given number of cycles, status becomes 1, the context stays usable."""
  import ctypes

  from jetstream_pytorch_b200 import _lib
  from jetstream_pytorch_b200.layers import TensorParallelSum, WeightOnlyPerChannelQuantizedLinear

  dev = torch.device("cuda", 0)
  lib = _lib.lib()
  # (sized for 512 channels on one rank = 256 channels on two; the wait: about 10 ms)
  tp = TensorParallelSum(512, 0, 1, lambda h: [h], wait_cycles=20_000_000)
  silent = ctypes.c_void_p()
  _lib.check(lib.jpt_peer_exchange_alloc(tp.struct.buffer_bytes, ctypes.byref(silent)))
  try:
    tp.struct.world = 2
    tp.struct.buffers[1] = silent.value
    x, wq, sc = _case(1, 0)
    lin = WeightOnlyPerChannelQuantizedLinear(x.shape[1], 256, device=dev)
    lin._load_quantized_weights(wq, sc)
    y = lin(x.to(dev), tp=tp)
    torch.cuda.synchronize(dev)
    assert tp.status() == 1
    # what had arrived is this rank's own partial: the single-GPU result
    assert torch.equal(y, lin(x.to(dev)))
  finally:
    tp.struct.world = 1
    lib.jpt_peer_exchange_free(silent)
    tp.close()
