"""The bounded waits of the kernels that wait on another GPU, made to run out
on purpose on ONE GPU: a world-of-two amax exchange whose second rank does not
exist (its buffer is a local allocation nobody writes).  The launch must
return, report through the status word, and leave the exchange usable."""

import time

import pytest
import torch

from oracle.quant import quantize_decode

pytestmark = pytest.mark.gpu

DEV = "cuda"


class _LoneRankExchange:
  """Rank 0 of a world of 2; the "peer" buffer is local memory nobody writes.
  Both buffers are plain zero-filled device tensors (the exchange only needs
  8-byte aligned device memory of jpt_peer_exchange_bytes() bytes)."""

  def __init__(self, batch, wait_cycles):
    from jetstream_pytorch_b200 import _lib

    nbytes = _lib.lib().jpt_peer_exchange_bytes(batch, 2)
    assert nbytes % 8 == 0
    self.own = torch.zeros(nbytes // 8, dtype=torch.int64, device=DEV)
    self.other = torch.zeros(nbytes // 8, dtype=torch.int64, device=DEV)
    self.struct = _lib.PeerExchangeStruct()
    self.struct.rank, self.struct.world, self.struct.batch = 0, 2, batch
    self.struct.buffers[0], self.struct.buffers[1] = self.own.data_ptr(), self.other.data_ptr()
    self.struct.wait_cycles = wait_cycles
    self.batch = batch

  def status(self):
    from jetstream_pytorch_b200 import _lib

    return _lib.lib().jpt_peer_exchange_status(self.own.data_ptr(), _lib.stream())

  def write_peer_words(self, epoch, amax):
    """What rank 1 would have stored into rank 0's buffer for launch `epoch`:
    64 bytes of state, then slots[epoch & 1][writer rank][2 B] of 64-bit words
    (epoch << 32 | float bits of the partial amax), K row then V row."""
    bits = amax.to(DEV, torch.float32).reshape(-1).view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    first = 8 + ((epoch & 1) * 2 + 1) * (2 * self.batch)
    self.own[first:first + 2 * self.batch] = bits | (epoch << 32)

  def close(self):
    torch.cuda.synchronize()


def test_peer_wait_runs_out_reports_and_recovers():
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData

  b, h, s, d = 16, 4, 64, 128
  g = torch.Generator().manual_seed(81)
  xk = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
  xv = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
  pos = torch.randint(0, s, (b,), generator=g)
  data = JetEngineEnvironmentData(batch_size=b, cache_sequence_length=s, ring_buffer=False, testing=True)
  data.quant_config.enable_kv_quantization = True
  env = JetEngineEnvironment(data, device=DEV)

  def fresh_cache():
    return Int8KVCacheGenerate(torch.zeros(b, h, s, d, dtype=torch.int8, device=DEV),
                               torch.zeros(b, h, s, d, dtype=torch.int8, device=DEV),
                               torch.ones(b, 1, s, 1, dtype=torch.bfloat16, device=DEV),
                               torch.ones(b, 1, s, 1, dtype=torch.bfloat16, device=DEV), pos.to(DEV), env=env)

  px = _LoneRankExchange(b, wait_cycles=4_000_000)  # about 2 ms at 2 GHz
  try:
    assert px.status() == 0
    # 1. nobody answers: the launch gives up after the limit, goes on with its own amax
    cache = fresh_cache()
    t0 = time.perf_counter()
    r = cache.update(xk.to(DEV), xv.to(DEV), 0, peers=px)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0, "the bounded wait did not end in time"
    assert px.status() == 1
    kq, ks = quantize_decode(xk)
    vq, vs = quantize_decode(xv)
    assert torch.equal(r[2].cpu(), kq) and torch.equal(r[3].cpu(), vq)
    assert torch.equal(r[6].cpu(), ks) and torch.equal(r[7].cpu(), vs)
    # 2. the launch number advanced all the same: a second launch whose peer words are
    #    present pairs up at once and uses the larger of the two maxima
    peer_amax = torch.stack([xk.float().abs().amax(dim=(1, 2, 3)) * 2.0, xv.float().abs().amax(dim=(1, 2, 3)) * 0.5])
    px.write_peer_words(2, peer_amax)
    cache = fresh_cache()
    local = cache.local_amax(xk.to(DEV), xv.to(DEV))
    expected = fresh_cache().update(xk.to(DEV), xv.to(DEV), 0, amax=torch.maximum(local, peer_amax.to(DEV)))
    t0 = time.perf_counter()
    r = cache.update(xk.to(DEV), xv.to(DEV), 0, peers=px)
    torch.cuda.synchronize()
    for got, want in zip(r, expected):
      assert torch.equal(got, want)
    assert not torch.equal(r[6].cpu(), ks), "the peer's larger K amax must change the scale"
  finally:
    px.close()


def test_attention_status_word_of_the_builtin_scratch_is_readable():
  from jetstream_pytorch_b200 import _lib
  from jetstream_pytorch_b200 import attention_kernel as ak

  assert _lib.lib().jpt_flash_decode_status(None, _lib.stream()) == 0
  assert ak.kernel_status() == 0
