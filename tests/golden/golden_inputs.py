"""Seeded inputs of the ragged-attention golden cases.

The large cases (head_dim 128, cache length 1024) would make the fixture file
several megabytes, so `ragged.npz` stores only the reference's OUTPUTS plus a
checksum of the inputs; `make_golden.py` and the tests both rebuild the inputs
from the generators here and the tests refuse to run on a checksum mismatch.
"""

import torch

# name -> geometry and validity ranges.  `ring`: the case runs the ring-buffer
# kernel body (valid [start, end) or wrapped, start == end empty); otherwise the
# left-aligned one (valid [0, end), start ignored).
RAGGED_CASES = {
    "left_i8_d128": dict(seed=101, b=5, hq=16, hkv=2, s=1024, d=128, bk=512, kv="int8", q=torch.bfloat16,
                         start=[0, 0, 0, 0, 0], end=[1024, 513, 1, 300, 0]),
    "left_bf16_d128": dict(seed=102, b=5, hq=16, hkv=2, s=1024, d=128, bk=512, kv="float", q=torch.bfloat16,
                           start=[0, 0, 0, 0, 0], end=[1024, 513, 1, 300, 0]),
    "left_i8_stacked": dict(seed=103, b=3, hq=8, hkv=2, s=64, d=16, bk=16, kv="int8", q=torch.bfloat16,
                            start=[0, 0, 0], end=[64, 17, 33], layers=2, layer=1),
    "left_f32_small": dict(seed=104, b=3, hq=4, hkv=4, t=2, s=48, d=16, bk=16, kv="float", q=torch.float32,
                           start=[0, 0, 0], end=[48, 5, 16]),
    "ring_i8_d128": dict(seed=105, b=6, hq=8, hkv=2, s=1024, d=128, bk=512, kv="int8", q=torch.bfloat16, ring=True,
                         start=[0, 100, 900, 500, 1023, 0], end=[1024, 700, 200, 500, 1, 1]),
    "ring_bf16_small": dict(seed=106, b=5, hq=4, hkv=2, s=64, d=16, bk=16, kv="float", q=torch.bfloat16, ring=True,
                            start=[0, 10, 50, 7, 63], end=[64, 40, 20, 7, 2]),
}


def ragged_inputs(name):
  """Returns dict(q [B,Hq,T,D], k, v [B,Hkv,S,D] (stacked: [NL,...]), ks, vs
  [B,1,S,1] bf16 or None, start, end int32 [B], bk, layer, ring)."""
  c = RAGGED_CASES[name]
  g = torch.Generator().manual_seed(c["seed"])
  b, hq, hkv, s, d, t = c["b"], c["hq"], c["hkv"], c["s"], c["d"], c.get("t", 1)
  lead = (c["layers"],) if "layers" in c else ()
  q = torch.randn(b, hq, t, d, generator=g).to(c["q"])
  if c["kv"] == "int8":
    k = torch.randint(-127, 128, lead + (b, hkv, s, d), generator=g, dtype=torch.int8)
    v = torch.randint(-127, 128, lead + (b, hkv, s, d), generator=g, dtype=torch.int8)
    ks = (torch.rand(lead + (b, 1, s, 1), generator=g) * 0.03 + 0.005).to(torch.bfloat16)
    vs = (torch.rand(lead + (b, 1, s, 1), generator=g) * 0.03 + 0.005).to(torch.bfloat16)
  else:
    k = torch.randn(lead + (b, hkv, s, d), generator=g).to(c["q"])
    v = torch.randn(lead + (b, hkv, s, d), generator=g).to(c["q"])
    ks = vs = None
  return dict(q=q, k=k, v=v, ks=ks, vs=vs, start=torch.tensor(c["start"], dtype=torch.int32),
              end=torch.tensor(c["end"], dtype=torch.int32), bk=c["bk"], layer=c.get("layer", 0),
              ring=c.get("ring", False))


def checksum(inputs):
  """Order-sensitive 64-bit checksum of the tensors of `inputs`."""
  total = 0
  for key in ("q", "k", "v", "ks", "vs"):
    t = inputs[key]
    if t is None:
      continue
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
      t = t.view(torch.int16)
    elif t.dtype == torch.float32:
      t = t.view(torch.int32)
    flat = t.reshape(-1).to(torch.int64)
    w = (torch.arange(flat.numel(), dtype=torch.int64) % 8191) + 1
    total = (total * 31 + int((flat * w).sum().item())) % (1 << 61)
  return total
