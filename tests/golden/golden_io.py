"""Save / load golden fixtures as .npz files of plain integer / float arrays.

bf16 tensors are stored as their 16-bit patterns under the key `<name>__bf16`.
"""

import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def save(name, tensors):
  out = {}
  for k, v in tensors.items():
    if isinstance(v, torch.Tensor):
      v = v.detach().as_subclass(torch.Tensor).contiguous()
      if v.dtype == torch.bfloat16:
        out[k + "__bf16"] = v.view(torch.int16).numpy()
      else:
        out[k] = v.numpy()
    else:
      out[k] = np.asarray(v)
  np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)


def load(name):
  data = np.load(os.path.join(HERE, name + ".npz"))
  out = {}
  for k in data.files:
    if k.endswith("__bf16"):
      out[k[:-6]] = torch.from_numpy(data[k].copy()).view(torch.bfloat16)
    else:
      arr = data[k]
      out[k] = torch.from_numpy(arr.copy()) if arr.ndim else arr.item()
  return out
