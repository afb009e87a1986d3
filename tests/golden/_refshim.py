"""Torch-backed stand-ins for the packages the reference imports but this
machine lacks (jax, jax.numpy, jax.experimental.pallas, torch_xla2), so that the
reference's own modules can be imported UNMODIFIED from a read-only checkout and
the parts of them that are plain torch / numpy can be executed to produce golden
vectors.

Only `make_golden.py` (run once, on a machine that has the reference checkout)
uses this file.  Nothing here is arithmetic of its own: every function forwards
to the torch op with the same meaning, arrays are torch tensors carrying the two
jax-array idioms the reference uses (`x.at[idx].set(v)`, `x.jax()`, `x._elem =`).
The Pallas kernels and `jax.random` are NOT emulated; calling them raises.
"""

import contextlib
import sys
import types

import numpy as np
import torch


class JTensor(torch.Tensor):
  """torch.Tensor with the jax-array / XLATensor2 idioms the reference uses."""

  @staticmethod
  def wrap(t):
    if isinstance(t, JTensor):
      return t
    if isinstance(t, torch.Tensor):
      return t.as_subclass(JTensor)
    return t

  def jax(self):
    return self

  @property
  def _elem(self):
    return self

  @_elem.setter
  def _elem(self, value):
    # `tensor._elem = new_array` rebinds the wrapped array in XLATensor2.
    self.data = torch.as_tensor(value).data

  @property
  def at(self):
    return _At(self)

  def transpose(self, *axes):
    if len(axes) == 1 and isinstance(axes[0], (tuple, list)):
      return self.permute(*axes[0])
    if len(axes) == self.ndim and self.ndim != 2:
      return self.permute(*axes)
    return super().transpose(*axes)

  def astype(self, dtype):
    return self.to(dtype)

  def block_until_ready(self):
    return self


class _At:

  def __init__(self, arr):
    self.arr = arr

  def __getitem__(self, idx):
    return _AtIdx(self.arr, idx)


class _AtIdx:

  def __init__(self, arr, idx):
    self.arr, self.idx = arr, idx

  def set(self, value):
    out = self.arr.clone()
    idx = self.idx
    if not isinstance(idx, tuple):
      idx = (idx,)
    idx = tuple(
        torch.as_tensor(np.asarray(i)) if isinstance(i, (list, np.ndarray)) else i
        for i in idx
    )
    value = torch.as_tensor(value)
    out[idx] = value.to(out.dtype)
    return JTensor.wrap(out)


def _tree_map(fn, tree):
  if isinstance(tree, (list, tuple)):
    return type(tree)(_tree_map(fn, t) for t in tree)
  if isinstance(tree, dict):
    return {k: _tree_map(fn, v) for k, v in tree.items()}
  return fn(tree)


def _mod(name):
  m = types.ModuleType(name)
  sys.modules[name] = m
  return m


def _unavailable(what):

  def f(*a, **k):
    raise RuntimeError(f"{what} is not emulated by the import shim")

  return f


def install():
  """Registers the stand-in modules in sys.modules (idempotent)."""
  if "jax" in sys.modules and getattr(sys.modules["jax"], "_IS_SHIM", False):
    return
  jax = _mod("jax")
  jax._IS_SHIM = True

  def jit(f=None, **_kw):
    if f is None:
      return lambda g: g
    return f

  jax.jit = jit
  jax.named_scope = lambda name: contextlib.nullcontext()
  jax.Array = torch.Tensor
  jax.vmap = _unavailable("jax.vmap")
  jax.default_device = lambda d: contextlib.nullcontext()
  jax.devices = lambda *a: ["cpu"]
  jax.config = types.SimpleNamespace(update=lambda *a, **k: None)
  jax.ShapeDtypeStruct = lambda shape, dtype: (shape, dtype)

  tree_util = _mod("jax.tree_util")
  tree_util.register_pytree_node = lambda *a, **k: None
  tree_util.tree_map = _tree_map
  jax.tree_util = tree_util

  sharding = _mod("jax.sharding")

  class _Dummy:

    def __init__(self, *a, **k):
      pass

  sharding.Mesh = _Dummy
  sharding.PartitionSpec = _Dummy
  sharding.NamedSharding = _Dummy
  sharding.Sharding = _Dummy
  jax.sharding = sharding

  lax = _mod("jax.lax")

  def dynamic_update_slice(operand, update, start_indices):
    out = operand.clone()
    sl = []
    for s, n, full in zip(start_indices, update.shape, operand.shape):
      s = int(s)
      s = max(0, min(s, full - n))  # jax clamps start indices
      sl.append(slice(s, s + n))
    out[tuple(sl)] = update.to(out.dtype)
    return JTensor.wrap(out)

  def dynamic_slice_in_dim(operand, start_index, slice_size, axis=0):
    start_index = int(start_index)
    return JTensor.wrap(operand.narrow(axis, start_index, slice_size))

  lax.dynamic_update_slice = dynamic_update_slice
  lax.dynamic_slice_in_dim = dynamic_slice_in_dim
  lax.with_sharding_constraint = lambda x, s: x
  lax.div = lambda a, b: torch.div(a, b, rounding_mode="trunc")
  lax.cond = lambda p, t, f, *ops: t(*ops) if bool(p) else f(*ops)
  jax.lax = lax

  rnd = _mod("jax.random")
  rnd.key = rnd.PRNGKey = rnd.split = rnd.uniform = rnd.normal = _unavailable(
      "jax.random"
  )
  jax.random = rnd

  jnp = _mod("jax.numpy")
  jnp.bfloat16, jnp.float32, jnp.float16 = (
      torch.bfloat16,
      torch.float32,
      torch.float16,
  )
  jnp.int8, jnp.int32, jnp.int64 = torch.int8, torch.int32, torch.int64
  jnp.inf = float("inf")

  def _w(fn):
    return lambda *a, **k: JTensor.wrap(fn(*a, **k))

  def _strip_device(k):
    k.pop("device", None)
    return k

  jnp.arange = lambda *a, **k: JTensor.wrap(torch.arange(*a, **_strip_device(k)))
  jnp.zeros = lambda shape, dtype=torch.float32, **k: JTensor.wrap(
      torch.zeros(tuple(shape), dtype=dtype)
  )
  jnp.ones = lambda shape, dtype=torch.float32, **k: JTensor.wrap(
      torch.ones(tuple(shape), dtype=dtype)
  )
  jnp.full = lambda shape, v, dtype=None, **k: JTensor.wrap(
      torch.full(tuple(shape), v, dtype=dtype)
  )
  jnp.asarray = jnp.array = lambda x, dtype=None: JTensor.wrap(
      torch.as_tensor(np.asarray(x) if not isinstance(x, torch.Tensor) else x)
      if dtype is None
      else torch.as_tensor(
          np.asarray(x) if not isinstance(x, torch.Tensor) else x
      ).to(dtype)
  )
  jnp.reshape = lambda x, shape: JTensor.wrap(x.reshape(tuple(shape)))
  jnp.squeeze = lambda x, axis=None: JTensor.wrap(
      x.squeeze() if axis is None else x.squeeze(axis)
  )
  jnp.expand_dims = lambda x, axis: JTensor.wrap(x.unsqueeze(axis))
  jnp.transpose = lambda x, axes: JTensor.wrap(x.permute(*axes))
  jnp.where = _w(torch.where)
  jnp.logical_and = _w(torch.logical_and)
  jnp.logical_or = _w(torch.logical_or)
  jnp.array_equal = lambda a, b: bool(
      torch.equal(torch.as_tensor(a).float(), torch.as_tensor(b).float())
  )
  jnp.zeros_like = _w(torch.zeros_like)
  jnp.concatenate = lambda xs, axis=0: JTensor.wrap(torch.cat(list(xs), axis))

  def pad(array, pad_width, mode="constant"):
    assert mode == "constant"
    flat = []
    for lo, hi in reversed(pad_width):
      flat += [lo, hi]
    return JTensor.wrap(torch.nn.functional.pad(array, flat))

  jnp.pad = pad
  jax.numpy = jnp

  exp = _mod("jax.experimental")
  jax.experimental = exp
  pallas = _mod("jax.experimental.pallas")
  pallas.pallas_call = _unavailable("pallas")
  pallas.program_id = _unavailable("pallas")
  pallas.when = _unavailable("pallas")
  pallas.BlockSpec = _unavailable("pallas")
  exp.pallas = pallas
  tpu = _mod("jax.experimental.pallas.tpu")
  tpu.PrefetchScalarGridSpec = _unavailable("pallas")
  pallas.tpu = tpu
  _mod("jax.experimental.pallas.ops")
  _mod("jax.experimental.pallas.ops.tpu")
  _mod("jax.experimental.pallas.ops.tpu.paged_attention")
  pak = _mod(
      "jax.experimental.pallas.ops.tpu.paged_attention.paged_attention_kernel"
  )
  pak.paged_attention = _unavailable("pallas paged_attention")
  sm = _mod("jax.experimental.shard_map")
  sm.shard_map = lambda f, mesh=None, in_specs=None, out_specs=None, **k: f
  exp.shard_map = sm

  x2 = _mod("torch_xla2")

  class _Env:

    def __enter__(self):
      return self

    def __exit__(self, *a):
      return False

    def j2t_iso(self, tree):
      return _tree_map(JTensor.wrap, tree)

    t2j_iso = j2t_iso
    to_xla = j2t_iso

  _env = _Env()
  x2.default_env = lambda: _env
  interop = _mod("torch_xla2.interop")
  interop.call_jax = lambda f, *a, **k: f(*a, **k)
  interop.call_torch = lambda f, *a, **k: f(*a, **k)
  x2.interop = interop
  tensor = _mod("torch_xla2.tensor")
  tensor.XLATensor2 = JTensor
  tensor.t2j = JTensor.wrap
  tensor.j2t = JTensor.wrap
  x2.tensor = tensor


def import_reference(reference_root):
  """Returns (cache_manager, page_attention_manager, attention_kernel, quantize)
  imported from `<reference_root>/jetstream_pt` with the shim installed."""
  install()
  if reference_root not in sys.path:
    sys.path.insert(0, reference_root)
  # The package __init__ pulls in the serving engine (absent dependencies);
  # register an empty package object so only the submodules asked for load.
  import importlib
  import os

  pkg = types.ModuleType("jetstream_pt")
  pkg.__path__ = [os.path.join(reference_root, "jetstream_pt")]
  sys.modules["jetstream_pt"] = pkg
  mods = []
  for name in (
      "torchjax",
      "quantize",
      "page_attention_manager",
      "cache_manager",
      "attention_kernel",
  ):
    mods.append(importlib.import_module(f"jetstream_pt.{name}"))
  _, quantize, pam, cm, ak = mods
  return cm, pam, ak, quantize
