"""Builds libjpt_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m jetstream_pytorch_b200.build [--force]
"""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libjpt_b200.so")

SOURCES = [
    "kv_update.cu",
    "prefill_insert.cu",
    "attention_generic.cu",
    "attention_mma.cu",
    "attention_umma.cu",
    "w8a16_linear.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]

# The quantisers must round exactly like the reference: never fast math, and no
# fused multiply-add contraction across the rounding steps in those two files.
EXTRA_FLAGS = {
    "kv_update.cu": ["--fmad=false"],
    "prefill_insert.cu": ["--fmad=false"],
}


def _stale():
  if not os.path.exists(LIB):
    return True
  t = os.path.getmtime(LIB)
  deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
  deps += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
  deps.append(os.path.abspath(__file__))
  return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
  """Compiles every .cu under csrc/ into one shared library; returns its path."""
  if not force and not _stale():
    return LIB
  nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
  objs = []
  build_dir = os.path.join(HERE, "build")
  os.makedirs(build_dir, exist_ok=True)
  procs = []
  for src in SOURCES:
    obj = os.path.join(build_dir, src.replace(".cu", ".o"))
    cmd = [nvcc, *NVCC_FLAGS, *EXTRA_FLAGS.get(src, []), *os.environ.get("JPT_NVCC_FLAGS", "").split(), "-I", INCLUDE, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
      cmd += ["-Xptxas", "-v"]
    procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs.append(obj)
  for src, pr in procs:
    out, _ = pr.communicate()
    if verbose and out:
      print(out)
    if pr.returncode != 0:
      raise RuntimeError(f"nvcc failed on {src}:\n{out}")
  cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
  out = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
  if out.returncode != 0:
    raise RuntimeError(f"link failed:\n{out.stdout}")
  return LIB


if __name__ == "__main__":
  print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
