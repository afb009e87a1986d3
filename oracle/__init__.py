"""CPU oracle for the KV-cache hot path of jetstream-pytorch.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
package; it exists so that tests, the smoke check and the benchmark's CPU
baseline leg have something independent to compare the CUDA path against.

Every function is a functional (no in-place mutation of its arguments) torch-CPU
or numpy restatement of one reference function and cites the reference lines it
follows (paths relative to the reference project root, e.g.
`jetstream_pt/cache_manager.py:532-537`).

Parity status: PINNED for the quantisers, the dense / int8 cache update and
finalize, the page manager, paged insert / append, dense_attention and
flash_attention -- the restatements are checked bit-for-bit (attention: to fp32
round-off) against vectors produced by executing the reference's own modules
(`tests/golden/make_golden.py`) and against the reference's own known-answer
tests.  UNPINNED for the two Pallas-TPU ragged kernels and the third-party paged
attention kernel, which cannot be executed without JAX; those are restated from
the kernel bodies and cross-checked only against the pinned dense attention.
"""

from oracle.quant import quantize_decode, quantize_insert  # noqa: F401
