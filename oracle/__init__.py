"""CPU restatement of the reference's compressed-KV hot path (numpy).

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this: it is
the checker that the parity tests, the smoke check and the benchmark's CPU
baseline leg compare against or time.  Every function names the reference
lines it follows.

Parity status
-------------
* bit layouts (``layouts``), FP32 attention (``attention``), the unstructured
  FP16 encoder and the K-path Lloyd iteration are pinned against outputs of the
  reference's own CPU-runnable Python (``reskv.reference``,
  ``reskv.compression._encode`` / ``cluster``), stored under ``tests/golden/``
  by ``tests/golden/make_golden.py``.
* the packers that exist in the reference only as CUDA kernels
  (``compress_fp16``, ``compress_structured_int4``, ``compress_quantized``) and
  the V-path Lloyd iteration (CUDA-only ``bmm(out_dtype=)``) cannot run in a
  GPU-less container.  Their restatements are pinned one step removed: what they
  emit is decoded by the reference's own ``reconstruct`` and compared with the
  selection/quantisation rule applied directly (also in the golden files).
  Division is IEEE here, while the reference compiles with ``--use_fast_math``;
  quantised codes whose quotient lies within an ulp of a rounding boundary are
  therefore "parity unpinned".
* cluster *assignments* are not pinned by any reference test (the reference's
  tests inject clustering); the contract restated here is "exact nearest centre,
  lowest index on ties".
"""

from . import attention, encode, kmeans, layouts  # noqa: F401
