"""CPU oracle for the quantized-linear path (TEST INFRASTRUCTURE, not product code).

Everything under ``oracle/`` is a numpy / torch-CPU restatement of the reference's
quantize -> pack -> block-scaled GEMM -> epilogue arithmetic.  It exists only to check
the CUDA path: ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import it; the product package never does.

Parity status per format
------------------------
* ``rowscale`` (per-row UE8M0) and ``blk16`` (per 16-column UE8M0, row-pair on the A side):
  PINNED.  ``tests/golden/make_golden.py`` runs the reference's own Triton quantizers
  (``veloxvoice/kernels/ops/triton_ops.py:8-124,169-293``) and ``mxfp4_dequant``
  (``triton_ops.py:296-309``) through Triton's CPU interpreter and stores their bytes
  in ``tests/golden/*.npz``; ``tests/test_oracle_golden.py`` checks this oracle against them.
* ``mx32``, ``nv16``, ``fp8_1x128``: the reference has no code for these formats, so
  PARITY UNPINNED at the reference.  They are defined here by extension of the reference's
  E2M1 rounding rule and scale rule, and pinned only by this oracle's own fixtures.
"""
