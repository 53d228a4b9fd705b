"""CPU oracle for the low-precision GEMM path. TEST INFRASTRUCTURE ONLY.

This package restates, in numpy, the arithmetic of the reference's quantize /
dequantize kernels and the fp32 reference GEMMs they are checked against.  It
is the checker for the CUDA kernels: only the test-suite, the smoke check and
the benchmark's CPU-baseline leg may import it.  The product package never
does; it fails loudly when its CUDA library is missing.

Pinning status (what the restatement has been checked against):

* tensorwise / rowwise FP8: pinned against golden vectors produced by the
  reference's own pure-torch reference (tests/pytorch/ref/quantization_ref.py)
  -- see tests/golden/make_golden.py.
* blockwise FP8 (1-D, dual, 128x128 weight, segment-M): pinned against golden
  vectors produced by running the reference's own Triton kernels
  (primus_turbo/triton/quantization/quant_blockwise.py) under the Triton CPU
  interpreter.
* blockwise / tensorwise / rowwise GEMM semantics: pinned (to fp32 tolerance)
  against the reference's Triton GEMM kernels under the same interpreter.
* MXFP8 / MXFP4 (ue8m0 scale, e4m3 / e5m2 / e2m1 conversion): the scale
  computation is restated bit for bit from the kernel source; the final
  fp32 -> fp8 / fp4 rounding is done in the reference by AMD CDNA4 convert
  instructions whose tie rule is in no source file of the reference.  The
  oracle assumes IEEE round-to-nearest-even then saturate-to-finite (the OCP
  MX rule).  PARITY UNPINNED for that rounding step; the reference's own
  round-trip tolerances are what is checked.
"""
