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
* MXFP8 / MXFP4: the ue8m0 scale rule (compute_tile_scale) and the scale decode
  (e8m0_to_scale) are pinned against the reference's own C++ functions compiled
  on the host (oracle/build_ref.py -> oracle/_ref, vectors in
  tests/golden/mx.npz: 36864 amax patterns x 3 formats, all 256 scale bytes);
  the dequantizer against the reference's torch `_dequant_mxfp8`; the padded
  row-wise / column-wise / batched layouts against `mxfp8_padded_ref` /
  `mxfp4_padded_ref` of the reference's tests.  The final fp32 -> fp8 / fp4
  rounding is done in the reference by AMD CDNA4 convert instructions whose
  tie rule is in no source file of the reference; the oracle assumes IEEE
  round-to-nearest-even then saturate-to-finite (the OCP MX rule).  PARITY
  UNPINNED for that one step (the convert's tie rule); the reference's own
  round-trip tolerances are what is checked there.
"""
