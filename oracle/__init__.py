"""CPU restatement of tinygrad's quantized-LLM inference hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this
directory: it is the checker that the CUDA path is compared against, and the
timed CPU baseline of the benchmark.  Every function cites the reference
file:line (paths relative to the tinygrad source tree) whose arithmetic it
restates.

Parity pins: the functions here are checked in ``tests/test_oracle.py`` against
(a) golden vectors produced by running the reference itself on its uop
interpreter device (``tests/golden/make_golden.py`` made them), (b) the
reference's own known-answer vectors (test/unit/test_gguf.py:36-40) and
(c) the gguf-py library the reference's tests compare against
(test/unit/test_gguf.py:50-64).  The grouped MXFP8 GEMM + expert routing
composition has no test in the reference: that part is "parity unpinned"
beyond the pinned pieces it is composed of.
"""
