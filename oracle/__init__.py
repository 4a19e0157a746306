"""CPU oracle for the quantized block-forward hot path.

TEST INFRASTRUCTURE ONLY.  Everything under this package is a checker: the tests, the
smoke check and the CPU-baseline leg of the benchmark import it; the product path
(`x17ai_b200`) never does and fails loudly when its CUDA library is missing.
`build_ref.py` (not imported here) compiles the reference's own kernels into `_ref/` as a second
checker for the GPU tests.
"""
from . import attn, formats, gemm, rms_norm  # noqa: F401
