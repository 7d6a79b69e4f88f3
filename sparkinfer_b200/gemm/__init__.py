"""GEMM op group: ``blockscaled``, ``mxfp8_linear``, ``block_fp8_linear``,
``tensor_fp8_linear``."""
