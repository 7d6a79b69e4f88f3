"""CPU oracle of the block-scaled GEMM path: test infrastructure only (see blockscaled_oracle)."""
