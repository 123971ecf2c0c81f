"""CPU oracle of the GEMM hot path: test infrastructure only (see opengemm_oracle.py)."""
