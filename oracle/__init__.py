"""CPU oracle of the NVFP4 hot path: test infrastructure only (see nvfp4_oracle.py)."""
