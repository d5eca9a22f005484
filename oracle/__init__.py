"""Test-only CPU oracle for the GEMM path (see gemm_oracle.py).  Not part of the product."""
