"""CPU checker for the MoonPoly GEMM path (test infrastructure only)."""
