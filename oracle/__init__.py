"""Parity checker for the GEMM path (test infrastructure, never imported by decx_b200)."""
