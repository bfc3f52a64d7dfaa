"""Packed groupwise formats and the fused decode GEMV entry points."""
