"""B200-native packed groupwise INT2 / INT4 decode GEMV behind the reference's Linear wrappers.

The package mirrors the part of ``ai_accel_lab`` that sits on the small-M decode path:

  kernels.groupwise_int2 / kernels.groupwise_int4   packed formats, quantisers, dequantisation
  kernels.decode_int2                               ``decode_int2_linear`` (fused M <= 4 GEMV)
  optimize.hybrid_int2 / optimize.hybrid_int4       ``HybridInt2Linear`` / ``HybridInt4Linear``
  runtime_v5                                        StaticCache + compiled (CUDA-graph) decode

All device work goes through one C-ABI shared library of hand-written sm_100a kernels
(``libqgemv_b200.so``, built from ``csrc/`` by ``ai_accel_studio_b200.build``).  There is no
Triton, no backend dispatch and no CPU fallback: computing on a CPU tensor raises.
"""
__version__ = "0.1.0"
