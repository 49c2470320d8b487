"""jatai_b200: the integer-only (INT8 mantissa + block exponent) training hot path of Jatai on B200.

Public surface (mirrors the reference's jatai_cuda package for this path):
  jatai_b200.ops       BLK, E_ZERO, GA, ATENCAO_LIMITE, g_rms, define_blk, OpsCuda
  jatai_b200.registro  Registro, ErroJatai
  jatai_b200.modelo    Modelo, PassoGravado
  jatai_b200.paralelo  data-parallel step with a bit-exact gradient reduction
The compute lives in libjatai_b200.so (hand-written sm_100a CUDA behind a C ABI, include/jatai_b200.h).
"""
from . import ops, registro  # noqa: F401
