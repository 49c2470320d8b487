"""The C restatement of the GEMM specification (oracle/gemm_ref.c) pinned to the int64 torch restatement
(oracle/spec.py), which the reference's own fixtures pin in turn.  The C version is the checker at sizes where the
torch one is too slow, so it has to give the same bits: block and raw outputs, a long K with exponents spread by 12,
all-zero blocks, saturated mantissas, external row maxima, a row slab."""
import ctypes
import os
import subprocess

import pytest
import torch

import casos
from oracle import spec

RAIZ = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    so = os.path.join(RAIZ, "oracle", "liboracle_gemm.so")
    subprocess.run(["make", "-C", os.path.join(RAIZ, "oracle")], check=True, capture_output=True)
    l = ctypes.CDLL(so)
    l.oracle_gemm.restype = ctypes.c_int
    return l


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _c_gemm(lib, A, B, blk, cru, RA=None, RB=None, m0=0, m1=None):
    M, K = A[0].shape
    N = B[0].shape[0]
    m1 = M if m1 is None else m1
    if cru:
        acc, e = torch.zeros(M, N, dtype=torch.int32), torch.zeros(M, N, dtype=torch.int16)
        assert lib.oracle_gemm(_p(A[0]), _p(A[1]), _p(B[0]), _p(B[1]), M, N, K, blk, _p(RA), _p(RB), _p(acc), _p(e), None, None, m0, m1) == 0
        return acc, e
    Cm, CE = torch.zeros(M, N, dtype=torch.int8), torch.zeros(M, N // blk, dtype=torch.int8)
    assert lib.oracle_gemm(_p(A[0]), _p(A[1]), _p(B[0]), _p(B[1]), M, N, K, blk, _p(RA), _p(RB), None, None, _p(Cm), _p(CE), m0, m1) == 0
    return Cm, CE


@pytest.mark.parametrize("cru", [False, True])
@pytest.mark.parametrize("blk,M,K,N,esp,zera", [(32, 64, 4096, 128, 12, 0.0), (32, 96, 512, 256, 4, 0.3), (128, 64, 4096, 128, 12, 0.2),
                                                (32, 64, 2048, 128, 0, 0.0), (128, 128, 1024, 256, 6, 0.0)])
def test_c_igual_ao_spec(lib, blk, M, K, N, esp, zera, cru):
    G = casos.Gen(1000 + blk + M + K + N + esp, blk)
    A, B = G.bloco(M, K, espalha=esp, zera=zera), G.bloco(N, K, espalha=esp, zera=zera)
    ref = spec.Spec(blk).gemm(A, B, cru=cru)
    got = _c_gemm(lib, A, B, blk, cru)
    for i, (a, b) in enumerate(zip(got, ref)):
        assert torch.equal(a, b), f"output {i} differs"


def test_c_mantissas_saturadas(lib):
    """Every mantissa +-127 with one common exponent: the largest partial products and no alignment shift at all."""
    G = casos.Gen(5, 32)
    A, B = casos._satura(G.bloco(64, 1024, espalha=0)), casos._satura(G.bloco(128, 1024, espalha=0))
    for cru in (False, True):
        for a, b in zip(_c_gemm(lib, A, B, 32, cru), spec.Spec(32).gemm(A, B, cru=cru)):
            assert torch.equal(a, b)


def test_c_maximos_externos_e_faixa(lib):
    """External row maxima (what a data-parallel rank passes) and a slab of rows: rows outside the slab stay untouched."""
    G = casos.Gen(6, 32)
    A, B = G.bloco(128, 512, espalha=8), G.bloco(128, 512, espalha=8)
    RA = (A[1].amax(1) + 3).to(torch.int8).contiguous()
    RB = (B[1].amax(1) + 1).to(torch.int8).contiguous()
    ref = spec.Spec(32).gemm(A, B, cru=True, RA=RA, RB=RB)
    acc, e = _c_gemm(lib, A, B, 32, True, RA, RB, m0=32, m1=96)
    assert torch.equal(acc[32:96], ref[0][32:96]) and torch.equal(e[32:96], ref[1][32:96])
    assert int(acc[:32].abs().sum()) == 0 and int(acc[96:].abs().sum()) == 0
