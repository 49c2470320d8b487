"""jt_atencao_back_fixo: the attention backward for callers that cannot allocate device memory (for instance a
process whose memory was budgeted and carved up before start-up, or code that runs where cudaMalloc is not
allowed).  It keeps its workspace in a fixed device array inside the library.  Called here through the C ABI with raw
pointers, twice in a row with different problems, and compared bit for bit with jt_atencao_back on the same inputs;
an over-size problem must be refused.  Collected last on purpose."""
import ctypes
import tempfile

import pytest
import torch

import casos

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def test_atencao_back_sem_alocar():
    from jatai_b200 import ops, registro
    ops.define_blk(32)
    reg = registro.Registro(tempfile.mkdtemp(), "fixo", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    lib = oc.lib
    lib.jt_atencao_back_fixo.restype = ctypes.c_int
    reg.novo_passo(0)
    for n, (Bt, T, H, D, limite) in enumerate([(2, 128, 2, 128, 0), (1, 256, 8, 128, 1), (2, 512, 8, 128, 0), (2, 512, 8, 128, 1), (2, 128, 2, 128, 0)]):
        G = casos.Gen(900 + n, 32)
        M = Bt * T
        qkv = tuple(t.cuda() for t in G.bloco(M, 3 * D, espalha=5, zera=0.05))
        go = tuple(t.cuda() for t in G.bloco(M, D, e0=-20, espalha=6))
        _, P = oc.atencao(qkv, Bt, T, H)
        ops.ATENCAO_LIMITE = bool(limite)
        try:
            ref_acc, ref_e = oc.atencao_back(go, qkv, P, Bt, T, H)
        finally:
            ops.ATENCAO_LIMITE = False
        acc = torch.full((M, 3 * D), 12345, dtype=torch.int32, device="cuda")
        e = torch.full((M, 3 * D), -1, dtype=torch.int16, device="cuda")
        rc = lib.jt_atencao_back_fixo(_p(go[0]), _p(go[1]), _p(qkv[0]), _p(qkv[1]), _p(P), _p(acc), _p(e), ctypes.c_int(Bt), ctypes.c_int(T),
                                      ctypes.c_int(H), ctypes.c_int(D), ctypes.c_int(ops.GA), ctypes.c_int(limite), ctypes.c_int(0))
        assert rc == 0, f"call {n}: cudaError {rc}"
        torch.cuda.synchronize()
        assert torch.equal(acc, ref_acc), f"call {n}: accumulators differ from jt_atencao_back"
        assert torch.equal(e, ref_e), f"call {n}: exponents differ from jt_atencao_back"
    # Bt*H*(8+T) = 64*64*1032 ints > 2^20: refused before anything is launched (pointers are never touched)
    rc = lib.jt_atencao_back_fixo(None, None, None, None, None, None, None, ctypes.c_int(64), ctypes.c_int(1024), ctypes.c_int(64),
                                  ctypes.c_int(4096), ctypes.c_int(4), ctypes.c_int(0), ctypes.c_int(0))
    assert rc == 1
    assert lib.jt_erro_le((ctypes.c_longlong * 6)()) == 0
