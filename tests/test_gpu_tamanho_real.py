"""Parity at the full sizes of the reference benchmarks, where the CPU oracle is too slow to run whole:
  * config 2 GEMM shapes (K up to 16384): row slabs against the C restatement, all rows against a linearity-free
    property (two K halves with common row maxima add up to the full raw GEMM);
  * config 3/5 attention shape (T = 1024, head dim 64): one sequence against the int64 oracle evaluated on the GPU;
  * config 4: three whole training steps of the 12-layer model with every operation double-run against the int64
    oracle evaluated on the GPU."""
import ctypes
import os
import subprocess
import tempfile

import pytest
import torch

import casos
from oracle import spec

pytestmark = pytest.mark.gpu
RAIZ = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def amb():
    from jatai_b200 import ops, registro
    ops.define_blk(32)
    reg = registro.Registro(tempfile.mkdtemp(), "real", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    reg.novo_passo(0)
    yield ops, oc, reg
    oc.lib.jt_gemm_via(0)


def _oraculo_c():
    so = os.path.join(RAIZ, "oracle", "liboracle_gemm.so")
    if not os.path.exists(so):
        subprocess.run(["make", "-C", os.path.join(RAIZ, "oracle")], check=True, capture_output=True)
    lib = ctypes.CDLL(so)
    lib.oracle_gemm.restype = ctypes.c_int
    return lib


def _bloco(R, C, seed):
    g = torch.Generator().manual_seed(seed)
    m = torch.randint(-127, 128, (R, C), generator=g, dtype=torch.int32).to(torch.int8)
    E = torch.randint(-12, -3, (R, C // 32), generator=g).to(torch.int8)
    return m, E


@pytest.mark.parametrize("M,K,N,cru", [(16384, 4096, 4096, False), (16384, 4096, 16384, False), (4096, 16384, 4096, True), (16384, 16384, 4096, False)])
def test_gemm_config2(amb, M, K, N, cru):
    ops, oc, reg = amb
    reg.novo_passo(0)
    A, B = _bloco(M, K, 1), _bloco(N, K, 2)
    Ag, Bg = tuple(t.cuda() for t in A), tuple(t.cuda() for t in B)
    out = oc.gemm(Ag, Bg, cru=cru)
    torch.cuda.synchronize()
    assert reg.lib.jt_erro_le((ctypes.c_longlong * 6)()) == 0
    # slabs of 64 rows at the start, the middle and the end, against the C restatement of the specification
    lib = _oraculo_c()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    for m0 in (0, (M // 2 // 64) * 64 + 64, M - 64):
        m1 = m0 + 64
        if cru:
            acc = torch.zeros(M, N, dtype=torch.int32)
            e = torch.zeros(M, N, dtype=torch.int16)
            assert lib.oracle_gemm(p(A[0]), p(A[1]), p(B[0]), p(B[1]), M, N, K, 32, None, None, p(acc), p(e), None, None, m0, m1) == 0
            assert torch.equal(out[0][m0:m1].cpu(), acc[m0:m1]) and torch.equal(out[1][m0:m1].cpu(), e[m0:m1]), f"rows {m0}..{m1}"
        else:
            Cm = torch.zeros(M, N, dtype=torch.int8)
            CE = torch.zeros(M, N // 32, dtype=torch.int8)
            assert lib.oracle_gemm(p(A[0]), p(A[1]), p(B[0]), p(B[1]), M, N, K, 32, None, None, None, None, p(Cm), p(CE), m0, m1) == 0
            assert torch.equal(out[0][m0:m1].cpu(), Cm[m0:m1]) and torch.equal(out[1][m0:m1].cpu(), CE[m0:m1]), f"rows {m0}..{m1}"
    # every row: the raw GEMM equals the sum of its two K halves computed with the full row maxima
    if cru:
        RA, RB = oc.max_linha(Ag), oc.max_linha(Bg)
        soma = None
        for h in range(2):
            a = (Ag[0][:, h * K // 2:(h + 1) * K // 2].contiguous(), Ag[1][:, h * K // 64:(h + 1) * K // 64].contiguous())
            b = (Bg[0][:, h * K // 2:(h + 1) * K // 2].contiguous(), Bg[1][:, h * K // 64:(h + 1) * K // 64].contiguous())
            acc, e = oc.gemm(a, b, cru=True, RA=RA, RB=RB)
            soma = acc if soma is None else soma + acc
            assert torch.equal(e, out[1])
        assert torch.equal(soma, out[0])


def test_atencao_T1024(amb):
    """Attention forward and backward at T = 1024, head dim 64 (16 heads, D = 1024, 2 sequences) against the int64
    oracle evaluated on the GPU."""
    ops, oc, reg = amb
    reg.novo_passo(0)
    Bt, T, H, D = 2, 1024, 16, 1024
    G = casos.Gen(77, 32)
    qkv = tuple(t.cuda() for t in G.bloco(Bt * T, 3 * D, espalha=4, zera=0.02))
    go = tuple(t.cuda() for t in G.bloco(Bt * T, D, e0=-20, espalha=5))
    s = spec.Spec(32)
    (oc_c, P_c) = oc.atencao(qkv, Bt, T, H)
    g_c = oc.atencao_back(go, qkv, P_c, Bt, T, H)
    torch.cuda.synchronize()
    for b in range(Bt):         # one sequence at a time keeps the oracle's (H, T, T) int64 tensors small
        sl = slice(b * T, (b + 1) * T)
        q1, g1 = tuple(t[sl].contiguous() for t in qkv), tuple(t[sl].contiguous() for t in go)
        (o_r, P_r) = s.atencao(q1, 1, T, H)
        assert torch.equal(oc_c[0][sl], o_r[0]) and torch.equal(oc_c[1][sl], o_r[1]) and torch.equal(P_c[b * H:(b + 1) * H], P_r)
        g_r = s.atencao_back(g1, q1, P_r, 1, T, H)
        assert torch.equal(g_c[0][sl], g_r[0]) and torch.equal(g_c[1][sl], g_r[1])


def test_config4_tres_passos_conferidos(amb):
    """Benchmark configuration 4 (12 layers, D=512, 8 heads, T=256, batch 8): three training steps, every operation checked
    bit for bit against the int64 oracle running on the same GPU."""
    import conferido
    from jatai_b200 import modelo, ops, registro

    class NaGpu(conferido.OpsConferido):
        def __getattr__(self, op):
            fc, fr = getattr(self.c, op), getattr(self.r, op)

            def f(*args, **kw):
                copia = [tuple(t.clone() for t in a) if isinstance(a, tuple) and op in ("momento", "peso", "momento_peso") else a for a in args]
                out_r = fr(*copia, **kw)
                out_c = fc(*args, **kw)
                torch.cuda.synchronize()
                for i, (a, b) in enumerate(zip(casos.plano(out_c), casos.plano(out_r))):
                    assert a.dtype == b.dtype and torch.equal(a, b), f"op '{op}' output {i} differs from the oracle"
                self.n[op] = self.n.get(op, 0) + 1
                return out_c
            return f

    ops.define_blk(32)
    reg = registro.Registro(tempfile.mkdtemp(), "c4", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    m = modelo.Modelo(256, 512, 8, 2048, 12, 0, "cuda", NaGpu(oc, spec.Spec(32)), reg)
    g = torch.Generator().manual_seed(1)
    perdas = []
    for p in range(3):
        x = torch.randint(0, 256, (8, 257), generator=g)
        reg.novo_passo(p)
        perdas.append(float(m.passo(x[:, :-1].contiguous().cuda(), x[:, 1:].contiguous().cuda(), k_lr=4)))
        reg.fim_passo()
    assert all(p == p and 3.0 < p < 7.0 for p in perdas), perdas
    assert m.ops.n["gemm"] >= 3 * 49 and m.ops.n["atencao_back_quant"] == 36
