"""Benchmark configuration 3 at its own sizes (16384 tokens x D = 1024, FF = 4096, vocabulary 256, a 12 M-element weight
tensor, block 32): every fused bandwidth op against the int64 oracle evaluated on the GPU, bit for bit.  The small-size table
(tests/casos.py) covers the edge cases; this covers the grids, row counts and 64-bit offsets of the benchmark shapes."""
import tempfile

import pytest
import torch

import casos
from oracle import spec

pytestmark = pytest.mark.gpu
M, D, FF, V = 16384, 1024, 4096, 256
RW, CW = 3072, 4096                      # 12 M elements


@pytest.fixture(scope="module")
def amb():
    from jatai_b200 import ops, registro
    ops.define_blk(32)
    reg = registro.Registro(tempfile.mkdtemp(), "c3", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    reg.novo_passo(0)
    return oc, reg, spec.Spec(32)


def _gpu(t):
    return tuple(x.cuda() for x in t)


def _igual(nome, a, b):
    a, b = casos.plano(a), casos.plano(b)
    assert len(a) == len(b)
    for i, (x, y) in enumerate(zip(a, b)):
        assert x.dtype == y.dtype and x.shape == y.shape and torch.equal(x, y), f"{nome}: output {i} differs ({int((x != y).sum())} of {x.numel()})"


def _fim(reg):
    import ctypes
    torch.cuda.synchronize()
    assert reg.lib.jt_erro_le((ctypes.c_longlong * 6)()) == 0


def test_rms_e_rms_back(amb):
    oc, reg, s = amb
    G = casos.Gen(301, 32)
    x, g = _gpu(G.bloco(M, D, espalha=6, zera=0.05)), _gpu(G.bloco(M, D, e0=-20, espalha=6))
    y, cache = oc.rms(x)
    _igual("rms", (y, cache), s.rms(x))
    _igual("rms_back", oc.rms_back(g, y, cache), s.rms_back(g, y, cache))
    _igual("rms_back_soma", oc.rms_back_soma(x, g, y, cache), s.rms_back_soma(x, g, y, cache))
    _fim(reg)


def test_soma_quant(amb):
    oc, reg, s = amb
    G = casos.Gen(302, 32)
    a, b = _gpu(G.bloco(M, D, espalha=10, zera=0.1)), _gpu(G.bloco(M, D, espalha=10, zera=0.1))
    _igual("soma", oc.soma(a, b), s.soma(a, b))
    c = _gpu(G.cru(M, D))
    _igual("quant", oc.quant(c), s.quant(c))
    _fim(reg)


def test_relu2_e_back(amb):
    oc, reg, s = amb
    G = casos.Gen(303, 32)
    h, g = _gpu(G.bloco(M, FF, zera=0.1)), _gpu(G.bloco(M, FF, e0=-18))
    _igual("relu2", oc.relu2(h), s.relu2(h))
    _igual("relu2_back", oc.relu2_back(g, h), s.relu2_back(g, h))
    _fim(reg)


def test_transpoe(amb):
    oc, reg, s = amb
    x = _gpu(casos.Gen(304, 32).bloco(M, FF, espalha=8, zera=0.1))
    _igual("transpoe", oc.transpoe(x), s.transpoe(x))
    _fim(reg)


def test_softmax_ce_embed_um_quente(amb):
    oc, reg, s = amb
    G = casos.Gen(305, 32)
    lg, alvo = _gpu(G.cru(M, V, bits=22, e0=-20)), G.tok(M, V).cuda()
    _igual("softmax_ce", oc.softmax_ce(lg, alvo), s.softmax_ce(lg, alvo))
    w = _gpu(G.bloco(V, D))
    _igual("embed", oc.embed(w, alvo), s.embed(w, alvo))
    _igual("um_quente", oc.um_quente(alvo, V), s.um_quente(alvo, V))
    _fim(reg)


@pytest.mark.parametrize("ef", [True, False])
def test_momento_peso(amb, ef):
    oc, reg, s = amb
    G = casos.Gen(306, 32)
    gr = _gpu(G.cru(RW, CW, bits=26, e0=-45))
    mom, w, res = G.bloco(RW, CW, e0=-40, zera=0.05), G.bloco(RW, CW, e0=-9), G.bloco(RW, CW, e0=-20, zera=0.1)
    copia = lambda t: tuple(x.clone().cuda() for x in t)
    m_r = s.momento(gr, copia(mom))
    w_r = s.peso(copia(w), m_r, copia(res), 4, ef)
    m_c = oc.momento(gr, copia(mom))
    _igual("momento", m_c, m_r)
    _igual("peso", oc.peso(copia(w), m_c, copia(res), 4, ef), w_r)
    _igual("momento_peso", oc.momento_peso(gr, copia(mom), copia(w), copia(res), 4, ef), (m_r, *w_r))
    _fim(reg)
