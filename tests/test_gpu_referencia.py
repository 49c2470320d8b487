"""The reference's own code as caller and as checker.

(1) Its Python callers, unmodified, on this library: the operator launcher `ops.OpsCuda` + the checked variant
    `OpsConferido` running its op test list (jatai_cuda/teste_ops.py:51-120, 53 cases), two `conferir` steps of its
    `modelo.Modelo` (jatai_cuda/treino_cuda.py:48-60), its `PassoGravado` (modelo.py:143-180) and the sentinel-in-a-graph
    scenario (teste_erro_grafo.py) - each in a child process (tests/ref_chamadores.py).
(2) Its CUDA library (compiled for sm_100a by the oracle's recipe) against this one, operation by operation, through one
    launcher class, in the configuration it supports (block 128, head dimension 4, T = 128): all 18 operations.
Both need oracle/_ref (built where a reference checkout exists; it travels with the repository's built files)."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

import casos

pytestmark = pytest.mark.gpu
RAIZ = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_PY = os.path.join(RAIZ, "oracle", "_ref", "jatai_cuda")
REF_SO = os.path.join(RAIZ, "oracle", "_ref", "libjatai_ref.so")


def _filho(modo, limite_s=900):
    if not os.path.exists(os.path.join(REF_PY, "ops.py")):
        pytest.skip("oracle/_ref/jatai_cuda not staged (needs the reference checkout at build time)")
    r = subprocess.run([sys.executable, os.path.join(RAIZ, "tests", "ref_chamadores.py"), modo], capture_output=True, text=True, timeout=limite_s)
    assert r.returncode == 0, f"{modo}: exit {r.returncode}\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    return r.stdout


def test_teste_ops_da_referencia():
    saida = _filho("teste_ops")
    assert "53 de 53 casos bateram bit a bit" in saida, saida[-2000:]


def test_conferir_da_referencia():
    assert "1044 operations identical" in _filho("conferir")


def test_passo_gravado_da_referencia():
    assert "3 steps eager == 1 eager + 2 replays" in _filho("grafo")


def test_erro_no_grafo_da_referencia():
    _filho("erro_grafo")


# --------------------------------------------------------------------------------------------- library against library
@pytest.fixture(scope="module")
def par():
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libjatai_ref.so not built (needs the reference checkout at build time)")
    from jatai_b200 import ops, registro
    ops.define_blk(128)
    rn = registro.Registro(tempfile.mkdtemp(), "nossa", vigiar=True, eco=False, salvar=False)
    rr = registro.Registro(tempfile.mkdtemp(), "ref", vigiar=True, eco=False, salvar=False)
    ocr = ops.OpsCuda(rr, biblioteca=REF_SO)
    oc = ops.OpsCuda(rn)                 # created last: the module-level library handle is this library's
    rn.novo_passo(0)
    rr.novo_passo(0)
    yield ops, oc, ocr
    ops.define_blk(32)


def _gpu(a):
    if torch.is_tensor(a):
        return a.cuda().contiguous()
    if isinstance(a, tuple):
        return tuple(_gpu(x) for x in a)
    return a


class _ComLimite:
    def __init__(self, ops, oc):
        self._ops, self._oc = ops, oc

    def __getattr__(self, n):
        return getattr(self._oc, n)

    @property
    def limite(self):
        return self._ops.ATENCAO_LIMITE

    @limite.setter
    def limite(self, v):
        self._ops.ATENCAO_LIMITE = bool(v)


# the reference's model size: Bt, T, H, D, FF, V = 8, 128, 64, 256, 1024, 256 (jatai_cuda/teste_ops.py:55); 4 sequences keep it quick
TABELA = [(n, f) for n, _, f in casos.tabela(128, Bt=4, T=128, D=256, FF=1024, V=256, hd=4)]


@pytest.mark.parametrize("nome,f", TABELA, ids=[n for n, _ in TABELA])
def test_biblioteca_da_referencia(par, nome, f):
    """Every case of the table (all 18 operations, the attention pair with exact and upper-bound shifts) on the reference's
    compiled kernels and on this library: identical bits."""
    ops, oc, ocr = par
    G = casos.Gen(casos.semente(nome), 128)
    op, args, kw = f(G)
    a = casos.roda(_ComLimite(ops, oc), op, tuple(_gpu(x) for x in args), kw)
    b = casos.roda(_ComLimite(ops, ocr), op, tuple(_gpu(x) for x in args), kw)
    torch.cuda.synchronize()
    assert len(a) == len(b)
    for i, (x, y) in enumerate(zip(a, b)):
        assert x.dtype == y.dtype and torch.equal(x, y), f"{nome}: output {i} differs from the reference's kernels ({int((x != y).sum())} of {x.numel()})"
