"""The 600-step regression of the reference (jatai_cuda/RELATORIO_TECNICO.md:784-790: the same run must give the same numbers
with the graph on or off), on benchmark configuration 4 with seeded random byte tokens standing in for the corpus:
  * run A replays the recorded CUDA graph, except steps 0, 1, 100, 300 and 599, which run eagerly with every operation
    double-run against the int64 oracle on the GPU (the reference's `conferir`);
  * run B executes all 600 steps eagerly, unchecked.
Both must reach identical state digests (weights + momentum + residual) after steps 100, 300 and 600 and identical loss traces."""
import tempfile

import pytest
import torch

import gpu_util as gu
from oracle import spec

pytestmark = pytest.mark.gpu
CFG = dict(V=256, D=512, H=8, FF=2048, L=12)
Bt, T, K_LR, PASSOS = 8, 256, 4, 600
CONFERIDOS = (0, 1, 100, 300, 599)
MARCOS = (100, 300, 600)


def _novo():
    from jatai_b200 import modelo, ops, registro
    ops.define_blk(32)
    reg = registro.Registro(tempfile.mkdtemp(), "t600", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    reg.novo_passo(0)
    return modelo.Modelo(CFG["V"], CFG["D"], CFG["H"], CFG["FF"], CFG["L"], 0, "cuda", oc, reg), reg, oc


def _lote(p):
    return gu.lote(1000 + p, Bt, T)


def test_traco_600_passos():
    from jatai_b200 import modelo
    a, rega, oca = _novo()
    conferido = gu.ConferidoNaGpu(oca, spec.Spec(32))
    grafo, perdas_a, marcos_a = None, [], {}
    for p in range(PASSOS):
        rega.novo_passo(p)
        if p in CONFERIDOS:
            a.ops = conferido
            perda = a.passo(*_lote(p), k_lr=K_LR)
            a.ops = oca
        else:
            if grafo is None:
                grafo = modelo.PassoGravado(a, Bt, T, K_LR)
            perda = grafo(*_lote(p))
        perdas_a.append(float(perda))
        rega.fim_passo()
        if p + 1 in MARCOS:
            marcos_a[p + 1] = gu.digest_estado(a)
    assert sum(conferido.n.values()) == len(CONFERIDOS) * sum(conferido.n.values()) // len(CONFERIDOS) > 0
    del grafo, a
    torch.cuda.empty_cache()
    b, regb, _ = _novo()
    perdas_b, marcos_b = [], {}
    for p in range(PASSOS):
        regb.novo_passo(p)
        perdas_b.append(float(b.passo(*_lote(p), k_lr=K_LR)))
        regb.fim_passo()
        if p + 1 in MARCOS:
            marcos_b[p + 1] = gu.digest_estado(b)
    assert marcos_a == marcos_b, f"state digests differ: {marcos_a} vs {marcos_b}"
    assert perdas_a == perdas_b
    assert all(x == x for x in perdas_a) and perdas_a[-1] < perdas_a[0] + 0.5
