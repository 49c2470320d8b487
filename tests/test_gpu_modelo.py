"""The whole training step on the GPU: every operation of two steps double-run against the oracle, the CUDA-graph
replay against eager execution, and the device sentinel inside a replayed graph."""
import tempfile

import pytest
import torch

from oracle import spec

pytestmark = pytest.mark.gpu
CFG = dict(V=256, D=128, H=2, FF=256, L=2)      # head dimension 64, block 32
BT, T = 2, 64


def _lote(seed, dev="cuda"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, CFG["V"], (BT, T + 1), generator=g)
    return x[:, :-1].contiguous().to(dev), x[:, 1:].contiguous().to(dev)


def _novo(ops_obj=None, vigiar=False):
    from jatai_b200 import modelo, ops, registro
    ops.define_blk(32)
    reg = registro.Registro(tempfile.mkdtemp(), "m", vigiar=vigiar, eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    reg.novo_passo(0)
    m = modelo.Modelo(CFG["V"], CFG["D"], CFG["H"], CFG["FF"], CFG["L"], 0, "cuda", ops_obj(oc) if ops_obj else oc, reg)
    return m, reg, oc


def _estado(m):
    return [t.clone() for n in sorted(m.p) for par in (m.p[n], m.mom[n], m.res[n]) for t in par]


def test_passo_conferido():
    """Two full steps (forward, backward, optimiser) with every operation checked bit for bit against the oracle."""
    import conferido
    m, reg, oc = _novo(lambda oc: conferido.OpsConferido(oc, spec.Spec(32)), vigiar=True)
    tok, alvo = _lote(1)
    for p in range(2):
        reg.novo_passo(p)
        perda = float(m.passo(tok, alvo, k_lr=4))
        reg.fim_passo()
        assert perda == perda and perda < 10
    n = m.ops.n
    assert n["gemm"] >= 2 * (1 + 1 + 4 * CFG["L"] + CFG["L"] * 2) and n["atencao_quant"] == 2 * CFG["L"] and n["momento_peso"] == 2 * (4 * CFG["L"] + 2)


def test_grafo_igual_ao_eager():
    from jatai_b200 import modelo
    a, rega, _ = _novo()
    b, regb, _ = _novo()
    lotes = [_lote(s) for s in (1, 2, 3)]
    pa = []
    for p, (tok, alvo) in enumerate(lotes):
        rega.novo_passo(p)
        pa.append(float(a.passo(tok, alvo, k_lr=4)))
        rega.fim_passo()
    regb.novo_passo(0)
    pb = [float(b.passo(*lotes[0], k_lr=4))]
    regb.fim_passo()
    g = modelo.PassoGravado(b, BT, T, 4)
    for p, (tok, alvo) in enumerate(lotes[1:], 1):
        regb.novo_passo(p)
        pb.append(float(g(tok, alvo)))
        regb.fim_passo()
    assert pa == pb
    for i, (x, y) in enumerate(zip(_estado(a), _estado(b))):
        assert torch.equal(x, y), f"state tensor {i}: graph replay differs from eager"


def test_sentinela_dentro_do_grafo():
    """An invalid token in a replayed graph is reported with operation, section and position (the reference's
    teste_erro_grafo.py); the kernels record and go on, nothing traps."""
    from jatai_b200 import modelo
    from jatai_b200.registro import ErroJatai
    m, reg, _ = _novo()
    tok, alvo = _lote(1)
    reg.novo_passo(0)
    m.passo(tok, alvo, k_lr=4)
    reg.fim_passo()
    g = modelo.PassoGravado(m, BT, T, 4)
    ruim = tok.clone()
    ruim[1, 17] = 300
    reg.novo_passo(1)
    g(ruim, alvo)
    with pytest.raises(ErroJatai) as ei:
        reg.fim_passo()
    msg = str(ei.value)
    assert "embed" in msg and "forward / embedding" in msg and f"linha {T + 17}, coluna 0" in msg and "300" in msg
