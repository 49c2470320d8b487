"""Host logic of the training step on CPU: the model code driven by the oracle, and the data-parallel reduction
with two gloo ranks against one process on the concatenated batch (must be bit-identical)."""
import os
import sys
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import spec

CFG = dict(V=128, D=64, H=4, FF=128, L=2)       # head dimension 16, block 32
BT, T = 4, 32


def _modelo(redutor=None):
    from jatai_b200 import modelo, ops, registro
    ops.BLK = 32
    reg = registro.Registro(tempfile.mkdtemp(), "cpu", eco=False)
    return modelo.Modelo(CFG["V"], CFG["D"], CFG["H"], CFG["FF"], CFG["L"], 0, "cpu", spec.Spec(32), reg, redutor=redutor)


def _lote(seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, CFG["V"], (BT, T + 1), generator=g)
    return x[:, :-1].contiguous(), x[:, 1:].contiguous()


def _estado(m):
    return [t.clone() for n in sorted(m.p) for par in (m.p[n], m.mom[n], m.res[n]) for t in par]


def test_passo_no_oraculo_muda_pesos_e_reduz_perda():
    m = _modelo()
    tok, alvo = _lote(1)
    antes = _estado(m)
    p0 = float(m.passo(tok, alvo, k_lr=4))
    for _ in range(3):
        m.passo(tok, alvo, k_lr=4)
    p1 = float(m.passo(tok, alvo))
    assert any(not torch.equal(a, b) for a, b in zip(antes, _estado(m)))
    assert p1 < p0, f"loss did not go down on a repeated batch: {p0} -> {p1}"
    assert abs(p0 - 4.85) < 0.5          # ~ln(128) at initialisation


def _rank(rank, mundo, porta, saida):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(porta))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dist.init_process_group("gloo", rank=rank, world_size=mundo)
    from jatai_b200 import paralelo
    m = _modelo(paralelo.Redutor())
    tok, alvo = _lote(1)
    fatia = slice(rank * BT // mundo, (rank + 1) * BT // mundo)
    perdas = []
    for _ in range(2):
        perdas.append(float(paralelo.media_da_perda(m.passo(tok[fatia], alvo[fatia], k_lr=4))))
    torch.save({"estado": _estado(m), "perdas": perdas}, os.path.join(saida, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_dp_duas_ranks_igual_a_um_processo():
    saida = tempfile.mkdtemp()
    porta = 29500 + os.getpid() % 2000
    mp.spawn(_rank, args=(2, porta, saida), nprocs=2, join=True)
    m = _modelo()
    tok, alvo = _lote(1)
    perdas = [float(m.passo(tok, alvo, k_lr=4)) for _ in range(2)]
    ref = _estado(m)
    for r in range(2):
        d = torch.load(os.path.join(saida, f"r{r}.pt"))
        assert len(d["estado"]) == len(ref)
        for i, (a, b) in enumerate(zip(d["estado"], ref)):
            assert torch.equal(a, b), f"rank {r}: state tensor {i} differs from the single-process run"
        assert all(abs(a - b) < 1e-9 for a, b in zip(d["perdas"], perdas))


def test_regua_float_acompanha_o_modelo_inteiro():
    """The float32 yard-stick starts from the integer model's weights: its loss at initialisation is the integer model's
    (up to the integer rounding), and one of its SGD steps lowers it on a repeated batch."""
    from jatai_b200 import regua
    m = _modelo()
    tok, alvo = _lote(1)
    p_int = float(m.passo(tok, alvo))
    pf = regua.PassoFloat(m, 4)
    p_f = float(pf.m(tok, alvo))
    assert abs(p_f - p_int) < 0.05, (p_f, p_int)
    for _ in range(3):
        pf(tok, alvo)
    assert float(pf.m(tok, alvo)) < p_f
