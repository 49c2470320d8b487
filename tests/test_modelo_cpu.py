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


class _SpecComMaximos(spec.Spec):
    """The oracle with the launcher's fused entry: transpositions that also leave the row maxima in the caller's views (which
    the reducer has pre-set to -128)."""
    usos = 0

    def transpoe2_max(self, X1, X2, R1, R2):
        Y1, Y2 = self.transpoe2(X1, X2)
        assert int(R1.max()) == -128 and int(R2.max()) == -128, "the reducer must hand out slices pre-set to -128"
        R1.copy_(torch.maximum(R1, self.max_linha(Y1)))
        R2.copy_(torch.maximum(R2, self.max_linha(Y2)))
        _SpecComMaximos.usos += 1
        return Y1, Y2


CFG2 = dict(V=256, D=256, H=4, FF=256, L=1)      # every width a multiple of 256: the fused transposition applies
BT2, T2 = 4, 64


def _modelo2(ops_, redutor=None):
    from jatai_b200 import modelo, ops, registro
    ops.BLK = 32
    reg = registro.Registro(tempfile.mkdtemp(), "cpu", eco=False)
    return modelo.Modelo(CFG2["V"], CFG2["D"], CFG2["H"], CFG2["FF"], CFG2["L"], 0, "cpu", ops_, reg, redutor=redutor)


def _lote2(seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, CFG2["V"], (BT2, T2 + 1), generator=g)
    return x[:, :-1].contiguous(), x[:, 1:].contiguous()


def _rank2(rank, mundo, porta, saida):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(porta))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dist.init_process_group("gloo", rank=rank, world_size=mundo)
    from jatai_b200 import paralelo
    m = _modelo2(_SpecComMaximos(32), paralelo.Redutor())
    tok, alvo = _lote2(3)
    fatia = slice(rank * BT2 // mundo, (rank + 1) * BT2 // mundo)
    for _ in range(2):
        m.passo(tok[fatia], alvo[fatia], k_lr=4)
    torch.save({"estado": _estado(m), "usos": _SpecComMaximos.usos}, os.path.join(saida, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_dp_maximos_escritos_no_lugar_pela_transposicao():
    """Data parallel with a launcher that offers transpoe2_max: from the second step on the row maxima of the weight-gradient
    operands are written straight into the reducer's buffer (no max_linha, no copy), and the state stays bit-identical to one
    process on the concatenated batch."""
    saida = tempfile.mkdtemp()
    porta = 31500 + os.getpid() % 2000
    mp.spawn(_rank2, args=(2, porta, saida), nprocs=2, join=True)
    m = _modelo2(spec.Spec(32))
    tok, alvo = _lote2(3)
    for _ in range(2):
        m.passo(tok, alvo, k_lr=4)
    ref = _estado(m)
    for r in range(2):
        d = torch.load(os.path.join(saida, f"r{r}.pt"))
        assert d["usos"] > 0, "the fused transposition was never used"
        for i, (a, b) in enumerate(zip(d["estado"], ref)):
            assert torch.equal(a, b), f"rank {r}: state tensor {i} differs from the single-process run"
