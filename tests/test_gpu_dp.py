"""Data parallel on real GPUs (needs >= 2): two NCCL ranks, each with half of the sequences, must end two steps with
exactly the weights, momentum and residual of one GPU running the whole batch (one eager step, then two steps
replayed from CUDA graphs with the collectives between the graphs)."""
import os
import sys
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
CFG = dict(V=256, D=128, H=2, FF=256, L=2)
BT, T = 4, 64          # 2 sequences = 128 tokens per rank (the transposition tile is 128 rows)


def _lote(seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, CFG["V"], (BT, T + 1), generator=g)
    return x[:, :-1].contiguous(), x[:, 1:].contiguous()


def _estado(m):
    return [t.detach().cpu().clone() for n in sorted(m.p) for par in (m.p[n], m.mom[n], m.res[n]) for t in par]


def _roda(dev, redutor, fatia):
    from jatai_b200 import modelo, ops, registro
    ops.define_blk(32)
    reg = registro.Registro(tempfile.mkdtemp(), "dp", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    m = modelo.Modelo(CFG["V"], CFG["D"], CFG["H"], CFG["FF"], CFG["L"], 0, dev, oc, reg, redutor=redutor)
    lotes = [_lote(s) for s in (1, 2, 3)]
    reg.novo_passo(0)
    m.passo(lotes[0][0][fatia].to(dev), lotes[0][1][fatia].to(dev), k_lr=4)           # eager
    reg.fim_passo()
    gravado = modelo.PassoGravado(m, fatia.stop - fatia.start, T, 4)                   # then replayed graphs
    for p, (tok, alvo) in enumerate(lotes[1:], 1):
        reg.novo_passo(p)
        gravado(tok[fatia].to(dev), alvo[fatia].to(dev))
        reg.fim_passo()
    return _estado(m)


def _rank(rank, mundo, porta, saida):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(porta), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=mundo, device_id=torch.device("cuda", rank))
    from jatai_b200 import paralelo
    est = _roda(torch.device("cuda", rank), paralelo.Redutor(), slice(rank * BT // mundo, (rank + 1) * BT // mundo))
    torch.save(est, os.path.join(saida, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_dp_nccl_igual_a_uma_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    saida = tempfile.mkdtemp()
    mp.spawn(_rank, args=(2, 29600 + os.getpid() % 2000, saida), nprocs=2, join=True)
    ref = _roda(torch.device("cuda", 0), None, slice(0, BT))
    for r in range(2):
        est = torch.load(os.path.join(saida, f"r{r}.pt"))
        for i, (a, b) in enumerate(zip(est, ref)):
            assert torch.equal(a, b), f"rank {r}: state tensor {i} differs from the single-GPU run"
