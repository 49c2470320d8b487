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


# ---------------------------------------------------------------------------------------------- the 600-step trace, data parallel
CFG4 = dict(V=256, D=512, H=8, FF=2048, L=12)
BT4, T4, MARCOS = 8, 256, (100, 300, 600)


def _traco(dev, redutor, fatia, passos=600):
    """Benchmark configuration 4 for `passos` steps (one eager, the rest replayed); digests of the training state at the marks."""
    import gpu_util as gu
    from jatai_b200 import modelo, ops, registro
    ops.define_blk(32)
    reg = registro.Registro(tempfile.mkdtemp(), "dp600", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    m = modelo.Modelo(CFG4["V"], CFG4["D"], CFG4["H"], CFG4["FF"], CFG4["L"], 0, dev, oc, reg, redutor=redutor)
    gravado, marcos = None, {}
    for p in range(passos):
        tok, alvo = gu.lote(1000 + p, BT4, T4, dev="cpu")
        tok, alvo = tok[fatia].to(dev), alvo[fatia].to(dev)
        reg.novo_passo(p)
        if p == 0:
            m.passo(tok, alvo, k_lr=4)
        else:
            if gravado is None:
                gravado = modelo.PassoGravado(m, fatia.stop - fatia.start, T4, 4)
            gravado(tok, alvo)
        reg.fim_passo()
        if p + 1 in MARCOS:
            marcos[p + 1] = gu.digest_estado(m)
    return marcos


def _rank600(rank, mundo, porta, saida):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(porta), NCCL_NVLS_ENABLE="0")
    raiz = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [raiz, os.path.join(raiz, "tests")]
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=mundo, device_id=torch.device("cuda", rank))
    from jatai_b200 import paralelo
    marcos = _traco(torch.device("cuda", rank), paralelo.Redutor(), slice(rank * BT4 // mundo, (rank + 1) * BT4 // mundo))
    torch.save(marcos, os.path.join(saida, f"m{rank}.pt"))
    dist.destroy_process_group()


def test_dp_traco_600_passos():
    """600 steps of configuration 4 on 2 NCCL ranks (4 sequences each) reach, after steps 100, 300 and 600, the state digests
    of one GPU running the 8 sequences (the same seeded batches as tests/test_gpu_traco600.py)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    saida = tempfile.mkdtemp()
    mp.spawn(_rank600, args=(2, 31600 + os.getpid() % 2000, saida), nprocs=2, join=True)
    ref = _traco(torch.device("cuda", 0), None, slice(0, BT4))
    for r in range(2):
        assert torch.load(os.path.join(saida, f"m{r}.pt")) == ref, f"rank {r}: state digests differ from the single-GPU run"
