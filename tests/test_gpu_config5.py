"""Benchmark configuration 5's shape (D = 1024, 16 heads of 64, T = 1024, FF = 4096, 16 sequences = 16384 tokens per GPU, block 32):
two training steps of a 2-layer model with every operation double-run against the int64 oracle evaluated on the GPU (its
attention one sequence at a time), and the full 24 layers replayed from a CUDA graph against eager execution."""
import tempfile

import pytest
import torch

import gpu_util as gu
from oracle import spec

pytestmark = pytest.mark.gpu
V, D, H, FF, Bt, T = 256, 1024, 16, 4096, 16, 1024


def _novo(L, embrulho=None):
    from jatai_b200 import modelo, ops, registro
    ops.define_blk(32)
    reg = registro.Registro(tempfile.mkdtemp(), "c5", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    reg.novo_passo(0)
    return modelo.Modelo(V, D, H, FF, L, 0, "cuda", embrulho(oc) if embrulho else oc, reg), reg


def test_config5_dois_passos_conferidos():
    m, reg = _novo(2, lambda oc: gu.ConferidoNaGpu(oc, spec.Spec(32), por_sequencia=True))
    perdas = []
    for p in range(2):
        reg.novo_passo(p)
        perdas.append(float(m.passo(*gu.lote(11 + p, Bt, T), k_lr=4)))
        reg.fim_passo()
    assert all(3.0 < x < 8.0 for x in perdas), perdas
    n = m.ops.n
    assert n["atencao_quant"] == 4 and n["atencao_back_quant"] == 4 and n["momento_peso"] == 2 * 10 and n["gemm"] >= 2 * (1 + 1 + 4 * 2 + 2 * 2)


def test_config5_grafo_igual_ao_eager_24_camadas():
    from jatai_b200 import modelo
    lotes = [gu.lote(s, Bt, T) for s in (1, 2, 3)]
    a, rega = _novo(24)
    pa = []
    for p, lt in enumerate(lotes):
        rega.novo_passo(p)
        pa.append(float(a.passo(*lt, k_lr=4)))
        rega.fim_passo()
    da = gu.digest_estado(a)
    del a
    torch.cuda.empty_cache()
    b, regb = _novo(24)
    regb.novo_passo(0)
    pb = [float(b.passo(*lotes[0], k_lr=4))]
    regb.fim_passo()
    g = modelo.PassoGravado(b, Bt, T, 4)
    for p, lt in enumerate(lotes[1:], 1):
        regb.novo_passo(p)
        pb.append(float(g(*lt)))
        regb.fim_passo()
    assert pa == pb
    assert gu.digest_estado(b) == da, "graph replay differs from eager execution"
