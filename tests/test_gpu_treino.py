"""The training driver end to end on the GPU (small model, synthetic bytes): eager first step, recorded graph,
validation, checkpoint, and a resumed run that continues bit for bit."""
import argparse
import os
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(pasta, **kw):
    a = argparse.Namespace(dados=None, V=256, D=128, H=2, FF=256, L=2, T=64, blk=32, pasta=pasta, salvar=None, retomar=None, eager=False)
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_treinar_salvar_retomar():
    from jatai_b200 import treino
    pasta = tempfile.mkdtemp()
    inteiro, meio = os.path.join(pasta, "inteiro.pt"), os.path.join(pasta, "meio.pt")
    treino.treinar(_args(pasta, salvar=inteiro), 4, 6, 2)                 # 6 steps in one go
    treino.treinar(_args(pasta, salvar=meio), 4, 3, 2)                    # 3 steps, save ...
    retomado = os.path.join(pasta, "retomado.pt")
    treino.treinar(_args(pasta, retomar=meio, salvar=retomado), 4, 6, 2)  # ... resume and do the other 3
    a, b = torch.load(inteiro), torch.load(retomado)
    for grupo in ("pesos", "momento", "residuo"):
        for n in a[grupo]:
            for x, y in zip(a[grupo][n], b[grupo][n]):
                assert torch.equal(x, y), f"{grupo}/{n} differs between the uninterrupted and the resumed run"
    assert torch.equal(a["gerador"], b["gerador"])


def test_velocidade():
    from jatai_b200 import treino
    treino.velocidade(_args(tempfile.mkdtemp()), 2)
