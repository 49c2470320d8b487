"""Data loader (the reference's recipe on a toy corpus) and bit-exact checkpoint / resume, on CPU with the oracle."""
import json
import os
import tempfile

import torch

from oracle import spec


def test_carregar_e_lote():
    from jatai_b200 import dados
    pasta = tempfile.mkdtemp()
    for lingua in ("Portuguese", "English"):
        with open(os.path.join(pasta, f"{lingua}.jsonl"), "w", encoding="utf-8") as fh:
            for i in range(45):
                fh.write(json.dumps({"text": f"{lingua} documento {i} ação"}) + "\n")
    treino, val = dados.carregar(pasta)
    assert treino.dtype == torch.long and int(treino.max()) < 256
    doc0 = "Portuguese documento 0 ação".encode() + b"\n\n"
    assert bytes(val[:len(doc0)].tolist()) == doc0                    # documents 0, 20, 40 of each language validate
    assert len(val) == sum(len(f"{l} documento {i} ação".encode()) + 2 for l in ("Portuguese", "English") for i in (0, 20, 40))
    g = torch.Generator().manual_seed(3)
    x, y = dados.lote(treino, g, 4, 16)
    assert x.shape == (4, 16) and torch.equal(x[:, 1:], y[:, :-1])


def _modelo():
    from jatai_b200 import modelo, ops, registro
    ops.BLK = 32
    reg = registro.Registro(tempfile.mkdtemp(), "ck", eco=False)
    return modelo.Modelo(128, 64, 4, 128, 1, 0, "cpu", spec.Spec(32), reg)


def _estado(m):
    return [t.clone() for n in sorted(m.p) for par in (m.p[n], m.mom[n], m.res[n]) for t in par]


def test_retomar_continua_bit_a_bit():
    from jatai_b200 import dados, estado
    fonte = dados.sintetico(5000, 9) % 128
    a, ga = _modelo(), torch.Generator().manual_seed(1)
    for _ in range(2):
        a.passo(*dados.lote(fonte, ga, 2, 32), k_lr=4)
    arq = os.path.join(tempfile.mkdtemp(), "ck.pt")
    estado.salva(a, arq, 2, ga)
    for _ in range(2):
        a.passo(*dados.lote(fonte, ga, 2, 32), k_lr=4)
    b, gb = _modelo(), torch.Generator().manual_seed(999)
    assert estado.restaura(b, arq, gb) == 2
    for _ in range(2):
        b.passo(*dados.lote(fonte, gb, 2, 32), k_lr=4)
    for i, (x, y) in enumerate(zip(_estado(a), _estado(b))):
        assert torch.equal(x, y), f"state tensor {i} differs after resume"


def test_restaura_le_o_arquivo_de_pesos_da_referencia():
    """The reference's weight file (noite.py:88-91: modo, L, FF, pesos, residuo) loads: weights and residual as stored, momentum
    from zero, step 0, with a warning that the continuation is not bit-exact; a file for another depth is refused."""
    import pytest
    from jatai_b200 import dados, estado, ops
    fonte = dados.sintetico(3000, 5) % 128
    a, ga = _modelo(), torch.Generator().manual_seed(1)
    for _ in range(2):
        a.passo(*dados.lote(fonte, ga, 2, 32), k_lr=4)
    arq = os.path.join(tempfile.mkdtemp(), "ref_pesos.pt")
    torch.save({"modo": "int8", "L": a.L, "FF": a.FF, "pesos": {k: (m.cpu(), e.cpu()) for k, (m, e) in a.p.items()},
                "residuo": {k: (m.cpu(), e.cpu()) for k, (m, e) in a.res.items()}}, arq)
    b = _modelo()
    with pytest.warns(UserWarning, match="not bit-exact"):
        assert estado.restaura(b, arq) == 0
    for n in a.p:
        assert all(torch.equal(x, y) for x, y in zip(a.p[n], b.p[n])) and all(torch.equal(x, y) for x, y in zip(a.res[n], b.res[n]))
        assert int(b.mom[n][0].abs().max()) == 0 and bool((b.mom[n][1] == ops.E_ZERO).all())
    b.passo(*dados.lote(fonte, ga, 2, 32), k_lr=4)                # and the model trains on from there
    torch.save({"modo": "int8", "L": a.L + 1, "FF": a.FF, "pesos": {}, "residuo": {}}, arq)
    with pytest.raises(ValueError):
        estado.restaura(_modelo(), arq)


def test_corpus_no_dispositivo_corta_os_mesmos_lotes():
    """The device-resident corpus draws the windows of the plain loader (same generator, same batches)."""
    from jatai_b200 import dados
    fonte = dados.sintetico(3000, 4)
    c = dados.Corpus(fonte)
    ga, gb = torch.Generator().manual_seed(5), torch.Generator().manual_seed(5)
    for _ in range(3):
        xa, ya = dados.lote(fonte, ga, 3, 24)
        xb, yb = c.lote(gb, 3, 24)
        assert xb.dtype == torch.long and torch.equal(xa, xb) and torch.equal(ya, yb)
