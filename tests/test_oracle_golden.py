"""The oracle (oracle/spec.py) against the fixtures produced by the reference's own OpsRef."""
import json
import os

import pytest

import casos
import golden_util as gu
from oracle import spec


def _ids(blk):
    return [n for n, _, _ in casos.tabela(blk)]


@pytest.mark.parametrize("blk", [128, 32])
def test_fixture_covers_table(blk):
    meta, _ = gu.carrega(blk)
    assert sorted(meta) == sorted(_ids(blk))


@pytest.mark.parametrize("nome,blk,f", casos.tabela(128) + casos.tabela(32), ids=_ids(128) + _ids(32))
def test_spec_matches_reference(nome, blk, f):
    meta, arrs = gu.carrega(blk)
    G = casos.Gen(casos.semente(nome), blk)
    op, args, kw = f(G)
    gu.confere_entradas(nome, meta[nome], args)
    outs = casos.roda(spec.Spec(blk), op, args, kw)
    gu.confere_saidas(nome, meta[nome], arrs, outs)


def test_config1_block32_digests():
    """Benchmark configuration 1 (M=2048, K=N=512, block 32): Y, dX and raw dW of the oracle hash to the reference's."""
    with open(os.path.join(gu.AQUI, "config1_b32.json")) as fh:
        rec = json.load(fh)
    X, W, dY = casos.config1(32)
    assert [gu.digest(t) for t in (*X, *W, *dY)] == rec["in"]
    s = spec.Spec(32)
    assert [gu.digest(t) for t in s.gemm(X, W)] == rec["Y"]
    assert [gu.digest(t) for t in s.gemm(dY, s.transpoe(W))] == rec["dX"]
    assert [gu.digest(t) for t in s.gemm(s.transpoe(dY), s.transpoe(X), cru=True)] == rec["dW"]
