"""Loading and comparing the golden fixtures (tests/golden/*.npz + *.json)."""
import hashlib
import json
import os

import numpy as np
import torch

AQUI = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def digest(t):
    a = t.detach().cpu().contiguous().numpy()
    return hashlib.sha256(str(a.dtype).encode() + str(a.shape).encode() + a.tobytes()).hexdigest()


def carrega(blk):
    with open(os.path.join(AQUI, f"ops_b{blk}.json")) as fh:
        meta = json.load(fh)
    arrs = np.load(os.path.join(AQUI, f"ops_b{blk}.npz"))
    return meta, arrs


def confere_saidas(nome, rec, arrs, outs):
    assert len(outs) == len(rec["out"]), f"{nome}: {len(outs)} outputs, fixture has {len(rec['out'])}"
    for i, (t, r) in enumerate(zip(outs, rec["out"])):
        if "sha256" in r:
            assert digest(t) == r["sha256"], f"{nome}: output {i} differs from the reference (digest)"
        else:
            ref = torch.from_numpy(arrs[r["key"]])
            got = t.detach().cpu()
            assert got.dtype == ref.dtype and got.shape == ref.shape, f"{nome}: output {i} {got.dtype}{tuple(got.shape)} vs {ref.dtype}{tuple(ref.shape)}"
            dif = got != ref
            assert not dif.any(), (f"{nome}: output {i}: {int(dif.sum())} of {ref.numel()} differ; first at "
                                   f"{dif.nonzero()[0].tolist()}: got {got[tuple(dif.nonzero()[0])].item()} ref {ref[tuple(dif.nonzero()[0])].item()}")


def confere_entradas(nome, rec, args):
    import casos
    ins = [digest(t) for t in casos.plano([a for a in args if not isinstance(a, (int, bool))])]
    assert ins == rec["in"], f"{nome}: the seeded inputs differ from the ones the fixture was made with"
