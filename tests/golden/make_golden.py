"""Generate the golden fixtures by running the REFERENCE's own int64 specification.

Run in a container that has the reference checkout (it is imported, never copied):

    python tests/golden/make_golden.py /path/to/reference

For every case of tests/casos.py the reference `OpsRef` (jatai_cuda/ops.py:92-290) is executed on the
seeded inputs and its outputs are stored:
  * ops_b128.npz : the reference exactly as shipped (BLK = 128).
  * ops_b32.npz  : the same code with its block constant set to 32 (ops.BLK = 32 and the bound default
                   of ops.expande, the only two places the constant is captured).
  * config1_b32.json : SHA-256 of every output of benchmark configuration 1 (M=2048, K=N=512, block 32).
Outputs larger than 32 KiB are stored as SHA-256 digests; input digests are stored for all cases so a
change in the random generator is detected instead of silently comparing different inputs.
"""
import hashlib
import json
import os
import sys

import numpy as np
import torch

AQUI = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(AQUI))
import casos  # noqa: E402


def digest(t):
    a = t.detach().cpu().contiguous().numpy()
    return hashlib.sha256(str(a.dtype).encode() + str(a.shape).encode() + a.tobytes()).hexdigest()


class Adaptador:
    """The reference's OpsRef plus the `limite` switch, which the reference keeps in a module global."""

    def __init__(self, O):
        self._O, self._r = O, O.OpsRef()

    def __getattr__(self, n):
        return getattr(self._r, n)

    @property
    def limite(self):
        return self._O.ATENCAO_LIMITE

    @limite.setter
    def limite(self, v):
        self._O.ATENCAO_LIMITE = bool(v)


def define_blk(O, blk):
    O.BLK = blk
    O.expande.__defaults__ = (blk,)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <reference checkout>")
    ref = sys.argv[1]
    sys.path.insert(0, os.path.join(ref, "jatai_cuda"))
    import ops as O
    ops = Adaptador(O)
    for blk in (128, 32):
        define_blk(O, blk)
        arrs, meta = {}, {}
        for nome, b, f in casos.tabela(blk):
            G = casos.Gen(casos.semente(nome), b)
            op, args, kw = f(G)
            outs = casos.roda(ops, op, args, kw)
            ins = [digest(t) for t in casos.plano([a for a in args if not isinstance(a, (int, bool))])]
            rec = {"op": op, "in": ins, "out": []}
            for i, t in enumerate(outs):
                if t.numel() * t.element_size() > 32768:
                    rec["out"].append({"sha256": digest(t)})
                else:
                    k = f"{nome}#{i}"
                    arrs[k] = t.cpu().numpy()
                    rec["out"].append({"key": k})
            meta[nome] = rec
            print(f"  {nome}: {op} -> {len(outs)} outputs")
        np.savez_compressed(os.path.join(AQUI, f"ops_b{blk}.npz"), **arrs)
        with open(os.path.join(AQUI, f"ops_b{blk}.json"), "w") as fh:
            json.dump(meta, fh, indent=1, sort_keys=True)
    # benchmark configuration 1 at block 32: Y = X.W^T, dX = dY.T(W)^T, dW = T(dY).T(X)^T raw (modelo.py:110-113)
    define_blk(O, 32)
    X, W, dY = casos.config1(32)
    r = O.OpsRef()
    Y = r.gemm(X, W)
    dX = r.gemm(dY, r.transpoe(W))
    dW = r.gemm(r.transpoe(dY), r.transpoe(X), cru=True)
    rec = {"in": [digest(t) for t in (*X, *W, *dY)],
           "Y": [digest(t) for t in Y], "dX": [digest(t) for t in dX], "dW": [digest(t) for t in dW]}
    with open(os.path.join(AQUI, "config1_b32.json"), "w") as fh:
        json.dump(rec, fh, indent=1, sort_keys=True)
    define_blk(O, 128)
    print("fixtures written to", AQUI)


if __name__ == "__main__":
    main()
