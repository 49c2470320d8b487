"""Runs the REFERENCE's own Python callers - its operator API (`ops.OpsCuda`, `OpsConferido`), model (`modelo.Modelo`,
`PassoGravado`), registry and op test list (`teste_ops.py`), staged unmodified under oracle/_ref/jatai_cuda by the oracle's
recipe - on THIS library.  The only change is the one a maintainer makes (the binding stub of the integration notes): the path
the reference hands to ctypes.CDLL is answered with libjatai_b200.so, and jt_blk(128) selects the reference's tensor format.

    python tests/ref_chamadores.py teste_ops | conferir | grafo | erro_grafo

Test infrastructure: started as a child process by tests/test_gpu_referencia.py (the reference's module names - ops, modelo,
registro - would clash with nothing here, but its module-level state is kept out of the test process).  Exit code 0 = passed.
"""
import ctypes
import os
import runpy
import sys
import tempfile

RAIZ = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(RAIZ, "oracle", "_ref", "jatai_cuda")
NOSSA = os.path.join(RAIZ, "jatai_b200", "libjatai_b200.so")

_CDLL = ctypes.CDLL


class CDLLTrocada(_CDLL):
    """ctypes.CDLL that opens this library where the reference asks for its own, and selects block length 128."""

    def __init__(self, nome, *a, **kw):
        troca = isinstance(nome, str) and os.path.basename(nome) == "libjatai.so"
        super().__init__(NOSSA if troca else nome, *a, **kw)
        if troca:
            self.jt_blk.restype = ctypes.c_int
            assert self.jt_blk(128) == 0


def prepara():
    ctypes.CDLL = CDLLTrocada
    sys.path.insert(0, REF)
    os.chdir(tempfile.mkdtemp())          # the reference writes its logs under ./logs


def lote(torch, seed, Bt, T, V=256):
    x = torch.randint(0, V, (Bt, T + 1), generator=torch.Generator().manual_seed(seed))
    return x[:, :-1].contiguous().cuda(), x[:, 1:].contiguous().cuda()


def estado(torch, m):
    return [t.clone() for n in sorted(m.p) for par in (m.p[n], m.mom[n], m.res[n]) for t in par]


def main(modo):
    prepara()
    if modo == "teste_ops":
        # the reference's 53 known-shape cases through its OpsConferido; the script ends with sys.exit(number of failures != 0)
        runpy.run_path(os.path.join(REF, "teste_ops.py"), run_name="__main__")
        return 1                          # not reached: teste_ops.py always calls sys.exit
    import torch
    import ops as O
    from modelo import Modelo, PassoGravado
    from registro import Registro, ErroJatai
    V, D, H, T, FF, L = 256, 256, 64, 128, 1024, 12          # jatai_cuda/treino_cuda.py:31-33
    if modo == "conferir":
        # jatai_cuda/treino_cuda.py:48-60 on random tokens: two full training steps, every operation double-run against OpsRef
        reg = Registro("logs", "conferir", vigiar=True, eco=False)
        ops = O.OpsConferido(reg)
        m = Modelo(V, D, H, FF, L, 0, "cuda", ops, reg)
        for p in range(2):
            reg.novo_passo(p)
            perda = float(m.passo(*lote(torch, 1 + p, 8, T), k_lr=4))
            reg.fim_passo()
            assert perda == perda and 3.0 < perda < 8.0, perda
        n = sum(ops.n.values())
        print(f"conferir: {n} operations identical over 2 steps: " + ", ".join(f"{k} {v}" for k, v in sorted(ops.n.items())))
        assert n == 1044, n              # the count the reference's report states for two steps of this model
        return 0
    if modo == "grafo":
        # eager steps and replays of the reference's PassoGravado leave identical weights, momentum and residual
        def novo(nome):
            reg = Registro("logs", nome, eco=False)
            return Modelo(V, D, H, FF, L, 0, "cuda", O.OpsCuda(reg), reg), reg
        a, rega = novo("eager")
        b, regb = novo("grafo")
        lotes = [lote(torch, s, 8, T) for s in (1, 2, 3)]
        for p, lt in enumerate(lotes):
            rega.novo_passo(p)
            a.passo(*lt, k_lr=4)
            rega.fim_passo()
        regb.novo_passo(0)
        b.passo(*lotes[0], k_lr=4)
        regb.fim_passo()
        g = PassoGravado(b, 8, T, 4)
        for p, lt in enumerate(lotes[1:], 1):
            regb.novo_passo(p)
            g(*lt)
            regb.fim_passo()
        for i, (x, y) in enumerate(zip(estado(torch, a), estado(torch, b))):
            assert torch.equal(x, y), f"state tensor {i}: graph replay differs from eager"
        print(f"grafo: {len(g.lancamentos)} launches recorded; 3 steps eager == 1 eager + 2 replays")
        return 0
    if modo == "erro_grafo":
        # the scenario of jatai_cuda/teste_erro_grafo.py:14-29 (token 300 at (3, 17) inside a replayed graph) on random tokens
        reg = Registro("logs", "erro_grafo", eco=False)
        m = Modelo(V, D, H, FF, L, 0, "cuda", O.OpsCuda(reg), reg)
        tok, alvo = lote(torch, 1, 8, T)
        reg.novo_passo(0)
        m.passo(tok, alvo, k_lr=4)
        reg.fim_passo()
        g = PassoGravado(m, 8, T, 4)
        reg.novo_passo(1)
        g(tok, alvo)
        reg.fim_passo()
        ruim = tok.clone()
        ruim[3, 17] = 300
        reg.novo_passo(2)
        try:
            g(ruim, alvo)
            reg.fim_passo()
        except ErroJatai as e:
            msg = str(e)
            ok = "forward / embedding" in msg and "linha 401, coluna 0" in msg and "valor    : 300" in msg and "embed" in msg
            print(msg)
            return 0 if ok else 1
        print("sentinel not raised")
        return 1
    raise SystemExit(f"unknown mode {modo}")


if __name__ == "__main__":
    sys.exit(main(sys.argv[1]))
