"""Training driver on the CUDA kernels: the `treinar` and `velocidade` modes of the reference's
jatai_cuda/treino_cuda.py (:63-116, :119-165) with the model size, block length and data source as options.

    python -m jatai_b200.treino treinar <k> <passos> [Bt] [--dados PASTA] [--D 512 --H 8 --FF 2048 --L 12 --T 256]
                                        [--salvar ARQ] [--retomar ARQ] [--eager]
    python -m jatai_b200.treino velocidade [Bt] [...]

Without --dados (and without $JATAI_DADOS) uniform random bytes stand in for the corpus.  One step in a hundred runs
eagerly with statistics or per-operation timing; the others replay the recorded CUDA graph.  The device error record
is read after every step.  (The reference's `conferir` mode - every operation double-run against the specification -
lives in tests/, because the specification is test infrastructure here.)
"""
import argparse
import math
import os
import time

import torch

from . import dados as D_, estado, modelo as M_, ops as O, registro as R_

EVAL_CADA, N_EVAL, STAT_CADA = 100, 8, 100


def _args():
    ap = argparse.ArgumentParser()
    ap.add_argument("modo", choices=["treinar", "velocidade"])
    ap.add_argument("nums", nargs="*", type=int)
    ap.add_argument("--dados", default=os.environ.get("JATAI_DADOS"))
    for n, v in (("V", 256), ("D", 512), ("H", 8), ("FF", 2048), ("L", 12), ("T", 256), ("blk", 32)):
        ap.add_argument(f"--{n}", type=int, default=v)
    ap.add_argument("--pasta", default="logs")
    ap.add_argument("--salvar")
    ap.add_argument("--retomar")
    ap.add_argument("--eager", action="store_true")
    return ap.parse_args()


def _fontes(a):
    if a.dados:
        return D_.carregar(a.dados)
    return D_.sintetico(4_000_000, 1), D_.sintetico(400_000, 2)


def treinar(a, k, passos, Bt):
    O.define_blk(a.blk)
    reg = R_.Registro(a.pasta, f"treino_k{k}_bt{Bt}")
    ops = O.OpsCuda(reg)
    treino, val = _fontes(a)
    m = M_.Modelo(a.V, a.D, a.H, a.FF, a.L, 0, "cuda", ops, reg)
    ger = torch.Generator().manual_seed(1)
    p0 = estado.restaura(m, a.retomar, ger) if a.retomar else 0
    ger_val = torch.Generator().manual_seed(123)
    lotes_val = [D_.lote(val, ger_val, 8, a.T, "cuda") for _ in range(N_EVAL)]
    reg.info(f"INT8 training | lr 2^-{k} | {Bt} x {a.T} = {Bt * a.T} tokens per step | steps {p0}..{passos} | block {a.blk}")
    csv = open(os.path.join(a.pasta, f"treino_k{k}_bt{Bt}.csv"), "a")
    if p0 == 0:
        csv.write("passo,loss_treino,loss_val,tokens_por_s\n")
    acum = n_acum = tok_cont = 0
    t_treino, melhor, grafo = 0.0, float("inf"), None
    for p in range(p0, passos + 1):
        if p % EVAL_CADA == 0:
            reg.novo_passo(p)
            with reg.trecho("validacao"):
                pv = float(sum(m.passo(*b) for b in lotes_val)) / N_EVAL
            reg.fim_passo()
            tps, pt = tok_cont / max(t_treino, 1e-9), acum / max(n_acum, 1)
            reg.info(f"passo {p:5d} | loss treino {pt:.4f} | loss val {pv:.4f} | {tps:,.0f} tokens/s", loss_val=pv, loss_treino=pt, tps=tps)
            csv.write(f"{p},{pt:.5f},{pv:.5f},{tps:.1f}\n")
            csv.flush()
            if not math.isfinite(pv):
                reg.falha(f"validation loss is not finite: {pv}")
            if pv > 1.5 * melhor:
                reg.aviso(f"validation loss rose from {melhor:.4f} to {pv:.4f}: diverging?")
            melhor = min(melhor, pv)
            acum = n_acum = tok_cont = 0
            t_treino = 0.0
        if p == passos:
            break
        reg.novo_passo(p)
        tok, alvo = D_.lote(treino, ger, Bt, a.T, "cuda")
        normal = grafo is None or p % STAT_CADA in (0, 1)
        m.estatisticas = p % STAT_CADA == 0
        reg.perfil = p % STAT_CADA == 1
        torch.cuda.synchronize()
        t0 = time.time()
        perda = float(m.passo(tok, alvo, k_lr=k) if normal else grafo(tok, alvo))
        if grafo is None and not a.eager:
            reg.fim_passo()
            grafo = M_.PassoGravado(m, Bt, a.T, k)
        reg.fim_passo()                              # synchronises and reads the kernels' sentinel record
        t_treino += time.time() - t0
        if reg.perfil:
            reg.relatorio_tempos(1)
        if not math.isfinite(perda):
            reg.falha(f"training loss is not finite: {perda}")
        acum += perda
        n_acum += 1
        tok_cont += Bt * a.T
    csv.close()
    if a.salvar:
        estado.salva(m, a.salvar, passos, ger)
        reg.info(f"state saved to {a.salvar}")


def velocidade(a, Bt):
    """tokens/s of the whole training step (forward + backward + update), eager and replayed from a CUDA graph."""
    O.define_blk(a.blk)
    reg = R_.Registro(a.pasta, f"velocidade_bt{Bt}")
    ops = O.OpsCuda(reg)
    treino, _ = _fontes(a)
    ger = torch.Generator().manual_seed(1)
    lotes = [D_.lote(treino, ger, Bt, a.T, "cuda") for _ in range(6)]
    m = M_.Modelo(a.V, a.D, a.H, a.FF, a.L, 0, "cuda", ops, reg)

    def mede(f, n=30):
        f(lotes[0])
        torch.cuda.synchronize()
        t0 = time.time()
        for i in range(n):
            f(lotes[1 + i % 5])
        torch.cuda.synchronize()
        return Bt * a.T * n / (time.time() - t0)

    def passo_eager(b):
        reg.novo_passo(0)
        m.passo(*b, k_lr=4)
        reg.fim_passo()
    t_eager = mede(passo_eager)
    reg.perfil = True
    passo_eager(lotes[0])
    reg.relatorio_tempos(1)
    reg.perfil = False
    reg.novo_passo(0)
    grafo = M_.PassoGravado(m, Bt, a.T, 4)

    def passo_grafo(b):
        reg.novo_passo(0)
        grafo(*b)
        reg.fim_passo()
    t_grafo = mede(passo_grafo)
    reg.info(f"batch {Bt} x {a.T} = {Bt * a.T} tokens | INT8 CUDA {t_eager:,.0f} tokens/s eager, {t_grafo:,.0f} with a CUDA graph",
             int8=t_eager, int8_grafo=t_grafo)


def main():
    a = _args()
    os.makedirs(a.pasta, exist_ok=True)
    if a.modo == "treinar":
        k, passos = a.nums[0], a.nums[1]
        treinar(a, k, passos, a.nums[2] if len(a.nums) > 2 else 8)
    else:
        velocidade(a, a.nums[0] if a.nums else 8)


if __name__ == "__main__":
    main()
