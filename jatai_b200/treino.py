"""Training driver on the CUDA kernels.

    python -m jatai_b200.treino treinar <k> <passos> [Bt] [--dados PASTA] [--D 512 --H 8 --FF 2048 --L 12 --T 256]
                                        [--salvar ARQ] [--retomar ARQ] [--eager]
    python -m jatai_b200.treino velocidade [Bt] [...]

The command line, the log lines and the CSV (`passo,loss_treino,loss_val,tokens_por_s`) are those of the reference's
driver (jatai_cuda/treino_cuda.py:63-165: modes `treinar` and `velocidade`), so its plotting and summary scripts read the
output.  The model size, the block length and the data source, constants over there, are options here; without --dados
(and without $JATAI_DADOS) uniform random bytes stand in for the corpus.  The reference's third mode, `conferir` (every
operation double-run against the specification), lives in tests/: the specification is test infrastructure here.

How a run is organised: a `Sessao` owns model, data and the recorded step.  Step 0 runs eagerly (it sizes workspaces), the
step is then recorded in a CUDA graph and replayed; every `CADA`-th step and the one after it run eagerly again, one with
per-tensor statistics, one with per-operation timing.  The device error record is read after every step.  Validation
every `CADA` steps on fixed batches.  A checkpoint holds weights, momentum, residual and the sampler's generator, so a
resumed run continues bit for bit.
"""
import argparse
import math
import os
import time

import torch

from . import dados as D_, estado, modelo as M_, ops as O, registro as R_

CADA, LOTES_VAL = 100, 8


def _args(argv=None):
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
    return ap.parse_args(argv)


class Sessao:
    """Model + data + recorded step of one run."""

    def __init__(self, a, rotulo, Bt):
        O.define_blk(a.blk)
        os.makedirs(a.pasta, exist_ok=True)
        self.a, self.Bt, self.T = a, Bt, a.T
        self.reg = R_.Registro(a.pasta, rotulo)
        self.ops = O.OpsCuda(self.reg)
        if a.dados:
            self.treino, self.val = D_.carregar(a.dados, dev="cuda", como_corpus=True)
        else:
            self.treino, self.val = D_.Corpus(D_.sintetico(4_000_000, 1), "cuda"), D_.Corpus(D_.sintetico(400_000, 2), "cuda")
        self.m = M_.Modelo(a.V, a.D, a.H, a.FF, a.L, 0, "cuda", self.ops, self.reg)
        self.amostrador = torch.Generator().manual_seed(1)
        self.gravado = None

    def lote(self):
        return self.treino.lote(self.amostrador, self.Bt, self.T)

    def lotes_de_validacao(self):
        g = torch.Generator().manual_seed(123)
        return [self.val.lote(g, 8, self.T) for _ in range(LOTES_VAL)]

    def passo(self, p, k, lote, eager=False, estatisticas=False, perfil=False):
        """One training step; returns (loss, seconds) with the device drained and its error record read."""
        reg, m = self.reg, self.m
        reg.novo_passo(p)
        m.estatisticas, reg.perfil = estatisticas, perfil
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        if eager or self.gravado is None:
            perda = m.passo(*lote, k_lr=k)
        else:
            perda = self.gravado(*lote)
        perda = float(perda)
        reg.fim_passo()
        dt = time.perf_counter() - t0
        if perfil:
            reg.relatorio_tempos(1)
        m.estatisticas, reg.perfil = False, False
        return perda, dt

    def grava(self, k):
        self.gravado = M_.PassoGravado(self.m, self.Bt, self.T, k)

    def valida(self, p, lotes):
        self.reg.novo_passo(p)
        with self.reg.trecho("validacao"):
            total = sum(float(self.m.passo(*b)) for b in lotes)
        self.reg.fim_passo()
        return total / len(lotes)


class _Media:
    def __init__(self):
        self.zera()

    def zera(self):
        self.soma, self.n, self.tokens, self.segundos = 0.0, 0, 0, 0.0

    def junta(self, perda, tokens, segundos):
        self.soma += perda
        self.n += 1
        self.tokens += tokens
        self.segundos += segundos


def treinar(a, k, passos, Bt):
    s = Sessao(a, f"treino_k{k}_bt{Bt}", Bt)
    reg = s.reg
    inicio = estado.restaura(s.m, a.retomar, s.amostrador) if a.retomar else 0
    lotes_val = s.lotes_de_validacao()
    reg.info(f"INT8 training | lr 2^-{k} | {Bt} x {a.T} = {Bt * a.T} tokens per step | steps {inicio}..{passos} | block {a.blk}")
    media, melhor = _Media(), float("inf")
    with open(os.path.join(a.pasta, f"treino_k{k}_bt{Bt}.csv"), "a") as csv:
        if inicio == 0:
            csv.write("passo,loss_treino,loss_val,tokens_por_s\n")
        for p in range(inicio, passos + 1):
            if p % CADA == 0:
                pv = s.valida(p, lotes_val)
                tps, pt = media.tokens / max(media.segundos, 1e-9), media.soma / max(media.n, 1)
                reg.info(f"passo {p:5d} | loss treino {pt:.4f} | loss val {pv:.4f} | {tps:,.0f} tokens/s", loss_val=pv, loss_treino=pt, tps=tps)
                csv.write(f"{p},{pt:.5f},{pv:.5f},{tps:.1f}\n")
                csv.flush()
                if not math.isfinite(pv):
                    reg.falha(f"validation loss is not finite: {pv}")
                if pv > 1.5 * melhor:
                    reg.aviso(f"validation loss rose from {melhor:.4f} to {pv:.4f}: diverging?")
                melhor = min(melhor, pv)
                media.zera()
            if p == passos:
                break
            resto = p % CADA
            perda, dt = s.passo(p, k, s.lote(), eager=resto in (0, 1), estatisticas=resto == 0, perfil=resto == 1)
            if s.gravado is None and not a.eager:
                s.grava(k)
            if not math.isfinite(perda):
                reg.falha(f"training loss is not finite: {perda}")
            media.junta(perda, Bt * a.T, dt)
    if a.salvar:
        estado.salva(s.m, a.salvar, passos, s.amostrador)
        reg.info(f"state saved to {a.salvar}")


def velocidade(a, Bt, n=30):
    """tokens/s of the whole training step (forward + backward + update), eager and replayed from a CUDA graph."""
    s = Sessao(a, f"velocidade_bt{Bt}", Bt)
    lotes = [s.lote() for _ in range(6)]

    def taxa(eager):
        s.passo(0, 4, lotes[0], eager=eager)
        return Bt * a.T * n / sum(s.passo(0, 4, lotes[1 + i % 5], eager=eager)[1] for i in range(n))

    t_eager = taxa(True)
    s.passo(0, 4, lotes[0], eager=True, perfil=True)
    s.reg.novo_passo(0)
    s.grava(4)
    t_grafo = taxa(False)
    # the float32 yard-stick: the same model in plain PyTorch, from the same weights, same batches
    from . import regua
    pf = regua.PassoFloat(s.m, 4)
    pf(*lotes[0])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(n):
        pf(*lotes[1 + i % 5])
    torch.cuda.synchronize()
    t_f32 = Bt * a.T * n / (time.perf_counter() - t0)
    s.reg.info(f"batch {Bt} x {a.T} = {Bt * a.T} tokens | INT8 CUDA {t_eager:,.0f} tokens/s eager, {t_grafo:,.0f} with a CUDA graph | "
               f"float32 PyTorch {t_f32:,.0f} tokens/s | INT8 / float32 = {t_eager / t_f32:.2f}x ({t_grafo / t_f32:.2f}x with the graph)",
               int8=t_eager, int8_grafo=t_grafo, f32=t_f32)
    return t_eager, t_grafo, t_f32


def main(argv=None):
    a = _args(argv)
    if a.modo == "treinar":
        k, passos = a.nums[0], a.nums[1]
        treinar(a, k, passos, a.nums[2] if len(a.nums) > 2 else 8)
    else:
        velocidade(a, a.nums[0] if a.nums else 8)


if __name__ == "__main__":
    main()
