"""Launch registry and diagnostics for the integer training kernels.

Host-side counterpart of the reference's jatai_cuda/registro.py with the same public names, so the
operator classes and `modelo.py`-style callers are interchangeable:

    Registro(pasta, nome, lib=None, vigiar=False, perfil=False, eco=True)
      .trecho(nome)            context manager: section label stack ("forward / camada 3 / mlp")
      .novo_passo(p)           start a step: forget the launch list, clear the device error record
      .registra(op, ent, forma) -> kid     called before a launch; kid is passed to the kernel
      .depois(kid, cuda_rc)    called after it: checks the return code (and the device record when vigiar)
      .confere_device()        read the device error record (synchronises) and raise ErroJatai on a sentinel
      .fim_passo()             once per step: confere_device + accumulate per-op times when perfil
      .confere_bloco / .confere_cru / .exige / .falha / .aviso / .info / .estatistica / .relatorio_tempos
    ErroJatai                  the exception every check raises

What differs from the reference: the exponent block length comes from `ops.BLK` at call time (the reference
hard-codes 128 at registro.py:171-173,202), sentinel code 7 (a bounded wait inside a kernel expired) is known,
and dumping a failing kernel's inputs to disk can be switched off (`salvar=False`).
"""
import contextlib
import ctypes
import json
import os
import time

import torch

# device sentinel codes (jatai_cuda/registro.py:28-35 for 1..6)
CODIGOS = {
    1: "accumulator reached 2^30 (would overflow the int32 register)",
    2: "block exponent above 126 (INT8 exponent overflow; below -126 a block is flushed to zero)",
    3: "mantissa outside +-127 even after raising the exponent",
    4: "division by zero (softmax sum <= 0)",
    5: "left shift would lose bits (result >= 2^30)",
    6: "invalid argument (token or target outside the vocabulary)",
    7: "a bounded wait inside a kernel expired (pipeline stalled); that kernel's output is invalid",
}


class ErroJatai(RuntimeError):
    """Raised by every check of the registry; the message names step, section, operation and position."""


def _bloco():
    from . import ops
    return ops.BLK


def _formas(entradas):
    return {k: (tuple(v.shape) if torch.is_tensor(v) else v) for k, v in entradas.items()}


def _defeitos_bloco(t, blk):
    """List of format defects of a (mantissa, exponent) pair; empty when it is a valid block tensor."""
    m, E = t
    if not (torch.is_tensor(m) and torch.is_tensor(E)):
        return [f"expected two tensors, got {type(m).__name__} and {type(E).__name__}"]
    d = []
    for nome, x in (("mantissa", m), ("exponent", E)):
        if x.dtype != torch.int8:
            d.append(f"{nome} dtype {x.dtype} (expected int8)")
        if not x.is_cuda:
            d.append(f"{nome} not on the GPU")
        if not x.is_contiguous():
            d.append(f"{nome} not contiguous")
    if m.dim() != 2:
        d.append(f"mantissa has {m.dim()} dimensions (expected 2)")
    elif m.shape[1] % blk:
        d.append(f"{m.shape[1]} columns is not a multiple of the block length {blk}")
    elif tuple(E.shape) != (m.shape[0], m.shape[1] // blk):
        d.append(f"exponent shape {tuple(E.shape)}, expected {(m.shape[0], m.shape[1] // blk)}")
    return d


def _defeitos_cru(t):
    acc, e = t
    d = []
    if acc.dtype != torch.int32:
        d.append(f"accumulator dtype {acc.dtype} (expected int32)")
    if e.dtype != torch.int16:
        d.append(f"exponent dtype {e.dtype} (expected int16)")
    if acc.shape != e.shape:
        d.append(f"shapes differ: {tuple(acc.shape)} and {tuple(e.shape)}")
    if not (acc.is_cuda and e.is_cuda):
        d.append("not on the GPU")
    if not (acc.is_contiguous() and e.is_contiguous()):
        d.append("not contiguous")
    return d


class Registro:
    def __init__(self, pasta, nome, lib=None, vigiar=False, perfil=False, eco=True, salvar=True):
        os.makedirs(pasta, exist_ok=True)
        self.pasta, self.nome, self.lib = pasta, nome, lib
        self.vigiar, self.perfil, self.eco, self.salvar = vigiar, perfil, eco, salvar
        self.arq = open(os.path.join(pasta, f"{nome}.jsonl"), "a")
        self.pilha = []            # section labels
        self.lancamentos = []      # one dict per launch of the current step: op, trecho, entradas, forma
        self.passo = None
        self.eventos = []          # (op, start event, end event) when perfil
        self.tempos = {}           # op -> accumulated ms

    # ---------------------------------------------------------------- log file and messages
    def escreve(self, tipo, **campos):
        linha = dict(hora=time.strftime("%H:%M:%S"), tipo=tipo, passo=self.passo, trecho=self.onde())
        linha.update(campos)
        self.arq.write(json.dumps(linha, ensure_ascii=False, default=str) + "\n")
        self.arq.flush()
        return linha

    def info(self, msg, **campos):
        self.escreve("info", msg=msg, **campos)
        if self.eco:
            print(msg, flush=True)

    def aviso(self, msg, **campos):
        self.escreve("aviso", msg=msg, **campos)
        print(f"[AVISO] passo {self.passo} | {self.onde()} | {msg}", flush=True)

    def falha(self, msg, **campos):
        self.escreve("erro", msg=msg, **campos)
        raise ErroJatai(f"\n[ERRO] passo {self.passo} | {self.onde()}\n{msg}")

    def exige(self, condicao, msg):
        if not condicao:
            self.falha(msg)

    def onde(self):
        return " / ".join(self.pilha) if self.pilha else "-"

    @contextlib.contextmanager
    def trecho(self, nome):
        self.pilha.append(nome)
        try:
            yield
        finally:
            self.pilha.pop()

    # ---------------------------------------------------------------- launches
    def novo_passo(self, passo):
        self.passo, self.lancamentos, self.eventos = passo, [], []
        if self.lib is not None:
            self.lib.jt_erro_limpa()

    def registra(self, op, entradas, forma_saida):
        self.lancamentos.append(dict(op=op, trecho=self.onde(), entradas=entradas, forma=forma_saida))
        if self.perfil:
            par = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            par[0].record()
            self.eventos.append((op,) + par)
        return len(self.lancamentos) - 1

    def depois(self, kid, codigo_cuda):
        if self.perfil:
            self.eventos[-1][2].record()
        if codigo_cuda:
            lanc = self.lancamentos[kid]
            self.falha(f"CUDA refused the launch of '{lanc['op']}' (cudaError {codigo_cuda}). "
                       f"Input shapes: {_formas(lanc['entradas'])}")
        if self.vigiar:
            self.confere_device()

    def _descreve(self, kid):
        if 0 <= kid < len(self.lancamentos):
            return f"{self.lancamentos[kid]['op']} em {self.lancamentos[kid]['trecho']}"
        return "-"

    def confere_device(self):
        """Read the device error record (this synchronises the GPU); raise if a kernel left a sentinel."""
        rec = (ctypes.c_longlong * 6)()
        n = self.lib.jt_erro_le(rec)
        if n == 0:
            return
        if n < 0:
            self.falha(f"CUDA error {-n} while reading the device error record; an earlier kernel probably aborted. "
                       f"Last launch: {self._descreve(len(self.lancamentos) - 1)}")
        codigo, kid, idx, valor, aux = rec[1], rec[2], rec[3], rec[4], rec[5]
        texto = CODIGOS.get(codigo, f"codigo {codigo}")
        if not 0 <= kid < len(self.lancamentos):
            self.falha(f"{texto} in a kernel with unknown launch id {kid} (idx {idx}, value {valor})")
        lanc = self.lancamentos[kid]
        forma = lanc["forma"]
        if forma and len(forma) == 2:
            posicao = f"linha {idx // forma[1]}, coluna {idx % forma[1]} (forma {tuple(forma)})"
        else:
            posicao = f"indice {idx}"
        destino = self._salva_entradas(lanc) if self.salvar else "(not saved)"
        relato = "\n".join([
            texto,
            f"  operacao : {lanc['op']}",
            f"  trecho   : {lanc['trecho']}",
            f"  posicao  : {posicao}",
            f"  valor    : {valor}   (dado extra: {aux})",
            f"  eventos  : {n} in this step (only the first one is detailed)",
            f"  entradas : {_formas(lanc['entradas'])}",
            f"  salvas em: {destino}",
        ])
        self.pilha = [lanc["trecho"]]      # blame the section of the failing kernel, not the place of the check
        self.falha(relato, codigo=codigo, op=lanc["op"], idx=idx, valor=valor, aux=aux)

    def _salva_entradas(self, lanc):
        caminho = os.path.join(self.pasta, f"erro_passo{self.passo}_{lanc['op']}.pt")
        try:
            torch.save({k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in lanc["entradas"].items()}, caminho)
            return caminho
        except Exception as e:             # a failed dump must not hide the original error
            return f"(not saved: {e})"

    def fim_passo(self):
        if self.lib is not None:
            self.confere_device()
        if self.perfil:
            torch.cuda.synchronize()
            for op, ini, fim in self.eventos:
                self.tempos[op] = self.tempos.get(op, 0.0) + ini.elapsed_time(fim)

    def relatorio_tempos(self, passos):
        if not self.tempos:
            return
        total = sum(self.tempos.values())
        corpo = [f"  {op:16s} {ms / passos:8.3f} ms/passo  {100 * ms / total:5.1f}%"
                 for op, ms in sorted(self.tempos.items(), key=lambda kv: -kv[1])]
        corpo.append(f"  {'total':16s} {total / passos:8.3f} ms/passo")
        self.info("GPU time per operation:\n" + "\n".join(corpo), tempos={k: v / passos for k, v in self.tempos.items()})
        self.tempos = {}

    # ---------------------------------------------------------------- format checks
    def confere_bloco(self, nome, t):
        d = _defeitos_bloco(t, _bloco())
        if d:
            self.falha(f"argument '{nome}' is not a valid block tensor: " + "; ".join(d))

    def confere_cru(self, nome, t):
        d = _defeitos_cru(t)
        if d:
            self.falha(f"argument '{nome}' is not a valid raw tensor: " + "; ".join(d))

    # ---------------------------------------------------------------- statistics (report only)
    def estatistica(self, nome, t, zeros_normais=False):
        """Zero fraction, zeroed-block fraction and exponent range of a block tensor, with anomaly warnings."""
        m, E = t
        vivos = E != -127
        algum = bool(vivos.any())
        rec = dict(
            nome=nome,
            zeros=round(float((m == 0).float().mean()), 4),
            blocos_zerados=round(float((~vivos).float().mean()), 4),
            exp_min=int(E[vivos].min()) if algum else None,
            exp_max=int(E[vivos].max()) if algum else None,
            maior_mantissa_media=round(float(m.abs().reshape(m.shape[0], -1, _bloco()).amax(-1).float().mean()), 1),
        )
        self.escreve("estatistica", **rec)
        if not algum:
            self.aviso(f"'{nome}' came out entirely zero")
        elif rec["zeros"] > 0.5 and not zeros_normais:
            self.aviso(f"'{nome}' is {rec['zeros']:.0%} zeros: are small values vanishing in the rounding?")
        if algum and rec["exp_min"] < -110:
            self.aviso(f"'{nome}' has exponent {rec['exp_min']}, close to the INT8 limit of -126")
        return rec
