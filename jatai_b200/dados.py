"""Byte-level training data for the integer model.

`Corpus` keeps a document collection as ONE uint8 tensor resident on the training device and cuts batches out of it there: a
batch is Bt windows of T + 1 consecutive bytes, gathered by one indexing kernel from window starts drawn on the host with a
seeded generator (so a run is reproducible and a checkpoint only has to store the generator state).  Inputs are the first T
bytes of a window, targets the last T.

The split and the draw follow the reference's recipe (treino_int8_gpu/treino.py:29-44), so that the same files and the same
seed give the same batches as its loader: of each language file the first 3000 JSON lines are read, every document gets a
blank line appended, every 20th document goes to validation, and the window starts are `randint(0, len - T - 1)` of a CPU
generator.  Where no corpus is available `sintetico` supplies uniform random bytes.
"""
import json
import os

import torch

LINGUAS = ("Portuguese", "English")
MAX_LINHAS, UM_EM_VAL = 3000, 20


def _documentos(caminho, limite):
    """Yields (index, utf-8 bytes + blank line) of the first `limite` JSON lines of a file."""
    with open(caminho, encoding="utf-8") as fh:
        for i, linha in zip(range(limite), fh):
            yield i, json.loads(linha)["text"].encode("utf-8") + b"\n\n"


class Corpus:
    """A byte stream on a device, with the batch cutter."""

    def __init__(self, octetos, dev="cpu"):
        if isinstance(octetos, (bytes, bytearray)):
            octetos = torch.frombuffer(bytearray(octetos), dtype=torch.uint8)
        self.dados = octetos.to(torch.uint8).to(dev).contiguous()
        self._passos = {}

    def __len__(self):
        return self.dados.numel()

    def para(self, dev):
        return Corpus(self.dados, dev)

    def longos(self):
        """The stream as int64 on its device (the form the reference loader returns)."""
        return self.dados.to(torch.long)

    def lote(self, gerador, Bt, T, dev=None):
        inicio = torch.randint(0, len(self) - T - 1, (Bt,), generator=gerador)
        passo = self._passos.get(T)
        if passo is None:
            passo = self._passos[T] = torch.arange(T + 1, device=self.dados.device)
        janela = self.dados[inicio.to(self.dados.device)[:, None] + passo].to(torch.long)
        if dev is not None:
            janela = janela.to(dev)
        return janela[:, :-1], janela[:, 1:]


def carregar(pasta=None, linguas=LINGUAS, dev="cpu", como_corpus=False):
    """(train, validation) of a corpus folder: int64 byte tensors, or `Corpus` objects on `dev` with como_corpus=True."""
    pasta = pasta or os.environ.get("JATAI_DADOS", "dados")
    partes = {False: [], True: []}
    for lingua in linguas:
        for i, doc in _documentos(os.path.join(pasta, f"{lingua}.jsonl"), MAX_LINHAS):
            partes[i % UM_EM_VAL == 0].append(doc)
    treino, val = Corpus(b"".join(partes[False]), dev), Corpus(b"".join(partes[True]), dev)
    return (treino, val) if como_corpus else (treino.longos(), val.longos())


def sintetico(n, semente=0):
    """n uniform random bytes as an int64 tensor (the stand-in used when the corpus is absent)."""
    return torch.randint(0, 256, (n,), generator=torch.Generator().manual_seed(semente))


def lote(dados, gerador, Bt, T, dev="cpu"):
    """A batch from a 1-D tensor of byte values (any integer dtype) or a `Corpus`; same draw as `Corpus.lote`."""
    if isinstance(dados, Corpus):
        return dados.lote(gerador, Bt, T, dev)
    inicio = torch.randint(0, len(dados) - T - 1, (Bt,), generator=gerador)
    janela = dados[inicio[:, None] + torch.arange(T + 1)].to(dev)
    return janela[:, :-1], janela[:, 1:]
