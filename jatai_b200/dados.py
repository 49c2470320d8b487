"""Byte-level training data: the loader and batch sampler of the reference (treino_int8_gpu/treino.py:29-44).

`carregar(pasta)` reads Portuguese.jsonl and English.jsonl (one JSON object with a "text" field per line), takes
the first 3000 lines of each, appends a blank line to every document and sends one document in 20 to the
validation split; both splits come back as 1-D int64 tensors of byte values.  `lote(dados, gerador, Bt, T)` draws
Bt windows of T+1 bytes and returns inputs and targets shifted by one.  The reference keeps T and BT as module
globals; here they are arguments.  `sintetico` stands in for the corpus where it is not available (benchmarks).
"""
import json
import os

import torch

LINGUAS = ("Portuguese", "English")
MAX_LINHAS, UM_EM_VAL = 3000, 20


def carregar(pasta=None, linguas=LINGUAS):
    pasta = pasta or os.environ.get("JATAI_DADOS", "dados")
    treino, val = bytearray(), bytearray()
    for lingua in linguas:
        caminho = os.path.join(pasta, f"{lingua}.jsonl")
        with open(caminho, encoding="utf-8") as fh:
            for i, linha in enumerate(fh):
                if i >= MAX_LINHAS:
                    break
                doc = json.loads(linha)["text"].encode("utf-8") + b"\n\n"
                (val if i % UM_EM_VAL == 0 else treino).extend(doc)
    return torch.tensor(list(treino), dtype=torch.long), torch.tensor(list(val), dtype=torch.long)


def sintetico(n, semente=0):
    """n uniform random bytes (the stand-in used when the corpus is absent)."""
    return torch.randint(0, 256, (n,), generator=torch.Generator().manual_seed(semente))


def lote(dados, gerador, Bt, T, dev="cpu"):
    ini = torch.randint(0, len(dados) - T - 1, (Bt,), generator=gerador)
    x = torch.stack([dados[i:i + T + 1] for i in ini.tolist()]).to(dev)
    return x[:, :-1], x[:, 1:]
