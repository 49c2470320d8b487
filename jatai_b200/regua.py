"""float32 yard-stick of the integer model: the same Transformer in plain PyTorch (autograd, fp32), started from the integer
model's dequantised weights.  It plays the role of the reference's `ModeloFloat` (treino_int8_gpu/jatai_int8.py:399-428, used
by jatai_cuda/treino_cuda.py:153-165): the speed every INT8 number is quoted against, and the loss curve the integer run is
compared with.  Architecture as in `modelo.Modelo`: pre-norm, RMSNorm without gain, causal attention with ALiBi, ReLU^2 MLP,
byte vocabulary.  ALiBi: the integer model subtracts (i - j) << incl from scores counted in 1/256, i.e. the slope of head h is
2^(incl - 8) with incl = max(8 - h // 8, 0); scores are divided by sqrt(head dim).  Nothing here is on the integer hot path.
"""
import math

import torch
import torch.nn.functional as F


def _deq(t):
    m, E = t
    blk = m.shape[1] // E.shape[1]
    return m.float() * torch.exp2(E.float()).repeat_interleave(blk, dim=1)


class ModeloFloat(torch.nn.Module):
    def __init__(self, inteiro):
        """`inteiro`: a modelo.Modelo whose current weights become the float parameters."""
        super().__init__()
        self.D, self.H, self.L = inteiro.D, inteiro.H, inteiro.L
        self.w = torch.nn.ParameterDict({n: torch.nn.Parameter(_deq(t)) for n, t in inteiro.p.items()})
        incl = torch.tensor([max(8 - h // 8, 0) for h in range(self.H)], dtype=torch.float32)
        self.register_buffer("inclinacao", torch.exp2(incl - 8).to(next(iter(self.w.values())).device))

    def forward(self, tok, alvo):
        Bt, T = tok.shape
        H, hd = self.H, self.D // self.H
        norma = lambda x: x * torch.rsqrt((x * x).mean(-1, keepdim=True))
        dist = (torch.arange(T, device=tok.device)[:, None] - torch.arange(T, device=tok.device)[None, :]).float()
        vies = -self.inclinacao[:, None, None] * dist                    # [H, T, T]; the causal mask removes the negative distances
        x = self.w["emb"][tok]
        for l in range(self.L):
            q, k, v = (norma(x) @ self.w[f"Wqkv{l}"].t()).reshape(Bt, T, 3, H, hd).permute(2, 0, 3, 1, 4)
            z = q @ k.transpose(-1, -2) / math.sqrt(hd) + vies
            a = torch.softmax(z.masked_fill(dist < 0, float("-inf")), -1)
            x = x + (a @ v).transpose(1, 2).reshape(Bt, T, self.D) @ self.w[f"Wo{l}"].t()
            x = x + torch.relu(norma(x) @ self.w[f"Wup{l}"].t()).square() @ self.w[f"Wd{l}"].t()
        return F.cross_entropy((norma(x) @ self.w["out"].t()).reshape(-1, self.w["out"].shape[0]), alvo.reshape(-1))


class PassoFloat:
    """One SGD step (momentum 7/8, learning rate 2^-k: the integer optimiser's constants) of the float yard-stick."""

    def __init__(self, inteiro, k_lr):
        self.m = ModeloFloat(inteiro)
        self.opt = torch.optim.SGD(self.m.parameters(), lr=2.0 ** -k_lr, momentum=0.875)

    def __call__(self, tok, alvo):
        perda = self.m(tok, alvo)
        self.opt.zero_grad(set_to_none=True)
        perda.backward()
        self.opt.step()
        return perda.detach()
