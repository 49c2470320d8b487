"""Helpers of the GPU tests: the checked operator object with the int64 oracle evaluated on the same GPU (test infrastructure)."""
import hashlib

import torch

import casos


class ConferidoNaGpu:
    """Every operation runs on the CUDA launcher and on the oracle, both on the GPU tensors, and must agree bit for bit (the role of
    the reference's OpsConferido, jatai_cuda/ops.py:532-566).  `por_sequencia`: the oracle's attention runs one sequence at a
    time, which keeps its (heads, T, T) int64 tensors small at T = 1024."""
    nome = "conferido"

    def __init__(self, cuda_ops, oraculo, por_sequencia=False):
        self.c, self.r, self.por_sequencia = cuda_ops, oraculo, por_sequencia
        self.lib = cuda_ops.lib
        self.n = {}

    def _atencao_r(self, op, args):
        if op == "atencao_quant":
            o, P = self._atencao_r("atencao", args)
            return self.r.quant(o), P
        if op == "atencao_back_quant":
            return self.r.quant(self._atencao_r("atencao_back", args))
        if op == "atencao":
            qkv, Bt, T, H = args
            partes = [self.r.atencao(tuple(t[b * T:(b + 1) * T].contiguous() for t in qkv), 1, T, H) for b in range(Bt)]
            o = tuple(torch.cat([p[0][i] for p in partes]) for i in range(2))
            return o, torch.cat([p[1] for p in partes])
        go, qkv, P, Bt, T, H = args
        partes = [self.r.atencao_back(tuple(t[b * T:(b + 1) * T].contiguous() for t in go), tuple(t[b * T:(b + 1) * T].contiguous() for t in qkv),
                                      P[b * H:(b + 1) * H], 1, T, H) for b in range(Bt)]
        return tuple(torch.cat([p[i] for p in partes]) for i in range(2))

    def __getattr__(self, op):
        fc, fr = getattr(self.c, op), getattr(self.r, op)

        def f(*args, **kw):
            copia = [tuple(t.clone() for t in a) if isinstance(a, tuple) and op in ("momento", "peso", "momento_peso") else a for a in args]
            if self.por_sequencia and op in ("atencao", "atencao_back", "atencao_quant", "atencao_back_quant"):
                out_r = self._atencao_r(op, copia)
            else:
                out_r = fr(*copia, **kw)
            out_c = fc(*args, **kw)
            torch.cuda.synchronize()
            for i, (a, b) in enumerate(zip(casos.plano(out_c), casos.plano(out_r))):
                if not (a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)):
                    dif = (a != b) if a.shape == b.shape else None
                    raise AssertionError(f"op '{op}' output {i} differs from the oracle ({int(dif.sum()) if dif is not None else '?'} of {a.numel()})")
            self.n[op] = self.n.get(op, 0) + 1
            return out_c
        return f


def digest_estado(m):
    """SHA-256 over weights, momentum and residual of a model (mantissas and exponents, in name order)."""
    h = hashlib.sha256()
    for n in sorted(m.p):
        for par in (m.p[n], m.mom[n], m.res[n]):
            for t in par:
                h.update(t.detach().cpu().numpy().tobytes())
    return h.hexdigest()


def lote(seed, Bt, T, V=256, dev="cuda"):
    x = torch.randint(0, V, (Bt, T + 1), generator=torch.Generator().manual_seed(seed))
    return x[:, :-1].contiguous().to(dev), x[:, 1:].contiguous().to(dev)
