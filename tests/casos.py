"""Seeded input generators and the case table shared by the golden-fixture script and the tests.

The generators follow the recipe of the reference's op tests (jatai_cuda/teste_ops.py:18-31):
uniform int8 mantissas in [-mmax, mmax], one exponent per block e0 +- espalha, optionally a
fraction of all-zero blocks (E = -127); raw tensors = uniform int32 below 2^bits with a per-element
int16 exponent e0 +- 3.  The block length is a parameter here (the reference hard-wires 128).

A case is (name, blk, builder); builder(G) returns (op, args, kwargs) where args are CPU tensors /
tuples / ints in the order of the operator API.  Every case builds its own generator from its name,
so cases are independent of each other and of execution order.
"""
import zlib

import torch

E_ZERO = -127


class Gen:
    def __init__(self, seed, blk):
        self.g = torch.Generator(device="cpu").manual_seed(seed)
        self.blk = blk

    def bloco(self, R, C, espalha=4, zera=0.0, e0=-10, mmax=127, faixa=None):
        blk = self.blk
        m = torch.randint(-mmax, mmax + 1, (R, C), generator=self.g, dtype=torch.int32).to(torch.int8)
        if faixa is not None:          # explicit exponent range [lo, hi], as benchmark configuration 1 states it
            E = torch.randint(faixa[0], faixa[1] + 1, (R, C // blk), generator=self.g).to(torch.int8)
        else:
            E = (e0 + torch.randint(-espalha, espalha + 1, (R, C // blk), generator=self.g)).to(torch.int8)
        if zera:
            z = torch.rand(R, C // blk, generator=self.g) < zera
            m = m.reshape(R, C // blk, blk).masked_fill(z[..., None], 0).reshape(R, C)
            E = E.masked_fill(z, E_ZERO)
        return m.contiguous(), E.contiguous()

    def cru(self, R, C, bits=24, e0=-30):
        acc = torch.randint(-(1 << bits), 1 << bits, (R, C), generator=self.g, dtype=torch.int32)
        e = (e0 + torch.randint(-3, 4, (R, C), generator=self.g)).to(torch.int16)
        return acc.contiguous(), e.contiguous()

    def tok(self, M, V):
        return torch.randint(0, V, (M,), generator=self.g).to(torch.int32)

    def zeros_cru(self, R, C):
        return torch.zeros(R, C, dtype=torch.int32), torch.zeros(R, C, dtype=torch.int16)

    def zeros_bloco(self, R, C):
        return torch.zeros(R, C, dtype=torch.int8), torch.full((R, C // self.blk), E_ZERO, dtype=torch.int8)


def semente(nome):
    return zlib.crc32(nome.encode()) & 0x7FFFFFFF


def tabela(blk, Bt=2, T=64, D=128, FF=256, V=128, hd=4):
    """The edge-case list of teste_ops.py:56-98 at reduced sizes (fixtures must stay small).

    `chain` entries need an earlier op's output (rms -> rms_back, atencao -> atencao_back); they are
    encoded as op names the runner understands.
    """
    M = Bt * T
    H = D // hd
    c = []

    def caso(nome, f):
        c.append((f"b{blk}/{nome}", blk, f))

    caso("gemm", lambda G: ("gemm", (G.bloco(M, D), G.bloco(3 * D, D)), {}))
    caso("gemm espalha 6", lambda G: ("gemm", (G.bloco(2 * M, D, espalha=6), G.bloco(FF, D)), {}))
    caso("gemm cru", lambda G: ("gemm", (G.bloco(2 * M, D), G.bloco(FF, D)), dict(cru=True)))
    caso("gemm blocos zerados", lambda G: ("gemm", (G.bloco(M, D, zera=0.3), G.bloco(D, D, zera=0.3)), {}))
    caso("gemm K longo espalha 12", lambda G: ("gemm", (G.bloco(M, 4 * FF, espalha=12), G.bloco(D, 4 * FF, espalha=12)), {}))
    caso("gemm cru K=tokens", lambda G: ("gemm", (G.bloco(D, M), G.bloco(FF, M)), dict(cru=True)))
    caso("gemm cru espalha 8", lambda G: ("gemm", (G.bloco(D, 4 * M, espalha=8), G.bloco(D, 4 * M, espalha=8)), dict(cru=True)))
    caso("gemm cru zerados", lambda G: ("gemm", (G.bloco(D, 4 * M, zera=0.4), G.bloco(3 * D, 4 * M, zera=0.4)), dict(cru=True)))
    caso("gemm mantissas no limite", lambda G: ("gemm", (_satura(G.bloco(M, D, espalha=0)), _satura(G.bloco(D, D, espalha=0))), {}))
    caso("gemm_soma", lambda G: ("gemm_soma", (G.bloco(M, D), G.bloco(D, D), G.bloco(M, D, espalha=10, zera=0.1)), {}))
    caso("gemm_soma residuo distante", lambda G: ("gemm_soma", (G.bloco(M, FF), G.bloco(D, FF), G.bloco(M, D, e0=8, espalha=20, zera=0.2)), {}))
    caso("gemm_relu2", lambda G: ("gemm_relu2", (G.bloco(M, D, zera=0.1), G.bloco(FF, D)), {}))
    caso("gemm_relu2 underflow", lambda G: ("gemm_relu2", (G.bloco(M, D, e0=-40), G.bloco(FF, D, e0=-40)), {}))
    caso("gemm_relu2_back", lambda G: ("gemm_relu2_back", (G.bloco(M, D), G.bloco(FF, D), G.bloco(M, FF, zera=0.1)), {}))
    caso("transpoe", lambda G: ("transpoe", (G.bloco(M, 3 * D, espalha=8, zera=0.1),), {}))
    caso("quant", lambda G: ("quant", (G.cru(M, D),), {}))
    caso("quant zeros", lambda G: ("quant", (G.zeros_cru(M, D),), {}))
    caso("soma", lambda G: ("soma", (G.bloco(M, D, espalha=10, zera=0.1), G.bloco(M, D, espalha=10, zera=0.1)), {}))
    caso("relu2", lambda G: ("relu2", (G.bloco(M, FF, zera=0.1),), {}))
    caso("relu2 underflow", lambda G: ("relu2", (G.bloco(M, FF, e0=-62, espalha=3),), {}))
    caso("relu2_back", lambda G: ("relu2_back", (G.bloco(M, FF), G.bloco(M, FF)), {}))
    caso("um_quente", lambda G: ("um_quente", (G.tok(M, V), V), {}))
    caso("embed", lambda G: ("embed", (G.bloco(V, D), G.tok(M, V)), {}))
    caso("rms", lambda G: ("rms", (G.bloco(M, D, espalha=6, zera=0.2),), {}))
    caso("rms mantissas pequenas", lambda G: ("rms", (G.bloco(M, D, mmax=3),), {}))
    caso("rms_back", lambda G: ("rms>rms_back", (G.bloco(M, D), G.bloco(M, D, espalha=6)), {}))
    caso("softmax_ce", lambda G: ("softmax_ce", (G.cru(M, V, bits=22, e0=-20), G.tok(M, V)), {}))
    caso("softmax_ce concentrado", lambda G: ("softmax_ce", (G.cru(M, V, bits=24, e0=-16), G.tok(M, V)), {}))
    caso("momento", lambda G: ("momento", (G.cru(D, D, bits=28, e0=-50), G.bloco(D, D, e0=-40)), {}))
    caso("momento underflow", lambda G: ("momento", (G.zeros_cru(D, D), G.bloco(D, D, e0=-122, espalha=3)), {}))
    caso("momento do zero", lambda G: ("momento", (G.cru(D, D, bits=20), G.zeros_bloco(D, D)), {}))
    caso("peso ef", lambda G: ("peso", (G.bloco(D, D, e0=-9), G.bloco(D, D, e0=-15), G.bloco(D, D, e0=-20, zera=0.3), 4, True), {}))
    caso("peso sem ef", lambda G: ("peso", (G.bloco(D, D, e0=-9), G.bloco(D, D, e0=-15), G.bloco(D, D), 4, False), {}))
    caso("peso passo grande", lambda G: ("peso", (G.bloco(D, D, e0=-12), G.bloco(D, D, e0=-2), G.bloco(D, D, e0=-20), 1, True), {}))
    # attention: forward alone, and forward -> backward chains (P of the forward feeds the backward)
    caso("atencao", lambda G: ("atencao", (G.bloco(M, 3 * D, espalha=3), Bt, T, H), {}))
    caso("atencao concentrada", lambda G: ("atencao", (G.bloco(M, 3 * D, e0=-3), Bt, T, H), {}))
    caso("atencao shift esq pequeno", lambda G: ("atencao", (G.bloco(M, 3 * D, e0=0, espalha=1), Bt, T, H), {}))
    caso("atencao shift esq grande", lambda G: ("atencao", (G.bloco(M, 3 * D, e0=4, espalha=1, mmax=3), Bt, T, H), {}))
    caso("atencao espalhada", lambda G: ("atencao", (G.bloco(M, 3 * D, espalha=12, zera=0.1), Bt, T, H), {}))
    caso("atencao_back", lambda G: ("atencao>atencao_back", (G.bloco(M, 3 * D), G.bloco(M, D, e0=-20), Bt, T, H), {}))
    caso("atencao_back espalhada", lambda G: ("atencao>atencao_back", (G.bloco(M, 3 * D, espalha=12, zera=0.1), G.bloco(M, D, e0=-20, espalha=12, zera=0.1), Bt, T, H), {}))
    caso("atencao_back limite", lambda G: ("atencao>atencao_back", (G.bloco(M, 3 * D), G.bloco(M, D, e0=-20), Bt, T, H), dict(limite=True)))
    caso("atencao_back limite espalhada", lambda G: ("atencao>atencao_back", (G.bloco(M, 3 * D, espalha=12, zera=0.1), G.bloco(M, D, e0=-20, espalha=12, zera=0.1), Bt, T, H), dict(limite=True)))
    return c


def _satura(t):
    """Every mantissa at +-127: the largest exact partial products a K-block can produce."""
    m, E = t
    return torch.where(m >= 0, torch.full_like(m, 127), torch.full_like(m, -127)), E


def config1(blk=32):
    """Benchmark configuration 1: one linear layer forward + both backward GEMMs, M=2048, K=N=512,
    mantissas uniform in [-127,127], one exponent per K-block uniform in [-12,-4], seed 0."""
    G = Gen(0, blk)
    X = G.bloco(2048, 512, faixa=(-12, -4))
    W = G.bloco(512, 512, faixa=(-12, -4))
    dY = G.bloco(2048, 512, faixa=(-12, -4))
    return X, W, dY


def roda(ops, op, args, kw):
    """Run one table entry on an operator object (spec, reference or CUDA); returns a flat tensor list."""
    kw = dict(kw)
    lim = kw.pop("limite", False)
    if op == "rms>rms_back":
        x, g = args
        y, cache = ops.rms(x)
        out = ops.rms_back(g, y, cache)
    elif op == "atencao>atencao_back":
        qkv, go, Bt, T, H = args
        _, P = ops.atencao(qkv, Bt, T, H)
        antes = _limite(ops, lim)
        try:
            out = ops.atencao_back(go, qkv, P, Bt, T, H)
        finally:
            _limite(ops, antes)
    elif op in ("momento", "peso"):                 # in-place ops: work on copies
        copia = [tuple(t.clone() for t in a) if isinstance(a, tuple) else a for a in args]
        out = getattr(ops, op)(*copia, **kw)
    else:
        out = getattr(ops, op)(*args, **kw)
    return plano(out)


def _limite(ops, novo):
    antes = getattr(ops, "limite", False)
    if hasattr(ops, "limite"):
        ops.limite = novo
    return antes


def plano(x):
    if torch.is_tensor(x):
        return [x]
    return [t for y in x for t in plano(y)]
