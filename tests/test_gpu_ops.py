"""Parity of the CUDA kernels with the oracle, through the C ABI (jatai_b200.ops.OpsCuda -> libjatai_b200.so).

Every case of tests/casos.py (the reference's own edge-case list at reduced sizes) runs at block 32 and 128 and
must equal, bit for bit, (a) the oracle on the same seeded inputs and (b) the committed golden outputs that the
reference's OpsRef produced.  GEMMs additionally run on each of the three kernel paths.
"""
import os
import tempfile

import pytest
import torch

import casos
import golden_util as gu
from oracle import spec

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def amb():
    from jatai_b200 import ops, registro
    reg = registro.Registro(tempfile.mkdtemp(), "teste", vigiar=True, eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    reg.novo_passo(0)
    yield ops, oc, reg
    ops.define_blk(32)
    oc.lib.jt_gemm_via(0)


def para_gpu(a):
    if torch.is_tensor(a):
        return a.to(DEV).contiguous()
    if isinstance(a, tuple):
        return tuple(para_gpu(x) for x in a)
    return a


class Adapt:
    """OpsCuda with the `limite` attribute casos.roda toggles (a module global in the operator module)."""

    def __init__(self, ops, oc):
        self._ops, self._oc = ops, oc

    def __getattr__(self, n):
        return getattr(self._oc, n)

    @property
    def limite(self):
        return self._ops.ATENCAO_LIMITE

    @limite.setter
    def limite(self, v):
        self._ops.ATENCAO_LIMITE = bool(v)


def _ids(blk):
    return [n for n, _, _ in casos.tabela(blk)]


def compara(nome, outs, refs):
    assert len(outs) == len(refs)
    for i, (a, b) in enumerate(zip(outs, refs)):
        a, b = a.cpu(), b.cpu()
        assert a.dtype == b.dtype and a.shape == b.shape, f"{nome} out {i}: {a.dtype}{tuple(a.shape)} vs {b.dtype}{tuple(b.shape)}"
        dif = a != b
        if dif.any():
            p = tuple(dif.nonzero()[0].tolist())
            raise AssertionError(f"{nome} out {i}: {int(dif.sum())} of {a.numel()} differ; first at {p}: cuda {a[p].item()} oracle {b[p].item()}")


@pytest.mark.parametrize("nome,blk,f", casos.tabela(32) + casos.tabela(128), ids=_ids(32) + _ids(128))
def test_tabela(amb, nome, blk, f):
    ops, oc, reg = amb
    ops.define_blk(blk)
    oc.lib.jt_gemm_via(0)
    reg.novo_passo(0)
    G = casos.Gen(casos.semente(nome), blk)
    op, args, kw = f(G)
    outs = casos.roda(Adapt(ops, oc), op, tuple(para_gpu(a) for a in args), kw)
    torch.cuda.synchronize()
    refs = casos.roda(spec.Spec(blk), op, args, kw)
    compara(nome, outs, refs)
    meta, arrs = gu.carrega(blk)
    gu.confere_saidas(nome, meta[nome], arrs, outs)


GEMMS = [(n, b, f) for n, b, f in casos.tabela(32) + casos.tabela(128) if "/gemm" in n]


@pytest.mark.parametrize("via", [1, 2, 3])
@pytest.mark.parametrize("nome,blk,f", GEMMS, ids=[n for n, _, _ in GEMMS])
def test_gemm_vias(amb, nome, blk, f, via):
    """via 1 = tensor core forced (block 32: FMA rounding with its range check, which the saturated-mantissa case sends to the
    conversion; block 128: conversion), 2 = CUDA cores, 3 = tensor core with the conversion everywhere."""
    ops, oc, reg = amb
    ops.define_blk(blk)
    assert oc.lib.jt_gemm_via(via) == 0
    try:
        reg.novo_passo(0)
        G = casos.Gen(casos.semente(nome), blk)
        op, args, kw = f(G)
        outs = casos.roda(oc, op, tuple(para_gpu(a) for a in args), kw)
        torch.cuda.synchronize()
        compara(f"{nome} via {via}", outs, casos.roda(spec.Spec(blk), op, args, kw))
    finally:
        oc.lib.jt_gemm_via(0)


def test_config1(amb):
    """Benchmark configuration 1: linear layer forward + both backward GEMMs at block 32, against the reference digests."""
    import json
    ops, oc, reg = amb
    ops.define_blk(32)
    reg.novo_passo(0)
    with open(os.path.join(gu.AQUI, "config1_b32.json")) as fh:
        rec = json.load(fh)
    X, W, dY = (para_gpu(t) for t in casos.config1(32))
    Y = oc.gemm(X, W)
    dX = oc.gemm(dY, oc.transpoe(W))
    dW = oc.gemm(oc.transpoe(dY), oc.transpoe(X), cru=True)
    torch.cuda.synchronize()
    assert [gu.digest(t) for t in Y] == rec["Y"]
    assert [gu.digest(t) for t in dX] == rec["dX"]
    assert [gu.digest(t) for t in dW] == rec["dW"]


@pytest.mark.parametrize("blk", [32, 128])
@pytest.mark.parametrize("M,N,K,cru", [(256, 256, 1024, False), (512, 384, 512, True), (128, 128, 4096, True), (1024, 1536, 512, False),
                                       (64, 128, 256, False), (192, 256, 384, True)])
def test_gemm_formas(amb, blk, M, N, K, cru):
    """Shape sweep against the oracle evaluated on the GPU in int64 (includes split-K raw outputs and the
    shapes only the CUDA-core path takes: M or K not a multiple of 128)."""
    ops, oc, reg = amb
    ops.define_blk(blk)
    reg.novo_passo(0)
    G = casos.Gen(1000 + M + N + K, blk)
    A, B = para_gpu(G.bloco(M, K, faixa=(-12, -4))), para_gpu(G.bloco(N, K, espalha=6, zera=0.05))
    out = oc.gemm(A, B, cru=cru)
    torch.cuda.synchronize()
    compara(f"gemm {M}x{N}x{K}", casos.plano(out), casos.plano(spec.Spec(blk).gemm(A, B, cru=cru)))


def test_gemm_maximos_externos(amb):
    """Row maxima supplied by the caller (the data-parallel path): two K halves with the global maxima add up to
    the full GEMM, bit for bit."""
    ops, oc, reg = amb
    ops.define_blk(32)
    reg.novo_passo(0)
    G = casos.Gen(77, 32)
    A, B = para_gpu(G.bloco(256, 1024, espalha=8)), para_gpu(G.bloco(128, 1024, espalha=8))
    RA, RB = oc.max_linha(A), oc.max_linha(B)
    assert torch.equal(RA.cpu(), A[1].cpu().amax(1)) and torch.equal(RB.cpu(), B[1].cpu().amax(1))
    inteiro = oc.gemm(A, B, cru=True)
    soma = None
    for h in range(2):
        a = (A[0][:, h * 512:(h + 1) * 512].contiguous(), A[1][:, h * 16:(h + 1) * 16].contiguous())
        b = (B[0][:, h * 512:(h + 1) * 512].contiguous(), B[1][:, h * 16:(h + 1) * 16].contiguous())
        acc, e = oc.gemm(a, b, cru=True, RA=RA, RB=RB)
        assert torch.equal(e, inteiro[1])
        soma = acc if soma is None else soma + acc
    assert torch.equal(soma, inteiro[0])


def test_sentinela_token_invalido(amb):
    """An out-of-range token is recorded (code 6) and reported with operation and position; nothing traps."""
    from jatai_b200.registro import ErroJatai
    ops, oc, reg = amb
    ops.define_blk(32)
    reg.novo_passo(0)
    G = casos.Gen(5, 32)
    W = para_gpu(G.bloco(256, 128))
    tok = G.tok(64, 256)
    tok[17] = 300
    reg.vigiar = False
    try:
        X = oc.embed(W, tok.to(DEV))
        with pytest.raises(ErroJatai) as ei:
            reg.confere_device()
        assert "embed" in str(ei.value) and "linha 17" in str(ei.value) and "300" in str(ei.value)
        assert int(X[0][17].abs().sum()) == 0 and int(X[1][17, 0]) == -127
    finally:
        reg.vigiar = True
        reg.novo_passo(0)


def test_referencia_compat(amb):
    """Compatibility format (block 128): the reference's own CUDA library, compiled for sm_100a from its source,
    is driven through the same operator class and must agree with this library bit for bit."""
    caminho = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libjatai_ref.so")
    if not os.path.exists(caminho):
        pytest.skip("oracle/_ref/libjatai_ref.so not built (needs the reference checkout at build time)")
    from jatai_b200 import registro
    ops, oc, reg = amb
    ops.define_blk(128)
    reg.novo_passo(0)
    reg2 = registro.Registro(tempfile.mkdtemp(), "ref", vigiar=True, eco=False, salvar=False)
    ocr = ops.OpsCuda(reg2, biblioteca=caminho)
    ops.OpsCuda.lib_global = oc.lib
    reg2.novo_passo(0)
    G = casos.Gen(9, 128)
    M, D, FF = 256, 256, 1024
    x, w1, w2, r = para_gpu(G.bloco(M, D)), para_gpu(G.bloco(FF, D)), para_gpu(G.bloco(D, FF)), para_gpu(G.bloco(M, D, espalha=8))
    for nome, f in [("gemm", lambda o: o.gemm(x, w1)), ("gemm_cru", lambda o: o.gemm(x, w1, cru=True)),
                    ("gemm_relu2", lambda o: o.gemm_relu2(x, w1)), ("gemm_soma", lambda o: o.gemm_soma(o.gemm_relu2(x, w1)[1], w2, r)),
                    ("transpoe", lambda o: o.transpoe(w1)), ("rms", lambda o: o.rms(x)), ("soma", lambda o: o.soma(x, r))]:
        a, b = casos.plano(f(oc)), casos.plano(f(ocr))
        torch.cuda.synchronize()
        compara(f"ref/{nome}", a, b)


ATENCOES = [  # blk, Bt, T, H, D  (head dim D/H in {4, 16, 64}; T also off the 128 grid; block 128 with wide heads)
    (32, 2, 64, 4, 64), (32, 2, 128, 2, 128), (32, 1, 256, 8, 512), (32, 1, 160, 2, 128), (32, 2, 96, 16, 64),
    (128, 2, 64, 2, 128), (128, 1, 192, 8, 128), (32, 1, 512, 2, 128), (32, 1, 192, 2, 128), (128, 1, 320, 2, 128), (32, 3, 128, 1, 64),
]


@pytest.mark.parametrize("limite", [False, True])
@pytest.mark.parametrize("blk,Bt,T,H,D", ATENCOES)
def test_atencao_generalizada(amb, blk, Bt, T, H, D, limite):
    """Attention forward + backward at head dimensions and sequence lengths the reference kernels do not reach,
    against the generalised oracle (which reduces to the reference at head dimension 4)."""
    ops, oc, reg = amb
    ops.define_blk(blk)
    reg.novo_passo(0)
    G = casos.Gen(31 * T + H + D + blk, blk)
    M = Bt * T
    qkv, go = G.bloco(M, 3 * D, espalha=5, zera=0.05), G.bloco(M, D, e0=-20, espalha=6, zera=0.05)
    s = spec.Spec(blk, limite=limite)
    (o_r, P_r) = s.atencao(qkv, Bt, T, H)
    g_r = s.atencao_back(go, qkv, P_r, Bt, T, H)
    ops.ATENCAO_LIMITE = limite
    try:
        o_c, P_c = oc.atencao(para_gpu(qkv), Bt, T, H)
        g_c = oc.atencao_back(para_gpu(go), para_gpu(qkv), P_c, Bt, T, H)
        torch.cuda.synchronize()
    finally:
        ops.ATENCAO_LIMITE = False
    compara(f"atencao {blk}/{Bt}/{T}/{H}/{D}", [*o_c, P_c], [*o_r, P_r])
    compara(f"atencao_back {blk}/{Bt}/{T}/{H}/{D} limite={limite}", list(g_c), list(g_r))


@pytest.mark.parametrize("R,C,esp,zera", [(256, 512, 4, 0.0), (128, 1024, 12, 0.1), (384, 256, 60, 0.3), (128, 256, 0, 0.0), (256, 768, 25, 0.5)])
def test_transpoe_largo(amb, R, C, esp, zera):
    """The wide-tile block-32 transposition (fp32 exact quantiser) against the oracle, including exponent spreads
    beyond what fp32 can align (integer path) and mostly-zero tensors."""
    ops, oc, reg = amb
    ops.define_blk(32)
    reg.novo_passo(0)
    G = casos.Gen(4000 + R + C + esp, 32)
    X = G.bloco(R, C, espalha=esp, zera=zera, e0=-5)
    out = oc.transpoe(para_gpu(X))
    torch.cuda.synchronize()
    compara(f"transpoe {R}x{C} esp {esp}", list(out), list(spec.Spec(32).transpoe(X)))


GEMMS32 = [(n, b, f) for n, b, f in casos.tabela(32) if "/gemm" in n]


@pytest.mark.parametrize("tn", [64, 128])
@pytest.mark.parametrize("nome,blk,f", GEMMS32, ids=[n for n, _, _ in GEMMS32])
def test_gemm_largura_do_tile(amb, nome, blk, f, tn):
    """Both tile widths of the tensor-core GEMM (64 and 128 columns), forced, on every GEMM case of the table."""
    ops, oc, reg = amb
    ops.define_blk(32)
    oc.lib.jt_gemm_via(0)
    assert oc.lib.jt_gemm_tn(tn) == 0
    try:
        reg.novo_passo(0)
        G = casos.Gen(casos.semente(nome), blk)
        op, args, kw = f(G)
        outs = casos.roda(oc, op, tuple(para_gpu(a) for a in args), kw)
        torch.cuda.synchronize()
        compara(f"{nome} tn {tn}", outs, casos.roda(spec.Spec(blk), op, args, kw))
    finally:
        oc.lib.jt_gemm_tn(0)


@pytest.mark.parametrize("tn", [64, 128])
@pytest.mark.parametrize("caso", ["expoentes afastados", "linhas nulas", "acumuladores grandes"])
@pytest.mark.parametrize("op", ["gemm", "gemm_soma", "gemm_relu2", "gemm_relu2_back"])
def test_gemm_estagio_de_saida(amb, op, caso, tn):
    """The output stage of the tensor-core GEMM quantises in fp32 when that is exact and in integers otherwise.  These
    inputs force the integer side: column exponents of one block more than 64 apart, all-zero rows of B (row maximum
    -127 next to ordinary rows), accumulators at or above 2^24 - each against the specification."""
    ops, oc, reg = amb
    ops.define_blk(32)
    oc.lib.jt_gemm_via(0)
    assert oc.lib.jt_gemm_tn(tn) == 0
    try:
        reg.novo_passo(0)
        G = casos.Gen(4242, 32)
        M, K, N = 256, 512, 256
        A, B = G.bloco(M, K, espalha=2), G.bloco(N, K, espalha=2)
        if caso == "expoentes afastados":
            B[1][0::2] -= 50                      # even rows of B 70 exponents below the odd ones, inside every block of columns
            B[1][1::2] += 20                      # (output exponents stay far from the int8 limits, squared too)
        elif caso == "linhas nulas":
            B[0][::3] = 0
            B[1][::3] = -127
        else:
            A = (torch.full_like(A[0], 127), torch.full_like(A[1], -8))
            B = (torch.full_like(B[0], 127), torch.full_like(B[1], -8))
        X = G.bloco(M, N, espalha=3)
        args = {"gemm": (A, B), "gemm_soma": (A, B, X), "gemm_relu2": (A, B), "gemm_relu2_back": (A, B, X)}[op]
        outs = casos.roda(oc, op, tuple(para_gpu(a) for a in args), {})
        torch.cuda.synchronize()
        compara(f"{op} {caso} tn {tn}", outs, casos.roda(spec.Spec(32), op, args, {}))
    finally:
        oc.lib.jt_gemm_tn(0)


@pytest.mark.parametrize("blk", [32, 128])
@pytest.mark.parametrize("ef", [0, 1])
def test_momento_peso_junto(amb, blk, ef):
    """The fused optimiser launch gives the bits of momento followed by peso (and of the specification), including
    zero blocks of momentum and residual and gradients of very different magnitudes."""
    ops, oc, reg = amb
    ops.define_blk(blk)
    try:
        reg.novo_passo(0)
        G = casos.Gen(77 + blk + ef, blk)
        R_, C_ = 256, 512
        grad = G.cru(R_, C_, bits=26, e0=-35)
        grad[0][::7] = 0
        mom, w, res = G.bloco(R_, C_, espalha=6, zera=0.1, e0=-14), G.bloco(R_, C_, espalha=3, e0=-9), G.bloco(R_, C_, espalha=5, zera=0.2, e0=-17)
        copia = lambda t: tuple(x.clone().cuda() for x in t)
        g_d = para_gpu(grad)
        m1, w1, r1 = copia(mom), copia(w), copia(res)
        m1 = oc.momento(g_d, m1)
        w1, r1 = oc.peso(w1, m1, r1, 4, ef)
        m2, w2, r2 = oc.momento_peso(g_d, copia(mom), copia(w), copia(res), 4, ef)
        torch.cuda.synchronize()
        ref = spec.Spec(blk).momento_peso(grad, mom, w, res, 4, ef)
        compara(f"momento_peso blk {blk} ef {ef} (vs separate launches)", casos.plano((m2, w2, r2)), casos.plano((m1, w1, r1)))
        compara(f"momento_peso blk {blk} ef {ef} (vs specification)", casos.plano((m2, w2, r2)), casos.plano(ref))
    finally:
        ops.define_blk(32)


@pytest.mark.parametrize("blk,R,C1,C2", [(32, 256, 256, 512), (32, 2048, 512, 1536), (32, 2048, 256, 512), (32, 4096, 2048, 512),
                                         (32, 8192, 2048, 2048), (32, 256, 192, 512), (128, 256, 256, 512)])
def test_transpoe_par(amb, blk, R, C1, C2):
    """The paired transposition launch gives the bits of two single launches and of the specification, for every tile
    height it picks, unequal widths, a width that falls back to the generic kernel, and block 128."""
    ops, oc, reg = amb
    ops.define_blk(blk)
    try:
        reg.novo_passo(0)
        G = casos.Gen(500 + R + C1 + C2, blk)
        X1, X2 = G.bloco(R, C1, espalha=8, zera=0.1), G.bloco(R, C2, espalha=3, zera=0.05)
        d1, d2 = para_gpu(X1), para_gpu(X2)
        juntos = oc.transpoe2(d1, d2)
        separados = (oc.transpoe(d1), oc.transpoe(d2))
        torch.cuda.synchronize()
        compara(f"transpoe2 {R}x({C1},{C2}) blk {blk} (vs single launches)", casos.plano(juntos), casos.plano(separados))
        compara(f"transpoe2 {R}x({C1},{C2}) blk {blk} (vs specification)", casos.plano(juntos), casos.plano(spec.Spec(blk).transpoe2(X1, X2)))
    finally:
        ops.define_blk(32)


@pytest.mark.parametrize("blk,M,D", [(32, 256, 512), (32, 128, 1024), (32, 64, 2048), (32, 40, 256), (128, 256, 512)])
def test_rms_back_soma_junto(amb, blk, M, D):
    """The fused RMSNorm-backward + residual-add launch gives the bits of the two launches and of the specification
    (rows that do not fill the last CTA, every row width the kernel is instantiated for, zero blocks in the residual)."""
    ops, oc, reg = amb
    ops.define_blk(blk)
    try:
        reg.novo_passo(0)
        G = casos.Gen(900 + M + D, blk)
        x = G.bloco(M, D, espalha=5, zera=0.1, e0=-12)
        y, cache = spec.Spec(blk).rms(x)
        g, res = G.bloco(M, D, espalha=4, e0=-20), G.bloco(M, D, espalha=6, zera=0.15, e0=-19)
        dg, dy, dc, dr = para_gpu(g), para_gpu(y), tuple(t.cuda() for t in cache), para_gpu(res)
        junto = oc.rms_back_soma(dr, dg, dy, dc)
        separado = oc.soma(dr, oc.rms_back(dg, dy, dc))
        torch.cuda.synchronize()
        compara(f"rms_back_soma {M}x{D} blk {blk} (vs two launches)", casos.plano(junto), casos.plano(separado))
        compara(f"rms_back_soma {M}x{D} blk {blk} (vs specification)", casos.plano(junto), casos.plano(spec.Spec(blk).rms_back_soma(res, g, y, cache)))
    finally:
        ops.define_blk(32)


@pytest.mark.parametrize("tn", [64, 128])
@pytest.mark.parametrize("caso", ["tudo +127", "sinais alternados", "uma linha saturada", "um bloco saturado por linha"])
def test_gemm_produtos_parciais_grandes(amb, caso, tn):
    """Partial products at and above 2^18 with no alignment shift (s = 0): the inputs on which rounding by an FMA against
    1.5*2^23 would leave its exact range.  The kernel must find them (a range check on the biased patterns) and round those
    columns by conversion - in whole tiles, in single rows and in single K-blocks, for positive and negative products."""
    ops, oc, reg = amb
    ops.define_blk(32)
    oc.lib.jt_gemm_via(0)
    assert oc.lib.jt_gemm_tn(tn) == 0
    try:
        reg.novo_passo(0)
        G = casos.Gen(8181, 32)
        M, K, N = 256, 512, 256
        A, B = G.bloco(M, K, espalha=0), G.bloco(N, K, espalha=0)
        if caso == "tudo +127":
            A, B = (torch.full_like(A[0], 127), A[1]), (torch.full_like(B[0], 127), B[1])
        elif caso == "sinais alternados":            # every K-block of a row entirely +127 or -127: products of both signs at 32 * 127^2
            sa = (torch.arange(K // 32) % 2 * 2 - 1).repeat_interleave(32).to(torch.int8)
            A = ((127 * sa).expand(M, K).contiguous(), A[1])
            B = (torch.where(torch.arange(N)[:, None] % 3 == 0, -127, 127).to(torch.int8).expand(N, K).contiguous(), B[1])
        elif caso == "uma linha saturada":
            A[0][37] = 127
            B[0][101] = -127
        else:                                         # one saturated K-block per row, at a different place in every row
            for i in range(M):
                b = i % (K // 32)
                A[0][i, 32 * b:32 * b + 32] = 127 if i % 2 else -127
            B = (torch.full_like(B[0], 127), B[1])
        for cru in (False, True):
            outs = casos.plano(oc.gemm(para_gpu(A), para_gpu(B), cru=cru))
            torch.cuda.synchronize()
            compara(f"gemm {caso} tn {tn} cru {cru}", outs, casos.plano(spec.Spec(32).gemm(A, B, cru=cru)))
    finally:
        oc.lib.jt_gemm_tn(0)


@pytest.mark.parametrize("limite", [False, True])
@pytest.mark.parametrize("blk,Bt,T,H,D", [(32, 2, 128, 2, 128), (32, 1, 192, 2, 128), (32, 1, 160, 2, 128), (32, 2, 256, 8, 512), (128, 2, 128, 2, 128),
                                         (32, 1, 704, 1, 64), (32, 1, 320, 3, 192)])
def test_atencao_nucleos_tensor_e_cuda(amb, blk, Bt, T, H, D, limite):
    """Head dimension 64 has two implementations - tensor cores (the default) and the CUDA-core kernels (jt_atencao_via(1),
    also what the no-allocation entry point runs, and what sequence lengths that are no multiple of 64 get): forward and backward
    must agree bit for bit, on sequence lengths that fill whole key chunks and on ones that do not."""
    ops, oc, reg = amb
    ops.define_blk(blk)
    reg.novo_passo(0)
    G = casos.Gen(7 * T + H + D + blk, blk)
    M = Bt * T
    qkv, go = para_gpu(G.bloco(M, 3 * D, espalha=6, zera=0.05)), para_gpu(G.bloco(M, D, e0=-20, espalha=6, zera=0.05))
    ops.ATENCAO_LIMITE = limite
    saidas = []
    try:
        for via in (0, 1):
            assert oc.lib.jt_atencao_via(via) == 0
            o, P = oc.atencao(qkv, Bt, T, H)
            g = oc.atencao_back(go, qkv, P, Bt, T, H)
            torch.cuda.synchronize()
            saidas.append([*o, P, *g])
    finally:
        ops.ATENCAO_LIMITE = False
        oc.lib.jt_atencao_via(0)
        ops.define_blk(32)
    compara(f"atencao tensor x cuda {blk}/{Bt}/{T}/{H}/{D} limite={limite}", saidas[0], saidas[1])


@pytest.mark.parametrize("limite", [False, True])
@pytest.mark.parametrize("Bt,T,H,D", [(2, 128, 2, 128), (1, 256, 8, 512), (1, 192, 2, 128), (1, 1024, 1, 64)])
def test_atencao_com_quant_fundido(amb, Bt, T, H, D, limite):
    """The attention kernels that write their outputs already quantised (block length 32, head dimension 64) against
    quant(atencao(...)) / quant(atencao_back(...)) of the specification, including rows whose block of 32 columns is entirely
    zero and key tiles that end beyond T."""
    ops, oc, reg = amb
    ops.define_blk(32)
    reg.novo_passo(0)
    G = casos.Gen(11 * T + H + D, 32)
    M = Bt * T
    qkv, go = G.bloco(M, 3 * D, espalha=5, zera=0.1), G.bloco(M, D, e0=-20, espalha=6, zera=0.1)
    s = spec.Spec(32, limite=limite)
    o_r, P_r = s.atencao_quant(qkv, Bt, T, H)
    g_r = s.atencao_back_quant(go, qkv, P_r, Bt, T, H)
    ops.ATENCAO_LIMITE = limite
    try:
        o_c, P_c = oc.atencao_quant(para_gpu(qkv), Bt, T, H)
        g_c = oc.atencao_back_quant(para_gpu(go), para_gpu(qkv), P_c, Bt, T, H)
        torch.cuda.synchronize()
    finally:
        ops.ATENCAO_LIMITE = False
    assert reg.lancamentos[-1]["op"] == "atencao_back_quant"          # the fused entry point ran, not the composition
    compara(f"atencao_quant {Bt}/{T}/{H}/{D}", [*o_c, P_c], [*o_r, P_r])
    compara(f"atencao_back_quant {Bt}/{T}/{H}/{D} limite={limite}", list(g_c), list(g_r))


@pytest.mark.gpu
def test_espera_limitada_desiste_e_o_contexto_segue(amb):
    """The bounded wait of the tensor-core kernels on its own: one warp waits on a barrier that nothing completes, gives up
    after the (shortened) limit, records code 7 at place 99 and returns; the next GEMM is bit-exact as ever.  No copy,
    MMA or second CTA is involved, and the wait is the library's own `espera`."""
    import ctypes
    import json
    import time
    ops, oc, reg = amb
    lib = oc.lib
    ops.define_blk(32)
    torch.cuda.synchronize()
    assert lib.jt_erro_limpa() == 0
    saiu = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert lib.jt_espera_limite(ctypes.c_longlong(2_000_000)) == 0          # about a millisecond
    try:
        t0 = time.time()
        assert lib.jt_teste_espera(ctypes.c_void_p(saiu.data_ptr()), ctypes.c_int(5)) == 0
        torch.cuda.synchronize()
        dt = time.time() - t0
        out = (ctypes.c_longlong * 6)()
        n = lib.jt_erro_le(out)
        assert saiu.item() == 2, "the wait must give up"
        assert n >= 1 and out[1] == 7 and out[2] == 5 and out[3] == 99, list(out)
        assert dt < 2.0, f"gave up after {dt:.2f} s with a limit of about 1 ms"
    finally:
        assert lib.jt_espera_limite(ctypes.c_longlong(0)) == 0
        assert lib.jt_erro_limpa() == 0
    reg.novo_passo(0)
    with open(os.path.join(gu.AQUI, "config1_b32.json")) as fh:
        rec = json.load(fh)
    X, W, _ = (para_gpu(t) for t in casos.config1(32))
    Y = oc.gemm(X, W)
    torch.cuda.synchronize()
    assert [gu.digest(t) for t in Y] == rec["Y"]


@pytest.mark.gpu
@pytest.mark.parametrize("R,C1,C2,esp", [(256, 256, 512, 8), (2048, 512, 1536, 3), (128, 256, 256, 40), (4096, 2048, 512, 60), (8192, 2048, 2048, 5)])
def test_transpoe_par_com_maximos(amb, R, C1, C2, esp):
    """jt_transpoe2_max = jt_transpoe2 followed by jt_max_linha of both results, bit for bit, with the maxima written (as a
    maximum into a buffer pre-set to -128) by the transposition kernel itself: every tile height, exponents far apart (the
    integer path of the kernel), all-zero blocks."""
    ops, oc, reg = amb
    ops.define_blk(32)
    reg.novo_passo(0)
    G = casos.Gen(900 + R + C1 + C2, 32)
    d1, d2 = para_gpu(G.bloco(R, C1, espalha=esp, zera=0.1)), para_gpu(G.bloco(R, C2, espalha=3, zera=0.3))
    separados = oc.transpoe2(d1, d2)
    r1, r2 = oc.max_linha(separados[0]), oc.max_linha(separados[1])
    buf = torch.full((C1 + C2 + 256,), -128, dtype=torch.int8, device=DEV)
    juntos = oc.transpoe2_max(d1, d2, buf[256:256 + C1], buf[256 + C1:])
    torch.cuda.synchronize()
    assert juntos is not None
    compara(f"transpoe2_max {R}x({C1},{C2})", casos.plano(juntos), casos.plano(separados))
    assert torch.equal(buf[256:256 + C1], r1) and torch.equal(buf[256 + C1:], r2)
    assert bool((buf[:256] == -128).all())
    assert oc.transpoe2_max(para_gpu(G.bloco(128, 192, espalha=2, zera=0.0)), para_gpu(G.bloco(128, 256, espalha=2, zera=0.0)), buf[:192], buf[256:512]) is None


@pytest.mark.gpu
def test_gemm_abandona_uma_espera_e_o_seguinte_e_exato(amb):
    """The abort path of the tensor-core GEMM itself: with its operand loads switched off (nothing asynchronous in flight) and
    the wait limit shortened, the MMA warp's first wait runs out, the CTAs record code 7 with the launch id of that GEMM,
    every warp leaves through the normal exit and the launch returns; the next GEMM is bit-exact."""
    import ctypes
    import json
    import time
    ops, oc, reg = amb
    lib = oc.lib
    ops.define_blk(32)
    X, W, _ = (para_gpu(t) for t in casos.config1(32))
    torch.cuda.synchronize()
    assert lib.jt_erro_limpa() == 0
    vigiar, reg.vigiar = reg.vigiar, False                       # the registry would raise on the record this test provokes
    assert lib.jt_espera_limite(ctypes.c_longlong(2_000_000)) == 0 and lib.jt_gemm_sem_cargas(1) == 0
    try:
        reg.novo_passo(0)
        t0 = time.time()
        oc.gemm(X, W)
        kid = len(reg.lancamentos) - 1
        torch.cuda.synchronize()
        dt = time.time() - t0
        out = (ctypes.c_longlong * 6)()
        n = lib.jt_erro_le(out)
        assert n >= 1 and out[1] == 7 and out[2] == kid, list(out)
        assert dt < 5.0, f"the aborted GEMM took {dt:.2f} s with a limit of about 1 ms"
    finally:
        assert lib.jt_gemm_sem_cargas(0) == 0 and lib.jt_espera_limite(ctypes.c_longlong(0)) == 0
        assert lib.jt_erro_limpa() == 0
        reg.vigiar = vigiar
    reg.novo_passo(0)
    with open(os.path.join(gu.AQUI, "config1_b32.json")) as fh:
        rec = json.load(fh)
    Y = oc.gemm(X, W)
    torch.cuda.synchronize()
    assert [gu.digest(t) for t in Y] == rec["Y"]


@pytest.mark.gpu
@pytest.mark.parametrize("mmax,esp,T", [(127, 5, 1024), (9, 2, 1024), (2, 0, 768), (40, 12, 512)])
def test_atencao_pedacos_de_chaves_sem_efeito(amb, mmax, esp, T):
    """The forward leaves out key chunks its norm bound proves to have P = 0 exactly: large and tiny q, k magnitudes (the bound
    decides how many chunks stay), several sequence lengths, against the oracle bit for bit (P included), and the backward on
    that P."""
    ops, oc, reg = amb
    ops.define_blk(32)
    reg.novo_passo(0)
    Bt, H, D = 1, 2, 128
    G = casos.Gen(77 + mmax + T, 32)
    qkv, go = G.bloco(Bt * T, 3 * D, espalha=esp, zera=0.02, mmax=mmax), G.bloco(Bt * T, D, e0=-20, espalha=4)
    s = spec.Spec(32)
    o_r, P_r = s.atencao(qkv, Bt, T, H)
    g_r = s.atencao_back(go, qkv, P_r, Bt, T, H)
    o_c, P_c = oc.atencao(para_gpu(qkv), Bt, T, H)
    g_c = oc.atencao_back(para_gpu(go), para_gpu(qkv), P_c, Bt, T, H)
    torch.cuda.synchronize()
    compara(f"atencao mmax {mmax} T {T}", [*o_c, P_c], [*o_r, P_r])
    compara(f"atencao_back mmax {mmax} T {T}", list(g_c), list(g_r))


@pytest.mark.gpu
def test_atencao_back_com_P_alterado(amb):
    """The backward works from the P it is given: with whole tiles of P zeroed by hand (tiles its zero map then leaves out, tiles
    next to the diagonal, a whole key range) it still equals the oracle's backward on that same P."""
    ops, oc, reg = amb
    ops.define_blk(32)
    reg.novo_passo(0)
    Bt, T, H, D = 1, 1024, 2, 128
    G = casos.Gen(4242, 32)
    qkv, go = G.bloco(Bt * T, 3 * D, espalha=3, zera=0.02, mmax=30), G.bloco(Bt * T, D, e0=-20, espalha=4)
    s = spec.Spec(32)
    _, P = s.atencao(qkv, Bt, T, H)
    P = P.clone()                                    # [Bt*H, T (keys), T (queries)]
    P[0, 0:128, 256:] = 0                            # a far key range for all later queries
    P[0, 512:576, 576:640] = 0                       # the tile right of a diagonal tile
    P[1, 640:704, 640:704] = 0                       # a diagonal tile itself
    P[1, :, 896:960] = 0                             # every key of one query tile
    g_r = s.atencao_back(go, qkv, P, Bt, T, H)
    g_c = oc.atencao_back(para_gpu(go), para_gpu(qkv), para_gpu(P), Bt, T, H)
    torch.cuda.synchronize()
    compara("atencao_back with hand-zeroed tiles of P", list(g_c), list(g_r))
