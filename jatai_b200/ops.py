"""Operator API of the integer training step on B200: the host-side mirror of jatai_cuda/ops.py.

`OpsCuda(reg)` has the method names, argument meaning, return values and error behaviour of the reference's
`OpsCuda` (jatai_cuda/ops.py:294-515): every method checks its inputs through the registry, allocates its
outputs as torch tensors, registers the launch (-> kid) and calls one `jt_*` entry point of
libjatai_b200.so with raw device pointers.  A model written against the reference operator API
(`modelo.py`) therefore runs unchanged on these kernels.

Formats: Bloco = (m int8 [R,C], E int8 [R,C/BLK]), value m * 2^E, zero block E = -127;
         Cru = (acc int32 [R,C], e int16 [R,C]).

Module-level names kept from the reference: BLK, E_ZERO, GA, ATENCAO_LIMITE, g_rms, OpsCuda (class attribute
lib_global).  New: define_blk (the reference's block length is a compile-time 128; here 32 is native and 128
is the compatibility format), and optional arguments for the data-parallel step (RA / RB of `gemm`, log2M of
`softmax_ce`).  There is no CPU path: constructing OpsCuda without the compiled library, or calling it with
CPU tensors, raises.
"""
import ctypes
import math
import os

import torch

BLK = 32
E_ZERO = -127
GA = 4                     # guard bits of q/k/v/dO aligned inside a head (reference ops.py:20)
ATENCAO_LIMITE = False     # attention backward: shifts from upper bounds instead of exact maxima (ops.py:21-23)
AQUI = os.path.dirname(os.path.abspath(__file__))
BIBLIOTECA = os.path.join(AQUI, "libjatai_b200.so")

_INT_FUNCS = ("jt_gemm", "jt_gemm_f", "jt_gemm_ext", "jt_max_linha", "jt_quant", "jt_soma", "jt_relu2", "jt_relu2_back",
              "jt_momento", "jt_peso", "jt_momento_peso", "jt_transpoe", "jt_transpoe2", "jt_embed", "jt_um_quente", "jt_rms", "jt_rms_back", "jt_rms_back_soma", "jt_atencao",
              "jt_atencao_back", "jt_softmax_ce", "jt_erro_le", "jt_erro_limpa", "jt_sincroniza", "jt_para16", "jt_para8",
              "jt_soma16", "jt_res_estocastico", "jt_blk", "jt_blk_atual", "jt_gemm_via", "jt_gemm_tn", "jt_atencao_back_fixo", "jt_atencao_via", "jt_atencao_quant", "jt_atencao_back_quant",
              "jt_espera_limite", "jt_teste_espera", "jt_transpoe2_max", "jt_pdl", "jt_gemm_sem_cargas")


def g_rms(D):
    """(guard bits of RMSNorm forward, of its backward) for D columns; reference ops.py:28-30."""
    nb = D // BLK
    return 2 * ((8 - int(math.log2(nb))) // 2), 14 - int(math.log2(D))


def carrega_biblioteca(caminho=None):
    """dlopen the C-ABI library and declare the return types.  Raises if it has not been built."""
    caminho = caminho or BIBLIOTECA
    if not os.path.exists(caminho):
        raise RuntimeError(f"{caminho} not found: build it with `python -m jatai_b200.build` (needs nvcc, sm_100a)")
    lib = ctypes.CDLL(caminho)
    lib.jt_stream.argtypes = [ctypes.c_void_p]
    lib.jt_stream.restype = None
    lib.jt_erro_le.argtypes = [ctypes.c_void_p]
    for f in _INT_FUNCS:
        if hasattr(lib, f):
            getattr(lib, f).restype = ctypes.c_int
    return lib


def define_blk(blk, lib=None):
    """Select the exponent block length (32 or 128) for this module and for the library."""
    global BLK
    if blk not in (32, 128):
        raise ValueError("block length must be 32 or 128")
    BLK = blk
    lib = lib or getattr(OpsCuda, "lib_global", None)
    if lib is not None and hasattr(lib, "jt_blk"):
        if lib.jt_blk(blk) != 0:
            raise RuntimeError(f"library refused block length {blk}")
    elif lib is not None and blk != 128:
        raise RuntimeError("this library has a fixed block length of 128")


def _ptr(x):
    if x is None:
        return ctypes.c_void_p(0)
    if torch.is_tensor(x):
        return ctypes.c_void_p(x.data_ptr() if x.numel() else 0)
    raise TypeError(type(x))


class OpsCuda:
    """Launcher of the CUDA kernels; interface of the reference's OpsCuda (ops.py:294-515)."""
    nome = "cuda"
    lib_global = None

    def __init__(self, reg, biblioteca=None):
        if not torch.cuda.is_available():
            raise RuntimeError("OpsCuda needs a CUDA device; there is no CPU implementation in this package")
        self.reg = reg
        self.lib = carrega_biblioteca(biblioteca)
        reg.lib = self.lib
        self.lib.jt_erro_limpa()
        OpsCuda.lib_global = self.lib
        if hasattr(self.lib, "jt_blk"):
            if self.lib.jt_blk(BLK) != 0:
                raise RuntimeError(f"library refused block length {BLK}")
        elif BLK != 128:
            raise RuntimeError("this library has a fixed block length of 128; call ops.define_blk(128) first")
        if hasattr(self.lib, "jt_pdl"):                           # programmatic dependent launches: JT_PDL=0 switches them off
            self.lib.jt_pdl(0 if os.environ.get("JT_PDL", "1") == "0" else 1)
        # a library with only the reference's entry points: the fused extras read as absent, callers fall back to the separate operations
        for metodo, fn in (("transpoe2", "jt_transpoe2"), ("momento_peso", "jt_momento_peso"), ("rms_back_soma", "jt_rms_back_soma"),
                           ("max_linha", "jt_max_linha"), ("atencao_quant", "jt_atencao_quant"), ("atencao_back_quant", "jt_atencao_back_quant")):
            if not hasattr(self.lib, fn):
                setattr(self, metodo, None)

    # ------------------------------------------------------------------ plumbing
    def _lanca(self, op, fn, ponteiros, inteiros, entradas, forma, longos=()):
        """ponteiros: tensors / None; inteiros: C ints (indices in `longos` are long long); kid goes last."""
        kid = self.reg.registra(op, entradas, forma)
        args = [_ptr(p) for p in ponteiros]
        args += [ctypes.c_longlong(v) if i in longos else ctypes.c_int(v) for i, v in enumerate(inteiros)]
        rc = getattr(self.lib, fn)(*args, ctypes.c_int(kid))
        self.reg.depois(kid, rc)

    @staticmethod
    def _bloco_vazio(R, C, dev):
        return torch.empty(R, C, dtype=torch.int8, device=dev), torch.empty(R, C // BLK, dtype=torch.int8, device=dev)

    @staticmethod
    def _cru_vazio(R, C, dev):
        return torch.empty(R, C, dtype=torch.int32, device=dev), torch.empty(R, C, dtype=torch.int16, device=dev)

    # ------------------------------------------------------------------ GEMM family
    def _gemm(self, op, modo, A, B, X=None, duas=False, RA=None, RB=None):
        reg = self.reg
        reg.confere_bloco("A", A)
        reg.confere_bloco("B", B)
        (a, ea), (b, eb) = A, B
        M, K = a.shape
        N = b.shape[0]
        reg.exige(b.shape[1] == K, f"{op}: K differs, A {tuple(a.shape)} x B {tuple(b.shape)}")
        reg.exige(M % 64 == 0 and N % 128 == 0 and K % BLK == 0,
                  f"{op}: M must be a multiple of 64, N of 128, K of {BLK} (M={M}, N={N}, K={K})")
        ent = dict(A=a, EA=ea, B=b, EB=eb)
        if X is not None:
            reg.confere_bloco("X", X)
            reg.exige(tuple(X[0].shape) == (M, N), f"{op}: X has shape {tuple(X[0].shape)}, expected {(M, N)}")
            ent.update(X=X[0], XE=X[1])
        for nome, r, n in (("RA", RA, M), ("RB", RB, N)):
            if r is not None:
                reg.exige(r.dtype == torch.int8 and r.is_cuda and r.is_contiguous() and r.numel() == n,
                          f"{op}: {nome} must be a contiguous int8 CUDA tensor with {n} elements")
        dev = a.device
        Cb = Cr = C2 = (None, None)
        if modo == 1:
            Cr = self._cru_vazio(M, N, dev)
        else:
            Cb = self._bloco_vazio(M, N, dev)
        if duas:
            C2 = self._bloco_vazio(M, N, dev)
        x = X if X is not None else (None, None)
        if hasattr(self.lib, "jt_gemm_ext"):
            self._lanca(op, "jt_gemm_ext", (a, ea, b, eb, Cb[0], Cb[1], Cr[0], Cr[1], x[0], x[1], C2[0], C2[1], RA, RB),
                        (M, N, K, modo), ent, (M, N))
        else:       # a library with only the reference's entry points (no external row maxima)
            reg.exige(RA is None and RB is None, f"{op}: this library has no jt_gemm_ext (RA / RB unsupported)")
            self._lanca(op, "jt_gemm_f", (a, ea, b, eb, Cb[0], Cb[1], Cr[0], Cr[1], x[0], x[1], C2[0], C2[1]),
                        (M, N, K, modo), ent, (M, N))
        if modo == 1:
            return Cr
        return (Cb, C2) if duas else Cb

    def gemm(self, A, B, cru=False, RA=None, RB=None):
        """C = A . B^T, operands blocked along K.  cru=True: raw int32 accumulators + int16 exponents.
        RA / RB (optional int8 vectors): row-maximum exponents to align to instead of the operands' own
        (a data-parallel rank passes the maxima over all ranks)."""
        return self._gemm("gemm_cru" if cru else "gemm", 1 if cru else 0, A, B, RA=RA, RB=RB)

    def gemm_soma(self, A, B, X):
        return self._gemm("gemm_soma", 2, A, B, X=X)

    def gemm_relu2(self, A, B):
        return self._gemm("gemm_relu2", 3, A, B, duas=True)

    def gemm_relu2_back(self, A, B, Hh):
        return self._gemm("gemm_relu2_back", 4, A, B, X=Hh)

    def max_linha(self, X):
        """Row-maximum exponents (int8 [R]) of a block tensor: the RA / RB a GEMM derives from its operand."""
        self.reg.confere_bloco("X", X)
        E = X[1]
        R = torch.empty(E.shape[0], dtype=torch.int8, device=E.device)
        self._lanca("max_linha", "jt_max_linha", (E, R), (E.shape[0], E.shape[1]), dict(E=E), (E.shape[0], 1))
        return R

    def transpoe(self, X):
        self.reg.confere_bloco("X", X)
        m, E = X
        R, C = m.shape
        self.reg.exige(R % 128 == 0 and C % 64 == 0, f"transpoe: rows {R} must be a multiple of 128 and columns {C} of 64")
        Y = self._bloco_vazio(C, R, m.device)
        self._lanca("transpoe", "jt_transpoe", (m, E, Y[0], Y[1]), (R, C), dict(X=m, EX=E), (C, R))
        return Y

    def transpoe2(self, X1, X2):
        """(transpoe(X1), transpoe(X2)) for two block tensors with the same number of rows, in one launch (an addition of
        this library; the two operands of a weight-gradient GEMM)."""
        self.reg.confere_bloco("X1", X1)
        self.reg.confere_bloco("X2", X2)
        (m1, E1), (m2, E2) = X1, X2
        R, C1 = m1.shape
        C2 = m2.shape[1]
        self.reg.exige(m2.shape[0] == R, f"transpoe2: row counts differ ({R} and {m2.shape[0]})")
        self.reg.exige(R % 128 == 0 and C1 % 64 == 0 and C2 % 64 == 0, f"transpoe2: rows {R} must be a multiple of 128 and columns {C1}, {C2} of 64")
        Y1, Y2 = self._bloco_vazio(C1, R, m1.device), self._bloco_vazio(C2, R, m1.device)
        self._lanca("transpoe2", "jt_transpoe2", (m1, E1, Y1[0], Y1[1], m2, E2, Y2[0], Y2[1]), (C1, C2, R), dict(X1=m1, EX1=E1, X2=m2, EX2=E2),
                    (C1 + C2, R))
        return Y1, Y2

    def transpoe2_max(self, X1, X2, R1, R2):
        """transpoe2, and the row maxima of both results (max_linha) written into R1 [C1] / R2 [C2] - int8 views the caller has
        pre-set to -128 (data parallel: slices of the buffer of its MAX collective).  None where this library or these
        shapes do not offer it (the caller then uses transpoe2 and max_linha)."""
        (m1, E1), (m2, E2) = X1, X2
        R, C1 = m1.shape
        C2 = m2.shape[1]
        if BLK != 32 or C1 % 256 or C2 % 256 or R % 128 or m2.shape[0] != R or not hasattr(self.lib, "jt_transpoe2_max"):
            return None
        self.reg.confere_bloco("X1", X1)
        self.reg.confere_bloco("X2", X2)
        self.reg.exige(R1.numel() == C1 and R2.numel() == C2 and R1.dtype == torch.int8 and R2.dtype == torch.int8 and
                       R1.data_ptr() % 4 == 0 and R2.data_ptr() % 4 == 0, "transpoe2_max: row-maximum views of the wrong size, type or alignment")
        Y1, Y2 = self._bloco_vazio(C1, R, m1.device), self._bloco_vazio(C2, R, m1.device)
        self._lanca("transpoe2", "jt_transpoe2_max", (m1, E1, Y1[0], Y1[1], m2, E2, Y2[0], Y2[1], R1, R2), (C1, C2, R),
                    dict(X1=m1, EX1=E1, X2=m2, EX2=E2), (C1 + C2, R))
        return Y1, Y2

    # ------------------------------------------------------------------ block elementwise
    def quant(self, Cc):
        self.reg.confere_cru("C", Cc)
        acc, e = Cc
        R, C = acc.shape
        self.reg.exige(C % BLK == 0, f"quant: {C} columns is not a multiple of {BLK}")
        Y = self._bloco_vazio(R, C, acc.device)
        self._lanca("quant", "jt_quant", (acc, e, Y[0], Y[1]), (R * C // BLK,), dict(acc=acc, e=e), (R, C), longos=(0,))
        return Y

    def _elemento(self, op, fn, tensores, nomes):
        for n, t in zip(nomes, tensores):
            self.reg.confere_bloco(n, t)
        forma = tuple(tensores[0][0].shape)
        for n, t in zip(nomes[1:], tensores[1:]):
            self.reg.exige(tuple(t[0].shape) == forma, f"{op}: '{n}' has shape {tuple(t[0].shape)}, expected {forma}")
        Y = self._bloco_vazio(*forma, tensores[0][0].device)
        ptrs = [x for t in tensores for x in t] + [Y[0], Y[1]]
        ent = {f"{n}{s}": x for n, t in zip(nomes, tensores) for s, x in zip(("", "E"), t)}
        self._lanca(op, fn, ptrs, (tensores[0][0].numel() // BLK,), ent, forma, longos=(0,))
        return Y

    def soma(self, X, Y):
        return self._elemento("soma", "jt_soma", (X, Y), ("x", "y"))

    def relu2(self, Hh):
        return self._elemento("relu2", "jt_relu2", (Hh,), ("h",))

    def relu2_back(self, Gg, Hh):
        return self._elemento("relu2_back", "jt_relu2_back", (Gg, Hh), ("g", "h"))

    def embed(self, W, tok):
        self.reg.confere_bloco("W", W)
        m, E = W
        V, D = m.shape
        M = tok.numel()
        X = self._bloco_vazio(M, D, m.device)
        self._lanca("embed", "jt_embed", (m, E, tok, X[0], X[1]), (M, D, V), dict(W=m, tok=tok), (M, D))
        return X

    def um_quente(self, tok, V):
        M = tok.numel()
        U = self._bloco_vazio(M, V, tok.device)
        self._lanca("um_quente", "jt_um_quente", (tok, U[0], U[1]), (M, V), dict(tok=tok), (M, V))
        return U

    # ------------------------------------------------------------------ RMSNorm
    def rms(self, X):
        self.reg.confere_bloco("x", X)
        m, E = X
        M, D = m.shape
        self.reg.exige(D <= 2048 and D & (D - 1) == 0, f"rms: D={D} must be a power of two <= 2048")
        G, _ = g_rms(D)
        Y = self._bloco_vazio(M, D, m.device)
        r = torch.empty(M, dtype=torch.int32, device=m.device)
        emax = torch.empty(M, dtype=torch.int32, device=m.device)
        self._lanca("rms", "jt_rms", (m, E, Y[0], Y[1], r, emax), (M, D, int(math.log2(D)), G), dict(x=m, xE=E), (M, D))
        return Y, (r, emax)

    def rms_back(self, Gg, Y, cache):
        self.reg.confere_bloco("g", Gg)
        self.reg.confere_bloco("y", Y)
        (g, gE), (y, yE) = Gg, Y
        M, D = g.shape
        G, GB = g_rms(D)
        O = self._bloco_vazio(M, D, g.device)
        self._lanca("rms_back", "jt_rms_back", (g, gE, y, yE, cache[0], cache[1], O[0], O[1]), (M, D, int(math.log2(D)), G, GB),
                    dict(g=g, gE=gE, y=y, yE=yE, r=cache[0], emax=cache[1]), (M, D))
        return O

    def rms_back_soma(self, X, Gg, Y, cache):
        """soma(X, rms_back(Gg, Y, cache)) in one launch (an addition of this library; same results)."""
        for n, t in (("x", X), ("g", Gg), ("y", Y)):
            self.reg.confere_bloco(n, t)
        (g, gE), (y, yE) = Gg, Y
        M, D = g.shape
        self.reg.exige(tuple(X[0].shape) == (M, D), f"rms_back_soma: x has shape {tuple(X[0].shape)}, expected {(M, D)}")
        G, GB = g_rms(D)
        O = self._bloco_vazio(M, D, g.device)
        self._lanca("rms_back_soma", "jt_rms_back_soma", (g, gE, y, yE, cache[0], cache[1], X[0], X[1], O[0], O[1]),
                    (M, D, int(math.log2(D)), G, GB), dict(g=g, gE=gE, y=y, yE=yE, r=cache[0], emax=cache[1], x=X[0], xE=X[1]), (M, D))
        return O

    # ------------------------------------------------------------------ attention
    def atencao(self, QKV, Bt, T, H):
        self.reg.confere_bloco("qkv", QKV)
        m, E = QKV
        D = m.shape[1] // 3
        hd = D // H
        self.reg.exige(m.shape[0] == Bt * T and H * hd == D and hd in (4, 16, 64) and T % 32 == 0 and T <= 1024,
                       f"atencao: rows {m.shape[0]} (= Bt*T = {Bt * T}), head dim {hd} (4, 16 or 64), T={T} (multiple of 32, <= 1024)")
        oacc, oe = self._cru_vazio(Bt * T, D, m.device)
        P = torch.empty(Bt * H, T, T, dtype=torch.uint8, device=m.device)
        self._lanca("atencao", "jt_atencao", (m, E, oacc, oe, P), (Bt, T, H, D, GA), dict(qkv=m, qkvE=E), (Bt * T, D))
        return (oacc, oe), P

    def atencao_back(self, GO, QKV, P, Bt, T, H):
        self.reg.confere_bloco("go", GO)
        self.reg.confere_bloco("qkv", QKV)
        (gm, gE), (m, E) = GO, QKV
        D = gm.shape[1]
        acc, e = self._cru_vazio(Bt * T, 3 * D, m.device)
        self._lanca("atencao_back", "jt_atencao_back", (gm, gE, m, E, P, acc, e), (Bt, T, H, D, GA, int(ATENCAO_LIMITE)),
                    dict(go=gm, goE=gE, qkv=m, qkvE=E, P=P), (Bt * T, 3 * D))
        return acc, e

    def _atencao_fundida(self, T, H, D):
        """Whether the library quantises the attention outputs in its own output stage for this shape (else: two launches)."""
        return BLK == 32 and D == 64 * H and T % 64 == 0 and 128 <= T <= 1024

    def atencao_quant(self, QKV, Bt, T, H):
        """(quant(O), P) of atencao(QKV, Bt, T, H): one launch where the library offers it (an addition of this library; same results)."""
        D = QKV[0].shape[1] // 3
        if not self._atencao_fundida(T, H, D):
            oc, P = self.atencao(QKV, Bt, T, H)
            return self.quant(oc), P
        self.reg.confere_bloco("qkv", QKV)
        m, E = QKV
        self.reg.exige(m.shape[0] == Bt * T, f"atencao_quant: rows {m.shape[0]} (= Bt*T = {Bt * T})")
        O = self._bloco_vazio(Bt * T, D, m.device)
        P = torch.empty(Bt * H, T, T, dtype=torch.uint8, device=m.device)
        self._lanca("atencao_quant", "jt_atencao_quant", (m, E, O[0], O[1], P), (Bt, T, H, D, GA), dict(qkv=m, qkvE=E), (Bt * T, D))
        return O, P

    def atencao_back_quant(self, GO, QKV, P, Bt, T, H):
        """quant(atencao_back(GO, QKV, P, Bt, T, H)): one launch sequence without the raw intermediate where the library offers it."""
        D = GO[0].shape[1]
        if not self._atencao_fundida(T, H, D):
            return self.quant(self.atencao_back(GO, QKV, P, Bt, T, H))
        self.reg.confere_bloco("go", GO)
        self.reg.confere_bloco("qkv", QKV)
        (gm, gE), (m, E) = GO, QKV
        G = self._bloco_vazio(Bt * T, 3 * D, m.device)
        self._lanca("atencao_back_quant", "jt_atencao_back_quant", (gm, gE, m, E, P, G[0], G[1]), (Bt, T, H, D, GA, int(ATENCAO_LIMITE)),
                    dict(go=gm, goE=gE, qkv=m, qkvE=E, P=P), (Bt * T, 3 * D))
        return G

    # ------------------------------------------------------------------ loss and optimiser
    def softmax_ce(self, L, alvo, log2M=None):
        """log2M: log2 of the token count the gradient is averaged over (default: rows of L; a data-parallel
        rank passes the global count)."""
        self.reg.confere_cru("logits", L)
        acc, e = L
        M, V = acc.shape
        if log2M is None:
            self.reg.exige(M & (M - 1) == 0, f"softmax_ce: {M} rows is not a power of two")
            log2M = int(math.log2(M))
        self.reg.exige(V <= 2048 and V % BLK == 0, f"softmax_ce: V={V}")
        g = self._bloco_vazio(M, V, acc.device)
        d = torch.empty(M, dtype=torch.int32, device=acc.device)
        s = torch.empty(M, dtype=torch.int32, device=acc.device)
        self._lanca("softmax_ce", "jt_softmax_ce", (acc, e, alvo, g[0], g[1], d, s), (M, V, log2M), dict(acc=acc, e=e, alvo=alvo), (M, V))
        return g, d, s

    def momento(self, Gc, Mom):
        self.reg.confere_cru("grad", Gc)
        self.reg.confere_bloco("momento", Mom)
        self.reg.exige(tuple(Gc[0].shape) == tuple(Mom[0].shape), "momento: gradient and momentum shapes differ")
        self._lanca("momento", "jt_momento", (Gc[0], Gc[1], Mom[0], Mom[1]), (Mom[0].numel() // BLK,), dict(g=Gc[0], ge=Gc[1]),
                    tuple(Mom[0].shape), longos=(0,))
        return Mom

    def momento_peso(self, Gc, Mom, W, R, k, ef):
        """momento(Gc, Mom) followed by peso(W, Mom, R, k, ef) in one launch (an addition of this library; same results).
        Returns (Mom, W, R), all updated in place."""
        self.reg.confere_cru("grad", Gc)
        for n, t in (("W", W), ("momento", Mom), ("residuo", R)):
            self.reg.confere_bloco(n, t)
        self.reg.exige(tuple(Gc[0].shape) == tuple(Mom[0].shape) == tuple(W[0].shape), "momento_peso: gradient, momentum and weight shapes differ")
        self._lanca("momento_peso", "jt_momento_peso", (Gc[0], Gc[1], Mom[0], Mom[1], W[0], W[1], R[0], R[1]),
                    (k, int(ef), W[0].numel() // BLK), dict(g=Gc[0], ge=Gc[1]), tuple(W[0].shape), longos=(2,))
        return Mom, W, R

    def peso(self, W, Mom, R, k, ef):
        for n, t in (("W", W), ("momento", Mom), ("residuo", R)):
            self.reg.confere_bloco(n, t)
        self._lanca("peso", "jt_peso", (W[0], W[1], Mom[0], Mom[1], R[0], R[1]), (k, int(ef), W[0].numel() // BLK), dict(),
                    tuple(W[0].shape), longos=(2,))
        return W, R
