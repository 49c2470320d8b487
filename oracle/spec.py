"""TEST INFRASTRUCTURE - int64 restatement of the reference's integer training arithmetic.

This module is the checker, never the product: only tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py may import it.  The library in jatai_b200/ never does.

It restates, operation by operation, the executable specification `OpsRef` of the reference
(jatai_cuda/ops.py:92-290) and its primitives (ops.py:34-89) with the three constants the
reference hard-wires turned into parameters:

  blk       exponent block length along the last dimension   (reference: 128, ops.py:17)
  head dim  D // H in attention                              (reference: 4, ops.py:188,195)
  T         sequence length                                  (reference kernels: <= 128)

At blk=128, head dim 4 every function below must return exactly what `OpsRef` returns; that is
pinned by tests/test_oracle_golden.py against fixtures produced by importing the reference itself
(tests/golden/make_golden.py).  At blk=32 the fixtures come from the same reference code with its
block constant patched (ops.BLK = 32 and the default of ops.expande), which covers every op
except attention; for attention at head dim > 4 no reference implementation exists, so those
cases are "parity unpinned" beyond the head-dim-4 reduction (see the notes in `Spec.atencao`).

Formats (ops.py:9): Bloco = (m int8 [R,C], E int8 [R,C/blk]), value m * 2^E, all-zero block has
E = -127; Cru = (acc int32 [R,C], e int16 [R,C]).
"""
import math

import torch

I64 = torch.int64
E_ZERO = -127
_NONE = -100000          # "no non-zero element in this block" marker (ops.py:19)
GA = 4                   # guard bits of q/k/v/dO aligned inside a head (ops.py:20)
GG = 4                   # guard bits of a GEMM partial product (ops.py:104)


# ----------------------------------------------------------------------------- primitives
def bitlen(x):
    """Number of bits of |x| (0 for 0).  ops.py:34-39."""
    a = x.abs().to(I64)
    n = torch.zeros_like(a)
    for step in (32, 16, 8, 4, 2, 1):
        n = n + step * ((a >> (n + step)) != 0)
    return n + (a != 0)


def rnd(x, s):
    """x * 2^-s rounded half-to-even; s <= 0 is an exact left shift.  ops.py:42-51."""
    x = x.to(I64)
    s = torch.as_tensor(s, dtype=I64, device=x.device).expand_as(x)
    r = s.clamp(0, 62)
    fl = x >> r                                   # floor
    rem = x - (fl << r)                           # 0 <= rem < 2^r
    half = torch.where(r > 0, torch.ones_like(r) << (r - 1).clamp(min=0), torch.zeros_like(r))
    up = (rem > half) | ((rem == half) & ((fl & 1) == 1))
    right = fl + (up & (r > 0)).to(I64)
    return torch.where(s > 0, right, x << (-s).clamp(0, 62))


def expande(E, blk):
    """Per-block exponents -> per-element exponents.  ops.py:54-55."""
    return E.to(I64).repeat_interleave(blk, dim=-1)


def quant(v, e, blk):
    """int64 values with per-element exponent -> Bloco along the last dim.  ops.py:58-72.

    top = max over non-zero elements of e + bitlen(v); E = top - 7; one retry with E + 1 if a
    mantissa exceeds 127 after rounding; E < -126 flushes the block to zero (E = -127).
    """
    v = v.to(I64)
    e = torch.as_tensor(e, dtype=I64, device=v.device).expand_as(v)
    shape = v.shape[:-1] + (v.shape[-1] // blk, blk)
    top = torch.where(v != 0, e + bitlen(v), torch.full_like(v, _NONE)).reshape(shape).amax(-1)
    empty = top == _NONE
    E = top - 7
    q = rnd(v, expande(E, blk) - e)
    E = E + (q.abs().reshape(shape).amax(-1) > 127).to(I64)
    q = rnd(v, expande(E, blk) - e)
    dead = empty | (E < -126)
    E = torch.where(dead, torch.full_like(E, E_ZERO), E)
    q = torch.where(expande(dead.to(I64), blk) == 1, torch.zeros_like(q), q)
    return q.clamp(-127, 127).to(torch.int8).contiguous(), E.to(torch.int8).contiguous()


def exp_int(d):
    """Q15 exp(-d/256) for d >= 0: power-of-two shift + cubic polynomial.  ops.py:75-81."""
    t = d.clamp(max=6000) * 23637
    n = t >> 22
    f = (t & ((1 << 22) - 1)) >> 7
    p = torch.full_like(f, -1295)
    for c in (7556, -22645, 32765):
        p = ((p * f) >> 15) + c
    return torch.where(n > 30, torch.zeros_like(p), p >> n.clamp(max=30))


def isqrt(n):
    """Integer square root by 10 Newton steps from a power-of-two start.  ops.py:84-89."""
    n = n.clamp(min=0)
    x = torch.ones_like(n) << ((bitlen(n) + 1) // 2)
    for _ in range(10):
        x = torch.minimum(x, (x + n // x.clamp(min=1)) >> 1)
    return x.clamp(min=1)


def g_rms(D, blk):
    """Guard bits of RMSNorm forward / backward.  ops.py:28-30."""
    nb = D // blk
    return 2 * ((8 - int(math.log2(nb))) // 2), 14 - int(math.log2(D))


def _ilog2(n):
    k = int(n).bit_length() - 1
    assert 1 << k == n, f"{n} is not a power of two"
    return k


def _matmul_exact(a, b):
    """Exact integer a @ b^T for small-magnitude int tensors, through float64 (|result| < 2^53)."""
    return (a.to(torch.float64) @ b.to(torch.float64).t()).to(I64)


# ----------------------------------------------------------------------------- the operations
class Spec:
    """The 18 operations of the reference operator API, in int64, parametric in the block length.

    Signatures follow `OpsRef` (ops.py:92-290) so the parity tests read like the reference's
    own (`teste_ops.py`).  `limite` mirrors the module switch ATENCAO_LIMITE (ops.py:23).
    """
    nome = "spec"

    def __init__(self, blk=32, limite=False):
        self.blk = blk
        self.limite = limite

    # -- GEMM family -------------------------------------------------------------------------
    def gemm_acc(self, A, B, RA=None, RB=None):
        """Raw accumulator and base exponent of C = A . B^T.  ops.py:95-105.

        For every K-block the exact int8 dot product p is shifted left by GG and rounded by
        (RA_i - ea_ib) + (RB_j - eb_jb) before it is added.  RA / RB default to the row maxima
        of the exponents; a data-parallel rank passes the maxima over all ranks instead.
        """
        (a, ea), (b, eb) = A, B
        blk = self.blk
        M, K = a.shape
        ea, eb = ea.to(I64), eb.to(I64)
        RA = ea.amax(1) if RA is None else RA.to(I64)
        RB = eb.amax(1) if RB is None else RB.to(I64)
        acc = torch.zeros(M, b.shape[0], dtype=I64, device=a.device)
        for j in range(K // blk):
            sl = slice(j * blk, (j + 1) * blk)
            p = _matmul_exact(a[:, sl], b[:, sl])
            s = (RA - ea[:, j])[:, None] + (RB - eb[:, j])[None, :]
            acc += rnd(p << GG, s)
        return acc, RA[:, None] + RB[None, :] - GG

    def gemm(self, A, B, cru=False, RA=None, RB=None):
        acc, base = self.gemm_acc(A, B, RA, RB)
        if cru:                                                     # ops.py:106-107
            return acc.to(torch.int32), base.clamp(min=-30000).to(torch.int16)
        return quant(acc, base, self.blk)                           # ops.py:108

    def gemm_soma(self, A, B, X):                                   # ops.py:111-112
        return self.soma(X, self.gemm(A, B))

    def gemm_relu2(self, A, B):                                     # ops.py:114-116
        h = self.gemm(A, B)
        return h, self.relu2(h)

    def gemm_relu2_back(self, A, B, Hh):                            # ops.py:118-119
        return self.relu2_back(self.gemm(A, B), Hh)

    def max_linha(self, X):
        """Row-maximum exponents of a block tensor: the RA / RB of gemm_acc (ops.py:98)."""
        return X[1].amax(1).to(torch.int8)

    def rms_back_soma(self, X, Gg, Y, cache):
        """soma(X, rms_back(Gg, Y, cache)) (the CUDA library offers the pair as one launch)."""
        return self.soma(X, self.rms_back(Gg, Y, cache))

    def atencao_quant(self, QKV, Bt, T, H):
        """(quant(O), P) of atencao (the CUDA library offers the pair without the raw intermediate)."""
        oc, P = self.atencao(QKV, Bt, T, H)
        return self.quant(oc), P

    def atencao_back_quant(self, GO, QKV, P, Bt, T, H):
        return self.quant(self.atencao_back(GO, QKV, P, Bt, T, H))

    def transpoe2(self, X1, X2):
        """Two transpositions (the CUDA library offers the pair as one launch)."""
        return self.transpoe(X1), self.transpoe(X2)

    def transpoe(self, X):                                          # ops.py:121-123
        m, E = X
        return quant(m.to(I64).t().contiguous(), expande(E, self.blk).t().contiguous(), self.blk)

    # -- block elementwise -------------------------------------------------------------------
    def quant(self, C):                                             # ops.py:125-126
        return quant(C[0], C[1].to(I64), self.blk)

    def soma(self, X, Y):                                           # ops.py:128-132
        (xm, xE), (ym, yE) = X, Y
        blk = self.blk
        ec = torch.maximum(xE.to(I64), yE.to(I64)) - 21
        ece = expande(ec, blk)
        v = rnd(xm, ece - expande(xE, blk)) + rnd(ym, ece - expande(yE, blk))
        return quant(v, ece, blk)

    def relu2(self, Hh):                                            # ops.py:134-137
        m, E = Hh
        r = m.to(I64).clamp(min=0)
        return quant(r * r, 2 * expande(E, self.blk), self.blk)

    def relu2_back(self, Gg, Hh):                                   # ops.py:139-141
        (g, gE), (h, hE) = Gg, Hh
        v = g.to(I64) * h.to(I64).clamp(min=0) * 2
        return quant(v, expande(gE, self.blk) + expande(hE, self.blk), self.blk)

    def embed(self, W, tok):                                        # ops.py:143-145
        m, E = W
        idx = tok.long()
        return m[idx].contiguous(), E[idx].contiguous()

    def um_quente(self, tok, V):                                    # ops.py:147-151
        M = tok.numel()
        U = torch.zeros(M, V, dtype=torch.int8, device=tok.device)
        U[torch.arange(M, device=tok.device), tok.long()] = 1
        return U, torch.zeros(M, V // self.blk, dtype=torch.int8, device=tok.device)

    # -- RMSNorm -----------------------------------------------------------------------------
    def rms(self, X):                                               # ops.py:153-165
        m, E = X
        blk = self.blk
        R, D = m.shape
        G, _ = g_rms(D, blk)
        x, eb = m.to(I64), E.to(I64)
        sq = (x * x).reshape(R, D // blk, blk).sum(-1)
        emax = eb.amax(1, keepdim=True)
        ss = rnd(sq << G, 2 * (emax - eb)).sum(1)
        r = isqrt(ss >> _ilog2(D))
        k = bitlen(r) + 10
        inv = (torch.ones_like(k) << k) // r
        Y = quant(x * inv[:, None], expande(eb, blk) - k[:, None] - emax + G // 2, blk)
        return Y, (r.to(torch.int32), emax[:, 0].to(torch.int32))

    def rms_back(self, Gg, Y, cache):                               # ops.py:167-184
        (g, gE), (y, yE) = Gg, Y
        blk = self.blk
        r, emax = cache[0].to(I64), cache[1].to(I64)
        R, D = g.shape
        G, GB = g_rms(D, blk)
        lg = _ilog2(D)
        g, y, gE, yE = g.to(I64), y.to(I64), gE.to(I64), yE.to(I64)
        esum = gE + yE
        smax = esum.amax(1, keepdim=True)
        S = rnd((g * y) << GB, expande(smax - esum, blk)).sum(1)
        eS = smax[:, 0] - GB - lg
        sh = (bitlen(S) - 15).clamp(min=0)
        S, eS = rnd(S, sh), eS + sh
        ec = torch.maximum(gE + 7, yE + eS[:, None] + 22) - 28
        inner = rnd(g, expande(ec - gE, blk)) - rnd(y * S[:, None], expande(ec - (yE + eS[:, None]), blk))
        sh2 = (bitlen(inner) - 18).clamp(min=0)
        inner = rnd(inner, sh2)
        k = bitlen(r) + 10
        inv = (torch.ones_like(k) << k) // r
        return quant(inner * inv[:, None], expande(ec, blk) + sh2 - k[:, None] - (emax[:, None] - G // 2), blk)

    # -- attention ---------------------------------------------------------------------------
    def _alinha(self, m, E, Bt, T, H, col0, D):
        """One of q / k / v / dO, per (sequence, head), aligned to a single exponent.

        ops.py:186-192 at head dim 4: the head's 4 mantissas share one block exponent; every
        token is shifted (with GA guard bits) onto the largest exponent of that head in that
        sequence.  Generalisation: the exponent is taken per element (a head of hd > blk
        columns spans hd/blk blocks) and the maximum runs over all tokens and all columns of
        the head.  With hd dividing blk this is the reference rule unchanged.
        Returns (aligned int64 [Bt,H,T,hd], exponent int64 [Bt,H,1]).
        """
        hd = D // H
        x = m.to(I64)[:, col0:col0 + D].reshape(Bt, T, H, hd).permute(0, 2, 1, 3)
        ex = expande(E, self.blk)[:, col0:col0 + D].reshape(Bt, T, H, hd).permute(0, 2, 1, 3)
        top = ex.amax((-2, -1), keepdim=True)
        return rnd(x << GA, top - ex), top[..., 0] - GA

    @staticmethod
    def _incl(H, dev):
        """ALiBi slope exponent per head: distance is multiplied by 2^incl in 1/256 units.

        ops.py:208 writes 8 - h // 8 (for its 64 heads: 8 groups, slopes 2^0 .. 2^-7).  The formula is
        kept literally for every head count, because the reference evaluates exactly this expression
        for any H it accepts (H <= 64); with H = 8 every head therefore has slope 1.
        """
        h = torch.arange(H, device=dev)
        return (8 - h // 8).clamp(min=0)[:, None, None]

    def atencao(self, QKV, Bt, T, H):                               # ops.py:198-219
        m, E = QKV
        D = m.shape[1] // 3
        hd = D // H
        lg = _ilog2(hd)
        assert lg % 2 == 0, "head dim must be a power of 4 (1/sqrt(hd) has to be a power of two)"
        qa, eq = self._alinha(m, E, Bt, T, H, 0, D)
        ka, ek = self._alinha(m, E, Bt, T, H, D, D)
        va, ev = self._alinha(m, E, Bt, T, H, 2 * D, D)
        dev = m.device
        i = torch.arange(T, device=dev)
        dist = i[:, None] - i[None, :]
        fut = dist < 0
        prod = torch.matmul(qa.to(torch.float64), ka.to(torch.float64).transpose(-1, -2)).to(I64)
        # score in 1/256 units: prod * 2^(eq+ek) / sqrt(hd) * 256   (ops.py:209 with lg/2 = 1)
        u = rnd(prod, -(eq + ek - lg // 2 + 8)[..., None]) - (dist.clamp(min=0)[None] << self._incl(H, dev))
        u = torch.where(fut, torch.full_like(u, -(2**31 - 1)), u)
        mx = u.amax(-1, keepdim=True)
        ex = torch.where(fut, torch.zeros_like(u), exp_int(mx - u) >> 3)
        inv = (1 << 28) // ex.sum(-1, keepdim=True)
        P = torch.where(fut, torch.zeros_like(u), ((ex * inv + (1 << 19)) >> 20).clamp(max=255))
        o = torch.matmul(P.to(torch.float64), va.to(torch.float64)).to(I64)          # (Bt,H,T,hd), < 2^53
        oacc = o.permute(0, 2, 1, 3).reshape(Bt * T, D)
        oe = (ev - 8)[..., None].expand(Bt, H, T, hd).permute(0, 2, 1, 3).reshape(Bt * T, D)
        Pt = P.transpose(-1, -2).reshape(Bt * H, T, T)              # stored key-major: [j][i]
        return (oacc.to(torch.int32).contiguous(), oe.to(torch.int16).contiguous()), Pt.to(torch.uint8).contiguous()

    def atencao_back(self, GO, QKV, P, Bt, T, H):                   # ops.py:221-258
        (gm, gE), (m, E) = GO, QKV
        D = gm.shape[1]
        hd = D // H
        goa, ego = self._alinha(gm, gE, Bt, T, H, 0, D)
        qa, eq = self._alinha(m, E, Bt, T, H, 0, D)
        ka, ek = self._alinha(m, E, Bt, T, H, D, D)
        va, ev = self._alinha(m, E, Bt, T, H, 2 * D, D)
        f64 = torch.float64
        Pl = P.to(I64).reshape(Bt, H, T, T).transpose(-1, -2)        # P[i][j]
        gP = torch.matmul(goa.to(f64), va.to(f64).transpose(-1, -2)).to(I64)
        t = torch.arange(T, device=gm.device)
        causal = t[:, None] >= t[None, :]
        zero = torch.zeros_like(gP)
        if self.limite:          # |gP_ij| <= max_i ||dO_i||_inf * max_j ||v_j||_1        (ops.py:231-233)
            lim = goa.abs().amax((-2, -1)) * va.abs().sum(-1).amax(-1)
            sh = (bitlen(lim)[..., None, None] - 15).clamp(min=0)
        else:                    # exact causal maximum                                    (ops.py:235)
            sh = (bitlen(torch.where(causal, gP.abs(), zero).amax((-2, -1), keepdim=True)) - 15).clamp(min=0)
        gP = rnd(gP, sh)
        egp = ego + ev + sh[..., 0]
        sl = rnd((Pl * gP).sum(-1, keepdim=True), 8)
        dS = Pl * (gP - sl)
        if self.limite:                                                                   # ops.py:240-242
            lim2 = Pl.amax((-2, -1)) * (torch.where(causal, gP.abs(), zero).amax((-2, -1)) + sl.abs().amax((-2, -1)))
            sh2 = (bitlen(lim2)[..., None, None] - 12).clamp(min=0)
        else:                                                                             # ops.py:244
            sh2 = (bitlen(dS.abs().amax((-2, -1), keepdim=True)) - 12).clamp(min=0)
        dS = rnd(dS, sh2)
        eds = egp - 9 + sh2[..., 0]
        dSf, Plf = dS.to(f64), Pl.to(f64)
        gq = torch.matmul(dSf, ka.to(f64)).to(I64)
        gk = torch.matmul(dSf.transpose(-1, -2), qa.to(f64)).to(I64)
        gv = torch.matmul(Plf.transpose(-1, -2), goa.to(f64)).to(I64)

        def lin(x):
            return x.permute(0, 2, 1, 3).reshape(Bt * T, D)

        def exps(e):
            return lin(e[..., None].expand(Bt, H, T, hd))
        acc = torch.cat([lin(gq), lin(gk), lin(gv)], 1)
        e = torch.cat([exps(eds + ek), exps(eds + eq), exps(ego - 8)], 1)
        return acc.to(torch.int32).contiguous(), e.to(torch.int16).contiguous()

    # -- loss --------------------------------------------------------------------------------
    def softmax_ce(self, L, alvo, log2M=None):                      # ops.py:260-271
        """`log2M` defaults to log2 of the local row count; a data-parallel rank passes the
        log2 of the global token count so that the gradient scale matches the full batch."""
        acc, e = L
        M = acc.shape[0]
        if log2M is None:
            log2M = _ilog2(M)
        u = rnd(acc, -(e.to(I64) + 8))
        umax = u.amax(1, keepdim=True)
        ex = exp_int(umax - u) >> 3
        s = ex.sum(1, keepdim=True)
        v = (ex * ((1 << 28) // s) + (1 << 15)) >> 16
        rows = torch.arange(M, device=acc.device)
        v[rows, alvo.long()] -= 4096
        g = quant(v, -12 - log2M, self.blk)
        return g, (umax[:, 0] - u[rows, alvo.long()]).to(torch.int32), s[:, 0].to(torch.int32)

    # -- optimiser ---------------------------------------------------------------------------
    def momento(self, Gc, Mom):                                     # ops.py:273-278
        (g, ge), (mm, mE) = Gc, Mom
        g, ge = g.to(I64), ge.to(I64)
        em = expande(mE, self.blk) - 3
        ec = torch.maximum(em + 10, ge + bitlen(g)) - 28
        return quant(rnd(mm.to(I64) * 7, ec - em) + rnd(g, ec - ge), ec, self.blk)

    def peso(self, W, Mom, R, k, ef):                               # ops.py:280-290
        (w, wE), (mm, mE), (r, rE) = W, Mom, R
        blk = self.blk
        ew, em = expande(wE, blk), expande(mE, blk) - k
        er = expande(rE, blk) if ef else torch.full_like(ew, E_ZERO)
        ec = torch.maximum(torch.maximum(ew + 7, em + 7), er + 7) - 27
        alvo = rnd(w, ec - ew) - rnd(mm, ec - em)
        if ef:
            alvo = alvo + rnd(r, ec - er)
        w2, wE2 = quant(alvo, ec, blk)
        if not ef:
            return (w2, wE2), R
        back = torch.where(w2 == 0, torch.zeros_like(alvo), rnd(w2, ec - expande(wE2, blk)))
        return (w2, wE2), quant(alvo - back, ec, blk)

    def momento_peso(self, Gc, Mom, W, R, k, ef):
        """The optimiser step of one weight: momento then peso on its result (ops.py:273-290 composed; the CUDA library
        offers the pair as one launch)."""
        Mom2 = self.momento(Gc, Mom)
        W2, R2 = self.peso(W, Mom2, R, k, ef)
        return Mom2, W2, R2
