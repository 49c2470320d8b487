"""The integer-only Transformer training step, written purely against the operator API.

Host-side mirror of the reference's jatai_cuda/modelo.py (Modelo :29-140, PassoGravado :143-180): pre-norm
Transformer, RMSNorm without gain, causal ALiBi attention, ReLU^2 MLP, byte vocabulary, q/k/v in one [3D, D]
matrix; SGD with momentum 7/8, learning rate 2^-k, error feedback on the weights.  The same code runs on the
CUDA launcher (`ops.OpsCuda`) and on any object with the same methods (the tests drive it with the int64
oracle on CPU), because it only ever calls `self.ops.<op>(...)` and the registry's `trecho()`.

Same constructor, same `passo(tok, alvo, k_lr)`, same weight names and the same seeded initialisation (generator
and draw order of modelo.py:16-19,32-40) as the reference, so a run here and a run of the reference model start
from identical weights.  Not included: the reference's opt-in 16-bit residual stream (JATAI_RES16).

Data parallel: pass `redutor` (see jatai_b200.paralelo).  Every op except the weight-gradient GEMMs is per token
or per sequence; the weight-gradient GEMM reduces over tokens, so ranks first agree on the row-maximum exponents
(MAX), run the GEMM on their own tokens with those, and add the int32 partial sums (SUM).  A weight gradient feeds
nothing but the optimiser, so all weight-gradient GEMMs are deferred to the end of the backward: a data-parallel step
is forward + backward with no communication, ONE MAX collective, the deferred GEMMs, ONE SUM collective, the
optimiser.  Integer addition is associative, so the result is bit-identical to one GPU running the concatenated batch.
"""
import math

import os
import torch

from . import ops as O


def inicial(g, linhas, fan_in, dev, emb=False):
    """Seeded initial weight block tensor: mantissa round(32 N(0,1)), one exponent for the whole tensor."""
    e = -5 if emb else -int(round(math.log2(32 * math.sqrt(fan_in))))
    m = torch.round(torch.randn(linhas, fan_in, generator=g) * 32).clamp(-127, 127).to(torch.int8)
    E = torch.full((linhas, fan_in // O.BLK), e, dtype=torch.int8, device=dev)
    return m.to(dev).contiguous(), E


def zeros_como(t):
    return torch.zeros_like(t[0]), torch.full_like(t[1], O.E_ZERO)


class Modelo:
    def __init__(self, V, D, H, FF, L, semente, dev, ops, reg, redutor=None):
        self.V, self.D, self.H, self.FF, self.L = V, D, H, FF, L
        self.dev, self.ops, self.reg, self.redutor = dev, ops, reg, redutor
        g = torch.Generator().manual_seed(semente)
        p = {"emb": inicial(g, V, D, dev, emb=True)}
        for l in range(L):
            qkv = [inicial(g, D, D, dev) for _ in range(3)]
            p[f"Wqkv{l}"] = (torch.cat([t[0] for t in qkv]).contiguous(), torch.cat([t[1] for t in qkv]).contiguous())
            p[f"Wo{l}"] = inicial(g, D, D, dev)
            p[f"Wup{l}"] = inicial(g, FF, D, dev)
            p[f"Wd{l}"] = inicial(g, D, FF, dev)
        p["out"] = inicial(g, V, D, dev)
        self.p = p
        self.mom = {n: zeros_como(t) for n, t in p.items()}
        self.res = {n: zeros_como(t) for n, t in p.items()}
        self.error_feedback = True
        self.estatisticas = False
        # second stream for the weight-gradient GEMMs (single GPU, CUDA launcher only)
        usa_lado = hasattr(ops, "lib") and torch.device(dev).type == "cuda"
        self._lado = torch.cuda.Stream(device=dev) if usa_lado else None
        self._pendente, self._feitos, self._k_lr_lado = None, set(), None
        na_gpu = redutor is not None and hasattr(ops, "lib") and torch.device(dev).type == "cuda"
        self._ramos = [torch.cuda.Stream(device=dev) for _ in range(3)] if na_gpu else []

    # ------------------------------------------------------------------ helpers
    def _st(self, nome, t, zeros_normais=False):
        if self.estatisticas:
            self.reg.estatistica(nome, t, zeros_normais)

    def _soma_rms_back(self, gx, gn, y, cache):
        """gx + rms_back(gn, y, cache): one launch where the operator object offers the pair."""
        junto = getattr(self.ops, "rms_back_soma", None)
        if junto is not None:
            return junto(gx, gn, y, cache)
        return self.ops.soma(gx, self.ops.rms_back(gn, y, cache))

    def _atencao_quant(self, qkv, Bt, T):
        """quant(atencao(qkv)) and P: one launch where the operator object offers the pair."""
        junto = getattr(self.ops, "atencao_quant", None)
        if junto is not None:
            return junto(qkv, Bt, T, self.H)
        oc, P = self.ops.atencao(qkv, Bt, T, self.H)
        return self.ops.quant(oc), P

    def _atencao_back_quant(self, go, qkv, P, Bt, T):
        junto = getattr(self.ops, "atencao_back_quant", None)
        if junto is not None:
            return junto(go, qkv, P, Bt, T, self.H)
        return self.ops.quant(self.ops.atencao_back(go, qkv, P, Bt, T, self.H))

    def _transpoe_par(self, gy, x):
        """Both operands of a weight-gradient GEMM transposed: one launch where the operator object offers the pair."""
        par = getattr(self.ops, "transpoe2", None)
        if par is not None and gy[0].shape[0] == x[0].shape[0]:
            return par(gy, x)
        return self.ops.transpoe(gy), self.ops.transpoe(x)

    def _transpoe_par_max(self, gy, x):
        """Data parallel: both operands of a weight-gradient GEMM transposed, with their row maxima - written by the
        transposition itself into the reducer's buffer where the launcher and the reducer offer that, by max_linha otherwise."""
        ops, red = self.ops, self.redutor
        junto, fatias = getattr(ops, "transpoe2_max", None), getattr(red, "fatias_max", None)
        if junto is not None and fatias is not None and gy[0].shape[0] == x[0].shape[0] and gy[0].shape[1] % 256 == 0 and x[0].shape[1] % 256 == 0:
            f = fatias(gy[0].shape[1], x[0].shape[1])
            if f is not None:
                par = junto(gy, x, f[0], f[1])
                if par is not None:
                    return par[0], par[1], f[0], f[1]
                a, b = self._transpoe_par(gy, x)                    # the slices are taken: fill them the long way
                f[0].copy_(ops.max_linha(a))
                f[1].copy_(ops.max_linha(b))
                return a, b, f[0], f[1]
        a, b = self._transpoe_par(gy, x)
        return a, b, ops.max_linha(a), ops.max_linha(b)

    def _grad_peso(self, nome, gy, x):
        """dW = gy^T . x as a raw tensor.  Both operands are transposed so that the reduced dimension (tokens)
        is the blocked one.  Data parallel: the GEMM is deferred - only the transposed operands and their row
        maxima are kept - because a weight gradient feeds nothing but the optimiser; all of them run after the
        backward, between the two collectives of the step (see `_gemms_adiados`)."""
        ops = self.ops
        if self._lado is None:
            if self.redutor is None:
                a, b = self._transpoe_par(gy, x)
                self._grads[nome] = ops.gemm(a, b, cru=True)
            else:
                self._adiados.append((nome, *self._transpoe_par_max(gy, x)))
            return
        # A weight gradient is a leaf of the backward graph: its two transpositions and its GEMM run on a second
        # stream, next to the dX chain, and fill SMs the small GEMMs of that chain leave idle.  Under capture the
        # second stream becomes a parallel branch of the CUDA graph.
        principal = torch.cuda.current_stream()
        self._lado.wait_stream(principal)
        for t in (*gy, *x):
            t.record_stream(self._lado)
        with torch.cuda.stream(self._lado):
            ops.lib.jt_stream(self._lado.cuda_stream)
            try:
                self._otimiza_pendente()
                if self.redutor is None:
                    a, b = self._transpoe_par(gy, x)
                    self._grads[nome] = ops.gemm(a, b, cru=True)
                    self._pendente = nome
                else:       # data parallel: only the transpositions and the row maxima now, the GEMM after the exchange
                    self._adiados.append((nome, *self._transpoe_par_max(gy, x)))
            finally:
                ops.lib.jt_stream(principal.cuda_stream)

    def _pesos_transpostos(self):
        """The backward multiplies by every weight transposed (and re-quantised along the new rows).  The weights do not change
        between the start of a step and their own update, so on the CUDA launcher all those transpositions are issued at the
        start of the step on the second stream, beside the forward pass, instead of inside the backward's dependency chain.
        Returns {id of the weight's mantissa tensor: transposed block tensor} (empty where there is no second stream)."""
        if self._lado is None:
            return {}
        ops, principal = self.ops, torch.cuda.current_stream()
        self._lado.wait_stream(principal)
        wt = {}
        with torch.cuda.stream(self._lado):
            ops.lib.jt_stream(self._lado.cuda_stream)
            try:
                with self.reg.trecho("pesos transpostos"):
                    for n, w in self.p.items():
                        if n != "emb":
                            wt[id(w[0])] = t = ops.transpoe(w)
                            for x in t:
                                x.record_stream(principal)
            finally:
                ops.lib.jt_stream(principal.cuda_stream)
        return wt

    def _otimiza_pendente(self):
        """Single GPU, on the second stream: the optimiser step of the weight whose gradient was computed by the
        previous call.  Safe because the second stream has just waited for the main stream, and by then the main
        stream has queued its last read of that weight in this step (each weight is read once in the forward and
        once, transposed, in the backward, right after its own `_grad_peso` call)."""
        n = self._pendente
        if n is None or self._k_lr_lado is None:
            return
        with self.reg.trecho("otimizador"), self.reg.trecho(n):
            self._otimiza({n: self._grads[n]}, self._k_lr_lado)
        self._feitos.add(n)
        self._pendente = None

    def _gemms_adiados(self, maximos, inicio=0, fim=None):
        """Data parallel, after the MAX collective: the weight-gradient GEMMs [inicio, fim) of the deferred list (all of
        them by default) with the global row maxima.  The GEMMs are independent of each other, so on the GPU they are
        dealt round-robin to a few streams (parallel branches of the CUDA graph when recording) and joined at the end.
        The list is cleared when its last GEMM has been issued."""
        ops = self.ops
        fim = len(self._adiados) if fim is None else fim
        principal = torch.cuda.current_stream() if self._ramos else None
        for r in self._ramos:
            r.wait_stream(principal)
        for i, ((nome, a, b, _, _), (RA, RB)) in enumerate(zip(self._adiados[inicio:fim], maximos[inicio:fim])):
            with self.reg.trecho(nome):
                if not self._ramos:
                    self._grads[nome] = ops.gemm(a, b, cru=True, RA=RA, RB=RB)
                    continue
                ramo = self._ramos[i % len(self._ramos)]
                for t in (*a, *b, RA, RB):
                    t.record_stream(ramo)
                with torch.cuda.stream(ramo):
                    ops.lib.jt_stream(ramo.cuda_stream)
                    try:
                        self._grads[nome] = ops.gemm(a, b, cru=True, RA=RA, RB=RB)
                    finally:
                        ops.lib.jt_stream(principal.cuda_stream)
        for r in self._ramos:
            principal.wait_stream(r)
        if fim == len(self._adiados):
            self._adiados = []

    def _otimiza(self, grads, k_lr):
        ops = self.ops
        junto = getattr(ops, "momento_peso", None)        # one launch for the pair where the library has it
        for n, gr in grads.items():
            with self.reg.trecho(n):
                if junto is not None:
                    self.mom[n], self.p[n], self.res[n] = junto(gr, self.mom[n], self.p[n], self.res[n], k_lr, self.error_feedback)
                    continue
                self.mom[n] = ops.momento(gr, self.mom[n])
                self.p[n], self.res[n] = ops.peso(self.p[n], self.mom[n], self.res[n], k_lr, self.error_feedback)

    # ------------------------------------------------------------------ the step
    def passo(self, tok, alvo, k_lr=None):
        """Forward (+ backward and update when k_lr is given).  Returns the loss as a tensor (report only, float)."""
        perda = self.frente_tras(tok, alvo, treina=k_lr is not None, k_lr=k_lr)
        if k_lr is None:
            return perda
        grads = {n: g for n, g in self._grads.items() if n not in self._feitos}       # the rest (all of them without a second stream)
        if self.redutor is not None:
            with self.reg.trecho("gradientes de peso"):
                self._gemms_adiados(self.redutor.maximos_tudo([(ra, rb) for _, _, _, ra, rb in self._adiados]))
                grads = self.redutor.soma_tudo(self._grads)
        with self.reg.trecho("otimizador"):
            self._otimiza(grads, k_lr)
        return perda

    def frente_tras(self, tok, alvo, treina=True, k_lr=None):
        """Forward and (if `treina`) backward.  Weight gradients land in self._grads (single GPU) or, data parallel,
        their operands in self._adiados.  No communication happens here.  With `k_lr` on a single GPU the optimiser
        step of each weight also runs here, on the second stream, as soon as its gradient exists."""
        for _ in self.em_trechos(tok, alvo, treina=treina, k_lr=k_lr):
            pass
        return self._perda

    def cortes(self, grupos):
        """Layer indices after which the backward is cut so that it falls into `grupos` pieces of consecutive layers (the
        backward walks the layers from the last to the first; the output head belongs to the first piece, the embedding to
        the last)."""
        ordem = list(reversed(range(self.L)))
        grupos = max(1, min(grupos, self.L))
        return {ordem[len(ordem) * g // grupos - 1] for g in range(1, grupos)}

    def em_trechos(self, tok, alvo, treina=True, k_lr=None, cortes=()):
        """`frente_tras` as a generator: it yields after the backward of every layer listed in `cortes`, with the side
        stream joined, so that a caller can end a CUDA graph there and put a collective between two pieces (data
        parallel: the weight-gradient operands of the piece just finished are the new entries of self._adiados).  The loss
        tensor is left in self._perda."""
        ops, reg, p = self.ops, self.reg, self.p
        Bt, T = tok.shape
        tok = tok.reshape(-1).to(torch.int32).contiguous()
        alvo = alvo.reshape(-1).to(torch.int32).contiguous()
        self._grads, self._adiados = {}, []
        self._pendente, self._feitos = None, set()
        self._k_lr_lado = k_lr if (self.redutor is None and self._lado is not None) else None
        inicio = getattr(self.redutor, "inicio_passo", None) if treina else None
        if inicio is not None:
            inicio()                                               # data parallel: the buffer of row maxima starts the step at -128
        guardados = []
        wt = self._pesos_transpostos() if treina else {}
        with reg.trecho("forward"):
            with reg.trecho("embedding"):
                x = ops.embed(p["emb"], tok)
            for l in range(self.L):
                with reg.trecho(f"camada {l}"):
                    with reg.trecho("atencao"):
                        n1, c1 = ops.rms(x)
                        qkv = ops.gemm(n1, p[f"Wqkv{l}"])
                        om, P = self._atencao_quant(qkv, Bt, T)
                        x = ops.gemm_soma(om, p[f"Wo{l}"], x)
                        self._st(f"c{l}.qkv", qkv); self._st(f"c{l}.atencao_saida", om); self._st(f"c{l}.residuo1", x)
                    with reg.trecho("mlp"):
                        n2, c2 = ops.rms(x)
                        h, a = ops.gemm_relu2(n2, p[f"Wup{l}"])
                        x = ops.gemm_soma(a, p[f"Wd{l}"], x)
                        self._st(f"c{l}.relu2", a, zeros_normais=True); self._st(f"c{l}.residuo2", x)
                guardados.append((n1, c1, qkv, P, om, n2, c2, h, a))
            with reg.trecho("saida"):
                nf, cf = ops.rms(x)
                logits = ops.gemm(nf, p["out"], cru=True)
                if self.redutor is None:
                    g, d_alvo, soma = ops.softmax_ce(logits, alvo)
                else:
                    g, d_alvo, soma = ops.softmax_ce(logits, alvo, log2M=self.redutor.log2_tokens(tok.numel()))
        # loss report: stays on the device; the caller converts after the step without stalling the queue
        self._perda = perda = (d_alvo.double() / 256 + torch.log(soma.double() / 4096)).mean()
        if not treina:
            return
        if self._lado is not None and wt:
            torch.cuda.current_stream().wait_stream(self._lado)         # the transposed weights are ready (they were, long ago)
        T_ = lambda w: wt[id(w[0])] if id(w[0]) in wt else ops.transpoe(w)
        with reg.trecho("backward"):
            with reg.trecho("saida"):
                self._grad_peso("out", g, nf)
                gx = ops.rms_back(ops.gemm(g, T_(p["out"])), nf, cf)
                self._st("grad_saida", gx)
            for l in reversed(range(self.L)):
                n1, c1, qkv, P, om, n2, c2, h, a = guardados[l]
                with reg.trecho(f"camada {l}"):
                    with reg.trecho("mlp"):
                        self._grad_peso(f"Wd{l}", gx, a)
                        gh = ops.gemm_relu2_back(gx, T_(p[f"Wd{l}"]), h)
                        self._grad_peso(f"Wup{l}", gh, n2)
                        gn = ops.gemm(gh, T_(p[f"Wup{l}"]))
                        gx = self._soma_rms_back(gx, gn, n2, c2)
                        self._st(f"c{l}.grad_mlp", gh, zeros_normais=True)
                    with reg.trecho("atencao"):
                        self._grad_peso(f"Wo{l}", gx, om)
                        go = ops.gemm(gx, T_(p[f"Wo{l}"]))
                        gq = self._atencao_back_quant(go, qkv, P, Bt, T)
                        self._grad_peso(f"Wqkv{l}", gq, n1)
                        gn = ops.gemm(gq, T_(p[f"Wqkv{l}"]))
                        gx = self._soma_rms_back(gx, gn, n1, c1)
                        self._st(f"c{l}.grad_qkv", gq); self._st(f"c{l}.grad_residuo", gx)
                if l in cortes:
                    if self._lado is not None:
                        torch.cuda.current_stream().wait_stream(self._lado)
                    yield l
            with reg.trecho("embedding"):
                self._grad_peso("emb", ops.um_quente(tok, self.V), gx)
        if self._lado is not None:
            if self._pendente is not None and self._k_lr_lado is not None:
                principal = torch.cuda.current_stream()
                self._lado.wait_stream(principal)
                with torch.cuda.stream(self._lado):
                    ops.lib.jt_stream(self._lado.cuda_stream)
                    try:
                        self._otimiza_pendente()
                    finally:
                        ops.lib.jt_stream(principal.cuda_stream)
            torch.cuda.current_stream().wait_stream(self._lado)          # join the weight-gradient branch


class PassoGravado:
    """One training step recorded in a CUDA graph and replayed: the few hundred launches become one call.

    Recording executes nothing (weights do not change while recording).  Everything the step allocates lives in
    the graph's pool at fixed addresses; weights, momentum and residual are updated in place by the kernels, so
    the graph stays valid.  Inputs go to fixed buffers (copy_) before each replay.  The launch list of the
    recording is kept: the launch ids are baked into the kernel arguments, so a sentinel raised during a replay
    names the same operation and section as it would in eager mode.  Run one eager step before recording (the
    attention sizes its workspace on first use, which a capture does not allow).

    Data parallel: no collective is ever part of a captured graph; the step is cut into GRUPOS pieces of consecutive layers
    and recorded as 3 graphs per piece, with the collectives issued eagerly between the replays:
        M_g  forward (g = 0) and the backward of piece g, the transpositions of its weight-gradient operands on the side
             branch, writing their row maxima into the piece's slice of the flat buffer                     main stream
        MAX  all-reduce of that slice (a few KB, on a communicator of its own)
        D_g  the weight-gradient GEMMs of piece g with the global maxima, sums packed into the flat buffer   second stream
        SUM  all-reduce of the piece's int32 sums (asynchronous)
        O_g  the optimiser step of the piece's weights                                                      third stream
    The main stream goes straight on to M_{g+1} after queueing MAX_g, so the weight-gradient GEMMs, the gradient traffic and
    the optimiser of piece g run beside the backward of piece g + 1, as the single-GPU step runs them beside its backward;
    only the last piece's tail is exposed.  The backward never reads a weight again after its own piece (it multiplies by
    the transposed copies made at the start of the step), so O_g may update it while the backward goes on.
    """

    GRUPOS = int(os.environ.get("JT_GRUPOS", "12"))         # data parallel: pieces of consecutive layers (measured: 12 beats 4 and 6)

    def __init__(self, modelo, Bt, T, k_lr):
        self.m, self.reg, self.k_lr = modelo, modelo.reg, k_lr
        lib = modelo.ops.lib
        self.tok = torch.zeros(Bt, T, dtype=torch.long, device=modelo.dev)
        self.alvo = torch.zeros(Bt, T, dtype=torch.long, device=modelo.dev)
        est, vig, perf = modelo.estatisticas, self.reg.vigiar, self.reg.perfil
        modelo.estatisticas, self.reg.vigiar, self.reg.perfil = False, False, False     # nothing that synchronises while recording
        torch.cuda.synchronize()
        self.reg.lancamentos = []
        red = modelo.redutor
        try:
            if red is None:
                self.grafos = [torch.cuda.CUDAGraph()]
                with torch.cuda.graph(self.grafos[0]):
                    lib.jt_stream(torch.cuda.current_stream().cuda_stream)
                    self.perda = modelo.passo(self.tok, self.alvo, k_lr=k_lr)
            else:
                # The reducer's flat buffers must already exist with their final sizes (one eager step has run), so the
                # graphs see fixed addresses.
                assert getattr(red, "_max", None) is not None and getattr(red, "_plano", None) is not None, \
                    "run one eager data-parallel step before recording"
                cortes = modelo.cortes(self.GRUPOS)
                ng = len(cortes) + 1
                trechos = modelo.em_trechos(self.tok, self.alvo, treina=True, k_lr=None, cortes=cortes)
                self._M, self._D, self._O, self._fatias_max, self._fatias = [], [], [], [], []
                grupos, n0, o_max, pool_m = [], 0, 0, None
                for g in range(ng):
                    gm = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gm, **({} if pool_m is None else {"pool": pool_m})):
                        lib.jt_stream(torch.cuda.current_stream().cuda_stream)
                        next(trechos, None)
                        novos = modelo._adiados[n0:]
                        o1 = red.empacota_maximos([(ra, rb) for _, _, _, ra, rb in novos], o_max)
                    pool_m = gm.pool()
                    self._M.append(gm)
                    self._fatias_max.append((o_max, o1))
                    grupos.append((n0, n0 + len(novos)))
                    n0, o_max = n0 + len(novos), o1
                assert next(trechos, "fim") == "fim" and o_max == red._max.numel()
                self.perda = modelo._perda
                adiados = list(modelo._adiados)                       # every operand the later graphs read stays referenced here
                maximos = red.vistas_maximos([(ra, rb) for _, _, _, ra, rb in adiados])
                nomes = [a[0] for a in adiados]
                self._lado = torch.cuda.Stream(device=modelo.dev)
                self._lado2 = torch.cuda.Stream(device=modelo.dev)
                pool_l, pool_o, vistas_g = None, None, []
                for g, (a0, a1) in enumerate(grupos):
                    with torch.cuda.stream(self._lado):
                        gd = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(gd, stream=self._lado, **({} if pool_l is None else {"pool": pool_l})):
                            lib.jt_stream(torch.cuda.current_stream().cuda_stream)
                            modelo._adiados = adiados
                            modelo._gemms_adiados(maximos, a0, a1)
                            v, fatia = red.empacota_grupo({k: modelo._grads[k] for k in nomes[a0:a1]}, modelo._grads)
                        pool_l = gd.pool()
                    # the optimiser graphs run on a third stream with a pool of their own: while piece g's sums are on the wire
                    # and being applied, the second stream already runs the GEMMs of piece g + 1
                    with torch.cuda.stream(self._lado2):
                        go = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(go, stream=self._lado2, **({} if pool_o is None else {"pool": pool_o})):
                            lib.jt_stream(torch.cuda.current_stream().cuda_stream)
                            with self.reg.trecho("otimizador"):
                                modelo._otimiza(v, k_lr)
                        pool_o = go.pool()
                    self._D.append(gd)
                    self._O.append(go)
                    self._fatias.append(fatia)
                    vistas_g.append(v)
                self._vivos = (adiados, vistas_g, dict(modelo._grads), maximos)
                self.grafos = self._M + self._D + self._O
        finally:
            lib.jt_stream(None)
            modelo.estatisticas, self.reg.vigiar, self.reg.perfil = est, vig, perf
        self.lancamentos = list(self.reg.lancamentos)
        self.coletivos_por_passo = 0 if red is None else 2 * len(self._M)
        self.reg.info(f"step recorded in {len(self.grafos)} CUDA graph(s): {len(self.lancamentos)} launches", lancamentos=len(self.lancamentos))

    def __call__(self, tok, alvo):
        self.tok.copy_(tok)
        self.alvo.copy_(alvo)
        self.reg.lancamentos = self.lancamentos
        if len(self.grafos) == 1:
            self.grafos[0].replay()
            return self.perda
        red = self.m.redutor
        principal = torch.cuda.current_stream()
        for gm, gd, go, fmax, fsoma in zip(self._M, self._D, self._O, self._fatias_max, self._fatias):
            gm.replay()
            pronto_max = red.reduz_maximos_fatia(*fmax)           # asynchronous, ordered after the piece just queued
            with torch.cuda.stream(self._lado):
                pronto_max.wait()
                gd.replay()
                pronto = red.reduz_fatia(*fsoma)                  # asynchronous: ordered after this piece's GEMMs
            with torch.cuda.stream(self._lado2):
                pronto.wait()                                     # the second stream does not wait for the sums: it goes on
                go.replay()                                       # with the next piece's GEMMs
        principal.wait_stream(self._lado)
        principal.wait_stream(self._lado2)                        # the next step reads every weight
        return self.perda
