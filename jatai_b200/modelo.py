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

    def _transpoe_par(self, gy, x):
        """Both operands of a weight-gradient GEMM transposed: one launch where the operator object offers the pair."""
        par = getattr(self.ops, "transpoe2", None)
        if par is not None and gy[0].shape[0] == x[0].shape[0]:
            return par(gy, x)
        return self.ops.transpoe(gy), self.ops.transpoe(x)

    def _grad_peso(self, nome, gy, x):
        """dW = gy^T . x as a raw tensor.  Both operands are transposed so that the reduced dimension (tokens)
        is the blocked one.  Data parallel: the GEMM is deferred - only the transposed operands and their row
        maxima are kept - because a weight gradient feeds nothing but the optimiser; all of them run after the
        backward, between the two collectives of the step (see `_gemms_adiados`)."""
        ops = self.ops
        if self._lado is None:
            a, b = self._transpoe_par(gy, x)
            if self.redutor is None:
                self._grads[nome] = ops.gemm(a, b, cru=True)
            else:
                self._adiados.append((nome, a, b, ops.max_linha(a), ops.max_linha(b)))
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
                a, b = self._transpoe_par(gy, x)
                if self.redutor is None:
                    self._grads[nome] = ops.gemm(a, b, cru=True)
                    self._pendente = nome
                else:       # data parallel: only the transpositions and the row maxima now, the GEMM after the exchange
                    self._adiados.append((nome, a, b, ops.max_linha(a), ops.max_linha(b)))
            finally:
                ops.lib.jt_stream(principal.cuda_stream)

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
        ops, reg, p = self.ops, self.reg, self.p
        Bt, T = tok.shape
        tok = tok.reshape(-1).to(torch.int32).contiguous()
        alvo = alvo.reshape(-1).to(torch.int32).contiguous()
        self._grads, self._adiados = {}, []
        self._pendente, self._feitos = None, set()
        self._k_lr_lado = k_lr if (self.redutor is None and self._lado is not None) else None
        guardados = []
        with reg.trecho("forward"):
            with reg.trecho("embedding"):
                x = ops.embed(p["emb"], tok)
            for l in range(self.L):
                with reg.trecho(f"camada {l}"):
                    with reg.trecho("atencao"):
                        n1, c1 = ops.rms(x)
                        qkv = ops.gemm(n1, p[f"Wqkv{l}"])
                        oc, P = ops.atencao(qkv, Bt, T, self.H)
                        om = ops.quant(oc)
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
        perda = (d_alvo.double() / 256 + torch.log(soma.double() / 4096)).mean()
        if not treina:
            return perda
        T_ = ops.transpoe
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
                        gq = ops.quant(ops.atencao_back(go, qkv, P, Bt, T, self.H))
                        self._grad_peso(f"Wqkv{l}", gq, n1)
                        gn = ops.gemm(gq, T_(p[f"Wqkv{l}"]))
                        gx = self._soma_rms_back(gx, gn, n1, c1)
                        self._st(f"c{l}.grad_qkv", gq); self._st(f"c{l}.grad_residuo", gx)
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
        return perda


class PassoGravado:
    """One training step recorded in a CUDA graph and replayed: the few hundred launches become one call.

    Recording executes nothing (weights do not change while recording).  Everything the step allocates lives in
    the graph's pool at fixed addresses; weights, momentum and residual are updated in place by the kernels, so
    the graph stays valid.  Inputs go to fixed buffers (copy_) before each replay.  The launch list of the
    recording is kept: the launch ids are baked into the kernel arguments, so a sentinel raised during a replay
    names the same operation and section as it would in eager mode.  Run one eager step before recording (the
    attention backward sizes its workspace on first use, which a capture does not allow).  Data parallel: the
    step is recorded as 1 + 2 GRUPOS graphs (forward+backward | per group of weights: deferred weight-gradient GEMMs
    | optimiser) and the collectives run eagerly between the replays: one MAX for the whole step, then one SUM per
    group, which overlaps the next group's GEMMs while the group's optimiser step follows on a second stream.
    """

    GRUPOS = 4          # data parallel: pieces the weight-gradient tail (GEMMs | SUM collective | optimiser) is pipelined in

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
                # Data parallel: three graphs with the two collectives issued eagerly between them, so that no
                # collective is ever part of a captured graph.  The reducer's flat buffers must already exist with
                # their final sizes (one eager step has run), so the graphs see fixed addresses.
                assert getattr(red, "_max", None) is not None and getattr(red, "_plano", None) is not None, \
                    "run one eager data-parallel step before recording"
                g0 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g0):
                    lib.jt_stream(torch.cuda.current_stream().cuda_stream)
                    self.perda = modelo.frente_tras(self.tok, self.alvo)
                    pares = [(ra, rb) for _, _, _, ra, rb in modelo._adiados]
                    red.empacota_maximos(pares)
                # The tail is cut into groups of consecutive weights: while group g's sums cross the wire, group
                # g+1's GEMMs run, and group g's optimiser step runs on a second stream as soon as its sums are in.
                # The GEMM graphs share graph 0's pool (replayed in recording order on one stream); the optimiser
                # graphs have a pool of their own (they run beside the GEMM graphs).
                n = len(pares)
                ng = min(self.GRUPOS, n)
                cortes = [n * g // ng for g in range(ng + 1)]
                maximos = red.vistas_maximos(pares)
                nomes = [a[0] for a in modelo._adiados]
                self._gemm, self._otim, self._fatias, vistas_g = [], [], [], []
                for g in range(ng):
                    gg = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gg, pool=g0.pool()):
                        lib.jt_stream(torch.cuda.current_stream().cuda_stream)
                        modelo._gemms_adiados(maximos, cortes[g], cortes[g + 1])
                        v, fatia = red.empacota_grupo({k: modelo._grads[k] for k in nomes[cortes[g]:cortes[g + 1]]}, modelo._grads)
                    self._gemm.append(gg)
                    self._fatias.append(fatia)
                    vistas_g.append(v)
                self._vivos = (vistas_g, dict(modelo._grads))        # keeps every tensor the graphs read at its address
                self._lado = torch.cuda.Stream(device=modelo.dev)
                pool_o = None
                for g in range(ng):
                    go = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(go, **({} if pool_o is None else {"pool": pool_o})):
                        lib.jt_stream(torch.cuda.current_stream().cuda_stream)
                        with self.reg.trecho("otimizador"):
                            modelo._otimiza(vistas_g[g], k_lr)
                    pool_o = go.pool()
                    self._otim.append(go)
                self.grafos = [g0] + self._gemm + self._otim
        finally:
            lib.jt_stream(None)
            modelo.estatisticas, self.reg.vigiar, self.reg.perfil = est, vig, perf
        self.lancamentos = list(self.reg.lancamentos)
        self.coletivos_por_passo = 0 if red is None else 1 + len(self._fatias)
        self.reg.info(f"step recorded in {len(self.grafos)} CUDA graph(s): {len(self.lancamentos)} launches", lancamentos=len(self.lancamentos))

    def __call__(self, tok, alvo):
        self.tok.copy_(tok)
        self.alvo.copy_(alvo)
        self.reg.lancamentos = self.lancamentos
        if len(self.grafos) == 1:
            self.grafos[0].replay()
        else:
            red = self.m.redutor
            principal = torch.cuda.current_stream()
            self.grafos[0].replay()
            red.reduz_maximos()
            for g, (gg, go, fatia) in enumerate(zip(self._gemm, self._otim, self._fatias)):
                gg.replay()
                pronto = red.reduz_fatia(*fatia)                  # asynchronous: ordered after this group's GEMMs
                if g == 0:
                    self._lado.wait_stream(principal)             # the optimiser may not overtake the backward's last read of a weight
                with torch.cuda.stream(self._lado):
                    pronto.wait()
                    go.replay()
            principal.wait_stream(self._lado)
        return self.perda
