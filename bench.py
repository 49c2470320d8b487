"""Benchmark of the integer training hot path on B200.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload gemm|passo]

Workloads (synthetic data with the shapes and value distributions the reference benchmarks use: mantissas uniform in
[-127,127], one exponent per 32-element K-block uniform in [-12,-4], seeded):
  passo  (default) one full training step of the 12-layer model (D=512, 8 heads, T=256, batch 8 = 2048 tokens per GPU),
         replayed from a CUDA graph; metric = tokens/s.
  gemm   block-32 INT8 GEMM trio of one linear layer at (M,K,N) = (16384,4096,4096):
         Y = X.W^T, dX = dY.T(W)^T, dW = T(dY).T(X)^T raw.  A step = the three GEMMs; metric = TOPS (2.M.N.K each).
  ops    the bandwidth-bound fused ops at 16384 tokens x D=1024: achieved HBM GB/s per op (single GPU).
With N > 1 (torchrun, one rank per GPU): gemm runs independent replicas (the path has no exchange step);
passo is data parallel with the bit-exact gradient reduction of jatai_b200.paralelo.

`--impl reference` times the CPU restatement of the reference specification (oracle/, all host threads) on a
bounded sample of the same workload; it is the only mode in which this file executes anything under oracle/
apart from the `cpu_baseline` leg of the default mode.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import torch

RAIZ = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, RAIZ)

FORMA = dict(M=16384, K=4096, N=4096)
BLK = 32


# ------------------------------------------------------------------------------------------------ helpers
def picos():
    """Roofline denominators: measured on this pool when the driver wrote them, else the stated fallback."""
    try:
        with open(os.path.join(RAIZ, "MEASURED_PEAKS.json")) as fh:
            p = json.load(fh)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sust=p.get("bf16_tflops_sustained"), origem="measured")
    except Exception:
        return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sust=1400.0, origem="fallback")


class Relogios:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    CAMPOS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, indice):
        self.linhas, self.p = [], None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={indice}", f"--query-gpu={self.CAMPOS}", "--format=csv,noheader,nounits",
                                       "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._le, daemon=True)
            self.t.start()
        except Exception:
            self.p = None

    def _le(self):
        for ln in self.p.stdout:
            self.linhas.append(ln.strip())

    def fim(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=2)
        except Exception:
            self.p.kill()
        sm, mx, razoes = [], None, set()
        nomes = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.linhas:
            c = [x.strip() for x in ln.split(",")]
            if len(c) < 6:
                continue
            try:
                sm.append(float(c[0]))
                mx = float(c[1])
            except ValueError:
                continue
            for n, v in zip(nomes, c[2:6]):
                if v.lower().startswith("active"):
                    razoes.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(razoes), "samples": len(sm)}


def gera_bloco(R, C, seed, dev, pinned=False):
    g = torch.Generator(device="cpu").manual_seed(seed)
    m = torch.randint(-127, 128, (R, C), generator=g, dtype=torch.int32).to(torch.int8)
    E = torch.randint(-12, -3, (R, C // BLK), generator=g).to(torch.int8)
    if pinned:
        return m.pin_memory(), E.pin_memory()
    return m.to(dev), E.to(dev)


def dist_info():
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    mundo = int(os.environ.get("WORLD_SIZE", "1"))
    return rank, local, mundo


def barreira(mundo):
    if mundo > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_ranks(ms, mundo, dev):
    if mundo == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


# ------------------------------------------------------------------------------------------------ CPU arm
def oracle_gemm_lib():
    so = os.path.join(RAIZ, "oracle", "liboracle_gemm.so")
    if not os.path.exists(so):
        subprocess.run(["make", "-C", os.path.join(RAIZ, "oracle")], check=True, capture_output=True)
    lib = ctypes.CDLL(so)
    lib.oracle_gemm.restype = ctypes.c_int
    lib.oracle_threads.restype = ctypes.c_int
    return lib


def cpu_gemm_amostra(linhas):
    """Times the C restatement of the GEMM specification on `linhas` rows of the forward GEMM.  Returns (TOPS, s, threads)."""
    lib = oracle_gemm_lib()
    K, N = FORMA["K"], FORMA["N"]
    X = gera_bloco(linhas, K, 11, "cpu")
    W = gera_bloco(N, K, 12, "cpu")
    Cm = torch.empty(linhas, N, dtype=torch.int8)
    CE = torch.empty(linhas, N // BLK, dtype=torch.int8)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    t0 = time.perf_counter()
    rc = lib.oracle_gemm(p(X[0]), p(X[1]), p(W[0]), p(W[1]), linhas, N, K, BLK, None, None, None, None, p(Cm), p(CE), 0, linhas)
    dt = time.perf_counter() - t0
    assert rc == 0
    return 2.0 * linhas * N * K / dt / 1e12, dt, lib.oracle_threads()


def braco_referencia(args):
    """`--impl reference`: the CPU restatement of the reference specification, all host threads, bounded sample."""
    rank, _, mundo = dist_info()
    if rank != 0:
        return
    linhas = 1024
    tempos = []
    for i in range(args.warmup + args.steps):
        tops, dt, th = cpu_gemm_amostra(linhas)
        if i >= args.warmup:
            tempos.append((tops, dt))
    tops = sum(t for t, _ in tempos) / len(tempos)
    ms = 1e3 * sum(d for _, d in tempos) / len(tempos)
    amostra = f"{linhas} of {FORMA['M']} rows of the forward GEMM (K={FORMA['K']}, N={FORMA['N']}) per step"
    print(json.dumps({
        "impl": "reference", "metric": "int8_b32_gemm_tops", "value": tops, "unit": "TOPS", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+int32",
        "data": "synthetic", "config": {"workload": "gemm_b32_16384x4096x4096", "sample": amostra},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": th, "kind": "port", "sample": amostra},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}))


# ------------------------------------------------------------------------------------------------ our arm
def braco_gemm(args):
    rank, local, mundo = dist_info()
    if mundo > 1:
        torch.cuda.set_device(local)
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local if mundo > 1 else 0)
    torch.cuda.set_device(dev)
    from jatai_b200 import ops, registro
    ops.define_blk(BLK)
    reg = registro.Registro(tempfile.mkdtemp(), f"bench{rank}", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    oc.lib.jt_stream(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if args.via is not None:
        assert oc.lib.jt_gemm_via(args.via) == 0
    M, K, N = FORMA["M"], FORMA["K"], FORMA["N"]
    reg.novo_passo(0)
    # operands of the three GEMMs, resident; 288 MB of mantissas per step > L2 (126 MB), so no flush is needed
    X, W, dY = gera_bloco(M, K, 1 + rank, dev), gera_bloco(N, K, 2, dev), gera_bloco(M, N, 3 + rank, dev)
    Wt, dYt, Xt = oc.transpoe(W), oc.transpoe(dY), oc.transpoe(X)
    torch.cuda.synchronize()
    ops_por_gemm = 2.0 * M * N * K
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def passo(tempos=None):
        reg.lancamentos = []
        a, b, c, d = ev(), ev(), ev(), ev()
        a.record()
        Y = oc.gemm(X, W)
        b.record()
        dX = oc.gemm(dY, Wt)
        c.record()
        dW = oc.gemm(dYt, Xt, cru=True)
        d.record()
        if tempos is not None:
            tempos.append((a, b, c, d))
        return Y, dX, dW

    for _ in range(max(args.warmup, 3)):
        passo()
    barreira(mundo)
    rel = Relogios(dev.index or 0)
    tempos = []
    ini, fim = ev(), ev()
    ini.record()
    for _ in range(args.steps):
        passo(tempos)
    fim.record()
    barreira(mundo)
    ms_total = max_ranks(ini.elapsed_time(fim), mundo, dev)
    clocks = rel.fim()
    ms_passo = ms_total / args.steps
    tops = mundo * 3 * ops_por_gemm / (ms_passo * 1e-3) / 1e12
    por_gemm = [sum(t[i].elapsed_time(t[i + 1]) for t in tempos) / len(tempos) for i in range(3)]
    n = reg.lib.jt_erro_le((ctypes.c_longlong * 6)())
    assert n == 0, f"device error record has {n} events"

    # end to end through the operator API with HOST buffers: H2D of the six operands, three GEMMs, D2H of the results
    Xh, Wh, dYh = gera_bloco(M, K, 1 + rank, dev, True), gera_bloco(N, K, 2, dev, True), gera_bloco(M, N, 3 + rank, dev, True)
    Yh = (torch.empty(M, N, dtype=torch.int8).pin_memory(), torch.empty(M, N // BLK, dtype=torch.int8).pin_memory())
    dXh = (torch.empty(M, K, dtype=torch.int8).pin_memory(), torch.empty(M, K // BLK, dtype=torch.int8).pin_memory())
    dWh = (torch.empty(N, K, dtype=torch.int32).pin_memory(), torch.empty(N, K, dtype=torch.int16).pin_memory())

    def passo_e2e():
        reg.lancamentos = []
        x = tuple(t.to(dev, non_blocking=True) for t in Xh)
        w = tuple(t.to(dev, non_blocking=True) for t in Wh)
        dy = tuple(t.to(dev, non_blocking=True) for t in dYh)
        wt, dyt, xt = oc.transpoe(w), oc.transpoe(dy), oc.transpoe(x)
        Y = oc.gemm(x, w)
        dX = oc.gemm(dy, wt)
        dW = oc.gemm(dyt, xt, cru=True)
        for h, d in ((Yh, Y), (dXh, dX), (dWh, dW)):
            h[0].copy_(d[0], non_blocking=True)
            h[1].copy_(d[1], non_blocking=True)

    h2d = sum(t.numel() * t.element_size() for par in (Xh, Wh, dYh) for t in par)
    d2h = sum(t.numel() * t.element_size() for par in (Yh, dXh, dWh) for t in par)
    for _ in range(2):
        passo_e2e()
    barreira(mundo)
    e_steps = max(2, min(args.steps, 5))
    ini.record()
    for _ in range(e_steps):
        passo_e2e()
    fim.record()
    barreira(mundo)
    ms_e2e = max_ranks(ini.elapsed_time(fim), mundo, dev) / e_steps
    tops_e2e = mundo * 3 * ops_por_gemm / (ms_e2e * 1e-3) / 1e12

    if mundo > 1:
        torch.distributed.destroy_process_group()
    if rank != 0:
        return
    pk = picos()
    pico_i8 = 2.0 * pk["bf16"]
    ach = ops_por_gemm / (por_gemm[0] * 1e-3) / 1e12
    saida = {
        "metric": "int8_b32_gemm_tops", "value": tops, "unit": "TOPS", "n_gpus": mundo, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_passo, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+int32",
        "data": "synthetic",
        "config": {"workload": f"gemm_b32_{M}x{K}x{N}", "shape_MKN": [M, K, N], "block": BLK, "gemms_per_step": ["Y=X.W^T", "dX=dY.W", "dW=dY^T.X raw"],
                   "l2": "inputs larger than L2 (288 MB of operands per step)", "parallelism": f"replicas x{mundo}",
                   "via": args.via if args.via is not None else 0},
        "ms_per_gemm": {"fwd": por_gemm[0], "dX": por_gemm[1], "dW_raw": por_gemm[2]},
        "roofline": {"bound": "tensor", "achieved": ach, "peak": pico_i8, "unit": "TOPS", "frac": ach / pico_i8, "traffic": None,
                     "kernel": "k_gemm_tc<32,0> forward GEMM", "peak_source": f"2 x cuBLAS bf16 burst ({pk['origem']}): kind::i8 issues at twice the bf16 rate",
                     "alu_bound_note": "every 32-wide K slice is drained from tensor memory and rounded on the CUDA cores: M*N*K/32 element-steps"},
        "clocks": clocks,
        "e2e": {"value": tops_e2e, "unit": "TOPS", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e,
                "includes": "H2D of X, W, dY from pinned memory, 3 transposes, 3 GEMMs, D2H of Y, dX, dW"},
        "gpu_launches": 3 * args.steps,
    }
    if mundo == 1 and not args.sem_cpu:
        try:
            ctops, dt, th = cpu_gemm_amostra(2048)
            saida["cpu_baseline"] = {"value": ctops, "unit": "TOPS", "cores": th, "kind": "port",
                                     "sample": f"2048 of {M} rows of the forward GEMM, C restatement of the int64 spec, {dt:.1f} s"}
        except Exception as e:      # the baseline is a reported extra; the GPU numbers stand without it
            saida["cpu_baseline"] = {"value": None, "unit": "TOPS", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    print(json.dumps(saida))


# ------------------------------------------------------------------------------------------------ training step
TRAFEGO_GEMMS_PASSO = 601.5e6        # bytes per step, measured with ncu on this workload (see roofline.traffic_note)
PASSO = dict(V=256, D=512, H=8, FF=2048, L=12, Bt=8, T=256, k_lr=4)      # benchmark configuration 4 of the reference


def lote_tokens(seed, Bt, T, V):
    """Uniform random byte tokens; inputs and targets shifted by one (the reference's batch recipe, treino.py:41-44)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, V, (Bt, T + 1), generator=g)
    return x[:, :-1].contiguous(), x[:, 1:].contiguous()


def cpu_passo_amostra(L_am=2, Bt_am=2):
    """Times the int64 restatement of the specification on a reduced model (same D, heads, T, FF; fewer layers and
    sequences), scaled to the full step by layer and sequence count.  Returns (tokens/s scaled, seconds, threads, text)."""
    from jatai_b200 import modelo, ops, registro
    from oracle import spec
    c = PASSO
    antes = ops.BLK
    ops.BLK = BLK
    try:
        reg = registro.Registro(tempfile.mkdtemp(), "cpu", eco=False)
        m = modelo.Modelo(c["V"], c["D"], c["H"], c["FF"], L_am, 0, "cpu", spec.Spec(BLK), reg)
        tok, alvo = lote_tokens(1, Bt_am, c["T"], c["V"])
        t0 = time.perf_counter()
        m.passo(tok, alvo, k_lr=c["k_lr"])
        dt = time.perf_counter() - t0
    finally:
        ops.BLK = antes
    # per-layer work dominates; embedding/logits (1 of ~13 layer-equivalents) are counted with the layers
    escala = (c["L"] / L_am)
    tps = Bt_am * c["T"] / (dt * escala)
    return tps, dt, torch.get_num_threads(), (f"{L_am} of {c['L']} layers, {Bt_am} of {c['Bt']} sequences of T={c['T']}, int64 torch restatement "
                                              f"of the spec, {dt:.1f} s; tokens/s scaled by the layer count")


def braco_referencia_passo(args):
    rank, _, _ = dist_info()
    if rank != 0:
        return
    vals = []
    for i in range(min(args.warmup, 1) + min(args.steps, 3)):
        tps, dt, th, txt = cpu_passo_amostra()
        if i >= min(args.warmup, 1):
            vals.append((tps, dt))
    tps = sum(v for v, _ in vals) / len(vals)
    c = PASSO
    print(json.dumps({
        "impl": "reference", "metric": "train_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(vals),
        "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * sum(d for _, d in vals) / len(vals), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8+int32", "data": "synthetic",
        "config": {"workload": f"passo_{c['L']}L_D{c['D']}_H{c['H']}_T{c['T']}_Bt{c['Bt']}_b{BLK}", "sample": txt},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": th, "kind": "port", "sample": txt},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}))


def resumo_perfil(reg, pk):
    """Per-operation GPU time of one eager step (CUDA events around every launch) and the roofline of the GEMMs."""
    tempos, ops_gemm, ms_gemm = {}, 0.0, 0.0
    for (op, ini, fim), lanc in zip(reg.eventos, reg.lancamentos):
        ms = ini.elapsed_time(fim)
        tempos[op] = tempos.get(op, 0.0) + ms
        if op.startswith("gemm"):
            a, b = lanc["entradas"]["A"], lanc["entradas"]["B"]
            ops_gemm += 2.0 * a.shape[0] * a.shape[1] * b.shape[0]
            ms_gemm += ms
    total = sum(tempos.values())
    ordem = sorted(tempos.items(), key=lambda kv: -kv[1])
    return {"ms_per_op": {k: round(v, 4) for k, v in ordem}, "ms_total": total, "gemm_ops": ops_gemm, "gemm_ms": ms_gemm}


def tempo_gemms(oc, reg):
    """GPU time of all block GEMMs of the step just run, back to back: the recorded launches are issued again, with
    their own operands, into one CUDA graph (no host gaps between them) and the graph is timed with CUDA events."""
    chamadas = []
    for lanc in reg.lancamentos:
        if not lanc["op"].startswith("gemm"):
            continue
        e = lanc["entradas"]
        chamadas.append((lanc["op"], (e["A"], e["EA"]), (e["B"], e["EB"]), (e["X"], e["XE"]) if "X" in e else None))

    def roda():
        for op, A, B, X in chamadas:
            if op == "gemm":
                oc.gemm(A, B)
            elif op == "gemm_cru":
                oc.gemm(A, B, cru=True)
            elif op == "gemm_soma":
                oc.gemm_soma(A, B, X)
            elif op == "gemm_relu2":
                oc.gemm_relu2(A, B)
            else:
                oc.gemm_relu2_back(A, B, X)
        reg.lancamentos = []

    roda()
    torch.cuda.synchronize()
    st, gr = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    ini, fim = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(st):
        try:
            with torch.cuda.graph(gr, stream=st):
                oc.lib.jt_stream(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                roda()
        finally:
            oc.lib.jt_stream(None)
        gr.replay()
        reps = 3
        ini.record()
        for _ in range(reps):
            gr.replay()
        fim.record()
    torch.cuda.synchronize()
    return ini.elapsed_time(fim) / reps, len(chamadas)


def braco_passo(args):
    rank, local, mundo = dist_info()
    if mundo > 1:
        torch.cuda.set_device(local)
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local if mundo > 1 else 0)
    torch.cuda.set_device(dev)
    from jatai_b200 import modelo, ops, paralelo, registro
    ops.define_blk(BLK)
    c = PASSO
    reg = registro.Registro(tempfile.mkdtemp(), f"passo{rank}", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    if args.via is not None:
        assert oc.lib.jt_gemm_via(args.via) == 0
    red = paralelo.Redutor() if mundo > 1 else None
    m = modelo.Modelo(c["V"], c["D"], c["H"], c["FF"], c["L"], 0, dev, oc, reg, redutor=red)
    Bt, T = c["Bt"], c["T"]
    lotes = [tuple(t.to(dev) for t in lote_tokens(100 * rank + i, Bt, T, c["V"])) for i in range(8)]
    # one eager step with per-launch events: sizes the attention workspace, gives the per-op breakdown
    reg.novo_passo(0)
    m.passo(*lotes[0], k_lr=c["k_lr"])                # first step pays the one-time costs (workspace, kernel attributes)
    reg.fim_passo()
    reg.perfil = True
    reg.novo_passo(1)
    m.passo(*lotes[1], k_lr=c["k_lr"])
    reg.fim_passo()
    perfil = resumo_perfil(reg, picos())
    lancamentos = len(reg.lancamentos)
    reg.perfil = False
    reg.tempos = {}
    gemm_ms, n_gemms = tempo_gemms(oc, reg)
    passo_fn = None
    modo = "eager"
    if not args.eager:
        try:
            gravado = modelo.PassoGravado(m, Bt, T, c["k_lr"])
            passo_fn, modo = gravado, "cuda_graph"
        except Exception as e:          # capture refused (e.g. a collective that can not be captured): run eagerly, say so
            modo = f"eager (graph capture failed: {type(e).__name__})"
    if passo_fn is None:
        def passo_fn(tok, alvo):
            reg.lancamentos = []
            return m.passo(tok, alvo, k_lr=c["k_lr"])
    ev = lambda: torch.cuda.Event(enable_timing=True)
    W = max(args.warmup, 3)
    for i in range(W):
        passo_fn(*lotes[i % 8])
    barreira(mundo)
    rel = Relogios(dev.index or 0)
    ini, fim = ev(), ev()
    ini.record()
    for i in range(args.steps):
        perda = passo_fn(*lotes[i % 8])
    fim.record()
    barreira(mundo)
    ms = max_ranks(ini.elapsed_time(fim), mundo, dev) / args.steps
    clocks = rel.fim()
    n_err = reg.lib.jt_erro_le((ctypes.c_longlong * 6)())
    assert n_err == 0, f"device error record has {n_err} events"
    tps = mundo * Bt * T / (ms * 1e-3)
    # end to end: tokens come from pinned host memory every step and the loss is read back every step
    hospedeiro = [tuple(t.pin_memory() for t in lote_tokens(100 * rank + i, Bt, T, c["V"])) for i in range(8)]
    perdas = []

    def passo_e2e(i):
        tok, alvo = hospedeiro[i % 8]
        p = passo_fn(tok.to(dev, non_blocking=True), alvo.to(dev, non_blocking=True))
        perdas.append(float(p))                      # device -> host read of the step's result (synchronises)

    for i in range(2):
        passo_e2e(i)
    barreira(mundo)
    ini.record()
    for i in range(args.steps):
        passo_e2e(i)
    fim.record()
    barreira(mundo)
    ms_e2e = max_ranks(ini.elapsed_time(fim), mundo, dev) / args.steps
    perda_f = float(perda)
    if mundo > 1:
        torch.distributed.destroy_process_group()
    if rank != 0:
        return
    pk = picos()
    pico_i8 = 2.0 * pk["bf16_sust"] if pk.get("bf16_sust") else 2.0 * pk["bf16"]
    ach = perfil["gemm_ops"] / (gemm_ms * 1e-3) / 1e12 if gemm_ms else None
    saida = {
        "metric": "train_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": mundo, "steps": args.steps, "warmup": W,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+int32", "data": "synthetic",
        "config": {"workload": f"passo_{c['L']}L_D{c['D']}_H{c['H']}_T{c['T']}_Bt{c['Bt']}_b{BLK}", "tokens_per_gpu_step": Bt * T,
                   "global_tokens_per_step": mundo * Bt * T, "block": BLK, "mode": modo, "parallelism": f"dp{mundo}",
                   "l2": "weights + momentum + residual + activations of a step exceed L2 (about 0.6 GB touched per step)",
                   "init": "seeded random weights (reference recipe), uniform random byte tokens"},
        "loss_last": perda_f, "launches_per_step": lancamentos,
        "roofline": {"bound": "tensor", "achieved": ach, "peak": pico_i8, "unit": "TOPS", "frac": (ach / pico_i8) if ach else None,
                     "traffic": TRAFEGO_GEMMS_PASSO if (mundo == 1 and args.via is None and BLK == 32) else None,
                     "traffic_note": "DRAM bytes read + written by the step's 148 GEMM launches, one ncu pass (cold L2 per launch; the outputs stay in L2): profiles/k_gemm_tc_b32.md",
                     "kernel": f"all {n_gemms} block GEMMs of one step (k_gemm_tc), issued back to back from one CUDA graph with the step's own operands",
                     "peak_source": f"2 x cuBLAS bf16 sustained ({pk['origem']})", "gemm_ms_per_step": gemm_ms},
        "ms_per_op_eager": perfil["ms_per_op"], "clocks": clocks,
        "e2e": {"value": mundo * Bt * T / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * Bt * T * 8, "d2h_bytes_per_step": 8,
                "ms_per_step": ms_e2e, "includes": "tokens and targets from pinned host memory, the step, loss read back to the host every step"},
        "gpu_launches": lancamentos * args.steps,
    }
    if red is not None:
        saida["wire"] = {"collectives_per_step": 1 + (len(passo_fn._fatias) if modo == "cuda_graph" else 1), "max_bytes_per_step": int(red._max.numel()), "sum_bytes_per_step": int(red._plano.numel()) * 4}
    if mundo == 1 and not args.sem_cpu:
        try:
            ctps, dt, th, txt = cpu_passo_amostra()
            saida["cpu_baseline"] = {"value": ctps, "unit": "tokens/s", "cores": th, "kind": "port", "sample": txt}
        except Exception as e:
            saida["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    print(json.dumps(saida))


# ------------------------------------------------------------------------------------------------ fused op suite
def braco_ops(args):
    """Benchmark configuration 3: the bandwidth-bound ops at 16384 tokens x D=1024 (block 32); achieved HBM GB/s per op from
    the algorithmic bytes (inputs read once + outputs written once).  Inputs rotate over enough copies to exceed L2."""
    rank, local, mundo = dist_info()
    dev = torch.device("cuda", local if mundo > 1 else 0)
    torch.cuda.set_device(dev)
    from jatai_b200 import ops, registro
    ops.define_blk(BLK)
    reg = registro.Registro(tempfile.mkdtemp(), f"ops{rank}", eco=False, salvar=False)
    oc = ops.OpsCuda(reg)
    reg.novo_passo(0)
    M, D, FF, V, NW = 16384, 1024, 4096, 256, 12 * 1024 * 1024
    g = torch.Generator().manual_seed(7)

    def bloco(R, C, e0=-10, esp=4):
        m = torch.randint(-127, 128, (R, C), generator=g, dtype=torch.int32).to(torch.int8).to(dev)
        E = (e0 + torch.randint(-esp, esp + 1, (R, C // BLK), generator=g)).to(torch.int8).to(dev)
        return m, E

    def cru(R, C, bits=24, e0=-30):
        a = torch.randint(-(1 << bits), 1 << bits, (R, C), generator=g, dtype=torch.int32).to(dev)
        e = (e0 + torch.randint(-3, 4, (R, C), generator=g)).to(torch.int16).to(dev)
        return a, e

    b1 = 1 + 1.0 / BLK                       # bytes per element of a block tensor
    casos_ = []                               # (name, bytes, [callable per buffer copy])

    def copias(f, n):
        return [f() for _ in range(n)]

    x = copias(lambda: bloco(M, D), 6)
    casos_.append(("rms", M * (2 * D * b1 + 8), [lambda t=t: oc.rms(t) for t in x]))
    ys = [oc.rms(t) for t in x]
    gs = copias(lambda: bloco(M, D, e0=-20), 6)
    casos_.append(("rms_back", M * (3 * D * b1 + 8), [lambda a=a, y=y: oc.rms_back(a, y[0], y[1]) for a, y in zip(gs, ys)]))
    casos_.append(("soma", 3 * M * D * b1, [lambda a=a, b=b: oc.soma(a, b) for a, b in zip(x, gs)]))
    h = copias(lambda: bloco(M, FF), 3)
    h2 = copias(lambda: bloco(M, FF), 3)
    casos_.append(("relu2", 2 * M * FF * b1, [lambda t=t: oc.relu2(t) for t in h]))
    casos_.append(("relu2_back", 3 * M * FF * b1, [lambda a=a, b=b: oc.relu2_back(a, b) for a, b in zip(h, h2)]))
    casos_.append(("transpoe", 2 * M * FF * b1, [lambda t=t: oc.transpoe(t) for t in h]))
    c = copias(lambda: cru(M, D), 3)
    casos_.append(("quant", M * D * (6 + b1), [lambda t=t: oc.quant(t) for t in c]))
    lg = copias(lambda: cru(M, V, bits=22, e0=-20), 12)
    alvo = torch.randint(0, V, (M,), generator=g).to(torch.int32).to(dev)
    casos_.append(("softmax_ce", M * (V * 6 + 4 + V * b1 + 8), [lambda t=t: oc.softmax_ce(t, alvo) for t in lg]))
    gw = copias(lambda: cru(3072, 4096, bits=26, e0=-45), 3)
    mom = copias(lambda: bloco(3072, 4096, e0=-40), 3)
    w = copias(lambda: bloco(3072, 4096, e0=-9), 3)
    res = copias(lambda: bloco(3072, 4096, e0=-20), 3)
    casos_.append(("momento", NW * (6 + 2 * b1), [lambda a=a, b=b: oc.momento(a, b) for a, b in zip(gw, mom)]))
    casos_.append(("peso", NW * 5 * b1, [lambda a=a, b=b, r=r: oc.peso(a, b, r, 4, True) for a, b, r in zip(w, mom, res)]))
    Bt, T, H = 16, 1024, 16
    qkv = copias(lambda: bloco(M, 3 * D, esp=3), 2)
    casos_.append(("atencao (16 seq x 16 heads x T=1024, hd 64)", M * 3 * D * b1 + M * D * 6 + Bt * H * T * T,
                   [lambda t=t: oc.atencao(t, Bt, T, H) for t in qkv]))
    pk = picos()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    tabela, tot_b, tot_ms = {}, 0.0, 0.0
    reps = max(args.steps, 5)
    corrente = torch.cuda.Stream()
    for nome, nbytes, fs in casos_:
        for i in range(max(args.warmup, 3)):
            reg.lancamentos = []
            fs[i % len(fs)]()
        torch.cuda.synchronize()
        # the calls are recorded in a CUDA graph and the replay is timed: kernels of 10-100 us would otherwise be
        # timed at the rate the Python launcher can enqueue them
        grafo = torch.cuda.CUDAGraph()
        with torch.cuda.stream(corrente):
            with torch.cuda.graph(grafo, stream=corrente):
                oc.lib.jt_stream(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                saidas = []
                for i in range(reps):
                    reg.lancamentos = []
                    saidas.append(fs[i % len(fs)]())
            oc.lib.jt_stream(None)
            grafo.replay()
            torch.cuda.synchronize()
            a, b = ev(), ev()
            a.record()
            grafo.replay()
            b.record()
        torch.cuda.synchronize()
        del saidas, grafo
        ms = a.elapsed_time(b) / reps
        gbs = nbytes / (ms * 1e-3) / 1e9
        tabela[nome] = {"ms": round(ms, 4), "MB": round(nbytes / 1e6, 1), "GB/s": round(gbs, 1), "frac_of_measured_hbm": round(gbs / pk["hbm_gbs"], 3)}
        tot_b += nbytes
        tot_ms += ms
    n = reg.lib.jt_erro_le((ctypes.c_longlong * 6)())
    assert n == 0, f"device error record has {n} events"
    if rank != 0:
        return
    agg = tot_b / (tot_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "fused_ops_hbm_gbs", "value": agg, "unit": "GB/s", "n_gpus": 1, "steps": reps, "warmup": max(args.warmup, 3), "ms_per_step": tot_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+int32", "data": "synthetic",
        "config": {"workload": "ops_16384tok_D1024_b32", "l2": "inputs rotate over copies totalling more than L2 (126 MB)",
                   "timing": "each op recorded `steps` times in a CUDA graph over rotating inputs; the replay is timed with CUDA events"},
        "per_op": tabela,
        "roofline": {"bound": "hbm", "achieved": agg, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": agg / pk["hbm_gbs"], "traffic": None,
                     "peak_source": f"STREAM-style copy ({pk['origem']})"},
        "gpu_launches": reps * len(casos_)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="passo", choices=["gemm", "passo", "ops"])
    ap.add_argument("--via", type=int, default=None, help="force a GEMM path (jt_gemm_via)")
    ap.add_argument("--eager", action="store_true", help="passo: no CUDA graph")
    ap.add_argument("--forma", type=int, nargs=3, default=None, metavar=("M", "K", "N"), help="gemm: another shape (profiling captures)")
    ap.add_argument("--sem-cpu", dest="sem_cpu", action="store_true", help="skip the cpu_baseline leg")
    args = ap.parse_args()
    if args.forma:
        FORMA.update(M=args.forma[0], K=args.forma[1], N=args.forma[2])
    if args.impl == "reference":
        return braco_referencia_passo(args) if args.workload == "passo" else braco_referencia(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    if args.workload == "passo":
        return braco_passo(args)
    if args.workload == "ops":
        return braco_ops(args)
    return braco_gemm(args)


if __name__ == "__main__":
    main()
