"""Benchmark of the integer training hot path on B200.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload passo|gemm|ops] [--config c4|c5|compat]

Synthetic data with the shapes and value distributions the reference benchmarks use (mantissas uniform in [-127,127],
one exponent per 32-element block uniform in [-12,-4], seeded; uniform random byte tokens) stands in for the corpus.

Workloads:
  passo  (default) one full training step replayed from a CUDA graph; metric = tokens/s.  The headline configuration is
         c4 = 12 layers, D=512, 8 heads, T=256, batch 8 = 2048 tokens per GPU (benchmark configuration 4).  The line also
         carries, under "extra", short timed legs of the other benchmark configurations:
           config5  24 layers, D=1024, 16 heads, T=1024, 16 sequences = 16384 tokens per GPU (data parallel when N > 1)
           config2  block-32 GEMM sweep (N = 1 only): three shapes x {Y, dX, dW raw}, GEMM alone and GEMM + its transposes
           config3  the bandwidth-bound fused ops at 16384 tokens x D=1024 (N = 1 only): achieved HBM GB/s per op
           compat   the reference's own model size (D=256, 64 heads of 4, T=128, block 128; N = 1 only)
         `--config c5` / `--config compat` make that configuration the headline instead; `--sem-extras` drops the legs.
  gemm   the GEMM trio of one linear layer at (M,K,N) = (16384,4096,4096); metric = TOPS (2.M.N.K each).
  ops    configuration 3 alone.
With N > 1 (torchrun, one rank per GPU) passo is data parallel with the bit-exact gradient reduction of
jatai_b200.paralelo (weak scaling); after the timed region the ranks compare a SHA-256 of weights, momentum and residual.

`--impl reference` times the CPU restatement of the reference specification (oracle/, all host threads) on a bounded
sample of the same workload and, when the reference's own CUDA library was compiled (oracle/_ref), that library on the
GPU in the one configuration it supports (compat).  Apart from the `cpu_baseline` leg of the default mode this is the
only mode in which this file executes anything under oracle/.
"""
import argparse
import ctypes
import hashlib
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
CONFIGS = {
    # benchmark configuration 4: the headline
    "c4": dict(V=256, D=512, H=8, FF=2048, L=12, Bt=8, T=256, k_lr=4, blk=32),
    # benchmark configuration 5: 16384 tokens per GPU
    "c5": dict(V=256, D=1024, H=16, FF=4096, L=24, Bt=16, T=1024, k_lr=4, blk=32),
    # the reference library's own size (jatai_cuda/treino_cuda.py:31-33), 2048 tokens per step, block 128
    "compat": dict(V=256, D=256, H=64, FF=1024, L=12, Bt=16, T=128, k_lr=4, blk=128),
}
SWEEP = [(16384, 4096, 4096), (16384, 4096, 16384), (16384, 16384, 4096)]        # benchmark configuration 2
# DRAM bytes read + written per launch of the tensor-core GEMM, from one ncu capture (1 launch, --clock-control none,
# cold L2) of the 4096 x 4096 x 4096 block GEMM; other shapes scale by their algorithmic bytes (traffic grows with them)
TRAFEGO_NCU = dict(bytes=35.2e6, forma=(4096, 4096, 4096), fonte="ncu dram__bytes_read.sum + dram__bytes_write.sum, k_gemm_tc 4096x4096x4096, 1 launch")


# ------------------------------------------------------------------------------------------------ helpers
def picos():
    """Roofline denominators: measured on this pool when the driver wrote them, else the stated fallback."""
    try:
        with open(os.path.join(RAIZ, "MEASURED_PEAKS.json")) as fh:
            p = json.load(fh)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sust=p.get("bf16_tflops_sustained") or p["bf16_tflops"], origem="measured")
    except Exception:
        return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sust=1400.0, origem="fallback")


def nome_passo(c):
    return f"passo_{c['L']}L_D{c['D']}_H{c['H']}_T{c['T']}_Bt{c['Bt']}_b{c['blk']}"


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


def gera_bloco(R, C, seed, dev, pinned=False, blk=BLK):
    g = torch.Generator(device="cpu").manual_seed(seed)
    m = torch.randint(-127, 128, (R, C), generator=g, dtype=torch.int32).to(torch.int8)
    E = torch.randint(-12, -3, (R, C // blk), generator=g).to(torch.int8)
    if pinned:
        return m.pin_memory(), E.pin_memory()
    return m.to(dev), E.to(dev)


def dist_info():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


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


def ev():
    return torch.cuda.Event(enable_timing=True)


def inicia_gpu():
    rank, local, mundo = dist_info()
    if mundo > 1:
        torch.cuda.set_device(local)
        if not torch.distributed.is_initialized():
            torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local if mundo > 1 else 0)
    torch.cuda.set_device(dev)
    return rank, mundo, dev


def lanca_ops(blk, rotulo, biblioteca=None):
    from jatai_b200 import ops, registro
    ops.define_blk(blk)
    reg = registro.Registro(tempfile.mkdtemp(), rotulo, eco=False, salvar=False)
    oc = ops.OpsCuda(reg, biblioteca=biblioteca)
    reg.novo_passo(0)
    return ops, oc, reg


def sem_erros(reg, onde):
    n = reg.lib.jt_erro_le((ctypes.c_longlong * 6)())
    assert n == 0, f"{onde}: device error record has {n} events"


def n_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ------------------------------------------------------------------------------------------------ CPU legs (the oracle, timed)
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


def braco_referencia_gemm(args):
    """`--impl reference --workload gemm`: the C restatement of the GEMM specification, all host threads, bounded sample."""
    rank, _, _ = dist_info()
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


def lote_tokens(seed, Bt, T, V):
    """Uniform random byte tokens; inputs and targets shifted by one (the reference's batch recipe, treino.py:41-44)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, V, (Bt, T + 1), generator=g)
    return x[:, :-1].contiguous(), x[:, 1:].contiguous()


def cpu_passo_amostra(c, Bt_am=2):
    """Times the int64 restatement of the specification on reduced models (same D, heads, T, FF; 1 and 2 layers, Bt_am
    sequences) with every host thread.  The difference of the two timings is the cost of one layer, the rest is the part
    that does not grow with depth (embedding, logits, loss, their gradients and updates); the full step is estimated as
    rest + L x layer, for Bt_am sequences.  Returns (tokens/s, seconds spent, threads, description)."""
    from jatai_b200 import modelo, ops, registro
    from oracle import spec
    th = n_threads()
    torch.set_num_threads(th)
    antes = ops.BLK
    ops.BLK = c["blk"]
    tempos = {}
    try:
        tok, alvo = lote_tokens(1, Bt_am, c["T"], c["V"])
        for L_am in (1, 2):
            reg = registro.Registro(tempfile.mkdtemp(), "cpu", eco=False)
            m = modelo.Modelo(c["V"], c["D"], c["H"], c["FF"], L_am, 0, "cpu", spec.Spec(c["blk"]), reg)
            t0 = time.perf_counter()
            m.passo(tok, alvo, k_lr=c["k_lr"])
            tempos[L_am] = time.perf_counter() - t0
    finally:
        ops.BLK = antes
    camada = max(tempos[2] - tempos[1], 1e-9)
    resto = max(tempos[1] - camada, 0.0)
    total = resto + c["L"] * camada
    tps = Bt_am * c["T"] / total
    txt = (f"int64 torch restatement of the spec on {th} threads: {Bt_am} of {c['Bt']} sequences of T={c['T']}, models of 1 and 2 layers "
           f"({tempos[1]:.1f} s, {tempos[2]:.1f} s) -> layer {camada:.2f} s, depth-independent part {resto:.2f} s, step = rest + {c['L']} x layer; "
           f"same_config: false (sampled sequences and layers)")
    return tps, tempos[1] + tempos[2], th, txt


def gpu_compat_referencia(steps):
    """The reference's own CUDA library (dp4a kernels, compiled for sm_100a into oracle/_ref by the oracle's recipe) on the one
    configuration it supports, through the same launcher and model code: tokens/s of the graph-replayed step, or None."""
    so = os.path.join(RAIZ, "oracle", "_ref", "libjatai_ref.so")
    if not (os.path.exists(so) and torch.cuda.is_available()):
        return None
    torch.cuda.set_device(0)
    r = mede_passo(CONFIGS["compat"], 0, 1, torch.device("cuda", 0), steps=max(steps, 5), warmup=3, biblioteca=so, perfil=False, e2e=False)
    return {"tokens_per_s": r["tps"], "ms_per_step": r["ms"], "launches_per_step": r["lancamentos"], "library": "oracle/_ref/libjatai_ref.so (reference jatai_cuda.cu, sm_100a)",
            "config": nome_passo(CONFIGS["compat"])}


def braco_referencia_passo(args):
    rank, _, _ = dist_info()
    if rank != 0:
        return
    c = CONFIGS[args.config]
    vals = []
    w = min(args.warmup, 1)
    for i in range(w + min(args.steps, 2)):
        tps, dt, th, txt = cpu_passo_amostra(c)
        if i >= w:
            vals.append((tps, dt))
    tps = sum(v for v, _ in vals) / len(vals)
    saida = {
        "impl": "reference", "metric": "train_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(vals),
        "warmup": w, "ms_per_step": 1e3 * c["Bt"] * c["T"] / tps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8+int32", "data": "synthetic", "same_config": False,
        "config": {"workload": nome_passo(c), "sample": txt},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": th, "kind": "port", "sample": txt},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    try:
        comp = gpu_compat_referencia(args.steps)
        if comp is not None:
            saida["extra"] = {"compat_reference_kernels": comp}
    except Exception as e:
        saida["extra"] = {"compat_reference_kernels": {"failed": f"{type(e).__name__}: {e}"}}
    print(json.dumps(saida))


# ------------------------------------------------------------------------------------------------ GEMM workload
def bytes_gemm(M, K, N, blk, cru):
    """Algorithmic bytes of one block GEMM: operands and exponents in, output out."""
    b1 = 1 + 1.0 / blk
    return (M * K + N * K) * b1 + M * N * (6 if cru else b1)


def braco_gemm(args):
    rank, mundo, dev = inicia_gpu()
    ops, oc, reg = lanca_ops(BLK, f"bench{rank}")
    oc.lib.jt_stream(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if args.via is not None:
        assert oc.lib.jt_gemm_via(args.via) == 0
    M, K, N = FORMA["M"], FORMA["K"], FORMA["N"]
    # operands of the three GEMMs, resident; 288 MB of mantissas per step > L2 (126 MB), so no flush is needed
    X, W, dY = gera_bloco(M, K, 1 + rank, dev), gera_bloco(N, K, 2, dev), gera_bloco(M, N, 3 + rank, dev)
    Wt, dYt, Xt = oc.transpoe(W), oc.transpoe(dY), oc.transpoe(X)
    torch.cuda.synchronize()
    ops_por_gemm = 2.0 * M * N * K

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
    sem_erros(reg, "gemm")

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
    alg = bytes_gemm(M, K, N, BLK, False)
    saida = {
        "metric": "int8_b32_gemm_tops", "value": tops, "unit": "TOPS", "n_gpus": mundo, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_passo, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+int32",
        "data": "synthetic",
        "config": {"workload": f"gemm_b32_{M}x{K}x{N}", "shape_MKN": [M, K, N], "block": BLK, "gemms_per_step": ["Y=X.W^T", "dX=dY.W", "dW=dY^T.X raw"],
                   "l2": "inputs larger than L2 (288 MB of operands per step)", "parallelism": f"replicas x{mundo}",
                   "via": args.via if args.via is not None else 0},
        "ms_per_gemm": {"fwd": por_gemm[0], "dX": por_gemm[1], "dW_raw": por_gemm[2]},
        "roofline": {"bound": "tensor", "achieved": ach, "peak": pico_i8, "unit": "TOPS", "frac": ach / pico_i8,
                     "frac_of_2x_bf16_sustained": ach / (2.0 * pk["bf16_sust"]),
                     "traffic": TRAFEGO_NCU["bytes"] * alg / bytes_gemm(*TRAFEGO_NCU["forma"], BLK, False), "traffic_source": TRAFEGO_NCU["fonte"] + ", scaled by algorithmic bytes",
                     "algorithmic_bytes": alg,
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


def mede_sweep(oc, reg, dev, reps=3):
    """Benchmark configuration 2: for each (M,K,N) the three GEMMs of a linear layer in the C[rows,cols] = A[rows,red] . B[cols,red]^T
    convention - Y[M,N] (red K), dX[M,K] (red N, B = T(W)), dW raw [N,K] (red M, A = T(dY), B = T(X)) - timed alone and with the
    transpositions they need (the method of the reference's bench_formas.py:56).  2.M.N.K operations each."""
    pk = picos()
    pico = 2.0 * pk["bf16"]
    saida = {}

    def cronometra(f):
        f()
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for _ in range(reps):
            reg.lancamentos = []
            f()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    for (M, K, N) in SWEEP:
        X, W, dY = gera_bloco(M, K, 21, dev), gera_bloco(N, K, 22, dev), gera_bloco(M, N, 23, dev)
        Wt = oc.transpoe(W)
        dYt, Xt = oc.transpoe2(dY, X)
        ops_ = 2.0 * M * N * K
        linhas = {}
        for nome, so, com in (("Y", lambda: oc.gemm(X, W), None),
                              ("dX", lambda: oc.gemm(dY, Wt), lambda: oc.gemm(dY, oc.transpoe(W))),
                              ("dW_raw", lambda: oc.gemm(dYt, Xt, cru=True), lambda: oc.gemm(*oc.transpoe2(dY, X), cru=True))):
            ms = cronometra(so)
            tops = ops_ / (ms * 1e-3) / 1e12
            linhas[nome] = {"ms": round(ms, 4), "TOPS": round(tops, 1), "frac_of_2x_bf16_burst": round(tops / pico, 4)}
            if com is not None:
                ms2 = cronometra(com)
                linhas[nome].update({"ms_with_transposes": round(ms2, 4), "TOPS_with_transposes": round(ops_ / (ms2 * 1e-3) / 1e12, 1)})
        saida[f"{M}x{K}x{N}"] = linhas
        del X, W, dY, Wt, dYt, Xt
        torch.cuda.empty_cache()
    sem_erros(reg, "config2")
    return {"shapes_MKN": saida, "peak_TOPS": pico, "peak_source": f"2 x cuBLAS bf16 burst ({pk['origem']})", "reps": reps,
            "l2": "operands of every GEMM exceed L2", "ops": "2*M*N*K per GEMM"}


# ------------------------------------------------------------------------------------------------ training step
def nucleos_por_passo(reg, c):
    """Kernels of this library launched per step: one per recorded operation, except the attention on the tensor-core
    path (head dimension 64, T >= 128), whose forward is 2 launches (operand preparation + the kernel) and whose backward is
    5 (preparation, three row phases, the key-tile kernel), 6 with the map of zero tiles of P from T = 512 on.  The split-K memsets are not counted."""
    from jatai_b200 import ops
    n = len(reg.lancamentos)
    if ops.BLK == 32 and c["D"] == 64 * c["H"] and c["T"] % 64 == 0 and 128 <= c["T"] <= 1024:
        for lanc in reg.lancamentos:
            if lanc["op"].startswith("atencao_back"):
                n += 4 if (ops.ATENCAO_LIMITE or c["T"] <= 256) else 5
            elif lanc["op"].startswith("atencao"):
                n += 1
    return n


def resumo_perfil(reg):
    """Per-operation GPU time of one eager step (CUDA events around every launch), operation count and algorithmic bytes of its GEMMs."""
    tempos, ops_gemm, ms_gemm, alg = {}, 0.0, 0.0, 0.0
    from jatai_b200 import ops
    for (op, ini, fim), lanc in zip(reg.eventos, reg.lancamentos):
        ms = ini.elapsed_time(fim)
        tempos[op] = tempos.get(op, 0.0) + ms
        if op.startswith("gemm"):
            a, b = lanc["entradas"]["A"], lanc["entradas"]["B"]
            ops_gemm += 2.0 * a.shape[0] * a.shape[1] * b.shape[0]
            alg += bytes_gemm(a.shape[0], a.shape[1], b.shape[0], ops.BLK, op == "gemm_cru")
            ms_gemm += ms
    ordem = sorted(tempos.items(), key=lambda kv: -kv[1])
    return {"ms_per_op": {k: round(v, 4) for k, v in ordem}, "ms_total": sum(tempos.values()), "gemm_ops": ops_gemm, "gemm_ms": ms_gemm, "gemm_bytes": alg}


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
    ini, fim = ev(), ev()
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


def digest_estado(m):
    """SHA-256 over weights, momentum and residual (mantissas and exponents, in name order)."""
    h = hashlib.sha256()
    for n in sorted(m.p):
        for par in (m.p[n], m.mom[n], m.res[n]):
            for t in par:
                h.update(t.detach().cpu().numpy().tobytes())
    return h.digest()


def mede_passo(c, rank, mundo, dev, steps, warmup, via=None, eager=False, biblioteca=None, perfil=True, e2e=True, gemms=False):
    """One configuration of the training step: eager steps (workspace sizing, per-op profile), graph capture, timed replays
    with device-resident tokens, then the same through host buffers.  Returns a dict of measurements."""
    from jatai_b200 import modelo, paralelo
    ops, oc, reg = lanca_ops(c["blk"], f"passo{rank}", biblioteca)
    if via is not None:
        assert oc.lib.jt_gemm_via(via) == 0
    red = paralelo.Redutor() if mundo > 1 else None
    m = modelo.Modelo(c["V"], c["D"], c["H"], c["FF"], c["L"], 0, dev, oc, reg, redutor=red)
    Bt, T = c["Bt"], c["T"]
    lotes = [tuple(t.to(dev) for t in lote_tokens(100 * rank + i, Bt, T, c["V"])) for i in range(8)]
    r = {}
    reg.novo_passo(0)
    m.passo(*lotes[0], k_lr=c["k_lr"])                # first step pays the one-time costs (workspace, kernel attributes)
    reg.fim_passo()
    reg.perfil = perfil
    reg.novo_passo(1)
    m.passo(*lotes[1], k_lr=c["k_lr"])
    reg.fim_passo()
    r["lancamentos"] = nucleos_por_passo(reg, c)
    if perfil:
        r["perfil"] = resumo_perfil(reg)
    reg.perfil = False
    reg.tempos = {}
    if gemms:
        r["gemm_ms"], r["n_gemms"] = tempo_gemms(oc, reg)
    passo_fn, modo = None, "eager"
    if not eager:
        try:
            passo_fn, modo = modelo.PassoGravado(m, Bt, T, c["k_lr"]), "cuda_graph"
        except Exception as e:          # capture refused: run eagerly, say so
            modo = f"eager (graph capture failed: {type(e).__name__}: {e})"
    if passo_fn is None:
        def passo_fn(tok, alvo):
            reg.lancamentos = []
            return m.passo(tok, alvo, k_lr=c["k_lr"])
    r["modo"] = modo
    for i in range(warmup):
        passo_fn(*lotes[i % 8])
    barreira(mundo)
    rel = Relogios(dev.index or 0)
    ini, fim = ev(), ev()
    ini.record()
    for i in range(steps):
        perda = passo_fn(*lotes[i % 8])
    fim.record()
    barreira(mundo)
    r["ms"] = max_ranks(ini.elapsed_time(fim), mundo, dev) / steps
    r["clocks"] = rel.fim()
    sem_erros(reg, nome_passo(c))
    r["tps"] = mundo * Bt * T / (r["ms"] * 1e-3)
    r["perda"] = float(perda)
    if e2e:
        # end to end: tokens come from pinned host memory every step and the loss is read back every step
        hospedeiro = [tuple(t.pin_memory() for t in lote_tokens(100 * rank + i, Bt, T, c["V"])) for i in range(8)]

        def passo_e2e(i):
            tok, alvo = hospedeiro[i % 8]
            return float(passo_fn(tok.to(dev, non_blocking=True), alvo.to(dev, non_blocking=True)))      # device -> host read (synchronises)

        for i in range(2):
            passo_e2e(i)
        barreira(mundo)
        ini.record()
        for i in range(steps):
            passo_e2e(i)
        fim.record()
        barreira(mundo)
        r["ms_e2e"] = max_ranks(ini.elapsed_time(fim), mundo, dev) / steps
        r["tps_e2e"] = mundo * Bt * T / (r["ms_e2e"] * 1e-3)
        r["h2d"], r["d2h"] = 2 * Bt * T * 8, 8
    if red is not None:
        # every rank applied the same update to the same sums: the training state must be identical everywhere
        meu = torch.tensor(list(digest_estado(m)), dtype=torch.uint8, device=dev)
        todos = [torch.empty_like(meu) for _ in range(mundo)]
        torch.distributed.all_gather(todos, meu)
        r["estado_igual"] = all(torch.equal(t, todos[0]) for t in todos)
        r["fio"] = {"collectives_per_step": getattr(passo_fn, "coletivos_por_passo", None), "max_bytes_per_step": int(red._max.numel()),
                    "sum_bytes_per_step": int(getattr(red, "bytes_soma_passo", 0) or red._plano.numel() * 4)}
    del passo_fn, m, lotes
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return r


def braco_passo(args):
    rank, mundo, dev = inicia_gpu()
    c = CONFIGS[args.config]
    pk = picos()
    W = max(args.warmup, 3)
    r = mede_passo(c, rank, mundo, dev, args.steps, W, via=args.via, eager=args.eager, gemms=True, biblioteca=args.biblioteca)
    Bt, T = c["Bt"], c["T"]
    pf = r["perfil"]
    ach = pf["gemm_ops"] / (r["gemm_ms"] * 1e-3) / 1e12 if r.get("gemm_ms") else None
    pico_b, pico_s = 2.0 * pk["bf16"], 2.0 * pk["bf16_sust"]
    saida = {
        "metric": "train_tokens_per_s", "value": r["tps"], "unit": "tokens/s", "n_gpus": mundo, "steps": args.steps, "warmup": W,
        "ms_per_step": r["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+int32", "data": "synthetic",
        "config": {"workload": nome_passo(c), "tokens_per_gpu_step": Bt * T, "global_tokens_per_step": mundo * Bt * T, "block": c["blk"],
                   "mode": r["modo"], "parallelism": f"dp{mundo}",
                   "l2": "weights + momentum + residual + activations of a step exceed L2 (about 0.6 GB touched per step at the smallest configuration)",
                   "init": "seeded random weights (reference recipe), uniform random byte tokens"},
        "roofline": {"bound": "tensor", "achieved": ach, "peak": pico_s, "unit": "TOPS", "frac": (ach / pico_s) if ach else None,
                     "frac_of_2x_bf16_burst": (ach / pico_b) if ach else None,
                     "traffic": TRAFEGO_NCU["bytes"] * pf["gemm_bytes"] / bytes_gemm(*TRAFEGO_NCU["forma"], BLK, False) if mundo == 1 else None,
                     "traffic_source": TRAFEGO_NCU["fonte"] + "; scaled to the step's GEMM launches by their algorithmic bytes (cold-L2 figure: inside the step most operands are still in L2)",
                     "algorithmic_bytes": pf["gemm_bytes"],
                     "kernel": f"all {r.get('n_gemms')} block GEMMs of one step (k_gemm_tc), issued back to back from one CUDA graph with the step's own operands",
                     "peak_source": f"2 x cuBLAS bf16 sustained ({pk['origem']}); frac_of_2x_bf16_burst uses the burst figure", "gemm_ms_per_step": r.get("gemm_ms")},
        "clocks": r["clocks"],
        "e2e": {"value": r["tps_e2e"], "unit": "tokens/s", "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"],
                "ms_per_step": r["ms_e2e"], "includes": "tokens and targets from pinned host memory, the step, loss read back to the host every step"},
        "gpu_launches": r["lancamentos"] * args.steps,
        "extra": {"launches_per_step": r["lancamentos"], "loss_last": r["perda"], "ms_per_op_eager": pf["ms_per_op"]},
    }
    if mundo > 1:
        saida["extra"]["dp_state_identical"] = r["estado_igual"]
        saida["extra"]["wire"] = r["fio"]
    ex = saida["extra"]
    if not args.sem_extras:
        def tenta(nome, f):
            t0 = time.perf_counter()
            try:
                ex[nome] = f()
            except Exception as e:            # an extra leg never takes the headline down with it
                ex[nome] = {"failed": f"{type(e).__name__}: {e}"}
            if isinstance(ex[nome], dict):
                ex[nome]["leg_seconds"] = round(time.perf_counter() - t0, 1)
            torch.cuda.empty_cache()

        if args.config != "c5":
            def perna5():
                c5 = CONFIGS["c5"]
                r5 = mede_passo(c5, rank, mundo, dev, steps=3, warmup=1, via=args.via)
                d = {"workload": nome_passo(c5), "tokens_per_s": r5["tps"], "ms_per_step": r5["ms"], "e2e_tokens_per_s": r5["tps_e2e"], "steps": 3, "warmup": 1,
                     "mode": r5["modo"], "parallelism": f"dp{mundo}", "tokens_per_gpu_step": c5["Bt"] * c5["T"], "launches_per_step": r5["lancamentos"],
                     "loss_last": r5["perda"], "ms_per_op_eager": r5["perfil"]["ms_per_op"], "clocks": r5["clocks"]}
                if mundo > 1:
                    d["dp_state_identical"], d["wire"] = r5["estado_igual"], r5["fio"]
                return d
            tenta("config5", perna5)
        if mundo == 1:
            def perna2():
                _, oc, reg = lanca_ops(BLK, "sweep")
                return mede_sweep(oc, reg, dev)
            tenta("config2", perna2)
            tenta("config3", lambda: mede_ops(dev, reps=8, warmup=3))
            if args.config != "compat":
                def perna_c():
                    cc = CONFIGS["compat"]
                    rc = mede_passo(cc, 0, 1, dev, steps=10, warmup=3, perfil=False, e2e=False)
                    return {"workload": nome_passo(cc), "tokens_per_s": rc["tps"], "ms_per_step": rc["ms"], "launches_per_step": rc["lancamentos"], "mode": rc["modo"],
                            "note": "the reference library's own model size and tensor format (block 128, head dimension 4, T=128), on this library; "
                                    "`--impl reference` reports the reference's dp4a kernels on the same configuration"}
                tenta("compat", perna_c)
    if mundo > 1:
        torch.distributed.destroy_process_group()
    if rank != 0:
        return
    if mundo == 1 and not args.sem_cpu:
        try:
            ctps, dt, th, txt = cpu_passo_amostra(c)
            saida["cpu_baseline"] = {"value": ctps, "unit": "tokens/s", "cores": th, "kind": "port", "sample": txt}
        except Exception as e:
            saida["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    print(json.dumps(saida))


# ------------------------------------------------------------------------------------------------ fused op suite
def mede_ops(dev, reps=12, warmup=3, tokens=16384):
    """Benchmark configuration 3: the bandwidth-bound ops at 16384 tokens x D=1024 (block 32); achieved HBM GB/s per op from
    the algorithmic bytes (inputs read once + outputs written once).  Inputs rotate over enough copies to exceed L2."""
    ops, oc, reg = lanca_ops(BLK, "ops")
    M, D, FF, V, NW = tokens, 1024, 4096, 256, 12 * 1024 * 1024
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
    x2 = copias(lambda: bloco(M, D), 6)          # both operands of the add from the stated distribution (block exponents uniform over 9 values)
    casos_.append(("soma", 3 * M * D * b1, [lambda a=a, b=b: oc.soma(a, b) for a, b in zip(x, x2)]))
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
    casos_.append(("momento_peso (one launch)", NW * (6 + 7 * b1), [lambda a=a, b=b, ww=ww, r=r: oc.momento_peso(a, b, ww, r, 4, True) for a, b, ww, r in zip(gw, mom, w, res)]))
    Bt, T, H = 16, 1024, 16
    M_ops, M = M, Bt * T                       # the attention keeps its shape whatever the row count of the other ops
    qkv = copias(lambda: bloco(M, 3 * D, esp=3), 2)
    b_at = M * 3 * D * b1 + M * D * 6 + Bt * H * T * T
    casos_.append(("atencao (16 seq x 16 heads x T=1024, hd 64)", b_at, [lambda t=t: oc.atencao(t, Bt, T, H) for t in qkv]))
    saidas_at = [oc.atencao(t, Bt, T, H) for t in qkv]
    go = copias(lambda: bloco(M, D, e0=-20), 2)
    casos_.append(("atencao_back (same shape)", M * 3 * D * b1 + M * D * b1 + Bt * H * T * T + M * 3 * D * 6,
                   [lambda t=t, gg=gg, s=s: oc.atencao_back(gg, t, s[1], Bt, T, H) for t, gg, s in zip(qkv, go, saidas_at)]))
    pk = picos()
    tabela, tot_b, tot_ms = {}, 0.0, 0.0
    corrente = torch.cuda.Stream()
    n_lanc = 0
    for nome, nbytes, fs in casos_:
        for i in range(warmup):
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
        n_lanc += reps
        if not nome.startswith("atencao"):             # the attention kernels are contractions, not bandwidth ops: listed, not aggregated
            tot_b += nbytes
            tot_ms += ms
    sem_erros(reg, "config3")
    agg = tot_b / (tot_ms * 1e-3) / 1e9
    return {"per_op": tabela, "aggregate_GBs": agg, "aggregate_frac_of_measured_hbm": agg / pk["hbm_gbs"], "hbm_peak_GBs": pk["hbm_gbs"],
            "peak_source": f"STREAM-style copy ({pk['origem']})", "reps": reps, "ms_total": tot_ms, "launches": n_lanc,
            "workload": f"ops_{M_ops}tok_D1024_b32", "l2": "inputs rotate over copies totalling more than L2 (126 MB)",
            "timing": "each op recorded `reps` times in a CUDA graph over rotating inputs; the replay is timed with CUDA events",
            "aggregate_note": "bandwidth ops only; the two attention lines are contractions and are listed for their time"}


def braco_ops(args):
    rank, mundo, dev = inicia_gpu()
    r = mede_ops(dev, reps=max(args.steps, 5), warmup=max(args.warmup, 3), tokens=args.tokens)
    if rank != 0:
        return
    print(json.dumps({
        "metric": "fused_ops_hbm_gbs", "value": r["aggregate_GBs"], "unit": "GB/s", "n_gpus": 1, "steps": r["reps"], "warmup": max(args.warmup, 3),
        "ms_per_step": r["ms_total"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+int32", "data": "synthetic",
        "config": {"workload": r["workload"], "l2": r["l2"], "timing": r["timing"]},
        "per_op": r["per_op"],
        "roofline": {"bound": "hbm", "achieved": r["aggregate_GBs"], "peak": r["hbm_peak_GBs"], "unit": "GB/s", "frac": r["aggregate_frac_of_measured_hbm"],
                     "traffic": None, "peak_source": r["peak_source"]},
        "gpu_launches": r["launches"]}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="passo", choices=["gemm", "passo", "ops"])
    ap.add_argument("--config", default="c4", choices=sorted(CONFIGS), help="passo: which configuration is the headline")
    ap.add_argument("--via", type=int, default=None, help="force a GEMM path (jt_gemm_via)")
    ap.add_argument("--eager", action="store_true", help="passo: no CUDA graph")
    ap.add_argument("--forma", type=int, nargs=3, default=None, metavar=("M", "K", "N"), help="gemm: another shape (profiling captures)")
    ap.add_argument("--tokens", type=int, default=16384, help="ops: rows of the op suite (configuration 3 is 16384; larger sizes show the kernels without the launch overhead)")
    ap.add_argument("--sem-cpu", dest="sem_cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--sem-extras", dest="sem_extras", action="store_true", help="passo: headline only, no extra legs")
    ap.add_argument("--biblioteca", default=None, help="passo: another library with the same C ABI (diagnostics; block length of --config must suit it)")
    args = ap.parse_args()
    if args.forma:
        FORMA.update(M=args.forma[0], K=args.forma[1], N=args.forma[2])
    if args.impl == "reference":
        return braco_referencia_passo(args) if args.workload == "passo" else braco_referencia_gemm(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    if args.workload == "passo":
        return braco_passo(args)
    if args.workload == "ops":
        return braco_ops(args)
    return braco_gemm(args)


if __name__ == "__main__":
    main()
