"""Checkpoint and bit-exact resume of the integer training state.

The reference saves only weights and error-feedback residual, at the end of its long runs (jatai_cuda/noite.py:88-91),
and has no resume.  A resumed run can only continue bit for bit if the momentum and the state of the batch sampler's
random generator are restored as well, so all four are saved here.  Every tensor is an integer tensor: a checkpoint
is exact by construction, on any device.
"""
import torch


def salva(modelo, caminho, passo=0, gerador=None, extra=None):
    cpu = lambda d: {n: tuple(t.detach().cpu() for t in par) for n, par in d.items()}
    torch.save({
        "formato": 1, "passo": passo, "blk": int(modelo.p["emb"][0].shape[1] // modelo.p["emb"][1].shape[1]),
        "config": dict(V=modelo.V, D=modelo.D, H=modelo.H, FF=modelo.FF, L=modelo.L),
        "pesos": cpu(modelo.p), "momento": cpu(modelo.mom), "residuo": cpu(modelo.res),
        "gerador": gerador.get_state() if gerador is not None else None, "extra": extra,
    }, caminho)


def restaura(modelo, caminho, gerador=None):
    """Loads a checkpoint into an existing model of the same configuration, in place (a recorded CUDA graph stays
    valid).  Returns the step number stored with it.

    Also reads the reference's weight file (jatai_cuda/noite.py:88-91: {"modo", "L", "FF", "pesos", "residuo"}, no momentum, no
    step, no sampler state): weights and residual are loaded, the momentum starts from zero blocks and 0 is returned - a
    run continued from such a file is NOT a bit-exact continuation of the run that wrote it (a warning says so)."""
    d = torch.load(caminho, map_location="cpu")
    if "config" not in d and "pesos" in d and "residuo" in d:
        import warnings
        from . import ops as O
        if d.get("modo", "int8") != "int8" or d.get("L", modelo.L) != modelo.L or d.get("FF", modelo.FF) != modelo.FF:
            raise ValueError(f"reference weight file is for modo={d.get('modo')}, L={d.get('L')}, FF={d.get('FF')}; the model has L={modelo.L}, FF={modelo.FF}")
        warnings.warn("reference weight file: no momentum, step or sampler state in it - the momentum starts from zero, the "
                      "continuation is not bit-exact")
        _copia(modelo.p, d["pesos"])
        _copia(modelo.res, d["residuo"])
        for m, E in modelo.mom.values():
            m.zero_()
            E.fill_(O.E_ZERO)
        return 0
    cfg = dict(V=modelo.V, D=modelo.D, H=modelo.H, FF=modelo.FF, L=modelo.L)
    if d["config"] != cfg:
        raise ValueError(f"checkpoint is for {d['config']}, the model is {cfg}")
    for destino, origem in ((modelo.p, d["pesos"]), (modelo.mom, d["momento"]), (modelo.res, d["residuo"])):
        _copia(destino, origem)
    if gerador is not None and d["gerador"] is not None:
        gerador.set_state(d["gerador"])
    return d["passo"]


def _copia(destino, origem):
    for n, par in origem.items():
        if n not in destino:
            raise ValueError(f"tensor '{n}' of the checkpoint does not exist in the model")
        for t, s in zip(destino[n], par):
            if t.shape != s.shape or t.dtype != s.dtype:
                raise ValueError(f"tensor '{n}' of the checkpoint has shape {tuple(s.shape)}, the model {tuple(t.shape)} (block length differs?)")
            t.copy_(s)
