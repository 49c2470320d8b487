"""Checked operator object: every operation runs on the CUDA launcher and on the oracle with the same inputs and
must agree bit for bit (the role of the reference's OpsConferido, jatai_cuda/ops.py:532-566).  Test infrastructure."""
import torch

import casos


def _cpu(a):
    if torch.is_tensor(a):
        return a.detach().cpu()
    if isinstance(a, tuple):
        return tuple(_cpu(x) for x in a)
    return a


class OpsConferido:
    nome = "conferido"

    def __init__(self, cuda_ops, oraculo):
        self.c, self.r = cuda_ops, oraculo
        self.lib = cuda_ops.lib
        self.n = {}

    def __getattr__(self, op):
        fc, fr = getattr(self.c, op), getattr(self.r, op)

        def f(*args, **kw):
            cpu_args = [_cpu(a) for a in args]
            if op in ("momento", "peso", "momento_peso"):                       # in-place on the device: the oracle works on copies
                cpu_args = [tuple(t.clone() for t in a) if isinstance(a, tuple) else a for a in cpu_args]
            kw_r = {k: _cpu(v) for k, v in kw.items()}
            out_r = fr(*cpu_args, **kw_r)
            out_c = fc(*args, **kw)
            torch.cuda.synchronize()
            for i, (a, b) in enumerate(zip(casos.plano(out_c), casos.plano(out_r))):
                a = a.cpu()
                if a.shape != b.shape or a.dtype != b.dtype or not torch.equal(a, b):
                    dif = (a != b) if a.shape == b.shape else None
                    onde = tuple(dif.nonzero()[0].tolist()) if dif is not None and dif.any() else None
                    raise AssertionError(f"op '{op}' output {i}: {int(dif.sum()) if dif is not None else '?'} of {a.numel()} differ"
                                         f" (first at {onde}: cuda {a[onde].item() if onde else '?'} oracle {b[onde].item() if onde else '?'})")
            self.n[op] = self.n.get(op, 0) + 1
            return out_c
        return f
