"""Data-parallel training step with a deterministic, bit-exact gradient reduction.

One process per GPU (torch.distributed; NCCL over NVLink on the GPUs, gloo for the CPU tests).  The reference has no
multi-GPU code; the scheme follows from its own split-K argument (jatai_cuda/jatai_cuda.cu:214-216): any partition
of the reduced dimension of a block GEMM gives bit-identical sums PROVIDED every part aligns its partial products
to the same row-maximum exponents.  In the weight-gradient GEMM the reduced dimension is the token axis, and data
parallelism is exactly a partition of it.  So, per weight tensor:
  1. each rank computes the row maxima of its own operands (jt_max_linha) during the backward,
  2. after the backward, ONE all-reduce MAX of all those int8 vectors of the step (tens of KB),
  3. each rank runs the (deferred) GEMMs on its tokens with the global maxima -> int32 partial sums with one
     common exponent,
  4. after the backward, ONE all-reduce SUM of all int32 sums of the step (a flat buffer): exact, and the same
     bits whatever order the library adds in,
  5. every rank applies the same momentum / weight update, so weights stay identical without a broadcast.
Requirements: equal token counts per rank, a multiple of 128 (the transposition tile); the global token count a
power of two (softmax_ce averages by a shift).  The result equals one GPU running the concatenated batch.
"""
import math

import torch
import torch.distributed as dist


class Redutor:
    """The three hooks jatai_b200.modelo.Modelo calls when it runs data parallel."""

    def __init__(self, grupo=None):
        assert dist.is_initialized(), "initialise torch.distributed first"
        self.grupo = grupo
        self.mundo = dist.get_world_size(grupo)
        # the small MAX exchanges get a communicator of their own, so that they never queue behind a gradient SUM in flight
        self.grupo_max = dist.new_group(ranks=dist.get_process_group_ranks(grupo) if grupo is not None else None)
        self.bytes_max = 0        # bytes this rank put on the wire, per kind (for the bench report)
        self.bytes_soma = 0
        self.chamadas = 0

    def log2_tokens(self, locais):
        n = locais * self.mundo
        k = int(math.log2(n))
        assert 1 << k == n, f"global token count {n} is not a power of two"
        return k

    def maximos_tudo(self, pares):
        """Global row-maximum exponents of all deferred weight-gradient GEMMs of a step, as ONE collective.
        `pares` = [(RA_local, RB_local), ...] int8 vectors; returns the same structure with the maxima over ranks
        (views of a flat buffer kept between steps, so a captured graph finds them at fixed addresses)."""
        total = sum(ra.numel() + rb.numel() for ra, rb in pares)
        dev = pares[0][0].device
        if getattr(self, "_max", None) is None or self._max.numel() != total or self._max.device != dev:
            self._max = torch.empty(total, dtype=torch.int8, device=dev)
        self.empacota_maximos(pares)
        self.reduz_maximos()
        return self.vistas_maximos(pares)

    def inicio_passo(self):
        """Start of a training step: once the flat buffer of row maxima exists (from the second step on) it is pre-set to -128
        so that the transposition kernels can write their maxima straight into it (`fatias_max`)."""
        self._cursor_max = 0
        if getattr(self, "_max", None) is not None:
            self._max.fill_(-128)

    def fatias_max(self, na, nb):
        """The next two slices (na and nb int8 entries) of the flat buffer, in the order the step produces its weight-gradient
        operands - the same order `empacota_maximos` uses - or None while the buffer does not exist yet (first step) or the
        request does not fit (the caller then computes the maxima apart and they are copied in)."""
        m = getattr(self, "_max", None)
        o = getattr(self, "_cursor_max", None)
        if m is None or o is None or o + na + nb > m.numel() or o % 4 or na % 4:
            self._cursor_max = None                                  # out of step with the plan: no more in-place slices this step
            return None
        self._cursor_max = o + na + nb
        return m[o:o + na], m[o + na:o + na + nb]

    def empacota_maximos(self, pares, o=0):
        """Puts local maxima into the flat buffer from offset `o` on (those written in place by `fatias_max` are there
        already); returns the offset after them."""
        base = self._max.data_ptr()
        for ra, rb in pares:
            for r in (ra, rb):
                if r.data_ptr() != base + o:
                    self._max[o:o + r.numel()].copy_(r)
                o += r.numel()
        return o

    def vistas_maximos(self, pares):
        o, out = 0, []
        for ra, rb in pares:
            a = self._max[o:o + ra.numel()]
            b = self._max[o + ra.numel():o + ra.numel() + rb.numel()]
            out.append((a, b))
            o += ra.numel() + rb.numel()
        return out

    def reduz_maximos(self):
        dist.all_reduce(self._max, op=dist.ReduceOp.MAX, group=self.grupo_max)
        self.bytes_max += self._max.numel()
        self.chamadas += 1

    def reduz_maximos_fatia(self, o0, o1):
        """MAX over ranks of one slice of the flat buffer of maxima, asynchronously; returns the work handle."""
        w = dist.all_reduce(self._max[o0:o1], op=dist.ReduceOp.MAX, group=self.grupo_max, async_op=True)
        self.bytes_max += o1 - o0
        self.chamadas += 1
        return w

    def soma_tudo(self, grads):
        """Exact integer sum over ranks of every weight gradient of a step, as ONE collective: the int32 partial
        accumulators are packed into a flat buffer (kept between steps), all-reduced with SUM and handed back as
        views.  The exponents are equal on all ranks by construction and are not exchanged."""
        vistas = self.empacota_somas(grads)
        self.reduz_somas()
        return vistas

    def empacota_somas(self, grads):
        total = sum(acc.numel() for acc, _ in grads.values())
        algum = next(iter(grads.values()))[0]
        if getattr(self, "_plano", None) is None or self._plano.numel() != total or self._plano.device != algum.device:
            self._plano = torch.empty(total, dtype=torch.int32, device=algum.device)
        self._total_plano = total
        o, vistas = 0, {}
        for n, (acc, e) in grads.items():
            v = self._plano[o:o + acc.numel()].view(acc.shape)
            v.copy_(acc)
            vistas[n] = (v, e)
            o += acc.numel()
        return vistas

    def empacota_grupo(self, grupo, todos):
        """empacota_somas for one group of consecutive gradients.  `todos` fixes the layout of the flat buffer: it holds,
        in order, every gradient up to and including this group (later ones are not needed to place it).  Returns the
        group's views and its (start, end) in the buffer, which an eager step has already sized."""
        total = getattr(self, "_total_plano", None)
        assert getattr(self, "_plano", None) is not None and total is not None, "run one eager data-parallel step first"
        nomes = list(todos.keys())
        primeiro = nomes.index(next(iter(grupo)))
        o = sum(todos[n][0].numel() for n in nomes[:primeiro])
        o0, vistas = o, {}
        for n, (acc, e) in grupo.items():
            v = self._plano[o:o + acc.numel()].view(acc.shape)
            v.copy_(acc)
            vistas[n] = (v, e)
            o += acc.numel()
        assert o <= total
        return vistas, (o0, o)

    def reduz_fatia(self, o0, o1):
        """SUM over ranks of one slice of the flat buffer, asynchronously: returns the work handle; `wait()` on it makes
        the then-current stream wait for the result."""
        w = dist.all_reduce(self._plano[o0:o1], op=dist.ReduceOp.SUM, group=self.grupo, async_op=True)
        self.bytes_soma += (o1 - o0) * 4
        self.chamadas += 1
        return w

    def reduz_somas(self):
        dist.all_reduce(self._plano, op=dist.ReduceOp.SUM, group=self.grupo)
        self.bytes_soma += self._plano.numel() * 4
        self.chamadas += 1


def media_da_perda(perda, grupo=None):
    """Mean loss over all ranks (report only)."""
    t = perda.detach().clone()
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=grupo)
    return t / dist.get_world_size(grupo)
