"""Data-parallel training step with a deterministic, bit-exact gradient reduction.

One process per GPU (torch.distributed; NCCL over NVLink on the GPUs, gloo for the CPU tests).  The reference has no
multi-GPU code; the scheme follows from its own split-K argument (jatai_cuda/jatai_cuda.cu:214-216): any partition
of the reduced dimension of a block GEMM gives bit-identical sums PROVIDED every part aligns its partial products
to the same row-maximum exponents.  In the weight-gradient GEMM the reduced dimension is the token axis, and data
parallelism is exactly a partition of it.  So, per weight tensor:
  1. each rank computes the row maxima of its own operands (jt_max_linha),
  2. all-reduce MAX of those int8 vectors (a few KB),
  3. each rank runs the GEMM on its tokens with the global maxima -> int32 partial sums with one common exponent,
  4. all-reduce SUM of the int32 sums: exact, and the same bits whatever order the library adds in,
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
        self.bytes_max = 0        # bytes this rank put on the wire, per kind (for the bench report)
        self.bytes_soma = 0
        self.chamadas = 0

    def log2_tokens(self, locais):
        n = locais * self.mundo
        k = int(math.log2(n))
        assert 1 << k == n, f"global token count {n} is not a power of two"
        return k

    def maximos(self, RA, RB):
        """Global row-maximum exponents of both GEMM operands, one collective for the pair."""
        junto = torch.cat([RA, RB])
        dist.all_reduce(junto, op=dist.ReduceOp.MAX, group=self.grupo)
        self.bytes_max += junto.numel()
        self.chamadas += 1
        return junto[:RA.numel()].contiguous(), junto[RA.numel():].contiguous()

    def soma(self, acc):
        """Exact integer sum of the ranks' int32 partial accumulators (in place)."""
        dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.grupo)
        self.bytes_soma += acc.numel() * 4
        self.chamadas += 1
        return acc


def media_da_perda(perda, grupo=None):
    """Mean loss over all ranks (report only)."""
    t = perda.detach().clone()
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=grupo)
    return t / dist.get_world_size(grupo)
