"""The C-ABI library loads and exports every symbol include/jatai_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

RAIZ = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def simbolos_do_header():
    txt = open(os.path.join(RAIZ, "include", "jatai_b200.h")).read()
    return sorted(set(re.findall(r"\b(jt_[a-z0-9_]+)\s*\(", txt)))


def test_header_tem_as_entradas_da_referencia():
    nomes = simbolos_do_header()
    for n in ("jt_erro_le", "jt_erro_limpa", "jt_sincroniza", "jt_stream", "jt_gemm_split", "jt_gemm_bm", "jt_atencao_linhas", "jt_gemm_f",
              "jt_gemm", "jt_quant", "jt_soma", "jt_relu2", "jt_relu2_back", "jt_momento", "jt_peso", "jt_transpoe", "jt_embed",
              "jt_um_quente", "jt_rms", "jt_rms_back", "jt_atencao", "jt_atencao_back", "jt_softmax_ce", "jt_para16", "jt_para8",
              "jt_soma16", "jt_res_estocastico"):
        assert n in nomes, f"{n} (an entry point of the reference ABI) is not declared"


def test_biblioteca_exporta_tudo():
    from jatai_b200 import build
    so = build.build()
    lib = ctypes.CDLL(so)
    faltam = [n for n in simbolos_do_header() if not hasattr(lib, n)]
    assert not faltam, f"declared but not exported: {faltam}"


def test_ops_sem_gpu_falha_alto():
    """No CPU fallback: constructing the launcher without a CUDA device raises."""
    import pytest
    import torch
    if torch.cuda.is_available():
        pytest.skip("has a GPU")
    from jatai_b200 import ops, registro
    import tempfile
    with pytest.raises(RuntimeError):
        ops.OpsCuda(registro.Registro(tempfile.mkdtemp(), "x", eco=False))
