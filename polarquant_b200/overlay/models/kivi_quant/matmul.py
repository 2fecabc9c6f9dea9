"""Stand-in for the KIVI kernels the reference imports unconditionally
(models/modeling_llama_polar.py:19, benchmark/benchmark_matmul.py:9) but does not ship."""


def _absent(*args, **kwargs):
    raise NotImplementedError("kivi_quant is a third-party package the reference does not vendor; "
                              "the polar key-cache path never calls it")


cuda_bmm_fA_qB_outer = _absent
triton_bmm_fA_qB_outer = _absent
