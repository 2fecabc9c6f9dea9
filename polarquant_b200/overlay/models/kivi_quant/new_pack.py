"""Stand-in for the KIVI packer the reference imports unconditionally
(models/modeling_llama_polar.py:18) but does not ship."""


def triton_quantize_and_pack_along_last_dim(*args, **kwargs):
    raise NotImplementedError("kivi_quant is a third-party package the reference does not vendor; "
                              "the polar key-cache path never calls it")
