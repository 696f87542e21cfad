from .k2_fused import swiglu_quant_channelwise_out  # noqa: F401
