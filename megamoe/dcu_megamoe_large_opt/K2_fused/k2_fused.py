"""`from megamoe.dcu_megamoe_large_opt.K2_fused.k2_fused import swiglu_quant_channelwise_out` as the reference's test
does (tests/test_mega_moe_dcu.py:32); the kernel is mm_swiglu_quant_channelwise of the B200 library."""
from deepgemm_b200.megamoe import swiglu_quant_channelwise_out  # noqa: F401
