from .marlin import mul_2_4, bmm_2_4, sbmm_2_4, sbmm_2_4_multilaunch
from .punica import add_lora_sgmv_cutlass, add_lora_bgmv

__all__ = ["mul_2_4", "bmm_2_4", "sbmm_2_4", "sbmm_2_4_multilaunch", "add_lora_sgmv_cutlass", "add_lora_bgmv"]
