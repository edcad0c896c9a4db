from .marlin import mul_2_4, bmm_2_4, sbmm_2_4, sbmm_2_4_multilaunch
from .punica import add_lora_sgmv_cutlass, add_lora_bgmv

__all__ = ["mul_2_4", "bmm_2_4", "sbmm_2_4", "sbmm_2_4_multilaunch", "add_lora_sgmv_cutlass", "add_lora_bgmv"]
from .activations import QuickGELU
from .rotary_embedding import rotary_embedding, batched_rotary_embedding

__all__ += ["QuickGELU", "rotary_embedding", "batched_rotary_embedding"]
