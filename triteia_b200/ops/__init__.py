"""Public op API — the names exported by the reference's triteia/python/ops/__init__.py:1-8."""
from .matmul.sparse_low_precision import matmul_4bit_2_4
from .matmul.bmm import bmm_4bit_2_4, bmm_4bit_2_4_forloop
from .matmul.sbmm import (sbmm_16bit_forloop, sbmm_4bit_2_4_forloop, sbmm_4bit_2_4_multilaunch,
                          sbmm_4bit_2_4_native, sbmm_4bit_2_4_segments, sbmm_indexed)
from .matmul.lora import lora_forloop, lora_bgmv, lora_sgmv, lora_indexed
from .matmul.ldmm import ldmm, baseline_ldmm
from .utils.sparsity import mask_creator
from .utils.generator import (gen_lora_16_bit, gen_batched_lora_16_bit, gen_sparse_quant4_NT,
                              gen_batched_sparse_quant4_NT, generate_model_distribution, fp16_to_sparse,
                              torch_weight_to_sparse_marlin, random_packed_deltas)

# spellings used by the benchmark description of this path
matmul_4bit_2of4 = matmul_4bit_2_4
sbmm_4bit_2of4_forloop = sbmm_4bit_2_4_forloop
sbmm_4bit_2of4_multilaunch = sbmm_4bit_2_4_multilaunch
sbmm_4bit_2of4_native = sbmm_4bit_2_4_native
