"""d2dmoe_b200: the D2DMoE dynamic-k MoE-FFN inference layer on B200 (sm_100a).

Importing the package loads the in-tree CUDA library; there is no other backend.
"""
from . import ops  # noqa: F401  (loads the library, raises if it is missing)
from .moe import (MOE_IMPL_MAP, B200GluExperts, B200KernelExperts, MoeficationMoE,  # noqa: F401
                  MoeficationRouter, add_routers, add_save_output_norm_hook, bind_upstream,
                  fused_gemma_decoder_forward, fused_gpt_block_forward,
                  fused_vit_block_forward)

__all__ = ["MoeficationMoE", "MoeficationRouter", "B200KernelExperts", "B200GluExperts",
           "MOE_IMPL_MAP", "add_routers", "add_save_output_norm_hook", "bind_upstream", "fused_vit_block_forward", "fused_gpt_block_forward",
           "fused_gemma_decoder_forward", "ops"]
