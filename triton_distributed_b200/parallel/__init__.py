"""Parallel layers: TP (MLP / attention / MoE), EP, SP (flash-decode, all-gather attention, Ulysses), PP transport
(the reference's ``triton_dist.layers.nvidia``)."""
from .tp_mlp import TP_MLP  # noqa: F401
from .tp_attn import TP_Attn  # noqa: F401
from .tp_moe import TP_MoE  # noqa: F401
from .ep_layer import EPAll2AllLayer, EP_MoE  # noqa: F401
from .sp_flash_decode import SpGQAFlashDecodeAttention  # noqa: F401
from .sp_attention import (SPAllGatherAttentionContextIntraNode, create_sp_ag_attention_context_intra_node,  # noqa: F401
                           create_sp_ag_attention_context_inter_node, fused_sp_ag_attn_intra_node,
                           fused_sp_ag_attn_inter_node)
from .ulysses import SpUlysessQKVGemmAll2AllKernel, SpUlysessOAll2AllGemmKernel  # noqa: F401
from .pp import CommOp  # noqa: F401
from .gemm_ar_layer import GemmARLayer, AllGatherLayer  # noqa: F401
