"""Overlapped ops, collectives and single-GPU kernels (the reference's ``triton_dist.kernels.nvidia``)."""
from .gemm import (gemm, linear, gemm_reference, new_stall_counters, summarize_stall_counters,  # noqa: F401
                   STALL_COUNTERS)
from .ag_gemm import (AllGatherGEMMTensorParallelContext, create_ag_gemm_context, ag_gemm,  # noqa: F401
                      ag_gemm_reference)
from .gemm_rs import (GEMMReduceScatterTensorParallelContext, create_gemm_rs_context, gemm_rs,  # noqa: F401
                      gemm_rs_reference)
from .allreduce import (AllReduceMethod, AllReduceContext, create_allreduce_ctx, all_reduce,  # noqa: F401
                        get_auto_allreduce_method)
from .reduce_scatter import (ReduceScatter2DContext, create_reduce_scater_2d_ctx, create_reduce_scatter_2d_ctx,  # noqa: F401
                             reduce_scatter_2d_op, ring_reduce)
from .allgather import (AllGatherMethod, get_auto_all_gather_method, FastAllGatherContext,  # noqa: F401
                        create_fast_allgather_context, fast_allgather, all_gather_ll, all_gather,
                        cp_engine_producer_all_gather_intra_node,
                        cp_engine_producer_all_gather_inter_node)
from .elementwise import (rmsnorm, silu_mul, residual_add, qk_norm_rope_kv, embedding, argmax, sample_token,  # noqa: F401
                          abs_sum)
from .attention import (flash_attn_varlen, gqa_fwd_batch_decode, gqa_fwd_batch_decode_intra_rank,  # noqa: F401
                        gqa_fwd_batch_decode_persistent, attention_reference, merge_attention_partials,
                        dense_block_table, decode_workspace, pick_kv_splits)
from .gemv import (GemvARContext, create_gemv_ar_context, gemv_fused, gemv_reference, gemv_supported,  # noqa: F401
                   GEMV_FAST_M, GEMV_MAX_M)
from .gemm_ar import (GemmARContext, LLGemmARContext, create_gemm_ar_context, create_ll_gemm_ar_context,  # noqa: F401
                      gemm_allreduce_op, low_latency_gemm_allreduce_op, skinny_gemm, gemm_ar_reference)
from .moe import (topk_router, sort_topk_ids_align_block_size, calc_gather_scatter_index, group_gemm_sorted,  # noqa: F401
                  gather_sorted, reduce_topk, unsort, MoESort, create_ag_group_gemm_context, ag_group_gemm,
                  create_moe_rs_context, create_moe_ar_context, run_moe_reduce_rs, run_moe_reduce_ar,
                  topk_router_reference, group_gemm_reference, moe_reduce_reference)
from .ep_a2a import (AllToAllContext, EpRecv, create_all_to_all_context, ep_dispatch, ep_combine, fast_all_to_all,  # noqa: F401
                     all_to_all_post_process, fp8_quant, fp8_dequant)
from .all_to_all import (AllToAllSingle2DContext, create_all_to_all_single_2d_context, all_to_all_single_2d)  # noqa: F401

from .gdn import (chunk_gated_delta_rule_fwd, gated_delta_rule_chunked, gated_delta_rule_recurrent,  # noqa: F401,E402
                  prepare_chunk_indices, prepare_lens)
from .fp8 import (ag_gemm_fp8, dequantize_act_1x128, dequantize_weight_128x128, gemm_fp8_blockscaled,  # noqa: F401,E402
                  gemm_fp8_blockscaled_reference, quantize_act_1x128, quantize_weight_128x128,
                  create_ag_gemm_fp8_context, create_gemm_rs_fp8_context, gemm_rs_fp8, ag_gemm_fp8_reference,
                  gemm_rs_fp8_reference, AGGemmFp8Context, GemmRSFp8Context)
from .moe import (tile_arrival_order, tile_schedule, sort_topk_ids_staged, group_gemm_gather,  # noqa: F401,E402
                  MoESort, MoEAgScatterGroupGemmContext, MoEReduceRSContext)
