"""The public names a user of the reference imports (kernels/nvidia/__init__.py:25-92, layers/nvidia/__init__.py:25-30,
utils.py, models/__init__.py, mega_triton_kernel/models) exist here under the same names."""
import pytest


def test_reference_api_names_exist():
    import triton_distributed_b200 as tdb
    from triton_distributed_b200 import language, mega, models, ops, parallel, tools, utils

    names = {
        tdb: ["initialize_distributed", "finalize_distributed", "nvshmem_create_tensor", "nvshmem_create_tensors",
              "nvshmem_free_tensor_sync", "nvshmem_barrier_all_on_stream"],
        language: ["wait", "consume_token", "notify", "symm_at", "rank", "num_ranks"],
        ops: ["create_ag_gemm_context", "ag_gemm", "create_gemm_rs_context", "gemm_rs", "create_gemm_ar_context",
              "create_ll_gemm_ar_context", "gemm_allreduce_op", "low_latency_gemm_allreduce_op", "create_allreduce_ctx",
              "all_reduce", "AllReduceMethod", "get_auto_allreduce_method", "create_fast_allgather_context",
              "fast_allgather", "cp_engine_producer_all_gather_intra_node", "cp_engine_producer_all_gather_inter_node",
              "AllGatherMethod", "get_auto_all_gather_method", "create_reduce_scater_2d_ctx", "reduce_scatter_2d_op",
              "ring_reduce", "create_all_to_all_context", "fast_all_to_all", "all_to_all_post_process",
              "create_all_to_all_single_2d_context", "all_to_all_single_2d", "create_ag_group_gemm_context",
              "ag_group_gemm", "create_moe_rs_context", "run_moe_reduce_rs", "run_moe_reduce_ar", "gqa_fwd_batch_decode",
              "gqa_fwd_batch_decode_intra_rank", "gqa_fwd_batch_decode_persistent"],
        parallel: ["GemmARLayer", "AllGatherLayer", "EPAll2AllLayer", "SpGQAFlashDecodeAttention",
                   "create_sp_ag_attention_context_intra_node", "create_sp_ag_attention_context_inter_node",
                   "fused_sp_ag_attn_intra_node", "fused_sp_ag_attn_inter_node", "SpUlysessQKVGemmAll2AllKernel",
                   "SpUlysessOAll2AllGemmKernel", "CommOp", "TP_MLP", "TP_Attn", "TP_MoE"],
        models: ["AutoLLM", "DenseLLM", "Qwen3MoE", "KV_Cache", "Engine", "ModelConfig"],
        mega: ["ModelBuilder", "Qwen3Model"],
        tools: ["contextual_autotune"],
        utils: ["group_profile", "perf_func", "dist_print", "assert_allclose", "bitwise_equal"],
    }
    missing = [f"{mod.__name__}.{n}" for mod, ns in names.items() for n in ns if not hasattr(mod, n)]
    assert not missing, missing

    tp = ["_init_parameters", "_init_ctx", "_init_AR_ctx", "_init_gemm_ar_ctx", "torch_fwd", "dist_triton_fwd",
          "dist_triton_AR_fwd", "dist_triton_gemm_ar_fwd"]
    methods = [
        (parallel.TP_MLP, tp), (parallel.TP_Attn, tp),
        (parallel.TP_MoE, ["_init_parameters", "_init_ctx", "torch_fwd", "dist_triton_fwd"]),
        (parallel.CommOp, ["read", "set_signal", "wait_signal"]),
        (parallel.EPAll2AllLayer, ["dispatch", "combine"]),
        (models.DenseLLM, ["set_fwd", "inference"]), (models.Engine, ["serve"]),
        (mega.ModelBuilder, ["compile", "run", "dump_trace", "get_sm_activity", "make_fc1", "make_fc2", "make_qkv_proj",
                             "make_o_proj", "make_linear", "make_flash_decode", "make_silu_mul_up",
                             "make_qk_norm_rope_update_kvcache", "make_rms_norm", "make_add",
                             "make_barrier_all_intra_node", "make_allreduce", "make_prefetch", "make_flash_attn",
                             "make_qkv_pack_flash_attn", "make_qkv_pack_qk_norm_rope_split_v"]),
        (mega.Qwen3Model, ["mega_forwrad"]),
        (parallel.SpUlysessQKVGemmAll2AllKernel, ["forward", "pre_attn_a2a", "qkv_pack_a2a"]),
        (parallel.SpUlysessOAll2AllGemmKernel, ["forward", "post_attn_a2a"]),
    ]
    missing = [f"{cls.__name__}.{m}" for cls, ms in methods for m in ms if not hasattr(cls, m)]
    assert not missing, missing


def test_decode_only_megakernel_says_so():
    from triton_distributed_b200.mega import ModelBuilder

    for name in ("make_flash_attn", "make_qkv_pack_flash_attn", "make_qkv_pack_qk_norm_rope_split_v"):
        with pytest.raises(NotImplementedError, match="decode-only"):
            getattr(ModelBuilder, name)(object.__new__(ModelBuilder))


def test_consume_token_returns_its_value():
    from triton_distributed_b200 import language

    assert language.consume_token(7, token=object()) == 7
