"""The public names and call signatures a user of the reference relies on (its modules, file by file)."""
import inspect

import torch


def _params(fn):
    return list(inspect.signature(fn).parameters)


def test_process_group_manager_surface():
    from picotron_b200 import process_group_manager as pgm
    assert _params(pgm.setup_process_group_manager) == ["tp_size", "cp_size", "pp_size", "dp_size"]
    pgm.reset()
    g = pgm.get()                                                     # single-process stand-in: same attribute surface
    for a in ("global_rank", "world_size", "local_rank", "tp_rank", "cp_rank", "pp_rank", "dp_rank", "tp_group", "cp_group",
              "pp_group", "dp_group", "cp_dp_group", "pp_dp_group", "tp_world_size", "cp_world_size", "pp_world_size",
              "dp_world_size", "cp_dp_world_size", "tp_first_rank", "tp_last_rank", "cp_send_rank", "cp_recv_rank",
              "pp_is_first_stage", "pp_is_last_stage", "pp_next_rank", "pp_prev_rank"):
        assert hasattr(g, a), a
    assert str(g).startswith("TP(1)-CP(1)-PP(1)-DP(1)-Rank(")


def test_parallel_module_surface():
    from picotron_b200.parallel import (bucket, context_parallel, cp_communications, data_parallel, pipeline_parallel,
                                        pp_communications, tensor_parallel, tp_communications)
    assert _params(tensor_parallel.apply_tensor_parallel) == ["model"]
    assert _params(tensor_parallel.ColumnParallelLinear.__init__)[1:] == ["in_features", "out_features", "bias", "gather_output",
                                                                         "async_all_reduce"]
    assert _params(tensor_parallel.RowParallelLinear.__init__)[1:] == ["in_features", "out_features", "bias"]
    assert _params(tensor_parallel.VocabParallelEmbedding.__init__)[1:] == [
        "num_embeddings", "embedding_dim", "padding_idx", "max_norm", "norm_type", "scale_grad_by_freq", "sparse"]
    for name in ("CopyToModelParallelRegion", "ReduceFromModelParallelRegion", "GatherFromModelParallelRegion",
                 "LinearWithAsyncAllReduce", "linear_with_all_reduce", "linear_with_async_all_reduce"):
        assert hasattr(tp_communications, name), name
    assert _params(pipeline_parallel.PipelineParallel.__init__)[1:] == ["model", "config"]
    assert _params(pipeline_parallel.PipelineParallel.forward)[1:4] == ["input_ids", "position_ids", "hidden_states"]
    assert _params(pipeline_parallel.PipelineParallel.backward)[1:] == ["input_tensor", "output_tensor", "output_tensor_grad"]
    for fn in (pipeline_parallel.train_step_pipeline_afab, pipeline_parallel.train_step_pipeline_1f1b):
        assert _params(fn) == ["model", "data_loader", "tensor_shapes", "device", "dtype"]
    assert _params(pp_communications.pipeline_communicate) == ["operation", "device", "dtype", "tensor", "shapes"]
    assert _params(pp_communications.bidirectional_pipeline_communicate) == ["operation", "send_tensor", "recv_shapes", "device",
                                                                            "dtype"]
    assert _params(context_parallel.apply_context_parallel) == ["model"]
    assert _params(context_parallel.ring_attention) == ["q", "k", "v", "sm_scale", "is_causal"]
    assert _params(context_parallel.update_rope_for_context_parallel) == ["cos", "sin"]
    cc = cp_communications.ContextCommunicate
    assert _params(cc.__init__)[1:] == ["msg"] and _params(cc.send_recv)[1:] == ["tensor_to_send", "recv_tensor"]
    assert callable(cc.commit) and callable(cc.wait)
    assert _params(data_parallel.DataParallelBucket.__init__)[1:4] == ["module", "bucket_cap_mb", "grad_type"]
    for m in ("no_sync", "reset", "backward", "forward"):
        assert hasattr(data_parallel.DataParallelBucket, m) and hasattr(data_parallel.DataParallelNaive, m) or m == "reset"
    assert _params(bucket.BucketManager.__init__)[1:5] == ["params", "process_group", "bucket_size", "grad_type"]
    for m in ("reset", "wait", "mark_param_as_ready"):
        assert hasattr(bucket.BucketManager, m), m


def test_model_state_and_utils_surface():
    from picotron_b200 import checkpoint, data, model, utils
    assert _params(model.Llama.forward)[1:4] == ["input_ids", "attention_mask", "position_ids"]
    assert _params(model.get_cos_sin) == ["seq_length", "head_dim", "base"]
    for n in ("Llama", "DecoderLayer", "Attention", "MLP", "Embedding", "FinalProjection", "TritonRMSNorm", "LlamaRMSNorm",
              "apply_rotary_pos_emb", "flash_attention"):
        assert hasattr(model, n), n
    cm = checkpoint.CheckpointManager
    assert _params(cm.save_checkpoint)[1:6] == ["model", "optimizer", "trained_steps", "trained_tokens", "out_dir"]
    assert _params(cm.load_checkpoint)[1:] == ["model", "optimizer", "out_dir"]
    assert _params(checkpoint.init_model_with_dematerialized_weights) == ["include_buffers"]
    assert _params(checkpoint.init_model_with_materialized_weights)[:3] == ["model", "model_config", "save_dir"]
    assert hasattr(checkpoint, "InitializationManager")
    assert _params(data.MicroBatchDataLoader.__init__)[1:9] == ["micro_batch_size", "seq_length", "dataset_name", "tokenizer_name",
                                                               "num_workers", "num_proc", "grad_acc_steps", "device"]
    for n in ("print", "set_all_seed", "to_readable_format", "get_mfu", "get_num_params", "assert_no_meta_tensors",
              "average_loss_across_dp_cp_ranks", "download_model"):
        assert hasattr(utils, n), n
    assert _params(utils.get_mfu)[:3] == ["tokens_per_second", "num_params", "model_config"]
    assert utils.to_readable_format(1_050_000) == "1.05M" and utils.to_readable_format(999) == "999.00"


def test_llama_forward_returns_logits_without_targets():
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.config import ModelConfig
    from picotron_b200.model import Llama
    pgm.reset()
    cfg = ModelConfig(hidden_size=32, intermediate_size=64, vocab_size=50, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=8)
    m = Llama(cfg)
    ids = torch.randint(0, 50, (2, 8))
    logits = m(input_ids=ids, attention_mask=None, position_ids=None)
    assert logits.shape == (2, 8, 50)
