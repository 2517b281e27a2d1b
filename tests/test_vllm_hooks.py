"""The vLLM hook layer on CPU: metadata split, cache specs, configuration checks (needs vLLM importable; no GPU).

Fabricated `CommonAttentionMetadata` stands in for what vLLM's model runner hands to a metadata builder."""

from types import SimpleNamespace

import pytest
import torch

pytest.importorskip("vllm", reason="the hook layer is written against vLLM's v1 interfaces")

from residualquant_b200 import cache_plan  # noqa: E402
from residualquant_b200 import vllm_hooks as H  # noqa: E402
from residualquant_b200.group import DeferredKVGroup  # noqa: E402
from vllm.v1.attention.backend import CommonAttentionMetadata  # noqa: E402

RECORDS = ((2, 32), (2, 32), (2, 32), (4, 32))


def _common(query_lens, seq_lens, blocks=4):
    starts = torch.tensor([0] + list(torch.tensor(query_lens).cumsum(0)), dtype=torch.int32)
    tokens = int(starts[-1])
    lens = torch.tensor(seq_lens, dtype=torch.int32)
    return CommonAttentionMetadata(
        query_start_loc=starts.clone(), query_start_loc_cpu=starts, seq_lens=lens, num_reqs=len(query_lens),
        num_actual_tokens=tokens, max_query_len=max(query_lens), max_seq_len=max(seq_lens),
        block_table_tensor=torch.arange(len(query_lens) * blocks, dtype=torch.int32).view(len(query_lens), blocks),
        slot_mapping=torch.arange(tokens, dtype=torch.int64), seq_lens_cpu_upper_bound=lens.clone())


def _builder():
    config = SimpleNamespace(parallel_config=SimpleNamespace(decode_context_parallel_size=1), speculative_config=None)
    spec = H.LoopCacheSpec(block_size=16, num_kv_heads=16, head_size=200, dtype=torch.uint8)
    return H.PackedBuilder(spec, ["layers.0.attn"], config, torch.device("cpu"))


def test_decode_only_batch_is_one_part_that_aliases_the_batch_tensors():
    common = _common([1, 1, 1], [40, 7, 300])
    metadata = _builder().build(0, common)
    assert len(metadata.parts) == 1 and metadata.request_metadata is metadata.parts
    begin, end, part = metadata.parts[0]
    assert (begin, end) == (0, 3) and part.max_query_len == 1
    # same storage: a CUDA-graph replay sees whatever the runner wrote into these tensors
    assert part.seq_lens.data_ptr() == common.seq_lens.data_ptr()
    assert part.block_table.data_ptr() == common.block_table_tensor.data_ptr()
    assert part.query_start_loc.data_ptr() == common.query_start_loc.data_ptr()


def test_mixed_batch_splits_into_decode_prefix_and_prompt_suffix():
    common = _common([1, 1, 21, 5], [150, 47, 21, 5])
    metadata = _builder().build(0, common)
    assert [(b, e) for b, e, _ in metadata.parts] == [(0, 2), (2, 28)]
    decode, prompts = metadata.parts[0][2], metadata.parts[1][2]
    assert decode.max_query_len == 1 and decode.seq_lens.tolist() == [150, 47]
    assert decode.query_start_loc.tolist() == [0, 1, 2] and decode.block_table.shape[0] == 2
    assert prompts.max_query_len == 21 and prompts.query_start_loc.tolist() == [0, 21, 26]   # rebased to the part
    assert prompts.seq_lens.tolist() == [21, 5] and prompts.slot_mapping.tolist() == list(range(2, 28))
    # prompts only
    only = _builder().build(0, _common([9, 4], [9, 4]))
    assert [(b, e) for b, e, _ in only.parts] == [(0, 13)]


def test_partial_prefill_is_rejected():
    with pytest.raises(ValueError, match="partial prefill"):
        _builder().build(0, _common([1, 8], [30, 20]))        # 8 new tokens of a 20-token sequence
    with pytest.raises(ValueError, match="must precede"):
        _builder().build(0, _common([6, 1], [6, 30]))         # the runner did not reorder the batch


def test_builder_contract():
    builder = _builder()
    assert builder.reorder_batch_threshold == 1 and builder.use_cascade_attention() is False
    from vllm.v1.attention.backend import AttentionCGSupport

    assert H.PackedBuilder.get_cudagraph_support(None, None) == AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE


def test_backend_contract_and_registration():
    B = H.PackedBackend
    assert B.get_kv_cache_shape(100, 16, 16, 200) == (2, 100, 16, 16, 200)        # packed_backend.py:222-223
    assert B.get_kv_cache_stride_order() == (0, 1, 2, 3, 4)
    assert B.get_impl_cls() is H.PackedImpl and B.get_builder_cls() is H.PackedBuilder
    assert B.forward_includes_kv_cache_update and B.accept_output_buffer
    assert B.reference_name == "LOOP_PACKED_ACCELERATED" and B.supports_head_size(224)
    H.register_packed_backend()
    from vllm.v1.attention.backends.registry import AttentionBackendEnum

    assert AttentionBackendEnum[B.get_name()].get_class() is B


def test_packed_layers_report_their_page_format():
    from vllm.v1.kv_cache_interface import FullAttentionSpec, UniformTypeKVCacheSpecs

    group = DeferredKVGroup(RECORDS, 16)
    native = FullAttentionSpec(block_size=16, num_kv_heads=16, head_size=128, dtype=torch.bfloat16)
    specs = {"a": native, "b": native, "c": native}
    layers = {"a": SimpleNamespace(packed_group=group), "b": SimpleNamespace(), "c": SimpleNamespace(packed_group=group)}
    out = H.packed_cache_specs(specs, layers, 16, 128)
    assert isinstance(out["a"], H.LoopCacheSpec) and out["b"] is native and out["a"] == out["c"]
    assert out["a"].head_size == 200 and out["a"].dtype == torch.uint8
    # one block of a packed owner: 2 planes x 16 heads x 16 tokens x 200 bytes, as the pool-sizing arithmetic has it
    owner = cache_plan.OwnerSpec(16, 128, 16, RECORDS)
    assert out["a"].page_size_bytes == owner.page_bytes == 2 * 16 * 16 * 200
    assert H.check_cache_specs(out, 8192) == 16
    # vLLM allocates owners of different page sizes under one block table by itself
    assert UniformTypeKVCacheSpecs.is_uniform_type(out)
    with pytest.raises(ValueError, match="block sizes differ"):
        H.check_cache_specs({**out, "d": FullAttentionSpec(block_size=32, num_kv_heads=16, head_size=128, dtype=torch.bfloat16)}, 8192)
    with pytest.raises(ValueError, match="full-attention"):
        H.check_cache_specs({"w": FullAttentionSpec(block_size=16, num_kv_heads=16, head_size=128, dtype=torch.bfloat16,
                                                     sliding_window=512)}, 8192)


def test_configuration_checks():
    good = {"packed_groups": [[[2, 32]] * 3 + [[4, 32]]], "coefficient_method": "ls", "reference_mode": "anchor",
            "anchor_index": 3}
    assert H.validate_config(good, 4) == [RECORDS]
    with pytest.raises(ValueError, match="every model recurrence"):
        H.validate_config(good, 8)
    with pytest.raises(ValueError, match="anchor_index=0"):
        H.validate_config({**good, "reference_mode": "adjacent"}, 4)
    with pytest.raises(ValueError, match="coefficient"):
        H.validate_config({**good, "coefficient_method": "median"}, 4)
    with pytest.raises(ValueError, match="at least one record"):
        H.validate_config({**good, "packed_groups": [[]]}, 0)
    with pytest.raises(ValueError, match="Unknown"):
        H.validate_config({**good, "bf16_variant": 1}, 4)
    # Huginn numbering: 2 prelude + 2 coda slots, then recurrence-major
    assert H.slot_index(4, 0, 4, 0) == 4 and H.slot_index(4, 3, 4, 2) == 18
    assert H.serving_settings({"max_num_batched_tokens": 2048}, good) == {
        "max_num_batched_tokens": 4096, "block_size": 32, "enable_prefix_caching": False, "enable_chunked_prefill": False}
    assert H.serving_settings({"block_size": 16}, None) == {"block_size": 16}


def test_scheduler_accepts_whole_prompts_only():
    cache = SimpleNamespace(enable_prefix_caching=False)
    sched = SimpleNamespace(max_num_batched_tokens=8192, max_model_len=4096, long_prefill_token_threshold=0,
                            enable_chunked_prefill=True)
    H.check_scheduler_config(sched, cache)
    assert sched.enable_chunked_prefill is False
    with pytest.raises(ValueError, match="at least max_model_len"):
        H.check_scheduler_config(SimpleNamespace(max_num_batched_tokens=1024, max_model_len=4096,
                                                 long_prefill_token_threshold=0), cache)
    with pytest.raises(ValueError, match="partial long prefills"):
        H.check_scheduler_config(SimpleNamespace(max_num_batched_tokens=8192, max_model_len=4096,
                                                 long_prefill_token_threshold=512), cache)
    with pytest.raises(ValueError, match="prefixes"):
        H.check_scheduler_config(sched, SimpleNamespace(enable_prefix_caching=True))
    from vllm.v1.core.sched.scheduler import Scheduler

    assert issubclass(H.FullPromptScheduler, Scheduler)


def test_implementation_rejects_what_the_kernel_does_not_do():
    H.PackedImpl(16, 128, 128 ** -0.5, 16)
    with pytest.raises(ValueError, match="matching Q/K/V"):
        H.PackedImpl(16, 128, 1.0, 4)
    with pytest.raises(ValueError, match="window"):
        H.PackedImpl(16, 128, 1.0, 16, sliding_window=1024)
    impl = H.PackedImpl(16, 128, 1.0, 16)
    with pytest.raises(ValueError, match="BF16 output"):
        impl.forward(None, None, None, None, None, None, output=None)
    sentinel = object()
    assert impl.forward(None, None, None, None, None, None, output=sentinel) is sentinel    # profiling run: no metadata


def test_reference_module_name_resolves_to_this_library():
    """The reference's hook imports `residual_quantization._cuda` (packed_backend.py:17-20)."""
    from residual_quantization._cuda import attention, quantize
    from residualquant_b200 import _cuda

    assert attention is _cuda.attention and quantize is _cuda.quantize
