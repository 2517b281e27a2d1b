"""vLLM attention-backend hook for the packed-KV kernels, written against vLLM 0.22 (`vllm.v1`).

What the reference's plugin does with vLLM 0.10.2 (plugins/residual_quantization/src/residual_quantization/):

  packed_backend.py   `PackedBackend` / `PackedBuilder` / `PackedImpl`: an attention backend whose cache is
                      uint8 [2, blocks, heads, block_size, page_width], whose metadata splits a reordered batch into
                      its decode prefix and its full-prompt suffix, and whose forward runs the packed decode
                      attention (or flash-attn for prompts) and then stages / quantizes the new K/V.
  install_model.py    `install_model_attention`: swaps that backend into the `Attention` layers of a looped model,
                      one `DeferredKVGroup` per (physical layer, group of loops); the loops after the first share the
                      first one's cache.
  install_cache.py    `LoopCacheSpec` + allocator hooks: every owner layer gets a cache of its own packed format while
                      all owners share one block-ID space; kernels are warmed up before vLLM sizes the pool.
  scheduler.py        `FullPromptScheduler`: whole prompts only (no chunked prefill, no prefix caching).

The same pieces here, on the interfaces of vLLM 0.22.  Two things are simpler than in the reference because vLLM grew
them natively: a group of full-attention layers with DIFFERENT page sizes is allocated by vLLM itself
(`UniformTypeKVCacheSpecs`), so only `get_kv_cache_spec` has to be taught the packed page width, and a backend may own
its cache update (`forward_includes_kv_cache_update`).  The builder and the implementation derive from vLLM's abstract
base classes, not from its flash-attn backend: the packed kernel needs none of that backend's scheduling state.

Importing this module needs vLLM; nothing else in the package does.
"""

from __future__ import annotations

import inspect
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
from vllm.v1.attention.backend import (
    AttentionBackend,
    AttentionCGSupport,
    AttentionImpl,
    AttentionMetadata,
    AttentionMetadataBuilder,
    AttentionType,
    CommonAttentionMetadata,
)
from vllm.v1.kv_cache_interface import FullAttentionSpec
from vllm.v1.worker.ubatch_utils import UBatchSlice, split_attn_metadata

from . import _cuda
from .group import DeferredKVGroup, batch_slices

__all__ = (
    "PackedBackend", "PackedBuilder", "PackedImpl", "PackedMetadata", "LoopCacheSpec", "FullPromptScheduler",
    "install_model_attention", "install_vllm_cache_hooks", "packed_cache_specs", "warmup_packed_kernels",
    "serving_settings", "REFERENCE_BACKEND_NAME",
)

# the name the reference registers its backend under (packed_backend.py:206-207); vLLM 0.22 identifies third-party
# backends by the enum member CUSTOM instead, so this name is kept as an attribute
REFERENCE_BACKEND_NAME = "LOOP_PACKED_ACCELERATED"
CONFIG_KEYS = ("packed_groups", "coefficient_method", "reference_mode", "anchor_index", "rotation_artifact",
               "prefill_cpu_offload", "prefill_offload_chunk_tokens", "prefill_offload_lookahead")


# ----------------------------------------------------------------------------------------------------------
# metadata
# ----------------------------------------------------------------------------------------------------------


@dataclass
class PackedMetadata(AttentionMetadata):
    """What one attention call needs.  `parts` lists the batch's runs of one kind -- the decode prefix, the
    full-prompt suffix -- as (first token, last token, metadata of that run); a decode-only batch has one part that
    aliases the batch's own (CUDA-graph static) tensors."""

    num_actual_tokens: int
    max_query_len: int
    query_start_loc: torch.Tensor
    seq_lens: torch.Tensor
    block_table: torch.Tensor
    slot_mapping: torch.Tensor
    parts: List[Tuple[int, int, "PackedMetadata"]] = field(default_factory=list)

    @property
    def request_metadata(self):
        """The reference's name for `parts` (packed_backend.py:160-199)."""
        return self.parts


def _metadata_of(common: CommonAttentionMetadata) -> PackedMetadata:
    return PackedMetadata(
        num_actual_tokens=common.num_actual_tokens,
        max_query_len=common.max_query_len,
        query_start_loc=common.query_start_loc,
        seq_lens=common.seq_lens,
        block_table=common.block_table_tensor,
        slot_mapping=common.slot_mapping,
    )


class PackedBuilder(AttentionMetadataBuilder[PackedMetadata]):
    """Decode-only batches are CUDA-graph capturable; batches with prompts run eagerly and are split.

    vLLM puts the one-token requests first (`reorder_batch_threshold = 1`), so a mixed batch is a decode prefix
    followed by whole prompts.  A request with several query tokens that is not a whole prompt (chunked or recomputed
    prefill) is rejected: the quantizer needs every loop's K/V of a token at once (packed_backend.py:175-178)."""

    _cudagraph_support = AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE
    reorder_batch_threshold = 1

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        self._init_reorder_batch_threshold(1)

    def use_cascade_attention(self, *args, **kwargs) -> bool:
        return False

    @staticmethod
    def split(common: CommonAttentionMetadata) -> List[Tuple[int, int, CommonAttentionMetadata]]:
        """(first token, last token, metadata) of the decode prefix and of the full-prompt suffix."""
        if common.max_query_len == 1:
            # decode: nothing is read on the host, so stale CPU copies under graph replay do no harm
            return [(0, common.num_actual_tokens, common)]
        starts = common.query_start_loc_cpu[: common.num_reqs + 1].tolist()
        lengths = common.seq_lens_cpu_upper_bound
        if lengths is None:
            lengths = common.seq_lens.to("cpu")     # prompts only: an eager, synchronizing step anyway
            common = common.replace(seq_lens_cpu_upper_bound=lengths)
        runs = batch_slices(starts, lengths[: common.num_reqs].tolist())
        slices = [UBatchSlice(slice(run.first_request, run.last_request), slice(run.first_token, run.last_token))
                  for run in runs]
        return [(run.first_token, run.last_token, part)
                for run, part in zip(runs, split_attn_metadata(slices, common))]

    def build(self, common_prefix_len: int, common_attn_metadata: CommonAttentionMetadata,
              fast_build: bool = False) -> PackedMetadata:
        metadata = _metadata_of(common_attn_metadata)
        metadata.parts = [(begin, end, _metadata_of(part)) for begin, end, part in self.split(common_attn_metadata)]
        return metadata


# ----------------------------------------------------------------------------------------------------------
# implementation
# ----------------------------------------------------------------------------------------------------------


def _flash_prefill(query, key, value, output, metadata: PackedMetadata, scale: float) -> None:
    """Whole prompts attend to themselves causally over their raw bf16 K/V (library kernel, outside the packed path;
    the reference calls the same function: packed_backend.py:62-76)."""
    from vllm.v1.attention.backends.fa_utils import flash_attn_varlen_func, get_flash_attn_version

    flash_attn_varlen_func(
        q=query, k=key, v=value, out=output,
        cu_seqlens_q=metadata.query_start_loc, cu_seqlens_k=metadata.query_start_loc,
        max_seqlen_q=metadata.max_query_len, max_seqlen_k=metadata.max_query_len,
        softmax_scale=scale, causal=True, fa_version=get_flash_attn_version(),
    )


class PackedImpl(AttentionImpl[PackedMetadata]):
    """One attention slot (one loop of one KV group).  The layer object carries `packed_group`,
    `group_loop_index`, `key_rotation`, `value_rotation`, `key_mean` (set by `install_model_attention`)."""

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: Optional[int] = None,
                 alibi_slopes=None, sliding_window=None, kv_cache_dtype: str = "auto", logits_soft_cap=None,
                 attn_type: str = AttentionType.DECODER, kv_sharing_target_layer_name: Optional[str] = None,
                 prefill=None, **unused) -> None:
        if num_kv_heads not in (None, num_heads):
            raise ValueError("Packed attention requires matching Q/K/V head counts")
        if alibi_slopes is not None or sliding_window is not None or logits_soft_cap:
            raise ValueError("Packed attention is plain causal softmax attention: no ALiBi, window or soft cap")
        if attn_type != AttentionType.DECODER:
            raise ValueError("Packed attention serves decoder self-attention only")
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_heads
        self.kv_cache_dtype = kv_cache_dtype
        self.kv_sharing_target_layer_name = kv_sharing_target_layer_name
        self.prefill = prefill or _flash_prefill

    def forward(self, layer, query, key, value, kv_cache, attn_metadata: Optional[PackedMetadata], output=None,
                output_scale=None, output_block_scale=None):
        if output is None or output_scale is not None or output_block_scale is not None:
            raise ValueError("BF16 output required")
        if attn_metadata is None:        # vLLM's memory-profiling run
            return output
        group: DeferredKVGroup = layer.packed_group
        records = [list(r) for r in group.records]
        tokens = attn_metadata.slot_mapping.numel()
        offload = group.prefill_offload is not None and attn_metadata.max_query_len > 1
        completing = len(group.pending) + 1 == len(group.records)
        ring = offload and len(group.records) > 1 and getattr(group.prefill_offload, "lookahead_enabled", False)
        if ring and completing:
            group.prefill_offload.prepare(group, tokens)
        for begin, end, part in attn_metadata.parts:
            if part.max_query_len > 1:
                self.prefill(query[begin:end], key[begin:end], value[begin:end], output[begin:end], part, self.scale)
            else:
                _cuda.attention(query[begin:end], key[begin:end], value[begin:end], kv_cache, output[begin:end],
                                part.query_start_loc, part.seq_lens, part.block_table, layer.key_rotation,
                                layer.value_rotation, layer.key_mean, records, group.reference_mode, group.anchor_index,
                                layer.group_loop_index)
        # the new K/V: held back until the group's last loop, then all records are quantized in one call
        staged = group.stage(key[:tokens], value[:tokens], offload=offload)
        if staged is None:
            if ring and len(group.pending) + 1 == len(group.records):
                group.prefill_offload.preload(group, tokens)
            return output
        if ring and completing:
            chunks = group.prefill_offload.chunks(staged, attn_metadata.slot_mapping, group=group)
        elif offload and len(staged) > 1:
            chunks = group.prefill_offload.chunks(staged, attn_metadata.slot_mapping)
        else:
            chunks = ((staged, attn_metadata.slot_mapping),)
        for chunk_records, chunk_slots in chunks:
            _cuda.quantize(chunk_records, kv_cache, chunk_slots, layer.key_rotation, layer.value_rotation, layer.key_mean,
                           records, group.reference_mode, group.anchor_index, group.coefficient_method)
        return output


class PackedBackend(AttentionBackend):
    """Packed recurrent attention with its own cache layout and metadata."""

    accept_output_buffer = True
    forward_includes_kv_cache_update = True       # forward stages / quantizes the new K/V itself
    supported_dtypes = [torch.bfloat16]
    reference_name = REFERENCE_BACKEND_NAME

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_impl_cls():
        return PackedImpl

    @staticmethod
    def get_builder_cls():
        return PackedBuilder

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> Tuple[int, ...]:
        """`head_size` is the page width in bytes here (see `LoopCacheSpec`): uint8
        [2, blocks, heads, block_size, page_width], the layout of common/cache.cuh:71-106."""
        return (2, num_blocks, num_kv_heads, block_size, head_size)

    @staticmethod
    def get_kv_cache_stride_order(include_num_layers_dimension: bool = False) -> Tuple[int, ...]:
        if include_num_layers_dimension:
            return (0, 1, 2, 3, 4, 5)
        return (0, 1, 2, 3, 4)

    @classmethod
    def supports_head_size(cls, head_size: int) -> bool:
        return True

    @classmethod
    def supports_kv_cache_dtype(cls, kv_cache_dtype) -> bool:
        return kv_cache_dtype in (None, "auto", "bfloat16")


def register_packed_backend() -> None:
    """Make `AttentionBackendEnum.CUSTOM` resolve to `PackedBackend`."""
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    register_backend(AttentionBackendEnum.CUSTOM, f"{PackedBackend.__module__}.{PackedBackend.__qualname__}")


# ----------------------------------------------------------------------------------------------------------
# cache specification
# ----------------------------------------------------------------------------------------------------------


@dataclass(frozen=True, kw_only=True)
class LoopCacheSpec(FullAttentionSpec):
    """A packed owner layer: uint8 pages, `head_size` = bytes per token of one (head, plane)."""


def packed_cache_specs(specs: Dict[str, object], layers: Dict[str, object], heads: int, head_dim: int) -> Dict[str, object]:
    """Replace the spec of every layer that carries a `packed_group` by its packed page format
    (install_cache.py:111-137).  `specs` maps owner layer names to vLLM's own specs."""
    result = dict(specs)
    for name in specs:
        layer = layers.get(name)
        group = getattr(layer, "packed_group", None)
        if group is None:
            continue
        result[name] = LoopCacheSpec(block_size=group.page_tokens, num_kv_heads=heads,
                                     head_size=group.page_width(head_dim), dtype=torch.uint8)
    return result


def check_cache_specs(specs: Dict[str, object], max_model_len: int) -> int:
    """The conditions the reference's allocator checks before it shares block IDs between owners of different
    formats (install_cache.py:38-63).  Returns the common block size."""
    for spec in specs.values():
        if (not isinstance(spec, FullAttentionSpec) or spec.sliding_window is not None
                or spec.attention_chunk_size is not None):
            raise ValueError("Only native/packed full-attention caches are supported")
    block_sizes = {spec.block_size for spec in specs.values()}
    if len(block_sizes) != 1:
        raise ValueError("Group token block sizes differ")
    return block_sizes.pop()


@torch.inference_mode()
def warmup_packed_kernels(layers: Sequence[object], device) -> int:
    """One tiny quantize and one attention per loop for every distinct kernel variant among `layers`, so that lazily
    loaded CUDA modules and the library's scratch buffer exist before vLLM measures free memory and before any graph
    capture (install_cache.py:187-256).  Returns the number of variants touched."""
    seen = set()
    for layer in layers:
        group = getattr(layer, "packed_group", None)
        if group is None:
            continue
        heads, dim = layer.num_kv_heads, layer.head_size
        signature = (heads, dim, group.records, group.page_tokens, group.reference_mode, group.anchor_index,
                     group.coefficient_method, layer.key_mean is not None, id(layer.key_rotation), id(layer.value_rotation))
        if signature in seen:
            continue
        seen.add(signature)
        records = [list(r) for r in group.records]
        x = torch.zeros((1, heads, dim), dtype=torch.bfloat16, device=device)
        out = torch.empty_like(x)
        cache = torch.zeros(group.cache_shape(1, heads, dim), dtype=torch.uint8, device=device)
        slots = torch.zeros(1, dtype=torch.int64, device=device)
        starts = torch.tensor([0, 1], dtype=torch.int32, device=device)
        lengths = torch.ones(1, dtype=torch.int32, device=device)
        table = torch.zeros((1, 1), dtype=torch.int32, device=device)
        _cuda.quantize([(x, x)] * len(records), cache, slots, layer.key_rotation, layer.value_rotation, layer.key_mean,
                       records, group.reference_mode, group.anchor_index, group.coefficient_method)
        for loop in range(len(records)):
            _cuda.attention(x, x, x, cache, out, starts, lengths, table, layer.key_rotation, layer.value_rotation,
                            layer.key_mean, records, group.reference_mode, group.anchor_index, loop)
    if seen:
        torch.cuda.synchronize(device)
    return len(seen)


_hooks_installed = False


def install_vllm_cache_hooks() -> None:
    """Process-local patches of vLLM's GPU model runner: packed layers report their packed page format, and the packed
    kernels are warmed up at the end of the memory-profiling run.  Importing this module patches nothing."""
    global _hooks_installed
    if _hooks_installed:
        return
    from vllm.config import get_layers_from_vllm_config
    from vllm.model_executor.layers.attention_layer_base import AttentionLayerBase
    from vllm.v1.worker.gpu_model_runner import GPUModelRunner

    original_profile = GPUModelRunner.profile_run
    original_specs = GPUModelRunner.get_kv_cache_spec

    def profile_run(runner, *args, **kwargs):
        result = original_profile(runner, *args, **kwargs)
        layers = get_layers_from_vllm_config(runner.vllm_config, AttentionLayerBase)
        warmup_packed_kernels(list(layers.values()), runner.device)
        return result

    def get_kv_cache_spec(runner):
        specs = original_specs(runner)
        layers = get_layers_from_vllm_config(runner.vllm_config, AttentionLayerBase, list(specs))
        model = runner.vllm_config.model_config.hf_config
        heads = model.num_attention_heads
        specs = packed_cache_specs(specs, layers, heads, model.hidden_size // heads)
        if any(isinstance(spec, LoopCacheSpec) for spec in specs.values()):
            if runner.vllm_config.parallel_config.decode_context_parallel_size != 1:
                raise ValueError("Packed mixed storage requires DCP1")
            check_cache_specs(specs, runner.vllm_config.model_config.max_model_len)
        return specs

    GPUModelRunner.profile_run = profile_run
    GPUModelRunner.get_kv_cache_spec = get_kv_cache_spec
    register_packed_backend()
    _cuda.set_stable_metadata(True)   # vLLM writes lengths, tables and slots once per step, before the forward pass
    _hooks_installed = True


# ----------------------------------------------------------------------------------------------------------
# binding groups to the attention layers of a looped model
# ----------------------------------------------------------------------------------------------------------


def validate_config(config: dict, recurrences: int) -> List[Tuple[Tuple[int, int], ...]]:
    """Checks of install_model.py:133-150 on the `residual_quantization` section of vLLM's additional config."""
    unknown = [key for key in config if key not in CONFIG_KEYS]
    if unknown:
        raise ValueError(f"Unknown residual_quantization settings: {unknown}")
    if config["reference_mode"] not in ("adjacent", "anchor"):
        raise ValueError("Unsupported reference")
    if config["reference_mode"] == "adjacent" and config["anchor_index"] != 0:
        raise ValueError("Adjacent reference currently requires anchor_index=0")
    if config["coefficient_method"] not in ("unit", "norm", "ls"):
        raise ValueError("Unsupported coefficient method")
    schedules = config["packed_groups"]
    if not schedules or any(not records for records in schedules):
        raise ValueError("Every packed group must contain at least one record")
    if sum(map(len, schedules)) != recurrences:
        raise ValueError("Packed groups must describe every model recurrence exactly once")
    return [tuple(tuple(int(v) for v in record) for record in schedule) for schedule in schedules]


def slot_index(recurrent_slots_start: int, recurrence: int, layers_per_recurrence: int, layer: int) -> int:
    """Index of the attention slot of (recurrence, physical layer): slots are numbered recurrence-major after the
    prelude and coda slots (install_model.py:183-204)."""
    return recurrent_slots_start + recurrence * layers_per_recurrence + layer


def _prefill_offload(config: dict, vllm_config, pending_records: int, heads: int, head_dim: int):
    enabled = config.get("prefill_cpu_offload", False)
    chunk_tokens = config.get("prefill_offload_chunk_tokens", 512)
    lookahead = config.get("prefill_offload_lookahead", True)
    if not isinstance(enabled, bool):
        raise ValueError("prefill_cpu_offload must be a boolean")
    if type(chunk_tokens) is not int or chunk_tokens <= 0:
        raise ValueError("prefill_offload_chunk_tokens must be a positive integer")
    if not isinstance(lookahead, bool):
        raise ValueError("prefill_offload_lookahead must be a boolean")
    if not enabled or pending_records == 0:
        return None
    from vllm.config import CUDAGraphMode

    from .prefill_offload import PrefillHostStage

    if vllm_config.compilation_config.cudagraph_mode.mixed_mode() == CUDAGraphMode.FULL:
        raise ValueError("Prefill CPU offload requires eager prefill attention; "
                         "use FULL_DECODE_ONLY, PIECEWISE or NONE CUDA graphs")
    stage = PrefillHostStage(chunk_tokens)
    stage.lookahead_enabled = lookahead
    stage.reserve(vllm_config.scheduler_config.max_num_batched_tokens, pending_records, heads, head_dim)
    return stage


def install_model_attention(config: dict, data: Optional[dict], vllm_config, attention_settings: Dict[str, dict]) -> None:
    """Give every recurrent `Attention` layer of a loaded looped model the packed backend, its group state, rotations
    and key means; call after weight loading and before vLLM allocates the KV pool (install_model.py:120-221).

    config              the `residual_quantization` section (CONFIG_KEYS)
    data                calibrated artifact or None: key_rotations [layers, H, D, D] (shared by the groups) or
                        [groups, layers, H, D, D]; value_rotations likewise or None (absorbed into the weights);
                        key_means fp32 [recurrences, layers, H, D]
    attention_settings  layer name -> the arguments its `Attention.__init__` was called with (captured by the loader)
    """
    from vllm.config import get_layers_from_vllm_config
    from vllm.model_executor.layers.attention.attention import Attention, validate_kv_sharing_target
    from vllm.model_executor.models.utils import extract_layer_index
    from vllm.v1.attention.backends.registry import AttentionBackendEnum

    from . import rotation as rotation_registry

    model = vllm_config.model_config.hf_config
    page_tokens = vllm_config.cache_config.block_size
    layers_per_recurrence = model.n_layers_in_recurrent_block
    recurrent_slots_start = model.n_layers_in_prelude + model.n_layers_in_coda
    schedules = validate_config(config, model.mean_recurrence)
    heads = model.num_attention_heads
    offload = _prefill_offload(config, vllm_config, max(map(len, schedules)) - 1, heads, model.hidden_size // heads)

    context = vllm_config.compilation_config.static_forward_context
    slots = {extract_layer_index(layer.layer_name): layer
             for layer in get_layers_from_vllm_config(vllm_config, Attention).values()}
    parameters = inspect.signature(PackedImpl.__init__).parameters
    register_packed_backend()

    def device_rotation(matrix):
        """fp16 on the GPU; a matrix that is a signed Hadamard matrix is registered once, so that the kernels run their
        fused Walsh-Hadamard transform instead of the dense product."""
        matrix = matrix.contiguous().cuda().half()
        rotation_registry.register_rotation(matrix)
        return matrix

    shared_key_rotations = None
    if data is not None and data["key_rotations"].ndim == 4:
        shared_key_rotations = [device_rotation(m) for m in data["key_rotations"]]

    first_recurrence = 0
    for group_index, records in enumerate(schedules):
        key_rotations, value_rotations, key_means = shared_key_rotations, None, None
        if data is not None:
            key_means = data["key_means"][first_recurrence:first_recurrence + len(records)]
            if data["key_rotations"].ndim == 5:
                key_rotations = [device_rotation(m) for m in data["key_rotations"][group_index]]
            if data.get("value_rotations") is not None:
                value_rotations = [device_rotation(m) for m in data["value_rotations"][group_index]]
        chain: List[DeferredKVGroup] = []
        for layer_index in range(layers_per_recurrence):
            group = DeferredKVGroup(records, page_tokens, config["reference_mode"], config["anchor_index"],
                                    config["coefficient_method"], offload)
            if offload is not None and offload.lookahead_enabled:
                group.offload_chain, group.offload_index = chain, layer_index
                chain.append(group)
            owner_name = slots[slot_index(recurrent_slots_start, first_recurrence, layers_per_recurrence, layer_index)].layer_name
            key_mean = None
            if key_means is not None:
                key_mean = key_means[:, layer_index].contiguous().cuda()
            for loop, _ in enumerate(records):
                layer = slots[slot_index(recurrent_slots_start, first_recurrence + loop, layers_per_recurrence, layer_index)]
                owner = owner_name if loop > 0 else None
                if owner is not None:
                    validate_kv_sharing_target(layer.layer_name, owner, context)
                settings = dict(attention_settings[layer.layer_name])
                extra = settings.pop("extra_impl_args", None) or {}
                settings.update(num_heads=layer.num_heads, head_size=layer.head_size, num_kv_heads=layer.num_kv_heads,
                                sliding_window=layer.sliding_window, kv_cache_dtype=layer.kv_cache_dtype,
                                attn_type=layer.attn_type, kv_sharing_target_layer_name=owner)
                layer.impl = PackedImpl(**{name: settings[name] for name in parameters if name in settings}, **extra)
                layer.attn_backend = PackedBackend
                layer.backend = AttentionBackendEnum.CUSTOM
                layer.use_output = PackedBackend.accept_output_buffer
                layer.kv_sharing_target_layer_name = owner
                layer.packed_group = group
                layer.group_loop_index = loop
                layer.key_rotation = key_rotations[layer_index] if key_rotations is not None else None
                layer.value_rotation = value_rotations[layer_index] if value_rotations is not None else None
                layer.key_mean = key_mean
        first_recurrence += len(records)


# ----------------------------------------------------------------------------------------------------------
# scheduler and serving settings
# ----------------------------------------------------------------------------------------------------------


def check_scheduler_config(scheduler_config, cache_config) -> None:
    """Whole prompts only: the quantizer needs a token's K/V of every loop in one step (scheduler.py:11-20)."""
    if scheduler_config.max_num_batched_tokens < scheduler_config.max_model_len:
        raise ValueError("Full prompts require a budget of at least max_model_len")
    if scheduler_config.long_prefill_token_threshold:
        raise ValueError("Packed KV does not support partial long prefills")
    if cache_config.enable_prefix_caching:
        raise ValueError("Packed KV does not support cached prompt prefixes")
    scheduler_config.enable_chunked_prefill = False
    if hasattr(scheduler_config, "chunked_prefill_enabled"):
        scheduler_config.chunked_prefill_enabled = False


def _scheduler_class():
    from vllm.v1.core.sched.scheduler import Scheduler

    class FullPromptScheduler(Scheduler):
        """Admit full prompts together with decode requests; never a partial prefill."""

        def __init__(self, vllm_config, *args, **kwargs):
            check_scheduler_config(vllm_config.scheduler_config, vllm_config.cache_config)
            super().__init__(vllm_config, *args, **kwargs)

    return FullPromptScheduler


def __getattr__(name):
    # vLLM's scheduler module is heavy to import; build the subclass on first use
    if name == "FullPromptScheduler":
        cls = _scheduler_class()
        globals()[name] = cls
        return cls
    raise AttributeError(name)


def serving_settings(settings: dict, config: Optional[dict]) -> dict:
    """Engine arguments a packed configuration forces (scripts/evaluation/server_client.py:73-81): block size 32
    unless chosen, no prefix caching, no chunked prefill, and a token budget that holds a whole prompt."""
    settings = dict(settings)
    if config and config.get("packed_groups"):
        settings.setdefault("block_size", 32)
        settings.update(enable_prefix_caching=False, enable_chunked_prefill=False,
                        max_num_batched_tokens=max(4096, settings.get("max_num_batched_tokens", 0)))
    return settings
