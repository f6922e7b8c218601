"""vLLM attention backend ``CUSTOM`` over ``pth_flash_attn_fwd`` on B200 (sm_100a).

Counterpart of the reference's backend module (python/pth_flash_attn/vllm_backend.py:
builder 230-459, backend class 462-566, Impl 569-796), for the same job: serve vLLM's paged
``int8_per_token_head`` cache, as vLLM's own writer fills it, with this library's kernels.
The cache spec, the page layout and the quantising writer stay vLLM's (the classes derive
from the Triton backend's, exactly because the write side must not change); only the read
side is replaced.

How a step runs:

* ``PthFlashAttnMetadataBuilder.build`` turns the batch into at most two :class:`OpCall`
  records - the decode-like requests (query length up to the reorder threshold, which
  includes speculative verification) and the prefill requests behind them - each with the
  launch plan of its own padded descriptor (``planner.plan_launch``).  The split exists
  because the op's split workspace is ``[S, T, Hq, D]``: a decode slice wants many pieces
  of few tokens, a prefill slice one piece of many tokens.  The second call's
  ``query_start_loc`` is rebased on the device into a persistent buffer (the host copy may
  be ahead of the device one under adaptive verification).
* ``PthFlashAttnImpl.forward`` issues those calls.  It allocates nothing and reads no device
  data: the workspace was reserved when the layer was constructed (inside the window whose
  memory vLLM's KV-cache budget accounts for), the cache views are built once per cache
  tensor, and every per-step tensor is a view of vLLM's persistent buffers.  A decode-only
  step is therefore capturable in a CUDA graph (``UNIFORM_BATCH``).

What is refused, with a reason, at construction or at ``build``: cascade attention, DCP /
PCP, dual-batch overlap, R-SWA, ALiBi, soft caps, sinks, fused output quantisation,
per-request causal masks, encoder attention, and a sliding window or non-causal attention
at a head size without a windowed kernel.  Devices whose compute capability is not 10.x are
refused by ``supports_compute_capability``.

This module makes no ``torch.cuda`` call; device questions go through vLLM's platform
object.
"""
from __future__ import annotations

import dataclasses
import inspect
from typing import Any, ClassVar

import torch
from vllm.config import VllmConfig, get_current_vllm_config_or_none
from vllm.logger import init_logger
from vllm.platforms import current_platform
from vllm.v1.attention.backend import (
    AttentionCGSupport,
    AttentionMetadataBuilder,
    AttentionType,
    CommonAttentionMetadata,
    MultipleOf,
)
from vllm.v1.attention.backends.triton_attn import TritonAttentionBackend, TritonAttentionImpl
from vllm.v1.attention.backends.utils import get_num_attention_heads_from_layers, split_decodes_and_prefills
from vllm.v1.kv_cache_interface import KVQuantMode
from vllm.v1.worker.workspace import current_workspace_manager, is_workspace_manager_initialized

from . import ops, planner

logger = init_logger(f"vllm.{__name__}")

BACKEND_NAME = "CUSTOM"                 # the enum member vLLM reserves for plugins
KV_CACHE_DTYPE = "int8_per_token_head"  # the one cache format served
KERNEL_BLOCK_MULTIPLE = 16              # page sizes are multiples of 16 slots
SUPPORTED_CC_MAJOR = 10                 # sm_100a
SCALE_BYTES = 4                         # one fp32 scale behind the int8 row of a head


# --------------------------------------------------------------------------
# sizes taken from the configuration
# --------------------------------------------------------------------------
def verify_query_len(vllm_config: VllmConfig) -> int:
    """Query tokens of a decode request: 1, plus the draft tokens under speculation."""
    spec = getattr(vllm_config, "speculative_config", None)
    drafts = getattr(spec, "num_speculative_tokens", None) if spec is not None else None
    return 1 + (int(drafts) if drafts else 0)


def _num_sms(device: torch.device | None = None) -> int:
    index = getattr(device, "index", None)
    if index is None:
        index = torch.accelerator.current_device_index()
    return int(current_platform.num_compute_units(index))


def reserved_token_splits(vllm_config: VllmConfig, *, num_kv_heads: int, head_size: int, num_sms: int) -> int:
    """Token-splits of workspace a layer reserves: enough for every decode-like plan."""
    return planner.workspace_token_splits(
        max_num_seqs=int(vllm_config.scheduler_config.max_num_seqs), q_dec_max=verify_query_len(vllm_config),
        Hkv=num_kv_heads, D=head_size, num_sms=num_sms)


def group_window(kv_cache_spec: Any) -> int:
    """Sliding window of the layers of a KV-cache group (0: none)."""
    return int(getattr(kv_cache_spec, "sliding_window", None) or 0)


def _heads_per_kv(num_q_heads: int, num_kv_heads: int) -> int:
    if num_kv_heads < 1 or num_q_heads % num_kv_heads:
        raise ValueError(f"pth_flash_attn: Hq = {num_q_heads} is not a positive multiple of Hkv = {num_kv_heads}")
    group = num_q_heads // num_kv_heads
    if group > planner.MAX_ROWS_PER_CTA:
        raise ValueError(f"pth_flash_attn: G = Hq / Hkv = {group} exceeds {planner.MAX_ROWS_PER_CTA}")
    return group


def _windowed_refusal(what: str, head_size: int) -> str:
    sizes = ", ".join(str(d) for d in planner.WINDOWED_HEAD_SIZES)
    return f"{what} at head size {head_size} (windowed kernels exist for D = {sizes} only)"


# --------------------------------------------------------------------------
# cache views
# --------------------------------------------------------------------------
def cache_views(kv_cache: torch.Tensor, head_size: int) -> tuple[torch.Tensor, ...]:
    """``(k, v, k_scale, v_scale)`` views of one layer's ``int8_per_token_head`` cache.

    The op takes logical ``[blocks, slots, kv heads, D]`` int8 and ``[blocks, slots, kv heads]``
    fp32 tensors of any strides.  vLLM has shipped two physical layouts of this cache, told
    apart by rank:

    * ``[blocks, kv heads, slots, 2 * (D + 4)]`` - one packed cell ``K | k_scale | V |
      v_scale`` per (head, slot); the layout the reference's reader is written for
      (python/pth_flash_attn/vllm_backend.py:680-702, docs/integration.md:45-50);
    * ``[blocks, 2, slots, kv heads, D + 4]`` - a K half and a V half per block, each row
      followed by its scale.
    No byte is copied in either case.
    """
    if kv_cache.dtype not in (torch.int8, torch.uint8):
        raise NotImplementedError(f"pth_flash_attn: cache dtype {kv_cache.dtype} is not int8")
    data = kv_cache if kv_cache.dtype == torch.int8 else kv_cache.view(torch.int8)
    row = head_size + SCALE_BYTES
    as_f32 = torch.tensor([], dtype=torch.float32, device=kv_cache.device).set_(kv_cache.untyped_storage())
    base = kv_cache.storage_offset()

    def scales(first_byte: int, strides: tuple[int, int, int], shape: tuple[int, int, int]) -> torch.Tensor:
        if (base + first_byte) % 4 or any(s % 4 for s in strides):
            raise NotImplementedError("pth_flash_attn: cache scales are not 4-byte aligned")
        return torch.as_strided(as_f32, shape, tuple(s // 4 for s in strides), (base + first_byte) // 4)

    if data.dim() == 4 and data.shape[-1] == 2 * row:
        blocks, heads, slots, _ = data.shape
        sb, sh, ss, _ = data.stride()
        cells = data.permute(0, 2, 1, 3)  # [blocks, slots, heads, cell]
        shape = (blocks, slots, heads)
        return (cells[..., :head_size], cells[..., row:row + head_size],
                scales(head_size, (sb, ss, sh), shape), scales(row + head_size, (sb, ss, sh), shape))
    if data.dim() == 5 and data.shape[1] == 2 and data.shape[-1] == row:
        blocks, _, slots, heads, _ = data.shape
        sb, s2, ss, sh, _ = data.stride()
        shape = (blocks, slots, heads)
        return (data[:, 0, :, :, :head_size], data[:, 1, :, :, :head_size],
                scales(head_size, (sb, ss, sh), shape), scales(s2 + head_size, (sb, ss, sh), shape))
    raise NotImplementedError(f"pth_flash_attn: unknown int8_per_token_head cache shape {tuple(kv_cache.shape)}")


# --------------------------------------------------------------------------
# metadata
# --------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class OpCall:
    """Everything one ``pth_flash_attn_fwd`` call needs besides the layer's own tensors."""

    plan: planner.LaunchPlan
    tokens: slice                    # rows of query / output this call covers
    max_query_len: int
    query_start_loc: torch.Tensor    # int32 [requests + 1], starting at 0
    seq_lens: torch.Tensor           # int32 [requests]
    block_table: torch.Tensor        # int32 [>= requests, blocks]


@dataclasses.dataclass
class PthAttnMetadata:
    """One step's metadata: the fields vLLM's runners read, plus the op calls."""

    num_actual_tokens: int
    max_query_len: int
    query_start_loc: torch.Tensor
    max_seq_len: int
    seq_lens: torch.Tensor
    block_table: torch.Tensor
    slot_mapping: torch.Tensor
    causal: bool
    calls: tuple[OpCall, ...]
    use_cascade: bool = False
    common_prefix_len: int = 0

    @property
    def decode(self) -> OpCall | None:
        """The call over the decode-like requests, if the step has one."""
        return next((c for c in self.calls if not c.plan.is_prefill), None)

    @property
    def prefill(self) -> OpCall | None:
        return next((c for c in self.calls if c.plan.is_prefill), None)


class PthFlashAttnMetadataBuilder(AttentionMetadataBuilder[PthAttnMetadata]):
    """Plans the op calls of a step; owns one small persistent buffer."""

    # decode batches of one uniform query length replay as full graphs; a step with a
    # prefill runs piecewise
    _cudagraph_support: ClassVar[AttentionCGSupport] = AttentionCGSupport.UNIFORM_BATCH
    supports_draft_decode_metadata_update = True

    def __init__(self, kv_cache_spec: Any, layer_names: list[str], vllm_config: VllmConfig,
                 device: torch.device) -> None:
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        parallel = vllm_config.parallel_config
        if getattr(parallel, "use_ubatching", False) or getattr(parallel, "num_ubatches", 1) > 1:
            raise NotImplementedError("pth_flash_attn: dual-batch overlap is not supported (one workspace per layer)")
        model = vllm_config.model_config
        if getattr(model, "rswa_window", None) is not None:
            raise NotImplementedError("pth_flash_attn: R-SWA is not supported")
        q_heads = (get_num_attention_heads_from_layers(vllm_config, layer_names)
                   or model.get_num_attention_heads(parallel))
        self.num_kv_heads = int(kv_cache_spec.num_kv_heads)
        self.head_size = int(kv_cache_spec.head_size)
        self.group = _heads_per_kv(int(q_heads), self.num_kv_heads)
        if self.head_size not in planner.SUPPORTED_HEAD_SIZES:
            raise NotImplementedError(
                f"pth_flash_attn: head size {self.head_size} is not one of {planner.SUPPORTED_HEAD_SIZES}")
        self.window = group_window(kv_cache_spec)
        if self.window and self.head_size not in planner.WINDOWED_HEAD_SIZES:
            raise NotImplementedError("pth_flash_attn: " + _windowed_refusal("sliding window", self.head_size))
        # a request is decode-like while its query fits one 64-row tile; a speculative
        # verification of 1 + k tokens counts as a decode too
        self._init_reorder_batch_threshold(planner.max_tokens_per_tile(self.group), supports_spec_as_decode=True)
        self.num_sms = _num_sms(device)
        self.ws_token_splits = reserved_token_splits(vllm_config, num_kv_heads=self.num_kv_heads,
                                                     head_size=self.head_size, num_sms=self.num_sms)
        self._rebased_qsl = torch.zeros(int(vllm_config.scheduler_config.max_num_seqs) + 1, dtype=torch.int32,
                                        device=device)

    @classmethod
    def get_varlen_cudagraph_max_query_len(cls, vllm_config: VllmConfig, kv_cache_spec: Any) -> int:
        """Longest decode query a full graph covers: the reorder threshold, from the config."""
        heads = vllm_config.model_config.get_num_attention_heads(vllm_config.parallel_config)
        group = _heads_per_kv(int(heads), int(kv_cache_spec.num_kv_heads))
        return max(planner.max_tokens_per_tile(group), verify_query_len(vllm_config))

    def _call(self, cam: CommonAttentionMetadata, requests: slice, tokens: slice, max_query_len: int,
              is_prefill: bool) -> OpCall:
        count = requests.stop - requests.start
        plan = planner.plan_launch(
            num_tokens=tokens.stop - tokens.start, num_reqs=count, max_query_len=max_query_len, G=self.group,
            Hkv=self.num_kv_heads, D=self.head_size, num_sms=self.num_sms, is_prefill=is_prefill,
            ws_token_splits=self.ws_token_splits, window=self.window)
        starts = cam.query_start_loc
        if requests.start == 0:
            qsl = starts if starts.shape[0] == count + 1 else starts[:count + 1]
        else:
            if count + 1 > self._rebased_qsl.shape[0]:
                raise RuntimeError(f"pth_flash_attn: {count} prefill requests exceed max_num_seqs = "
                                   f"{self._rebased_qsl.shape[0] - 1}")
            qsl = self._rebased_qsl[:count + 1]
            first = requests.start
            torch.sub(starts[first:requests.stop + 1], starts[first:first + 1], out=qsl)  # on the device
        return OpCall(plan=plan, tokens=tokens, max_query_len=max_query_len, query_start_loc=qsl,
                      seq_lens=cam.seq_lens[requests], block_table=cam.block_table_tensor[requests])

    def build(self, common_prefix_len: int, common_attn_metadata: CommonAttentionMetadata,
              fast_build: bool = False) -> PthAttnMetadata:
        cam = common_attn_metadata
        if common_prefix_len > 0:
            raise NotImplementedError("pth_flash_attn: cascade attention")
        causal = cam.causal
        if not isinstance(causal, bool):
            raise NotImplementedError(
                f"pth_flash_attn: per-request causal masks are not supported (got {type(causal).__name__})")
        if not causal and self.head_size not in planner.WINDOWED_HEAD_SIZES:
            raise NotImplementedError("pth_flash_attn: " + _windowed_refusal("non-causal attention", self.head_size))
        if getattr(cam, "rswa_prefix_lens", None) is not None:
            raise NotImplementedError("pth_flash_attn: R-SWA is not supported")
        doc_ranges = getattr(cam, "mm_req_doc_ranges", None)
        if doc_ranges and any(doc_ranges.values()):
            raise NotImplementedError("pth_flash_attn: bidirectional multimodal prefix ranges are not supported")

        decodes, prefills, decode_tokens, _ = split_decodes_and_prefills(
            cam, decode_threshold=self.reorder_batch_threshold or 1)
        decodes, decode_tokens = int(decodes), int(decode_tokens)
        requests, tokens = int(cam.num_reqs), int(cam.num_actual_tokens)
        calls = []
        if decodes > 0 and decode_tokens > 0:
            if prefills == 0:
                longest = int(cam.max_query_len)
            else:  # bound of the decode part alone, from the HOST copy of the starts (no sync)
                host = cam.query_start_loc_cpu
                longest = int((host[1:decodes + 1] - host[:decodes]).max())
            calls.append(self._call(cam, slice(0, decodes), slice(0, decode_tokens), max(longest, 1), False))
        if prefills > 0 and tokens > decode_tokens:
            calls.append(self._call(cam, slice(decodes, requests), slice(decode_tokens, tokens),
                                    int(cam.max_query_len), True))
        return PthAttnMetadata(
            num_actual_tokens=tokens, max_query_len=int(cam.max_query_len), query_start_loc=cam.query_start_loc,
            max_seq_len=int(cam.max_seq_len), seq_lens=cam.seq_lens, block_table=cam.block_table_tensor,
            slot_mapping=cam.slot_mapping, causal=causal, calls=tuple(calls))

    def build_for_cudagraph_capture(self, common_attn_metadata: CommonAttentionMetadata) -> PthAttnMetadata:
        """As :meth:`build`; lengths of 1 keep the capture run short (the plan ignores them)."""
        metadata = self.build(0, common_attn_metadata)
        metadata.seq_lens.fill_(1)
        return metadata

    def update_draft_decode_metadata(self, _metadata: PthAttnMetadata) -> None:
        """Every step-dependent field is a persistent device buffer: nothing to refresh."""


# --------------------------------------------------------------------------
# backend and implementation
# --------------------------------------------------------------------------
class PthFlashAttnBackend(TritonAttentionBackend):
    """``CUSTOM``: vLLM's cache format and writer, this library's reader."""

    supported_dtypes: ClassVar[list[torch.dtype]] = [torch.float16, torch.bfloat16]
    supported_kv_cache_dtypes: ClassVar[list] = [KV_CACHE_DTYPE]

    @staticmethod
    def get_name() -> str:
        return BACKEND_NAME

    @staticmethod
    def get_impl_cls() -> type["PthFlashAttnImpl"]:
        return PthFlashAttnImpl

    @staticmethod
    def get_builder_cls() -> type[PthFlashAttnMetadataBuilder]:
        return PthFlashAttnMetadataBuilder

    @staticmethod
    def get_supported_kernel_block_sizes(kv_cache_spec: Any = None) -> list:
        return [MultipleOf(KERNEL_BLOCK_MULTIPLE)]

    @classmethod
    def supports_block_size(cls, block_size: int | None) -> bool:
        return block_size is None or block_size % KERNEL_BLOCK_MULTIPLE == 0

    @classmethod
    def supports_head_size(cls, head_size: int) -> bool:
        return head_size in planner.SUPPORTED_HEAD_SIZES

    @classmethod
    def supports_attn_type(cls, attn_type: str) -> bool:
        return attn_type == AttentionType.DECODER

    @classmethod
    def supports_non_causal(cls) -> bool:
        return True   # at the windowed head sizes; validate_configuration refuses the others

    @classmethod
    def supports_sliding_window(cls) -> bool:
        return True   # as above

    @classmethod
    def supports_rswa(cls) -> bool:
        return False

    @classmethod
    def supports_sink(cls) -> bool:
        return False

    @classmethod
    def supports_mm_prefix(cls) -> bool:
        return False

    @classmethod
    def supports_alibi_sqrt(cls) -> bool:
        return False

    @classmethod
    def supports_batch_invariance(cls) -> bool:
        return False  # how a request is cut into pieces depends on the rest of the batch

    @classmethod
    def supports_compute_capability(cls, capability: Any) -> bool:
        return capability.major == SUPPORTED_CC_MAJOR and ops.is_available()

    @classmethod
    def validate_configuration(cls, *args: Any, **kwargs: Any) -> list[str]:
        """vLLM's reasons plus the head-size condition of windows and non-causal attention."""
        base = super().validate_configuration
        reasons = list(base(*args, **kwargs))
        bound = inspect.signature(base).bind(*args, **kwargs)
        bound.apply_defaults()
        given = bound.arguments
        head_size = given.get("head_size")
        if head_size in planner.SUPPORTED_HEAD_SIZES and head_size not in planner.WINDOWED_HEAD_SIZES:
            if given.get("has_sliding_window"):
                reasons.append(_windowed_refusal("sliding window", head_size))
            if given.get("use_non_causal"):
                reasons.append(_windowed_refusal("non-causal attention", head_size))
        return reasons


class PthFlashAttnImpl(TritonAttentionImpl):
    """Reads the cache with ``pth_flash_attn_fwd``; writes it exactly as the Triton backend does."""

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                 alibi_slopes: list[float] | None, sliding_window: int | None, kv_cache_dtype: str,
                 logits_soft_cap: float | None = None, attn_type: str = AttentionType.DECODER,
                 kv_sharing_target_layer_name: str | None = None, sinks: torch.Tensor | None = None,
                 use_alibi_sqrt: bool = False, chunk_lookback: int = -1) -> None:
        refused = []
        if alibi_slopes is not None or use_alibi_sqrt:
            refused.append("ALiBi")
        if sliding_window is not None and sliding_window < 1:
            refused.append(f"sliding window {sliding_window}")
        elif sliding_window is not None and head_size not in planner.WINDOWED_HEAD_SIZES:
            refused.append(_windowed_refusal("sliding window", head_size))
        if logits_soft_cap:
            refused.append("logits soft cap")
        if sinks is not None:
            refused.append("attention sinks")
        if chunk_lookback != -1:
            refused.append("chunk lookback")
        if attn_type != AttentionType.DECODER:
            refused.append(f"attention type {attn_type}")
        if kv_cache_dtype != KV_CACHE_DTYPE:
            refused.append(f"kv_cache_dtype {kv_cache_dtype}")
        if head_size not in planner.SUPPORTED_HEAD_SIZES:
            refused.append(f"head size {head_size}")
        if refused:  # before anything is reserved: a wrong selection fails at load with its reasons
            raise NotImplementedError("pth_flash_attn does not support: " + ", ".join(refused))
        _heads_per_kv(num_heads, num_kv_heads)
        super().__init__(num_heads, head_size, scale, num_kv_heads, alibi_slopes, sliding_window, kv_cache_dtype,
                         logits_soft_cap, attn_type, kv_sharing_target_layer_name, sinks, use_alibi_sqrt,
                         chunk_lookback)
        if getattr(self, "dcp_world_size", 1) > 1 or getattr(self, "pcp_world_size", 1) > 1:
            raise NotImplementedError("pth_flash_attn: DCP / PCP are not supported")
        if self._kv_quant_mode != KVQuantMode.INT8_PER_TOKEN_HEAD:
            raise NotImplementedError("pth_flash_attn: int8_per_token_head only")
        self.supports_quant_query_input = False   # the query stays 16-bit
        self.window = int(sliding_window or 0)    # (vLLM's own field is a (left, right) pair)
        self._views: tuple[int, tuple[torch.Tensor, ...]] | None = None
        self._ws_token_splits = 0
        self._no_workspace: torch.Tensor | None = None
        self._reserve_workspace(get_current_vllm_config_or_none())

    def _reserve_workspace(self, vllm_config: VllmConfig | None) -> None:
        """Reserve the split workspace now, while vLLM is still measuring the model's memory."""
        if vllm_config is None or not is_workspace_manager_initialized():
            return
        self._ws_token_splits = reserved_token_splits(vllm_config, num_kv_heads=self.num_kv_heads,
                                                      head_size=self.head_size, num_sms=_num_sms())
        o_shape, lse_shape = planner.workspace_shapes(ws_token_splits=self._ws_token_splits, Hq=self.num_heads,
                                                      D=self.head_size)
        ws_o, _ = current_workspace_manager().get_simultaneous((o_shape, torch.float32), (lse_shape, torch.float32))
        self._no_workspace = torch.empty(0, dtype=torch.float32, device=ws_o.device)
        logger.info("pth_flash_attn: reserved %d token-splits of split workspace (Hq=%d, D=%d, %.2f MiB)",
                    self._ws_token_splits, self.num_heads, self.head_size,
                    planner.workspace_bytes(ws_token_splits=self._ws_token_splits, Hq=self.num_heads,
                                            D=self.head_size) / 2 ** 20)

    def _caches(self, kv_cache: torch.Tensor) -> tuple[torch.Tensor, ...]:
        key = kv_cache.data_ptr()
        if self._views is None or self._views[0] != key:
            self._views = (key, cache_views(kv_cache, self.head_size))
        return self._views[1]

    def _run(self, call: OpCall, query: torch.Tensor, output: torch.Tensor, caches: tuple[torch.Tensor, ...],
             causal: bool) -> None:
        plan = call.plan
        if plan.num_splits > 1:
            if self._ws_token_splits and plan.ws_token_splits_used > self._ws_token_splits:
                raise RuntimeError(f"pth_flash_attn: launch needs {plan.ws_token_splits_used} token-splits, "
                                   f"{self._ws_token_splits} were reserved")
            ws_o, ws_lse = current_workspace_manager().get_simultaneous(
                (plan.ws_o_shape, torch.float32), (plan.ws_lse_shape, torch.float32))
        else:
            if self._no_workspace is None:
                self._no_workspace = torch.empty(0, dtype=torch.float32, device=query.device)
            ws_o = ws_lse = self._no_workspace
        whole = call.tokens.start == 0 and call.tokens.stop == query.shape[0]
        k, v, ks, vs = caches
        ops.pth_flash_attn_fwd(output if whole else output[call.tokens], query if whole else query[call.tokens],
                               k, v, ks, vs, call.block_table, call.seq_lens, call.query_start_loc,
                               call.max_query_len, plan.wm, plan.num_splits, self.scale, ws_o, ws_lse,
                               self.window, causal)

    def forward(self, layer: torch.nn.Module, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                kv_cache: torch.Tensor, attn_metadata: PthAttnMetadata | None, output: torch.Tensor,
                output_scale: torch.Tensor | None = None,
                output_block_scale: torch.Tensor | None = None) -> torch.Tensor:
        """The step's op calls (at most two), writing ``output`` in place.  ``key`` / ``value``
        are unused: the cache is written by ``do_kv_cache_update``."""
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("pth_flash_attn: fused output quantisation is not supported")
        if attn_metadata is None:   # vLLM's memory-profile run
            return output.fill_(0)
        caches = self._caches(kv_cache)
        for call in attn_metadata.calls:
            self._run(call, query, output, caches, attn_metadata.causal)
        return output
