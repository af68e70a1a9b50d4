"""KV connector in vLLM's v1 connector interface.

``B200KVConnector`` derives from ``KVConnectorBase_V1`` and maps its scheduler-side and
worker-side calls onto :class:`P2PKVConnector` (``kv_transfer/connector.py``): blocks are
pulled GPU-to-GPU over NVLink by the consumer, the producer only parks finished requests'
blocks until the consumer acknowledges the pull.  Registered with vLLM's factory under the
names ``P2PKVConnector`` and ``LLMDataDistConnector`` (``kv_transfer/register.py``), with the
same ``kv_transfer_params`` wire format as the reference
(omni_npu/connector/llmdatadist_connector_v1.py:85-90,284-290).
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Set, Tuple

import torch

from .. import compat
from ..config import CacheConfig, EngineConfig, KVTransferConfig, ParallelConfig
from .connector import ConnectorMetadata, P2PKVConnector

if compat.vllm_available():
    from vllm.distributed.kv_transfer.kv_connector.v1.base import (KVConnectorBase_V1, KVConnectorMetadata,
                                                                    KVConnectorRole)
else:
    class KVConnectorBase_V1:  # type: ignore[no-redef]
        def __init__(self, vllm_config=None, role=None, kv_cache_config=None) -> None:
            self._connector_metadata = None
            self._role = role

        @property
        def role(self):
            return self._role

    class KVConnectorMetadata:  # type: ignore[no-redef]
        pass

    class KVConnectorRole:  # type: ignore[no-redef]
        SCHEDULER, WORKER = 0, 1


class B200ConnectorMetadata(KVConnectorMetadata):
    def __init__(self, inner: ConnectorMetadata) -> None:
        self.inner = inner


def engine_config_from_vllm(vllm_config) -> EngineConfig:
    """The few fields the connector needs, taken from a vLLM config object."""
    kt = vllm_config.kv_transfer_config
    cache = getattr(vllm_config, "cache_config", None)
    par = getattr(vllm_config, "parallel_config", None)
    cfg = EngineConfig(
        cache=CacheConfig(block_size=int(getattr(cache, "block_size", 16) or 16)),
        parallel=ParallelConfig(tensor_parallel_size=int(getattr(par, "tensor_parallel_size", 1) or 1)),
        kv_transfer=KVTransferConfig(
            kv_connector=getattr(kt, "kv_connector", "P2PKVConnector"), kv_role=getattr(kt, "kv_role", None),
            kv_rank=getattr(kt, "kv_rank", 0), kv_parallel_size=getattr(kt, "kv_parallel_size", 1),
            kv_ip=getattr(kt, "kv_ip", "127.0.0.1"), kv_port=int(getattr(kt, "kv_port", 14579)),
            kv_connector_extra_config=dict(getattr(kt, "kv_connector_extra_config", {}) or {})),
        additional_config=dict(getattr(vllm_config, "additional_config", None) or {}))
    return cfg


class B200KVConnector(KVConnectorBase_V1):
    def __init__(self, vllm_config, role, kv_cache_config=None) -> None:
        try:
            super().__init__(vllm_config, role, kv_cache_config)
        except TypeError:                                 # older base: (vllm_config, role)
            super().__init__(vllm_config, role)
        if not hasattr(self, "role"):                     # vLLM's base exposes ``role`` as a read-only property
            self._role = role
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.impl = P2PKVConnector(engine_config_from_vllm(vllm_config),
                                   device if role == KVConnectorRole.WORKER else torch.device("cpu"))
        # the control endpoint / heartbeat thread start when the KV caches are registered

    # ------------------------------------------------------------ scheduler side
    def get_num_new_matched_tokens(self, request, num_computed_tokens: int) -> Tuple[Optional[int], bool]:
        return self.impl.get_num_new_matched_tokens(request, num_computed_tokens)

    def update_state_after_alloc(self, request, blocks, num_external_tokens: int) -> None:
        ids = blocks.get_block_ids()[0] if hasattr(blocks, "get_block_ids") else list(blocks)
        self.impl.update_state_after_alloc(request, list(ids), num_external_tokens)

    def build_connector_meta(self, scheduler_output) -> B200ConnectorMetadata:
        return B200ConnectorMetadata(self.impl.build_connector_meta(scheduler_output))

    def request_finished(self, request, block_ids) -> Tuple[bool, Optional[Dict[str, Any]]]:
        delay, params = self.impl.request_finished(request, list(block_ids))
        return bool(delay), params                        # True: vLLM frees the blocks when told (get_finished)

    # --------------------------------------------------------------- worker side
    def register_kv_caches(self, kv_caches: Dict[str, torch.Tensor]) -> None:
        # layer name -> cache tensor; keep the layer order stable on both instances
        self.impl.register_kv_caches([kv_caches[k] for k in sorted(kv_caches)])

    def start_load_kv(self, forward_context=None, **kwargs: Any) -> None:
        md = getattr(self, "_connector_metadata", None)
        if isinstance(md, B200ConnectorMetadata):
            self.impl.start_load_kv(md.inner)

    def wait_for_layer_load(self, layer_name: str) -> None:
        self.impl.wait_for_layer_load(layer_name)

    def save_kv_layer(self, layer_name: str, kv_layer: torch.Tensor, attn_metadata=None, **kwargs: Any) -> None:
        self.impl.save_kv_layer(layer_name, kv_layer, attn_metadata)

    def wait_for_save(self) -> None:
        self.impl.wait_for_save()

    def get_finished(self, finished_req_ids: Set[str]) -> Tuple[Optional[Set[str]], Optional[Set[str]]]:
        sending, recving = self.impl.get_finished()
        return sending or None, recving or None

    def shutdown(self) -> None:
        self.impl.close()
