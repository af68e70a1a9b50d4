"""Registration of the KV connector with vLLM's connector factory
(counterpart of omni_npu/connector/register.py:37-51).  The connector is
reachable as ``P2PKVConnector`` (GPU-to-GPU pulls) and ``HostPoolKVConnector`` (blocks
travel through a pinned host pool) and, for drop-in compatibility with launch scripts
written for the reference, as ``LLMDataDistConnector`` / ``OmniCacheConnector``."""
from __future__ import annotations

from .. import compat

CONNECTOR_NAMES = ("P2PKVConnector", "LLMDataDistConnector", "HostPoolKVConnector", "OmniCacheConnector")
MODULE = "omni_npu_b200.kv_transfer.vllm_connector"


def register_connectors() -> bool:
    if not compat.vllm_available():
        return False
    try:
        factory = compat.kv_connector_factory()
    except ImportError:
        return False
    ok = False
    for name in CONNECTOR_NAMES:
        try:
            registry = getattr(factory, "_registry", {})
            if name in registry:
                ok = True
                continue
            factory.register_connector(name, MODULE, "B200KVConnector")
            ok = True
        except Exception:
            pass
    return ok
