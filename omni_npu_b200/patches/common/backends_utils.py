"""``CommonAttentionMetadata.unpadded`` keeps the padded metadata.

vLLM trims the per-step attention metadata to the actual request / token counts before it hands
it to backends that do not run padded.  The attention backends of this package replay whole
decode steps as CUDA graphs captured at padded batch sizes and read lengths, slots and block
tables from device buffers of that padded size (padding rows carry slot -1 and length 0), so the
trimmed copy would describe other tensors than the captured kernels read.  The patch makes
``unpadded`` return the object unchanged.
(reference: omni_npu/vllm_patches/patches/common/patch_backends_utils.py:6-15)
"""
from __future__ import annotations

from ... import compat
from ..core import Patch, register_patch

if compat.vllm_available():
    try:
        from vllm.v1.attention.backends.utils import CommonAttentionMetadata as _Meta

        if hasattr(_Meta, "unpadded"):
            @register_patch("PaddedAttentionMetadataPatch", _Meta)
            class PaddedAttentionMetadataPatch(Patch):
                attributes = ["unpadded"]

                def unpadded(self, num_actual_tokens: int, num_actual_reqs: int):
                    return self
    except Exception:  # pragma: no cover - depends on the vLLM version
        pass
