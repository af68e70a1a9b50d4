"""Graph-mode configuration of the platform.

On B200 a decode step is a CUDA graph; there is no tracing compiler on the hot path.  What
remains configurable is which batch sizes are captured ("gears"), how a batch is padded to
a gear, and whether prefill bypasses graphs (it always does: it is ragged and
compute-bound).  ``B200CompilationConfig`` carries that and validates it once, in place of
the reference's ``NPUCompilationConfig`` with its GE / torchair switches
(omni_npu/compilation/ge_compile_config.py:17-106).
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional

MAX_GEAR_NUM = 64


@dataclass
class B200CompilationConfig:
    cudagraph_mode: str = "FULL_DECODE_ONLY"        # NONE | FULL_DECODE_ONLY
    decode_gear_list: List[int] = field(default_factory=list)    # captured decode batch sizes
    max_capture_size: int = 256
    bypass_prefill: bool = True
    graph_debug: bool = False                       # check that input addresses do not move

    @classmethod
    def from_additional_config(cls, additional: Optional[Mapping[str, Any]], max_num_seqs: int = 256
                               ) -> "B200CompilationConfig":
        d: Dict[str, Any] = dict((additional or {}).get("graph_config", additional or {}))
        cfg = cls(cudagraph_mode=d.get("cudagraph_mode", "FULL_DECODE_ONLY"),
                  decode_gear_list=sorted(set(int(x) for x in d.get("decode_gear_list", []))),
                  max_capture_size=int(d.get("max_capture_size", 256)),
                  bypass_prefill=bool(d.get("bypass_prefill", True)),
                  graph_debug=bool(d.get("graph_debug", False)))
        cfg.validate(max_num_seqs)
        return cfg

    def validate(self, max_num_seqs: int) -> None:
        if self.cudagraph_mode not in ("NONE", "FULL_DECODE_ONLY"):
            raise ValueError(f"unknown cudagraph_mode {self.cudagraph_mode!r}")
        if len(self.decode_gear_list) > MAX_GEAR_NUM:
            raise ValueError(f"at most {MAX_GEAR_NUM} decode gears, got {len(self.decode_gear_list)}")
        if any(g <= 0 for g in self.decode_gear_list):
            raise ValueError("decode gears must be positive")
        if self.decode_gear_list and self.decode_gear_list[-1] < max_num_seqs:
            # the largest gear must cover a full batch, as the reference insists
            self.decode_gear_list.append(max_num_seqs)

    def gears(self, max_num_seqs: int) -> List[int]:
        """The batch sizes to capture: the configured gears, or 1, 2, 4, 8, then steps of 8 /
        16 up to the largest batch."""
        if self.cudagraph_mode == "NONE":
            return []
        if self.decode_gear_list:
            return [g for g in self.decode_gear_list if g <= max(max_num_seqs, 1)] or [max_num_seqs]
        sizes, s = [], 1
        top = min(max_num_seqs, self.max_capture_size)
        while s < top:
            sizes.append(s)
            s = s * 2 if s < 8 else s + 8 if s < 64 else s + 16
        sizes.append(top)
        return sizes

    def pad_to_gear(self, batch_size: int, gears: List[int]) -> Optional[int]:
        """Smallest gear that holds the batch, or None (run eagerly)."""
        i = bisect.bisect_left(gears, batch_size)
        return gears[i] if i < len(gears) else None
