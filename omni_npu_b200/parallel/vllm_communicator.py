"""vLLM device-communicator adapter.

vLLM creates one communicator per process group from the class path the platform returns
(``Platform.get_device_communicator_cls``).  ``B200VllmCommunicator`` derives from vLLM's
base class and forwards every collective to :class:`B200Communicator`, so model code running
under vLLM gets the peer-memory all-reduce (push / one-shot / two-shot kernels), the fused
all-reduce + residual + RMSNorm and the expert-parallel dispatch / combine kernels.
Counterpart of ``NPUCommunicator`` (omni_npu/distributed/communicator.py:23-284), which
vLLM loads the same way (omni_npu/platform.py:136-139).
"""
from __future__ import annotations

from typing import List, Optional, Union

import torch

from .. import compat
from .communicator import B200Communicator

if compat.vllm_available():
    from vllm.distributed.device_communicators.base_device_communicator import DeviceCommunicatorBase as _Base
else:                                                    # importable without vLLM (tests, docs)
    class _Base:                                         # type: ignore[no-redef]
        def __init__(self, cpu_group=None, device=None, device_group=None, unique_name: str = "", **kw) -> None:
            self.cpu_group, self.device, self.device_group, self.unique_name = cpu_group, device, device_group, unique_name


class B200VllmCommunicator(_Base):
    def __init__(self, cpu_group, device: Optional[torch.device] = None, device_group=None,
                 unique_name: str = "", **kw) -> None:
        try:
            super().__init__(cpu_group, device, device_group, unique_name, **kw)
        except TypeError:                                # older base signature
            super().__init__(cpu_group, device, device_group, unique_name)
        self.impl = B200Communicator(cpu_group, device, device_group, unique_name=unique_name)

    # ----------------------------------------------------------- collectives
    def all_reduce(self, input_: torch.Tensor) -> torch.Tensor:
        return self.impl.all_reduce(input_)

    def all_gather(self, input_: torch.Tensor, dim: int = -1) -> torch.Tensor:
        return self.impl.all_gather(input_, dim)

    def all_gatherv(self, input_: Union[torch.Tensor, List[torch.Tensor]], dim: int = 0,
                    sizes: Optional[List[int]] = None):
        return self.impl.all_gatherv(input_, dim, sizes)

    def reduce_scatter(self, input_: torch.Tensor, dim: int = -1) -> torch.Tensor:
        return self.impl.reduce_scatter(input_, dim)

    def reduce_scatterv(self, input_: torch.Tensor, dim: int = -1, sizes: Optional[List[int]] = None):
        return self.impl.reduce_scatterv(input_, dim, sizes)

    def gather(self, input_: torch.Tensor, dst: int = 0, dim: int = -1):
        return self.impl.gather(input_, dst, dim)

    def broadcast(self, input_: torch.Tensor, src: int = 0) -> torch.Tensor:
        return self.impl.broadcast(input_, src)

    def send(self, tensor: torch.Tensor, dst: Optional[int] = None) -> None:
        self.impl.send(tensor, dst)

    def recv(self, size: torch.Size, dtype: torch.dtype, src: Optional[int] = None) -> torch.Tensor:
        return self.impl.recv(size, dtype, src)

    def all_to_all(self, input_: torch.Tensor, scatter_dim: int = 0, gather_dim: int = -1,
                   scatter_sizes: Optional[List[int]] = None, gather_sizes: Optional[List[int]] = None):
        return self.impl.all_to_all(input_, scatter_dim, gather_dim, scatter_sizes, gather_sizes)

    # ---------------------------------------------------- expert parallelism
    def prepare_communication_buffer_for_model(self, model: torch.nn.Module) -> None:
        self.impl.prepare_communication_buffer_for_model(model)

    def dispatch(self, hidden_states: torch.Tensor, *args, **kw):
        return self.impl.dispatch(hidden_states, *args, **kw)

    def combine(self, hidden_states: torch.Tensor, *args, **kw):
        return self.impl.combine(hidden_states, *args, **kw)

    def destroy(self) -> None:
        self.impl.destroy()
