"""Communicator handles, the communication stream, domain-size queries and the device barrier
(reference: `deep_ep/comm/__init__.py`). The `HCCL*`/`hccl` names of the reference are kept as
aliases of the NCCL-flavoured names."""
from .barrier import barrier
from .handle import (
    CommHandle,
    HCCLCommHandle,
    NCCLCommHandle,
    destroy_all_managed_comm,
    destroy_all_managed_hccl_comm,
    get_comm_handle,
    get_hccl_comm_handle,
    get_logical_domain_size,
    get_physical_domain_size,
)
from .stream import get_comm_stream

__all__ = [
    'CommHandle', 'NCCLCommHandle', 'HCCLCommHandle', 'barrier', 'destroy_all_managed_comm',
    'destroy_all_managed_hccl_comm', 'get_comm_handle', 'get_hccl_comm_handle', 'get_comm_stream',
    'get_logical_domain_size', 'get_physical_domain_size',
]
