"""Distributed backends (single / DDP / FSDP) behind the reference's backend protocol."""
from .backends import (BACKEND_TYPE_TO_MODULE_MAP, DDPBackend, DistributedBackend, FSDPBackend,
                       SingleBackend, make_backend_from_args, registered_backends)

__all__ = ["BACKEND_TYPE_TO_MODULE_MAP", "DDPBackend", "DistributedBackend", "FSDPBackend", "SingleBackend",
           "make_backend_from_args", "registered_backends"]
