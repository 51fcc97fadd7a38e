from .ddp import GcowDDPState, compressed_allreduce_hook, wrap_ddp

__all__ = ["GcowDDPState", "compressed_allreduce_hook", "wrap_ddp"]
