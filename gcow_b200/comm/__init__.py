from .allreduce import CompressedAllReduce, CollectiveTimeout, nccl_allreduce_mean
from .oracle import allreduce_oracle, protocol_model

__all__ = ["CompressedAllReduce", "CollectiveTimeout", "nccl_allreduce_mean", "allreduce_oracle",
           "protocol_model"]
