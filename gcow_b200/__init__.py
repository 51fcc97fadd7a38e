"""gcow_b200 – gradient compression on the wire for B200 (sm_100a).

Public surface:

* ``compress`` / ``decompress`` – ZFP float32 block codec (1-D blocks of 4 and
  2-D blocks of 4x4; fixed-rate, fixed-accuracy and fixed-precision modes) on
  CUDA tensors (hand-written kernels) or CPU tensors (C++ oracle).
* ``ZfpParams`` – the four codec parameters and their mode setters.
* ``CompressedAllReduce`` / ``ddp_comm_hook`` – fused compressed gradient
  all-reduce over NVLink peer memory and its DistributedDataParallel hook.
* ``GcowConfig`` – one configuration object (environment ``GCOW_*`` < CLI).
"""
from .config import GcowConfig
from .codec import (ZfpParams, compress, decompress, compressed_nbytes, max_compressed_nbytes,
                    Compressed)

__all__ = ["GcowConfig", "ZfpParams", "compress", "decompress", "compressed_nbytes",
           "max_compressed_nbytes", "Compressed"]

__version__ = "0.1.0"
