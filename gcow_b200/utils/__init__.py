from .logging import MetricsLogger, AverageMeter, ProgressMeter, accuracy
from .checkpoint import save_checkpoint, load_checkpoint
from .tracing import nvtx_range, PhaseTimer, sample_clocks, ClockSampler

__all__ = ["MetricsLogger", "AverageMeter", "ProgressMeter", "accuracy", "save_checkpoint",
           "load_checkpoint", "nvtx_range", "PhaseTimer", "sample_clocks", "ClockSampler"]
