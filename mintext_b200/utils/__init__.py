from .filesize import parse_file_size
from .logging import MetricLogger
from .profiling import Profiler
from .pytree import calculate_tflops_per_device, calculate_tokens_per_device, check_nan, count_params

__all__ = ["MetricLogger", "Profiler", "count_params", "check_nan", "calculate_tflops_per_device",
           "calculate_tokens_per_device", "parse_file_size"]
