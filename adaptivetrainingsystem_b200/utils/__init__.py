from .profiler import PhaseTimer, measured_peaks, roofline_fraction, time_cuda
from .environment import get_system_info, validate_environment, estimate_training_time, print_system_diagnostics
from .export_utils import export_for_inference  # noqa: E402,F401
