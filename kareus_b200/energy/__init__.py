"""Online energy plane: NVML access, measurement windows, samplers, clock control, plan server."""
from .nvml import FakeNVML, RealNVML, NVMLError, get_nvml
from .monitor import EnergyMonitor, Measurement, Trial, measure
from .freq_controller import FrequencyController
from .pfo import PFOServer, PipelineFrequencyOptimizer, PointSolution
from .power import EnergyPoller, GpuStatsMonitor, PowerMonitor
