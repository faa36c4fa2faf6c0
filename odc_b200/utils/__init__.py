from .nvtx import nvtx_range, nvtx_record_function
from .clocks import ClockSampler
