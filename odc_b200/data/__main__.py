"""``python -m odc_b200.data``: predicted idle share of lock-step vs per-rank microbatching on sampled minibatches."""
from .packing import report_main

report_main()
