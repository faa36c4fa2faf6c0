from .dataset import BatchedDataset
from .packing import (balanced_partitions, bin_pack_decreasing, get_cost_fn, get_packing_function,
                      greedy_partition, imbalance_report, karmarkar_karp, rearrange_micro_batches)
from .synthetic import (LengthSpec, h2d_bytes, make_minibatch, make_minibatch_from_lengths, pack_microbatch,
                        sample_lengths, to_device)
