"""yali_b200: a Blackwell-native low-latency all-reduce library (one-shot Flash,
two-shot Stream, NVLS multimem and fused tensor-parallel kernels for sm_100a) with
a thin PyTorch layer.

    import yali_b200 as yali
    comm = yali.init_process_group()          # one GPU per process (torchrun)
    y = yali.all_reduce(x)                    # CUDA tensor: native kernels; CPU tensor: gloo
"""
from .parallel.comm import (Comm, destroy_process_group, get_default_comm, init_process_group)  # noqa: F401
from .ops.collectives import (all_gather, all_reduce, all_reduce_host, all_reduce_rmsnorm,  # noqa: F401
                              fused_linear_rmsnorm, reduce_scatter)  # noqa: F401
from .ops import reference  # noqa: F401

__version__ = "0.1.0"
