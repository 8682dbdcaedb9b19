from . import reference  # noqa: F401
from .collectives import all_gather, all_reduce, all_reduce_rmsnorm, reduce_scatter  # noqa: F401
