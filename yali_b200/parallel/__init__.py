from .comm import Comm, destroy_process_group, get_default_comm, init_process_group  # noqa: F401
