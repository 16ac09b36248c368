from .worker_group import SPMDWorkerGroup, init_spmd_process_group  # noqa: F401
