from .worker_group import ProcessWorkerGroup, create_colocated_worker_cls  # noqa: F401
