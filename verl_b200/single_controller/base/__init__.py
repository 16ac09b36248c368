from .decorator import Dispatch, Execute, register  # noqa: F401
from .worker import Worker  # noqa: F401
from .worker_group import ClassWithInitArgs, ResourcePool, WorkerGroup  # noqa: F401
