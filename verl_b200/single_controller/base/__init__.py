from .decorator import Dispatch, Execute, register  # noqa: F401
from .worker import Worker  # noqa: F401
from .worker_group import (ClassWithInitArgs, ResourcePool, ResourcePoolManager, SubResourcePool, WorkerGroup,  # noqa: F401
                           merge_resource_pool, split_resource_pool)
