from .base import ClassWithInitArgs, Dispatch, Execute, ResourcePool, Worker, WorkerGroup, register  # noqa: F401
