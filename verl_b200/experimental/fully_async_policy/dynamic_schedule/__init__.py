"""Dynamic GPU scheduling between training and generation: policy registry, built-in policies, resource controller."""

from .base import DynamicScheduleContext, DynamicSchedulePolicyBase, build_policy, register_policy, registered_policies  # noqa: F401
from .controller import DynamicResourceController, ResourceState  # noqa: F401
from .policies import DefaultDynamicSchedulePolicy, FixedRatioDynamicSchedulePolicy, StaticFullyAsyncPolicy  # noqa: F401
