"""Backend names of the reference that map onto this framework's two engines.

The reference ships several third-party training runtimes behind the same ``BaseEngine`` contract (``veomni``,
``torchtitan``, ``automodel``, ``mindspeed``, ``fsdp_turbo``: ``verl/workers/engine/*/transformer_impl.py``). There is one
native runtime here, so configs that name those backends run on the engine with the equivalent parallelism: sharded
data parallel (+Ulysses, +expert parallel) for the FSDP-family names, tensor/pipeline parallel for the Megatron family.
"""

from verl_b200.workers.engine.base import EngineRegistry
from verl_b200.workers.engine.fsdp.engine import FSDPEngine, FSDPEngineWithValueHead

FSDP_FAMILY = ["veomni", "torchtitan", "automodel", "fsdp_turbo"]
MEGATRON_FAMILY = ["mindspeed", "mcore"]

EngineRegistry.register(model_type="language_model", backend=FSDP_FAMILY, device=["cuda", "cpu"])(FSDPEngine)
EngineRegistry.register(model_type="value_model", backend=FSDP_FAMILY, device=["cuda", "cpu"])(FSDPEngineWithValueHead)


def _register_megatron_family():
    from verl_b200.workers.engine.megatron.engine import MegatronEngine, MegatronEngineWithValueHead

    EngineRegistry.register(model_type="language_model", backend=MEGATRON_FAMILY, device=["cuda", "cpu"])(MegatronEngine)
    EngineRegistry.register(model_type="value_model", backend=MEGATRON_FAMILY, device=["cuda", "cpu"])(MegatronEngineWithValueHead)


_register_megatron_family()
