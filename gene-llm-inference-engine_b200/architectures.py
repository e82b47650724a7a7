"""The architectures this engine can build, entered into the one registry.

Adding an architecture means: a typed configuration class with ``from_json``, ``to_json`` and
``model_spec`` (its config.json keys translated into parts), a weight plan (its tensor names mapped
onto the parameters of those parts), and one ``register_architecture`` call like the one below.
"""
from .config import Architecture, GekupelConfig, LlamaConfig, NipadraConfig, PinoraxConfig, FovezenConfig, register_architecture
from .weights.plan import gekupel_weight_plan, llama_weight_plan, nipadra_weight_plan, pinorax_weight_plan, fovezen_weight_plan

register_architecture(Architecture(
    name="LlamaForCausalLM", model_types=("llama",), config_class=LlamaConfig, weight_plan=llama_weight_plan))

register_architecture(Architecture(
    name="Nipadra", model_types=("nipadra",), config_class=NipadraConfig, weight_plan=nipadra_weight_plan))

register_architecture(Architecture(
    name="Gekupel", model_types=("gekupel",), config_class=GekupelConfig, weight_plan=gekupel_weight_plan))

register_architecture(Architecture(
    name="Pinorax", model_types=("pinorax",), config_class=PinoraxConfig, weight_plan=pinorax_weight_plan))

register_architecture(Architecture(
    name="Fovezen", model_types=("fovezen",), config_class=FovezenConfig, weight_plan=fovezen_weight_plan))
