"""Model registries (reference: maester/models/__init__.py:17-51).

``models_config[name][flavor]`` → args dataclass, ``model_name_to_cls[name]`` → model class,
``model_name_to_parallelize[name]`` → ``fn(model, world_mesh, parallel_dims, cfg)``,
``model_name_to_optimizers_builder[name]`` → ``fn(model, cfg, parallel_dims)``.
"""
from maester_b200.models.gemma import GemmaTextModel, gemma3_configs
from maester_b200.models.llama import Transformer, llama2_configs, llama3_configs, mistral_configs
from maester_b200.optimizers.container import build_optimizers
from maester_b200.parallel.parallelize import parallelize_deepseek, parallelize_gemma, parallelize_llama

models_config = {
    "llama2": llama2_configs,
    "llama3": llama3_configs,
    "mistral": mistral_configs,
    "gemma3": gemma3_configs,
}
model_name_to_cls = {
    "llama2": Transformer,
    "llama3": Transformer,
    "mistral": Transformer,
    "gemma3": GemmaTextModel,
}
model_name_to_parallelize = {
    "llama2": parallelize_llama,
    "llama3": parallelize_llama,
    "mistral": parallelize_llama,
    "gemma3": parallelize_gemma,
}
model_name_to_optimizers_builder = {
    "llama2": build_optimizers,
    "llama3": build_optimizers,
    "mistral": build_optimizers,
    "gemma3": build_optimizers,
}

try:  # MoE families register themselves when their modules are importable
    from maester_b200.models import _moe_registry  # noqa: F401
except ImportError:
    pass
