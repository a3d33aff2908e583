"""Registers the MoE model families in the registries of ``maester_b200.models``."""
from maester_b200 import models as _m
from maester_b200.models.deepseek import DeepSeekModel, build_deepseek_optimizers, deepseek_configs
from maester_b200.models.glm4 import Glm4MoeTextModel, glm4_configs
from maester_b200.parallel.parallelize import parallelize_deepseek

_m.models_config.update({"deepseek": deepseek_configs, "glm4": glm4_configs})
_m.model_name_to_cls.update({"deepseek": DeepSeekModel, "glm4": Glm4MoeTextModel})
_m.model_name_to_parallelize.update({"deepseek": parallelize_deepseek, "glm4": parallelize_deepseek})
_m.model_name_to_optimizers_builder.update({"deepseek": build_deepseek_optimizers, "glm4": build_deepseek_optimizers})
