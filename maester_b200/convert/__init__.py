"""Checkpoint conversion between Hugging Face safetensors and this framework's DCP checkpoints.

The reference ships one hand-written script per model family and direction
(scripts/convert/{llama,gemma,deepseek,glm4}/{to,from}_dcp.py).  Here each family is ONE declarative
specification (``families.py``): a table of key patterns with ``{L}`` (layer) and ``{E}`` (expert)
placeholders plus invertible tensor transforms (RoPE row permutation, q/k/v fusion, expert stacking).
Both directions are derived from the same table, so a round trip is the identity by construction.

    to_native(family, hf_state_dict, hf_config)  -> {fqn: tensor}      (what ``{"model": ...}`` holds)
    to_hf(family, native_state_dict, arch)       -> {hf key: tensor}

``io.py`` reads and writes sharded safetensors and reads a DCP checkpoint without building the model.
"""
from maester_b200.convert.rules import FamilySpec, Rule, to_hf, to_native  # noqa: F401
from maester_b200.convert.families import FAMILIES, arch_from_hf_config, arch_from_model_args  # noqa: F401
