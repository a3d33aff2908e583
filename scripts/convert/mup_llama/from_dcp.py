"""muP-trained Llama: DCP checkpoint -> Hugging Face ``mup_llama`` checkpoint.

The exported config carries the muP multipliers (``mup_input_alpha``, ``mup_output_alpha``,
``mup_width_mul``) and selects the ``mup_llama`` model type implemented in
``maester_b200/models/hf/modeling_mup_llama.py`` (reference: scripts/convert/llama/from_dcp_mup.py).
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", ".."))

from maester_b200.convert import cli  # noqa: E402
from maester_b200.convert import hf_config  # noqa: E402

if __name__ == "__main__":
    _orig = hf_config.hf_config_from_args
    cli.hf_config_from_args = lambda family, args, mup=False: _orig(family, args, mup=True)
    cli.from_dcp_main("llama")
