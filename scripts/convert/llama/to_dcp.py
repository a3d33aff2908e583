"""llama: Hugging Face safetensors -> DCP checkpoint (see maester_b200/convert/cli.py for the options)."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", ".."))

from maester_b200.convert.cli import to_dcp_main  # noqa: E402

if __name__ == "__main__":
    to_dcp_main("llama")
