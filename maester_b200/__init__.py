"""maester_b200: a Blackwell-native (sm_100a) LLM training framework.

Framework layer in PyTorch, hot paths in hand-written CUDA (``maester_b200/csrc``), one process per
GPU over ``torch.distributed``.  Public entry points mirror the reference project: ``train.py
jobs/<job>``, ``submit.py``, model registries in :mod:`maester_b200.models`.
"""
__version__ = "0.1.0"
