"""Host-side memory hygiene before the training loop (reference: maester/memory.py:36-39)."""
import gc

import torch


def cleanup_before_training() -> None:
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
