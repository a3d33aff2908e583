"""Hugging Face ``transformers`` model classes for serving checkpoints trained here."""
