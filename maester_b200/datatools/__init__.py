"""Offline data tooling: ingestion, shuffling/splitting, token statistics and inspection.

The reference keeps these as stand-alone scripts under ``scripts/``; here the logic is importable
(and tested) and the scripts of the same names are thin command-line wrappers.
"""
