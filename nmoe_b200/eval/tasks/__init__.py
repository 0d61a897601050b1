"""Prompt construction and answer extraction of the generation tasks."""
from . import gpqa, gsm8k, humaneval, span  # noqa: F401

REGISTRY = {"gsm8k": gsm8k, "gpqa": gpqa, "humaneval": humaneval, "span": span}
