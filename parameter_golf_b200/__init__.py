"""parameter_golf_b200 — a Blackwell-native small-GPT training, export and evaluation framework.

Python is the orchestration layer; the hot path is hand-written sm_100a CUDA
(`parameter_golf_b200.ops.native`), one process per GPU.
"""
__version__ = "0.1.0"
