"""A small, whole inference engine for the GPT-2 style decoder, written for NVIDIA B200."""

__version__ = "0.1.0"
