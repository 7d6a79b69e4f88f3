"""Quantization op group: ``nvfp4``, ``mxfp8``."""
