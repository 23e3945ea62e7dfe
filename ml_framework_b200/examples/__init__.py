"""Runnable examples: higher-order derivatives and quantization workflows."""
