"""Blackwell-native LM pretraining stack with the public surface of Jaxtitan."""

__version__ = "0.1.0"
