"""Agents built from the framework's streaming models."""
from .voice_agent import Pipeline, build_voice_agent  # noqa: F401
