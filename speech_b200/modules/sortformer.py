"""Sortformer building blocks (reference module path ``modules/sortformer_modules.py``)."""
from ..models.sortformer_models import SortformerModules  # noqa: F401
