"""Speaker-label model entry point (reference module path ``models/label_models.py``)."""
from .classification_models import EncDecSpeakerLabelModel  # noqa: F401
