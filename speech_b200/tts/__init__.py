"""Text-to-speech collection: audio codec, MagpieTTS, the classic FastPitch / HiFi-GAN / aligner stack and G2P."""
from .audio_codec import AudioCodecModel  # noqa: F401
from .classic import AlignerModel, DictG2p, FastPitchModel, HifiGanModel, PhonemeTokenizer  # noqa: F401
from .magpietts import MagpieTTSModel  # noqa: F401
