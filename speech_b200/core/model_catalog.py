"""Catalogue of published checkpoints by name, and their resolution to local files.

The reference lists its checkpoints per model class (``list_available_models`` returning ``PretrainedModelInfo`` records with an
NGC URL, e.g. ``asr/models/ctc_models.py``, ``asr/models/rnnt_bpe_models.py``, ``asr/models/label_models.py``) and downloads them
on ``from_pretrained``.  Here the names are kept in one table and resolved offline: a name maps to
``<cache>/<name>.nemo``, ``<cache>/<name>/<name>.nemo`` or a Hugging Face snapshot in the local hub cache, where ``<cache>`` is
``$NEMO_CACHE_DIR`` (or ``~/.cache/speech_b200``).  ``fetch`` uses a caller-supplied downloader so that deployments with network
access can fill the cache; nothing here opens a connection by itself.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

__all__ = ["CatalogEntry", "CATALOG", "cache_dir", "entries_for_class", "fetch", "resolve_local", "search"]

_NGC = "https://api.ngc.nvidia.com/v2/models/nvidia/nemo/{name}/versions/{version}/files/{name}.nemo"


@dataclass(frozen=True)
class CatalogEntry:
    name: str
    class_name: str
    description: str
    hf_id: Optional[str] = None
    version: str = "1.0.0"

    @property
    def location(self) -> str:
        return _NGC.format(name=self.name, version=self.version)


def _e(name, cls, desc, hf=None, version="1.0.0"):
    return CatalogEntry(name, cls, desc, hf, version)


CATALOG: List[CatalogEntry] = [
    # CTC
    _e("stt_en_conformer_ctc_small", "EncDecCTCModelBPE", "Conformer-CTC small, English", "nvidia/stt_en_conformer_ctc_small"),
    _e("stt_en_conformer_ctc_large", "EncDecCTCModelBPE", "Conformer-CTC large, English", "nvidia/stt_en_conformer_ctc_large"),
    _e("stt_en_fastconformer_ctc_large", "EncDecCTCModelBPE", "FastConformer-CTC large, English", "nvidia/stt_en_fastconformer_ctc_large"),
    _e("parakeet-ctc-0.6b", "EncDecCTCModelBPE", "FastConformer-CTC XL, English", "nvidia/parakeet-ctc-0.6b"),
    _e("parakeet-ctc-1.1b", "EncDecCTCModelBPE", "FastConformer-CTC XXL, English", "nvidia/parakeet-ctc-1.1b"),
    _e("QuartzNet15x5Base-En", "EncDecCTCModel", "QuartzNet 15x5, English characters", None, "1.0.0rc1"),
    _e("stt_en_jasper10x5dr", "EncDecCTCModel", "Jasper 10x5 dense residual, English characters"),
    _e("stt_en_citrinet_1024", "EncDecCTCModelBPE", "Citrinet-1024, English"),
    # transducer
    _e("stt_en_conformer_transducer_large", "EncDecRNNTBPEModel", "Conformer-Transducer large, English", "nvidia/stt_en_conformer_transducer_large"),
    _e("stt_en_fastconformer_transducer_large", "EncDecRNNTBPEModel", "FastConformer-Transducer large, English", "nvidia/stt_en_fastconformer_transducer_large"),
    _e("parakeet-rnnt-0.6b", "EncDecRNNTBPEModel", "FastConformer-Transducer XL, English", "nvidia/parakeet-rnnt-0.6b"),
    _e("parakeet-rnnt-1.1b", "EncDecRNNTBPEModel", "FastConformer-Transducer XXL, English", "nvidia/parakeet-rnnt-1.1b"),
    _e("parakeet-tdt-1.1b", "EncDecRNNTBPEModel", "FastConformer-TDT XXL, English", "nvidia/parakeet-tdt-1.1b"),
    _e("parakeet-tdt-0.6b-v2", "EncDecRNNTBPEModel", "FastConformer-TDT XL, English with punctuation and timestamps", "nvidia/parakeet-tdt-0.6b-v2"),
    _e("parakeet-tdt-0.6b-v3", "EncDecRNNTBPEModel", "FastConformer-TDT XL, 25 European languages", "nvidia/parakeet-tdt-0.6b-v3"),
    _e("stt_en_contextnet_1024", "EncDecRNNTBPEModel", "ContextNet-1024 transducer, English"),
    # hybrid
    _e("stt_en_fastconformer_hybrid_large_pc", "EncDecHybridRNNTCTCBPEModel", "FastConformer hybrid Transducer-CTC large with punctuation and capitalisation",
       "nvidia/stt_en_fastconformer_hybrid_large_pc"),
    _e("stt_en_fastconformer_hybrid_large_streaming_multi", "EncDecHybridRNNTCTCBPEModel", "cache-aware streaming FastConformer hybrid, several look-aheads",
       "nvidia/stt_en_fastconformer_hybrid_large_streaming_multi"),
    _e("parakeet-tdt_ctc-110m", "EncDecHybridRNNTCTCBPEModel", "FastConformer hybrid TDT-CTC 110M, English", "nvidia/parakeet-tdt_ctc-110m"),
    _e("parakeet-tdt_ctc-1.1b", "EncDecHybridRNNTCTCBPEModel", "FastConformer hybrid TDT-CTC XXL, English", "nvidia/parakeet-tdt_ctc-1.1b"),
    # attention encoder-decoder
    _e("canary-1b", "EncDecMultiTaskModel", "FastConformer + Transformer decoder, ASR and translation en/de/es/fr", "nvidia/canary-1b"),
    _e("canary-1b-flash", "EncDecMultiTaskModel", "Canary with a shallow decoder, 1B", "nvidia/canary-1b-flash"),
    _e("canary-180m-flash", "EncDecMultiTaskModel", "Canary with a shallow decoder, 180M", "nvidia/canary-180m-flash"),
    _e("canary-1b-v2", "EncDecMultiTaskModel", "Canary, 25 European languages", "nvidia/canary-1b-v2"),
    # speech LM
    _e("canary-qwen-2.5b", "SALM", "FastConformer encoder + Qwen LM with LoRA", "nvidia/canary-qwen-2.5b"),
    # speaker, diarization, VAD, classification
    _e("titanet_large", "EncDecSpeakerLabelModel", "TitaNet-L speaker embeddings", "nvidia/speakerverification_en_titanet_large"),
    _e("titanet_small", "EncDecSpeakerLabelModel", "TitaNet-S speaker embeddings"),
    _e("speakerverification_speakernet", "EncDecSpeakerLabelModel", "SpeakerNet verification"),
    _e("ecapa_tdnn", "EncDecSpeakerLabelModel", "ECAPA-TDNN speaker embeddings"),
    _e("langid_ambernet", "EncDecSpeakerLabelModel", "AmberNet spoken language identification", "nvidia/lang_id_ambernet"),
    _e("diar_sortformer_4spk-v1", "SortformerEncLabelModel", "Sortformer diarizer, up to 4 speakers", "nvidia/diar_sortformer_4spk-v1"),
    _e("diar_streaming_sortformer_4spk-v2", "SortformerEncLabelModel", "streaming Sortformer diarizer with speaker cache", "nvidia/diar_streaming_sortformer_4spk-v2"),
    _e("vad_multilingual_marblenet", "EncDecClassificationModel", "MarbleNet voice activity detection, multilingual"),
    _e("vad_multilingual_frame_marblenet", "EncDecFrameClassificationModel", "frame-level MarbleNet VAD", "nvidia/frame_vad_multilingual_marblenet_v2.0"),
    _e("commandrecognition_en_matchboxnet3x1x64_v2", "EncDecClassificationModel", "MatchboxNet speech commands"),
    # self-supervised
    _e("ssl_en_conformer_large", "SpeechEncDecSelfSupervisedModel", "Conformer large, contrastive + MLM pre-training"),
    _e("ssl_en_nest_large_v1.0", "EncDecDenoiseMaskedTokenPredModel", "NEST large self-supervised FastConformer", "nvidia/ssl_en_nest_large_v1.0"),
    # TTS and codecs
    _e("magpie_tts_multilingual_357m", "MagpieTTSModel", "MagpieTTS multilingual", "nvidia/magpie_tts_multilingual_357m"),
    _e("nemo-nano-codec-22khz-1.89kbps-21.5fps", "AudioCodecModel", "FSQ audio codec, 22.05 kHz, 8 codebooks", "nvidia/nemo-nano-codec-22khz-1.89kbps-21.5fps"),
    _e("audio_codec_22khz", "AudioCodecModel", "audio codec 22.05 kHz"),
    _e("mel_codec_44khz_medium", "AudioCodecModel", "mel codec 44.1 kHz"),
    _e("tts_en_fastpitch", "FastPitchModel", "FastPitch, LJSpeech"),
    _e("tts_en_hifigan", "HifiGanModel", "HiFi-GAN vocoder, LJSpeech"),
]

_BY_NAME: Dict[str, CatalogEntry] = {e.name: e for e in CATALOG}


def cache_dir() -> str:
    return os.environ.get("NEMO_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "speech_b200")


def entries_for_class(cls) -> List[CatalogEntry]:
    """Entries of exactly this class, as in the reference where each class lists its own checkpoints; the abstract ``ASRModel``
    answers for all its subclasses (its listing is what ``ASRModel.from_pretrained(name)`` dispatches on)."""
    if cls.__name__ == "ASRModel":
        subs, stack = set(), [cls]
        while stack:
            c = stack.pop()
            subs.add(c.__name__)
            stack.extend(c.__subclasses__())
        return [e for e in CATALOG if e.class_name in subs]
    return [e for e in CATALOG if e.class_name == cls.__name__]


def search(text: str) -> List[CatalogEntry]:
    t = text.lower()
    return [e for e in CATALOG if t in e.name.lower() or t in e.description.lower()]


def resolve_local(name: str) -> Optional[str]:
    """Path of the checkpoint called ``name`` (catalogue name or its Hugging Face id) if it is on this machine, else ``None``."""
    entry = _BY_NAME.get(name) or next((e for e in CATALOG if e.hf_id == name), None)
    base = entry.name if entry is not None else name.split("/")[-1]
    root = cache_dir()
    for cand in (os.path.join(root, f"{base}.nemo"), os.path.join(root, base, f"{base}.nemo"), os.path.join(root, base)):
        if os.path.isfile(cand) or (os.path.isdir(cand) and os.path.exists(os.path.join(cand, "model_config.yaml"))):
            return cand
    hf_id = entry.hf_id if entry is not None else (name if "/" in name else None)
    if hf_id:
        try:
            from huggingface_hub import snapshot_download

            snap = snapshot_download(repo_id=hf_id, local_files_only=True)
        except Exception:
            return None
        nemo = sorted(f for f in os.listdir(snap) if f.endswith(".nemo"))
        return os.path.join(snap, nemo[0]) if nemo else snap
    return None


def fetch(name: str, downloader: Callable[[str, str], None]) -> str:
    """Fills the cache: ``downloader(url, destination_path)`` is called once when the file is not there yet."""
    entry = _BY_NAME[name]
    dest = os.path.join(cache_dir(), f"{entry.name}.nemo")
    if not os.path.exists(dest):
        os.makedirs(os.path.dirname(dest), exist_ok=True)
        tmp = dest + ".part"
        downloader(entry.location, tmp)
        os.replace(tmp, dest)
    return dest
