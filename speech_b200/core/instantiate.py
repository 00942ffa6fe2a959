"""Allow-listed ``_target_`` instantiation.

Model configs name their building blocks by dotted class path.  Only paths under an
allow-listed prefix are ever imported, so a config cannot execute arbitrary code
(reference: ``nemo/core/classes/common.py:118-332``).  Class paths written by the
reference framework (``nemo.collections.asr.modules.ConformerEncoder`` ...) are mapped to
this package's classes through ``TARGET_ALIASES`` so ``.nemo`` files load in both
directions.
"""
from __future__ import annotations

import importlib
from typing import Any, Callable, Dict

from .config import DictConfig, ListConfig, OmegaConf, to_container

ALLOWED_PREFIXES = ["speech_b200.", "torch.optim.", "torch.nn.", "torch.distributed.fsdp."]

# reference class path -> class path in this package
TARGET_ALIASES: Dict[str, str] = {}


def register_alias(reference_path: str, local_path: str) -> None:
    TARGET_ALIASES[reference_path] = local_path


def allow_prefix(prefix: str) -> None:
    if prefix not in ALLOWED_PREFIXES:
        ALLOWED_PREFIXES.append(prefix)


def _install_default_aliases() -> None:
    a = register_alias
    M = "speech_b200.modules."
    for ref in ("nemo.collections.asr.modules.", "nemo.collections.asr.modules.audio_preprocessing."):
        a(ref + "AudioToMelSpectrogramPreprocessor", M + "preprocessor.AudioToMelSpectrogramPreprocessor")
        a(ref + "SpectrogramAugmentation", M + "spec_augment.SpectrogramAugmentation")
        a(ref + "AudioToMFCCPreprocessor", M + "preprocessor.AudioToMFCCPreprocessor")
    a("nemo.collections.asr.modules.ConformerEncoder", M + "conformer_encoder.ConformerEncoder")
    a("nemo.collections.asr.modules.conformer_encoder.ConformerEncoder", M + "conformer_encoder.ConformerEncoder")
    a("nemo.collections.asr.modules.ConvASRDecoder", M + "ctc_decoder.ConvASRDecoder")
    a("nemo.collections.asr.modules.conv_asr.ConvASRDecoder", M + "ctc_decoder.ConvASRDecoder")
    a("nemo.collections.asr.modules.ConvASREncoder", M + "conv_asr.ConvASREncoder")
    a("nemo.collections.asr.modules.ConvASRDecoderClassification", M + "conv_asr.ConvASRDecoderClassification")
    a("nemo.collections.asr.modules.SpeakerDecoder", M + "conv_asr.SpeakerDecoder")
    a("nemo.collections.asr.modules.RNNTDecoder", M + "rnnt.RNNTDecoder")
    a("nemo.collections.asr.modules.rnnt.RNNTDecoder", M + "rnnt.RNNTDecoder")
    a("nemo.collections.asr.modules.RNNTJoint", M + "rnnt.RNNTJoint")
    a("nemo.collections.asr.modules.rnnt.RNNTJoint", M + "rnnt.RNNTJoint")
    a("nemo.collections.asr.modules.StatelessTransducerDecoder", M + "rnnt.StatelessTransducerDecoder")
    a("nemo.collections.asr.modules.SampledRNNTJoint", M + "rnnt.SampledRNNTJoint")
    a("nemo.collections.asr.modules.HATJoint", M + "rnnt.HATJoint")
    for ref, name in (("rnn_encoder.", "RNNEncoder"), ("lstm_decoder.", "LSTMDecoder"), ("transformer_encoder.", "TransformerEncoder"),
                      ("wav2vec_modules.", "ConvFeatureEncoder"), ("wav2vec_modules.", "Wav2VecTransformerEncoder"),
                      ("parallel_expert_encoder.", "ParallelExpertEncoder")):
        a("nemo.collections.asr.modules." + name, M + "extra_encoders." + name)
        a("nemo.collections.asr.modules." + ref + name, M + "extra_encoders." + name)
    a("nemo.collections.asr.modules.transformer.get_nemo_transformer", M + "transformer_nm.get_transformer")
    a("nemo.collections.asr.modules.transformer.transformer.TransformerDecoderNM", M + "transformer_nm.TransformerDecoderNM")
    a("nemo.collections.asr.modules.transformer.TransformerDecoderNM", M + "transformer_nm.TransformerDecoderNM")
    a("nemo.collections.asr.modules.transformer.TransformerEncoderNM", M + "transformer_nm.TransformerEncoderNM")
    a("nemo.collections.asr.parts.submodules.token_classifier.TokenClassifier", M + "transformer_nm.TokenClassifier")
    a("nemo.collections.common.parts.MultiLayerPerceptron", M + "transformer_nm.MultiLayerPerceptron")
    a("nemo.collections.asr.modules.SortformerModules", M + "sortformer.SortformerModules")
    a("nemo.collections.asr.modules.transformer.transformer_encoders.TransformerEncoder", M + "transformer.TransformerEncoder")
    a("nemo.collections.asr.losses.ctc.CTCLoss", "speech_b200.losses.ctc.CTCLoss")
    a("nemo.collections.asr.losses.rnnt.RNNTLoss", "speech_b200.losses.rnnt.RNNTLoss")
    a("nemo.collections.common.losses.SmoothedCrossEntropyLoss", "speech_b200.losses.cross_entropy.SmoothedCrossEntropyLoss")
    a("nemo.collections.common.losses.smoothed_cross_entropy.SmoothedCrossEntropyLoss",
      "speech_b200.losses.cross_entropy.SmoothedCrossEntropyLoss")
    MD = "speech_b200.models."
    a("nemo.collections.asr.models.EncDecCTCModel", MD + "ctc_models.EncDecCTCModel")
    a("nemo.collections.asr.models.EncDecCTCModelBPE", MD + "ctc_models.EncDecCTCModelBPE")
    a("nemo.collections.asr.models.ctc_models.EncDecCTCModel", MD + "ctc_models.EncDecCTCModel")
    a("nemo.collections.asr.models.ctc_bpe_models.EncDecCTCModelBPE", MD + "ctc_models.EncDecCTCModelBPE")
    a("nemo.collections.asr.models.EncDecRNNTModel", MD + "rnnt_models.EncDecRNNTModel")
    a("nemo.collections.asr.models.EncDecRNNTBPEModel", MD + "rnnt_models.EncDecRNNTBPEModel")
    a("nemo.collections.asr.models.rnnt_models.EncDecRNNTModel", MD + "rnnt_models.EncDecRNNTModel")
    a("nemo.collections.asr.models.rnnt_bpe_models.EncDecRNNTBPEModel", MD + "rnnt_models.EncDecRNNTBPEModel")
    a("nemo.collections.asr.models.EncDecHybridRNNTCTCModel", MD + "hybrid_models.EncDecHybridRNNTCTCModel")
    a("nemo.collections.asr.models.EncDecHybridRNNTCTCBPEModel", MD + "hybrid_models.EncDecHybridRNNTCTCBPEModel")
    a("nemo.collections.asr.models.hybrid_rnnt_ctc_models.EncDecHybridRNNTCTCModel", MD + "hybrid_models.EncDecHybridRNNTCTCModel")
    a("nemo.collections.asr.models.hybrid_rnnt_ctc_bpe_models.EncDecHybridRNNTCTCBPEModel",
      MD + "hybrid_models.EncDecHybridRNNTCTCBPEModel")
    a("nemo.collections.asr.models.EncDecMultiTaskModel", MD + "aed_models.EncDecMultiTaskModel")
    a("nemo.collections.asr.models.aed_multitask_models.EncDecMultiTaskModel", MD + "aed_models.EncDecMultiTaskModel")
    a("nemo.collections.asr.models.SortformerEncLabelModel", MD + "sortformer_models.SortformerEncLabelModel")
    a("nemo.collections.asr.models.EncDecSpeakerLabelModel", MD + "classification_models.EncDecSpeakerLabelModel")
    a("nemo.collections.asr.models.EncDecClassificationModel", MD + "classification_models.EncDecClassificationModel")
    for name, mod in (("EncDecFrameClassificationModel", "classification_models"), ("EncDecRegressionModel", "classification_models"),
                      ("SpeechEncDecSelfSupervisedModel", "ssl_models"), ("EncDecMaskedTokenPredModel", "ssl_models"),
                      ("EncDecDenoiseMaskedTokenPredModel", "ssl_models"), ("EncDecRNNTBPEModelWithPrompt", "asr_variants"),
                      ("EncDecHybridRNNTCTCBPEModelWithPrompt", "asr_variants"), ("EncDecRNNTBPEEOUModel", "asr_variants"),
                      ("EncDecHybridRNNTCTCBPEEOUModel", "asr_variants"), ("EncDecMultiTalkerRNNTBPEModel", "asr_variants"),
                      ("EncDecTransfModelBPE", "transformer_bpe_models"), ("ConfidenceEnsembleModel", "asr_variants"),
                      ("ClusteringDiarizer", "diarizers"), ("OnlineDiarizer", "diarizers")):
        a("nemo.collections.asr.models." + name, MD + mod + "." + name)
    for name in ("ConvASRDecoderReconstruction", "ECAPAEncoder", "ParallelConvASREncoder"):
        a("nemo.collections.asr.modules." + name, M + "conv_asr." + name)
    for name in ("RandomProjectionVectorQuantizer", "RandomBlockMasking", "MultiSoftmaxDecoder"):
        a("nemo.collections.asr.modules." + name, MD + "ssl_models." + name)
    a("nemo.collections.asr.losses.angularloss.AngularSoftmaxLoss", "speech_b200.losses.misc.AngularSoftmaxLoss")
    a("nemo.collections.asr.losses.AngularSoftmaxLoss", "speech_b200.losses.misc.AngularSoftmaxLoss")
    a("nemo.collections.asr.losses.bce_loss.BCELoss", "speech_b200.losses.misc.BCELoss")
    a("nemo.collections.asr.losses.ssl_losses.contrastive.ContrastiveLoss", "speech_b200.losses.misc.ContrastiveLoss")
    a("nemo.collections.asr.losses.ssl_losses.mlm.MLMLoss", "speech_b200.losses.misc.MLMLoss")
    a("nemo.collections.asr.losses.ssl_losses.mlm.MultiMLMLoss", "speech_b200.losses.misc.MultiMLMLoss")
    a("nemo.collections.speechlm2.models.SALM", "speech_b200.speechlm.salm.SALM")
    a("nemo.collections.tts.models.MagpieTTSModel", "speech_b200.tts.magpietts.MagpieTTSModel")
    a("nemo.collections.tts.models.AudioCodecModel", "speech_b200.tts.audio_codec.AudioCodecModel")
    a("nemo.core.optim.lr_scheduler.NoamAnnealing", "speech_b200.core.optim.lr_scheduler.NoamAnnealing")
    a("nemo.core.optim.lr_scheduler.CosineAnnealing", "speech_b200.core.optim.lr_scheduler.CosineAnnealing")


_install_default_aliases()


def resolve_target_path(path: str) -> str:
    return TARGET_ALIASES.get(path, path)


def is_allowed(path: str) -> bool:
    return any(path.startswith(p) for p in ALLOWED_PREFIXES)


def locate(path: str) -> Any:
    """Import the object named by a dotted path, after alias mapping and the allow-list check."""
    path = resolve_target_path(path)
    if not is_allowed(path):
        raise ValueError(
            f"Refusing to instantiate '{path}': not under an allow-listed prefix {ALLOWED_PREFIXES}. "
            f"Use speech_b200.core.instantiate.allow_prefix() to extend the list."
        )
    parts = path.split(".")
    for i in range(len(parts) - 1, 0, -1):
        try:
            obj = importlib.import_module(".".join(parts[:i]))
        except ModuleNotFoundError:
            continue
        for attr in parts[i:]:
            obj = getattr(obj, attr)
        return obj
    raise ImportError(f"Cannot locate '{path}'")


def instantiate(cfg: Any, *args: Any, _recursive_: bool = True, **overrides: Any) -> Any:
    """Build the object described by ``cfg`` (``{_target_: path, **kwargs}``)."""
    if cfg is None:
        return None
    if isinstance(cfg, (DictConfig, ListConfig)):
        cfg = to_container(cfg, resolve=True)
    if isinstance(cfg, list):
        return [instantiate(c) if isinstance(c, (dict, list)) else c for c in cfg]
    if not isinstance(cfg, dict):
        return cfg
    cfg = dict(cfg)
    target = cfg.pop("_target_", None)
    cfg.pop("_convert_", None)
    partial = cfg.pop("_partial_", False)
    recursive = cfg.pop("_recursive_", _recursive_)
    if target is None:
        if recursive:
            return {k: instantiate(v) if isinstance(v, dict) and "_target_" in v else v for k, v in cfg.items()}
        return cfg
    fn: Callable[..., Any] = locate(target) if isinstance(target, str) else target
    kwargs = {}
    for k, v in cfg.items():
        if recursive and isinstance(v, dict) and "_target_" in v:
            v = instantiate(v)
        elif recursive and isinstance(v, list):
            v = [instantiate(e) if isinstance(e, dict) and "_target_" in e else e for e in v]
        kwargs[k] = v
    kwargs.update(overrides)
    if partial:
        import functools

        return functools.partial(fn, *args, **kwargs)
    return fn(*args, **kwargs)


def safe_instantiate(cfg: Any, *args: Any, **kwargs: Any) -> Any:
    return instantiate(cfg, *args, **kwargs)


def from_config_dict(config: Any, **extra: Any) -> Any:
    """Build an object from the three config styles the reference accepts
    (``common.py:751-842``): ``_target_``; legacy ``cls`` + ``params``; ``target`` + cfg ctor."""
    if isinstance(config, (DictConfig,)):
        plain = to_container(config, resolve=True)
    else:
        plain = dict(config)
    if "_target_" in plain:
        return instantiate(plain, **extra)
    if "cls" in plain and "params" in plain:
        return locate(plain["cls"])(**plain["params"], **extra)
    if "target" in plain:
        cls = locate(plain["target"])
        return cls(cfg=OmegaConf.create(plain), **extra)
    raise ValueError(f"Config has no _target_/cls/target entry: {list(plain)}")
