"""Programmatic model configs for the FastConformer family.

Size table (d_model, heads, layers, conv kernel, prediction / joint width, LSTM layers) follows
``examples/asr/conf/fastconformer/fast-conformer_transducer_bpe.yaml:23-33`` of the reference; shared defaults:
``dw_striding`` 8x sub-sampling with 256 conv channels, ``ff_expansion_factor 4``, ``rel_pos`` attention with
untied biases, AdamW betas (0.9, 0.98) + Noam warm-up.  The YAML files under ``examples/asr/conf`` describe the
same models; these helpers exist so benchmarks and tests can build them without touching the file system.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

from ..core.config import DictConfig, OmegaConf

FASTCONFORMER_SIZES: Dict[str, Dict[str, Any]] = {
    "small": dict(d_model=176, n_heads=4, n_layers=16, conv_kernel_size=9, pred_hidden=320, pred_rnn_layers=1, xscaling=True),
    "medium": dict(d_model=256, n_heads=4, n_layers=16, conv_kernel_size=9, pred_hidden=640, pred_rnn_layers=1, xscaling=True),
    "large": dict(d_model=512, n_heads=8, n_layers=17, conv_kernel_size=9, pred_hidden=640, pred_rnn_layers=1, xscaling=True),
    "xlarge": dict(d_model=1024, n_heads=8, n_layers=24, conv_kernel_size=9, pred_hidden=640, pred_rnn_layers=2, xscaling=True),
    "xxlarge": dict(d_model=1024, n_heads=8, n_layers=42, conv_kernel_size=5, pred_hidden=640, pred_rnn_layers=2, xscaling=False),
}


def preprocessor_cfg(features: int = 80, sample_rate: int = 16000, dither: float = 1e-5, pad_to: int = 0) -> Dict[str, Any]:
    return {"_target_": "speech_b200.modules.preprocessor.AudioToMelSpectrogramPreprocessor", "sample_rate": sample_rate,
            "normalize": "per_feature", "window_size": 0.025, "window_stride": 0.01, "window": "hann",
            "features": features, "n_fft": 512, "frame_splicing": 1, "dither": dither, "pad_to": pad_to}


def encoder_cfg(size: str = "large", features: int = 80, dropout: float = 0.1, dropout_att: float = 0.1,
                n_layers: Optional[int] = None, causal: bool = False, att_context_size=None,
                att_context_style: str = "regular", conv_norm_type: str = "batch_norm", **over) -> Dict[str, Any]:
    s = dict(FASTCONFORMER_SIZES[size])
    cfg = {"_target_": "speech_b200.modules.conformer_encoder.ConformerEncoder", "feat_in": features, "feat_out": -1,
           "n_layers": n_layers or s["n_layers"], "d_model": s["d_model"], "subsampling": "dw_striding",
           "subsampling_factor": 8, "subsampling_conv_channels": 256, "causal_downsampling": causal,
           "ff_expansion_factor": 4, "self_attention_model": "rel_pos", "n_heads": s["n_heads"],
           "att_context_size": att_context_size or [-1, -1], "att_context_style": att_context_style,
           "xscaling": s["xscaling"], "untie_biases": True, "pos_emb_max_len": 5000,
           "conv_kernel_size": s["conv_kernel_size"], "conv_norm_type": conv_norm_type,
           "conv_context_size": "causal" if causal else None, "dropout": dropout, "dropout_pre_encoder": dropout,
           "dropout_emb": 0.0, "dropout_att": dropout_att, "stochastic_depth_drop_prob": 0.0}
    cfg.update(over)
    return cfg


def optim_cfg(lr: float = 1e-3, sched: Optional[str] = None, d_model: int = 512, warmup_steps: int = 10000,
              weight_decay: float = 1e-3, betas=(0.9, 0.98)) -> Dict[str, Any]:
    cfg: Dict[str, Any] = {"name": "adamw", "lr": lr, "betas": list(betas), "weight_decay": weight_decay}
    if sched == "noam":
        cfg["sched"] = {"name": "NoamAnnealing", "d_model": d_model, "warmup_steps": warmup_steps, "min_lr": 1e-6}
    elif sched == "cosine":
        cfg["sched"] = {"name": "CosineAnnealing", "warmup_steps": warmup_steps, "min_lr": 1e-6}
    return cfg


def fastconformer_ctc_config(size: str = "small", vocab_size: int = 128, features: int = 80, dropout: float = 0.0,
                             tokenizer: Optional[Dict[str, Any]] = None, lr: float = 1e-3, **enc_over) -> DictConfig:
    s = FASTCONFORMER_SIZES[size]
    tok = tokenizer or {"type": "synthetic", "vocab_size": vocab_size}
    return OmegaConf.create({
        "sample_rate": 16000, "log_prediction": False, "compute_train_wer": False,
        "tokenizer": tok,
        "preprocessor": preprocessor_cfg(features),
        "spec_augment": None,
        "encoder": encoder_cfg(size, features, dropout, dropout, **enc_over),
        "decoder": {"_target_": "speech_b200.modules.ctc_decoder.ConvASRDecoder", "feat_in": None, "num_classes": -1,
                    "vocabulary": []},
        "optim": optim_cfg(lr, None, s["d_model"], weight_decay=0.0),
    })


def fastconformer_transducer_config(size: str = "xlarge", vocab_size: int = 1024, features: int = 80,
                                    dropout: float = 0.1, loss: str = "tdt", durations=(0, 1, 2, 3, 4), sigma: float = 0.02,
                                    omega: float = 0.0, joint_hidden: int = 640, pred_rnn_layers: Optional[int] = None,
                                    tokenizer: Optional[Dict[str, Any]] = None, fused_batch_size: int = 4,
                                    lr: float = 5.0, sched: Optional[str] = "noam", n_layers: Optional[int] = None,
                                    hybrid_ctc_weight: Optional[float] = None, **enc_over) -> DictConfig:
    s = FASTCONFORMER_SIZES[size]
    tok = tokenizer or {"type": "synthetic", "vocab_size": vocab_size}
    loss_cfg: Dict[str, Any] = {"loss_name": "default"}
    if loss == "tdt":
        loss_cfg = {"loss_name": "tdt", "tdt_kwargs": {"fastemit_lambda": 0.0, "clamp": -1.0,
                                                        "durations": list(durations), "sigma": sigma, "omega": omega}}
    cfg = {
        "sample_rate": 16000, "log_prediction": False, "compute_train_wer": False, "compute_eval_loss": True,
        "model_defaults": {"enc_hidden": s["d_model"], "pred_hidden": s["pred_hidden"], "joint_hidden": joint_hidden},
        "tokenizer": tok,
        "preprocessor": preprocessor_cfg(features),
        "spec_augment": None,
        "encoder": encoder_cfg(size, features, dropout, dropout, n_layers=n_layers, **enc_over),
        "decoder": {"_target_": "speech_b200.modules.rnnt.RNNTDecoder", "normalization_mode": None,
                    "random_state_sampling": False, "blank_as_pad": True, "vocab_size": -1,
                    "prednet": {"pred_hidden": s["pred_hidden"], "pred_rnn_layers": pred_rnn_layers or s["pred_rnn_layers"],
                                "t_max": None, "dropout": 0.0}},
        "joint": {"_target_": "speech_b200.modules.rnnt.RNNTJoint", "log_softmax": None, "preserve_memory": False,
                  "fuse_loss_wer": True, "fused_batch_size": fused_batch_size, "num_classes": -1, "vocabulary": [],
                  "jointnet": {"joint_hidden": joint_hidden, "activation": "relu", "dropout": 0.0}},
        "decoding": {"strategy": "greedy_batch", "greedy": {"max_symbols": 10}},
        "loss": loss_cfg,
        "optim": optim_cfg(lr, sched, s["d_model"]),
    }
    if hybrid_ctc_weight is not None:
        cfg["aux_ctc"] = {"ctc_loss_weight": hybrid_ctc_weight, "use_cer": False, "ctc_reduction": "mean_batch",
                          "decoder": {"_target_": "speech_b200.modules.ctc_decoder.ConvASRDecoder", "feat_in": None,
                                      "num_classes": -1, "vocabulary": []},
                          "decoding": {"strategy": "greedy_batch"}}
    return OmegaConf.create(cfg)


def canary_aed_config(size: str = "xlarge", enc_layers: int = 32, dec_layers: int = 8, dec_hidden: int = 1024, dec_heads: int = 16,
                      dec_inner: int = 4096, vocab_size: int = 16384, features: int = 80, dropout: float = 0.1,
                      label_smoothing: float = 0.1, lr: float = 3e-4, optim_name: str = "adamw",
                      tokenizer: Optional[Dict[str, Any]] = None, max_sequence_length: int = 1024, **enc_over) -> DictConfig:
    """Canary-1B-v2-shape attention encoder-decoder (reference ``examples/asr/conf/speech_multitask/fast-conformer_aed.yaml``):
    FastConformer encoder, Transformer decoder with cross-attention and learned positions, tied output head, label-smoothed
    cross entropy."""
    s = FASTCONFORMER_SIZES[size]
    tok = tokenizer or {"type": "synthetic", "vocab_size": vocab_size}
    optim = optim_cfg(lr, None, s["d_model"])
    optim["name"] = optim_name
    return OmegaConf.create({
        "sample_rate": 16000, "log_prediction": False, "prompt_format": "canary2", "use_loss_mask_for_prompt": False,
        "model_defaults": {"asr_enc_hidden": s["d_model"], "lm_dec_hidden": dec_hidden},
        "tokenizer": tok,
        "preprocessor": preprocessor_cfg(features),
        "spec_augment": None,
        "encoder": encoder_cfg(size, features, dropout, dropout, n_layers=enc_layers, **enc_over),
        "transf_decoder": {"_target_": "speech_b200.modules.transformer_nm.get_transformer", "library": "nemo", "encoder": False,
                           "pre_ln_final_layer_norm": True,
                           "config_dict": {"max_sequence_length": max_sequence_length, "num_token_types": 0, "embedding_dropout": dropout,
                                           "learn_positional_encodings": True, "hidden_size": dec_hidden, "inner_size": dec_inner,
                                           "num_layers": dec_layers, "num_attention_heads": dec_heads, "ffn_dropout": dropout,
                                           "attn_score_dropout": dropout, "attn_layer_dropout": dropout, "hidden_act": "relu",
                                           "pre_ln": True, "vocab_size": vocab_size}},
        "head": {"num_layers": 1, "activation": "relu", "log_softmax": True, "dropout": 0.0},
        "loss": {"label_smoothing": label_smoothing},
        "decoding": {"strategy": "greedy", "greedy": {"max_generation_delta": 50}},
        "optim": optim,
    })
