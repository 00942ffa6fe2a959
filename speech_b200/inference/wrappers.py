"""Model wrappers used by the streaming pipelines: a uniform view of CTC / transducer models (geometry, tokenizer,
blank id) plus the two kinds of step they run — a cache-aware encoder chunk followed by decoding that continues from the
previous state, or a whole-window offline pass for buffered streaming.
Reference: ``inference/model_wrappers/{asr,cache_aware_asr,cache_aware_rnnt,cache_aware_ctc,rnnt,ctc}_inference_wrapper.py``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .. import ops
from .context_manager import CacheAwareContext


class ASRInferenceWrapper:
    def __init__(self, asr_model, device=None, compute_dtype: Optional[torch.dtype] = None, decoding_cfg=None):
        self.asr_model = asr_model
        self.device = torch.device(device) if device is not None else next(asr_model.parameters()).device
        self.compute_dtype = compute_dtype
        asr_model.to(self.device)
        asr_model.eval()
        if decoding_cfg is not None and hasattr(asr_model, "change_decoding_strategy"):
            asr_model.change_decoding_strategy(decoding_cfg)
        pre = asr_model.preprocessor
        feat = getattr(pre, "featurizer", pre)
        self.sample_rate = int(getattr(feat, "sample_rate", getattr(pre, "_sample_rate", 16000)))
        self.hop_length = int(getattr(feat, "hop_length", 160))
        self.window_stride = self.hop_length / self.sample_rate
        self.subsampling_factor = int(getattr(asr_model.encoder, "subsampling_factor", 1))
        self.seconds_per_timestep = self.window_stride * self.subsampling_factor

    # ------------------------------------------------------------------ vocabulary
    @property
    def tokenizer(self):
        return getattr(self.asr_model, "tokenizer", None)

    def ids_to_tokens(self, ids: List[int]) -> List[str]:
        return self.decoding.decode_ids_to_tokens(list(ids))

    def ids_to_text(self, ids: List[int]) -> str:
        return self.decoding.decode_tokens_to_str(list(ids))

    @property
    def decoding(self):
        m = self.asr_model
        if self.decoder_type == "ctc" and hasattr(m, "ctc_decoding"):
            return m.ctc_decoding
        return m.decoding

    @property
    def decoder_type(self) -> str:
        from ..models.ctc_models import EncDecCTCModel

        return getattr(self.asr_model, "cur_decoder", None) or ("ctc" if isinstance(self.asr_model, EncDecCTCModel) else "rnnt")

    @property
    def blank_id(self) -> int:
        return int(self.decoding.blank_id)

    def autocast(self):
        return ops.compute_dtype(self.compute_dtype)

    # ------------------------------------------------------------------ offline window pass (buffered streaming)
    @torch.no_grad()
    def encode_windows(self, windows: torch.Tensor, lengths: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Audio windows [B, n] → encoder output [B, D, T'] and lengths."""
        m = self.asr_model
        with self.autocast():
            feats, flen = m.preprocessor(input_signal=windows.to(self.device), length=lengths.to(self.device))
            enc, enc_len = m.encoder(audio_signal=feats, length=flen)
        return enc, enc_len

    @torch.no_grad()
    def ctc_frame_predictions(self, enc: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        m = self.asr_model
        dec = m.ctc_decoder if hasattr(m, "ctc_decoder") else m.decoder
        with self.autocast():
            lp = dec(encoder_output=enc).float()
        conf, pred = lp.max(dim=-1)
        return pred, conf.exp()

    @torch.no_grad()
    def rnnt_decode(self, enc: torch.Tensor, enc_len: torch.Tensor, partial=None):
        return self.asr_model.decoding.rnnt_decoder_predictions_tensor(enc, enc_len, return_hypotheses=True,
                                                                       partial_hypotheses=partial)


class CacheAwareASRInferenceWrapper(ASRInferenceWrapper):
    def __init__(self, asr_model, device=None, compute_dtype=None, decoding_cfg=None, att_context_size=None):
        super().__init__(asr_model, device, compute_dtype, decoding_cfg)
        enc = asr_model.encoder
        if not hasattr(enc, "cache_aware_stream_step"):
            raise ValueError("the model's encoder does not support cache-aware streaming")
        if att_context_size is not None:
            self.set_default_att_context_size(att_context_size)
        if enc.streaming_cfg is None:
            enc.setup_streaming_params()
        # the encoder step of a streaming batch repeats its shapes: replay it from CUDA graphs (SPEECH_B200_STREAM_GRAPHS=0 to disable)
        import os

        enc.stream_cuda_graphs = self.device.type == "cuda" and os.environ.get("SPEECH_B200_STREAM_GRAPHS", "1") != "0"

    def set_default_att_context_size(self, att_context_size) -> None:
        self.asr_model.encoder.set_default_att_context_size(list(att_context_size))
        self.asr_model.encoder.setup_streaming_params()

    @property
    def streaming_cfg(self):
        return self.asr_model.encoder.streaming_cfg

    @staticmethod
    def _pick(v, first: bool):
        return (v[0] if first else v[1]) if isinstance(v, (list, tuple)) else v

    def chunk_feature_frames(self, first: bool = False) -> int:
        return int(self._pick(self.streaming_cfg.chunk_size, first))

    def shift_feature_frames(self, first: bool = False) -> int:
        return int(self._pick(self.streaming_cfg.shift_size, first))

    def pre_encode_cache_frames(self) -> int:
        return int(self._pick(self.streaming_cfg.pre_encode_cache_size, False))

    def drop_extra_pre_encoded(self) -> int:
        return int(self.streaming_cfg.drop_extra_pre_encoded)

    def get_initial_cache_state(self, batch_size: int = 1):
        return self.asr_model.encoder.get_initial_cache_state(batch_size=batch_size, device=self.device)

    @torch.no_grad()
    def stream_step(self, features: torch.Tensor, lengths: torch.Tensor, context: CacheAwareContext,
                    previous_hypotheses=None, previous_pred_out=None, drop_extra_pre_encoded: Optional[int] = None,
                    keep_all_outputs: bool = False):
        """One chunk for a batch of streams.  Returns ``(hypotheses_or_frame_predictions, new_context, encoded_len)``."""
        m = self.asr_model
        with self.autocast():
            out = m.conformer_stream_step(
                processed_signal=features.to(self.device), processed_signal_length=lengths.to(self.device),
                cache_last_channel=context.cache_last_channel, cache_last_time=context.cache_last_time,
                cache_last_channel_len=context.cache_last_channel_len, keep_all_outputs=keep_all_outputs,
                previous_hypotheses=previous_hypotheses, previous_pred_out=previous_pred_out,
                drop_extra_pre_encoded=drop_extra_pre_encoded, return_transcription=True, return_log_probs=True)
        greedy, hyps, clc, clt, clcl, best, encoded, encoded_len = out
        return best, CacheAwareContext(clc, clt, clcl), encoded_len, greedy


class CacheAwareRNNTInferenceWrapper(CacheAwareASRInferenceWrapper):
    def build_malsd_computer(self, beam_size: int = 4, max_symbols_per_step: int = 10, fusion_models=None, fusion_models_alpha=None):
        """A batched beam-search computer over this model's prediction and joint networks (TDT durations picked up from the
        model's decoding config)."""
        from ..decoding.batched_beam import ModifiedALSDBatchedComputer

        m = self.asr_model
        durations = list(getattr(m.decoding, "durations", None) or [])
        return ModifiedALSDBatchedComputer(m.decoder, m.joint, self.blank_id, beam_size=beam_size, durations=durations,
                                           max_symbols_per_step=max_symbols_per_step, fusion_models=fusion_models,
                                           fusion_models_alpha=fusion_models_alpha)

    @torch.no_grad()
    def malsd_stream_step(self, malsd_computer, features: torch.Tensor, lengths: torch.Tensor, context: CacheAwareContext, carries: list,
                          drop_extra_pre_encoded: Optional[int] = None):
        """One chunk for a batch of streams under beam search.  ``carries[i]`` is stream i's beam state from its previous chunk
        (``None`` at the start of an utterance).  Returns ``(best, new_context, encoded_len, new_carries)`` with
        ``best[i] = (tokens, frame indices within the utterance, score)`` of the currently best entry of stream i's beam — the
        whole utterance so far, not only this chunk, because the best entry may change.
        Reference: ``inference/model_wrappers/cache_aware_rnnt_inference_wrapper.py`` ``malsd_stream_step``."""
        from ..decoding.batched_beam import MALSDCarry

        m = self.asr_model
        with self.autocast(), ops.compute_dtype(ops.get_compute_dtype()):
            encoded, encoded_len, clc, clt, clcl = m.encoder.cache_aware_stream_step(
                processed_signal=features.to(self.device), processed_signal_length=lengths.to(self.device),
                cache_last_channel=context.cache_last_channel, cache_last_time=context.cache_last_time,
                cache_last_channel_len=context.cache_last_channel_len, keep_all_outputs=False, drop_extra_pre_encoded=drop_extra_pre_encoded)
        enc = encoded.transpose(1, 2).float()
        fresh = [i for i, c in enumerate(carries) if c is None]
        if fresh:                                  # open a beam for the streams that start an utterance: zero frames decode nothing
            sub = torch.tensor(fresh, device=enc.device)
            malsd_computer(enc[sub, :0], torch.zeros(len(fresh), dtype=torch.long, device=enc.device))
            opened = malsd_computer.carry.split()
            carries = list(carries)
            for i, c in zip(fresh, opened):
                carries[i] = c
        hyps = malsd_computer(enc, encoded_len, MALSDCarry.merge(carries))
        new_carries = malsd_computer.carry.split()
        best = [h[0] if h else ([], [], 0.0) for h in hyps.to_hyps_list(score_norm=malsd_computer.score_norm)]
        return best, CacheAwareContext(clc, clt, clcl), encoded_len, new_carries


class CacheAwareCTCInferenceWrapper(CacheAwareASRInferenceWrapper):
    pass


class RNNTInferenceWrapper(ASRInferenceWrapper):
    pass


class CTCInferenceWrapper(ASRInferenceWrapper):
    pass
