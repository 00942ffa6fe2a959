"""Transducer inference from exported sub-networks.  ``export_transducer_subnets`` traces the encoder and one decoder+joint step as two
TorchScript files; ``TorchscriptGreedyBatchedRNNTInfer`` loads them and runs batched greedy decoding with no model class in sight, which
is how a deployment checks that the exported graphs reproduce the framework's transcripts.  ``ONNXGreedyBatchedRNNTInfer`` is the same
loop over ONNX Runtime sessions (it needs the ``onnxruntime`` package).
The step graph: ``(encoder frame [B, 1, D], last token [B, 1], h [L, B, H], c [L, B, H]) → (logits [B, V + 1 (+ durations)], h', c')``; the
start-of-sequence input is the blank token (its embedding row is zero) with a zero state.
Reference: ``asr/parts/submodules/rnnt_greedy_decoding.py`` (``ExportedModelGreedyBatchedRNNTInfer``, ``ONNXGreedyBatchedRNNTInfer``,
``TorchscriptGreedyBatchedRNNTInfer``), ``examples/asr/export/transducer/infer_transducer_{ts,onnx}.py``.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Tuple

import torch
from torch import nn


class _EncoderForExport(nn.Module):
    def __init__(self, encoder):
        super().__init__()
        self.encoder = encoder

    def forward(self, audio_signal: torch.Tensor, length: torch.Tensor):
        enc, enc_len = self.encoder(audio_signal=audio_signal, length=length)
        return enc, enc_len


class _DecoderJointStep(nn.Module):
    def __init__(self, decoder, joint):
        super().__init__()
        self.decoder, self.joint = decoder, joint

    def forward(self, enc_frame: torch.Tensor, token: torch.Tensor, h: torch.Tensor, c: torch.Tensor):
        g, (h2, c2) = self.decoder.predict(token, (h, c), add_sos=False)
        f = self.joint.project_encoder(enc_frame)
        logits = self.joint.joint_after_projection(f, self.joint.project_prednet(g))
        return logits[:, 0, 0, :], h2, c2


def export_transducer_subnets(model, out_dir: str, feat_frames: int = 64, batch: int = 2) -> Tuple[str, str]:
    """Writes ``encoder.ts`` and ``decoder_joint.ts`` under ``out_dir`` (traced on CPU copies of the inputs' device) and returns their paths."""
    os.makedirs(out_dir, exist_ok=True)
    model.eval()
    dev = next(model.parameters()).device
    feat_in = int(getattr(model.encoder, "_feat_in", getattr(model.encoder, "feat_in", 80)))
    feats, flen = torch.randn(batch, feat_in, feat_frames, device=dev), torch.full((batch,), feat_frames, dtype=torch.long, device=dev)
    enc_path, dj_path = os.path.join(out_dir, "encoder.ts"), os.path.join(out_dir, "decoder_joint.ts")
    with torch.no_grad():
        enc_mod = _EncoderForExport(model.encoder)
        torch.jit.trace(enc_mod, (feats, flen), check_trace=False, strict=False).save(enc_path)
        enc, _ = enc_mod(feats, flen)
        dec = model.decoder
        L, H = int(dec.pred_rnn_layers), int(dec.pred_hidden)
        step = _DecoderJointStep(dec, model.joint)
        blank = int(getattr(dec, "blank_idx", model.joint.num_classes_with_blank - 1))
        example = (enc[:, :, :1].transpose(1, 2).contiguous(), torch.full((batch, 1), blank, dtype=torch.long, device=dev),
                   torch.zeros(L, batch, H, device=dev), torch.zeros(L, batch, H, device=dev))
        was = getattr(model.joint, "log_softmax", None)
        model.joint.log_softmax = False                              # raw logits: the arg-max is all greedy decoding needs
        try:
            torch.jit.trace(step, example, check_trace=False, strict=False).save(dj_path)
        finally:
            model.joint.log_softmax = was
    return enc_path, dj_path


class ExportedModelGreedyBatchedRNNTInfer:
    """Greedy decoding over the two exported graphs.  Subclasses provide ``run_encoder`` and ``run_decoder_joint``.  ``durations`` (TDT) makes the
    last ``len(durations)`` outputs of the step the duration head: the frame pointer advances by the chosen duration."""

    def __init__(self, blank_id: int, pred_layers: int, pred_hidden: int, max_symbols_per_step: Optional[int] = 10, durations: Optional[Sequence[int]] = None):
        self.blank, self.L, self.H = int(blank_id), int(pred_layers), int(pred_hidden)
        self.max_symbols = max_symbols_per_step
        self.durations = list(durations or [])

    def run_encoder(self, audio_signal: torch.Tensor, length: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError

    def run_decoder_joint(self, enc_frame, token, h, c):
        raise NotImplementedError

    @torch.no_grad()
    def __call__(self, audio_signal: torch.Tensor, length: torch.Tensor) -> List[List[int]]:
        enc, enc_len = self.run_encoder(audio_signal, length)               # [B, D, T]
        enc = enc.transpose(1, 2)
        B, T, _ = enc.shape
        dev = enc.device
        h, c = torch.zeros(self.L, B, self.H, device=dev), torch.zeros(self.L, B, self.H, device=dev)
        last = torch.full((B, 1), self.blank, dtype=torch.long, device=dev)
        t = torch.zeros(B, dtype=torch.long, device=dev)
        emitted = torch.zeros(B, dtype=torch.long, device=dev)
        hyps: List[List[int]] = [[] for _ in range(B)]
        nd = len(self.durations)
        durs = torch.tensor(self.durations or [0], device=dev)
        while True:
            active = t < enc_len
            if not bool(active.any()):
                break
            frame = enc[torch.arange(B, device=dev), t.clamp(max=T - 1)].unsqueeze(1)
            logits, h2, c2 = self.run_decoder_joint(frame, last, h, c)
            tok_logits = logits[:, :logits.shape[1] - nd] if nd else logits
            k = tok_logits.argmax(-1)
            jump = durs[logits[:, -nd:].argmax(-1)] if nd else torch.zeros_like(k)
            is_blank = k == self.blank
            forced = emitted >= self.max_symbols if self.max_symbols else torch.zeros_like(is_blank)
            emit = active & ~is_blank & ~forced
            for b in emit.nonzero().flatten().tolist():
                hyps[b].append(int(k[b]))
            keep = emit.view(1, B, 1)
            h, c = torch.where(keep, h2, h), torch.where(keep, c2, c)
            last = torch.where(emit.view(B, 1), k.view(B, 1), last)
            if nd:
                step = torch.where(emit, jump, jump.clamp(min=1))             # a blank (or a forced move) always advances
                step = torch.where(forced & ~is_blank, torch.ones_like(step), step)
            else:
                step = (~emit).long()
            emitted = torch.where(step > 0, torch.zeros_like(emitted), emitted + emit.long())
            t = t + torch.where(active, step, torch.zeros_like(step))
        return hyps


class TorchscriptGreedyBatchedRNNTInfer(ExportedModelGreedyBatchedRNNTInfer):
    def __init__(self, encoder_model: str, decoder_joint_model: str, blank_id: int, pred_layers: int, pred_hidden: int, max_symbols_per_step: Optional[int] = 10,
                 durations: Optional[Sequence[int]] = None, device: str = "cpu"):
        super().__init__(blank_id, pred_layers, pred_hidden, max_symbols_per_step, durations)
        for p in (encoder_model, decoder_joint_model):
            if not os.path.isfile(p):
                raise FileNotFoundError(p)
        self.device = torch.device(device)
        self.encoder = torch.jit.load(encoder_model, map_location=self.device).eval()
        self.decoder_joint = torch.jit.load(decoder_joint_model, map_location=self.device).eval()

    def run_encoder(self, audio_signal, length):
        return self.encoder(audio_signal.to(self.device), length.to(self.device))

    def run_decoder_joint(self, enc_frame, token, h, c):
        return self.decoder_joint(enc_frame, token, h, c)


class ONNXGreedyBatchedRNNTInfer(ExportedModelGreedyBatchedRNNTInfer):
    """The same loop over ONNX Runtime sessions of ``encoder.onnx`` / ``decoder_joint.onnx`` (inputs in the order of the step graph)."""

    def __init__(self, encoder_model: str, decoder_joint_model: str, blank_id: int, pred_layers: int, pred_hidden: int, max_symbols_per_step: Optional[int] = 10,
                 durations: Optional[Sequence[int]] = None, providers: Optional[Sequence[str]] = None):
        super().__init__(blank_id, pred_layers, pred_hidden, max_symbols_per_step, durations)
        try:
            import onnxruntime as ort
        except ImportError as e:
            raise RuntimeError("decoding exported ONNX graphs needs the 'onnxruntime' package, which is not installed; use the TorchScript export instead") from e
        providers = list(providers or ["CUDAExecutionProvider", "CPUExecutionProvider"])
        self.encoder = ort.InferenceSession(encoder_model, providers=providers)
        self.decoder_joint = ort.InferenceSession(decoder_joint_model, providers=providers)

    @staticmethod
    def _run(session, tensors):
        feed = {i.name: t.cpu().numpy() for i, t in zip(session.get_inputs(), tensors)}
        return [torch.from_numpy(o) for o in session.run(None, feed)]

    def run_encoder(self, audio_signal, length):
        enc, enc_len = self._run(self.encoder, (audio_signal, length))
        return enc, enc_len

    def run_decoder_joint(self, enc_frame, token, h, c):
        return tuple(self._run(self.decoder_joint, (enc_frame, token, h, c)))
