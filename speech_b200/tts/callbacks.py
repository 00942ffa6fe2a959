"""Periodic logging of what a TTS / codec model produces during training: audio files and spectrogram / alignment images written
under the experiment directory (and handed to any attached logger that accepts them).

``LoggingCallback(generators, data_loader, epoch_frequency | log_epochs, output_dir)`` runs every generator on every batch of a small
fixed data loader at the chosen epochs.  Generators: ``VocoderArtifactGenerator`` (ground truth + vocoded audio),
``AudioCodecArtifactGenerator`` (reconstruction, optional token histogram), ``FastPitchArtifactGenerator`` (predicted mel, alignment,
optionally audio through a vocoder).  Images are written as portable grey maps (``.pgm``) — readable everywhere, no plotting library.

Reference: ``tts/parts/utils/callbacks.py``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..core.trainer import Callback
from ..data.audio_to_text import save_wav

__all__ = ["ArtifactGenerator", "AudioArtifact", "AudioCodecArtifactGenerator", "FastPitchArtifactGenerator", "ImageArtifact", "LoggingCallback",
           "VocoderArtifactGenerator", "create_id", "write_pgm"]


@dataclass
class AudioArtifact:
    id: str
    data: np.ndarray
    sample_rate: int
    filename: str


@dataclass
class ImageArtifact:
    id: str
    data: np.ndarray                        # [rows, cols], any range; normalised when written
    filename: str
    x_axis: str = ""
    y_axis: str = ""


def create_id(filepath: str) -> str:
    return os.path.splitext(str(filepath))[0].strip(os.sep).replace(os.sep, "_")


def write_pgm(path: str, image: np.ndarray, flip_rows: bool = True) -> None:
    """8-bit grey map; row 0 of a spectrogram (lowest frequency) goes to the bottom when ``flip_rows``."""
    x = np.asarray(image, dtype=np.float64)
    lo, hi = float(np.nanmin(x)), float(np.nanmax(x))
    g = np.zeros_like(x) if hi <= lo else (x - lo) / (hi - lo)
    g = (255 * np.nan_to_num(g)).astype(np.uint8)
    if flip_rows:
        g = g[::-1]
    with open(path, "wb") as f:
        f.write(f"P5\n{g.shape[1]} {g.shape[0]}\n255\n".encode())
        f.write(np.ascontiguousarray(g).tobytes())


class ArtifactGenerator:
    def generate_artifacts(self, model, batch: Any, initial_log: bool = False) -> Tuple[List[AudioArtifact], List[ImageArtifact]]:
        raise NotImplementedError


def _ids(batch, n: int) -> List[str]:
    if isinstance(batch, dict) and "audio_filepaths" in batch:
        return [create_id(p) for p in batch["audio_filepaths"]]
    return [f"item{i}" for i in range(n)]


def _audio_of(batch) -> Tuple[torch.Tensor, torch.Tensor]:
    if isinstance(batch, dict):
        return batch["audio"], batch["audio_lens"]
    return (batch[0], batch[1]) if len(batch) == 2 else (batch[2], batch[3])


class VocoderArtifactGenerator(ArtifactGenerator):
    """Mel of the recorded audio -> vocoder -> audio; the ground truth is saved at the first log only."""

    def generate_artifacts(self, model, batch, initial_log: bool = False):
        audio, lens = _audio_of(batch)
        dev = next(model.parameters()).device
        with torch.no_grad():
            mel = model.mel.mel(audio.to(dev))
            gen = model.convert_spectrogram_to_audio(mel)
        out: List[AudioArtifact] = []
        for i, uid in enumerate(_ids(batch, audio.shape[0])):
            n = int(lens[i])
            out.append(AudioArtifact(f"voc_{uid}", gen[i, :n].float().cpu().numpy(), model.sample_rate, f"voc_{uid}.wav"))
            if initial_log:
                out.append(AudioArtifact(f"gt_{uid}", audio[i, :n].float().cpu().numpy(), model.sample_rate, f"gt_{uid}.wav"))
        return out, []


class AudioCodecArtifactGenerator(ArtifactGenerator):
    def __init__(self, log_audio: bool = True, log_encoding: bool = False, log_dequantized: bool = False):
        self.log_audio, self.log_encoding, self.log_dequantized = log_audio, log_encoding, log_dequantized

    def generate_artifacts(self, model, batch, initial_log: bool = False):
        audio, lens = _audio_of(batch)
        dev = next(model.parameters()).device
        audios: List[AudioArtifact] = []
        images: List[ImageArtifact] = []
        with torch.no_grad():
            enc, enc_len = model.encode_audio(audio.to(dev), lens.to(dev))
            deq = enc
            if model.vector_quantizer is not None:
                deq, _ = model.vector_quantizer(enc, enc_len)
            gen, gen_len = model.audio_decoder(deq, enc_len)
        for i, uid in enumerate(_ids(batch, audio.shape[0])):
            if self.log_audio:
                audios.append(AudioArtifact(f"pred_{uid}", gen[i, : int(gen_len[i])].float().cpu().numpy(), model.sample_rate, f"pred_{uid}.wav"))
                if initial_log:
                    audios.append(AudioArtifact(f"gt_{uid}", audio[i, : int(lens[i])].float().cpu().numpy(), model.sample_rate, f"gt_{uid}.wav"))
            t = int(enc_len[i])
            if self.log_encoding:
                images.append(ImageArtifact(f"enc_{uid}", enc[i, :, :t].float().cpu().numpy(), f"enc_{uid}.pgm", "frames", "channels"))
            if self.log_dequantized:
                images.append(ImageArtifact(f"deq_{uid}", deq[i, :, :t].float().cpu().numpy(), f"deq_{uid}.pgm", "frames", "channels"))
        return audios, images


class FastPitchArtifactGenerator(ArtifactGenerator):
    """Predicted mel and hard alignment as images; audio when a ``vocoder`` (mel -> waveform callable or model) is given."""

    def __init__(self, log_spectrogram: bool = True, log_alignment: bool = True, vocoder: Optional[Any] = None, sample_rate: int = 22050):
        self.log_spec, self.log_align, self.vocoder, self.sr = log_spectrogram, log_alignment, vocoder, sample_rate

    def generate_artifacts(self, model, batch, initial_log: bool = False):
        text, text_len, audio, audio_len = batch[:4]
        dev = next(model.parameters()).device
        with torch.no_grad():
            mel_gt = model.mel.mel(audio.to(dev))
            mel_len = torch.div(audio_len, model.mel.hop, rounding_mode="floor") + 1
            o = model(text.to(dev), text_len.to(dev), mel_gt, mel_len.to(dev), pitch=None)
            free = model(text.to(dev), text_len.to(dev))
        audios, images = [], []
        for i, uid in enumerate(_ids(batch, text.shape[0])):
            if self.log_spec:
                images.append(ImageArtifact(f"spec_{uid}", free["mel"][i, :, : int(free["mel_len"][i])].float().cpu().numpy(), f"spec_{uid}.pgm", "frames", "mel bins"))
                if initial_log:
                    images.append(ImageArtifact(f"spec_gt_{uid}", mel_gt[i, :, : int(mel_len[i])].float().cpu().numpy(), f"spec_gt_{uid}.pgm", "frames", "mel bins"))
            if self.log_align and o["attn_hard"] is not None:
                images.append(ImageArtifact(f"align_{uid}", o["attn_hard"][i, : int(mel_len[i]), : int(text_len[i])].float().cpu().numpy().T, f"align_{uid}.pgm",
                                            "frames", "text tokens"))
            if self.vocoder is not None:
                wav = self.vocoder(free["mel"][i: i + 1, :, : int(free["mel_len"][i])])
                audios.append(AudioArtifact(f"pred_{uid}", wav[0].float().cpu().numpy(), self.sr, f"pred_{uid}.wav"))
        return audios, images


class LoggingCallback(Callback):
    def __init__(self, generators: Sequence[ArtifactGenerator], data_loader, log_epochs: Optional[Sequence[int]] = None, epoch_frequency: int = 1,
                 output_dir: Optional[str] = None, loggers: Optional[Sequence[Any]] = None, log_tensorboard: bool = False):
        self.generators, self.data_loader = list(generators), data_loader
        self.log_epochs = set(log_epochs) if log_epochs is not None else None
        self.freq, self.output_dir, self.loggers, self.log_tb = max(1, epoch_frequency), output_dir, list(loggers or []), log_tensorboard
        self._initial = True

    def _should_log(self, epoch: int) -> bool:
        return epoch in self.log_epochs if self.log_epochs is not None else epoch % self.freq == 0

    def _emit(self, audios: List[AudioArtifact], images: List[ImageArtifact], epoch: int, step: int):
        if self.output_dir:
            d = os.path.join(self.output_dir, f"epoch_{epoch}")
            os.makedirs(d, exist_ok=True)
            for a in audios:
                save_wav(os.path.join(d, a.filename), np.asarray(a.data, dtype=np.float32), a.sample_rate)
            for im in images:
                write_pgm(os.path.join(d, im.filename), im.data)
        for lg in self.loggers:
            exp = getattr(lg, "experiment", lg)
            for a in audios:
                if hasattr(exp, "add_audio"):
                    exp.add_audio(a.id, np.asarray(a.data), global_step=step, sample_rate=a.sample_rate)
            for im in images:
                if hasattr(exp, "add_image"):
                    x = np.asarray(im.data, dtype=np.float32)
                    x = (x - x.min()) / max(1e-9, float(x.max() - x.min()))
                    exp.add_image(im.id, x[None, ::-1].copy(), global_step=step)

    def on_train_epoch_end(self, trainer, model):
        epoch = int(trainer.current_epoch)
        if not getattr(trainer, "is_global_zero", True) or not self._should_log(epoch):
            return
        was = model.training
        model.eval()
        try:
            for batch in self.data_loader:
                for g in self.generators:
                    audios, images = g.generate_artifacts(model, batch, initial_log=self._initial)
                    self._emit(audios, images, epoch, int(trainer.global_step))
        finally:
            model.train(was)
        self._initial = False
