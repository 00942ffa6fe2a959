"""Streaming inference of an attention encoder-decoder model with a wait-k or AlignAtt policy: audio arrives in chunks, the decoder
emits tokens as soon as the policy allows, latency (average lagging) is reported with the transcripts.

python .../speech_to_text_aed_streaming_infer.py model_path=m.nemo dataset_manifest=test.json chunk_secs=1.0 \\
       decoding.streaming_policy=waitk decoding.waitk_lagging=2 [decoding.alignatt_thr=8]
(reference script: ``examples/asr/asr_chunked_inference/aed/speech_to_text_aed_streaming_infer.py``)."""
import json

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import load_audio, read_manifest
from speech_b200.decoding.aed_streaming import AEDStreamingDecodingConfig, GreedyBatchedStreamingAEDComputer
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate


def transcribe_stream(model, computer, audio, chunk_samples, sr):
    """Feed ``audio`` chunk by chunk: after every chunk the encoder runs over what has arrived (an offline encoder: the prefix is
    re-encoded) and the decoder emits what the policy allows.  Returns (text, length-adaptive average lagging in seconds)."""
    dev = next(model.parameters()).device
    prompt = model._default_prompt_ids(1, dev)
    state = computer.init_state(prompt)
    n = audio.numel()
    enc_len = None
    for end in range(chunk_samples, n + chunk_samples, chunk_samples):
        end = min(end, n)
        x = audio[:end].unsqueeze(0).to(dev)
        enc, enc_len, _ = model.encode_audio(input_signal=x, input_signal_length=torch.tensor([end], device=dev))
        last = torch.tensor([end >= n], device=dev)
        state = computer(enc, enc_len, last, state)
        if not bool(state.active_samples.any()):
            break
    ids = state.hypotheses(computer.eos)[0]
    frame_s = n / sr / max(1, int(enc_len[0]))
    return model.decoding.decode_tokens_to_str(ids), computer.compute_laal(state, enc_len, frame_s)[0]


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "dataset_manifest": None, "output_filename": "aed_streaming_transcripts.json",
                                            "chunk_secs": 1.0, "decoding": {"streaming_policy": "waitk", "waitk_lagging": 2, "alignatt_thr": 8}}), cfg)
    model = ASRModel.restore_from(cfg.model_path).eval()
    fields = AEDStreamingDecodingConfig.__dataclass_fields__
    dcfg = AEDStreamingDecodingConfig(**{k: v for k, v in OmegaConf.to_container(cfg.decoding).items() if k in fields})
    eos = model.tokenizer.eos_id
    computer = GreedyBatchedStreamingAEDComputer(model.transf_decoder.embedding, model.transf_decoder.decoder, model.log_softmax, eos, dcfg)
    sr = 16000
    items = read_manifest(cfg.dataset_manifest)
    out = []
    with torch.no_grad():
        for it in items:
            audio = torch.as_tensor(load_audio(it["audio_filepath"], target_sr=sr), dtype=torch.float32)
            text, lagging = transcribe_stream(model, computer, audio, int(cfg.chunk_secs * sr), sr)
            out.append(dict(it, pred_text=text, average_lagging_s=lagging))
    computer.close()
    with open(cfg.output_filename, "w", encoding="utf-8") as f:
        for r in out:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
    if all(it.get("text") for it in items):
        logging.info(f"WER: {100 * word_error_rate([r['pred_text'] for r in out], [it['text'] for it in items]):.2f}%")
    return out


if __name__ == "__main__":
    main()
