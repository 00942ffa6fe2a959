"""Evaluate SALM as a speech recogniser: generate transcripts for a manifest, report WER and RTFx.

python examples/speechlm2/salm_eval.py pretrained_name=ckpt.nemo inputs=test.json batch_size=16 max_new_tokens=128
(reference script: ``examples/speechlm2/salm_eval.py``; WER + RTFx ``:190-201``)."""
import json
import time

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import load_audio, read_manifest
from speech_b200.speechlm.salm import SALM
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"pretrained_name": None, "inputs": None, "batch_size": 16, "max_new_tokens": 128,
                                            "output_manifest": "generations.jsonl", "user_prompt": "Transcribe the following:",
                                            "system_prompt": None, "device": "cuda" if torch.cuda.is_available() else "cpu"}), cfg)
    model = SALM.restore_from(cfg.pretrained_name).to(cfg.device).eval()
    items = read_manifest(cfg.inputs)
    preds, audio_secs, t_total = [], 0.0, 0.0
    for s in range(0, len(items), cfg.batch_size):
        chunk = items[s:s + cfg.batch_size]
        auds = [torch.as_tensor(load_audio(it["audio_filepath"])) for it in chunk]
        lens = torch.tensor([a.numel() for a in auds])
        audio = torch.nn.utils.rnn.pad_sequence(auds, batch_first=True)
        turns = ([{"role": "system", "content": cfg.system_prompt}] if cfg.system_prompt else []) + \
            [{"role": "user", "content": f"{cfg.user_prompt} {model.audio_locator_tag}"}]
        if cfg.device == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        ids = model.generate([turns] * len(chunk), audios=audio, audio_lens=lens, max_new_tokens=cfg.max_new_tokens)
        if cfg.device == "cuda":
            torch.cuda.synchronize()
        t_total += time.perf_counter() - t0
        audio_secs += float(lens.sum()) / 16000
        for row in ids.cpu().tolist():
            row = [t for t in row if t not in (model.text_pad_id, model.text_eos_id)]
            preds.append(model.tokenizer.ids_to_text(row).strip())
    with open(cfg.output_manifest, "w", encoding="utf-8") as f:
        for it, p in zip(items, preds):
            f.write(json.dumps(dict(it, pred_text=p), ensure_ascii=False) + "\n")
    if all(it.get("text") for it in items):
        logging.info(f"WER: {100 * word_error_rate(preds, [it['text'] for it in items]):.2f}%")
    logging.info(f"RTFx: {audio_secs / max(t_total, 1e-9):.1f}")


if __name__ == "__main__":
    main()
