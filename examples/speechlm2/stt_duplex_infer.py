"""Run the duplex speech-to-text model over recordings: frame-synchronous decoding with a KV cache, optional text prompt, forced turn
taking and trailing silence so that the agent can finish; reports turn-taking accuracy / latency when the manifest carries the
user's end-of-turn time.

python examples/speechlm2/stt_duplex_infer.py pretrained_name=duplex.nemo inputs=test.json [system_prompt="..."] [pad_seconds=2.0] \\
       [force_turn_taking=true]
(reference script: ``examples/speechlm2/stt_duplex_infer.py``; engine ``speechlm2/streaming/duplex_stt_inference.py``)."""
import json

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import load_audio, read_manifest
from speech_b200.speechlm.duplex import DuplexSTTModel
from speech_b200.speechlm.duplex_streaming import DuplexSTTStreamingInference
from speech_b200.speechlm.metrics import TurnTakingMetrics
from speech_b200.utils.logging import logging


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"pretrained_name": None, "inputs": None, "output_manifest": "duplex_generations.jsonl", "batch_size": 8,
                                            "system_prompt": None, "pad_seconds": 2.0, "force_turn_taking": None,
                                            "device": "cuda" if torch.cuda.is_available() else "cpu"}), cfg)
    model = DuplexSTTModel.restore_from(cfg.pretrained_name).to(cfg.device).eval()
    engine = DuplexSTTStreamingInference(model, force_turn_taking=cfg.force_turn_taking)
    items = read_manifest(cfg.inputs)
    frame_s = model.perception.token_equivalent_duration
    tt = TurnTakingMetrics(eos_token_id=model.text_eos_id, bos_token_id=model.text_bos_id, latency_multiplier=frame_s)
    prompt = None
    if cfg.system_prompt and model.tokenizer is not None:
        prompt = torch.tensor(model.tokenizer.text_to_ids(cfg.system_prompt), dtype=torch.long)
    out = []
    for s in range(0, len(items), cfg.batch_size):
        chunk = items[s:s + cfg.batch_size]
        auds = [torch.as_tensor(load_audio(it["audio_filepath"])) for it in chunk]
        lens = torch.tensor([a.numel() for a in auds])
        audio = torch.nn.utils.rnn.pad_sequence(auds, batch_first=True).to(cfg.device)
        kw = {}
        if prompt is not None:
            kw = {"prompt_tokens": prompt.unsqueeze(0).expand(len(chunk), -1), "prompt_token_lens": torch.full((len(chunk),), prompt.numel())}
        res = engine.offline_inference(audio, lens.to(cfg.device), input_pad_len=int(cfg.pad_seconds * 16000), **kw)
        for i, it in enumerate(chunk):
            rec = dict(it, pred_text=res["text"][i])
            if "asr_text" in res:
                rec["pred_user_text"] = res["asr_text"][i]
            out.append(rec)
        if all("user_end_time" in it for it in chunk):
            # user channel for the metric: end-of-turn token at the annotated frame
            src = torch.full_like(res["tokens"], model.text_pad_id)
            for i, it in enumerate(chunk):
                f = min(src.shape[1] - 1, int(round(float(it["user_end_time"]) / frame_s)))
                src[i, f] = model.text_eos_id
            tt.update("inputs", src, res["tokens"])
    with open(cfg.output_manifest, "w", encoding="utf-8") as f:
        for r in out:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
    metrics = {k: float(v) for k, v in tt.compute().items()}
    if metrics:
        logging.info(f"turn taking: {metrics}")
    return out, metrics


if __name__ == "__main__":
    main()
