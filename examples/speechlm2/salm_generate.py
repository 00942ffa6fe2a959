"""Free-form generation with SALM from a JSON-lines file of conversations (reference script: ``examples/speechlm2/salm_generate.py``).

python examples/speechlm2/salm_generate.py pretrained_name=ckpt.nemo inputs=conversations.jsonl max_new_tokens=256"""
import json

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import load_audio
from speech_b200.speechlm.data import read_conversations
from speech_b200.speechlm.salm import SALM


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"pretrained_name": None, "inputs": None, "max_new_tokens": 256, "output_manifest": "generations.jsonl",
                                            "do_sample": False, "temperature": 1.0, "top_p": 1.0}), cfg)
    model = SALM.restore_from(cfg.pretrained_name).eval()
    with open(cfg.output_manifest, "w", encoding="utf-8") as out:
        for conv in read_conversations(cfg.inputs):
            turns, auds = [], []
            for t in conv["conversations"]:
                role = "assistant" if t["from"].lower() in ("assistant", "agent") else "user"
                if t.get("type") == "audio":
                    auds.append(torch.as_tensor(load_audio(t["value"])))
                    text = model.audio_locator_tag
                else:
                    text = t["value"]
                if turns and turns[-1]["role"] == role:
                    turns[-1]["content"] += " " + text
                else:
                    turns.append({"role": role, "content": text})
            if turns and turns[-1]["role"] == "assistant":
                turns = turns[:-1]
            audio = torch.nn.utils.rnn.pad_sequence(auds, batch_first=True) if auds else None
            lens = torch.tensor([a.numel() for a in auds]) if auds else None
            ids = model.generate([turns], audios=audio, audio_lens=lens, max_new_tokens=cfg.max_new_tokens, do_sample=cfg.do_sample,
                                 temperature=cfg.temperature, top_p=cfg.top_p)
            out.write(json.dumps({"id": conv.get("id"), "response": model.tokenizer.ids_to_text(ids[0].cpu().tolist())}, ensure_ascii=False) + "\n")


if __name__ == "__main__":
    main()
