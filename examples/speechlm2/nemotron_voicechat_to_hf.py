"""Export the duplex voice-chat stack as one Hugging Face style directory: the listening half's language model, its perception
weights, the speaking half and the codec, each as safetensors with a JSON manifest of what is where.

python examples/speechlm2/nemotron_voicechat_to_hf.py stt=duplex_stt.nemo tts=eartts.nemo [codec=codec.nemo] output_dir=voicechat_hf
(reference script: ``examples/speechlm2/nemotron_voicechat_to_hf.py``)."""
import json
import os

from speech_b200.core.config import OmegaConf, hydra_runner, to_container
from speech_b200.core.modelpt import ModelPT
from speech_b200.speechlm.duplex import DuplexSTTModel
from speech_b200.speechlm.ear_tts import DuplexEARTTS


def _save(sd, path):
    from safetensors.torch import save_file

    save_file({k: v.detach().cpu().contiguous() for k, v in sd.items()}, path)


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"stt": None, "tts": None, "codec": None, "output_dir": "voicechat_hf"}), cfg)
    os.makedirs(cfg.output_dir, exist_ok=True)
    stt = DuplexSTTModel.restore_from(cfg.stt, map_location="cpu").eval()
    tts = DuplexEARTTS.restore_from(cfg.tts, map_location="cpu").eval()
    parts = {}
    llm_dir = os.path.join(cfg.output_dir, "llm")
    if hasattr(stt.llm, "save_pretrained"):
        stt.llm.save_pretrained(llm_dir)
        parts["llm"] = "llm/"
    _save({k: v for k, v in stt.state_dict().items() if not k.startswith("llm.")}, os.path.join(cfg.output_dir, "stt_heads_and_perception.safetensors"))
    parts["stt_rest"] = "stt_heads_and_perception.safetensors"
    _save(tts.state_dict(), os.path.join(cfg.output_dir, "tts.safetensors"))
    parts["tts"] = "tts.safetensors"
    configs = {"stt": to_container(stt.cfg, resolve=True), "tts": to_container(tts.cfg, resolve=True)}
    if cfg.codec:
        codec = ModelPT.restore_from(cfg.codec, map_location="cpu").eval()
        _save(codec.state_dict(), os.path.join(cfg.output_dir, "codec.safetensors"))
        parts["codec"] = "codec.safetensors"
        configs["codec"] = to_container(codec.cfg, resolve=True)
    with open(os.path.join(cfg.output_dir, "config.json"), "w") as f:
        json.dump({"architectures": ["NemotronVoiceChat"], "parts": parts, "configs": configs}, f, indent=2, default=str)
    return parts


if __name__ == "__main__":
    main()
