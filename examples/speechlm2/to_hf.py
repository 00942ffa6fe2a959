"""Export a SALM checkpoint's language model (with LoRA merged) as a Hugging Face directory, plus the perception weights
(reference script: ``examples/speechlm2/to_hf.py``).

python examples/speechlm2/to_hf.py pretrained_name=ckpt.nemo output_dir=hf_model"""
import os

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.speechlm.lora import merge_lora
from speech_b200.speechlm.salm import SALM


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"pretrained_name": None, "output_dir": "hf_model"}), cfg)
    model = SALM.restore_from(cfg.pretrained_name).eval()
    merge_lora(model.llm)
    model.llm.model.embed_tokens = model.embed_tokens          # the table lives on the SALM during training
    model.llm.save_pretrained(cfg.output_dir)
    from safetensors.torch import save_file

    save_file({k: v.detach().cpu().contiguous() for k, v in model.perception.state_dict().items()},
              os.path.join(cfg.output_dir, "perception.safetensors"))


if __name__ == "__main__":
    main()
