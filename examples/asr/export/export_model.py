"""Export a model (or its encoder / decoder parts) to TorchScript or ONNX and verify the exported module against eager.

python examples/asr/export/export_model.py model_path=model.nemo output=model.ts [submodule=encoder] [check_trace=true]
(reference script: ``scripts/export.py``; exporter: ``core/classes/exportable.py``)."""
from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "output": "model.ts", "submodule": None, "check_trace": True}), cfg)
    model = ASRModel.restore_from(cfg.model_path, map_location="cpu").eval()
    target = getattr(model, cfg.submodule) if cfg.submodule else model
    files, notes = target.export(cfg.output, check_trace=bool(cfg.check_trace))
    for f, n in zip(files, notes):
        logging.info(f"{f}: {n}")


if __name__ == "__main__":
    main()
