"""Train SALM on a device mesh (fully-sharded / hybrid-sharded data parallel x tensor / sequence / context parallel, optional
expert parallelism for mixture-of-experts LLMs).

Usage: torchrun --nproc-per-node 8 examples/speechlm2/salm_automodel_train.py trainer.strategy.tp_size=2 \\
           model.pretrained_llm=/models/qwen model.pretrained_asr=asr.nemo model.train_ds.input_cfg=train.yaml
(reference script: ``examples/speechlm2/salm_train.py`` with ``SALMAutomodel`` and ``AutomodelParallelStrategy``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.speechlm.salm_automodel import SALMAutomodel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="salm_automodel")
def main(cfg):
    run_training(SALMAutomodel, cfg)


if __name__ == "__main__":
    main()
