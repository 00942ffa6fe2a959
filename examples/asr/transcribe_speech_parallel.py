"""Transcribe a manifest on all GPUs of a node: one rank per GPU, the manifest split by rank, one prediction file per rank and a
merged file written by rank 0 (with WER when the manifest has references).

python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/asr/transcribe_speech_parallel.py \
    model_path=model.nemo dataset_manifest=test.json output_dir=preds batch_size=32
(reference script: ``examples/asr/transcribe_speech_parallel.py``)."""
import json
import os

import torch
import torch.distributed as dist

from speech_b200 import ops
from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "dataset_manifest": None, "output_dir": "preds", "batch_size": 32,
                                            "compute_dtype": "bfloat16"}), cfg)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if cuda else torch.device("cpu")
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    model = ASRModel.restore_from(cfg.model_path, map_location=str(dev)).to(dev).eval()
    items = read_manifest(cfg.dataset_manifest)
    # longest first inside a rank keeps the padding low; round-robin over the sorted list balances the ranks
    order = sorted(range(len(items)), key=lambda i: -float(items[i].get("duration", 0.0) or 0.0))
    mine = order[rank::world]
    cdt = torch.bfloat16 if cuda and str(cfg.compute_dtype) == "bfloat16" else None
    with ops.compute_dtype(cdt):
        hyps = model.transcribe([items[i]["audio_filepath"] for i in mine], batch_size=int(cfg.batch_size))
    os.makedirs(cfg.output_dir, exist_ok=True)
    part = os.path.join(cfg.output_dir, f"predictions_rank{rank}.json")
    with open(part, "w", encoding="utf-8") as f:
        for i, h in zip(mine, hyps):
            f.write(json.dumps(dict(items[i], pred_text=h.text if hasattr(h, "text") else h, index=i), ensure_ascii=False) + "\n")
    if world > 1:
        dist.barrier()
    if rank == 0:
        rows = []
        for r in range(world):
            with open(os.path.join(cfg.output_dir, f"predictions_rank{r}.json"), encoding="utf-8") as f:
                rows += [json.loads(l) for l in f if l.strip()]
        rows.sort(key=lambda x: x["index"])
        with open(os.path.join(cfg.output_dir, "predictions_all.json"), "w", encoding="utf-8") as f:
            for x in rows:
                f.write(json.dumps(x, ensure_ascii=False) + "\n")
        if rows and rows[0].get("text"):
            logging.info(f"WER: {100 * word_error_rate([x['pred_text'] for x in rows], [x['text'] for x in rows]):.2f}%")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
