"""Average the weights of several checkpoints: ``python -m speech_b200.utils.checkpoint_averaging a.ckpt b.ckpt ... -o avg.ckpt``
or ``--nemo model.nemo --checkpoint-dir dir`` to write an averaged ``.nemo`` (reference: ``scripts/checkpoint_averaging``)."""
from __future__ import annotations

import argparse
import glob
import os
from typing import Dict, List, Sequence

import torch


def average_state_dicts(state_dicts: Sequence[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    n = len(state_dicts)
    if n == 0:
        raise ValueError("nothing to average")
    out: Dict[str, torch.Tensor] = {}
    for k, v in state_dicts[0].items():
        if torch.is_tensor(v) and v.is_floating_point():
            acc = v.detach().double().clone()
            for sd in state_dicts[1:]:
                acc += sd[k].detach().double()
            out[k] = (acc / n).to(v.dtype)
        else:
            out[k] = v.clone() if torch.is_tensor(v) else v       # integer buffers (step counters): keep the first
    return out


def load_weights(path: str) -> Dict[str, torch.Tensor]:
    ck = torch.load(path, map_location="cpu", weights_only=False)
    return ck["state_dict"] if isinstance(ck, dict) and "state_dict" in ck else ck


def main(argv=None):
    ap = argparse.ArgumentParser(prog="speech_b200.utils.checkpoint_averaging")
    ap.add_argument("checkpoints", nargs="*")
    ap.add_argument("--checkpoint-dir", help="average every *.ckpt in this directory (excluding *-last.ckpt)")
    ap.add_argument("--nemo", help="a .nemo file whose weights are replaced by the average")
    ap.add_argument("-o", "--output", required=True)
    a = ap.parse_args(argv)
    paths: List[str] = list(a.checkpoints)
    if a.checkpoint_dir:
        paths += [p for p in sorted(glob.glob(os.path.join(a.checkpoint_dir, "*.ckpt"))) if not p.endswith("-last.ckpt")]
    avg = average_state_dicts([load_weights(p) for p in paths])
    if a.nemo:
        from ..core.modelpt import ModelPT

        model = ModelPT.restore_from(a.nemo, map_location="cpu")
        model.load_state_dict(avg, strict=True)
        model.save_to(a.output)
    else:
        torch.save({"state_dict": avg}, a.output)
    print(f"averaged {len(paths)} checkpoints into {a.output}")


if __name__ == "__main__":
    main()
