"""Find the largest batch size per bucket that fits in device memory:
``python -m speech_b200.utils.oomptimizer --config-path conf.yaml --buckets 5.0 10.0 20.0 [--memory-fraction 0.9]``.

For every bucket (max input duration, and max output length from ``--ratio`` tokens per second) the search doubles the batch
size until a training step runs out of memory (or exceeds the memory budget), then bisects; one forward + backward +
optimizer step is executed per probe with synthetic inputs built from the model's ``oomptimizer_schema``.  Prints a
``bucket_batch_size=[...]`` line for the data config (reference: ``scripts/speech_recognition/oomptimizer.py``).  Probes only
catch the allocator's own out-of-memory error; they never push the device beyond the configured budget.
"""
from __future__ import annotations

import argparse
from typing import Callable, List, Optional, Sequence, Tuple

import torch


def find_max_batch(try_step: Callable[[int], bool], start: int = 1, limit: int = 4096) -> int:
    """``try_step(b)`` → True when batch size ``b`` fits.  Exponential growth, then bisection."""
    if not try_step(start):
        return 0
    lo, hi = start, None
    b = start
    while hi is None and b < limit:
        b = min(limit, b * 2)
        if try_step(b):
            lo = b
        else:
            hi = b
    if hi is None:
        return lo
    while hi - lo > max(1, lo // 16):
        mid = (lo + hi) // 2
        if try_step(mid):
            lo = mid
        else:
            hi = mid
    return lo


def make_step_probe(model, optimizer, make_batch: Callable[[int], Tuple], memory_budget_bytes: Optional[int] = None) -> Callable[[int], bool]:
    dev = next(model.parameters()).device

    def probe(b: int) -> bool:
        try:
            if dev.type == "cuda":
                torch.cuda.reset_peak_memory_stats(dev)
            batch = make_batch(b)
            out = model.training_step(batch, 0)
            out["loss"].backward()
            optimizer.step()
            optimizer.zero_grad()
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
                if memory_budget_bytes is not None and torch.cuda.max_memory_allocated(dev) > memory_budget_bytes:
                    return False
            return True
        except torch.cuda.OutOfMemoryError:
            optimizer.zero_grad()
            return False
        finally:
            if dev.type == "cuda":
                torch.cuda.empty_cache()

    return probe


def optimize_buckets(model, optimizer, buckets: Sequence[Tuple[float, int]], sample_rate: int = 16000,
                     memory_fraction: float = 0.9, start: int = 1) -> List[int]:
    from .misc import SequenceLengthResolver

    dev = next(model.parameters()).device
    budget = int(torch.cuda.get_device_properties(dev).total_memory * memory_fraction) if dev.type == "cuda" else None
    resolver = SequenceLengthResolver(model.oomptimizer_schema)
    names = [i["name"] for i in model.oomptimizer_schema["inputs"]]
    out = []
    for dur, toks in buckets:
        def make(b, dur=dur, toks=toks):
            d = resolver(b, int(dur * sample_rate), int(toks), device=dev)
            return tuple(d[n] for n in names)
        out.append(find_max_batch(make_step_probe(model, optimizer, make, budget), start))
    return out


def main(argv=None):
    from ..core.config import OmegaConf
    from ..core.instantiate import resolve_target_path
    import importlib

    ap = argparse.ArgumentParser(prog="speech_b200.utils.oomptimizer")
    ap.add_argument("--config-path", required=True)
    ap.add_argument("--module-name", default="speech_b200.models.EncDecRNNTBPEModel")
    ap.add_argument("--buckets", type=float, nargs="+", required=True, help="bucket upper bounds in seconds")
    ap.add_argument("--ratio", type=float, default=4.0, help="output tokens per second of audio")
    ap.add_argument("--memory-fraction", type=float, default=0.9)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    cfg = OmegaConf.load(a.config_path)
    mod, cls = resolve_target_path(a.module_name).rsplit(".", 1)
    model = getattr(importlib.import_module(mod), cls)(cfg.model if "model" in cfg else cfg).to(a.device).train()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-6)
    sizes = optimize_buckets(model, opt, [(d, max(1, int(d * a.ratio))) for d in a.buckets], memory_fraction=a.memory_fraction)
    print("bucket_duration_bins=[" + ",".join(str(d) for d in a.buckets) + "]")
    print("bucket_batch_size=[" + ",".join(str(s) for s in sizes) + "]")


if __name__ == "__main__":
    main()
