"""Smaller runtime utilities: sharded checkpoint IO with asynchronous finalisation, bf16-without-autocast precision, step-delta
timing, a sweep launcher, lifecycle telemetry, punctuation error rate.

Reference: ``utils/callbacks/dist_ckpt_io.py:72-202`` (sharded save / load + async finalize), ``utils/trainer_utils.py:115``
(``FlashPrecision``: ``bf16-flash`` casts the model once and runs without autocast), ``utils/exp_manager.py:414-469``
(``DeltaTimingCallback``), ``core/utils/process_launcher/launcher.py`` (multirun launcher), ``lightning/one_logger_callback.py``
(telemetry fan-out), ``collections/common/metrics/punct_er.py`` (punctuation error rates).
"""
from __future__ import annotations

import json
import os
import subprocess
import threading
import time
from collections import Counter
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch


# ------------------------------------------------------------------------------------------------ sharded checkpoint IO
class DistributedCheckpointIO:
    """Every rank writes the tensors it owns; rank 0 writes the index.  ``state`` maps names to tensors; ``owner(name)`` tells which
    rank stores a replicated tensor (default: a stable hash of the name, which spreads a replicated model over the ranks), while
    tensors listed in ``sharded`` are stored by every rank as its own piece (``name@rank``) and concatenated on load along
    ``sharded[name]``.  With ``async_save`` the file write happens on a background thread from a CPU copy taken synchronously;
    ``finalize()`` joins outstanding writes and only then publishes the index, so a directory with an index is complete."""

    def __init__(self, rank: int = 0, world_size: int = 1, async_save: bool = False, barrier: Optional[Callable[[], None]] = None):
        self.rank, self.world, self.async_save, self.barrier = rank, world_size, async_save, barrier
        self._pending: List[threading.Thread] = []
        self._index: Optional[Tuple[str, Dict[str, Any]]] = None

    @staticmethod
    def _owner(name: str, world: int) -> int:
        return sum(name.encode()) % world

    def save_checkpoint(self, state: Dict[str, torch.Tensor], path: str, sharded: Optional[Dict[str, int]] = None, extra: Optional[dict] = None) -> None:
        os.makedirs(path, exist_ok=True)
        sharded = sharded or {}
        mine = {}
        for k, v in state.items():
            if k in sharded:
                mine[f"{k}@{self.rank}"] = v.detach().to("cpu", copy=True)
            elif self._owner(k, self.world) == self.rank:
                mine[k] = v.detach().to("cpu", copy=True)
        fname = os.path.join(path, f"shard_{self.rank:05d}_of_{self.world:05d}.pt")

        def write():
            torch.save(mine, fname + ".tmp")
            os.replace(fname + ".tmp", fname)

        if self.async_save:
            t = threading.Thread(target=write, daemon=True)
            t.start()
            self._pending.append(t)
        else:
            write()
        index = {"world_size": self.world, "sharded": sharded, "names": sorted(state), "extra": extra or {}}
        self._index = (path, index)
        if not self.async_save:
            self.finalize()

    def finalize(self) -> None:
        for t in self._pending:
            t.join()
        self._pending.clear()
        if self.barrier is not None:
            self.barrier()
        if self._index is not None and self.rank == 0:
            path, index = self._index
            with open(os.path.join(path, "index.json.tmp"), "w") as f:
                json.dump(index, f)
            os.replace(os.path.join(path, "index.json.tmp"), os.path.join(path, "index.json"))
        self._index = None

    @staticmethod
    def is_complete(path: str) -> bool:
        return os.path.exists(os.path.join(path, "index.json"))

    @staticmethod
    def load_checkpoint(path: str, map_location="cpu") -> Tuple[Dict[str, torch.Tensor], dict]:
        """Full (unsharded) state, whatever the number of ranks that wrote it."""
        with open(os.path.join(path, "index.json")) as f:
            index = json.load(f)
        W = int(index["world_size"])
        parts: Dict[str, torch.Tensor] = {}
        for r in range(W):
            parts.update(torch.load(os.path.join(path, f"shard_{r:05d}_of_{W:05d}.pt"), map_location=map_location))
        out = {}
        for name in index["names"]:
            if name in index["sharded"]:
                out[name] = torch.cat([parts[f"{name}@{r}"] for r in range(W)], dim=int(index["sharded"][name]))
            else:
                out[name] = parts[name]
        return out, index.get("extra", {})


# ------------------------------------------------------------------------------------------------ precision
class FlashPrecision:
    """``bf16-flash``: parameters and buffers are cast to bf16 ONCE (normalisation layers and anything matching ``keep_fp32`` stay
    fp32), the forward runs without autocast, and the optimizer keeps its own fp32 state.  Batches are cast on the way in, except
    tensors whose key contains ``audio`` (waveforms keep fp32 for the front-end)."""

    precision = "bf16-flash"

    def __init__(self, keep_fp32: Sequence[str] = ("norm", "bn", "batch_norm")):
        self.keep = tuple(keep_fp32)

    def convert_module(self, module: torch.nn.Module) -> torch.nn.Module:
        for name, p in module.named_parameters():
            if p.is_floating_point() and not any(k in name.lower() for k in self.keep):
                p.data = p.data.to(torch.bfloat16)
        for name, b in module.named_buffers():
            if b.is_floating_point() and not any(k in name.lower() for k in self.keep):
                b.data = b.data.to(torch.bfloat16)
        return module

    def convert_input(self, batch):
        if isinstance(batch, dict):
            return {k: (v if "audio" in k or not torch.is_tensor(v) or not v.is_floating_point() else v.to(torch.bfloat16)) for k, v in batch.items()}
        if isinstance(batch, (list, tuple)):
            return type(batch)(self.convert_input(b) if isinstance(b, (dict, list, tuple)) else b for b in batch)
        return batch

    def forward_context(self):
        import contextlib

        return contextlib.nullcontext()


# ------------------------------------------------------------------------------------------------ timing / telemetry
class DeltaTimingCallback:
    """Logs the wall time between the ends of consecutive training (and validation) batches: includes data loading and everything
    else between steps, which per-step timers miss."""

    def __init__(self, clock: Callable[[], float] = time.perf_counter):
        self.clock, self._last = clock, {}

    def _tick(self, trainer, key: str):
        now = self.clock()
        prev = self._last.get(key)
        self._last[key] = now
        if prev is not None and hasattr(trainer, "callback_metrics"):
            trainer.callback_metrics[f"{key}_step_timing in s"] = now - prev

    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
        self._tick(trainer, "train")

    def on_validation_batch_end(self, trainer, model, outputs, batch, batch_idx, dataloader_idx=0):
        self._tick(trainer, "validation")

    def on_train_epoch_start(self, trainer, model):
        self._last.pop("train", None)


class TelemetryCallback:
    """Application life-cycle events (model / data / optimizer initialisation, checkpoint load / save, train start / end, app end)
    appended as JSON lines; plugs into ``CallbackGroup`` fan-out or a Trainer's callbacks."""

    EVENTS = ("on_app_start", "on_model_init_start", "on_model_init_end", "on_dataloader_init_start", "on_dataloader_init_end",
              "on_optimizer_init_start", "on_optimizer_init_end", "on_load_checkpoint_start", "on_load_checkpoint_end",
              "on_save_checkpoint_start", "on_save_checkpoint_end", "on_train_start", "on_train_end", "on_app_end")

    def __init__(self, path: Optional[str] = None, clock: Callable[[], float] = time.time, sink: Optional[Callable[[dict], None]] = None):
        self.path, self.clock, self.sink = path, clock, sink
        self.records: List[dict] = []
        for ev in self.EVENTS:
            setattr(self, ev, self._make(ev))

    def _make(self, ev: str):
        def hook(*args, **kw):
            rec = {"event": ev, "time": self.clock(), **{k: v for k, v in kw.items() if isinstance(v, (int, float, str, bool))}}
            self.records.append(rec)
            if self.sink is not None:
                self.sink(rec)
            if self.path:
                with open(self.path, "a") as f:
                    f.write(json.dumps(rec) + "\n")
        return hook

    def durations(self) -> Dict[str, float]:
        """Seconds between every ``*_start`` and its ``*_end``."""
        start, out = {}, {}
        for r in self.records:
            if r["event"].endswith("_start"):
                start[r["event"][:-6]] = r["time"]
            elif r["event"].endswith("_end") and r["event"][:-4] in start:
                out[r["event"][3:-4]] = r["time"] - start.pop(r["event"][:-4])
        return out


# ------------------------------------------------------------------------------------------------ sweep launcher
class ProcessLauncher:
    """Runs one process per override set (a multirun sweep), at most ``max_parallel`` at a time, each pinned to one entry of
    ``gpu_ids`` through ``CUDA_VISIBLE_DEVICES``.  Returns ``[(overrides, return code, log path)]`` in submission order."""

    def __init__(self, base_cmd: Sequence[str], gpu_ids: Optional[Sequence[int]] = None, max_parallel: Optional[int] = None, log_dir: str = "multirun",
                 env: Optional[Dict[str, str]] = None):
        self.base, self.gpus = list(base_cmd), list(gpu_ids) if gpu_ids is not None else [None]
        self.max_parallel = max_parallel or len(self.gpus)
        self.log_dir, self.env = log_dir, dict(env or {})

    @staticmethod
    def expand_sweep(sweep: Dict[str, Sequence[Any]]) -> List[List[str]]:
        """``{"a": [1, 2], "b": ["x"]}`` -> ``[["a=1", "b=x"], ["a=2", "b=x"]]`` (Cartesian product, first key slowest)."""
        out: List[List[str]] = [[]]
        for k, vals in sweep.items():
            out = [o + [f"{k}={v}"] for o in out for v in vals]
        return out

    def launch(self, jobs: Sequence[Sequence[str]], timeout: Optional[float] = None) -> List[Tuple[List[str], int, str]]:
        os.makedirs(self.log_dir, exist_ok=True)
        results: List[Optional[Tuple[List[str], int, str]]] = [None] * len(jobs)
        free = list(range(min(self.max_parallel, len(self.gpus))))
        running: Dict[int, Tuple[subprocess.Popen, int, Any]] = {}
        nxt = 0
        while nxt < len(jobs) or running:
            while nxt < len(jobs) and free:
                slot = free.pop()
                env = dict(os.environ, **self.env)
                if self.gpus[slot] is not None:
                    env["CUDA_VISIBLE_DEVICES"] = str(self.gpus[slot])
                log = os.path.join(self.log_dir, f"job_{nxt:04d}.log")
                fh = open(log, "w")
                running[nxt] = (subprocess.Popen(self.base + list(jobs[nxt]), stdout=fh, stderr=subprocess.STDOUT, env=env), slot, fh)
                results[nxt] = (list(jobs[nxt]), -1, log)
                nxt += 1
            done = [j for j, (p, _, _) in running.items() if p.poll() is not None]
            if not done:
                time.sleep(0.02)
                if timeout is not None:
                    timeout -= 0.02
                    if timeout <= 0:
                        for p, _, _ in running.values():
                            p.kill()            # the exact processes started above
                        timeout = None
                continue
            for j in done:
                p, slot, fh = running.pop(j)
                fh.close()
                results[j] = (results[j][0], int(p.returncode), results[j][2])
                free.append(slot)
        return [r for r in results if r is not None]


# ------------------------------------------------------------------------------------------------ punctuation error rate
def punctuation_error_rate(hypotheses: Sequence[str], references: Sequence[str], marks: str = ".,?") -> Dict[str, Any]:
    """Aligns the word sequences and compares the punctuation mark that follows each aligned word.  Per mark and overall:
    ``correct``, ``substitutions``, ``deletions`` (mark missing in the hypothesis), ``insertions`` and
    ``per = (S + D + I) / (C + S + D + I)``."""
    from .asr_evaluator import align_words

    def split(s: str):
        words, puncts = [], []
        for tok in s.split():
            m = ""
            while tok and tok[-1] in marks:
                m, tok = tok[-1], tok[:-1]
            if tok:
                words.append(tok.lower())
                puncts.append(m)
            elif words and m:
                puncts[-1] = m
        return words, puncts

    stats = {m: Counter() for m in marks}
    for h, r in zip(hypotheses, references):
        hw, hp = split(h)
        rw, rp = split(r)
        i = j = 0
        for op, _, _ in align_words(rw, hw):
            a = rp[i] if op in ("ok", "sub", "del") else ""
            b = hp[j] if op in ("ok", "sub", "ins") else ""
            i += op in ("ok", "sub", "del")
            j += op in ("ok", "sub", "ins")
            if a and a == b:
                stats[a]["correct"] += 1
            elif a and b:
                stats[a]["substitutions"] += 1
            elif a:
                stats[a]["deletions"] += 1
            elif b:
                stats[b]["insertions"] += 1
    out: Dict[str, Any] = {}
    tot = Counter()
    for m, c in stats.items():
        n = sum(c.values())
        out[m] = {**{k: c[k] for k in ("correct", "substitutions", "deletions", "insertions")}, "per": (n - c["correct"]) / n if n else 0.0}
        tot.update(c)
    n = sum(tot.values())
    out["overall"] = {**{k: tot[k] for k in ("correct", "substitutions", "deletions", "insertions")}, "per": (n - tot["correct"]) / n if n else 0.0}
    return out
