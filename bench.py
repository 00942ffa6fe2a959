#!/usr/bin/env python
"""Headline benchmark: Parakeet-TDT-0.6B-shape training throughput in audio-seconds per second.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run, one rank per GPU)

Model: FastConformer-XL encoder (24 layers, d_model 1024, 8 heads, FFN 4096, conv kernel 9, 8x dw-striding
sub-sampling with 256 channels, 80 mel bins), 2-layer LSTM prediction net (640), joint 640 + ReLU, vocabulary
1024 + blank, TDT durations {0..4}, sigma 0.02, AdamW + Noam warm-up, bf16 activations with fp32 master weights.
Data: synthetic N(0, 0.1^2) waveforms at 16 kHz, durations uniform 10-20 s, duration-bucketed to ~300 s of
audio per GPU per batch, transcripts of uniform-random ids at 3 tokens per second; random-init weights.

Two timed passes of exactly K steps each (after W warm-up steps), both bracketed by barrier + synchronize and
timed with CUDA events, max over ranks:
  * device pass  -> "value": batches already resident on the GPU;
  * end-to-end   -> "e2e":   through ``Trainer.fit``: every step copies its batch from pinned host memory and
                             reads the loss back to the host.
Activations of one step are several GB (>> 126 MB L2), so no explicit L2 flush is needed between steps.

``--impl reference`` reports why the reference framework cannot run here; ``--impl eager`` runs the
"reference-equivalent (eager PyTorch + NCCL)" arm: the same architecture, data and timing protocol built from the library
calls the reference makes (``baseline/reference_equivalent.py``: torch.stft, nn.Conv2d, nn.LSTM, matmul rel-pos attention,
SyncBatchNorm, DistributedDataParallel, torch.optim.AdamW, and the reference's own Numba TDT loss kernels).
"""
from __future__ import annotations

import argparse
import json
import os

# Load every kernel image when its module is loaded instead of on first launch: lazily loaded kernels are paged in from disk the
# first time a shape selects them, which on a freshly started machine lands inside the timed steps.  Must be set before CUDA starts.
os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="native", choices=["native", "eager", "reference"])
    ap.add_argument("--size", default="xlarge")
    ap.add_argument("--layers", type=int, default=None, help="override the number of encoder layers (debug only)")
    ap.add_argument("--batch-seconds", type=float, default=300.0)
    ap.add_argument("--dropout", type=float, default=0.1)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--config", default="tdt", choices=["tdt", "canary_fsdp"],
                    help="tdt: Parakeet-TDT-0.6B-shape, data parallel (the headline); canary_fsdp: Canary-1B-v2-shape AED, fully sharded "
                         "(ZeRO-3) at N > 1, ~600 s of 5-40 s audio per GPU")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            p = [x.strip() for x in l.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_batches(args, rank: int, world: int, vocab: int):
    """Seeded synthetic corpus -> duration-bucketed batches of ~batch_seconds (padded) for this rank, in pinned memory."""
    import numpy as np
    import torch

    g = np.random.default_rng(1234 + rank)
    canary = getattr(args, "config", "tdt") == "canary_fsdp"
    n_utts = 400
    lo, hi = (5.0, 40.0) if canary else (10.0, 20.0)
    durs = g.uniform(lo, hi, size=n_utts)
    edges = np.arange(lo + (5.0 if canary else 1.0), hi + 1e-6, 5.0 if canary else 1.0)
    bucket = np.searchsorted(edges, durs, side="right")
    batches = []
    for b in range(len(edges) + 1):
        idx = np.nonzero(bucket == b)[0]
        if len(idx) == 0:
            continue
        top = float(edges[b]) if b < len(edges) else hi
        per = max(1, int(args.batch_seconds // top))
        for s in range(0, len(idx) - per + 1, per):
            batches.append(idx[s:s + per])
    order = np.random.default_rng(99).permutation(len(batches))
    out = []
    for k in order[:16]:
        ids = batches[k]
        lens = (durs[ids] * 16000).astype(np.int64)
        L = int(lens.max())
        audio = torch.zeros(len(ids), L, dtype=torch.float32)
        ntok = np.maximum(1, np.round(durs[ids] * 3.0)).astype(np.int64) + (6 if canary else 0)
        toks = torch.zeros(len(ids), int(ntok.max()), dtype=torch.long)
        for i, (n, u) in enumerate(zip(lens, ntok)):
            audio[i, :n] = torch.from_numpy((g.standard_normal(n) * 0.1).astype(np.float32))
            if canary:    # six task / language tokens out of 32 special ids, then the transcript
                toks[i, :6] = torch.from_numpy(g.integers(1, 33, size=6))
                toks[i, 6:u] = torch.from_numpy(g.integers(33, vocab, size=u - 6))
            else:
                toks[i, :u] = torch.from_numpy(g.integers(0, vocab, size=u))
        batch = (audio, torch.from_numpy(lens), toks, torch.from_numpy(ntok))
        if torch.cuda.is_available():
            batch = tuple(t.pin_memory() for t in batch)
        out.append((batch, float(durs[ids].sum())))
    return out


def reference_arm():
    """The reference framework installs offline only without its dependencies; importing its core then fails."""
    sys.path.insert(0, os.path.join(REPO, "baseline", "_ref"))
    why = None
    try:
        import nemo.core  # noqa: F401
        import nemo.collections.asr  # noqa: F401
    except Exception as e:  # noqa: BLE001
        why = f"{type(e).__name__}: {e}"
    if why is None:
        why = "reference imported but its Lightning/Hydra/Lhotse training entry point is not runnable offline"
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference installs with --no-deps only; import fails (" + why + "); hydra-core, omegaconf, "
                      "lightning and lhotse are not in the offline wheelhouse"}))


class _Timed:
    """Trainer callback: CUDA events around steps [warmup, warmup+steps), one loss read-back per step."""

    def __init__(self, warmup, steps, durations):
        import torch

        self.warmup, self.steps, self.durations = warmup, steps, durations
        self.t0 = torch.cuda.Event(enable_timing=True)
        self.t1 = torch.cuda.Event(enable_timing=True)
        self.audio = 0.0
        self.losses = []
        self.d2h_bytes = 0
        # loss read-back is pipelined by one step: step i's loss is copied to pinned memory asynchronously and read on the
        # host at the end of step i+1 (the last one at the end of the timed region), so the host never drains the GPU
        # queue in the middle of the run
        self._pending = None
        self._host = torch.zeros(2, dtype=torch.float32).pin_memory()

    # the Trainer calls every hook by name; unknown hooks are simply absent
    def setup(self, trainer, model, stage): ...

    def on_train_batch_start(self, trainer, model, batch, batch_idx):
        import torch
        import torch.distributed as dist

        if batch_idx == self.warmup:
            if dist.is_initialized():
                dist.barrier()
            torch.cuda.synchronize()
            self.t0.record()

    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
        import torch
        import torch.distributed as dist

        loss = outputs["loss"].detach().float()
        if self._pending is not None:
            slot, ev = self._pending
            ev.synchronize()
            self.losses.append(float(self._host[slot]))  # device -> host read of the previous step's result
        slot = batch_idx % 2
        self._host[slot].copy_(loss, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._pending = (slot, ev)
        self.d2h_bytes = 4
        if self.warmup <= batch_idx < self.warmup + self.steps:
            self.audio += self.durations[batch_idx % len(self.durations)]
        if batch_idx == self.warmup + self.steps - 1:
            slot, ev = self._pending
            ev.synchronize()
            self.losses.append(float(self._host[slot]))
            self._pending = None
            self.t1.record()
            torch.cuda.synchronize()
            if dist.is_initialized():
                dist.barrier()


def eager_arm(args, rank, world, local, dev):
    """Reference-equivalent arm: plain loop, same batches, same timing (CUDA events, barrier + synchronize, max over ranks)."""
    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.join(REPO, "baseline"))
    import reference_equivalent as refeq

    torch.manual_seed(0)
    vocab = 1024
    model, step = refeq.build(dev, world, local, args.layers, args.dropout, os.path.join(REPO, "baseline", "_ref"))
    model.train()
    data = make_batches(args, rank, world, vocab)
    batches = [b for b, _ in data]
    durations = [d for _, d in data]
    h2d = sum(sum(t.numel() * t.element_size() for t in b) for b in batches) / len(batches)
    host = torch.zeros(1, dtype=torch.float32).pin_memory()

    def run(e2e: bool):
        resident = None if e2e else [tuple(t.to(dev) for t in b) for b in batches]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        audio, losses = 0.0, []
        sampler = ClockSampler(local)
        for i in range(args.warmup + args.steps):
            if i == args.warmup:
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                sampler.start()
                t0.record()
            k = i % len(batches)
            batch = tuple(t.to(dev, non_blocking=True) for t in batches[k]) if e2e else resident[k]
            loss = step(batch)
            if e2e:
                host.copy_(loss.float().view(1), non_blocking=False)   # the step's result is read on the host every step
                losses.append(float(host[0]))
            elif i in (args.warmup, args.warmup + args.steps - 1):
                losses.append(float(loss))
            if i >= args.warmup:
                audio += durations[k]
        t1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        clocks = sampler.stop()
        return t0.elapsed_time(t1), audio, clocks, losses

    # untimed pass over every batch shape (JIT compilation of the Numba kernels, cuDNN plans, allocator growth)
    saved = (args.warmup, args.steps)
    args.warmup, args.steps = 0, 16          # the same count on every rank (the ranks' batch lists differ in length)
    run(False)
    args.warmup, args.steps = saved
    ms, audio, clocks, losses = run(False)
    ms2, audio2, _, losses2 = (0.0, 0.0, None, []) if args.no_e2e else run(True)
    stats = torch.tensor([ms, audio, ms2, audio2], device=dev, dtype=torch.float64)
    if world > 1:
        mx, sm = stats.clone(), stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, audio, ms2, audio2 = float(mx[0]), float(sm[1]), float(mx[2]), float(sm[3])
    if rank == 0:
        out = {"metric": "TDT-0.6B train audio-sec/s", "value": round(audio / (ms / 1e3), 2), "unit": "audio-seconds/s",
               "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
               "impl": "eager", "label": "reference-equivalent (eager PyTorch + NCCL)",
               "config": {"model": "FastConformer-xlarge-TDT (24L d1024 8h ffn4096 k9, 2xLSTM640, joint640, vocab1024, durations 0-4, "
                                   "sigma 0.02)" if args.layers is None else f"DEBUG layers={args.layers}",
                          "global_batch": f"~{args.batch_seconds:.0f} s audio per GPU", "parallelism": f"dp{world}",
                          "dropout": args.dropout, "prednet_dropout": 0.0, "joint_dropout": 0.0,
                          "attention": "sdpa" if os.environ.get("REFEQ_SDPA", "0") == "1" else "matmul + rel_shift + softmax",
                          "loss": model.loss_kind, "fused_batch_size": model.fused,
                          "ddp": "torch DistributedDataParallel, 25 MB buckets, SyncBatchNorm" if world > 1 else "single process",
                          "optimizer": "torch.optim.AdamW + Noam, clip_grad_norm_ 1.0",
                          "l2": "no flush: per-step activations are several GB, far larger than the 126 MB L2"},
               "clocks": clocks, "gpu_launches": 0, "loss_first_last": [round(losses[0], 3), round(losses[-1], 3)]}
        if not args.no_e2e:
            out["e2e"] = {"value": round(audio2 / (ms2 / 1e3), 2), "unit": "audio-seconds/s", "h2d_bytes_per_step": int(h2d),
                          "d2h_bytes_per_step": 4, "ms_per_step": round(ms2 / args.steps, 3)}
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if os.environ.get("SPEECH_B200_BENCH_WATCHDOG"):
        # dumps every thread's Python stack if the run is still going after that many seconds (where a hang sits)
        import faulthandler

        faulthandler.dump_traceback_later(float(os.environ["SPEECH_B200_BENCH_WATCHDOG"]), repeat=True)
    if args.impl == "reference":
        return reference_arm()
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world)
    if args.impl == "eager":
        return eager_arm(args, rank, world, local, dev)
    # at N > 1 the gradient exchange must be the peer-memory kernel: a silent fall-back to NCCL would benchmark the baseline
    os.environ.setdefault("SPEECH_B200_PEER_ALLREDUCE_STRICT", "1")

    from speech_b200 import ops
    from speech_b200.core.trainer import Trainer
    from speech_b200.models import EncDecRNNTBPEModel
    from speech_b200.models.configs import fastconformer_transducer_config

    if args.impl == "native":
        ops.native.load()
    torch.manual_seed(0)
    canary = args.config == "canary_fsdp"
    if canary:
        from speech_b200.models.aed_models import EncDecMultiTaskModel
        from speech_b200.models.configs import canary_aed_config

        vocab = 16384
        if args.batch_seconds == 300.0:
            args.batch_seconds = 600.0
        cfg = canary_aed_config("xlarge", enc_layers=args.layers or 32, vocab_size=vocab, dropout=args.dropout,
                                optim_name="fully_sharded_adamw" if world > 1 else "adamw")
        model = EncDecMultiTaskModel(cfg)
    else:
        vocab = 1024
        cfg = fastconformer_transducer_config(args.size, vocab_size=vocab, dropout=args.dropout, loss="tdt", durations=(0, 1, 2, 3, 4),
                                              sigma=0.02, n_layers=args.layers, lr=5.0, sched="noam")
        model = EncDecRNNTBPEModel(cfg)
    data = make_batches(args, rank, world, vocab)
    batches = [b for b, _ in data]
    durations = [d for _, d in data]
    total_steps = args.warmup + args.steps
    h2d = sum(sum(t.numel() * t.element_size() for t in b) for b in batches) / len(batches)

    class Loader:
        def __init__(self, n):
            self.n = n

        def __len__(self):
            return self.n

        def __iter__(self):
            for i in range(self.n):
                yield batches[i % len(batches)]

    def run(e2e: bool):
        """K timed steps after W warm-up steps; returns (ms, audio seconds, launches, clocks)."""
        trainer = run.trainer
        timed = _Timed(args.warmup, args.steps, durations)
        trainer.callbacks = [timed]
        trainer.max_steps = trainer.global_step + total_steps
        if e2e:
            loader = Loader(total_steps)
        else:
            resident = [tuple(t.to(dev) for t in b) for b in batches]
            torch.cuda.synchronize()

            class Resident(Loader):
                def __iter__(self):
                    for i in range(self.n):
                        yield resident[i % len(resident)]

            loader = Resident(total_steps)
        model._train_dl = loader
        sampler = ClockSampler(local)
        launches0 = ops.native.launch_count if args.impl == "native" else 0
        sampler.start()
        trainer._fit_loop() if run.started else trainer.fit(model, train_dataloaders=loader)
        run.started = True
        clocks = sampler.stop()
        ms = timed.t0.elapsed_time(timed.t1)
        launches = (ops.native.launch_count - launches0) if args.impl == "native" else 0
        launches = int(launches * args.steps / total_steps)
        return ms, timed.audio, launches, clocks, timed.losses

    run.trainer = Trainer(max_steps=total_steps, precision="bf16-mixed", gradient_clip_val=1.0, log_every_n_steps=10 ** 9,
                          accelerator="gpu", sync_batchnorm=True, enable_checkpointing=False, logger=False)
    run.started = False
    # The 16 batches have 16 different shapes and only the first W of them are seen during warm-up: reserve the device memory
    # pool once (one large block handed back to the caching allocator, which then carves every later request out of it), so that
    # the first visit of a shape inside the timed region does not go to the driver for memory.
    if args.impl == "native" and os.environ.get("SPEECH_B200_BENCH_PRIME", "1") != "0":
        # bucketed batches: the shapes are known up front, so the convolution plans of the sub-sampling front end are built here
        model.to(dev)
        hop = 160
        shapes = sorted({(int(b[0].shape[0]), int(b[0].shape[1]) // hop + 1) for b in batches})
        model.encoder.pre_encode.prime_shapes(shapes, dev, torch.bfloat16)
        torch.cuda.synchronize()
    reserve_gb = float(os.environ.get("SPEECH_B200_BENCH_RESERVE_GB", "72"))
    if reserve_gb > 0:
        free_b, _ = torch.cuda.mem_get_info(dev)
        n = int(min(reserve_gb * 2 ** 30, 0.6 * free_b))
        block = torch.empty(n, dtype=torch.uint8, device=dev)
        del block

    # untimed pass over every batch shape: neither timed pass is the one that meets a shape (or a kernel image) first
    saved = (args.warmup, args.steps)
    n_pre = int(os.environ.get("SPEECH_B200_BENCH_PREPASS", "16"))
    args.warmup, args.steps = 0, n_pre       # the same count on every rank (the ranks' batch lists differ in length)
    total_steps = n_pre
    if n_pre > 0:
        run(e2e=False)
    run.trainer.current_epoch = 0
    args.warmup, args.steps = saved
    total_steps = args.warmup + args.steps
    allreduce_check = None
    if world > 1 and canary:
        gs = None
        if type(run.trainer.grad_sync).__name__ != "FSDP2GradSync":
            raise SystemExit(f"bench.py: strategy is {type(run.trainer.grad_sync).__name__}, not the fully-sharded engine")
    elif world > 1:
        gs = run.trainer.grad_sync
        if type(gs).__name__ != "PeerGradSync":
            if os.environ.get("SPEECH_B200_PEER_ALLREDUCE", "1") == "1":
                raise SystemExit(f"bench.py: gradient exchange is {type(gs).__name__}, not the peer-memory kernel")
            gs = None       # NCCL all-reduce requested explicitly (comparison runs): reported as such in config.grad_exchange
    if world > 1 and gs is not None:
        # first bucket of the peer all-reduce against NCCL on the same data
        n = gs.buckets[0]["view"].numel()
        g = torch.Generator(device=dev).manual_seed(4321 + rank)
        x = torch.randn(n, device=dev, generator=g)
        want = x / world
        dist.all_reduce(want)
        got = x.clone()
        gs.comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(gs.comm_stream):
            gs.reducer(got, 1.0 / world)
        torch.cuda.current_stream().wait_stream(gs.comm_stream)
        torch.cuda.synchronize()
        err = ((got - want).abs().max() / want.abs().max()).reshape(1)
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        allreduce_check = {"elements": int(n), "max_rel_err_vs_nccl": float(err), "note": "bf16 exchange: expected ~4e-3"}
    ms, audio, launches, clocks, losses = run(e2e=False)
    run.trainer.current_epoch = 0
    e2e = None
    if not args.no_e2e:
        ms2, audio2, _, _, losses2 = run(e2e=True)
    stats = torch.tensor([ms, audio, ms2 if not args.no_e2e else 0.0, audio2 if not args.no_e2e else 0.0], device=dev,
                         dtype=torch.float64)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, audio = float(mx[0]), float(sm[1])
        ms2, audio2 = float(mx[2]), float(sm[3])
    value = audio / (ms / 1e3)
    if args.impl == "native":
        ops.native.check_status()
    if rank == 0:
        out = {
            "metric": "Canary-1B AED train audio-sec/s" if canary else "TDT-0.6B train audio-sec/s", "value": round(value, 2),
            "unit": "audio-seconds/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": args.impl,
            "config": {"model": (("Canary-1B-v2 shape: FastConformer 32L d1024 8h ffn4096 k9 + Transformer decoder 8L d1024 16h ffn4096, vocab 16384, "
                                  "label smoothing 0.1") if canary else
                                 (f"FastConformer-{args.size}-TDT (24L d1024 8h ffn4096 k9, 2xLSTM640, joint640, vocab1024, "
                                  f"durations 0-4, sigma 0.02)")) if args.layers is None else f"DEBUG layers={args.layers}",
                       "global_batch": f"~{args.batch_seconds:.0f} s audio per GPU" + ("" if canary else " (15-27 utterances of 10-20 s)"),
                       "seq_len": "5-40 s audio, 6 prompt + ~3 tokens/s" if canary else "10-20 s audio = 125-250 encoder frames, 30-60 tokens",
                       "parallelism": (f"fsdp2 (ZeRO-3) over {world}" if (canary and world > 1) else f"dp{world}"), "dropout": args.dropout,
                       "prednet_dropout": None if canary else float(cfg.decoder.prednet.get("dropout", 0.0)),
                       "joint_dropout": None if canary else float(cfg.joint.jointnet.get("dropout", 0.0)),
                       "grad_exchange": (f"{type(run.trainer.grad_sync).__name__}: {run.trainer.grad_sync.launched_in_backward} of "
                                         f"{len(run.trainer.grad_sync.buckets)} buckets launched during backward"
                                         + (f", {run.trainer.grad_sync.reducer.ctas} CTAs" if hasattr(run.trainer.grad_sync, "reducer") else ""))
                       if world > 1 else "none",
                       "optimizer": (("fully sharded AdamW (ZeRO-3), constant lr 3e-4, clip 1.0" if world > 1 else "AdamW, constant lr 3e-4, clip 1.0")
                                     if canary else "AdamW+Noam, clip 1.0"),
                       "l2": "no flush: per-step activations are several GB, far larger than the 126 MB L2"},
            "clocks": clocks, "gpu_launches": launches,
            "loss_first_last": [round(losses[0], 3), round(losses[-1], 3)],
        }
        if allreduce_check is not None:
            out["allreduce_check"] = allreduce_check
        if canary and world > 1:
            out["fsdp_memory"] = run.trainer.optimizers[0].memory_report()
        if not args.no_e2e:
            out["e2e"] = {"value": round(audio2 / (ms2 / 1e3), 2), "unit": "audio-seconds/s", "h2d_bytes_per_step": int(h2d),
                          "d2h_bytes_per_step": 4, "ms_per_step": round(ms2 / args.steps, 3)}
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
