"""SALM training benchmark: speech-LLM of the Canary-Qwen-2.5B shape (FastConformer-xlarge 32-layer audio encoder + Qwen3-1.7B-shape
decoder-only LLM, random weights, bf16) on synthetic conversations; reports LLM input tokens per second.

    python bench_salm.py --steps 10 --warmup 3                                   # one GPU, replicated AdamW
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        bench_salm.py --gpus N --tp T --steps 10 --warmup 3                      # dp_shard = N / T fully sharded, tp = T

One conversation = a user turn with one audio clip of 5-20 s (12.5 audio tokens per second after 8x sub-sampling of 10 ms frames)
plus a short text prompt, and an assistant turn of ~3 tokens per second of audio.  A step = forward + backward + optimizer update
of ``--batch-tokens`` LLM positions per GPU.  Timed with CUDA events on the training stream between a barrier and a synchronize on
both sides, max over ranks; the value is the total over all GPUs.  Inputs are copied from pinned host memory every step and the
loss is read back every step (the timed region is the end-to-end step).
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch-tokens", type=int, default=8192)
    ap.add_argument("--llm-layers", type=int, default=28)
    ap.add_argument("--enc-layers", type=int, default=32)
    ap.add_argument("--sequence-parallel", action="store_true")
    ap.add_argument("--packed", action="store_true")
    ap.add_argument("--impl", default="native", choices=["native", "eager"],
                    help="eager: the reference-equivalent arm (eager PyTorch Conformer + Hugging Face Qwen3 + torch AdamW), one GPU")
    ap.add_argument("--profile", default="", help="after the timed steps, run two more under torch.profiler and write the top kernels by device time to this file")
    ap.add_argument("--smoke-cpu", action="store_true", help="tiny model on the CPU, host clock: checks the script, measures nothing")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    cpu = args.smoke_cpu
    dev = torch.device("cpu") if cpu else torch.device("cuda", local)
    if not cpu:
        torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("gloo") if cpu else dist.init_process_group("nccl", device_id=dev)
    from bench import ClockSampler
    from speech_b200 import ops
    from speech_b200.core.config import OmegaConf
    from speech_b200.models.configs import encoder_cfg, preprocessor_cfg
    from speech_b200.parallel.mesh import DeviceMesh
    from speech_b200.speechlm.data import SALMDataset
    from speech_b200.speechlm.salm_automodel import SALMAutomodel
    from speech_b200.tokenizers import ByteLevelTokenizer

    torch.manual_seed(0)
    llm = dict(vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=args.llm_layers, num_attention_heads=16,
               num_key_value_heads=8, head_dim=128, tie_word_embeddings=True, qk_norm=True, model_type="qwen3")
    pc = {"preprocessor": preprocessor_cfg(128), "encoder": encoder_cfg("xlarge", 128, 0.1, 0.1, n_layers=args.enc_layers),
          "modality_adapter": {"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 1024}}
    if cpu:
        llm = dict(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                   head_dim=8, tie_word_embeddings=True, qk_norm=True, model_type="qwen3")
        pc = {"preprocessor": preprocessor_cfg(32), "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
              "modality_adapter": {"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 176}}
    sharded = world // args.tp > 1
    cfg = OmegaConf.create({"audio_locator_tag": "<|audioplaceholder|>", "prompt_format": "qwen", "llm": llm, "perception": pc,
                            "freeze_params": [], "prevent_freeze_params": [], "sequence_parallel": bool(args.sequence_parallel),
                            "packed_sequences": {"enabled": bool(args.packed), "row_len": None},
                            "optim": {"name": "fully_sharded_adamw" if sharded else "adamw", "lr": 1e-4, "weight_decay": 0.01}})
    tok = ByteLevelTokenizer(special_tokens=["<pad>", "<s>", "</s>", "<|im_start|>", "<|im_end|>"])
    model = SALMAutomodel(cfg, tokenizer=tok)
    eager = None
    if args.impl == "eager":
        if world > 1:
            raise SystemExit("the reference-equivalent arm of this benchmark runs on one GPU")
        import sys

        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
        from reference_equivalent import RefEqSALM

        # the native model above is kept only for its tokenizer / prompt formatter / batch assembly; it never runs
        eager = RefEqSALM(llm, enc_layers=(1 if cpu else args.enc_layers), d_model=(176 if cpu else 1024), n_mels=(32 if cpu else 128),
                          dropout=0.1, placeholder_id=model.audio_locator_tag_id, pad_id=model.text_pad_id)
    mesh = None
    if world > 1:
        mesh = DeviceMesh({"dp_shard": world // args.tp, "tp": args.tp})
        model.configure_model(mesh)
    dp_rank = mesh.rank("dp_shard") if mesh is not None else 0
    n_params = sum(p.numel() for p in model.parameters())

    # synthetic conversations, packed greedily into batches of <= batch_tokens LLM positions
    rng = np.random.default_rng(1234 + dp_rank)
    words = ["alpha", "beta", "gamma", "delta", "kappa", "sigma", "omega", "theta"]
    convs = []
    for i in range(12 if cpu else 160):
        d = float(rng.uniform(0.5, 1.0) if cpu else rng.uniform(5.0, 20.0))
        n_ans = max(1, int(3.0 * d / 2))
        convs.append({"id": f"c{i}", "conversations": [
            {"from": "User", "type": "text", "value": "Transcribe the following:"},          # the audio turn below adds the locator tag
            {"from": "User", "type": "audio", "value": (rng.standard_normal(int(d * 16000)) * 0.1).astype(np.float32), "duration": d},
            {"from": "Assistant", "type": "text", "value": " ".join(rng.choice(words, n_ans))}]})
    ds = SALMDataset(convs, tok, model.prompt_formatter(), cfg.audio_locator_tag, model.text_pad_id)
    batches, cur, cur_tok = [], [], 0
    for i in range(len(ds)):
        n = int(ds.cost(i)) + 24
        if cur and (len(cur) + 1) * max(cur_tok, n) > args.batch_tokens:
            batches.append(ds.collate([ds[j] for j in cur]))
            cur, cur_tok = [], 0
        cur.append(i)
        cur_tok = max(cur_tok, n)
        if len(batches) >= 8:
            break
    if cur and not batches:
        batches.append(ds.collate([ds[j] for j in cur]))
    batches = [{k: (v.pin_memory() if (torch.is_tensor(v) and not cpu) else v) for k, v in b.items()} for b in batches[:8]]
    h2d = sum(sum(v.numel() * v.element_size() for v in b.values() if torch.is_tensor(v)) for b in batches) / len(batches)

    if eager is not None:
        n_params = sum(p.numel() for p in eager.parameters())
        eager.to(dev).train()
        eopt = torch.optim.AdamW(eager.parameters(), lr=1e-4, weight_decay=0.01)
    else:
        model.to(dev)
    model.train()
    import types

    object.__setattr__(model, "_trainer", types.SimpleNamespace(gradient_clip_val=1.0, global_step=0))    # clip value for the optimizer
    if eager is None:
        model.setup_optimization()
    opt = model._optimizer if eager is None else None
    sync = None
    if world > 1:
        from speech_b200.parallel.ddp import build_grad_sync

        sync = build_grad_sync(model, [opt], "auto", mesh.size("dp_shard"), dev) if sharded else None
    cdt = torch.bfloat16
    tokens_done = torch.zeros((), dtype=torch.float64, device=dev)
    host_loss = torch.zeros(1) if cpu else torch.zeros(1).pin_memory()

    def eager_step(i: int, count: bool):
        import contextlib

        b = {k: (v.to(dev, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batches[i % len(batches)].items()}
        with (contextlib.nullcontext() if cpu else torch.autocast("cuda", dtype=cdt)):
            loss, positions = eager(b["audios"], b["audio_lens"], b["input_ids"], b["loss_mask"])
        loss.backward()
        torch.nn.utils.clip_grad_norm_(eager.parameters(), 1.0)
        eopt.step()
        eopt.zero_grad(set_to_none=True)
        host_loss.copy_(loss.detach().float().view(1), non_blocking=True)
        if count:
            tokens_done.add_(float(positions))
        return {"loss": loss}

    def step(i: int, count: bool):
        if eager is not None:
            return eager_step(i, count)
        b = {k: (v.to(dev, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batches[i % len(batches)].items()}
        if sync is not None:
            sync.begin_step()
        import contextlib

        with (contextlib.nullcontext() if cpu else ops.compute_dtype(cdt)), (contextlib.nullcontext() if cpu else torch.autocast("cuda", dtype=cdt)):
            out = model.training_step(b, i)
        out["loss"].backward()
        model.on_after_backward()
        if sync is not None:
            sync.finish_step()
        if not getattr(opt, "max_grad_norm", 0.0):
            model.configure_gradient_clipping(opt, 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        host_loss.copy_(out["loss"].detach().float().view(1), non_blocking=True)
        if count:
            tokens_done.add_(float(model._logged_tokens))
        return out

    # positions processed per step = batch x sequence length of the LLM input (logged by the model)
    orig_log = model.log_dict
    def log_dict(d, *a, **k):
        model._logged_tokens = d.get("batch_size", 0.0) * d.get("sequence_length", 0.0)
    model.log_dict = log_dict

    for i in range(args.warmup):
        step(i, False)
    if world > 1:
        dist.barrier()
    losses = []
    if cpu:
        import time

        h0 = time.perf_counter()
        for i in range(args.warmup, args.warmup + args.steps):
            step(i, True)
            losses.append(float(host_loss[0]))
        ms = torch.tensor([(time.perf_counter() - h0) * 1e3], dtype=torch.float64)
        clocks, launches0 = None, 0
    else:
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        sampler.start()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = ops.native.launch_count
        t0.record()
        for i in range(args.warmup, args.warmup + args.steps):
            step(i, True)
            torch.cuda.current_stream().synchronize()            # the loss of this step is on the host
            losses.append(float(host_loss[0]))
        t1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = torch.tensor([t0.elapsed_time(t1)], dtype=torch.float64, device=dev)
    toks = tokens_done.clone().view(1)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        # tensor-parallel peers process the same tokens: count each data-parallel rank once
        if mesh.rank("tp") != 0:
            toks.zero_()
        dist.all_reduce(toks)
    if not cpu:
        ops.native.check_status()
    if rank == 0:
        print(json.dumps({
            "metric": "SALM (Canary-Qwen-2.5B shape) train tokens/s", "value": round(float(toks) / (float(ms) / 1e3), 1), "unit": "LLM input tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(float(ms) / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "native" if eager is None else "reference-equivalent (eager PyTorch Conformer + Hugging Face Qwen3 + torch.optim.AdamW)",
            "config": {"model": f"FastConformer-xlarge {args.enc_layers}L encoder + Qwen3-1.7B-shape LLM {args.llm_layers}L, {n_params / 1e9:.2f} B parameters on rank 0",
                       "global_batch": f"<= {args.batch_tokens} padded LLM positions per data-parallel rank", "seq_len": "5-20 s audio (63-250 audio tokens) + prompt + ~1.5 answer words/s",
                       "parallelism": f"dp_shard{world // args.tp} x tp{args.tp}" + (" + sp" if args.sequence_parallel else ""),
                       "optimizer": "torch.optim.AdamW" if eager is not None else ("fully sharded AdamW (ZeRO-3)" if sharded else "AdamW"), "packed": bool(args.packed),
                       "l2": "no flush: weights alone are several GB"},
            "clocks": clocks, "gpu_launches": 0 if cpu else int(ops.native.launch_count - launches0), "loss_first_last": [losses[0], losses[-1]],
            "e2e": {"value": round(float(toks) / (float(ms) / 1e3), 1), "unit": "LLM input tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4,
                    "note": "the timed region itself copies inputs from pinned memory and reads the loss back every step"}}))
    if args.profile and not cpu and rank == 0:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(2):
                step(args.warmup + args.steps + i, False)
            torch.cuda.synchronize()
        with open(args.profile, "w") as f:
            f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40, max_name_column_width=90))
        if os.environ.get("SPEECH_B200_BENCH_TRACE"):
            prof.export_chrome_trace(os.environ["SPEECH_B200_BENCH_TRACE"])      # kernel timeline per stream (.json or .json.gz)
    elif args.profile and not cpu:
        for i in range(2):
            step(args.warmup + args.steps + i, False)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
