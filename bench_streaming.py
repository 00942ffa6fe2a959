"""Streaming benchmark: cache-aware FastConformer-RNNT (0.6B shape) serving many concurrent synthetic streams on one GPU.

python bench_streaming.py --streams 256 --seconds 20 --lookahead 13

Model: 24 layers, d_model 1024, 8 heads, causal depthwise conv k=9, 8x sub-sampling, attention context [70, lookahead] (chunked),
1-layer LSTM prediction network 640, joint 640, vocabulary 1024 + blank; random weights, bf16.  Load: ``--streams`` streams of
``--seconds`` seconds of N(0, 0.1^2) audio each, fed chunk by chunk through the continuous-batching pipeline (the public
``PipelineBuilder`` API: feature extraction, encoder step with per-stream caches, label-looping greedy decode).  Prints one JSON
line: RTFx = audio seconds / seconds spent in ``transcribe_step`` (host clock around each step; every step ends with the token
read-back, i.e. a device synchronisation), the chunk duration, p50 / p99 step latency and whether p99 stays within the chunk
duration — the criterion for "this many streams in real time".
"""
from __future__ import annotations

import argparse
import json
import time

import numpy as np
import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--streams", type=int, default=256)
    ap.add_argument("--seconds", type=float, default=20.0)
    ap.add_argument("--lookahead", type=int, default=13, choices=[0, 1, 6, 13])
    ap.add_argument("--batch-size", type=int, default=0, help="streams per encoder step (default: all)")
    ap.add_argument("--size", default="xlarge")
    ap.add_argument("--cuda-graph-decoder", action="store_true")
    ap.add_argument("--blank-bias", type=float, default=6.0,
                    help="added to the joint's blank logit: untrained weights would otherwise emit max_symbols tokens on every frame, "
                         "which no trained model does; 6.0 gives a few tokens per second of audio")
    args = ap.parse_args()
    from speech_b200.core.config import OmegaConf
    from speech_b200.inference.pipelines import PipelineBuilder
    from speech_b200.models import EncDecRNNTBPEModel
    from speech_b200.models.configs import fastconformer_transducer_config

    torch.manual_seed(0)
    dev = torch.device("cuda:0")
    cfg = fastconformer_transducer_config(args.size, vocab_size=1024, dropout=0.0, loss="rnnt", pred_rnn_layers=1, causal=True,
                                          att_context_size=[70, args.lookahead], att_context_style="chunked_limited", conv_norm_type="layer_norm")
    model = EncDecRNNTBPEModel(cfg).eval().to(dev)
    if args.blank_bias:
        with torch.no_grad():
            model.joint.joint_net[-1].bias[model.joint.num_classes_with_blank - 1] += args.blank_bias
    bs = args.batch_size or args.streams
    pcfg = OmegaConf.create({
        "pipeline_type": "cache_aware", "asr_decoding_type": "rnnt", "asr_output_granularity": "word",
        "asr": {"device": "cuda:0", "compute_dtype": "bfloat16",
                "decoding": {"strategy": "greedy_batch", "greedy": {"use_cuda_graph_decoder": bool(args.cuda_graph_decoder), "max_symbols": 10}}},
        "streaming": {"sample_rate": 16000, "batch_size": bs, "num_slots": max(args.streams, bs), "att_context_size": [70, args.lookahead], "use_cache": True},
        "endpointing": {"stop_history_eou": -1, "residue_tokens_at_end": 2}, "confidence": {"aggregation": "mean"}})
    pipe = PipelineBuilder.build_pipeline(pcfg, asr_model=model)
    rng = np.random.default_rng(0)
    n = int(args.seconds * 16000)
    audio = [(rng.standard_normal(n) * 0.1).astype(np.float32) for _ in range(args.streams)]
    pipe.run([a[: 16000 * 3] for a in audio[: min(args.streams, bs)]])          # warm-up: kernels, graphs, allocator
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = pipe.run(audio)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    steps = np.asarray(pipe.step_times)
    hop_s = 0.01
    chunk_s = (1 + args.lookahead) * 8 * hop_s
    total_audio = args.streams * args.seconds
    res = {"metric": "cache-aware streaming RTFx", "value": round(float(pipe.rtfx()), 1), "unit": "audio-seconds/s", "n_gpus": 1,
           "streams": args.streams, "seconds_per_stream": args.seconds, "chunk_ms": round(chunk_s * 1e3, 1), "steps": int(steps.size),
           "step_ms_p50": round(float(np.percentile(steps, 50)) * 1e3, 2), "step_ms_p99": round(float(np.percentile(steps, 99)) * 1e3, 2),
           "step_ms_first": round(float(steps[0]) * 1e3, 2), "slowest_steps": [int(i) for i in np.argsort(steps)[-3:][::-1]], "step_ms_max_after_first": round(float(steps[1:].max()) * 1e3, 2) if steps.size > 1 else None,
           "real_time": bool(np.percentile(steps, 99) <= chunk_s), "rtfx_wall": round(total_audio / wall, 1), "dtype": "bf16", "data": "synthetic",
           "tokens_emitted": int(sum(len(o.text.split()) for o in out.values())), "blank_bias": args.blank_bias,
           "config": {"model": f"FastConformer-{args.size} cache-aware RNNT, att_context [70,{args.lookahead}]", "batch_size": bs}}
    print(json.dumps(res))


if __name__ == "__main__":
    main()
