"""Per-kernel device times of one Conformer layer inside the whole-layer executor: ``python -m speech_b200.ops.bench_layer``.

Runs a FastConformer layer (forward + backward, training mode with dropout) at the given shape through the native executor,
which records a CUDA event after every launch, and prints the time and — for the GEMMs — the achieved FLOP rate of every
kernel in issue order.  The inputs of consecutive kernels are the real intermediate tensors, so cache state matches training.
"""
from __future__ import annotations

import argparse
import re

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(prog="speech_b200.ops.bench_layer")
    ap.add_argument("--batch", type=int, default=20)
    ap.add_argument("--frames", type=int, default=188, help="encoder frames per utterance (after subsampling)")
    ap.add_argument("--d-model", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--dropout", type=float, default=0.1)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args(argv)
    from .. import ops
    from ..core.optim.fused_adamw import FusedAdamW
    from ..modules.attention import RelPositionalEncoding
    from ..modules.conformer_modules import ConformerLayer
    from . import native_layer

    torch.manual_seed(0)
    d, H, B, T = args.d_model, args.heads, args.batch, args.frames
    layer = ConformerLayer(d_model=d, d_ff=4 * d, n_heads=H, conv_kernel_size=9, dropout=args.dropout, dropout_att=args.dropout).cuda().train()
    fusion = [fg for m in layer.modules() if hasattr(m, "arena_fusion_groups") for fg in m.arena_fusion_groups()]
    opt = FusedAdamW(layer.parameters(), lr=1e-3, fusion_groups=fusion)
    pe = RelPositionalEncoding(d, 0.0)
    pe.extend_pe(T, "cuda")
    x = torch.randn(B, T, d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    _, pos = pe(x)
    lens = torch.randint(T // 2, T + 1, (B,), device="cuda")
    lens[0] = T
    pad = torch.arange(T, device="cuda")[None, :] >= lens[:, None]
    att = pad[:, None, :] | pad[:, :, None]
    wr = torch.randn(B, T, d, device="cuda", dtype=torch.bfloat16)

    def step():
        opt.zero_grad()
        with ops.compute_dtype(torch.bfloat16):
            y = layer(x, att_mask=att, pos_emb=pos, pad_mask=pad)
        y.backward(wr)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    native_layer.profile_sink = []
    for _ in range(args.iters):
        step()
    torch.cuda.synchronize()
    sink, native_layer.profile_sink = native_layer.profile_sink, None
    R = B * T
    for phase in ("forward", "backward"):
        runs = [r for p, r in sink if p == phase]
        n = len(runs[0])
        print(f"--- {phase}: {n} launches, B={B} T={T} d={d} (rows {R}), mean of {len(runs)} runs")
        total = 0.0
        for i in range(n):
            label = runs[0][i][0]
            ms = sum(r[i][1] for r in runs) / len(runs)
            total += ms
            m = re.search(r"(linear|dgrad|wgrad) (\d+)x(\d+)", label)
            rate = f"{2.0 * R * int(m.group(2)) * int(m.group(3)) / ms / 1e9:8.0f} TFLOP/s" if m else ""
            print(f"{i:3d} {label:34s} {ms * 1e3:9.1f} us {rate}")
        print(f"    total {total:.3f} ms")


if __name__ == "__main__":
    main()
