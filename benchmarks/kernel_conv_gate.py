"""Time the fused convolution + batch normalisation + ReLU (forward and backward) against the PyTorch layers.

    python benchmarks/kernel_conv_gate.py --batch 16384 --rows 4 --cols 128 --channels 8

Times are CUDA-event times after warm-up.  ``--fused_only`` skips the layers (for hardware-counter captures).
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source checkout

import torch
from torch import nn

from dice_embeddings_b200.ops import conv_gate


def _time(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=16384)
    ap.add_argument("--rows", type=int, default=4)
    ap.add_argument("--cols", type=int, default=128)
    ap.add_argument("--channels", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--fused_only", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    B, H, W, C = args.batch, args.rows, args.cols, args.channels
    torch.manual_seed(0)
    conv, bn = nn.Conv2d(1, C, 3, padding=1).to(dev), nn.BatchNorm2d(C).to(dev)
    x = torch.randn(B, H * W, device=dev, requires_grad=True)
    g = torch.randn(B, C * H * W, device=dev)
    assert conv_gate.supported(x, conv, bn, H, W), "shape not covered by the fused kernels"

    def fused():
        conv_gate.conv_gate_features(x, conv, bn, H, W).backward(g)

    def layers():
        torch.relu(bn(conv(x.view(B, 1, H, W)))).reshape(B, -1).backward(g)

    t_fused = _time(fused, args.iters)
    feature_bytes = 4.0 * B * C * H * W
    image_bytes = 4.0 * B * H * W
    # forward: image twice, features once; backward: (features + image) twice, image gradient once
    algorithmic = 3 * feature_bytes + 5 * image_bytes
    line = f"conv gate fwd+bwd B={B} {H}x{W} C={C}: fused {t_fused:.3f} ms ({algorithmic / t_fused / 1e9:.2f} TB/s)"
    if not args.fused_only:
        line += f", layers (TF32 convolution) {_time(layers, args.iters):.3f} ms"
        torch.backends.cudnn.allow_tf32 = False
        line += f", layers (fp32) {_time(layers, args.iters):.3f} ms"
    print(line)


if __name__ == "__main__":
    main()
