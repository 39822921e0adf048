"""Small Bidonex configurations and the glue between model folders and the plain implementation."""

from __future__ import annotations

import json
from pathlib import Path

import torch

from plain import bidonex_plain as plain


def attention(heads, kv_heads, dim, vdim, scale, softcap=None, conv=None, size=None, keep_first=0, ff=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        mixer["softcap"] = softcap
    if conv:
        mixer["conv"] = conv
    if size:
        mixer["mask"] = {"size": size, "keep_first": keep_first}
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads, dim, rank, ff=None):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "rank": rank},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(vocab, width, layers, max_positions=512, eps=1e-5):
    return {"architecture": "Bidonex", "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": eps}, "layers": layers}


# Value heads smaller and larger than key heads, one and several kv heads, windows shorter and longer
# than a page, more kept keys than the window is long, no kept keys, layers without a cap, a
# convolution, a mask or a feed-forward, head sizes that are no multiple of 8 or 32.
SMALL_A = config(211, 64, [
    delta(2, 16, 8, ff=96),
    attention(4, 2, 16, 24, 0.31, softcap=12.0, conv=3, size=12, keep_first=3, ff=96),
    delta(1, 40, 4),
    attention(3, 3, 20, 12, 0.2, conv=2, size=7, keep_first=0, ff=80),
    attention(2, 1, 8, 8, 0.5, softcap=30.0, ff=72),
])
SMALL_B = config(301, 96, [
    attention(2, 1, 24, 40, 0.25, softcap=8.0, conv=4, size=5, keep_first=9, ff=128),
    delta(3, 24, 16, ff=128),
    attention(6, 2, 12, 12, 0.4, conv=1, size=33, keep_first=1),
    delta(2, 80, 8, ff=64),
], eps=1e-6)
ONLY_DELTA = config(97, 48, [delta(2, 24, 8, ff=64), delta(3, 16, 4)])
ONLY_ATTENTION = config(97, 48, [attention(4, 2, 12, 20, 0.3, softcap=10.0, conv=3, size=10, keep_first=2, ff=64)])
# Head sizes that the tensor-core kernels take (32, 64, 128), keys and values of different sizes.
SMALL_C = config(257, 128, [
    attention(4, 2, 64, 64, 0.125, softcap=20.0, conv=3, size=24, keep_first=4, ff=256),
    delta(2, 64, 16, ff=256),
    attention(2, 1, 32, 128, 0.18, conv=2, size=70, keep_first=2, ff=256),
    attention(2, 2, 128, 32, 0.09, softcap=30.0),
])
SMALL = {"small_c": (SMALL_C, 16, 15), "small_a": (SMALL_A, 4, 11), "small_b": (SMALL_B, 16, 12), "only_delta": (ONLY_DELTA, 8, 13),
         "only_attention": (ONLY_ATTENTION, 4, 14)}       # config, page size, seed


def write_model(folder: Path, raw: dict, seed: int, dtype=torch.bfloat16, sharpen: float = 6.0) -> Path:
    """A random model folder whose numbers make faults visible: q and k projections scaled up (one
    key's score stands out, so a wrong, missing or extra key shows), sinks and distance slopes of
    a size that matters, a key projection of the delta rule that is not tiny."""
    from safetensors.torch import load_file, save_file

    from paged_attention_engine_b200.weights import write_random_model

    write_random_model(folder, raw, seed, dtype)
    path = str(Path(folder) / "model.safetensors")
    tensors = load_file(path)
    gen = torch.Generator().manual_seed(seed + 1000)
    for name in list(tensors):
        t = tensors[name].float()
        if name.endswith((".mix.q", ".mix.k", ".mix.r", ".mix.v", ".mix.a", ".mix.g", ".mix.w1", ".mix.w2")):
            t = t * sharpen
        elif name.endswith((".sink", ".r1", ".a.b", ".w0")):
            t = torch.randn(t.shape, generator=gen) * 1.5
        elif name.endswith(".temp"):
            t = 0.5 + torch.rand(t.shape, generator=gen) * 2.0
        tensors[name] = t.to(tensors[name].dtype)
    save_file(tensors, path)
    return Path(folder)


def read_model(folder: Path):
    from safetensors.torch import load_file

    return json.loads((Path(folder) / "config.json").read_text()), load_file(str(Path(folder) / "model.safetensors"))


def plain_logits(folder: Path, tokens) -> torch.Tensor:
    raw, tensors = read_model(folder)
    return plain.forward(raw, tensors, list(tokens)).float()


FP32_RTOL = 5e-5
BF16_RTOL = 2.0 ** -5


def tolerance(dtype, reference: torch.Tensor) -> float:
    top = max(1.0, float(reference.abs().max()))
    return (FP32_RTOL if dtype in (torch.float32, "float32") else BF16_RTOL) * top
