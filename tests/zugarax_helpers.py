"""Small Zugarax configurations and the glue between model folders and the plain implementation."""

from __future__ import annotations

import json
from pathlib import Path

import torch

from plain import zugarax_plain as plain


def _mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit} if ff else None


def attention(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, size=None, scaling=None, ff=None, limit=1.5):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if size:
        mixer["mask"] = {"size": size}
    return {"type": "attention", "mixer": mixer, "mlp": _mlp(ff, limit)}


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=50000.0, scaling=None, kv_from=None, ff=None, limit=1.5):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": _mlp(ff, limit)}


def memory(heads, dim, vdim, cap, ff=None, limit=1.5):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": _mlp(ff, limit)}


def config(vocab, width, layers, embedding_scale, eps=1e-5, softcap=None):
    out = {"architecture": "Zugarax", "vocab": vocab, "width": width, "embedding": {"scale": embedding_scale},
           "norm": {"eps": eps}, "layers": layers}
    if softcap:
        out["logit_softcap"] = softcap
    return out


# Odd head sizes, value heads smaller and larger than key heads, windows shorter and longer than a
# page, rotations over a part of a head and over all of it, with and without frequency scaling
# (short `original` lengths so that every band of the scaling is met within a few dozen positions),
# a latent that a later layer reads, layers without a feed-forward, one head, limits other than 1.
SMALL_A = config(211, 64, [
    attention(4, 2, 16, 24, 0.3, 8, base=100.0, size=12, scaling=(4.0, 0.5, 3.0, 24), ff=96, limit=0.7),
    latent(3, 8, 4, 12, 20, 0.35, scaling=(6.0, 16, 8.0, 2.0), ff=80, limit=2.5),
    memory(2, 12, 20, 3.0),
    attention(3, 3, 20, 12, 0.25, 20, base=500.0, ff=72),
    latent(2, 12, 4, 6, 20, 0.3, scaling=(6.0, 16, 8.0, 2.0), kv_from=1),
    memory(1, 24, 8, 15.0, ff=64, limit=1.0),
], 8.0, softcap=6.0)
# Head sizes that the tensor-core attention takes (32, 64, 128), a width that the tensor-core products take.
SMALL_B = config(257, 128, [
    latent(4, 32, 32, 32, 64, 0.125, scaling=(8.0, 32, 16.0, 1.0), ff=256),
    attention(4, 2, 64, 64, 0.125, 32, size=40, scaling=(8.0, 1.0, 4.0, 32), ff=256),
    memory(2, 32, 64, 15.0, ff=128),
    attention(2, 1, 32, 128, 0.18, 32, size=70, ff=256),
    latent(2, 16, 32, 64, 64, 0.2, scaling=(8.0, 32, 16.0, 1.0), kv_from=0, ff=128),
    attention(2, 2, 128, 32, 0.09, 64, size=5),
], 11.3, eps=1e-6, softcap=10.0)
# A latent wider than 256 channels, two latents of different sizes, no cap on the logits, no scaling anywhere.
SMALL_C = config(97, 48, [
    latent(2, 8, 16, 8, 288, 0.3, ff=64),
    memory(3, 16, 16, 6.0),
    latent(1, 24, 8, 40, 24, 0.2),
    latent(3, 8, 16, 8, 288, 0.3, kv_from=0, ff=64, limit=0.5),
], 6.9)
ONLY_MEMORY = config(97, 48, [memory(2, 24, 24, 4.0, ff=64), memory(3, 16, 40, 15.0)], 3.0, softcap=4.0)
ONLY_ATTENTION = config(97, 48, [attention(4, 2, 12, 20, 0.3, 6, size=10, scaling=(4.0, 1.0, 4.0, 16), ff=64, limit=0.8)], 7.0)
# Neither a rotation nor a window: attention that knows no positions but the causal order.
BARE_ATTENTION = config(97, 48, [attention(2, 1, 24, 24, 0.2, 8, ff=64), memory(2, 8, 12, 5.0)], 5.0)
del BARE_ATTENTION["layers"][0]["mixer"]["rot"]
ONLY_LATENT = config(97, 48, [latent(4, 12, 8, 20, 24, 0.3, scaling=(4.0, 16, 8.0, 1.0), ff=64)], 7.0)
SMALL = {"small_b": (SMALL_B, 16, 21), "small_a": (SMALL_A, 4, 22), "small_c": (SMALL_C, 8, 23), "only_memory": (ONLY_MEMORY, 8, 24),
         "only_attention": (ONLY_ATTENTION, 4, 25), "only_latent": (ONLY_LATENT, 16, 26), "bare_attention": (BARE_ATTENTION, 16, 27)}       # config, page size, seed


def write_model(folder: Path, raw: dict, seed: int, dtype=torch.bfloat16, sharpen: float = 6.0) -> Path:
    """A random model folder whose numbers make faults visible: query and key projections and
    their norm weights scaled up (one key's score stands out, so a wrong, missing or extra key
    shows and the sink's 1 matters or not from row to row), gate biases of a size that matters,
    feed-forward projections that reach their limits, logits that reach their cap."""
    from safetensors.torch import load_file, save_file

    from paged_attention_engine_b200.weights import write_random_model

    write_random_model(folder, raw, seed, dtype)
    path = str(Path(folder) / "model.safetensors")
    tensors = load_file(path)
    gen = torch.Generator().manual_seed(seed + 1000)
    for name in list(tensors):
        t = tensors[name].float()
        if name.endswith((".mix.q", ".mix.k", ".mix.v", ".mix.g", ".mix.dkv", ".mix.uk", ".mix.uv", ".mlp.gate", ".mlp.up")):
            t = t * sharpen
        elif name.endswith((".mix.i", ".mix.f")):
            # a gate's error adds up along the sequence inside an exponent: bfloat16 inputs allow less here
            t = t * sharpen / 3.0
        elif name.endswith((".q.norm", ".k.norm")):
            t = 1.0 + torch.rand(t.shape, generator=gen) * 1.5
        elif name.endswith((".i.b", ".f.b")):
            t = torch.randn(t.shape, generator=gen) * 1.5
        elif name.endswith(".b"):
            t = torch.randn(t.shape, generator=gen) * 0.3
        elif name == "head":
            t = t * 12.0
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
