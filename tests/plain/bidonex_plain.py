"""A plain, slow Bidonex: one function per mechanism, written from the design's equations.

Everything runs on the CPU in float64 over one whole sequence at a time, with explicit loops
over tokens where a recurrence or a window is involved. It shares no code with the engine:
it reads a dictionary of tensors by their checkpoint names and the config.json dictionary.

Notation: T tokens, W model width, H query heads, G key/value heads, d query/key size, dv
value size, positions p = 0..T-1.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def _f(t):
    return t.to(F)


def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(var + eps) * w + b, var = mean of squared deviations."""
    mean = x.mean(dim=-1, keepdim=True)
    dev = x - mean
    var = (dev * dev).mean(dim=-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * _f(weight) + _f(bias)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def causal_conv(u, taps_weight):
    """y[t, c] = sum_j w[c, j] * u[t - taps + 1 + j, c], zeros before the start. u [T, C], w [C, taps]."""
    w = _f(taps_weight)
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def dense_feed_forward(h, up, down):
    return gelu_erf(h @ _f(up).T) @ _f(down).T


def scored_attention(q, k, v, scale, temp=None, cap=None, r1=None, r2=None, sink=None, size=None, keep=0, rows=None):
    """Attention of queries q [T, H, d] over keys k [T, G, d] and values v [T, G, dv] of the same
    sequence under the score rule; `rows` limits the query positions that are computed (the others
    stay zero). Returns [T, H, dv]."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for head in range(H):
        g = head // (H // G)
        for i in (range(T) if rows is None else rows):
            scores, seen = [], []
            for j in range(i + 1):
                if size is not None and not (i - j < int(size) or j < keep):
                    continue
                s = float(q[i, head] @ k[j, g]) * scale
                if temp is not None:
                    s *= float(temp[head])
                if cap:
                    s = float(cap) * math.tanh(s / float(cap))
                if r1 is not None:
                    s -= float(r1[head]) * math.log(1.0 + float(r2[head]) * (i - j))
                scores.append(s)
                seen.append(j)
            m = max(scores + ([float(sink[head])] if sink is not None else []))
            weights = [math.exp(s - m) for s in scores]
            denominator = sum(weights) + (math.exp(float(sink[head]) - m) if sink is not None else 0.0)
            for wgt, j in zip(weights, seen):
                out[i, head] += (wgt / denominator) * v[j, g]
    return out


def windowed_sink_attention(h, tensors, prefix, mixer, eps):
    """The attention mixer over one whole sequence h [T, W]."""
    H, G, d = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"])
    dv = int(mixer["vdim"])
    T = h.shape[0]
    q = h @ _f(tensors[f"{prefix}.q"]).T
    k = h @ _f(tensors[f"{prefix}.k"]).T
    v = h @ _f(tensors[f"{prefix}.v"]).T
    if int(mixer.get("conv") or 0) >= 1:
        q = causal_conv(q, tensors[f"{prefix}.q.conv"])
        k = causal_conv(k, tensors[f"{prefix}.k.conv"])
        v = causal_conv(v, tensors[f"{prefix}.v.conv"])
    q = unit_rms(q.view(T, H, d), eps)
    k = unit_rms(k.view(T, G, d), eps)
    v = v.view(T, G, dv)
    mask = mixer.get("mask") or {}
    temp, r1, r2, sink = (_f(tensors[f"{prefix}.{n}"]) for n in ("temp", "r1", "r2", "sink"))
    out = scored_attention(q, k, v, float(mixer["scale"]), temp, mixer.get("softcap"), r1, r2, sink,
                           mask.get("size"), int(mask.get("keep_first") or 0))
    return out.reshape(T, H * dv) @ _f(tensors[f"{prefix}.o"]).T


def general_delta(h, tensors, prefix, mixer, eps):
    """The generalized delta rule over one whole sequence h [T, W], state from zero."""
    H, d = int(mixer["heads"]), int(mixer["dim"])
    T = h.shape[0]
    t = lambda n: _f(tensors[f"{prefix}.{n}"])
    r = (h @ t("r").T).view(T, H, d)
    k = (h @ t("k").T).view(T, H, d)
    v = (h @ t("v").T).view(T, H, d)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ t("w1").T) @ t("w2").T + t("w0"))).view(T, H, d)
    rate = torch.sigmoid(h @ t("a").T + t("a.b")).view(T, H, d)
    gate = torch.sigmoid(h @ t("g").T)
    out = torch.zeros(T, H, d, dtype=F)
    for head in range(H):
        S = torch.zeros(d, d, dtype=F)              # [key channel, value channel]
        for i in range(T):
            kk = k[i, head]
            u = kk / torch.sqrt((kk * kk).sum() + 1e-6)
            old = S
            S = decay[i, head][:, None] * old - torch.outer(rate[i, head] * u, u @ old) + torch.outer(kk, v[i, head])
            out[i, head] = S.T @ r[i, head]
    out = unit_rms(out, eps).reshape(T, H * d) * t("norm") * gate
    return out @ t("o").T


def forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] (float64) of one whole sequence; with `return_layers` also the residual
    stream after every layer [layers, T, W]."""
    eps = float(config["norm"]["eps"])
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    T = ids.numel()
    x = _f(tensors["embed"])[ids] + _f(tensors["pos"])[:T]
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}"
        h = layer_norm(x, tensors[f"{p}.norm1"], tensors[f"{p}.norm1.b"], eps)
        if layer["type"] == "attention":
            branch = windowed_sink_attention(h, tensors, f"{p}.mix", layer["mixer"], eps)
        elif layer["type"] == "general_delta":
            branch = general_delta(h, tensors, f"{p}.mix", layer["mixer"], eps)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        if layer.get("mlp") is not None:
            branch = branch + dense_feed_forward(h, tensors[f"{p}.mlp.up"], tensors[f"{p}.mlp.down"])
        x = x + branch
        after.append(x)
    x = layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], eps)
    logits = x @ _f(tensors["head"]).T
    return (logits, torch.stack(after)) if return_layers else logits
