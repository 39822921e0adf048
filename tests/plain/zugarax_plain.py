"""A plain, slow Zugarax: one function per mechanism, written from the design's equations.

Everything runs on the CPU in float64 over one whole sequence at a time, with explicit loops
over tokens where a recurrence or a window is involved. It shares no code with the engine:
it reads a dictionary of tensors by their checkpoint names and the config.json dictionary.

Notation: T tokens, W model width, H query heads, G key/value heads, d query/key size, dv
value size, r rotated size, c latent size, positions p = 0..T-1.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def _f(t):
    return t.to(F)


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis; w None: no weight."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * _f(weight)


# --------------------------------------------------------------------------- #
# Rotation frequencies
# --------------------------------------------------------------------------- #

def base_frequencies(dims, base):
    return [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]


def banded_frequencies(dims, base, factor, low, high, original):
    """Long wavelengths are slowed by `factor`, short ones kept, the band between them blended."""
    out = []
    for f in base_frequencies(dims, base):
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


def ramped_frequencies(dims, base, factor, original, fast, slow):
    """(frequencies, amplitude): a linear ramp over the pair index between the pairs that turn
    `fast` and `slow` times within `original` positions; cos and sin are multiplied by the amplitude."""
    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(base_frequencies(dims, base)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, layout, amplitude=1.0):
    """Rotates the first 2 * len(freqs) channels of x [T, heads, n]. layout "half": channel i
    pairs with i + len(freqs); "interleaved": channel 2i with 2i + 1."""
    x = x.clone()
    half = len(freqs)
    for t, p in enumerate(positions):
        for i, f in enumerate(freqs):
            a, b = (i, i + half) if layout == "half" else (2 * i, 2 * i + 1)
            c, s = math.cos(p * f) * amplitude, math.sin(p * f) * amplitude
            u, v = x[t, :, a].clone(), x[t, :, b].clone()
            x[t, :, a] = u * c - v * s
            x[t, :, b] = v * c + u * s
    return x


# --------------------------------------------------------------------------- #
# Attention
# --------------------------------------------------------------------------- #

def softmax_attention(q, k, v, scale, size=None, extra_one=False, rows=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]. Query i sees key j when j <= i and
    (size None or i - j < size). extra_one: the denominator also holds exp(0) = 1."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for head in range(H):
        g = head // (H // G)
        for i in (range(T) if rows is None else rows):
            first = 0 if size is None else max(0, i - int(size) + 1)
            s = (k[first:i + 1, g] @ q[i, head]) * scale
            top = max(float(s.max()), 0.0) if extra_one else float(s.max())
            e = torch.exp(s - top)
            denominator = e.sum() + (math.exp(-top) if extra_one else 0.0)
            out[i, head] = (e / denominator) @ v[first:i + 1, g]
    return out


def windowed_attention_mixer(h, tensors, prefix, m, eps, rows=None):
    """The gated, windowed, grouped-query attention with normed and partly rotated q and k."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = lambda n: _f(tensors[f"{prefix}.{n}"])
    q = rms_norm((h @ t("q").T).view(T, H, d), tensors[f"{prefix}.q.norm"], eps)
    k = rms_norm((h @ t("k").T).view(T, G, d), tensors[f"{prefix}.k.norm"], eps)
    v = (h @ t("v").T).view(T, G, dv)
    rot = m.get("rot")
    if rot is not None:
        sc = rot.get("scaling")
        freqs = (banded_frequencies(rot["dims"], rot["base"], sc["factor"], sc["low"], sc["high"], sc["original"])
                 if sc else base_frequencies(rot["dims"], rot["base"]))
        positions = list(range(T))
        q, k = rotate(q, positions, freqs, "half"), rotate(k, positions, freqs, "half")
    size = m["mask"]["size"] if m.get("mask") else None
    o = softmax_attention(q, k, v, m["scale"], size=size, extra_one=True, rows=rows)
    gate = torch.sigmoid(h @ t("g").T)
    return (o.reshape(T, H * dv) * gate) @ t("o").T


def latent_of(h, tensors, prefix, m, eps):
    """(latent [T, c], rotated shared key part [T, r]) of the layer that owns a down projection."""
    T = h.shape[0]
    c, r = m["kv_rank"], m["rot_dim"]
    down = h @ _f(tensors[f"{prefix}.dkv"]).T
    latent = rms_norm(down[:, :c], tensors[f"{prefix}.dkv.norm"], eps)
    freqs, amplitude = _latent_frequencies(m)
    shared = rotate(down[:, c:].reshape(T, 1, r), list(range(T)), freqs, "interleaved", amplitude).reshape(T, r)
    return latent, shared


def _latent_frequencies(m):
    rot = m["rot"]
    sc = rot.get("scaling")
    if sc:
        return ramped_frequencies(rot["dims"], rot["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"])
    return base_frequencies(rot["dims"], rot["base"]), 1.0


def latent_attention_mixer(h, tensors, prefix, m, latent, shared, rows=None):
    """Causal attention whose keys and values are expanded per head from a shared latent."""
    T = h.shape[0]
    H, d, r, dv, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    t = lambda n: _f(tensors[f"{prefix}.{n}"])
    q = (h @ t("q").T).view(T, H, d + r)
    freqs, amplitude = _latent_frequencies(m)
    q_rot = rotate(q[:, :, d:], list(range(T)), freqs, "interleaved", amplitude)
    k_flat = (latent @ t("uk").T).view(T, H, d)
    v = (latent @ t("uv").T).view(T, H, dv)
    q_full = torch.cat([q[:, :, :d], q_rot], dim=-1)
    k_full = torch.cat([k_flat, shared.view(T, 1, r).expand(T, H, r)], dim=-1)
    o = softmax_attention(q_full, k_full, v, m["scale"], rows=rows)
    return o.reshape(T, H * dv) @ t("o").T


# --------------------------------------------------------------------------- #
# Matrix memory
# --------------------------------------------------------------------------- #

def log_sigmoid(x):
    return -math.log1p(math.exp(-x)) if x > -30 else x


def matrix_memory_scan(q, k, v, i_pre, f_pre, cap, state=None):
    """q, k [T, H, d] (q already scaled), v [T, H, dv], gate pre-activations [T, H]. The state per
    head is (S [d, dv], n [d], m); returns (o [T, H, dv], state)."""
    T, H, d = q.shape
    dv = v.shape[2]
    if state is None:
        state = [(torch.zeros(d, dv, dtype=F), torch.zeros(d, dtype=F), 0.0) for _ in range(H)]
    out = torch.zeros(T, H, dv, dtype=F)
    state = list(state)
    for head in range(H):
        S, n, m = state[head]
        for t in range(T):
            i = cap * math.tanh(float(i_pre[t, head]) / cap)
            f = log_sigmoid(cap * math.tanh(float(f_pre[t, head]) / cap))
            m_new = max(f + m, i)
            keep, add = math.exp(f + m - m_new), math.exp(i - m_new)
            S = keep * S + add * torch.outer(k[t, head], v[t, head])
            n = keep * n + add * k[t, head]
            m = m_new
            below = max(abs(float(n @ q[t, head])), math.exp(-m)) + 1e-6
            out[t, head] = (S.T @ q[t, head]) / below
        state[head] = (S, n, m)
    return out, state


def matrix_memory_mixer(h, tensors, prefix, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    t = lambda n: _f(tensors[f"{prefix}.{n}"])
    q = (h @ t("q").T).view(T, H, d) * d ** -0.5
    k = (h @ t("k").T).view(T, H, d)
    v = (h @ t("v").T).view(T, H, dv)
    i_pre = h @ t("i").T + t("i.b")
    f_pre = h @ t("f").T + t("f.b")
    o, _ = matrix_memory_scan(q, k, v, i_pre, f_pre, float(m["gate_cap"]))
    o = rms_norm(o, None, eps).reshape(T, H * dv) * t("norm") * torch.sigmoid(h @ t("g").T)
    return o @ t("o").T


# --------------------------------------------------------------------------- #
# Feed-forward, whole model
# --------------------------------------------------------------------------- #

def clamped_glu_feed_forward(h, tensors, prefix, limit):
    t = lambda n: _f(tensors[f"{prefix}.{n}"])
    g = torch.clamp(h @ t("gate").T + t("gate.b"), max=limit)
    u = torch.clamp(h @ t("up").T + t("up.b"), min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t("down").T + t("down.b")


def forward(raw, tensors, tokens, layer_outputs=None):
    """Logits [T, vocab] in float64 for one sequence from position 0. `layer_outputs`, a list,
    receives the residual stream after every layer."""
    eps = float(raw["norm"]["eps"])
    x = _f(tensors["embed"])[list(tokens)] * float(raw["embedding"]["scale"])
    latents = {}
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = rms_norm(x, tensors[f"{p}.norm1"], eps)
        if layer["type"] == "attention":
            x = x + windowed_attention_mixer(h, tensors, f"{p}.mix", m, eps)
        elif layer["type"] == "latent_attention":
            source = m.get("kv_from")
            if source is None:
                latents[i] = latent_of(h, tensors, f"{p}.mix", m, eps)
                source = i
            x = x + latent_attention_mixer(h, tensors, f"{p}.mix", m, *latents[source])
        elif layer["type"] == "mlstm":
            x = x + matrix_memory_mixer(h, tensors, f"{p}.mix", m, eps)
        else:
            raise ValueError(f"layer {i}: type {layer['type']!r}")
        if layer.get("mlp") is not None:
            h = rms_norm(x, tensors[f"{p}.norm2"], eps)
            x = x + clamped_glu_feed_forward(h, tensors, f"{p}.mlp", float(layer["mlp"]["limit"]))
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    logits = rms_norm(x, tensors["final.norm"], eps) @ _f(tensors["head"]).T
    cap = raw.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
