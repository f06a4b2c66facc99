"""Plain, slow implementation of the Kufulix decoder for the tests.

Whole sequences, no cache, one function per mechanism, torch on the CPU in 64-bit.  It shares
no code with the package under test: it reads config.json and the safetensors file with its
own few lines and computes every layer with dense masks and loops over tokens and experts.

The design in this file's notation (rows are tokens, p: position, h: the normed input of a sublayer):

    norm       N(x; w) = x / sqrt(mean x^2 + eps) * (1 + w)
    embedding  x = N(E[token]; w_embed)
    layer      x <- x + mixer(N(x; w_1));  x <- x + ff(N(x; w_2))
               a layer with `weights_of: j` runs layer j's tensors on a cache and state of its own
    attention  q, k, v = W h + b;  turn the first `dims` columns of every head of q and k: pairs
               (i, i + dims/2), angle p * g_i;  s_ij = q_i . k_j * scale for the visible j;
               softmax;  query head a reads key/value head a // (heads / kv_heads)
               g_i:  f_i = base^(-2i/dims), l = 2 pi / f_i;  l < original/high: f_i;
                     l > original/low: f_i / factor;  else with t = (original/l - low) / (high - low):
                     (1 - t) f_i / factor + t f_i
      'attention' layers:  visible j <= i with i // size == j // size;  every head's output times
                           sigmoid(W_g h)[head];  then W_o
      left of 'parallel':  q and k of every head divided by their root mean square (+ eps inside the
                           root) times a weight of `dim` numbers, BEFORE turning;  visible
                           0 <= i - j < size;  then W_o
    right of 'parallel' (state-space duality)
               [z | x | B | C | dt] = W_in h;  (x, B, C) <- silu(causal conv over time + bias);
               dt <- softplus(dt + dt_bias);  per head a (group a // (heads / groups)):
               S_t = exp(-exp(A_log_a) dt_t) S_(t-1) + dt_t B_t x_t^T;  y_t = S_t^T C_t + D_a x_t;
               y <- y * silu(z);  y divided by its root mean square in `norm_groups` equal parts,
               times a weight;  then W_o
    parallel   left_scale * left + right_scale * right
    experts    z = W_r h;  s = softmax(z) over experts and identity experts;  c = s + correction;
               groups of neighbours, a group's score = its largest c;  outside the `keep` best
               groups c = -inf;  the `top` largest c are chosen;  weight_e = s_e / (sum of chosen s
               + 1e-20);  expert(h) = W_down relu(W_up h)^2;  the last `identity` router outputs are
               experts whose output is h itself
    output     logits = cap * tanh(H N(x; w_final) / cap)
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- loading
def read_tensors(path):
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        chunk = raw[8 + n + b:8 + n + e]
        if meta["dtype"] == "BF16":
            bits = np.frombuffer(chunk, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(chunk, dtype="<f4").copy())
        else:
            raise ValueError(meta["dtype"])
        out[name] = t.reshape(meta["shape"]).to(F64)
    return out


def load(model_dir):
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    return config, read_tensors(model_dir / "model.safetensors")


# -------------------------------------------------------------------------- mechanisms
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_plus_norm(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def turn_frequencies(rot):
    dims = int(rot["dims"])
    out = []
    scaling = rot.get("scaling")
    for i in range(dims // 2):
        f = float(rot["base"]) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            original = float(scaling["original"])
            length = 2.0 * math.pi / f
            if length < original / high:
                pass
            elif length > original / low:
                f = f / factor
            else:
                t = (original / length - low) / (high - low)
                f = (1.0 - t) * f / factor + t * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def turn(x, positions, rot):
    """x [tokens, heads, dim]: the first `dims` columns of every head, pairs (i, i + dims/2)."""
    if not rot or not int(rot["dims"]):
        return x
    dims = int(rot["dims"])
    half = dims // 2
    angle = positions.to(F64)[:, None] * turn_frequencies(rot)[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def window_mask(n, size):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & (i - j < size)


def chunk_mask(n, size):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & (i // size == j // size)


def softmax_attention(q, k, v, mask, scale):
    """q [n, heads, dim], k [n, kv_heads, dim], v [n, kv_heads, vdim] -> [n, heads, vdim]."""
    n, heads, _ = q.shape
    group = heads // k.shape[1]
    out = torch.zeros(n, heads, v.shape[-1], dtype=F64)
    for a in range(heads):
        s = (q[:, a] @ k[:, a // group].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, a // group]
    return out


def projections(h, w, prefix, m):
    n = h.shape[0]
    q = (h @ w[prefix + "q"].T + w[prefix + "q.b"]).view(n, m["heads"], m["dim"])
    k = (h @ w[prefix + "k"].T + w[prefix + "k.b"]).view(n, m["kv_heads"], m["dim"])
    v = (h @ w[prefix + "v"].T + w[prefix + "v.b"]).view(n, m["kv_heads"], m["vdim"])
    return q, k, v


def chunked_gated_attention(h, w, prefix, m):
    n = h.shape[0]
    positions = torch.arange(n)
    q, k, v = projections(h, w, prefix, m)
    q, k = turn(q, positions, m["rot"]), turn(k, positions, m["rot"])
    out = softmax_attention(q, k, v, chunk_mask(n, int(m["mask"]["size"])), float(m["scale"]))
    gate = torch.sigmoid(h @ w[prefix + "g"].T)                   # [n, heads]
    out = out * gate[:, :, None]
    return out.reshape(n, -1) @ w[prefix + "o"].T


def windowed_normed_attention(h, w, prefix, m, eps):
    n = h.shape[0]
    positions = torch.arange(n)
    q, k, v = projections(h, w, prefix, m)
    q = unit_rms(q, eps) * w[prefix + "q.norm"]
    k = unit_rms(k, eps) * w[prefix + "k.norm"]
    q, k = turn(q, positions, m["rot"]), turn(k, positions, m["rot"])
    out = softmax_attention(q, k, v, window_mask(n, int(m["mask"]["size"])), float(m["scale"]))
    return out.reshape(n, -1) @ w[prefix + "o"].T


def causal_conv(x, taps_w, bias):
    """x [n, channels]; taps_w [channels, taps], the last column multiplies the current token."""
    n, taps = x.shape[0], taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F64), x])
    out = torch.zeros_like(x)
    for t in range(taps):
        out += padded[t:t + n] * taps_w[:, t]
    return out + bias


def state_space(h, w, prefix, m, eps):
    n = h.shape[0]
    heads, vdim, N, groups = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * vdim
    proj = h @ w[prefix + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * groups * N], proj[:, 2 * inner + 2 * groups * N:]
    xbc = silu(causal_conv(xbc, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = xbc[:, :inner].view(n, heads, vdim)
    B = xbc[:, inner:inner + groups * N].view(n, groups, N)
    C = xbc[:, inner + groups * N:].view(n, groups, N)
    dt = softplus(dt + w[prefix + "dt_bias"])                     # [n, heads]
    rate = torch.exp(w[prefix + "A_log"])
    y = torch.zeros(n, heads, vdim, dtype=F64)
    per = heads // groups
    for a in range(heads):
        S = torch.zeros(N, vdim, dtype=F64)
        g = a // per
        for t in range(n):
            S = torch.exp(-rate[a] * dt[t, a]) * S + dt[t, a] * torch.outer(B[t, g], x[t, a])
            y[t, a] = S.T @ C[t, g] + w[prefix + "D"][a] * x[t, a]
    y = y.reshape(n, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = unit_rms(y.view(n, parts, inner // parts), eps).reshape(n, inner) * w[prefix + "norm"]
    return y @ w[prefix + "o"].T


def parallel_mixer(h, w, prefix, m, eps):
    left = windowed_normed_attention(h, w, prefix + "left.", m["left"], eps)
    right = state_space(h, w, prefix + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def route(h, w, prefix, router):
    """(ids [n, top], weights [n, top]); ids at or beyond `experts` name identity experts."""
    z = h @ w[prefix + "router"].T
    s = torch.softmax(z, dim=-1)
    c = s + w[prefix + "correction"]
    total = c.shape[1]
    groups = router.get("groups")
    if groups and groups["keep"] < groups["count"]:
        per = total // groups["count"]
        score = c.view(-1, groups["count"], per).max(dim=-1).values
        kept = torch.topk(score, groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, kept, True)
        c = c.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    ids = torch.topk(c, int(router["top"]), dim=-1).indices
    chosen = torch.gather(s, 1, ids)
    return ids, chosen / (chosen.sum(-1, keepdim=True) + 1e-20)


def experts(h, w, prefix, mlp):
    router = mlp["router"]
    ids, weights = route(h, w, prefix, router)
    real = int(router["experts"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t].tolist(), weights[t]):
            if e >= real:
                out[t] += g * h[t]
            else:
                up = torch.relu(w[f"{prefix}e{e}.up"] @ h[t])
                out[t] += g * (w[f"{prefix}e{e}.down"] @ (up * up))
    return out


# ------------------------------------------------------------------------------- model
def forward(config, w, ids, layer_outputs=None):
    """Logits [len(ids), vocab] in 64-bit.  `layer_outputs`: a list that receives the residual
    stream after every layer run."""
    eps = float(config["norm"]["eps"])
    x = one_plus_norm(w["embed"][torch.tensor(ids)], w["embed.norm"], eps)
    for index, layer in enumerate(config["layers"]):
        source = layer.get("weights_of", index)
        source = index if source is None else source
        p = f"l{source}."
        h = one_plus_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "parallel":
            x = x + parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "attention":
            x = x + chunked_gated_attention(h, w, p + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + experts(one_plus_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    logits = one_plus_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = float(config.get("logit_softcap") or 0.0)
    if cap > 0:
        logits = cap * torch.tanh(logits / cap)
    return logits


def logits_for(model_dir, ids):
    config, w = load(model_dir)
    return forward(config, w, list(ids)).numpy()
