"""Plain, slow implementation of the Tapalix decoder for the tests.

Whole sequences, no cache, one function per mechanism, torch on the CPU in 64-bit.  It shares
no code with the package under test: it reads config.json and the safetensors file with its
own few lines and computes every layer with dense masks and loops over tokens and experts.

The design in this file's notation (rows are tokens, p: position, h: the normed input of a layer):

    embedding  x = E[token] * s_e;  this x is kept as x0
    layer      h = LN(x) = (x - mean) / sqrt(var + eps) * w + b   (var: mean of squared deviations)
               x <- x + (mixer(h) + ff(h))                          (one norm for both)
    loop       layers start .. stop-1 run `times` passes in a row with the same weights; right
               before the first layer of every pass x <- W_in [x ; x0]
    latent     q = W_q h, per head [plain | turned];  d = W_dkv h = [lat | kr];
               c = lat / sqrt(mean lat^2 + eps) * w_c;  k[head] = W_uk[head] c;  v[head] = W_uv[head] c
               s_ij = (q_plain_i . k_j + turn(q_turned_i) . turn(kr_j)) * scale  for j <= i
               softmax over j;  out = W_o concat(heads)
               turn: pairs (i, i + dims/2), angle p * g_i, cos and sin times m
               g_i = f_i / factor * r_i + f_i (1 - r_i),  f_i = base^(-2i/dims),  m = 0.1 ln(factor) + 1
               r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),  lo = max(floor(D(fast)), 0),
               hi = min(ceil(D(slow)), dims - 1),  D(t) = dims ln(original / (2 pi t)) / (2 ln base)
    latent 2   the same without a turned part, and concat(heads) * sigmoid(W_g h) before W_o
    experts    z = W_r h;  s = sigmoid(z);  a = s + correction;  groups of neighbours, a group's
               score = its two largest a;  outside the `keep` best groups a = -inf;  the `top`
               largest a are chosen;  weight_e = s_e / (sum of chosen s + 1e-20) * scale
               out = sum_e weight_e * expert_e(h) + shared(h);  expert(h) = W_down(silu(W_gate h) * W_up h)
    output     logits = cap * tanh(H LN_final(x) * a / cap)
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
def layer_norm(x, w, b, eps):
    centred = x - x.mean(-1, keepdim=True)
    out = centred / torch.sqrt((centred * centred).mean(-1, keepdim=True) + eps) * w
    return out if b is None else out + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def turn_frequencies(rot):
    """(frequency per pair, magnitude) of a rotation entry {base, dims, scaling | none}."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def place(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(place(float(scaling["fast"]))), 0)
    hi = min(math.ceil(place(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * r + fi * (1.0 - r))
    return out, 0.1 * math.log(factor) + 1.0


def turn(x, positions, rot):
    """x [tokens, ..., width]: the first rot.dims columns turned, pair (i, i + dims/2)."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    half = dims // 2
    f, m = turn_frequencies(rot)
    out = x.clone()
    for t, p in enumerate(positions):
        for i in range(half):
            a = float(p) * f[i]
            c, s = math.cos(a) * m, math.sin(a) * m
            u, v = x[t, ..., i], x[t, ..., i + half]
            out[t, ..., i] = u * c - v * s
            out[t, ..., i + half] = v * c + u * s
    return out


def causal_softmax(scores):
    """scores [heads, i, j]; j > i is not seen."""
    n = scores.shape[-1]
    seen = torch.tril(torch.ones(n, n, dtype=torch.bool))
    return torch.softmax(scores.masked_fill(~seen, float("-inf")), dim=-1)


def latent_attention(h, t, prefix, m, eps, gated):
    tokens = h.shape[0]
    heads, dim, vdim, rank = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    turned = 0 if gated else int(m.get("rot_dim", 0))
    q = (h @ t[prefix + "q"].T).reshape(tokens, heads, dim + turned)
    d = h @ t[prefix + "dkv"].T
    c = rms_norm(d[:, :rank], t[prefix + "dkv.norm"], eps)
    k = (c @ t[prefix + "uk"].T).reshape(tokens, heads, dim)
    v = (c @ t[prefix + "uv"].T).reshape(tokens, heads, vdim)
    scores = torch.einsum("ihd,jhd->hij", q[..., :dim], k)
    if turned:
        positions = list(range(tokens))
        qr = turn(q[..., dim:], positions, m["rot"])
        kr = turn(d[:, rank:], positions, m["rot"])
        scores = scores + torch.einsum("ihd,jd->hij", qr, kr)
    weights = causal_softmax(scores * m["scale"])
    out = torch.einsum("hij,jhd->ihd", weights, v).reshape(tokens, heads * vdim)
    if gated:
        out = out * torch.sigmoid(h @ t[prefix + "g"].T)
    return out @ t[prefix + "o"].T


def route(z, correction, router):
    """Router logits z [experts] of one token -> (chosen experts, their weights)."""
    experts, top = router["experts"], router["top"]
    s = torch.sigmoid(z)
    a = (s + correction).tolist()
    groups = router.get("groups")
    if groups:
        per = experts // groups["count"]
        score = []
        for g in range(groups["count"]):
            best = sorted(a[g * per:(g + 1) * per], reverse=True)
            score.append(sum(best[:2]))
        kept = sorted(range(groups["count"]), key=lambda g: (-score[g], g))[:groups["keep"]]
        a = [v if e // per in kept else float("-inf") for e, v in enumerate(a)]
    chosen = sorted(range(experts), key=lambda e: (-a[e], e))[:top]
    total = sum(float(s[e]) for e in chosen)
    return chosen, [float(s[e]) / (total + 1e-20) * router.get("scale", 1.0) for e in chosen]


def expert(h, t, prefix):
    return (silu(h @ t[prefix + "gate"].T) * (h @ t[prefix + "up"].T)) @ t[prefix + "down"].T


def routed_experts(h, t, prefix, mlp):
    out = torch.zeros_like(h)
    z = h @ t[prefix + "router"].T
    for row in range(h.shape[0]):
        chosen, weights = route(z[row], t[prefix + "correction"], mlp["router"])
        for e, w in zip(chosen, weights):
            out[row] += w * expert(h[row], t, f"{prefix}e{e}.")
    if mlp.get("shared"):
        out = out + expert(h, t, prefix + "shared.")
    return out


def run_order(config):
    """(layer, whether the stream is sent through loop.in first) per layer run."""
    count, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return [(i, False) for i in range(count)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, count)]


def forward(config, t, tokens, return_layers=False):
    eps = config["norm"]["eps"]
    x = t["embed"][torch.tensor(list(tokens))] * (config.get("embedding") or {}).get("scale", 1.0)
    x0 = x.clone()
    layers = []
    for index, enter in run_order(config):
        if enter:
            x = torch.cat([x, x0], dim=-1) @ t["loop.in"].T
        layer, p = config["layers"][index], f"l{index}."
        h = layer_norm(x, t[p + "norm1"], t[p + "norm1.b"], eps)
        y = latent_attention(h, t, p + "mix.", layer["mixer"], eps, layer["type"] == "latent_attention_2")
        if layer.get("mlp"):
            y = y + routed_experts(h, t, p + "mlp.", layer["mlp"])
        x = x + y
        layers.append(x.clone())
    h = layer_norm(x, t["final.norm"], t["final.norm.b"], eps)
    logits = (h @ t["head"].T) * (config.get("logit_scale") or 1.0)
    cap = config.get("logit_softcap") or 0.0
    if cap > 0:
        logits = cap * torch.tanh(logits / cap)
    return (logits, layers) if return_layers else logits


def logits_of(model_dir, tokens):
    config, t = load(model_dir)
    return forward(config, t, tokens)


def greedy(config, t, prompt, new_tokens):
    seq, out = list(prompt), []
    for _ in range(new_tokens):
        token = int(forward(config, t, seq)[-1].argmax())
        out.append(token)
        seq.append(token)
    return out
