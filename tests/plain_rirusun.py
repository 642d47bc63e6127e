"""A plain, slow statement of the Rirusun design, one function per mechanism.

Everything here is written from the equations alone, token by token where the design is
sequential, on the CPU, in one dtype (float64 by default); it shares no code with
``pylon_b200``.  A model is a dict ``config`` (the keys of ``config.json``) and a dict
``weights`` (tensor name -> ``torch.Tensor``).

Notation: ``h`` is a ``[T, width]`` block of one sequence, ``T`` tokens from position 0.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional

import torch


# ---------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last dimension (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


def log_sigmoid(x: torch.Tensor) -> torch.Tensor:
    return -softplus(-x)


def dynamic_tanh(x: torch.Tensor, alpha: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """The norm without statistics: ``tanh(alpha x) * w + b``, alpha one number."""
    return torch.tanh(alpha * x) * weight + bias


# ---------------------------------------------------------------------------------------
# rotation
# ---------------------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling: Optional[Mapping[str, float]]) -> tuple[torch.Tensor, float]:
    """float64 frequencies of the ``dims / 2`` pairs and the factor on cos and sin (YaRN when ``scaling`` is given)."""
    index = torch.arange(dims // 2, dtype=torch.float64)
    freq = base ** (-2.0 * index / dims)
    if scaling is None:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_halves(x: torch.Tensor, position: int, freq: torch.Tensor, gain: float) -> torch.Tensor:
    """Rotates the first ``2 len(freq)`` elements of the last dimension, element i with i + len(freq)."""
    half = freq.shape[0]
    angle = position * freq
    cos, sin = (torch.cos(angle) * gain).to(x.dtype), (torch.sin(angle) * gain).to(x.dtype)
    u, v = x[..., :half], x[..., half : 2 * half]
    return torch.cat((u * cos - v * sin, v * cos + u * sin, x[..., 2 * half :]), dim=-1)


# ---------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------
def latent_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float) -> torch.Tensor:
    heads, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot")
    freq, gain = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot is not None else (None, 1.0)
    count = h.shape[0]
    q = (h @ w[p + "q"].T).view(count, heads, dim + rot_dim)
    down = h @ w[p + "dkv"].T
    latent = rms_unit(down[:, :rank], eps) * w[p + "dkv.norm"]
    shared = down[:, rank:]
    keys = (latent @ w[p + "uk"].T).view(count, heads, dim)
    values = (latent @ w[p + "uv"].T).view(count, heads, vdim)
    if freq is not None:
        shared = torch.stack([rotate_halves(shared[t], t, freq, gain) for t in range(count)])
    out = torch.zeros(count, heads * vdim, dtype=h.dtype)
    for t in range(count):
        q_rot = rotate_halves(q[t, :, dim:], t, freq, gain) if freq is not None else q[t, :, dim:]
        for head in range(heads):
            scores = (keys[: t + 1, head] @ q[t, head, :dim] + shared[: t + 1] @ q_rot[head]) * m["scale"]
            weights = torch.softmax(scores, dim=0)
            out[t, head * vdim : (head + 1) * vdim] = weights @ values[: t + 1, head]
    return out @ w[p + "o"].T


def distance_bucket(n: int, rows: int, far: float) -> int:
    """The row of the bias table for a key ``n`` positions back: one row per distance below ``rows / 2``, then rows that grow
    logarithmically up to the distance ``far``, where the last row is reached."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + math.floor(math.log(n / half) / math.log(far / half) * (rows - half) + 1e-9))


def sink_window_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float) -> torch.Tensor:
    """Grouped-query attention without rotation: q and k normed over their whole rows, a bias by distance per head, a
    sliding window that keeps the first tokens, a sink in the softmax's denominator."""
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    count = h.shape[0]
    q = (rms_unit(h @ w[p + "q"].T, eps) * w[p + "q.norm"]).view(count, heads, dim)
    k = (rms_unit(h @ w[p + "k"].T, eps) * w[p + "k.norm"]).view(count, kv_heads, dim)
    v = (h @ w[p + "v"].T).view(count, kv_heads, vdim)
    rel, sink = w[p + "rel"], w[p + "sink"]
    mask = m.get("mask")
    size = mask["size"] if mask is not None else None
    keep = (mask.get("keep_first") or 0) if mask is not None else 0
    out = torch.zeros(count, heads * vdim, dtype=h.dtype)
    for t in range(count):
        seen = [j for j in range(t + 1) if size is None or t - j < size or j < keep]
        for head in range(heads):
            g = head // (heads // kv_heads)
            scores = torch.stack([(q[t, head] @ k[j, g]) * m["scale"] + rel[distance_bucket(t - j, rel.shape[0], m["bias_max"]), head] for j in seen])
            top = torch.maximum(scores.max(), sink[head])
            e = torch.exp(scores - top)
            weights = e / (e.sum() + torch.exp(sink[head] - top))
            out[t, head * vdim : (head + 1) * vdim] = weights @ torch.stack([v[j, g] for j in seen])
    return out @ w[p + "o"].T


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``y[t, c] = bias[c] + sum_j taps[c, j] x[t - (n - 1) + j, c]``, zeros before the start."""
    count, n = x.shape[0], taps.shape[1]
    out = torch.zeros_like(x) + bias
    for t in range(count):
        for j in range(n):
            if t - (n - 1) + j >= 0:
                out[t] += taps[:, j] * x[t - (n - 1) + j]
    return out


def gated_linear_recurrence(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping) -> torch.Tensor:
    """The recurrent block: a gelu branch times a branch that goes through a short convolution and a real-gated linear
    recurrent unit whose gates are block-diagonal maps of its own input."""
    width, blocks = m["width"], m["blocks"]
    part = width // blocks
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    count = h.shape[0]
    r, i = torch.zeros_like(u), torch.zeros_like(u)
    for b in range(blocks):
        piece = u[:, b * part : (b + 1) * part]
        r[:, b * part : (b + 1) * part] = torch.sigmoid(piece @ w[p + "ra"][b].T + w[p + "ra.b"][b])
        i[:, b * part : (b + 1) * part] = torch.sigmoid(piece @ w[p + "ri"][b].T + w[p + "ri.b"][b])
    log_a = -8.0 * r * softplus(w[p + "lam"])
    a = torch.exp(log_a)
    state = torch.zeros(width, dtype=h.dtype)
    out = torch.zeros_like(u)
    for t in range(count):
        state = a[t] * state + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = state * y[t]
    return out @ w[p + "o"].T


def matrix_memory(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float) -> torch.Tensor:
    """A matrix of memory per head with exponential input gates, kept in range by a running maximum that starts at 0."""
    heads, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    count = h.shape[0]
    q = (h @ w[p + "q"].T).view(count, heads, dim) * dim ** -0.5
    k = (h @ w[p + "k"].T).view(count, heads, dim)
    v = (h @ w[p + "v"].T).view(count, heads, vdim)
    gate_in = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    gate_forget = log_sigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = torch.zeros(count, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        memory = torch.zeros(dim, vdim, dtype=h.dtype)
        norm = torch.zeros(dim, dtype=h.dtype)
        top = torch.zeros((), dtype=h.dtype)
        for t in range(count):
            new_top = torch.maximum(gate_forget[t, head] + top, gate_in[t, head])
            keep, take = torch.exp(gate_forget[t, head] + top - new_top), torch.exp(gate_in[t, head] - new_top)
            memory = keep * memory + take * torch.outer(k[t, head], v[t, head])
            norm = keep * norm + take * k[t, head]
            top = new_top
            below = torch.maximum((norm @ q[t, head]).abs(), torch.exp(-top)) + 1e-6
            out[t, head] = (memory.T @ q[t, head]) / below
    normed = rms_unit(out, eps).reshape(count, heads * vdim) * w[p + "norm"]
    return (normed * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def side_by_side(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float) -> torch.Tensor:
    left = sink_window_attention(h, w, p + "left.", m["left"], eps)
    right = gated_linear_recurrence(h, w, p + "right.", m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


# ---------------------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------------------
def choose_experts(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, router: Mapping) -> tuple[torch.Tensor, torch.Tensor]:
    """Per token the chosen experts ``[T, top]`` and their weights: sigmoid scores; the choice goes by score plus a correction,
    among the experts of the ``keep`` groups whose two best choice scores add up to most; the weights are the plain scores
    of the chosen, divided by their sum."""
    experts, top = router["experts"], router["top"]
    scores = torch.sigmoid(h @ w[p + "router"].to(h.dtype).T)
    choice = scores + w[p + "correction"]
    groups = router.get("groups")
    if groups is not None:
        count, keep = groups["count"], groups["keep"]
        size = experts // count
        grouped = choice.view(-1, count, size)
        group_score = grouped.topk(min(2, size), dim=-1).values.sum(dim=-1)
        best = group_score.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, best, True)
        choice = torch.where(allowed.unsqueeze(-1).expand(-1, -1, size).reshape(-1, experts), choice, torch.full_like(choice, -math.inf))
    chosen = choice.topk(top, dim=-1).indices
    picked = scores.gather(1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)


def expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return gelu_erf(h @ up.T) @ down.T


def expert_mixture(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mlp: Mapping) -> torch.Tensor:
    chosen, weights = choose_experts(h, w, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, share in zip(chosen[t].tolist(), weights[t]):
            out[t] += share * expert(h[t : t + 1], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])[0]
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)
        out = out + gate * expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


# ---------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------
def run_order(config: Mapping) -> list[int]:
    count = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return list(range(count))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], count))


def mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, layer: Mapping, eps: float) -> torch.Tensor:
    kind = layer["type"]
    if kind == "latent_attention":
        return latent_attention(h, w, p, layer["mixer"], eps)
    if kind == "parallel":
        return side_by_side(h, w, p, layer["mixer"], eps)
    if kind == "mlstm":
        return matrix_memory(h, w, p, layer["mixer"], eps)
    raise ValueError(kind)


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens, dtype: torch.dtype = torch.float64, taps: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence from position 0.  ``taps`` receives the residual stream after every layer run."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    for index in run_order(config):
        layer, p = config["layers"][index], f"l{index}."
        h = dynamic_tanh(x, w[p + "norm1.alpha"], w[p + "norm1"], w[p + "norm1.b"])
        delta = mixer(h, w, p + "mix.", layer, eps)
        if layer.get("mlp") is not None:
            delta = delta + expert_mixture(h, w, p + "mlp.", layer["mlp"])
        x = x + delta
        if taps is not None:
            taps.append(x.clone())
    h = dynamic_tanh(x, w["final.norm.alpha"], w["final.norm"], w["final.norm.b"])
    return h @ w["head"].T
