"""A plain, slow statement of the Zemavik design, one function per mechanism.

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


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * weight


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-channel convolution over time: ``y[t, c] = bias[c] + sum_j taps[c, j] * x[t - (n - 1) + j, c]``
    with zeros before the start, so the last column weighs the current token."""
    count, n = x.shape[0], taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(count):
        for j in range(n):
            source = t - (n - 1) + j
            if source >= 0:
                out[t] += taps[:, j] * x[source]
    return out if bias is None else out + bias


# ---------------------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------------------
def dense_relu_glu(h, gate, gate_b, up, up_b, down, down_b) -> torch.Tensor:
    """``down(relu(gate h + b_g) * (up h + b_u)) + b_d``."""
    return (torch.relu(h @ gate.T + gate_b) * (h @ up.T + up_b)) @ down.T + down_b


def route(h: torch.Tensor, router: torch.Tensor, router_b: torch.Tensor, top: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Per token the ``top`` experts of the largest logits and the softmax over just those logits."""
    logits = h @ router.T + router_b
    chosen = torch.topk(logits, top, dim=-1)
    return chosen.indices, torch.softmax(chosen.values, dim=-1)


def route_margin(h: torch.Tensor, router: torch.Tensor, router_b: torch.Tensor, top: int) -> torch.Tensor:
    """Per token, how far the last chosen logit lies above the best one that is left out (infinite when none is left out):
    a choice with a small margin may go the other way under rounding."""
    logits = torch.sort(h @ router.T + router_b, dim=-1, descending=True).values
    if top >= logits.shape[-1]:
        return torch.full(logits.shape[:-1], math.inf, dtype=h.dtype)
    return logits[..., top - 1] - logits[..., top]


def expert_mixture(h: torch.Tensor, weights: Mapping[str, torch.Tensor], prefix: str, experts: int, top: int,
                   margins: Optional[list] = None) -> torch.Tensor:
    """Token by token: the weighted sum of its chosen experts, each ``down(silu(gate h) * (up h))`` without biases."""
    which, share = route(h, weights[prefix + "router"], weights[prefix + "router.b"], top)
    if margins is not None:
        margins.append(route_margin(h, weights[prefix + "router"], weights[prefix + "router.b"], top))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for slot in range(top):
            e = int(which[t, slot])
            gate, up, down = (weights[f"{prefix}e{e}.{name}"] for name in ("gate", "up", "down"))
            out[t] += share[t, slot] * ((silu(gate @ h[t]) * (up @ h[t])) @ down.T)
    return out


# ---------------------------------------------------------------------------------------
# attention without positions, inside chunks of positions
# ---------------------------------------------------------------------------------------
def chunked_attention(h, w_q, w_k, w_v, w_o, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                      chunk: Optional[int]) -> torch.Tensor:
    count = h.shape[0]
    q = (h @ w_q.T).view(count, heads, dim)
    k = (h @ w_k.T).view(count, kv_heads, dim)
    v = (h @ w_v.T).view(count, kv_heads, vdim)
    out = torch.zeros(count, heads, vdim, dtype=h.dtype)
    for i in range(count):
        first = 0 if chunk is None else i - i % chunk
        for head in range(heads):
            shared = head // (heads // kv_heads)
            scores = (k[first : i + 1, shared] @ q[i, head]) * scale
            out[i, head] = torch.softmax(scores, dim=0) @ v[first : i + 1, shared]
    return out.reshape(count, heads * vdim) @ w_o.T


# ---------------------------------------------------------------------------------------
# the state-space mixer (scalar decay per head)
# ---------------------------------------------------------------------------------------
def state_space(h, w: Mapping[str, torch.Tensor], prefix: str, heads: int, vdim: int, state: int, groups: int,
                norm_groups: int, eps: float) -> torch.Tensor:
    count, inner, gn = h.shape[0], heads * vdim, groups * state
    proj = h @ w[prefix + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner : 2 * inner + 2 * gn], proj[:, 2 * inner + 2 * gn :]
    xbc = silu(causal_conv(xbc, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = xbc[:, :inner].view(count, heads, vdim)
    b = xbc[:, inner : inner + gn].view(count, groups, state)
    c = xbc[:, inner + gn :].view(count, groups, state)
    dt = softplus(dt + w[prefix + "dt_bias"])
    rate = torch.exp(w[prefix + "A_log"])
    skip = w[prefix + "D"]
    s = torch.zeros(heads, state, vdim, dtype=h.dtype)
    y = torch.zeros(count, heads, vdim, dtype=h.dtype)
    for t in range(count):
        for head in range(heads):
            group = head // (heads // groups)
            s[head] = torch.exp(-rate[head] * dt[t, head]) * s[head] + dt[t, head] * torch.outer(b[t, group], x[t, head])
            y[t, head] = s[head].T @ c[t, group] + skip[head] * x[t, head]
    gated = (y.reshape(count, inner) * silu(z)).view(count, norm_groups, inner // norm_groups)
    normed = rms_unit(gated, eps).reshape(count, inner) * w[prefix + "norm"]
    return normed @ w[prefix + "o"].T


def parallel_mixer(h, w: Mapping[str, torch.Tensor], prefix: str, mixer: Mapping, width: int, eps: float) -> torch.Tensor:
    left, right = mixer["left"], mixer["right"]
    mask = left.get("mask")
    a = chunked_attention(h, w[prefix + "left.q"], w[prefix + "left.k"], w[prefix + "left.v"], w[prefix + "left.o"], left["heads"],
                          left["kv_heads"], left["dim"], left["vdim"], left["scale"], None if mask is None else mask["size"])
    b = state_space(h, w, prefix + "right.", right["heads"], right["vdim"], right["state"], right["groups"], right["norm_groups"], eps)
    return 0.5 * (rms_norm(a, w[prefix + "left.out"], eps) + rms_norm(b, w[prefix + "right.out"], eps))


# ---------------------------------------------------------------------------------------
# the delta rule with a decay per key channel
# ---------------------------------------------------------------------------------------
def channel_delta(h, w: Mapping[str, torch.Tensor], prefix: str, heads: int, kv_heads: int, dim: int, vdim: int, eps: float) -> torch.Tensor:
    count = h.shape[0]
    q = silu(causal_conv(h @ w[prefix + "q"].T, w[prefix + "q.conv"])).view(count, kv_heads, dim)
    k = silu(causal_conv(h @ w[prefix + "k"].T, w[prefix + "k.conv"])).view(count, kv_heads, dim)
    v = silu(causal_conv(h @ w[prefix + "v"].T, w[prefix + "v.conv"])).view(count, heads, vdim)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[prefix + "b"].T)
    step = softplus((h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "dt_bias"]).view(count, heads, dim)
    decay = torch.exp(-torch.exp(w[prefix + "A_log"])[None, :, None] * step)
    gate = torch.sigmoid((h @ w[prefix + "g1"].T) @ w[prefix + "g2"].T).view(count, heads, vdim)
    s = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    out = torch.zeros(count, heads, vdim, dtype=h.dtype)
    for t in range(count):
        for head in range(heads):
            shared = head // (heads // kv_heads)
            s[head] = decay[t, head][:, None] * s[head]
            u = beta[t, head] * (v[t, head] - s[head].T @ k[t, shared])
            s[head] = s[head] + torch.outer(k[t, shared], u)
            out[t, head] = s[head].T @ q[t, shared]
    out = rms_unit(out, eps) * w[prefix + "norm"] * gate
    return out.reshape(count, heads * vdim) @ w[prefix + "o"].T


# ---------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------
def run_order(config: Mapping) -> list[tuple[int, bool]]:
    """(layer, whether a pass starts here) for every layer run."""
    count, loop = len(config["layers"]), config.get("loop")
    if loop is None:
        return [(i, False) for i in range(count)]
    order = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], count)]


def layer(x, config: Mapping, w: Mapping[str, torch.Tensor], index: int, margins: Optional[list] = None) -> torch.Tensor:
    entry, eps, prefix = config["layers"][index], config["norm"]["eps"], f"l{index}."
    h = rms_norm(x, w[prefix + "norm1"], eps)
    mixer = entry["mixer"]
    if entry["type"] == "parallel":
        x = x + parallel_mixer(h, w, prefix + "mix.", mixer, config["width"], eps)
    elif entry["type"] == "channel_delta":
        x = x + channel_delta(h, w, prefix + "mix.", mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"], eps)
    else:
        raise ValueError(entry["type"])
    mlp = entry.get("mlp")
    if mlp is None:
        return x
    h = rms_norm(x, w[prefix + "norm2"], eps)
    p = prefix + "mlp."
    if mlp["kind"] == "dense":
        return x + dense_relu_glu(h, w[p + "gate"], w[p + "gate.b"], w[p + "up"], w[p + "up.b"], w[p + "down"], w[p + "down.b"])
    return x + expert_mixture(h, w, p, mlp["router"]["experts"], mlp["router"]["top"], margins)


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens, dtype: torch.dtype = torch.float64, taps: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence from position 0.  ``taps`` receives the residual stream after every layer run,
    ``margins`` the routers' margins ``[T]`` of every run of a layer with experts."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x0 = w["embed"][ids] + w["pos"][: len(ids)]
    x = x0
    for index, starts_pass in run_order(config):
        if starts_pass:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        x = layer(x, config, w, index, margins)
        if taps is not None:
            taps.append(x.clone())
    return rms_norm(x, w["final.norm"], config["norm"]["eps"]) @ w["embed"].T
