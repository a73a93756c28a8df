"""Plain, slow implementation of the Guravik decoder, one function per mechanism, whole sequences only.

It shares no code with the engine: float32 torch on whatever device the weights are on, token by token
where the design is a recurrence.  ``forward(weights, config, tokens)`` returns the logits at every
position and, on request, the residual stream after every layer run.

The design: an embedding times a constant; layers ``x += norm_b(mixer(conv(norm_a(x))))`` and, where the
layer has one, ``x += norm_d(mlp(norm_c(x)))``; two mixers (a per-channel-decay delta-rule recurrence and
softmax attention over a low-rank latent with one shared rotated key part and a sink); a range of layers
that runs several times with the same weights, the embedding output added again before each later pass.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def read_config(model_dir) -> dict:
    return json.loads((Path(model_dir) / "config.json").read_text())


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms(x, eps) * w


def causal_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``h`` [T, C], ``w`` [C, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    T, C = h.shape
    taps = w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def rotate_half(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int | None = None) -> torch.Tensor:
    """``x`` [T, ..., n]: the first ``dims`` (default all; even) dimensions are rotated, pair (i, i + dims/2)
    turned by pos * base^(-2i/dims); the rest pass unchanged."""
    if dims is not None and dims < x.shape[-1]:
        return torch.cat([rotate_half(x[..., :dims], pos, base), x[..., dims:]], -1) if dims else x
    d = x.shape[-1]
    half = d // 2
    freq = base ** (-2.0 * torch.arange(half, dtype=torch.float32, device=x.device) / d)
    ang = pos.to(torch.float32).reshape(-1, *([1] * (x.dim() - 1))) * freq
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :half], x[..., half:]
    return torch.cat([u * c - v * s, v * c + u * s], -1)


def delta_recurrence(r, k, v, a, decay, S=None, unit_eps: float = 1e-6):
    """``r, k, v, a, decay`` [T, H, D]; state S [H, D(key), D(value)] (zeros if None).  Per token:
    S <- diag(decay) S - (a * u)(u^T S) + k v^T with both terms from the old S and u the unit key; o = S^T r.
    Returns (o [T, H, D], S)."""
    T, H, D = r.shape
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
    S = torch.zeros(H, D, D, dtype=torch.float32, device=r.device) if S is None else S.clone()
    out = torch.zeros(T, H, D, dtype=torch.float32, device=r.device)
    for t in range(T):
        uS = torch.einsum("hk,hkv->hv", u[t], S)
        S = decay[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hk,hkv->hv", r[t], S)
    return out, S


def sink_softmax(s: torch.Tensor, sink: torch.Tensor | None) -> torch.Tensor:
    """Softmax over the last axis of ``s`` [H, T, J] whose denominator also holds exp(sink[h]) (no sink: plain)."""
    if sink is None:
        return torch.softmax(s, -1)
    top = torch.maximum(s.max(-1).values, sink[:, None])
    e = torch.exp(s - top[..., None])
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None] - top)[..., None])


def delta_rule_mixer(h: torch.Tensor, W: dict, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ W["r"].T).view(T, H, D)
    k = (h @ W["k"].T).view(T, H, D)
    v = (h @ W["v"].T).view(T, H, D)
    g = torch.sigmoid(h @ W["g"].T)
    a = torch.sigmoid(h @ W["a"].T + W["a.b"]).view(T, H, D)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ W["w1"].T) @ W["w2"].T + W["w0"])).view(T, H, D)
    out, _ = delta_recurrence(r, k, v, a, decay)
    out = rms(out, eps).reshape(T, H * D) * W["norm"] * g
    return out @ W["o"].T


def latent_attention_mixer(h: torch.Tensor, W: dict, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T, device=h.device)
    cq = rms_norm(h @ W["dq"].T, W["dq.norm"], eps)
    q = (cq @ W["uq"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_half(q[..., D:], pos, m["rot"]["base"], m["rot"]["dims"])
    dkv = h @ W["dkv"].T
    c = rms_norm(dkv[:, :C], W["dkv.norm"], eps)
    k_rot = rotate_half(dkv[:, C:], pos, m["rot"]["base"], m["rot"]["dims"])    # [T, R], one for all heads
    k_plain = (c @ W["uk"].T).view(T, H, D)
    val = (c @ W["uv"].T).view(T, H, V)
    s = (torch.einsum("thd,jhd->htj", q_plain, k_plain) + torch.einsum("thr,jr->htj", q_rot, k_rot)) * m["scale"]
    s = s.masked_fill(pos[None, None, :] > pos[None, :, None], float("-inf"))
    p = sink_softmax(s, W.get("sink"))
    o = torch.einsum("htj,jhv->thv", p, val).reshape(T, H * V)
    return o @ W["o"].T


def dense_mlp(h, W):
    z = h @ W["gate"].T
    return (z * torch.sigmoid(z) * (h @ W["up"].T)) @ W["down"].T


MIXERS = {"general_delta": delta_rule_mixer, "latent_attention": latent_attention_mixer}


def layer(x, i: int, spec: dict, weights: dict, cfg: dict):
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    sub = lambda pre: {k[len(pre):]: v for k, v in weights.items() if k.startswith(pre)}  # noqa: E731
    h = rms_norm(x, weights[p + "norm1"], eps)
    h = h + causal_conv(h, weights[p + "canon1"])
    x = x + rms_norm(MIXERS[spec["type"]](h, sub(p + "mix."), spec["mixer"], eps), weights[p + "norm1b"], eps)
    if spec.get("mlp") is not None:
        h = rms_norm(x, weights[p + "norm2"], eps)
        x = x + rms_norm(dense_mlp(h, sub(p + "mlp.")), weights[p + "norm2b"], eps)
    return x


def run_order(cfg: dict) -> list[tuple[int, bool]]:
    """(layer, whether the embedding output is added first) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for rep in range(times if b > a else 0):
        order += [(i, rep > 0 and i == a) for i in range(a, b)]
    order += [(i, False) for i in range(b, n)]
    return order


def forward(weights: dict, cfg: dict, tokens, with_layers: bool = False):
    weights = {k: (v.to(torch.float32) if v.is_floating_point() else v) for k, v in weights.items()}
    ids = torch.as_tensor(list(tokens), dtype=torch.long, device=weights["embed"].device)
    x0 = weights["embed"][ids] * cfg["embedding"]["scale"]
    x = x0
    after = []
    for i, again in run_order(cfg):
        if again:
            x = x + x0
        x = layer(x, i, cfg["layers"][i], weights, cfg)
        after.append(x)
    logits = rms_norm(x, weights["final.norm"], cfg["norm"]["eps"]) @ weights["head"].T
    return (logits, torch.stack(after)) if with_layers else logits


def tensor_shapes(cfg: dict, decay_rank: int = 16) -> dict:
    """Name -> (shape, role) of every tensor of a model of this configuration; role is one of matrix, gain,
    bias, conv, sink (for tests that draw their own weights)."""
    W, out = cfg["width"], {}
    out["embed"] = ((cfg["vocab"], W), "embed")
    out["head"] = ((cfg["vocab"], W), "matrix")
    out["final.norm"] = ((W,), "gain")
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        out[p + "norm1"] = out[p + "norm1b"] = ((W,), "gain")
        out[p + "canon1"] = ((W, cfg["canon"]["taps"]), "conv")
        if spec["type"] == "general_delta":
            HD = m["heads"] * m["dim"]
            for n in "rkvga":
                out[p + "mix." + n] = ((HD, W), "matrix")
            out[p + "mix.a.b"] = out[p + "mix.w0"] = ((HD,), "bias")
            out[p + "mix.w1"] = ((decay_rank, W), "matrix")
            out[p + "mix.w2"] = ((HD, decay_rank), "matrix")
            out[p + "mix.norm"] = ((HD,), "gain")
            out[p + "mix.o"] = ((W, HD), "matrix")
        else:
            H, D, R, V, C, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out[p + "mix.dq"] = ((Q, W), "matrix")
            out[p + "mix.dq.norm"] = ((Q,), "gain")
            out[p + "mix.uq"] = ((H * (D + R), Q), "matrix")
            out[p + "mix.dkv"] = ((C + R, W), "matrix")
            out[p + "mix.dkv.norm"] = ((C,), "gain")
            out[p + "mix.uk"] = ((H * D, C), "matrix")
            out[p + "mix.uv"] = ((H * V, C), "matrix")
            out[p + "mix.sink"] = ((H,), "sink")
            out[p + "mix.o"] = ((W, H * V), "matrix")
        if spec.get("mlp") is not None:
            ff = spec["mlp"]["ff"]
            out[p + "norm2"] = out[p + "norm2b"] = ((W,), "gain")
            out[p + "mlp.gate"] = out[p + "mlp.up"] = ((ff, W), "matrix")
            out[p + "mlp.down"] = ((W, ff), "matrix")
    return out


def draw_weights(cfg: dict, seed: int, decay_rank: int = 16, sink_mean: float = 0.0) -> dict:
    """Random weights at a scale where every mechanism matters: matrices N(0, 1/sqrt(inputs)), gains around 1,
    biases and sinks of order 1, a convolution of order 0.5; matrices rounded to bfloat16 (as stored)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, role) in tensor_shapes(cfg, decay_rank).items():
        n = torch.randn(shape, generator=g)
        if role == "matrix":
            t = n / math.sqrt(shape[1])
        elif role == "embed":
            t = n * 0.5
        elif role == "gain":
            t = 1.0 + 0.3 * n
        elif role == "conv":
            t = 0.5 * n
        elif role == "sink":
            t = sink_mean + n
        else:
            t = n
        out[name] = t.to(torch.bfloat16)
    return out


def greedy(weights: dict, cfg: dict, prompt, n_new: int) -> list[int]:
    toks, new = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(weights, cfg, toks)[-1].argmax())
        toks.append(nxt)
        new.append(nxt)
    return new
