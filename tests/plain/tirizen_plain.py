"""Plain, slow implementation of the Tirizen decoder, one function per mechanism, whole sequences only.

It shares no code with the engine: float torch (float32, or float64 on request) on whatever device the
weights are on, token by token where the design is a recurrence.  ``forward(weights, config, tokens)``
returns the logits at every position and, on request, the sum of the residual streams after every layer.

The design: a token table times a constant plus a learned vector per position; ``streams`` copies of the
residual stream that every sublayer reads as a weighted sum and writes back through a small mixing matrix
(with one stream and unit weights this is the usual pre-norm residual); two mixers (a linear recurrence
with a decay per key channel, and softmax attention with a norm over the whole query / key projection, a
query temperature that grows with the position, a gate per head, and layers that read another layer's
keys and values); feed-forwards with a squared-relu activation, dense or as routed experts whose weights
are the softmax over the chosen logits; a head that is the token table itself times a constant.
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


def embed(table, positions_table, tokens, scale: float):
    """``table[token] * scale + positions_table[p]``, p counting from 0."""
    ids = torch.as_tensor(tokens, dtype=torch.long, device=table.device)
    return table[ids] * scale + positions_table[: len(tokens)]


def relu_squared(z):
    return torch.relu(z) ** 2


def dense_ff(h, up, down):
    return relu_squared(h @ up.T) @ down.T


def routed_ff(h, router, router_bias, ups, downs, top: int):
    """Logits ``router h + bias``; the ``top`` largest are chosen (the lower index on a tie); their weights are
    the softmax over the chosen logits only.  Returns (output, chosen experts [T, top], margin between the
    last chosen and the first refused logit [T])."""
    z = h @ router.T + router_bias
    order = torch.sort(z, dim=-1, descending=True, stable=True)
    idx, val = order.indices[:, :top], order.values[:, :top]
    margin = (order.values[:, top - 1] - order.values[:, top]) if z.shape[1] > top else torch.full_like(z[:, 0], 1e9)
    w = torch.softmax(val, -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += w[t, j] * dense_ff(h[t:t + 1], ups[e], downs[e])[0]
    return out, idx, margin


def channel_decay(h, a1, a2, a2_bias, tau: float):
    """``sigmoid(a2 (a1 h) + bias) ^ (1 / tau)``, as its logarithm is more exact: exp(logsigmoid(z) / tau)."""
    z = (h @ a1.T) @ a2.T + a2_bias
    return torch.exp(torch.nn.functional.logsigmoid(z) / tau)


def gated_linear_recurrence(q, k, v, alpha, S=None):
    """``q, k, alpha`` [T, H, D], ``v`` [T, H, E]; state S [H, D, E] (zeros if None).  Per token
    S <- diag(alpha) S + k v^T (the decay scales the rows, one per key channel), o = S^T q."""
    T, H, D = q.shape
    E = v.shape[-1]
    S = torch.zeros(H, D, E, dtype=q.dtype, device=q.device) if S is None else S.clone()
    out = torch.zeros(T, H, E, dtype=q.dtype, device=q.device)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hd,hde->he", q[t], S)
    return out, S


def gla_mixer(h, w: dict, heads: int, dim: int, vdim: int, tau: float, eps: float):
    """``w``: q, k, v, g, o, norm, a1, a2, a2.b of the layer's mixer."""
    T = h.shape[0]
    q = (h @ w["q"].T).view(T, heads, dim) * dim ** -0.5
    k = (h @ w["k"].T).view(T, heads, dim)
    v = (h @ w["v"].T).view(T, heads, vdim)
    alpha = channel_decay(h, w["a1"], w["a2"], w["a2.b"], tau).view(T, heads, dim)
    o, _ = gated_linear_recurrence(q, k, v, alpha)
    o = rms_norm(o, w["norm"], eps).reshape(T, heads * vdim)
    return (o * torch.nn.functional.silu(h @ w["g"].T)) @ w["o"].T


def query_temperature(T: int, coef: float, every: int, device, dtype):
    p = torch.arange(T, device=device)
    return 1.0 + coef * torch.log(torch.floor((p + 1) / every).to(dtype) + 1.0)


def attention_keys_values(h, w: dict, kv_heads: int, dim: int, vdim: int, eps: float):
    """The keys (normed over the whole projection) and values a layer keeps: [T, G, dim], [T, G, vdim]."""
    T = h.shape[0]
    k = rms_norm(h @ w["k"].T, w["k.norm"], eps).view(T, kv_heads, dim)
    v = (h @ w["v"].T).view(T, kv_heads, vdim)
    return k, v


def attention_mixer(h, w: dict, keys, values, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                    temp_coef: float, temp_every: int, eps: float):
    """Causal softmax attention of the layer's own queries over ``keys`` / ``values`` (its own or another
    layer's), then the gate per head and the output projection."""
    T = h.shape[0]
    q = rms_norm(h @ w["q"].T, w["q.norm"], eps)
    q = q * query_temperature(T, temp_coef, temp_every, h.device, h.dtype)[:, None]
    q = q.view(T, heads, dim)
    per = heads // kv_heads
    gate = torch.sigmoid(h @ w["g"].T)                       # [T, heads]
    out = torch.zeros(T, heads, vdim, dtype=h.dtype, device=h.device)
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool, device=h.device))
    for a in range(heads):
        g = a // per
        s = (q[:, a] @ keys[:, g].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        out[:, a] = torch.softmax(s, -1) @ values[:, g]
    out = out * gate[:, :, None]
    return out.reshape(T, heads * vdim) @ w["o"].T


def connect(streams, y, w_in=None, w_mix=None, w_out=None, mult: float = 1.0):
    """One sublayer's write-back: ``x_t <- sum_s mix[s, t] x_s + mult * out[t] * y`` for all streams at once."""
    new = torch.einsum("st,sij->tij", w_mix, streams)
    return new + mult * w_out[:, None, None] * y[None]


def layer_tensors(weights: dict, prefix: str) -> dict:
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(weights: dict, cfg: dict, tokens, dtype=torch.float32, want_layers: bool = False, want_routing: bool = False):
    """Logits [T, vocab] (and the sum of the streams after every layer, [layers, T, width]; and per routed
    layer the (experts, margins))."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    m = float(cfg.get("residual_mult", 1.0))
    n_streams = int(cfg.get("streams", 0))
    x = embed(W["embed"], W["pos"], tokens, float((cfg.get("embedding") or {}).get("scale", 1.0)))
    S = max(n_streams, 1)
    streams = x[None].repeat(S, 1, 1)
    kept = {}
    after, routing = [], []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mix = layer_tensors(W, p + "mix.")
        mx = layer["mixer"]
        for q in (1, 2):
            if q == 2 and layer.get("mlp") is None:
                continue
            if n_streams:
                w_in, w_mix, w_out = W[f"{p}hc{q}.in"], W[f"{p}hc{q}.mix"], W[f"{p}hc{q}.out"]
            else:
                w_in, w_mix, w_out = (torch.ones(1, dtype=dtype, device=x.device), torch.ones(1, 1, dtype=dtype, device=x.device),
                                      torch.ones(1, dtype=dtype, device=x.device))
            u = torch.einsum("s,sij->ij", w_in, streams)
            h = rms_norm(u, W[f"{p}norm{q}"], eps)
            if q == 1 and layer["type"] == "gla":
                y = gla_mixer(h, mix, mx["heads"], mx["dim"], mx["vdim"], float(mx["tau"]), eps)
            elif q == 1:
                if "kv_from" in mx and mx["kv_from"] is not None:
                    keys, values = kept[int(mx["kv_from"])]
                else:
                    keys, values = attention_keys_values(h, mix, mx["kv_heads"], mx["dim"], mx["vdim"], eps)
                    kept[i] = (keys, values)
                y = attention_mixer(h, mix, keys, values, mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"],
                                    float(mx["scale"]), float(mx["q_temp"]["coef"]), int(mx["q_temp"]["every"]), eps)
            else:
                mlp = layer["mlp"]
                if mlp["kind"] == "dense":
                    y = dense_ff(h, W[p + "mlp.up"], W[p + "mlp.down"])
                else:
                    E = int(mlp["router"]["experts"])
                    y, idx, margin = routed_ff(h, W[p + "mlp.router"], W[p + "mlp.router.b"],
                                               [W[f"{p}mlp.e{e}.up"] for e in range(E)],
                                               [W[f"{p}mlp.e{e}.down"] for e in range(E)], int(mlp["router"]["top"]))
                    routing.append((idx, margin))
            streams = connect(streams, y, w_in, w_mix, w_out, m)
        after.append(streams.sum(0))
    x = streams.sum(0)
    logits = (rms_norm(x, W["final.norm"], eps) @ W["embed"].T) * float(cfg.get("logit_scale", 1.0))
    out = [logits]
    if want_layers:
        out.append(torch.stack(after))
    if want_routing:
        out.append(routing)
    return out[0] if len(out) == 1 else tuple(out)
