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


def routed_ff(h, router, router_bias, ups, downs, top: int, chosen=None):
    """Logits ``router h + bias``; the ``top`` largest are chosen (the lower index on a tie); their weights are
    the softmax over the chosen logits only.  Returns (output, chosen experts [T, top], margin between the
    last chosen and the first refused logit [T]).  ``chosen`` [T, top]: take these experts instead of choosing
    (to follow an implementation whose rounding turned a close choice); the weights are still computed here."""
    z = h @ router.T + router_bias
    order = torch.sort(z, dim=-1, descending=True, stable=True)
    idx, val = order.indices[:, :top], order.values[:, :top]
    margin = (order.values[:, top - 1] - order.values[:, top]) if z.shape[1] > top else torch.full_like(z[:, 0], 1e9)
    if chosen is not None:
        idx = torch.as_tensor(chosen, dtype=torch.long, device=z.device)
        val = torch.gather(z, 1, idx)
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


def forward(weights: dict, cfg: dict, tokens, dtype=torch.float32, want_layers: bool = False, want_routing: bool = False,
            chosen=None):
    """Logits [T, vocab] (and the sum of the streams after every layer, [layers, T, width]; and per routed
    layer the (experts, margins)).  ``chosen``: per routed layer, in order, the experts [T, top] to take."""
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
                temp = mx.get("q_temp") or {"coef": 0.0, "every": 1}
                y = attention_mixer(h, mix, keys, values, mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"],
                                    float(mx["scale"]), float(temp["coef"]), int(temp["every"]), eps)
            else:
                mlp = layer["mlp"]
                if mlp["kind"] == "dense":
                    y = dense_ff(h, W[p + "mlp.up"], W[p + "mlp.down"])
                else:
                    E = int(mlp["router"]["experts"])
                    y, idx, margin = routed_ff(h, W[p + "mlp.router"], W[p + "mlp.router.b"],
                                               [W[f"{p}mlp.e{e}.up"] for e in range(E)],
                                               [W[f"{p}mlp.e{e}.down"] for e in range(E)], int(mlp["router"]["top"]),
                                               chosen=None if chosen is None else chosen[len(routing)])
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


def greedy(weights: dict, cfg: dict, prompt, n_new: int) -> list[int]:
    toks, new = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(weights, cfg, toks)[-1].argmax())
        toks.append(nxt)
        new.append(nxt)
    return new


def draw_weights(cfg: dict, seed: int, decay_rank: int = 8, matrix_dtype=torch.bfloat16) -> dict:
    """Random weights for a configuration, at scales where every mechanism matters: projections of unit gain,
    norm gains around 1, decays spread over (0.5, 1), connection weights away from 1 and the identity, router
    biases as large as the logits' spread, learned positions as large as the embedded tokens."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    width, vocab = cfg["width"], cfg["vocab"]

    def mat(name, out, inn, gain=1.0):
        W[name] = (torch.randn(out, inn, generator=g) * gain / math.sqrt(inn)).to(matrix_dtype)

    def vec(name, n, mean=1.0, spread=0.3):
        W[name] = (mean + spread * torch.randn(n, generator=g)).to(matrix_dtype)

    W["embed"] = (torch.randn(vocab, width, generator=g) * 0.5).to(matrix_dtype)
    W["pos"] = (torch.randn(cfg["max_positions"], width, generator=g) * 0.5).to(matrix_dtype)
    vec("final.norm", width)
    S = int(cfg.get("streams", 0))
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        vec(p + "norm1", width)
        if layer["type"] == "gla":
            HD, HE = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            mat(p + "mix.q", HD, width, 2.0); mat(p + "mix.k", HD, width, 2.0); mat(p + "mix.v", HE, width)
            mat(p + "mix.g", HE, width); mat(p + "mix.o", width, HE)
            vec(p + "mix.norm", m["vdim"])
            rank = m.get("decay_rank", decay_rank)
            mat(p + "mix.a1", rank, width); mat(p + "mix.a2", HD, rank, 2.0)
            vec(p + "mix.a2.b", HD, mean=2.0, spread=1.5)
        else:
            Q = m["heads"] * m["dim"]
            mat(p + "mix.q", Q, width); vec(p + "mix.q.norm", Q)
            mat(p + "mix.g", m["heads"], width, 2.0); mat(p + "mix.o", width, m["heads"] * m["vdim"])
            if m.get("kv_from") is None:
                K = m["kv_heads"] * m["dim"]
                mat(p + "mix.k", K, width); mat(p + "mix.v", m["kv_heads"] * m["vdim"], width); vec(p + "mix.k.norm", K)
        mlp = layer.get("mlp")
        if mlp is not None:
            vec(p + "norm2", width)
            if mlp["kind"] == "dense":
                mat(p + "mlp.up", mlp["ff"], width); mat(p + "mlp.down", width, mlp["ff"])
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                mat(p + "mlp.router", E, width); vec(p + "mlp.router.b", E, mean=0.0, spread=0.5)
                for e in range(E):
                    mat(f"{p}mlp.e{e}.up", ff, width); mat(f"{p}mlp.e{e}.down", width, ff)
        if S:
            for q in ("1", "2") if mlp is not None else ("1",):
                vec(f"{p}hc{q}.in", S, mean=0.6, spread=0.3)
                vec(f"{p}hc{q}.out", S, mean=0.8, spread=0.4)
                W[f"{p}hc{q}.mix"] = (0.7 * torch.eye(S) + 0.3 * torch.randn(S, S, generator=g) / math.sqrt(S)).to(matrix_dtype)
    return W
