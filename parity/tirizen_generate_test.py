"""Gate: the Tirizen decoder through the entry point gives the plain implementation's tokens and logits.

A small model (three residual streams; a gated-linear-attention layer with routed experts, an attention layer
with a dense feed-forward, an attention layer on the second layer's keys and values): greedy tokens of three
prompts fed in portions of 6 beside decoded tokens, pages of 4, two state slots that are used again; then the
logits of one prompt through the step function, whole and token by token."""
# parity-gate: gpu

from __future__ import annotations

import json
import tempfile
from pathlib import Path

from parity._gates import Checks

CONFIG = {
    "architecture": "Tirizen", "vocab": 90, "width": 48, "streams": 3, "residual_mult": 0.8, "logit_scale": 0.5,
    "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5}, "max_positions": 96,
    "layers": [
        {"type": "gla", "mixer": {"heads": 2, "dim": 16, "vdim": 24, "tau": 8.0},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 40},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.25, "q_temp": {"coef": 0.4, "every": 5}}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.25, "q_temp": {"coef": 0.2, "every": 9}, "kv_from": 1}},
    ],
}


def run() -> int:
    import torch

    from quanta_b200 import generate
    from quanta_b200.engine.generate import LLM
    from quanta_b200.weights.safetensors_io import write_safetensors
    from tests import helpers as H
    from tests.plain import tirizen_plain as P

    c = Checks("tirizen_generate_test")
    with tempfile.TemporaryDirectory() as d:
        weights = P.draw_weights(CONFIG, seed=5, decay_rank=4)
        write_safetensors(Path(d) / "model.safetensors", weights)
        (Path(d) / "config.json").write_text(json.dumps(CONFIG))
        llm = LLM(d, dtype="float32", page_size=4, num_pages=40, max_requests=2, max_step_tokens=12, prefill_chunk=6)
        prompts = [H.random_tokens(n, CONFIG["vocab"], 40 + i) for i, n in enumerate((5, 11, 16))]
        got = generate(llm, prompts, max_new_tokens=8, eos_id=[])
        for p, g in zip(prompts, got):
            c.ok(g == P.greedy(weights, CONFIG, p, 8), f"greedy tokens of a prompt of {len(p)}")
        c.ok(llm.engine.manager.stats()["live_requests"] == 0, "all slots released")
        reqs = {"a": H.random_tokens(33, CONFIG["vocab"], 7)}
        want = P.forward(weights, CONFIG, reqs["a"])
        for name, steps in (("whole", H.cut_whole(reqs)), ("token by token", H.cut_tail_decode(reqs, tail=1000))):
            rows = H.replay(llm.engine, steps)
            worst = max(float((rows[("a", i)] - want[i]).abs().max()) for i in range(33))
            c.ok(worst < 2e-4 * float(want.abs().max()), f"logits, {name}: {worst}")
        c.ok(torch.isfinite(want).all().item(), "finite logits")
    c.done()
    return 0


if __name__ == "__main__":
    raise SystemExit(run())
