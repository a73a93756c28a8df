"""The Tirizen decoder in the engine against the plain implementation (tests/plain/tirizen_plain.py).

Small configurations of the tests' own, weights drawn at a scale where every mechanism matters, and inputs
made so that a fault shows where random numbers would hide it (one key that outweighs hundreds, a query
temperature that jumps inside a portion, a state that must survive a portion of one token).
"""

import json
import math
import random

import pytest
import torch

from tests import helpers as H
from tests.plain import tirizen_plain as P

pytestmark = pytest.mark.gpu


def _attn(heads, kv_heads, dim, vdim, scale=None, temp=(0.35, 7), kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 1.0 / math.sqrt(dim)}
    if temp is not None:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _gla(heads, dim, vdim, tau=4.0, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _config(vocab, width, layers, streams, mult=1.0, scale=1.0, logit_scale=1.0, eps=1e-5, max_positions=256):
    cfg = {"architecture": "Tirizen", "vocab": vocab, "width": width, "layers": layers, "residual_mult": mult,
           "embedding": {"scale": scale}, "logit_scale": logit_scale, "norm": {"eps": eps}, "max_positions": max_positions}
    if streams:
        cfg["streams"] = streams
    return cfg


# Sizes that are no powers of two and differ from one another; they cover: one, two and four residual streams and
# none (the plain residual); value sizes unlike key sizes, in both mixers, and head sizes that are no multiple of
# 8 or 16 (the element-by-element paths); one kv head for all query heads, and as many as query heads; layers that
# read an earlier layer's keys and values (twice the same source); a query temperature that jumps every 3, 7 and 40
# positions and a layer without one; experts with top 1, top 2 and every expert chosen; layers without a
# feed-forward; widths that are no multiple of 8.
CONFIGS = {
    "A": (_config(97, 64, [_gla(2, 24, 16, mlp=_moe(6, 2, 24)), _attn(4, 2, 16, 24, mlp=_dense(40)),
                           _attn(4, 2, 16, 24, kv_from=1, temp=(0.5, 3), mlp=_moe(6, 2, 24)), _gla(3, 8, 8, tau=16.0)],
                  streams=3, mult=0.6, scale=4.0, logit_scale=0.5), 6),
    "B": (_config(130, 96, [_attn(6, 1, 16, 16, temp=None, mlp=_moe(5, 1, 32)), _gla(1, 40, 72, tau=1.0, mlp=_dense(56)),
                            _attn(2, 2, 32, 8, temp=(1.0, 40))], streams=0, mult=1.0, scale=1.0, logit_scale=2.0, eps=1e-6), 3),
    "C": (_config(61, 44, [_attn(3, 3, 12, 20, mlp=_moe(3, 3, 16)), _gla(2, 20, 12, tau=8.0, mlp=_moe(9, 4, 8)),
                           _attn(3, 3, 12, 20, kv_from=0, temp=(0.2, 7)), _attn(3, 3, 12, 20, kv_from=0, mlp=_dense(24))],
                  streams=1, mult=1.3, scale=2.0), 5),
    "D": (_config(77, 80, [_gla(2, 136, 40, tau=32.0), _attn(5, 5, 24, 24, mlp=_moe(12, 2, 40)), _gla(2, 16, 136, mlp=_dense(64))],
                  streams=4, mult=0.5, scale=8.0, logit_scale=0.25, eps=1e-4), 9),
    # shapes that the tensor-core kernels take in bfloat16: heads of 64 and 128 (keys and values alike), expert sizes
    # that are multiples of 8, with the shared keys and values read by a second layer
    "E": (_config(111, 128, [_attn(4, 2, 64, 64, mlp=_moe(8, 2, 32)), _gla(2, 32, 32, tau=12.0, mlp=_moe(8, 2, 64)),
                             _attn(4, 2, 64, 64, kv_from=0, mlp=_dense(96)), _attn(2, 1, 128, 128, temp=(0.2, 16), mlp=_moe(4, 2, 16))],
                  streams=2, mult=0.8, scale=3.0), 4),
    # no routed layer: in bfloat16 every position of every request is compared (no choice that rounding could turn)
    "F": (_config(83, 64, [_attn(4, 2, 32, 32, mlp=_dense(48)), _gla(2, 16, 24, tau=8.0, mlp=_dense(40)),
                           _attn(4, 2, 32, 32, kv_from=0, temp=(0.4, 16)), _attn(2, 2, 8, 12, temp=(0.25, 5), mlp=_dense(32))],
                  streams=3, mult=0.9, scale=4.0, logit_scale=0.75), 6),
}


def _folder(tmp_path_factory, name, cfg=None, seed=None):
    from quanta_b200.weights.safetensors_io import write_safetensors
    base, rank = CONFIGS[name]
    cfg = cfg or base
    d = tmp_path_factory.mktemp(f"tirizen_{name}")
    weights = P.draw_weights(cfg, seed=(200 + ord(name[0])) if seed is None else seed, decay_rank=rank)
    write_safetensors(d / "model.safetensors", weights)
    (d / "config.json").write_text(json.dumps(cfg))
    return d, weights, cfg


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {name: _folder(tmp_path_factory, name) for name in CONFIGS}


def _engine(folder, dtype, steps=None, page_size=16, slots=4, num_pages=None):
    from quanta_b200.engine.model import load_model
    from quanta_b200.engine.step import Engine
    model, _ = load_model(folder, dtype=dtype)
    if num_pages is None:
        num_pages = H.tokens_in_flight(steps, page_size) // page_size
    return Engine(model, num_pages=num_pages, page_size=page_size, max_requests=slots)


def _want(weights, cfg, reqs):
    """Logits of every position and, per position, the smallest routing margin of any layer at this position or
    an earlier one of the request (a choice that rounding turns changes that token's keys and values in the
    layers above, and with them every later position)."""
    out, margin = {}, {}
    for rid, toks in reqs.items():
        lg, routing = P.forward(weights, cfg, toks, want_routing=True)
        m = torch.stack([mg for _, mg in routing]).min(0).values if routing else torch.full((len(toks),), 1e9)
        m = torch.cummin(m, 0).values
        for i in range(len(toks)):
            out[(rid, i)] = lg[i]
            margin[(rid, i)] = float(m[i])
    return out, margin


def _replay_following_the_routing(eng, steps, weights, cfg, reqs):
    """Replay ``steps`` while the routed layers report what every token chose; then the plain implementation's
    logits with those choices forced.  In bfloat16 a close choice may turn, and the token's keys and values in the
    layers above, and with them every later position, then differ for a reason that is no fault; following the
    engine's choices compares everything else (the weights of the chosen experts included) at every position.
    Steps run kernel by kernel while the layers report."""
    routed = [eng.model.blocks[e.layer].feed_forward for e in eng.model.schedule
              if hasattr(eng.model.blocks[e.layer].feed_forward, "trace")]
    for part in routed:
        part.trace = []
    eng.use_graphs = False
    from quanta_b200.engine.step import StepEntry
    got, chosen, pos = {}, {rid: [[None] * len(t) for _ in routed] for rid, t in reqs.items()}, {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], tuple(e["want"])) for e in s["entries"]]
        logits = eng.step(entries, end=s["end"])
        eng.check()
        logits = logits.float().cpu() if logits is not None else None
        picks = [part.trace.pop(0).cpu() for part in routed]
        row = lrow = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = logits[lrow]
                lrow += 1
            for i in range(len(e["tokens"])):
                for l in range(len(routed)):
                    chosen[e["id"]][l][base + i] = picks[l][row].tolist()
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    want = {}
    for rid, toks in reqs.items():
        lg = P.forward(weights, cfg, toks, chosen=[torch.tensor(c) for c in chosen[rid]])
        for i in range(len(toks)):
            want[(rid, i)] = lg[i]
    return got, want


def _errors(got, want):
    err = {}
    for key, row in got.items():
        ref = want[key]
        d = row - ref
        e = float((d - d.mean()).pow(2).mean().sqrt() / ref.std())
        err[key] = e if e == e else math.inf
    return err


def _worst(got, want, margins=None, near_tie=0.0):
    """Largest difference of a row's logits (mean taken off) over the row's spread, and where; positions whose
    router margin is below ``near_tie`` (a choice that rounding may turn) are left out."""
    err = _errors(got, want)
    keys = [k for k in err if margins is None or margins[k] >= near_tie]
    assert len(keys) >= 0.25 * len(err), "too many positions after a close routing choice: the test would show nothing"
    where = max(keys, key=lambda k: err[k])
    return err[where], where


TOL = {"float32": 2e-4, "bfloat16": 0.12}
NEAR_TIE = {"float32": 1e-4}


def _requests(vocab, lengths, seed):
    return {f"r{i}": H.random_tokens(n, vocab, seed + i) for i, n in enumerate(lengths)}


# ---- whole models under every cutting ----------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_cuttings_agree_with_plain(models, name, dtype):
    folder, weights, cfg = models[name]
    reqs = _requests(cfg["vocab"], [1, 2, 37, 70, 5, 130], seed=11)
    want, margins = _want(weights, cfg, reqs)
    cuttings = {
        "whole": H.cut_whole(reqs),
        "decode": H.cut_tail_decode(reqs, tail=40),
        "portions": H.cut_portions(reqs, sizes=(7, 2, 13, 3, 1, 2, 29, 4, 16, 2)),
        "mixed": H.cut_mixed(reqs, max_live=3, seed=5, portion_sizes=(2, 3, 5, 8, 17, 33)),
    }
    for cut, steps in cuttings.items():
        # exactly the pages the cutting needs and three state slots: both are given back and used again
        eng = _engine(folder, dtype, steps, page_size=8 if name in "ACEF" else 16, slots=3)
        if dtype == "bfloat16":
            got, following = _replay_following_the_routing(eng, steps, weights, cfg, reqs)
            worst, where = _worst(got, following)
        else:
            got = H.replay(eng, steps)
            worst, where = _worst(got, want, margins, NEAR_TIE[dtype])
        assert len(got) == len(want)
        assert worst < TOL[dtype], f"{name} {dtype} {cut}: {worst} at {where}"
        eng.manager.check_invariants()
        assert eng.manager.stats()["live_requests"] == 0


ORDERS = {
    # no layer keeps keys and values (the cache manager has no page group), none has a state, one layer only,
    # two sources of shared keys and values read in turn, a shared source behind recurrent layers at the very end
    "recurrence_only": [_gla(2, 16, 16, mlp=_dense(32)), _gla(1, 32, 8)],
    "attention_only": [_attn(4, 2, 16, 16, mlp=_moe(4, 2, 16)), _attn(4, 2, 16, 16, kv_from=0)],
    "one_layer": [_gla(2, 16, 24, mlp=_moe(3, 1, 8))],
    "two_sources": [_attn(2, 1, 16, 16), _attn(4, 4, 8, 8), _attn(2, 1, 16, 16, kv_from=0), _attn(4, 4, 8, 8, kv_from=1),
                    _attn(2, 1, 16, 16, kv_from=0)],
    "shared_at_the_end": [_attn(2, 1, 32, 32), _gla(2, 8, 8), _gla(2, 8, 8, mlp=_dense(16)), _attn(2, 1, 32, 32, kv_from=0),
                          _attn(2, 1, 32, 32, kv_from=0, mlp=_dense(8))],
}


@pytest.mark.parametrize("order", list(ORDERS))
def test_other_orders_of_layers(tmp_path_factory, order):
    cfg = _config(67, 40, ORDERS[order], streams=2 if order != "one_layer" else 0, mult=0.8, scale=2.0)
    folder, weights, cfg = _folder(tmp_path_factory, "A", cfg=cfg, seed=3)
    reqs = _requests(cfg["vocab"], [1, 40, 90], seed=1)
    want, margins = _want(weights, cfg, reqs)
    steps = H.cut_mixed(reqs, max_live=3, seed=5, portion_sizes=(2, 3, 5, 8, 17))
    for dtype in ("float32", "bfloat16"):
        eng = _engine(folder, dtype, steps, slots=3)
        if dtype == "bfloat16":
            got, following = _replay_following_the_routing(eng, steps, weights, cfg, reqs)
            worst, where = _worst(got, following)
        else:
            got = H.replay(eng, steps)
            worst, where = _worst(got, want, margins, NEAR_TIE[dtype])
        assert worst < TOL[dtype], (order, dtype, worst, where)
        eng.manager.check_invariants()


def test_residual_stream_after_every_layer(models):
    """The sum of the streams after each layer (the model's own trace) against the plain implementation's."""
    from quanta_b200.engine.step import StepEntry
    folder, weights, cfg = models["A"]
    toks = H.random_tokens(29, cfg["vocab"], 3)
    _, layers = P.forward(weights, cfg, toks, want_layers=True)
    eng = _engine(folder, "float32", num_pages=8)
    eng.model.residual_trace = []
    eng.step([StepEntry("a", toks, (0,))], end=["a"])
    assert len(eng.model.residual_trace) == len(cfg["layers"])
    for i, got in enumerate(eng.model.residual_trace):
        assert torch.allclose(got.cpu(), layers[i], atol=2e-4 * float(layers[i].abs().max()), rtol=1e-4), i


def test_token_by_token_equals_whole_prompt(models):
    """Every token alone (the recurrence's state crosses a step at every token) against the prompt in one step."""
    folder, weights, cfg = models["A"]
    reqs = _requests(cfg["vocab"], [45], seed=3)
    one = H.cut_tail_decode(reqs, tail=1000)
    whole = H.cut_whole(reqs)
    a = H.replay(_engine(folder, "float32", one, page_size=4), one)
    b = H.replay(_engine(folder, "float32", whole, page_size=4), whole)
    worst, where = _worst(a, b)
    assert worst < 2e-5, (worst, where)


def test_batch_does_not_change_a_request(models):
    """Unequal requests in one batch against each alone, float32: the same numbers to rounding."""
    folder, weights, cfg = models["D"]
    reqs = _requests(cfg["vocab"], [33, 3, 90, 64], seed=21)
    together = [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()], "end": list(reqs)}]
    alone = H.cut_whole(reqs)
    a = H.replay(_engine(folder, "float32", together), together)
    b = H.replay(_engine(folder, "float32", alone), alone)
    worst, where = _worst(a, b)
    assert worst < 2e-5, (worst, where)


def test_long_decoding_through_captured_steps(models):
    """A short prompt and 150 single tokens (captured decode steps once the shape has been seen), for two requests
    side by side whose contexts cross pages, key tiles and steps of the query temperature at different steps."""
    folder, weights, cfg = models["F"]
    reqs = _requests(cfg["vocab"], [157, 171], seed=4)
    steps = [{"entries": [{"id": "r0", "tokens": reqs["r0"][:7], "want": [6]}, {"id": "r1", "tokens": reqs["r1"][:21], "want": [20]}],
              "end": []}]
    for i in range(150):
        steps.append({"entries": [{"id": "r0", "tokens": [reqs["r0"][7 + i]], "want": [0]},
                                  {"id": "r1", "tokens": [reqs["r1"][21 + i]], "want": [0]}], "end": []})
    want, margins = _want(weights, cfg, reqs)
    for dtype in ("float32", "bfloat16"):
        eng = _engine(folder, dtype, num_pages=64, page_size=8)
        got = H.replay(eng, steps)
        assert eng.stats()["graph_replays"] > 100
        worst, where = _worst(got, {k: want[k] for k in got})
        assert worst < TOL[dtype], (dtype, worst, where)


def test_slots_and_pages_are_used_again(models):
    """One slot and the pages of one request: five requests one after the other, each starting from a zero state
    although the slot and the pages still hold the last request's numbers."""
    folder, weights, cfg = models["A"]
    reqs = _requests(cfg["vocab"], [30, 30, 29, 31, 30], seed=9)
    steps = H.cut_portions(reqs, sizes=(9, 1, 20, 1))
    eng = _engine(folder, "float32", num_pages=8, page_size=4, slots=1)
    got = H.replay(eng, steps)
    want, margins = _want(weights, cfg, reqs)
    worst, where = _worst(got, want, margins, NEAR_TIE["float32"])
    assert worst < TOL["float32"], (worst, where)


def test_query_temperature_and_learned_positions_count(tmp_path_factory):
    """A temperature that jumps every 3 positions with a large coefficient, and positions as large as the tokens:
    portions that start and end on, before and after a jump agree with the plain implementation, and a model
    whose temperature is left out, or whose position table is shifted by one row, is far off."""
    cfg = _config(50, 48, [_attn(2, 1, 24, 24, temp=(2.0, 3), mlp=_dense(32)), _attn(2, 1, 24, 24, temp=(1.5, 4), kv_from=0)],
                  streams=2, scale=1.0, max_positions=64)
    folder, weights, cfg = _folder(tmp_path_factory, "A", cfg=cfg, seed=77)
    reqs = _requests(cfg["vocab"], [41], seed=2)
    steps = H.cut_portions(reqs, sizes=(2, 3, 1, 2, 4, 6, 1, 1, 1, 5, 3, 12))
    got = H.replay(_engine(folder, "float32", steps, page_size=4), steps)
    want, _ = _want(weights, cfg, reqs)
    worst, where = _worst(got, want)
    assert worst < TOL["float32"], (worst, where)
    no_temp = json.loads(json.dumps(cfg))
    for layer in no_temp["layers"]:
        layer["mixer"]["q_temp"]["coef"] = 0.0
    far, _ = _worst(got, _want(weights, no_temp, reqs)[0])
    assert far > 100 * TOL["float32"]
    shifted = dict(weights, pos=torch.roll(weights["pos"], 1, 0))
    far, _ = _worst(got, _want(shifted, cfg, reqs)[0])
    assert far > 100 * TOL["float32"]


def test_a_prompt_longer_than_the_position_table_is_refused(models):
    from quanta_b200.engine.step import StepEntry
    folder, weights, cfg = models["B"]
    eng = _engine(folder, "float32", num_pages=40)
    with pytest.raises(ValueError, match="positions"):
        eng.step([StepEntry("a", H.random_tokens(cfg["max_positions"] + 1, cfg["vocab"], 0), (0,))])


def test_greedy_generation_through_the_scheduler(models):
    from quanta_b200 import generate
    from quanta_b200.engine.generate import LLM
    folder, weights, cfg = models["A"]
    prompts = [H.random_tokens(n, cfg["vocab"], 40 + n) for n in (9, 23, 4)]
    llm = LLM(str(folder), dtype="float32", page_size=4, num_pages=40, max_requests=2, max_step_tokens=16, prefill_chunk=6)
    got = generate(llm, prompts, max_new_tokens=12, eos_id=[])
    for p, g in zip(prompts, got):
        assert g == P.greedy(weights, cfg, p, 12)
    assert llm.last_stats["cache"]["live_requests"] == 0


def test_command_line_and_random_weights(tmp_path):
    """``python -m quanta_b200 random-weights`` writes a folder for this architecture and ``generate`` runs it."""
    import subprocess
    import sys
    cfg, _ = CONFIGS["C"]
    (tmp_path / "c.json").write_text(json.dumps(cfg))
    out = tmp_path / "model"
    root = str(H.__file__).rsplit("/tests/", 1)[0]
    subprocess.run([sys.executable, "-m", "quanta_b200", "random-weights", "--config", str(tmp_path / "c.json"), "--seed", "3",
                    "--out", str(out)], check=True, cwd=root)
    r = subprocess.run([sys.executable, "-m", "quanta_b200", "generate", "--model", str(out), "--prompt-ids", "1,2,3,4,5",
                        "--max-new-tokens", "5", "--dtype", "float32", "--eos-id", "60"], check=True, capture_output=True,
                       text=True, cwd=root)
    ids = [int(x) for x in r.stdout.strip().split(",")]
    from safetensors.torch import load_file
    weights = load_file(str(out / "model.safetensors"))
    want = P.greedy(weights, json.loads((out / "config.json").read_text()), [1, 2, 3, 4, 5], 5)
    if 60 in want:
        want = want[: want.index(60)]
    assert ids == want


# ---- mechanisms alone ----------------------------------------------------------------------------------
def _ctx_arrays(lengths, slots, dev):
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)  # noqa: E731
    return i32(starts), i32(slots)


@pytest.mark.parametrize("dim,vdim,heads,rank", [(8, 8, 3, 4), (24, 16, 2, 7), (32, 32, 5, 12), (20, 72, 2, 5), (64, 40, 1, 16),
                                                 (136, 24, 2, 3), (16, 136, 1, 8), (128, 128, 2, 32)])
def test_gated_linear_recurrence_alone(dim, vdim, heads, rank):
    """The recurrence kernels against the plain loop: three requests of unequal length in two calls (the state
    crosses the call; one request brings a single token), decays from near 0.5 to near 1, key and value sizes
    that differ, stale numbers in the slots of no request."""
    from quanta_b200 import kernels
    dev = "cuda:0"
    g = torch.Generator().manual_seed(dim + vdim)
    HD, HE = heads * dim, heads * vdim
    lengths = [[19, 1, 40], [1, 30, 3]]
    total = [sum(x) for x in zip(*lengths)]
    n_all = sum(total)
    width = 2 * HD + HE + rank + 3
    proj = torch.randn(n_all, width, generator=g)             # q, k, v, the decay's inner values, columns not read
    w2 = torch.randn(HD, rank, generator=g)
    bias = 2.0 + 1.5 * torch.randn(HD, generator=g)
    tau, q_scale = 4.0, dim ** -0.5
    state = torch.full((4, heads, dim, vdim), 5.0, device=dev)
    slots = [2, 0, 3]
    for s in slots:
        state[s].zero_()
    rows_of, at = [], 0
    for r in range(3):
        rows_of.append(list(range(at, at + total[r])))
        at += total[r]
    got = torch.zeros(n_all, heads, vdim)
    done = [0, 0, 0]
    for call in lengths:
        idx = [i for r in range(3) for i in rows_of[r][done[r]: done[r] + call[r]]]
        starts, sl = _ctx_arrays(call, slots, dev)
        out = torch.empty(len(idx), heads, vdim, device=dev)
        kernels.gla(proj[idx].to(dev).contiguous(), (0, HD, 2 * HD), 2 * HD + HE, rank, w2.to(dev), bias.to(dev), state, out,
                    starts, sl, heads, dim, vdim, tau, q_scale)
        got[idx] = out.cpu()
        for r in range(3):
            done[r] += call[r]
    for r in range(3):
        rows = rows_of[r]
        q = proj[rows, :HD].view(-1, heads, dim) * q_scale
        k = proj[rows, HD: 2 * HD].view(-1, heads, dim)
        v = proj[rows, 2 * HD: 2 * HD + HE].view(-1, heads, vdim)
        z = proj[rows, 2 * HD + HE: 2 * HD + HE + rank] @ w2.T + bias
        alpha = torch.sigmoid(z.double()).pow(1.0 / tau).float().view(-1, heads, dim)
        want, S = P.gated_linear_recurrence(q, k, v, alpha)
        assert torch.allclose(got[rows], want, atol=2e-5 * float(want.abs().max()), rtol=1e-4), (r, dim, vdim)
        assert torch.allclose(state[slots[r]].cpu(), S, atol=2e-5 * float(S.abs().max()), rtol=1e-4)
    assert float(state[1].min()) == 5.0


@pytest.mark.parametrize("dim,vdim,heads", [(64, 64, 3), (24, 40, 2), (136, 16, 1)])
def test_long_portions_run_as_segments(dim, vdim, heads):
    """A step with long portions cuts every request into segments that run side by side (each from a zero state,
    then joined in order, then once more from their true start states): the same numbers, to rounding, as the one
    chain in time and as the plain loop; requests of 700, 1, 65 and 64 tokens in one call (segments that end on,
    before and after a border), states that are not zero when the call begins."""
    from quanta_b200 import kernels
    dev, rank = "cuda:0", 6
    g = torch.Generator().manual_seed(dim)
    HD, HE = heads * dim, heads * vdim
    lengths = [[5, 1, 3, 2], [700, 1, 65, 64]]
    total = [sum(x) for x in zip(*lengths)]
    n_all = sum(total)
    proj = torch.randn(n_all, 2 * HD + HE + rank, generator=g)
    w2 = torch.randn(HD, rank, generator=g)
    bias = 3.0 + 1.5 * torch.randn(HD, generator=g)
    tau, q_scale = 8.0, dim ** -0.5
    rows_of, at = [], 0
    for r in range(4):
        rows_of.append(list(range(at, at + total[r])))
        at += total[r]
    results = {}
    for segments in (None, False):
        state = torch.full((6, heads, dim, vdim), 5.0, device=dev)
        slots = [2, 0, 5, 3]
        for s in slots:
            state[s].zero_()
        got = torch.zeros(n_all, heads, vdim)
        done = [0] * 4
        for call in lengths:
            idx = [i for r in range(4) for i in rows_of[r][done[r]: done[r] + call[r]]]
            starts, sl = _ctx_arrays(call, slots, dev)
            out = torch.empty(len(idx), heads, vdim, device=dev)
            before = kernels.LAUNCHES
            kernels.gla(proj[idx].to(dev).contiguous(), (0, HD, 2 * HD), 2 * HD + HE, rank, w2.to(dev), bias.to(dev), state, out,
                        starts, sl, heads, dim, vdim, tau, q_scale, segments=segments)
            assert kernels.LAUNCHES - before == (5 if segments is None and len(idx) >= 512 else 2)
            got[idx] = out.cpu()
            for r in range(4):
                done[r] += call[r]
        results[segments] = (got, state.cpu())
        assert float(state[1].min()) == 5.0 and float(state[4].min()) == 5.0
    (a, sa), (b, sb) = results[None], results[False]
    assert torch.allclose(a, b, atol=2e-5 * float(b.abs().max()), rtol=1e-4)
    assert torch.allclose(sa, sb, atol=2e-5 * float(sb.abs().max()), rtol=1e-4)
    for r in range(4):
        rows = rows_of[r]
        q = proj[rows, :HD].view(-1, heads, dim) * q_scale
        k = proj[rows, HD: 2 * HD].view(-1, heads, dim)
        v = proj[rows, 2 * HD: 2 * HD + HE].view(-1, heads, vdim)
        z = proj[rows, 2 * HD + HE: 2 * HD + HE + rank] @ w2.T + bias
        alpha = torch.sigmoid(z.double()).pow(1.0 / tau).float().view(-1, heads, dim)
        want, _ = P.gated_linear_recurrence(q, k, v, alpha)
        assert torch.allclose(a[rows], want, atol=3e-5 * float(want.abs().max()), rtol=1e-4), r


def test_a_far_token_stays_in_the_recurrent_state():
    """With decays at 1 - 2e-4 a token 600 steps back still weighs 0.89: its value comes out when the query meets
    its key, through a state that crossed 40 calls of unequal size."""
    from quanta_b200 import kernels
    dev, heads, dim, vdim, rank = "cuda:0", 1, 16, 8, 2
    n = 601
    proj = torch.zeros(n, 2 * dim + vdim + rank)
    proj[0, dim: 2 * dim] = torch.eye(dim)[3]               # the first token's key: channel 3
    proj[0, 2 * dim: 2 * dim + vdim] = torch.arange(1, vdim + 1).float()
    proj[-1, :dim] = torch.eye(dim)[3]                      # the last token's query asks for it
    bias = torch.full((dim,), math.log(0.9968 / (1 - 0.9968)))          # sigmoid = 0.9968, tau 16: alpha = 0.9998
    state = torch.zeros(1, heads, dim, vdim, device=dev)
    outs, at, rng = [], 0, random.Random(0)
    while at < n:
        m = min(rng.choice([1, 1, 2, 7, 40]), n - at)
        starts, sl = _ctx_arrays([m], [0], dev)
        out = torch.empty(m, heads, vdim, device=dev)
        kernels.gla(proj[at: at + m].to(dev).contiguous(), (0, dim, 2 * dim), 2 * dim + vdim, rank, torch.zeros(dim, rank, device=dev),
                    bias.to(dev), state, out, starts, sl, heads, dim, vdim, 16.0, 1.0)
        outs.append(out.cpu())
        at += m
    got = torch.cat(outs)[-1, 0]
    alpha = 0.9968 ** (1 / 16)
    want = torch.arange(1, vdim + 1).float() * alpha ** 600
    assert 0.85 < alpha ** 600 < 0.93
    assert torch.allclose(got, want, rtol=2e-3)


@pytest.mark.parametrize("S,width,K", [(1, 48, 1), (3, 256, 2), (4, 1000, 1), (16, 64, 3)])
def test_streams_between_two_sublayers_in_one_launch(S, width, K):
    """Write-back of a sublayer's output through the mixing matrix, the read of the next sublayer and its norm:
    against plain arithmetic, for all rows and for chosen rows that leave the streams as they are."""
    from quanta_b200 import kernels
    dev = "cuda:0"
    g = torch.Generator().manual_seed(S * width)
    T = 9
    x = torch.randn(T, S, width, generator=g) * 3
    y = torch.randn(T, K, width, generator=g)
    mix, out_w, read_w = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    w = 1 + 0.3 * torch.randn(width, generator=g)
    mult = 0.7
    new = P.connect(x.permute(1, 0, 2), y.sum(1), None, mix, out_w, mult).permute(1, 0, 2)
    u = torch.einsum("s,tsi->ti", read_w, new)
    want = P.rms_norm(u, w, 1e-5)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        xd, out = x.to(dev), torch.empty(T, width, dtype=dtype, device=dev)
        kernels.streams_mix_rmsnorm(xd, y.to(dev), mix.to(dev), out_w.to(dev), mult, read_w.to(dev), w.to(dev), 1e-5, out)
        assert torch.allclose(xd.cpu(), new, atol=1e-5, rtol=1e-5)
        assert torch.allclose(out.float().cpu(), want, atol=tol * float(want.abs().max()), rtol=tol)
    rows = torch.tensor([7, 2], dtype=torch.int32, device=dev)
    xd, out = x.to(dev), torch.empty(2, width, device=dev)
    kernels.streams_mix_rmsnorm(xd, y.to(dev), mix.to(dev), out_w.to(dev), mult, None, w.to(dev), 1e-5, out, rows=rows, store=False)
    assert torch.equal(xd.cpu(), x)
    assert torch.allclose(out.cpu(), P.rms_norm(new.sum(1), w, 1e-5)[[7, 2]], atol=1e-5, rtol=1e-5)
    # no pending output: the read and the norm alone
    out = torch.empty(T, width, device=dev)
    kernels.streams_mix_rmsnorm(x.to(dev), None, None, None, 0.0, read_w.to(dev), w.to(dev), 1e-5, out)
    assert torch.allclose(out.cpu(), P.rms_norm(torch.einsum("s,tsi->ti", read_w, x), w, 1e-5), atol=1e-5, rtol=1e-5)


def test_embedding_with_learned_positions_and_copies():
    from quanta_b200 import kernels
    dev = "cuda:0"
    g = torch.Generator().manual_seed(0)
    for width in (40, 45):
        table, pos = torch.randn(30, width, generator=g), torch.randn(12, width, generator=g)
        ids = torch.tensor([3, 29, 0, 7], dtype=torch.int32, device=dev)
        at = torch.tensor([0, 11, 5, 6], dtype=torch.int32, device=dev)
        status = kernels.new_status(dev)
        for dtype in (torch.float32, torch.bfloat16):
            tb, pb = table.to(dev, dtype), pos.to(dev, dtype)
            h = torch.empty(4, 3, width, device=dev)
            kernels.embedding(h, tb, ids, status, 2.5, pb, at)
            want = tb.float()[ids.long()] * 2.5 + pb.float()[at.long()]
            for c in range(3):
                assert torch.allclose(h[:, c], want, atol=1e-6, rtol=1e-6)
        assert int(status.cpu()[0]) == 0
        h = torch.empty(1, width, device=dev)
        kernels.embedding(h, table.to(dev), ids[:1], status, 1.0, pos.to(dev), torch.tensor([12], dtype=torch.int32, device=dev))
        assert int(status.cpu()[0]) == 7          # a position past the table is refused, not read


def _paged(rows_per_req, heads, page_size, width, dtype, dev, ids):
    """Pages ``[n, heads, page_size, width]`` in the order ``ids`` holding each request's rows ``[n, heads, width]``."""
    need = [-(-r.shape[0] // page_size) for r in rows_per_req]
    pages = torch.zeros(len(ids), heads, page_size, width, dtype=dtype, device=dev)
    table = torch.full((len(rows_per_req), max(need)), -1, dtype=torch.int32)
    at = 0
    for r, rows in enumerate(rows_per_req):
        for p in range(need[r]):
            pid = ids[at]
            at += 1
            table[r, p] = pid
            chunk = rows[p * page_size: (p + 1) * page_size]
            pages[pid, :, : chunk.shape[0]] = chunk.permute(1, 0, 2).to(dev, dtype)
    return pages, table.to(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,vd", [(24, 40), (64, 64), (20, 12), (128, 16)])
def test_attention_finds_one_key_among_many(dtype, hd, vd):
    """Queries at positions just before, at and after page borders, each with ONE key (the first, one at a border,
    one far back, its own) made to outweigh some 700 others; single tokens of a long request and a portion of
    another in the same call; values of another size than the keys.  Against a plain softmax."""
    from quanta_b200 import kernels
    dev, nq, nkv, ps = "cuda:0", 6, 2, 16
    g = torch.Generator().manual_seed(hd)
    n0, n1 = 700, 130
    keys = [0.3 * torch.randn(n, nkv, hd, generator=g) for n in (n0, n1)]
    vals = [torch.randn(n, nkv, vd, generator=g) for n in (n0, n1)]
    queries = [(0, p, k) for p, k in ((699, 0), (698, 15), (697, 16), (696, 17), (695, 31), (694, 32), (693, 640), (692, 692),
                                      (31, 0), (32, 31), (33, 32), (0, 0), (15, 1), (16, 16), (17, 3))]
    queries += [(1, p, (p * 7) % (p + 1)) for p in range(97, 130)]
    for r, k in {(r, k) for r, _, k in queries}:
        keys[r][k] *= 2.5                   # a made key is longer than the others, so that none of them can outdo it
    if dtype == torch.bfloat16:
        keys, vals = [k.to(dtype).float() for k in keys], [v.to(dtype).float() for v in vals]
    T = len(queries)
    q = 0.3 * torch.randn(T, nq, hd, generator=g)
    for t, (r, p, k) in enumerate(queries):
        for h in range(nq):
            key = keys[r][k, h // 3]
            q[t, h] += (12.0 + h) * key / key.norm() ** 2
    if dtype == torch.bfloat16:
        q = q.to(dtype).float()
    ids = list(range(60))
    random.Random(hd).shuffle(ids)
    k_pages, table = _paged(keys, nkv, ps, hd, dtype, dev, ids)
    v_pages, _ = _paged(vals, nkv, ps, vd, dtype, dev, ids)
    tok_pos = torch.tensor([p for _, p, _ in queries], dtype=torch.int32, device=dev)
    tok_req = torch.tensor([r for r, _, _ in queries], dtype=torch.int32, device=dev)
    out = torch.empty(T, nq, vd, dtype=dtype, device=dev)
    status = kernels.new_status(dev)
    kernels.paged_attention_simt(q.to(dev, dtype), k_pages, v_pages, out, tok_pos, tok_req, table, 0.9, 0, status)
    assert int(status.cpu()[0]) == 0
    out = out.float().cpu()
    for t, (r, p, k) in enumerate(queries):
        for h in range(nq):
            s = (keys[r][: p + 1, h // 3] @ q[t, h]) * 0.9
            prob = torch.softmax(s, -1)
            assert int(prob.argmax()) == k
            want = prob @ vals[r][: p + 1, h // 3]
            tol = 1e-5 if dtype == torch.float32 else 1e-2
            assert torch.allclose(out[t, h], want, atol=tol, rtol=tol), (t, h, r, p, k)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,vd,own_kv,pad", [(4, 2, 16, 24, True, 4), (3, 3, 12, 20, True, 1), (6, 1, 16, 16, False, 2),
                                                    (2, 1, 64, 64, True, 0)])
def test_queries_keys_and_values_of_a_step(dtype, nq, nkv, hd, vd, own_kv, pad):
    """Rows of a fused projection (queries, keys, values of another head size, then columns that are something
    else): norm over the whole query / key projection, the query temperature at positions on both sides of its
    jumps, and keys and values into pages of their own sizes; also for a layer that brings no keys or values."""
    from quanta_b200 import kernels
    dev, ps, eps, coef, every = "cuda:0", 4, 1e-5, 0.8, 3
    g = torch.Generator().manual_seed(nq * hd)
    T = 13
    qn, kn, vn = nq * hd, (nkv * hd if own_kv else 0), (nkv * vd if own_kv else 0)
    rows = torch.randn(T, qn + kn + vn + pad, generator=g).to(dtype)
    wq, wk = 1 + 0.3 * torch.randn(qn, generator=g), 1 + 0.3 * torch.randn(nkv * hd, generator=g)
    pos = torch.arange(0, T, dtype=torch.int32) + 1            # positions 1..13: jumps at 2, 5, 8, 11
    table = torch.tensor([[3, 0, 2, 1]], dtype=torch.int32, device=dev)
    k_pages = torch.zeros(4, nkv, ps, hd, dtype=dtype, device=dev) if own_kv else None
    v_pages = torch.zeros(4, nkv, ps, vd, dtype=dtype, device=dev) if own_kv else None
    q_out = torch.empty(T, nq, hd, dtype=dtype, device=dev)
    status = kernels.new_status(dev)
    kernels.qknorm_rope_write(rows.to(dev), q_out, k_pages, v_pages, wq.to(dev), wk.to(dev) if own_kv else None,
                              kernels.NORM_PER_LAYER, eps, torch.empty(0, device=dev), None, pos.to(dev).view(T, 1), pos.to(dev),
                              torch.zeros(T, dtype=torch.int32, device=dev), table, nq, nkv, hd, 0, ps, status,
                              vd=vd, has_kv=own_kv, q_temp_coef=coef, q_temp_every=every)
    assert int(status.cpu()[0]) == 0
    r = rows.float()
    temp = 1.0 + coef * torch.log(torch.floor((pos.float() + 1) / every) + 1.0)
    want_q = P.rms_norm(r[:, :qn], wq, eps) * temp[:, None]
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(q_out.float().cpu().view(T, qn), want_q, atol=tol, rtol=tol)
    assert len(set(temp.tolist())) == 5
    if own_kv:
        want_k = P.rms_norm(r[:, qn: qn + kn], wk, eps).view(T, nkv, hd)
        want_v = r[:, qn + kn: qn + kn + vn].view(T, nkv, vd)
        for t in range(T):
            p = int(pos[t])
            page = int(table[0, p // ps])
            assert torch.allclose(k_pages[page, :, p % ps].float().cpu(), want_k[t], atol=tol, rtol=tol)
            assert torch.equal(v_pages[page, :, p % ps].float().cpu(), want_v[t])


@pytest.mark.parametrize("T", [5, 130])
@pytest.mark.parametrize("E,k", [(8, 2), (5, 1), (3, 3), (40, 6)])
def test_router_weights_are_the_softmax_over_the_chosen(T, E, k):
    """Choice by logit + bias (the lower index among equals), weights the softmax over the chosen values, on both
    routing kernels (the one launch of small steps and the selection of large ones)."""
    from quanta_b200 import kernels
    dev, K = "cuda:0", 64
    g = torch.Generator().manual_seed(E * k)
    x = torch.randn(T, K, generator=g)
    gate, bias = torch.randn(E, K, generator=g) / 8, torch.randn(E, generator=g)
    gate[1] = gate[0]
    bias[1] = bias[0]                                   # experts 0 and 1 always tie
    z = x @ gate.T + bias
    order = torch.sort(z, dim=-1, descending=True, stable=True)
    want_idx, want_w = order.indices[:, :k], torch.softmax(order.values[:, :k], -1)
    logits = torch.empty(T, E, device=dev)
    kernels.router_small(x.to(dev), gate.to(dev), bias.to(dev), logits)
    idx = torch.empty(T, k, dtype=torch.int32, device=dev)
    w = torch.empty(T, k, device=dev)
    kernels.router_topk(logits, bias.to(dev), idx, w, kernels.ROUTE_SOFTMAX_CHOSEN, 1.0)
    close = (order.values[:, :-1] - order.values[:, 1:]).abs().min(-1).values < 1e-5 if E > 1 else torch.zeros(T, dtype=torch.bool)
    tie01 = ((want_idx == 0).any(-1) | (want_idx == 1).any(-1))
    ok = ~close | tie01                                 # rows whose order rounding cannot turn (the made tie is exact)
    assert torch.equal(idx.cpu().long()[ok & ~close], want_idx[ok & ~close])
    assert torch.allclose(w.cpu()[ok & ~close], want_w[ok & ~close], atol=1e-5)
    both = (want_idx == 0).any(-1) & (want_idx == 1).any(-1)
    for t in torch.nonzero(both).flatten().tolist():
        row = idx[t].cpu().tolist()
        assert row.index(0) < row.index(1)
    if kernels.router_small_selects(T, E, k):
        idx2 = torch.empty(T, k, dtype=torch.int32, device=dev)
        w2 = torch.empty(T, k, device=dev)
        bm = 16
        plan_words, max_tiles = kernels.moe_plan_sizes(T * k, E, bm)
        ints = torch.zeros(plan_words + T * k + 2 * max_tiles, dtype=torch.int32, device=dev)
        counters = torch.zeros(64, dtype=torch.int32, device=dev)
        kernels.router_small(x.to(dev), gate.to(dev), bias.to(dev), logits, idx2, w2, kernels.ROUTE_SOFTMAX_CHOSEN, 1.0,
                             counters=counters, bm=bm, plan=ints[:plan_words], sorted_pair=ints[plan_words: plan_words + T * k],
                             tile_expert=ints[plan_words + T * k: plan_words + T * k + max_tiles],
                             tile_row0=ints[plan_words + T * k + max_tiles:], status=kernels.new_status(dev))
        assert torch.equal(idx2, idx) and torch.equal(w2, w)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,I,E,k", [(3, 64, 32, 6, 2), (70, 48, 24, 5, 1), (300, 128, 200, 4, 4), (1, 40, 12, 3, 3)])
def test_ungated_experts_alone(dtype, T, H, I, E, k):
    """The routed feed-forward part (router, plan, both products on whichever kernels the sizes take) against the
    plain one; the sizes reach the tcgen05 path (widths that are multiples of 8, bfloat16) and the CUDA cores."""
    from quanta_b200 import kernels
    from quanta_b200.parts.base import StepContext, make
    dev = "cuda:0"
    g = torch.Generator().manual_seed(T + H)
    names = {"gate": "r", "bias": "r.b", "up": "e{e}.up", "down": "e{e}.down"}
    part = make("feed_forward", ("softmax_topk_experts", dict(hidden_size=H, expert_size=I, n_experts=E, top_k=k, use_bias=True, names=names)))
    W = {"r": torch.randn(E, H, generator=g) / math.sqrt(H), "r.b": 0.5 * torch.randn(E, generator=g)}
    for e in range(E):
        W[f"e{e}.up"] = (torch.randn(I, H, generator=g) / math.sqrt(H)).to(torch.bfloat16).float()
        W[f"e{e}.down"] = (torch.randn(H, I, generator=g) / math.sqrt(I)).to(torch.bfloat16).float()
    kinds = {s.name: s.kind for s in part.tensor_specs()}
    part.load(lambda n: W[n].to(dev, dtype if kinds[n] == "matrix" else torch.float32))
    x = torch.randn(T, H, generator=g).to(dtype)
    ctx = StepContext(n_tokens=T, positions=None, tok_pos=None, tok_req=None, req_slot=None, req_start=None, req_len_after=None,
                      status=kernels.new_status(dev), dtype=dtype)
    y = part.forward(x.to(dev), ctx).float().sum(1).cpu()
    assert int(ctx.status.cpu()[0]) == 0
    want, _, margin = P.routed_ff(x.float(), W["r"], W["r.b"], [W[f"e{e}.up"] for e in range(E)],
                                  [W[f"e{e}.down"] for e in range(E)], k)
    clear = margin > (1e-4 if dtype == torch.float32 else 0.05)
    assert int(clear.sum()) >= 0.6 * T
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert torch.allclose(y[clear], want[clear], atol=tol * float(want.abs().max()), rtol=tol)
