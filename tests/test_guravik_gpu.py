"""The Guravik decoder in the engine against the plain implementation (tests/plain/guravik_plain.py).

Small configurations of the tests' own, weights drawn at a scale where every mechanism matters, and
inputs made so that a fault shows where random numbers would hide it (one key that outweighs hundreds,
a sink that dominates, a state that must survive a portion of one token).
"""

import json
import math
import random

import pytest
import torch

from tests import helpers as H
from tests.plain import guravik_plain as P

pytestmark = pytest.mark.gpu


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, rot_dims=None, base=10000.0, ff=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": 1.0 / math.sqrt(dim + rot_dim), "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _delta(heads, dim, ff=None):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _config(vocab, width, layers, taps, loop, scale=1.0, eps=1e-5):
    return {"architecture": "Guravik", "vocab": vocab, "width": width, "layers": layers, "canon": {"taps": taps},
            "loop": {"start": loop[0], "stop": loop[1], "times": loop[2]}, "embedding": {"scale": scale},
            "norm": {"eps": eps}}


# Sizes that are no powers of two, differ from one another, and cover: one head and nine (more than a block of
# the attention kernel takes), value size unlike key size, fewer rotated dimensions than the rotated part has,
# taps 1 to 4, a loop in the middle, over everything, and none, layers with and without a feed-forward.
CONFIGS = {
    "A": (_config(97, 64, [_delta(2, 24), _latent(3, 16, 8, 24, 20, 40, ff=48), _delta(1, 40, ff=32)], 4, (1, 3, 3), 3.0, 1e-6), 12),
    "B": (_config(130, 96, [_latent(1, 32, 16, 16, 48, 24, rot_dims=8), _latent(5, 8, 4, 12, 16, 72, ff=40), _delta(3, 72)],
                  1, (0, 0, 1), 1.0, 1e-5), 5),
    "C": (_config(61, 48, [_delta(4, 8, ff=24), _latent(9, 8, 8, 8, 24, 16, base=100.0)], 2, (0, 2, 2), 7.5, 1e-4), 16),
    "D": (_config(77, 80, [_latent(2, 24, 16, 40, 32, 136, ff=56), _delta(2, 136)], 3, (1, 2, 2), 2.0, 1e-5), 8),
    # latents that the tensor-core attention kernel takes in bfloat16 (64 and 128 wide, rotated parts of 16 and 32),
    # with 5 heads (a tile of 32 rows holds six tokens and a part of the seventh) and 16 (two tokens a tile)
    "E": (_config(111, 64, [_latent(5, 16, 16, 24, 24, 64, ff=40), _delta(2, 16), _latent(16, 8, 32, 8, 16, 128)], 3, (0, 2, 2),
                  4.0, 1e-5), 4),
}


def _folder(tmp_path_factory, name, sink_mean=0.0):
    from quanta_b200.weights.safetensors_io import write_safetensors
    cfg, rank = CONFIGS[name]
    d = tmp_path_factory.mktemp(f"guravik_{name}")
    weights = P.draw_weights(cfg, seed=100 + ord(name[0]), decay_rank=rank, sink_mean=sink_mean)
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
    out = {}
    for rid, toks in reqs.items():
        lg = P.forward(weights, cfg, toks)
        for i in range(len(toks)):
            out[(rid, i)] = lg[i]
    return out


def _worst(got, want):
    """Largest difference of a row's logits (mean taken off) over the row's spread, and where."""
    worst, where = 0.0, None
    for key, row in got.items():
        ref = want[key]
        d = row - ref
        e = float((d - d.mean()).pow(2).mean().sqrt() / ref.std())
        if not e == e:
            e = math.inf
        if e > worst:
            worst, where = e, key
    return worst, where


TOL = {"float32": 2e-4, "bfloat16": 0.12}


def _requests(vocab, lengths, seed):
    return {f"r{i}": H.random_tokens(n, vocab, seed + i) for i, n in enumerate(lengths)}


# ---- whole models under every cutting ----------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_cuttings_agree_with_plain(models, name, dtype):
    folder, weights, cfg = models[name]
    reqs = _requests(cfg["vocab"], [1, 2, 37, 70, 5, 130], seed=11)
    want = _want(weights, cfg, reqs)
    cuttings = {
        "whole": H.cut_whole(reqs),
        "decode": H.cut_tail_decode(reqs, tail=40),
        "portions": H.cut_portions(reqs, sizes=(7, 2, 13, 3, 1, 2, 29, 4, 16, 2)),
        "mixed": H.cut_mixed(reqs, max_live=3, seed=5, portion_sizes=(2, 3, 5, 8, 17, 33)),
    }
    for cut, steps in cuttings.items():
        # exactly the pages the cutting needs and three state slots: both are given back and used again
        eng = _engine(folder, dtype, steps, page_size=8 if name in "ACE" else 16, slots=3)
        got = H.replay(eng, steps)
        assert len(got) == len(want)
        worst, where = _worst(got, want)
        assert worst < TOL[dtype], f"{name} {dtype} {cut}: {worst} at {where}"
        eng.manager.check_invariants()
        assert eng.manager.stats()["live_requests"] == 0


def test_token_by_token_equals_whole_prompt(models):
    """Every token alone (the state and the convolution's inputs cross a step at every token) against the
    prompt in one step: float32 results agree to rounding."""
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
    """A short prompt and 150 single tokens (captured decode steps once the shape has been seen), for two
    requests side by side whose contexts cross pages and key tiles at different steps."""
    folder, weights, cfg = models["C"]
    reqs = _requests(cfg["vocab"], [157, 171], seed=4)
    steps = [{"entries": [{"id": "r0", "tokens": reqs["r0"][:7], "want": [6]}, {"id": "r1", "tokens": reqs["r1"][:21], "want": [20]}],
              "end": []}]
    for i in range(150):
        steps.append({"entries": [{"id": "r0", "tokens": [reqs["r0"][7 + i]], "want": [0]},
                                  {"id": "r1", "tokens": [reqs["r1"][21 + i]], "want": [0]}], "end": []})
    want = _want(weights, cfg, reqs)
    for dtype in ("float32", "bfloat16"):
        eng = _engine(folder, dtype, num_pages=64, page_size=8)
        got = H.replay(eng, steps)
        assert eng.stats()["graph_replays"] > 100
        worst, where = _worst(got, {k: want[k] for k in got})
        assert worst < TOL[dtype], (dtype, worst, where)


def test_slots_and_pages_are_used_again(models):
    """One slot and the pages of one request: five requests one after the other, each starting from a
    zero state although the slot and the pages still hold the last request's numbers."""
    folder, weights, cfg = models["A"]
    reqs = _requests(cfg["vocab"], [30, 30, 29, 31, 30], seed=9)
    steps = H.cut_portions(reqs, sizes=(9, 1, 20, 1))
    eng = _engine(folder, "float32", num_pages=8, page_size=4, slots=1)
    got = H.replay(eng, steps)
    worst, where = _worst(got, _want(weights, cfg, reqs))
    assert worst < TOL["float32"], (worst, where)


def test_sink_counts(tmp_path_factory):
    """With sinks far above every score the attention output nearly vanishes; leaving the sink out would
    change the logits by orders of magnitude more than the tolerance."""
    folder, weights, cfg = _folder(tmp_path_factory, "B", sink_mean=6.0)
    reqs = _requests(cfg["vocab"], [50], seed=2)
    steps = H.cut_portions(reqs, sizes=(17, 2, 31))
    got = H.replay(_engine(folder, "float32", steps), steps)
    want = _want(weights, cfg, reqs)
    worst, where = _worst(got, want)
    assert worst < TOL["float32"], (worst, where)
    no_sink = {k: v for k, v in weights.items() if not k.endswith(".sink")}
    for k in weights:
        if k.endswith(".sink"):
            no_sink[k] = torch.full_like(weights[k], -1e4)
    far, _ = _worst(got, _want(no_sink, cfg, reqs))
    assert far > 100 * TOL["float32"]


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
    subprocess.run([sys.executable, "-m", "quanta_b200", "random-weights", "--config", str(tmp_path / "c.json"), "--seed", "3",
                    "--out", str(out)], check=True, cwd=str(H.__file__).rsplit("/tests/", 1)[0])
    r = subprocess.run([sys.executable, "-m", "quanta_b200", "generate", "--model", str(out), "--prompt-ids", "1,2,3,4,5",
                        "--max-new-tokens", "5", "--dtype", "float32", "--eos-id", "60"], check=True, capture_output=True,
                       text=True, cwd=str(H.__file__).rsplit("/tests/", 1)[0])
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
    tok_req = [r for r, n in enumerate(lengths) for _ in range(n)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)  # noqa: E731
    return i32(tok_req), i32(starts), i32(slots)


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_short_convolution_alone(taps):
    """Portions of 1, 2 and more rows (shorter and longer than the history), three requests in one call, slots
    that are not in order, against the whole-sequence convolution."""
    from quanta_b200 import kernels
    dev, C = "cuda:0", 40
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(C, taps, generator=g)
    seqs = [torch.randn(n, C, generator=g) for n in (23, 9, 14)]
    want = [s + P.causal_conv(s, w) for s in seqs]
    state = torch.full((5, max(taps - 1, 0), C), 7.0, device=dev)     # stale numbers in every slot
    slots = [3, 0, 4]
    for s in slots:
        state[s].zero_()
    done = [0, 0, 0]
    cuts = [[1, 1, 2, 7, 1, 11], [2, 1, 6], [14]]
    got = [[], [], []]
    for step in range(6):
        rows = [r for r in range(3) if step < len(cuts[r])]
        lengths = [cuts[r][step] for r in rows]
        x = torch.cat([seqs[r][done[r]: done[r] + n] for r, n in zip(rows, lengths)]).to(dev)
        tok_req, starts, sl = _ctx_arrays(lengths, [slots[r] for r in rows], dev)
        out = torch.empty_like(x)
        kernels.short_conv(x.contiguous(), w.to(dev), state, out, tok_req, starts, sl)
        off = 0
        for r, n in zip(rows, lengths):
            got[r].append(out[off: off + n].cpu())
            off += n
            done[r] += n
    for r in range(3):
        assert torch.allclose(torch.cat(got[r]), want[r], atol=1e-5, rtol=1e-5)
    if taps > 1:
        assert float(state[1].min()) == 7.0 and float(state[2].min()) == 7.0     # slots of no request stay as they were


@pytest.mark.parametrize("dim,heads", [(8, 3), (24, 2), (48, 5), (64, 1), (72, 2), (128, 2), (136, 1)])
def test_delta_rule_alone(dim, heads):
    """The recurrence kernel against the plain loop: three requests of unequal length in two calls (the state
    crosses the call; one request brings a single token), decays near 1 and near exp(-0.6), removal rates over
    the whole range."""
    from quanta_b200 import kernels
    dev = "cuda:0"
    g = torch.Generator().manual_seed(dim)
    HD = heads * dim
    lengths = [[19, 1, 40], [1, 30, 3]]
    total = [sum(x) for x in zip(*lengths)]
    n_all = sum(total)
    proj = torch.randn(n_all, 4 * HD + 5, generator=g)           # r, k, v, a and columns that are not read
    proj[:, HD:2 * HD] *= 3.0
    wpre = 3.0 * torch.randn(n_all, HD, generator=g)
    a_b, w_b = torch.randn(HD, generator=g), torch.randn(HD, generator=g)
    scale = math.exp(-0.5)
    state = torch.full((4, heads, dim, dim), 5.0, device=dev)
    slots = [2, 0, 3]
    for s in slots:
        state[s].zero_()
    rows_of = []
    at = 0
    for r in range(3):
        rows_of.append(list(range(at, at + total[r])))
        at += total[r]
    got = torch.zeros(n_all, heads, dim)
    done = [0, 0, 0]
    for call in lengths:
        idx = [i for r in range(3) for i in rows_of[r][done[r]: done[r] + call[r]]]
        _, starts, sl = _ctx_arrays(call, slots, dev)
        out = torch.empty(len(idx), heads, dim, device=dev)
        kernels.delta_rule(proj[idx].to(dev).contiguous(), (0, HD, 2 * HD, 3 * HD), wpre[idx].to(dev).contiguous(), a_b.to(dev),
                           w_b.to(dev), state, out, starts, sl, heads, dim, scale, 1e-6)
        got[idx] = out.cpu()
        for r in range(3):
            done[r] += call[r]
    for r in range(3):
        rows = rows_of[r]
        view = lambda lo: proj[rows, lo: lo + HD].view(-1, heads, dim)  # noqa: E731
        a = torch.sigmoid(view(3 * HD) + a_b.view(heads, dim))
        decay = torch.exp(-scale * torch.sigmoid(wpre[rows].view(-1, heads, dim) + w_b.view(heads, dim)))
        want, S = P.delta_recurrence(view(0), view(HD), view(2 * HD), a, decay)
        assert torch.allclose(got[rows], want, atol=2e-4 * float(want.abs().max()), rtol=1e-4), (r, dim)
        assert torch.allclose(state[slots[r]].cpu(), S, atol=2e-4 * float(S.abs().max()), rtol=1e-4)
    assert float(state[1].min()) == 5.0


@pytest.mark.parametrize("width", [48, 256, 1000])
def test_post_norm_and_next_norm_in_one_launch(width):
    """A sublayer's output normed, added to the stream and the sum normed, in one kernel: against plain arithmetic,
    for all rows and for chosen rows that leave the stream as it is."""
    from quanta_b200 import kernels
    dev = "cuda:0"
    g = torch.Generator().manual_seed(width)
    T = 9
    h, y = torch.randn(T, width, generator=g) * 3, torch.randn(T, width, generator=g) * 0.01
    gy, w = 1 + 0.3 * torch.randn(width, generator=g), 1 + 0.3 * torch.randn(width, generator=g)
    summed = h + P.rms_norm(y, gy, 1e-6)
    want = P.rms_norm(summed, w, 1e-5)
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 1e-2)):
        hd, out = h.to(dev), torch.empty(T, width, dtype=dtype, device=dev)
        kernels.normed_add_rmsnorm(hd, y.to(dev), gy.to(dev), 1e-6, w.to(dev), 1e-5, out)
        assert torch.allclose(hd.cpu(), summed, atol=1e-6, rtol=1e-6)
        assert torch.allclose(out.float().cpu(), want, atol=tol, rtol=tol)
    rows = torch.tensor([7, 2], dtype=torch.int32, device=dev)
    hd, out = h.to(dev), torch.empty(2, width, device=dev)
    kernels.normed_add_rmsnorm(hd, y.to(dev), gy.to(dev), 1e-6, w.to(dev), 1e-5, out, rows=rows, store_h=False)
    assert torch.equal(hd.cpu(), h) and torch.allclose(out.cpu(), want[[7, 2]], atol=2e-6, rtol=2e-6)


def _paged_rows(rows_per_req, page_size, width, dtype, dev, seed):
    """Cache pages in a shuffled order holding ``rows_per_req`` (a list of [n, width] tensors)."""
    need = [-(-r.shape[0] // page_size) for r in rows_per_req]
    ids = list(range(sum(need) + 3))
    random.Random(seed).shuffle(ids)
    pages = torch.zeros(len(ids), 1, page_size, width, dtype=dtype, device=dev)
    table = torch.full((len(rows_per_req), max(need)), -1, dtype=torch.int32)
    at = 0
    for r, rows in enumerate(rows_per_req):
        for p in range(need[r]):
            pid = ids[at]
            at += 1
            table[r, p] = pid
            chunk = rows[p * page_size: (p + 1) * page_size]
            pages[pid, 0, : chunk.shape[0]] = chunk.to(dev, dtype)
    return pages, table.to(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_ranges", [1, 3, 16])
def test_latent_attention_finds_one_key_among_many(dtype, n_ranges):
    """Queries at positions just before, at and after page and tile borders, each with ONE key (the first, one at
    a border, one far back, its own) made to outweigh some 700 others; single tokens of a long request and a
    portion of another in the same call; nine heads; keys cut into 1, 3 and 16 ranges.  Against a plain softmax."""
    from quanta_b200 import kernels
    dev, Hh, C, R, ps = "cuda:0", 9, 40, 8, 16
    g = torch.Generator().manual_seed(n_ranges)
    n0, n1 = 700, 130
    rows = [0.3 * torch.randn(n0, C + R, generator=g), 0.3 * torch.randn(n1, C + R, generator=g)]
    if dtype == torch.bfloat16:
        rows = [r.to(dtype).float() for r in rows]
    queries = [(0, p, k) for p, k in ((699, 0), (698, 15), (697, 16), (696, 17), (695, 31), (694, 32), (693, 640), (692, 692),
                                      (31, 0), (32, 31), (33, 32), (0, 0), (15, 1), (16, 16), (17, 3))]
    queries += [(1, p, (p * 7) % (p + 1)) for p in range(97, 130)]          # a portion: positions 97..129 of request 1
    T = len(queries)
    q_lat = 0.3 * torch.randn(Hh, T, C, generator=g)
    q_rot = 0.3 * torch.randn(T, Hh, R, generator=g)
    for t, (r, p, k) in enumerate(queries):
        for h in range(Hh):
            key = rows[r][k]
            q_lat[h, t] += (6.0 + h) * key[:C] / key[:C].norm() ** 2 * 2.0
    if dtype == torch.bfloat16:
        q_lat = q_lat.to(dtype).float()
    sink = torch.randn(Hh, generator=g)
    scale = 0.7
    pages, table = _paged_rows(rows, ps, C + R, dtype, dev, seed=n_ranges)
    tok_pos = torch.tensor([p for _, p, _ in queries], dtype=torch.int32, device=dev)
    tok_req = torch.tensor([r for r, _, _ in queries], dtype=torch.int32, device=dev)
    out = torch.empty(Hh, T, C, dtype=dtype, device=dev)
    status = kernels.new_status(dev)
    kernels.latent_attend(q_lat.to(dev), q_rot.to(dev), pages, sink.to(dev), out, tok_pos, tok_req, table, scale, n_ranges, status)
    assert int(status.cpu()[0]) == 0
    out = out.float().cpu()
    for t, (r, p, k) in enumerate(queries):
        keys = rows[r][: p + 1]
        s = (torch.einsum("hc,jc->hj", q_lat[:, t], keys[:, :C]) + torch.einsum("hr,jr->hj", q_rot[t], keys[:, C:])) * scale
        prob = P.sink_softmax(s[:, None, :], sink)[:, 0]
        assert int(prob[-1].argmax()) == k                      # the made key does stand out
        want = prob @ keys[:, :C]
        tol = 1e-5 if dtype == torch.float32 else 8e-3
        assert torch.allclose(out[:, t], want, atol=tol, rtol=tol), (t, r, p, k, float((out[:, t] - want).abs().max()))


# (4, 64, 64): the kernel's dynamic shared memory is exactly 48 KB, beside which it has static shared memory
@pytest.mark.parametrize("heads,C,R", [(16, 64, 16), (5, 128, 32), (33, 256, 16), (3, 512, 64), (4, 64, 64)])
@pytest.mark.parametrize("n_ranges", [1, 5])
def test_latent_attention_on_the_tensor_cores(heads, C, R, n_ranges):
    """The tensor-core kernel against a plain softmax, and against the CUDA-core kernel: single tokens of a long
    request at positions around page and tile borders, a portion of another request and a third request of one
    token at position 0, each query with one made key (the first, at a border, far back, its own) that
    outweighs the rest; heads that fill a tile exactly, leave it ragged, and spill over."""
    from quanta_b200 import kernels
    dev, ps, dtype = "cuda:0", 16, torch.bfloat16
    g = torch.Generator().manual_seed(heads + n_ranges)
    rows = [(0.3 * torch.randn(n, C + R, generator=g)).to(dtype).float() for n in (700, 130, 1)]
    queries = [(0, p, k) for p, k in ((0, 0), (15, 1), (16, 16), (17, 3), (31, 0), (32, 31), (33, 32), (63, 0), (64, 64), (65, 63),
                                      (692, 692), (693, 640), (694, 32), (695, 31), (696, 17), (697, 16), (698, 15), (699, 0))]
    queries += [(1, p, (p * 7) % (p + 1)) for p in range(97, 130)]
    queries += [(2, 0, 0)]
    T = len(queries)
    req_start = torch.tensor([0, 18, 18 + 33, T], dtype=torch.int32, device=dev)
    q_lat = 0.3 * torch.randn(heads, T, C, generator=g)
    q_rot = 0.3 * torch.randn(T, heads, R, generator=g)
    for t, (r, p, k) in enumerate(queries):
        key = rows[r][k]
        for h in range(heads):
            q_lat[h, t] += (12.0 + (h % 7)) * key[:C] / key[:C].norm() ** 2
    sink = torch.randn(heads, generator=g)
    scale = 0.7
    pages, table = _paged_rows(rows, ps, C + R, dtype, dev, seed=heads)
    tok_pos = torch.tensor([p for _, p, _ in queries], dtype=torch.int32, device=dev)
    tok_req = torch.tensor([r for r, _, _ in queries], dtype=torch.int32, device=dev)
    status = kernels.new_status(dev)
    assert kernels.latent_attend_uses_tensor_cores(dtype, C, R)
    out = {}
    for tc in (True, False):
        o = torch.empty(heads, T, C, dtype=dtype, device=dev)
        kernels.latent_attend(q_lat.to(dev), q_rot.to(dev), pages, sink.to(dev), o, tok_pos, tok_req, table, scale, n_ranges,
                              status, req_start=req_start, tensor_cores=tc)
        out[tc] = o.float().cpu()
    assert int(status.cpu()[0]) == 0
    qb = (q_lat * scale).to(dtype).float() / scale          # the tensor-core kernel rounds the scaled query to bfloat16
    rb = (q_rot * scale).to(dtype).float() / scale
    for t, (r, p, k) in enumerate(queries):
        keys = rows[r][: p + 1]
        s = (torch.einsum("hc,jc->hj", qb[:, t], keys[:, :C]) + torch.einsum("hr,jr->hj", rb[t], keys[:, C:])) * scale
        prob = P.sink_softmax(s[:, None, :], sink)[:, 0]
        assert int(prob[-1].argmax()) == k
        want = prob @ keys[:, :C]
        assert torch.allclose(out[True][:, t], want, atol=6e-3, rtol=2e-2), (t, r, p, k, float((out[True][:, t] - want).abs().max()))
        assert torch.allclose(out[True][:, t], out[False][:, t], atol=1.5e-2, rtol=3e-2), (t, r, p, k)


def test_latent_rows_are_written_normed_and_rotated():
    """The cache row of a position: RMS norm with gain of the latent part, rotation of the first ``rotated`` of
    the shared key part by the position, the rest unchanged; positions on both sides of a page border."""
    from quanta_b200 import kernels
    dev, C, R, rd, ps, eps = "cuda:0", 24, 12, 8, 4, 1e-5
    g = torch.Generator().manual_seed(0)
    T = 11
    dkv = torch.randn(T, C + R, generator=g)
    gain = 1 + 0.3 * torch.randn(C, generator=g)
    base = 50.0
    inv_freq = base ** (-2.0 * torch.arange(rd // 2, dtype=torch.float32) / rd)
    pos = torch.arange(3, 3 + T)
    pages = torch.zeros(8, 1, ps, C + R, device=dev)
    table = torch.tensor([[5, 2, 7, 0]], dtype=torch.int32, device=dev)
    status = kernels.new_status(dev)
    kernels.latent_write(dkv.to(dev), gain.to(dev), inv_freq.to(dev), pages, pos.to(dev, torch.int32),
                         torch.zeros(T, dtype=torch.int32, device=dev), table, C, R, rd, ps, eps, status)
    want = torch.cat([P.rms_norm(dkv[:, :C], gain, eps), P.rotate_half(dkv[:, C:], pos, base, rd)], -1)
    for t in range(T):
        p = int(pos[t])
        got = pages[int(table[0, p // ps]), 0, p % ps].cpu()
        assert torch.allclose(got, want[t], atol=2e-6, rtol=1e-5), t
