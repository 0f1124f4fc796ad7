"""The Kunonex architecture against its plain restatement (plain_kunonex.py):
every mechanism alone through its part and kernels, then whole models of six
tiny configurations that differ in every size and option, stepped whole, token
by token, in portions down to two tokens, in mixed batches over a pool so
small that pages and state slots are used again, through bin/trace_run and
through Engine.generate.  Weights are random; attention is sharpened so that
single keys, far ones too, carry the result."""
from __future__ import annotations

import copy
import json
import random

import numpy as np
import pytest
import torch

import plain_kunonex as plain
from helpers import KX, TOL, TraceProcess, kunonex_tensors, load_kunonex_plain, make_kunonex_folder, random_tokens

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
PTOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}
NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


def _rel(got, want):
    got, want = torch.as_tensor(got).double().cpu(), torch.as_tensor(want).double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def _rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


# ------------------------------------------------------------------ CPU: configuration and spec
def test_config_is_read_from_its_own_keys():
    from inferflux_b200.config import ConfigError, KunonexConfig, build_spec, load_config
    cfg = load_config(copy.deepcopy(KX["A"]))
    assert isinstance(cfg, KunonexConfig) and cfg.width == 64 and cfg.vocab_size == 300 and cfg.norm_eps == 1e-5
    assert [l.type for l in cfg.layers] == ["latent_attention", "mingru", "latent_attention", "mingru"]
    assert cfg.layers[2].ff == 0 and cfg.layers[0].mixer["kv_rank"] == 40 and cfg.layers[0].mixer["scale"] == 0.31
    assert load_config(cfg.to_dict()) == cfg                                  # what it writes, it reads back
    spec = build_spec(cfg)
    # layers 1 and 2 run twice, a junction ahead of each pass; the junction is one more entry of the spec's layers
    assert [(r.layer, r.params.get("pass")) for r in spec.schedule] == [
        (0, None), (4, 0), (1, 0), (2, 0), (4, 1), (1, 1), (2, 1), (3, None)]
    assert [(i, t) for i, t in plain.layer_runs(KX["A"])] == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (3, None)]
    assert "feed_forward" not in spec.layers[2].parts and spec.layers[4].arrangement == "junction"
    unscaled = copy.deepcopy(KX["A"])
    del unscaled["layers"][0]["mixer"]["scale"]
    assert load_config(unscaled).layers[0].mixer["scale"] == 24 ** -0.5      # absent: one over the root of dim
    no_loop = build_spec(load_config(copy.deepcopy(KX["C"])))
    assert [r.layer for r in no_loop.schedule] == [0, 1, 2] and len(no_loop.layers) == 3
    for breaker, text in [(lambda d: d["layers"][0].update(type="conv"), "type"), (lambda d: d.pop("width"), "width"),
                          (lambda d: d["layers"][1]["mixer"].pop("width"), "width"),
                          (lambda d: d["loop"].update(stop=9), "loop"), (lambda d: d["norm"].pop("eps"), "eps"),
                          (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "kind")]:
        bad = copy.deepcopy(KX["A"])
        breaker(bad)
        with pytest.raises(ConfigError, match=text):
            load_config(bad)


def test_cache_and_state_plan():
    """Every run of a looped layer has a cache index or state tensors of its own; only the latent is paged."""
    from inferflux_b200.config import build_spec, load_config
    from inferflux_b200.engine import Model
    model = Model(build_spec(load_config(copy.deepcopy(KX["A"]))), torch.float32, "cpu")
    names = {w.name: tuple(w.shape) for w in model.weight_specs()}
    assert names["loop.in"] == (64, 128) and names["loop.step"] == (2, 64) and names["l0.mix.uk"] == (72, 40)
    assert names["l1.mix.z.b"] == (64,) and names["l0.mlp.act"] == (4,) and "l2.mlp.up" not in names
    assert names["head"] == (300, 64) and names["embed.norm"] == (64,) and names["l3.shift"] == (64,)
    # two cache groups (latents of 40 and of 24 elements), two runs of layer 2 in the second
    assert [n.streams[0].width for n in model.kv_needs] == [40, 24] and model.runs_per_group == [1, 2]
    states = [sorted(s.name for s in needs) for needs in model.state_needs]
    assert states == [["shift_prev"], [], ["gru", "shift_prev"], ["shift_prev"], [], ["gru", "shift_prev"], ["shift_prev"],
                      ["gru", "shift_prev"]]


def test_plain_recurrence_and_shift_carry_over():
    """The plain implementation's own consistency: a sequence cut in two, the state handed over."""
    w = {"m.z": _rand((6, 5), 1).double(), "m.z.b": _rand((6,), 2).double(), "m.x": _rand((6, 5), 3).double(),
         "m.x.b": _rand((6,), 4).double(), "m.g": _rand((6, 5), 5).double(), "m.o": _rand((5, 6), 6).double()}
    h = _rand((9, 5), 7).double()
    whole, last = plain.mingru(h, w, "m")
    a, s = plain.mingru(h[:4], w, "m")
    b, s2 = plain.mingru(h[4:], w, "m", s)
    assert torch.allclose(torch.cat([a, b]), whole) and torch.allclose(s2, last)
    mu = _rand((5,), 8).double()
    assert torch.allclose(torch.cat([plain.token_shift(h[:4], mu), plain.token_shift(h[4:], mu, h[3])]),
                          plain.token_shift(h, mu))
    u = torch.tensor([-2.0, 0.0, 3.0], dtype=torch.float64)         # the candidate is continuous at 0 and grows linearly above
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    assert torch.allclose(cand, torch.tensor([0.11920292, 0.5, 3.5], dtype=torch.float64))


# ------------------------------------------------------------------ GPU: the parts alone
gpu = pytest.mark.gpu


def _load(part, tensors, dtype):
    part.load({k: (v.to(dtype) if v.dim() > 1 else v.float()).to(DEV) for k, v in tensors.items()})


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [40, 50, 100, 1536, 9000])       # rows in registers, and (50, 9000) the plain kernel
def test_layernorm_alone(dtype, hidden):
    from inferflux_b200.parts import LayerNorm
    from inferflux_b200.parts.base import PartialSums
    part = LayerNorm(dict(weight_name="n", hidden=hidden, eps=3e-6), "l", dtype, DEV)
    assert [w.name for w in LayerNorm.weight_specs(part.params, "l")] == ["l.n"]
    w = 1 + _rand((hidden,), 1, 0.1)
    _load(part, {"l.n": w}, dtype)
    res = (_rand((9, hidden), 2) + 30.0).to(DEV)                   # a large mean: the variance must not cancel
    parts = _rand((3, 9, hidden), 3).to(DEV)
    want_res = res.cpu().double() + parts.cpu().double().sum(0)
    out32 = torch.empty((9, hidden), dtype=torch.float32, device=DEV)
    out = part.forward(res, PartialSums(parts), out32=out32)
    assert out.dtype == dtype and _rel(res, want_res) < 1e-6
    assert _rel(out, plain.layer_norm(want_res, w.double(), 3e-6)) < PTOL[dtype]
    assert _rel(out32, plain.layer_norm(want_res, w.double(), 3e-6)) < 2e-5
    rows = torch.tensor([7, 0, 7], dtype=torch.int32, device=DEV)
    before = res.clone()
    picked = part.forward(res, None, rows=rows)
    assert torch.equal(res, before) and _rel(picked, plain.layer_norm(want_res[[7, 0, 7]], w.double(), 3e-6)) < PTOL[dtype]


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_alone(dtype):
    from types import SimpleNamespace
    from inferflux_b200.parts import SinusoidNormEmbedding
    v, h = 77, 52
    table, w = _rand((v, h), 8).to(dtype).float(), 1 + _rand((h,), 9, 0.1)
    part = SinusoidNormEmbedding(dict(vocab=v, hidden=h, eps=1e-5, table="e", norm_weight="e.n"), "", dtype, DEV)
    _load(part, {"e": table, "e.n": w}, dtype)
    ids = torch.tensor([0, 76, 5, 5, 33], dtype=torch.int32, device=DEV)
    pos = torch.tensor([0, 1, 17, 4095, 100000], dtype=torch.int32, device=DEV)
    got = part.forward_step(SimpleNamespace(token_ids=ids, positions=pos))
    want = plain.embed({"embed": table.double(), "embed.norm": w.double()}, ids.cpu(), pos.cpu(), 1e-5)
    assert got.dtype == torch.float32 and _rel(got, want) < 2e-6


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter", [(3, 136), (40, 136), (5, 135), (9, 2304)])   # three kernels by the row's length
def test_polynorm_feed_forward_alone(dtype, rows, inter):
    from inferflux_b200.parts import PolyNormFF
    h = 96
    part = PolyNormFF(dict(name="mlp", hidden=h, intermediate=inter, eps=2e-6), "l", dtype, DEV)
    w = {"l.mlp.up": _rand((inter, h), 4, 0.2), "l.mlp.up.b": _rand((inter,), 5, 0.3), "l.mlp.down": _rand((h, inter), 6, 0.2),
         "l.mlp.down.b": _rand((h,), 7, 0.3), "l.mlp.act": torch.tensor([0.7, -0.4, 0.25, 0.1])}
    w = {k: (v.to(dtype).float() if v.dim() > 1 else v) for k, v in w.items()}
    _load(part, dict(w), dtype)
    x = _rand((rows, h), 8).to(dtype)
    got = part.forward(x.to(DEV), None)
    want = plain.dense_ff(x.double(), {k: v.double() for k, v in w.items()}, "l.mlp", 2e-6)
    assert got.dtype == torch.float32 and _rel(got, want) < PTOL[dtype]


def _runner_for(cfg, dtype, seed, tokens=512, **kw):
    from inferflux_b200.config import EngineConfig
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine import Model, StepRunner
    config, tensors = kunonex_tensors(cfg, seed, **kw)
    model = Model(build_spec(config), dtype, DEV)
    plain_w = {k: v.double() for k, v in tensors.items()}
    model.load({k: (v.to(dtype) if v.dim() > 1 else v.float()).to(DEV) for k, v in tensors.items()})
    runner = StepRunner(model, EngineConfig(dtype=NAME[dtype], kv_cache_tokens=tokens, max_seqs=4))
    return model, runner, plain_w


def _mixer_in_portions(model, runner, layer_run, x, portions, dtype):
    """Call one run's mixer alone on rows cut into portions of one request."""
    from inferflux_b200.engine import StepEntry
    from inferflux_b200.parts.base import PartialSums
    info = model.runs[layer_run]
    mixer = model.blocks[model.spec.schedule[layer_run].layer].mixer
    outs, pos = [], 0
    for n in portions:
        ctx = runner.build_context([StepEntry("r", [1] * n, [])])
        out = mixer.forward(x[pos:pos + n].to(dtype).to(DEV), ctx, info, None)
        outs.append(out.tensor.sum(0) if isinstance(out, PartialSums) else out.float())
        runner.kv.advance("r", n)
        pos += n
    runner.end("r")
    return torch.cat(outs)


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_mingru_alone(dtype):
    """A portion that the scan cuts into three segments, single tokens, two tokens, a portion that ends on a
    segment's edge; the state goes through the request's slot."""
    cfg = dict(KX["B"], layers=[KX["B"]["layers"][0]], loop=None)        # width 200: not a multiple of the block
    model, runner, w = _runner_for(cfg, dtype, 5)
    x = _rand((150 + 1 + 1 + 2 + 64 + 7, 96), 6).to(dtype)
    want, _ = plain.mingru(x.double(), w, "l0.mix")
    got = _mixer_in_portions(model, runner, 0, x, [150, 1, 1, 2, 64, 7], dtype)
    assert _rel(got, want) < PTOL[dtype]
    # the slot was given back: the next request starts from zero
    again = _mixer_in_portions(model, runner, 0, x[:10], [10], dtype)
    assert _rel(again, want[:10]) < PTOL[dtype]


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", [0, 2])            # KX_A's two attention layers: 3 heads of rank 40, one head of rank 24
def test_latent_attention_alone(dtype, which):
    """Portions that start and end inside pages of 16, single tokens across a page border, two tokens."""
    layer = KX["A"]["layers"][which]
    cfg = dict(KX["A"], layers=[layer], loop=None)
    model, runner, w = _runner_for(cfg, dtype, 11)
    portions = [21, 10, 1, 1, 2, 13, 16, 1]
    x = _rand((sum(portions), 64), 12).to(dtype)
    want = plain.latent_attention(x.double(), w, "l0.mix", layer["mixer"], 1e-5)
    got = _mixer_in_portions(model, runner, 0, x, portions, dtype)
    assert _rel(got, want) < PTOL[dtype]


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_finds_single_far_keys(dtype):
    """640 tokens.  Head 0's weights are set so that its score is the inner product of the query token's
    first half with the key token's second half (both at unit root mean square), and each of the last five
    tokens is given a first half that equals the second half of one chosen earlier token: the very first, the
    last of the first page, the first of the second, its neighbour, and one in the middle.  Each query then
    puts all of its weight on that one key among hundreds, so a key that is lost, doubled or shifted by one at
    a page's edge changes the result entirely.  The first of the five queries lies in a portion, the others
    are single tokens."""
    R, hidden, n = 32, 64, 640
    layer = dict(type="latent_attention", mixer=dict(heads=2, dim=R, vdim=24, kv_rank=R, q_rank=R, scale=1.0), mlp=None)
    cfg = dict(KX["C"], width=hidden, layers=[layer], loop=None)
    config, tensors = kunonex_tensors(cfg, 13)
    eye = torch.eye(R)
    tensors["l0.mix.dq"] = torch.cat([eye, torch.zeros(R, R)], 1).to(torch.bfloat16)
    tensors["l0.mix.dkv"] = torch.cat([torch.zeros(R, R), eye], 1).to(torch.bfloat16)
    tensors["l0.mix.dq.norm"] = torch.ones(R, dtype=torch.bfloat16)
    tensors["l0.mix.dkv.norm"] = torch.ones(R, dtype=torch.bfloat16)
    tensors["l0.mix.uq"][:R] = eye.to(torch.bfloat16)
    tensors["l0.mix.uk"][:R] = eye.to(torch.bfloat16)
    tensors["l0.mix.uv"] = _rand((2 * 24, R), 15, 0.5).to(torch.bfloat16)
    from inferflux_b200.config import EngineConfig
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine import Model, StepRunner
    model = Model(build_spec(config), dtype, DEV)
    w = {k: v.double() for k, v in tensors.items()}
    model.load({k: (v.to(dtype) if v.dim() > 1 else v.float()).to(DEV) for k, v in tensors.items()})
    runner = StepRunner(model, EngineConfig(dtype=NAME[dtype], kv_cache_tokens=1024, max_seqs=4))
    x = _rand((n, hidden), 14).to(torch.bfloat16).float()
    targets = [0, 15, 16, 17, 300]
    for q, t in zip(range(n - 5, n), targets):
        x[q, :R] = x[t, R:]
    want = plain.latent_attention(x.double(), w, "l0.mix", layer["mixer"], 1e-6)
    # in the plain implementation the chosen key carries the row: without it the result is another one
    for q, t in zip(range(n - 5, n), targets):
        other = x.clone()
        other[t, R:] = _rand((R,), 99 + t)
        moved = plain.latent_attention(other.double(), w, "l0.mix", layer["mixer"], 1e-6)[q]
        assert _rel(moved, want[q]) > 0.2, (q, t)
    got = _mixer_in_portions(model, runner, 0, x, [600, 36, 1, 1, 1, 1], dtype)
    for q in range(n - 5, n):
        assert _rel(got[q], want[q]) < PTOL[dtype], q
    assert _rel(got, want) < PTOL[dtype]


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_token_shift_and_fused_single_token_path(dtype):
    """The shift part over portions and single tokens, and the kernel that does sum, norm, shift and state
    update at once for a step of single tokens, against the plain functions."""
    from inferflux_b200.engine import StepEntry
    from inferflux_b200.kernels import ops
    cfg = dict(KX["C"], layers=[KX["C"]["layers"][1]], loop=None)
    model, runner, w = _runner_for(cfg, dtype, 21)
    block, info = model.blocks[0], model.runs[0]
    h = _rand((30, 40), 22)
    want = plain.token_shift(h.double(), w["l0.shift"])
    outs, pos = [], 0
    for n in (7, 1, 2, 1, 19):
        ctx = runner.build_context([StepEntry("r", [1] * n, [])])
        outs.append(block.shift.forward(h[pos:pos + n].to(DEV), ctx, info).float())
        runner.kv.advance("r", n)
        pos += n
    assert _rel(torch.cat(outs), want) < PTOL[dtype]
    runner.end("r")
    # fused: three requests, one token each, three steps
    res = _rand((3, 3, 40), 23) + 5.0
    delta = _rand((3, 3, 40), 24)
    normed = plain.layer_norm((res + delta).double(), w["l0.norm1"], 1e-6)            # [step, request, hidden]
    for step in range(3):
        ctx = runner.build_context([StepEntry(f"q{i}", [1], []) for i in range(3)])
        r = res[step].to(DEV).contiguous()
        out, shifted = torch.empty((3, 40), dtype=dtype, device=DEV), torch.empty((3, 40), dtype=dtype, device=DEV)
        ops.add_layernorm_shift1(r, delta[step].to(DEV).contiguous(), block.norm.weight, block.norm.eps, block.shift.mu,
                                 info.states["shift_prev"], ctx.entry_slot, out, shifted)
        before = normed[step - 1] if step else torch.zeros_like(normed[0])
        assert _rel(out, normed[step]) < PTOL[dtype]
        assert _rel(shifted, normed[step] + (before - normed[step]) * w["l0.shift"]) < PTOL[dtype]
        assert _rel(r, (res[step] + delta[step]).double()) < 1e-6
        for i in range(3):
            runner.kv.advance(f"q{i}", 1)


# ------------------------------------------------------------------ GPU: whole models through the step function
def _logits_in_steps(runner, rid, toks, sizes):
    from inferflux_b200.engine import StepEntry
    outs, pos, k = [], 0, 0
    while pos < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - pos)
        outs.append(runner.step([StepEntry(rid, toks[pos:pos + n], list(range(n)))]).clone())
        pos, k = pos + n, k + 1
    runner.end(rid)
    return torch.cat(outs)


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_model_whole_one_by_one_and_in_portions(dtype, name):
    """Every layer's residual stream is not compared here; the logits at every position are, for three ways
    of cutting the same prompt.  In float32 the three agree with each other almost to the bit."""
    cfg = KX[name]
    model, runner, w = _runner_for(cfg, dtype, ord(name), tokens=1024)
    toks = random_tokens(cfg["vocab"], 150, 31)
    want = plain.forward(cfg, w, toks)
    whole = _logits_in_steps(runner, "w", toks, [150])
    assert _rel(whole, want) < PTOL[dtype]
    if name == "E":
        mixer = model.blocks[0].mixer
        assert (mixer.ukv is not None) == (dtype == torch.bfloat16)    # bfloat16: portions go per head
    ones = _logits_in_steps(runner, "o", toks[:70], [1])              # the captured decode graph after three steps
    assert runner.graph_replays > 0 and _rel(ones, want[:70]) < PTOL[dtype]
    cut = _logits_in_steps(runner, "c", toks, [2, 3, 17, 1, 16, 5, 32, 2, 15, 64, 2])
    assert _rel(cut, want) < PTOL[dtype]
    if dtype == torch.float32:
        assert _rel(cut, whole) < 2e-6 and _rel(ones, whole[:70]) < 2e-6
    runner.kv.check(), runner.slots.check()


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["mingru", "latent_attention"])
def test_models_of_one_kind_of_mixer(dtype, kind):
    """Only recurrent layers (no paged cache at all: the step runs on state slots alone) and only attention
    layers (latents of three different ranks: three cache groups), each looped as a whole."""
    base = KX["A"]
    if kind == "mingru":
        layers = [base["layers"][1], base["layers"][3], dict(base["layers"][1], mlp=None)]
    else:
        layers = [base["layers"][0], base["layers"][2], KX["C"]["layers"][2] | {"mixer": dict(KX["C"]["layers"][2]["mixer"])}]
    cfg = dict(base, layers=layers, loop=dict(start=0, stop=3, times=2))
    model, runner, w = _runner_for(cfg, dtype, 33, tokens=512)
    assert len(model.kv_needs) == (0 if kind == "mingru" else 3)
    toks = random_tokens(cfg["vocab"], 90, 34)
    want = plain.forward(cfg, w, toks)
    assert _rel(_logits_in_steps(runner, "w", toks, [90]), want) < PTOL[dtype]
    assert _rel(_logits_in_steps(runner, "c", toks, [40, 1, 1, 1, 1, 2, 30, 1]), want) < PTOL[dtype]
    runner.kv.check(), runner.slots.check()
    if dtype == torch.float32:
        # the scheduler and the sampler over the same kind of model: what Engine.generate continues a prompt with
        # is what the step function's logits of prompt + continuation, run whole, have as their largest
        from inferflux_b200 import Engine, SamplingParams, StepEntry
        eng = Engine.from_config(dict(cfg), seed=2, dtype="float32", kv_cache_tokens=256, max_seqs=4, chunked_prefill_tokens=16)
        prompts = [random_tokens(cfg["vocab"], n, 35 + n) for n in (3, 37)]
        for p, g in zip(prompts, eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))):
            seq = p + g.tokens
            logits = eng.run_step([StepEntry("v", seq, list(range(len(p) - 1, len(seq) - 1)))])
            eng.runner.end("v")
            assert logits.argmax(-1).tolist() == g.tokens


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "E"])
def test_batches_of_unequal_requests_and_reused_slots(dtype, name):
    """Four requests of unequal length, portions beside single tokens, against each alone; then four more
    in the slots and pages the first ones gave back."""
    from inferflux_b200.engine import StepEntry
    cfg = KX[name]
    model, runner, w = _runner_for(cfg, dtype, 41, tokens=4 * 128)
    rng = random.Random(3)
    for round_ in range(2):
        lens = [97, 5, 64, 33] if round_ == 0 else [31, 120, 2, 70]
        reqs = {f"r{round_}{i}": random_tokens(cfg["vocab"], n, 50 + 10 * round_ + i) for i, n in enumerate(lens)}
        want = {r: plain.forward(cfg, w, t) for r, t in reqs.items()}
        at, got = {r: 0 for r in reqs}, {r: [] for r in reqs}
        while any(at[r] < len(reqs[r]) for r in reqs):
            entries = []
            for r, t in reqs.items():
                left = len(t) - at[r]
                if left == 0 or (rng.random() < 0.2 and len(entries)):
                    continue
                n = 1 if left <= 6 else min(left - 6, rng.choice([1, 2, 3, 16, 29]))
                entries.append(StepEntry(r, t[at[r]:at[r] + n], list(range(n))))
            logits = runner.step(entries)
            row = 0
            for e in entries:
                got[e.rid].append(logits[row:row + len(e.tokens)].clone())
                row += len(e.tokens)
                at[e.rid] += len(e.tokens)
        for r in reqs:
            assert _rel(torch.cat(got[r]), want[r]) < PTOL[dtype], r
            runner.end(r)
        runner.kv.check(), runner.slots.check()
    assert all(p.reuses > 0 for p in runner.kv.pools)


@gpu
def test_long_decoding_after_a_long_prompt():
    """600 tokens at once, then 200 one by one through the captured graph; attention is sharp, so a key that
    is lost or doubled at a page's edge shows."""
    cfg = KX["B"]
    model, runner, w = _runner_for(cfg, torch.float32, 51, tokens=1024)
    toks = random_tokens(cfg["vocab"], 800, 52)
    want = plain.forward(cfg, w, toks)
    got = _logits_in_steps(runner, "d", toks, [600] + [1] * 200)
    assert runner.graph_replays >= 190 and _rel(got, want) < 2e-5


# ------------------------------------------------------------------ GPU: bin/trace_run and Engine.generate
LENGTHS = {"A": [70, 33, 5, 130, 64, 97, 1], "B": [150, 40, 9, 65, 111]}


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_replay_mixed_with_page_and_slot_reuse(name, dtype):
    """The command-line replay: the config.json picks the architecture; four state slots, a pool of the four
    longest requests; every request twice, so pages and slots turn over."""
    cfg = KX[name]
    folder = make_kunonex_folder(cfg, seed=60 + ord(name))
    pcfg, w = load_kunonex_plain(folder)
    requests = [random_tokens(cfg["vocab"], n, 100 + i) for i, n in enumerate(LENGTHS[name])]
    refs = [plain.forward(pcfg, w, r).numpy() for r in requests]
    pool = sum((n + 63) // 64 * 64 for n in sorted(LENGTHS[name])[-4:])
    proc = TraceProcess(folder, dtype, pool)
    rng = random.Random(7)
    waiting = [(f"m{j}_{i}", i) for j, i in enumerate(list(range(len(requests))) * 2)]
    live, worst = {}, 0.0
    while waiting or live:
        while waiting and len(live) < 4:
            rid, i = waiting.pop(0)
            live[rid] = [i, 0]
        entries, ends, checks = [], [], []
        for rid, (i, pos) in list(live.items()):
            toks = requests[i]
            if rng.random() < 0.15 and len(live) > 1:
                continue
            left = len(toks) - pos
            n = 1 if left <= 20 else min(left - 20, rng.choice([2, 3, 7, 16, 29, 48]))
            want = list(range(n)) if n <= 3 else sorted(rng.sample(range(n), 3))
            entries.append(dict(id=rid, tokens=toks[pos:pos + n], want=want))
            checks.append((i, pos, want))
            live[rid][1] = pos + n
            if pos + n == len(toks):
                ends.append(rid)
                del live[rid]
        if not entries:
            continue
        got = proc.step(entries, end=ends)
        row = 0
        for i, pos, want in checks:
            for p in want:
                err = np.abs(got[row].astype(np.float64) - refs[i][pos + p]).max() / np.abs(refs[i]).max()
                worst = max(worst, err)
                row += 1
    stats = proc.stats()
    assert proc.close() == 0
    assert worst <= TOL[dtype], worst
    assert all(u > 0 for u in stats["page_reuses"]) and stats["pages_free"] == stats["pages_total"]


@gpu
def test_greedy_generation_through_the_engine():
    """Engine.from_pretrained picks the architecture by config.json; the scheduler cuts prompts into portions
    of 16 and batches them with decoding requests; float32 greedy continuations equal the plain ones."""
    from inferflux_b200 import Engine, SamplingParams
    cfg = KX["A"]
    folder = make_kunonex_folder(cfg, seed=71)
    pcfg, w = load_kunonex_plain(folder)
    prompts = [random_tokens(cfg["vocab"], n, 80 + n) for n in (5, 41, 17, 70, 3)]

    def plain_greedy(p, n):
        seq = list(p)
        for _ in range(n):
            seq.append(int(plain.forward(pcfg, w, seq)[-1].argmax()))
        return seq[len(p):]

    want = [plain_greedy(p, 12) for p in prompts]
    eng = Engine.from_pretrained(folder, dtype="float32", kv_cache_tokens=512, max_seqs=4, chunked_prefill_tokens=16)
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    assert [g.tokens for g in got] == want
    eng16 = Engine.from_pretrained(folder, dtype="bfloat16", kv_cache_tokens=512, max_seqs=4, chunked_prefill_tokens=16)
    for p, g in zip(prompts, eng16.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))):
        seq = list(p)
        for t in g.tokens:                       # a near tie may break differently: each token within tolerance of the best
            logits = plain.forward(pcfg, w, seq)[-1]
            assert float(logits.max() - logits[t]) <= 4e-2 * float(logits.abs().max())
            seq.append(t)
