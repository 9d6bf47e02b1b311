"""Pudadra through the engine against the plain implementation of ``plain_pudadra``.

Small configurations with random weights of their own: head counts, map and value sizes, rotated widths, windows,
convolution lengths, expert counts, groups and choices that differ from layer to layer and from test to test (also the
degenerate ones: one kv head, as many as heads, values as wide as both maps or not, one tap and none, no cap, no window,
no rotation, all groups kept, one expert chosen, no shared expert, a layer without a feed-forward, constants of 1).
Every mechanism alone; whole prompts against token-by-token decoding and portions down to two tokens; unequal requests in
one batch with pages and slots that are freed, poisoned and used again; keys made dominant just inside and just outside a
window, at page borders and far away, in prompts and for single tokens in splits; long decoding while windows pass over
decoded tokens; greedy generation through ``Engine.generate`` and the scheduler; the trace replay program.

In bfloat16 a router's close call may fall the other way than in the plain float64 implementation, which changes a
token's experts, not the arithmetic under test.  So the bfloat16 comparisons hand the plain implementation the experts
that the engine chose (read from the device lists of the feed-forward); float32 comparisons use the plain router.
"""

from __future__ import annotations

import copy
import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_pudadra as plain

ROOT = Path(__file__).resolve().parent.parent

SCALING = {"factor": 8.0, "low": 1.0, "high": 3.0, "original": 64}
ATT = plain.attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, diff=0.4, window=21, rot_dims=8, softcap=4.0, base=700.0,
                            scaling=SCALING, mlp=plain.dense_mlp(48))
ATT_B = plain.attention_layer(heads=3, kv_heads=3, dim=20, vdim=40, conv=2, diff=0.7, window=40, rot_dims=20, softcap=0.0, base=50000.0,
                              mlp=plain.moe_mlp(ff=24, experts=6, top=2, groups=(3, 2), shared=16))
ATT_C = plain.attention_layer(heads=6, kv_heads=1, dim=8, vdim=72, conv=1, diff=0.25, window=17, rot_dims=4, softcap=9.0, mlp=None)
ATT_PLAIN = plain.attention_layer(heads=2, kv_heads=2, dim=32, vdim=16, conv=0, diff=0.5, window=0, rot_dims=0, softcap=0.0,
                                  mlp=plain.moe_mlp(ff=16, experts=4, top=1, groups=None, shared=0))
LAT = plain.latent_layer(heads=3, dim=8, rot_dim=8, vdim=16, kv_rank=24, window=10, mlp=plain.moe_mlp(ff=16, experts=8, top=3, groups=(4, 2), shared=24))
LAT_B = plain.latent_layer(heads=5, dim=16, rot_dim=4, vdim=8, kv_rank=40, window=33, base=20000.0, mlp=plain.dense_mlp(40))
LAT_C = plain.latent_layer(heads=2, dim=24, rot_dim=16, vdim=24, kv_rank=16, window=0, mlp=plain.moe_mlp(ff=8, experts=3, top=3, groups=(3, 3), shared=8))

FULL = plain.make_config([ATT, LAT, ATT_B, LAT_B, ATT_C, ATT_PLAIN, LAT_C], width=80, vocab=203, eps=1e-5, residual_mult=0.4,
                         logit_scale=1.7)

ALONE = {
    "diff_attention_dense": plain.make_config([ATT]),
    "diff_all_kv_heads_two_taps_no_cap_grouped_experts": plain.make_config([ATT_B], width=72, residual_mult=1.0),
    "diff_one_kv_head_one_tap_wide_values_no_ffn": plain.make_config([ATT_C], width=48, logit_scale=1.0),
    "diff_no_conv_no_window_no_rotation_one_expert": plain.make_config([ATT_PLAIN]),
    "latent_window_grouped_experts": plain.make_config([LAT]),
    "latent_narrow_rotation_dense": plain.make_config([LAT_B], width=56),
    "latent_no_window_all_experts": plain.make_config([LAT_C], width=40),
}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from edgerag_b200.weights.safetensors_io import write_safetensors

    base = tmp_path_factory.mktemp("pudadra")
    made = {}

    def get(name: str, raw: dict, seed: int = 0, edit=None):
        if name not in made:
            folder = base / name
            folder.mkdir()
            tensors = plain.random_weights(raw, seed)
            if edit is not None:
                edit(tensors)
            (folder / "config.json").write_text(json.dumps(raw))
            write_safetensors(folder / "model.safetensors", tensors)
            made[name] = (folder, raw, tensors)
        return made[name]

    return get


class ChoiceLog:
    """Records, for every layer with routed experts, the experts the engine chose for the rows of every step."""

    def __init__(self, model) -> None:
        self.steps: list[dict[int, torch.Tensor]] = []
        for i, block in enumerate(model.blocks):
            if block.ffn is not None and hasattr(block.ffn, "n_experts"):
                block.ffn.forward = self._wrap(i, block.ffn)

    def _wrap(self, layer, ffn):
        inner = ffn.forward

        def forward(x, ctx):
            from edgerag_b200.ops import kernels

            out = inner(x, ctx)
            n = x.shape[0]
            lists = ctx.buf("moe.lists", (kernels.moe_lists_ints(n, ffn.n_experts, ffn.top),), torch.int32)
            if self.steps:
                self.steps[-1][layer] = lists[: n * ffn.top].reshape(n, ffn.top).cpu().clone()
            return out

        return forward

    def new_step(self) -> None:
        self.steps.append({})

    def of_rows(self, picks: list[tuple[int, int, int]]) -> dict[int, torch.Tensor]:
        layers = self.steps[picks[0][0]].keys()
        return {layer: torch.cat([self.steps[s][layer][first: first + n] for s, first, n in picks]) for layer in layers}


def make_engine(folder, dtype, **over):
    from edgerag_b200.engine.engine import Engine, EngineOptions

    opts = dict(dtype=dtype, block_size=16, num_blocks=64, max_batch_size=4, max_step_tokens=512, max_model_len=1 << 20,
                cuda_graphs=False, poison_freed_pages=True)
    opts.update(over)
    eng = Engine.from_pretrained(folder, EngineOptions(**opts))
    eng.log = ChoiceLog(eng.model)
    return eng


def feed(runner, rid, tokens, cuts, log: ChoiceLog | None = None):
    from edgerag_b200.engine.step import StepEntry

    rows, pos, picks = [], 0, []
    for c in cuts:
        c = min(c, len(tokens) - pos)
        if c <= 0:
            break
        if log is not None:
            log.new_step()
            picks.append((len(log.steps) - 1, 0, c))
        out = runner.step([StepEntry(rid, tokens=tokens[pos: pos + c], want=list(range(c)))])
        rows.append(out.float().cpu().clone())
        pos += c
    assert pos == len(tokens), "the cuts do not cover the tokens"
    return torch.cat(rows), (log.of_rows(picks) if log is not None and log.steps and log.steps[picks[0][0]] else None)


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)


#: float32 (worst row, mean over rows): only the order of sums differs from the plain implementation.
#: bfloat16 (mean over rows, worst row): activations are rounded to 8 bits between the products.
BANDS = {"float32": (2e-4, 4e-5), "bfloat16": (2.5e-2, 0.12)}


def assert_close(got, want, dtype, what=""):
    assert torch.isfinite(got).all(), f"{what} {dtype}: non-finite logits"
    e = row_errors(got, want)
    where = f"{what} {dtype}: worst {e.max():.2e} (row {int(e.argmax())}), mean {e.mean():.2e}"
    worst, mean = (BANDS[dtype][0], BANDS[dtype][1]) if dtype == "float32" else (BANDS[dtype][1], BANDS[dtype][0])
    assert e.max() <= worst and e.mean() <= mean, where


def tokens_for(raw, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, raw["vocab"], (n,), generator=g).tolist()


def check_request(eng, raw, tensors, toks, cuts, dtype, what):
    eng.runner.admit(what)
    got, chosen = feed(eng.runner, what, toks, cuts, eng.log if dtype == "bfloat16" else None)
    eng.runner.release(what)
    want = plain.forward(tensors, raw, toks, chosen=chosen)
    assert_close(got, want, dtype, what)
    eng.cache.check_invariants()


# --- configuration, plan, plain mechanisms (CPU) ---------------------------------------------------

def test_plan_names_every_tensor_and_declares_pages_and_records():
    from edgerag_b200.config.registry import architecture_of
    from edgerag_b200.models.decoder import DecoderModel

    arch = architecture_of(FULL)
    cfg = arch.read_config(FULL, "test")
    model = DecoderModel(arch.make_plan(cfg), torch.float32, torch.device("cpu"))
    specs = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert specs.pop("head") == (FULL["vocab"], FULL["width"])            # tied to the embedding where absent
    assert specs == plain.tensor_shapes(FULL)
    groups = {(g.n_kv_heads, g.head_dim, g.window, g.v_head_dim): g.n_layers for g in model.cache_layout.groups}
    assert groups == {(2, 32, 21, 24): 1, (1, 32, 10, 0): 1, (3, 40, 40, 40): 1, (1, 44, 33, 0): 1, (1, 16, 17, 72): 1,
                      (2, 64, 0, 16): 1, (1, 32, 0, 0): 1}
    states = {s.name: tuple(s.shape) for s in model.cache_layout.states}
    assert states == {"qkv_conv@0": (2, 4 * 32 + 2 * 32 + 2 * 24), "qkv_conv@2": (1, 3 * 40 + 3 * 40 + 3 * 40)}   # one tap: no record
    assert model.graph_safe
    assert model.blocks[0].update_scale == 0.4 and model.head.scale == 1.7


def test_configuration_errors_name_the_key():
    from edgerag_b200.config.model_config import ConfigError
    from edgerag_b200.models.pudadra import PudadraConfig

    def broken(change):
        raw = copy.deepcopy(plain.make_config([ATT, LAT, ATT_B]))
        change(raw)
        return raw

    cases = [
        (lambda r: r["layers"][0].update(type="mamba"), "unknown layer type"),
        (lambda r: r["layers"][0]["mixer"].pop("kv_heads"), "kv_heads"),
        (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads must divide"),
        (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
        (lambda r: r["layers"][0]["mixer"]["mask"].pop("size"), "size"),
        (lambda r: r["layers"][0]["mixer"].pop("diff"), "diff"),
        (lambda r: r["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
        (lambda r: r["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
        (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
        (lambda r: r["layers"][1]["mlp"].update(kind="glu"), "mlp.kind"),
        (lambda r: r["layers"][1]["mlp"]["router"].update(top=9), "router.top"),
        (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(count=3), "router.groups"),
        (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(keep=1), "router.groups"),
        (lambda r: r["layers"][2]["mlp"]["expert"].pop("ff"), "ff"),
        (lambda r: r.pop("norm"), "norm"),
        (lambda r: r.pop("width"), "width"),
    ]
    for change, word in cases:
        with pytest.raises(ConfigError, match=word):
            PudadraConfig.from_dict(broken(change), "t")


def test_plain_window_against_its_definition():
    m = plain.window_mask(30, 7)
    for i in range(30):
        for j in range(30):
            assert bool(m[i, j]) == (0 <= i - j < 7)
    assert m[10, 4] and not m[10, 3] and m[10, 10] and not m[10, 11]
    assert plain.window_mask(9, 0).equal(torch.tril(torch.ones(9, 9, dtype=torch.bool)))


def test_frequencies_keep_short_waves_and_stretch_long_ones():
    from edgerag_b200.parts.rope import rotary_frequencies

    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 100}
    f0 = plain.rot_frequencies(1000.0, 16)
    f = plain.rot_frequencies(1000.0, 16, sc)
    wave = 2 * math.pi / f0
    assert f0[0] == 1.0 and torch.allclose(f0[3], torch.tensor(1000.0 ** (-6 / 16), dtype=torch.float64))
    kinds = set()
    for i in range(8):
        if wave[i] < 25:
            assert f[i] == f0[i]; kinds.add("kept")
        elif wave[i] > 100:
            assert torch.allclose(f[i], f0[i] / 8); kinds.add("stretched")
        else:
            s = (100 / wave[i] - 1.0) / 3.0
            assert torch.allclose(f[i], (1 - s) * f0[i] / 8 + s * f0[i]) and f0[i] / 8 < f[i] < f0[i]; kinds.add("between")
    assert kinds == {"kept", "stretched", "between"}
    assert torch.allclose(rotary_frequencies(1000.0, 16, sc), f, rtol=1e-14, atol=0) and torch.equal(rotary_frequencies(1000.0, 16), f0)


def test_plain_rotations_pair_the_right_entries():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 2, 10, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 3, 8, 21])
    f = plain.rot_frequencies(100.0, 6)
    y, z = plain.rotate_halves(x, pos, f), plain.rotate_pairs(x, pos, f)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(z[..., 6:], x[..., 6:]) and torch.allclose(y[0], x[0])
    a = 21 * 100.0 ** (-2.0 / 6)
    assert torch.allclose(y[3, 1, 1], x[3, 1, 1] * math.cos(a) - x[3, 1, 4] * math.sin(a))       # halves: 1 with 4
    assert torch.allclose(y[3, 1, 4], x[3, 1, 4] * math.cos(a) + x[3, 1, 1] * math.sin(a))
    assert torch.allclose(z[3, 1, 2], x[3, 1, 2] * math.cos(a) - x[3, 1, 3] * math.sin(a))       # pairs: 2 with 3
    assert torch.allclose(z[3, 1, 3], x[3, 1, 3] * math.cos(a) + x[3, 1, 2] * math.sin(a))


def test_plain_convolution_is_causal_and_starts_from_zeros():
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    assert torch.allclose(plain.causal_conv(x, torch.tensor([[0.0, 0.0, 1.0]], dtype=torch.float64)), x)
    assert torch.allclose(plain.causal_conv(x, torch.tensor([[2.0, 0.0, 0.0]], dtype=torch.float64))[:, 0],
                          torch.tensor([0.0, 0.0, 2.0, 4.0, 6.0], dtype=torch.float64))


def test_plain_router_keeps_the_best_groups_and_does_not_renormalise():
    w = torch.zeros(6, 6, dtype=torch.float64)
    h = torch.tensor([[5.0, 1.0, 4.0, 3.9, 3.0, 2.9]], dtype=torch.float64)
    chosen, weight = plain.routed_choice(h, torch.eye(6, dtype=torch.float64), {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}})
    s = torch.softmax(h, -1)
    # groups (0,1) (2,3) (4,5) score 5, 4, 3: the last is out, so the third choice is expert 1, not 4
    assert chosen.tolist() == [[0, 2, 3]] and torch.allclose(weight, s[:, [0, 2, 3]]) and float(weight.sum()) < 1.0
    chosen, _ = plain.routed_choice(h, torch.eye(6, dtype=torch.float64), {"experts": 6, "top": 3})
    assert chosen.tolist() == [[0, 2, 3]]
    chosen, _ = plain.routed_choice(h, torch.eye(6, dtype=torch.float64), {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert chosen.tolist() == [[0, 1]]


def test_plain_difference_of_maps_by_hand():
    """One head, two tokens, no rotation or window: the second token's output from the two softmaxes by hand."""
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 2, "diff": 0.5, "scale": 1.0, "softcap": 0.0}
    w = {"p.q": torch.tensor([[1.0], [2.0]]), "p.k": torch.tensor([[1.0], [1.0]]), "p.v": torch.tensor([[1.0], [-1.0]]),
         "p.o": torch.eye(2), "p.lq1": torch.tensor([0.0]), "p.lk1": torch.tensor([0.0]), "p.lq2": torch.tensor([1.0]),
         "p.lk2": torch.tensor([math.log(0.5)])}
    h = torch.tensor([[1.0], [3.0]], dtype=torch.float64)
    lam = 1.0 - 0.5 + 0.5
    assert math.isclose(plain.diff_lambda(w, "p.", 0.5), lam)
    out = plain.diff_attention_mixer(h, w, "p.", m, 0.0)
    p1, p2 = torch.softmax(torch.tensor([3.0, 9.0], dtype=torch.float64), 0), torch.softmax(torch.tensor([6.0, 18.0], dtype=torch.float64), 0)
    v = torch.tensor([[1.0, -1.0], [3.0, -3.0]], dtype=torch.float64)
    o = p1 @ v - lam * (p2 @ v)
    assert torch.allclose(out[1], o / o.pow(2).mean().sqrt() * 0.5)


# --- every mechanism alone ------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_one_mechanism_alone(name, dtype, folders):
    folder, raw, tensors = folders(name, ALONE[name], seed=11)
    toks = tokens_for(raw, 75, 5)
    eng = make_engine(folder, dtype)
    check_request(eng, raw, tensors, toks, [75], dtype, f"{name} whole")
    check_request(eng, raw, tensors, toks, [17, 2, 1, 1, 16, 3, 1, 1, 1, 2, 20, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1], dtype, f"{name} in portions")


@pytest.mark.gpu
def test_layers_agree_with_plain_one_by_one(folders):
    """The residual stream after every layer (float32), with the pending update added."""
    from edgerag_b200.engine.step import StepEntry
    from edgerag_b200.parts.base import settle_update

    folder, raw, tensors = folders("full", FULL, seed=1)
    toks = tokens_for(raw, 50, 2)
    want: list = []
    plain.forward(tensors, raw, toks, layers_out=want)
    eng = make_engine(folder, "float32")
    r, model = eng.runner, eng.model
    r.admit("x")
    r.pools.zero_slots(r.cache.drain_new_slots())
    ctx, ordered = r.prepare([StepEntry("x", tokens=toks, want=[])])
    hidden = ctx.buf("model.hidden", (len(toks), model.hidden_size), torch.float32)
    model.embedding.forward(ctx, hidden)
    delta = None
    for run, call in enumerate(model.schedule):
        delta = model.blocks[call.layer].forward(hidden, delta, ctx, call)
        settle_update(hidden, delta, model.dtype)
        delta = None
        err = (hidden.cpu().double() - want[run]).abs().max() / want[run].abs().max()
        assert err < 2e-5, f"layer {call.layer}: {err:.2e}"
    r.finish(ordered)


# --- the whole model: prompts, decoding, portions, batches ------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_decoding_and_portions_agree_with_plain(dtype, folders):
    folder, raw, tensors = folders("full", FULL, seed=1)
    toks = tokens_for(raw, 150, 6)
    eng = make_engine(folder, dtype)
    for rid, cuts in (("whole", [150]), ("decode", [40] + [1] * 110), ("portions", [2, 31, 2, 16, 15, 1, 2, 33, 3, 2, 2, 17] + [1] * 30),
                      ("pairs", [2] * 75)):
        check_request(eng, raw, tensors, toks, cuts, dtype, rid)


@pytest.mark.gpu
@pytest.mark.parametrize("page", [4, 64])
def test_other_page_sizes(page, folders):
    folder, raw, tensors = folders("full", FULL, seed=1)
    toks = tokens_for(raw, 90, 8)
    eng = make_engine(folder, "float32", block_size=page, num_blocks=256 // page)
    check_request(eng, raw, tensors, toks, [33, 2, 1, 1, 19] + [1] * 34, "float32", f"pages of {page}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_equal_each_alone(dtype, folders):
    """Portions of some requests beside single tokens of others; a request pauses for a step; requests end and their
    pages and state slots go to new ones (four slots, six requests, freed pages poisoned).  A slot that is used again
    must start from zeros: a convolution's record left behind by the request before shows in the first rows."""
    from edgerag_b200.engine.step import StepEntry

    folder, raw, tensors = folders("full", FULL, seed=1)
    lens = {"a": 70, "b": 33, "c": 1, "d": 90, "e": 18, "f": 47}
    toks = {k: tokens_for(raw, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    eng = make_engine(folder, dtype, num_blocks=14)       # 224 tokens of pages: never room for all at once
    r = eng.runner
    plan = [
        [("a", 30), ("b", 2)], [("a", 1), ("b", 16), ("c", 1)], [("a", 17), ("b", 1)], [("b", 14), ("d", 40), ("a", 1)],
        [("a", 21), ("d", 1)], [("d", 33), ("e", 2)], [("d", 16), ("e", 1), ("f", 3)], [("e", 15), ("f", 1)], [("f", 43)],
    ]
    fed = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    picks = {k: [] for k in lens}
    slots_seen = {}
    for step in plan:
        entries = []
        for rid, n in step:
            if fed[rid] == 0:
                r.admit(rid)
                slots_seen[rid] = eng.cache.requests[rid].slot
            entries.append(StepEntry(rid, tokens=toks[rid][fed[rid]: fed[rid] + n], want=list(range(n))))
        eng.log.new_step()
        first_row, row = {}, 0                               # the runner puts single tokens first: every entry's rows in the step
        for rid, n in sorted(step, key=lambda e: e[1] != 1):
            first_row[rid] = row
            row += n
        out = r.step(entries).float().cpu()
        row = 0
        for rid, n in step:
            got[rid].append(out[row: row + n].clone())
            picks[rid].append((len(eng.log.steps) - 1, first_row[rid], n))
            row += n
            fed[rid] += n
            if fed[rid] == lens[rid]:
                r.release(rid)
        eng.cache.check_invariants()
    assert fed == lens
    assert len(set(slots_seen.values())) < len(lens), "no state slot was used twice"
    for rid in lens:
        chosen = eng.log.of_rows(picks[rid]) if dtype == "bfloat16" else None
        assert_close(torch.cat(got[rid]), plain.forward(tensors, raw, toks[rid], chosen=chosen), dtype, f"request {rid}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_while_windows_pass_over_decoded_tokens(dtype, folders):
    folder, raw, tensors = folders("full", FULL, seed=1)
    toks = tokens_for(raw, 260, 9)
    eng = make_engine(folder, dtype)
    check_request(eng, raw, tensors, toks, [3] + [1] * 257, dtype, "260 tokens, 257 of them one by one")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_sizes_of_a_larger_model(dtype, folders):
    """Maps of 64 with values of 128, windows longer than a split of keys, a prompt of several windows, more experts'
    rows than a tile: the sizes at which single tokens are cut into splits and the experts' products take the tensor cores."""
    raw = plain.make_config([
        plain.attention_layer(heads=4, kv_heads=2, dim=64, vdim=128, conv=4, diff=0.6, window=600, rot_dims=32, softcap=30.0,
                              base=300000.0, scaling={"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256},
                              mlp=plain.moe_mlp(ff=64, experts=8, top=2, groups=(4, 3), shared=128)),
        plain.latent_layer(heads=4, dim=32, rot_dim=32, vdim=32, kv_rank=64, window=256, mlp=plain.dense_mlp(256)),
        plain.attention_layer(heads=2, kv_heads=1, dim=32, vdim=192, conv=2, diff=0.3, window=0, rot_dims=32, softcap=0.0, mlp=None)],
        width=128, vocab=96)
    folder, raw, tensors = folders("larger", raw, seed=3)
    toks = tokens_for(raw, 1300, 9)
    eng = make_engine(folder, dtype, num_blocks=256, max_step_tokens=2048)
    check_request(eng, raw, tensors, toks, [1300], dtype, "whole")
    check_request(eng, raw, tensors, toks, [590, 2, 9, 257, 400, 30] + [1] * 12, dtype, "portions")
    check_request(eng, raw, tensors, toks[:700], [598] + [1] * 102, dtype, "decoding over a window's edge")


# --- kernels with inputs made so that a fault shows ---------------------------------------------------

def _paged(rows, page_size, dtype, shuffle_seed=0):
    """Scatter each sequence's rows [len, G, d] over shuffled pages; unused slots hold NaN.  (pages [P, G, page, d], tables)."""
    G, d = rows[0].shape[1:]
    need = [-(-r.shape[0] // page_size) for r in rows]
    order = torch.randperm(sum(need) + 3, generator=torch.Generator().manual_seed(shuffle_seed)).tolist()
    pages = torch.full((sum(need) + 3, G, page_size, d), float("nan"), dtype=torch.float64)
    tables = torch.zeros(len(rows), max(need), dtype=torch.int32)
    for s, r in enumerate(rows):
        for i in range(need[s]):
            page = order.pop()
            tables[s, i] = page
            part = r[i * page_size: (i + 1) * page_size]
            pages[page, :, : part.shape[0]] = part.transpose(0, 1)
    return pages.to(dtype).cuda(), tables.cuda()


def _diff_reference(q, keys, values, where, scale, window, cap, lam, eps, out_scale, rep):
    """q [n, H, 2, d]; keys[seq] [len, G, 2, d]; values[seq] [len, G, dv]; where[t] = (sequence, position)."""
    out = torch.zeros(q.shape[0], q.shape[1], values[0].shape[-1], dtype=torch.float64)
    for t, (seq, pos) in enumerate(where):
        see = [j for j in range(pos + 1) if not window or pos - j < window]
        for h in range(q.shape[1]):
            maps = []
            for m in range(2):
                s = keys[seq][see, h // rep, m] @ q[t, h, m] * scale
                if cap > 0:
                    s = cap * torch.tanh(s / cap)
                maps.append(torch.softmax(s, 0) @ values[seq][see, h // rep])
            o = maps[0] - lam * maps[1]
            out[t, h] = o / torch.sqrt(o.pow(2).mean() + eps) * out_scale
    return out


DIFF_CASES = [  # (heads, kv heads, map size, value size, page, window)
    (4, 2, 16, 24, 16, 24), (6, 1, 24, 72, 8, 17), (2, 2, 64, 128, 16, 64), (3, 3, 8, 10, 16, 9), (4, 2, 12, 25, 16, 1),
    (4, 1, 32, 64, 32, 130), (2, 1, 48, 96, 16, 0), (8, 2, 64, 200, 64, 100), (4, 2, 80, 40, 16, 70), (2, 2, 16, 8, 4, 33),
    (4, 1, 128, 128, 16, 200), (12, 1, 16, 32, 16, 40), (24, 1, 16, 16, 16, 30), (8, 1, 32, 64, 16, 90),
]


def _dominant_queries(case, lens, seed):
    """Queries whose first map looks for one key and whose second map looks for another: just inside and just outside the
    window, at a page's last and first slot, far back, at position 0 and at their own."""
    H, G, d, dv, page, window = case
    g = torch.Generator().manual_seed(seed)
    keys = [torch.randn(n, G, 2, d, generator=g, dtype=torch.float64) * 0.3 for n in lens]
    values = [torch.randn(n, G, dv, generator=g, dtype=torch.float64) for n in lens]
    w = window or 50
    queries, where = [], []
    for s, n in enumerate(lens):
        for pos in sorted({n - 1, n - 2, w, w - 1, w + 1, 2 * w, page - 1, page, 2 * page, 0, 1, n // 2}):
            if not 0 <= pos < n:
                continue
            first = pos - w + 1
            for target in (first, first - 1, first + 1, (pos // page) * page - 1, (pos // page) * page, 0, 1, pos, pos - 1):
                if 0 <= target <= pos:
                    q = torch.randn(H, 2, d, generator=g, dtype=torch.float64) * 0.3
                    other = max(0, min(pos, 2 * first - target))         # the second map looks to the other side of the edge
                    for h in range(H):
                        for m, tg in ((0, target), (1, other)):
                            kk = keys[s][tg, h // (H // G), m]
                            q[h, m] += 12.0 * kk / kk.norm() ** 2
                    queries.append(q)
                    where.append((s, pos))
    return torch.stack(queries), keys, values, where


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", DIFF_CASES)
def test_differential_attention_with_keys_made_dominant(case, dtype):
    """A kernel that reads a key behind the window, skips the window's first key or stops at a page's border returns
    another value row.  Rows of prompts in one walk, and single tokens in splits of two sizes."""
    from edgerag_b200.ops import kernels as k

    H, G, d, dv, page, window = case
    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    lens = [150, 77, 2 * (window or 50) + 3, 300]
    q, keys, values, where = _dominant_queries(case, lens, H * 100 + d + window)
    if dtype == "bfloat16":
        q, keys, values = q.to(tdt).double(), [x.to(tdt).double() for x in keys], [x.to(tdt).double() for x in values]
    lam, eps, out_scale, cap = 0.55, 1e-6, 0.7, 6.0
    want = _diff_reference(q, keys, values, where, 0.5, window, cap, lam, eps, out_scale, H // G)
    other = _diff_reference(q, keys, values, where, 0.5, window + 1 if window else 40, cap, lam, eps, out_scale, H // G)
    assert (want - other).abs().max() > 0.2, "the inputs do not tell a window from one that is a key longer"
    k_pages, tables = _paged([x.reshape(x.shape[0], G, 2 * d) for x in keys], page, tdt, 1)
    v_pages, tables_v = _paged(values, page, tdt, 1)
    assert torch.equal(tables, tables_v)
    n = len(where)
    seq = torch.tensor([s for s, _ in where], dtype=torch.int32).cuda()
    pos = torch.tensor([p for _, p in where], dtype=torch.int32).cuda()
    qd = q.reshape(n, H * 2 * d).to(tdt).cuda().contiguous()
    tol = 2e-5 if dtype == "float32" else 3e-2
    out = torch.empty(n, H * dv, dtype=tdt, device="cuda")
    k.diff_attention(qd, k_pages, v_pages, tables, seq, pos, out, H, 0.5, lam, eps, out_scale, 0, n, window=window, softcap=cap)
    assert (out.double().cpu().view(n, H, dv) - want).abs().max() < tol, "rows in one walk"
    for split in (64, 16):
        n_splits = -(-max(lens) // split) if not window else min(-(-max(lens) // split), (window - 1) // split + 2)
        part = torch.full((n * H * n_splits * k.diff_part_floats(dv),), float("nan"), dtype=torch.float32, device="cuda")
        out.fill_(float("nan"))
        k.diff_attention(qd, k_pages, v_pages, tables, seq, pos, out, H, 0.5, lam, eps, out_scale, 0, n, window=window, softcap=cap,
                         split_keys=split, n_splits=n_splits, part=part)
        assert (out.double().cpu().view(n, H, dv) - want).abs().max() < tol, f"splits of {split}"
    if k.diff_mma_supported(tdt, d, dv):
        # the tensor-core form takes whole portions: every sequence's last tokens as the step's rows, each looking for a key
        new = [70, 1, (window or 50) + 2, 129]
        g2 = torch.Generator().manual_seed(5)
        qs, wh = [], []
        for s_, n_ in enumerate(lens):
            for i, p_ in enumerate(range(n_ - new[s_], n_)):
                first = p_ - (window or 50) + 1
                target = max(0, min(p_, [first, first - 1, p_, (p_ // page) * page - 1, (p_ // page) * page, 0, first + 1][i % 7]))
                other_t = max(0, min(p_, 2 * first - target))
                qq = torch.randn(H, 2, d, generator=g2, dtype=torch.float64) * 0.3
                for h in range(H):
                    for m_, tg in ((0, target), (1, other_t)):
                        kk = keys[s_][tg, h // (H // G), m_]
                        qq[h, m_] += 12.0 * kk / kk.norm() ** 2
                qs.append(qq.to(tdt).double())
                wh.append((s_, p_))
        q2 = torch.stack(qs)
        want2 = _diff_reference(q2, keys, values, wh, 0.5, window, cap, lam, eps, out_scale, H // G)
        starts = torch.tensor([0] + list(np.cumsum(new)), dtype=torch.int32).cuda()
        pos2 = torch.tensor([p_ for _, p_ in wh], dtype=torch.int32).cuda()
        out2 = torch.full((len(wh), H * dv), float("nan"), dtype=tdt, device="cuda")
        q2d = q2.reshape(len(wh), -1).to(tdt).cuda().contiguous()
        k.diff_attention_mma(q2d, k_pages, v_pages, tables, starts, pos2, out2, H, 0.5, lam, eps, out_scale, 0, len(lens), 0, len(wh),
                             k.diff_mma_tiles(new, H // G), window=window, softcap=cap)
        assert (out2.double().cpu().view(len(wh), H, dv) - want2).abs().max() < tol, "tensor cores, portions"
        # single tokens: the last token of every sequence as a step of its own, in splits of two sizes
        last = [int(starts[i + 1]) - 1 for i in range(len(lens))]
        q1, pos1 = q2d[last].contiguous(), pos2[last].contiguous()
        starts1 = torch.arange(len(lens) + 1, dtype=torch.int32).cuda()
        for split in (64, 128):
            n_splits = -(-max(lens) // split) if not window else min(-(-max(lens) // split), (window - 1) // split + 2)
            part = torch.full((len(last) * H * n_splits * k.diff_part_floats(dv),), float("nan"), dtype=torch.float32, device="cuda")
            out1 = torch.full((len(last), H * dv), float("nan"), dtype=tdt, device="cuda")
            for rows in ((8, 16, 64) if H // G <= 8 else (16, 64)):
                out1.fill_(float("nan"))
                k.diff_attention_mma(q1, k_pages, v_pages, tables, starts1, pos1, out1, H, 0.5, lam, eps, out_scale, 0, len(lens), 0,
                                     len(last), k.diff_mma_tiles([1] * len(last), H // G, rows), window=window, softcap=cap,
                                     split_keys=split, n_splits=n_splits, part=part if n_splits > 1 else None, tile_rows=rows)
                assert (out1.double().cpu().view(len(last), H, dv) - want2[last]).abs().max() < tol, \
                    f"tensor cores, single tokens, splits of {split}, tiles of {rows} rows"
    # a range of rows in the middle of the batch leaves the others alone
    out.fill_(7.0)
    k.diff_attention(qd, k_pages, v_pages, tables, seq, pos, out, H, 0.5, lam, eps, out_scale, 5, n - 9, window=window, softcap=cap)
    got = out.double().cpu().view(n, H, dv)
    assert (got[5: n - 4] - want[5: n - 4]).abs().max() < tol and bool((got[:5] == 7).all()) and bool((got[n - 4:] == 7).all())


LATENT_CASES = [  # (heads, latent, rotated part, page, window)
    (4, 32, 16, 16, 24), (16, 64, 32, 16, 100), (3, 24, 8, 8, 9), (8, 128, 64, 32, 130), (5, 40, 8, 16, 1), (20, 64, 32, 16, 70),
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", LATENT_CASES)
def test_latent_attention_under_a_window_with_one_row_made_dominant(case, dtype):
    """The latent attention's kernels (general, and on tensor cores in bfloat16) under a window: rows of portions and
    single tokens in splits, each query looking for one cache row at the window's edge, a page's border or far back."""
    from edgerag_b200.ops import kernels as k

    H, R, dr, page, window = case
    Dk = R + dr
    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    g = torch.Generator().manual_seed(H + R + window)
    lens = [150, 77, 2 * window + 3, 300]
    rows = [(torch.randn(n, 1, Dk, generator=g, dtype=torch.float64) * 0.3).to(tdt).double() for n in lens]
    # portions: every sequence's last `new` tokens are the step's rows, in order (the tensor-core form takes whole portions)
    new = [40, 1, window + 2, 17]
    q_rows, where = [], []
    for s, n in enumerate(lens):
        for i, pos in enumerate(range(n - new[s], n)):
            first = pos - window + 1
            target = [first, first - 1, pos, (pos // page) * page - 1, (pos // page) * page, 0, first + 1][i % 7]
            target = max(0, min(pos, target))
            q = torch.randn(H, Dk, generator=g, dtype=torch.float64) * 0.3
            q += 12.0 * rows[s][target, 0] / rows[s][target, 0].norm() ** 2
            q_rows.append(q)
            where.append((s, pos))
    q = torch.stack(q_rows)

    def reference(win):
        out = torch.zeros(len(where), H, R, dtype=torch.float64)
        for t, (s, pos) in enumerate(where):
            see = [j for j in range(pos + 1) if pos - j < win]
            for h in range(H):
                out[t, h] = torch.softmax(rows[s][see, 0] @ q[t, h] * 0.5, 0) @ rows[s][see, 0, :R]
        return out

    want = reference(window)
    assert (want - reference(window + 1)).abs().max() > 0.1
    pages, tables = _paged(rows, page, tdt, 2)
    n = len(where)
    seq = torch.tensor([s for s, _ in where], dtype=torch.int32).cuda()
    pos = torch.tensor([p for _, p in where], dtype=torch.int32).cuda()
    starts = torch.tensor([0] + list(np.cumsum(new)), dtype=torch.int32).cuda()
    ql = q.float().cuda().contiguous()
    tol = 2e-5 if dtype == "float32" else 3e-2
    out = torch.empty(n, H, R, dtype=tdt, device="cuda")
    k.latent_attention(ql, pages, tables, seq, pos, out, 0.5, 0, n, window=window)
    assert (out.double().cpu() - want).abs().max() < tol, "general kernel, one walk"
    for split in (64, 128):
        n_splits = min(-(-max(lens) // split), (window - 1) // split + 2)
        part = torch.full((k.latent_scratch_floats(n, H, R, n_splits),), float("nan"), dtype=torch.float32, device="cuda")
        out.fill_(float("nan"))
        k.latent_attention(ql, pages, tables, seq, pos, out, 0.5, 0, n, window=window, split_keys=split, n_splits=n_splits, part=part)
        assert (out.double().cpu() - want).abs().max() < tol, f"general kernel, splits of {split}"
    if k.latent_mma_supported(tdt, R, dr):
        out.fill_(float("nan"))
        tiles = k.latent_mma_tiles(new, H, 2)
        k.latent_attention_mma(ql, pages, tables, starts, pos, out, 0.5, 0, len(lens), 0, n, tiles, 2, window=window)
        assert (out.double().cpu() - want).abs().max() < tol, "tensor cores, portions"
        # single tokens: the last token of every sequence as a step of its own, in splits
        last = [int(starts[s + 1]) - 1 for s in range(len(lens))]
        ql1 = ql[last].contiguous()
        pos1 = pos[last].contiguous()
        starts1 = torch.arange(len(lens) + 1, dtype=torch.int32).cuda()
        mt = 1 if H <= 16 else 2
        for split in (64, 128):
            n_splits = min(-(-max(lens) // split), (window - 1) // split + 2)
            part = torch.full((k.latent_scratch_floats(len(last), H, R, n_splits),), float("nan"), dtype=torch.float32, device="cuda")
            out1 = torch.full((len(last), H, R), float("nan"), dtype=tdt, device="cuda")
            k.latent_attention_mma(ql1, pages, tables, starts1, pos1, out1, 0.5, 0, len(lens), 0, len(last),
                                   k.latent_mma_tiles([1] * len(last), H, mt), mt, window=window, split_keys=split, n_splits=n_splits,
                                   part=part if n_splits > 1 else None)
            assert (out1.double().cpu() - want[last]).abs().max() < tol, f"tensor cores, single tokens, splits of {split}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2, 1, 8, 12, 3, 4, 16), (3, 3, 16, 40, 4, 16, 8), (4, 2, 24, 24, 2, 0, 16), (2, 2, 8, 8, 1, 8, 4)])
def test_prepare_convolves_from_the_record_rotates_and_writes_the_cache(sizes, dtype):
    """Two requests in portions: the convolution's inputs before a portion come from the request's record (which another
    request's slot beside it must not touch), the maps' halves are turned by the true positions, and keys and values land in
    the tokens' cache slots."""
    from edgerag_b200.ops import kernels as k

    H, G, d, dv, taps, rot, page = sizes
    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    g = torch.Generator().manual_seed(sum(sizes))
    C = (H + G) * 2 * d + G * dv
    ld = -(-C // 8) * 8
    lens = {0: 23, 1: 9}
    proj = {s: (torch.randn(n, ld, generator=g, dtype=torch.float64)).to(tdt).double() for s, n in lens.items()}
    conv_w = torch.randn(C, taps, generator=g, dtype=torch.float64).float().double()
    freq = plain.rot_frequencies(300.0, rot) if rot else None
    want_q, want_k, want_v = {}, {}, {}
    for s, n in lens.items():
        y = plain.causal_conv(proj[s][:, :C], conv_w)
        qq, kk = y[:, : H * 2 * d].reshape(n, H, 2, d), y[:, H * 2 * d: (H + G) * 2 * d].reshape(n, G, 2, d)
        if rot:
            qq, kk = plain.rotate_halves(qq, torch.arange(n), freq), plain.rotate_halves(kk, torch.arange(n), freq)
        want_q[s], want_k[s], want_v[s] = qq.reshape(n, -1), kk.reshape(n, G, 2 * d), y[:, (H + G) * 2 * d:].reshape(n, G, dv)
    n_pages = 8
    k_pages = torch.full((n_pages, G, page, 2 * d), float("nan"), dtype=tdt, device="cuda")
    v_pages = torch.full((n_pages, G, page, dv), float("nan"), dtype=tdt, device="cuda")
    state = torch.zeros(4, max(taps - 1, 1), C, dtype=torch.float32, device="cuda")[:, : taps - 1].contiguous() if taps > 1 else None
    if state is not None:
        state[1].fill_(float("nan"))            # a slot nobody uses
    slot_of, page_of = {0: 3, 1: 0}, {0: [5, 1, 6, 2, 7, 0][: -(-23 // page)], 1: [4, 3][: -(-9 // page)]}
    if page == 4:
        k_pages = torch.full((16, G, page, 2 * d), float("nan"), dtype=tdt, device="cuda")
        v_pages = torch.full((16, G, page, dv), float("nan"), dtype=tdt, device="cuda")
        page_of = {0: [5, 1, 6, 2, 7, 0], 1: [4, 3, 9]}
    fed = {0: 0, 1: 0}
    inv = freq.float().cuda() if rot else None
    for step in ([(0, 5), (1, 2)], [(1, 1), (0, 1)], [(0, 2), (1, 6)], [(0, 15)]):
        rows = torch.cat([proj[s][fed[s]: fed[s] + n] for s, n in step]).to(tdt).cuda().contiguous()
        total = rows.shape[0]
        seq_of = torch.tensor([i for i, (_, n) in enumerate(step) for _ in range(n)], dtype=torch.int32).cuda()
        starts = torch.tensor([0] + list(np.cumsum([n for _, n in step])), dtype=torch.int32).cuda()
        st_slots = torch.tensor([slot_of[s] for s, _ in step], dtype=torch.int32).cuda()
        posl = [p for s, n in step for p in range(fed[s], fed[s] + n)]
        slots = torch.tensor([page_of[s][p // page] * page + p % page for s, n in step for p in range(fed[s], fed[s] + n)],
                             dtype=torch.int32).cuda()
        q_out = torch.full((total, H * 2 * d), float("nan"), dtype=tdt, device="cuda")
        k.diff_prepare(rows, q_out, torch.tensor(posl, dtype=torch.int32).cuda(), H, G, d, dv, inv_freq=inv, rot_dims=rot,
                       conv_w=conv_w.float().cuda(), conv_state=state, seq_of_token=seq_of, seq_starts=starts, state_slots=st_slots,
                       slots=slots, k_pages=k_pages, v_pages=v_pages, page_size=page)
        if state is not None:
            k.conv_state_update(rows, 0, state, len(step), starts, st_slots)
        tol = 1e-5 if dtype == "float32" else 4e-2
        row = 0
        for s, n in step:
            assert (q_out[row: row + n].double().cpu() - want_q[s][fed[s]: fed[s] + n]).abs().max() < tol, (step, s)
            row += n
            fed[s] += n
    tol = 1e-5 if dtype == "float32" else 4e-2
    for s, n in lens.items():
        for p in range(n):
            pg, off = page_of[s][p // page], p % page
            assert (k_pages[pg, :, off].double().cpu() - want_k[s][p]).abs().max() < tol
            assert (v_pages[pg, :, off].double().cpu() - want_v[s][p]).abs().max() < tol
    if state is not None:
        assert torch.isnan(state[1]).all(), "a record of another slot was written"
        assert torch.allclose(state[3].double().cpu(), proj[0][23 - (taps - 1): 23, :C], atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(12, 4, (4, 3), 64), (6, 2, (3, 2), 40), (8, 3, None, 96), (16, 1, (8, 1), 128), (5, 5, (5, 5), 24),
                                   (64, 6, (8, 4), 256)])
def test_router_with_groups_and_both_product_paths(sizes, dtype):
    """Choices and weights against the plain router (inputs without close calls); the lists; the experts' products with
    the weight on the output, on the general kernels and (bfloat16) the tensor cores, for few and for many rows."""
    from edgerag_b200.ops import kernels as k

    E, top, groups, width = sizes
    ff = 24
    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    g = torch.Generator().manual_seed(E * 7 + top)
    router = {"experts": E, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    w_router = (torch.randn(E, width, generator=g) * 3.0 / math.sqrt(width)).float()
    w_up = (torch.randn(E, ff, width, generator=g) / math.sqrt(width)).to(tdt)
    w_down = (torch.randn(E, width, ff, generator=g) / math.sqrt(ff)).to(tdt)
    for n in (5, 200):
        x = torch.randn(n, width, generator=g).to(tdt)
        z = x.double() @ w_router.double().T
        chosen, weight = plain.routed_choice(x.double(), w_router, router)
        # leave out the rows with a close call between a chosen and an unchosen expert or group
        s = torch.softmax(z, -1)
        clear = torch.ones(n, dtype=torch.bool)
        for t in range(n):
            vals = torch.sort(z[t], descending=True).values
            if (vals[:-1] - vals[1:]).min() < 1e-3:
                clear[t] = False
        lists = torch.zeros(k.moe_lists_ints(n, E, top), dtype=torch.int32, device="cuda")
        score = torch.zeros(n * top, dtype=torch.float32, device="cuda")
        tc = k.moe_tc_supported(tdt, width, ff)
        tile_rows = k.moe_tc_tile_rows(n, E, top) if tc else 0
        k.moe_route(x.cuda(), w_router.cuda(), top, lists, score, tile_rows, scores="softmax", groups=groups)
        got_c = lists[: n * top].reshape(n, top).cpu()
        got_s = score.reshape(n, top).cpu()
        assert torch.equal(got_c[clear].long(), chosen[clear]), "choices"
        assert torch.allclose(got_s[clear].double(), weight[clear], rtol=2e-5, atol=1e-7), "weights are the softmax scores themselves"
        # the update from the engine's own choices
        want = torch.zeros(n, width, dtype=torch.float64)
        for t in range(n):
            for c in range(top):
                e = int(got_c[t, c])
                a = torch.relu(x[t].double() @ w_up[e].double().T) ** 2
                if dtype == "bfloat16":
                    a = a.to(tdt).double()
                want[t] += float(got_s[t, c]) * (a @ w_down[e].double().T)
        act = torch.empty(n * top, ff, dtype=tdt, device="cuda")
        parts = torch.full((top, n, width), float("nan"), dtype=torch.float32, device="cuda")
        if tc:
            xs = torch.empty(n * top, width, dtype=tdt, device="cuda")
            k.moe_tc_gather(x.cuda(), lists, None, E, top, xs)
            k.moe_tc_up_act(xs, w_up.cuda(), lists, top, tile_rows, act)
            k.moe_tc_down(act, w_down.cuda(), lists, top, tile_rows, parts, out_score=score)
            tol = 2e-2 * float(want.abs().max())
            assert (parts.sum(0).double().cpu() - want).abs().max() < tol, "tensor cores"
            k.moe_route(x.cuda(), w_router.cuda(), top, lists, score, scores="softmax", groups=groups)
            parts.fill_(float("nan"))
        k.moe_up_act(x.cuda(), w_up.cuda(), lists, top, act)
        k.moe_down(act, w_down.cuda(), lists, top, parts, out_score=score)
        tol = (2e-5 if dtype == "float32" else 2e-2) * float(want.abs().max())
        assert (parts.sum(0).double().cpu() - want).abs().max() < tol, "general kernels"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_activations_scaled_updates_and_scaled_logits(dtype):
    from edgerag_b200.ops import kernels as k

    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(7, 48, generator=g) * 2).to(tdt)
    tol = 1e-6 if dtype == "float32" else 2e-2
    out = torch.empty(7, 41, dtype=tdt, device="cuda")
    k.act_rows(x.cuda(), out, "gelu_erf")
    assert (out.double().cpu() - plain.gelu_erf(x.double()[:, :41])).abs().max() < tol
    k.act_rows(x.cuda(), out, "relu_squared", gate_col=41)
    want = plain.relu_squared(x.double()[:, :41]) * torch.sigmoid(x.double()[:, 41:42])
    assert (out.double().cpu() - want).abs().max() < tol * 8
    # hidden += m * delta inside the norm's kernel, rows and partial sums; and with no norm after
    hidden = torch.randn(5, 64, generator=g)
    delta = torch.randn(5, 64, generator=g).to(tdt)
    parts = torch.randn(3, 5, 64, generator=g)
    weight = torch.rand(64, generator=g) + 0.5
    for d_in, d_ref in ((delta.cuda(), delta.double()), (parts.cuda(), parts.sum(0).to(tdt).double())):
        h = hidden.clone().cuda()
        y = torch.empty(5, 64, dtype=tdt, device="cuda")
        k.add_rmsnorm(h, weight.cuda(), y, 1e-5, delta=d_in, exact=True, delta_scale=0.3)
        ref = hidden.double() + 0.3 * d_ref
        assert (h.double().cpu() - ref).abs().max() < 1e-6
        assert (y.double().cpu() - plain.rms_unit(ref, 1e-5) * weight.double()).abs().max() < tol * 4
        h = hidden.clone().cuda()
        k.residual_add(h, d_in, tdt, scale=0.3)
        assert (h.double().cpu() - ref).abs().max() < 1e-6
    logits = torch.randn(3, 16, generator=g).cuda()[:, :13]
    before = logits.clone()
    k.scale_rows(logits, 2.5, tdt)
    assert torch.allclose(logits, before * 2.5)


# --- models whose weights make a fault show -----------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_whose_scores_single_out_keys_at_the_windows_edge(dtype, folders):
    """Queries and keys scaled up (the cap then decides the largest scores) so that single keys carry a row: the plain
    model with a window one shorter or one longer gives clearly other logits, the engine must give these."""
    layers = [plain.attention_layer(heads=2, kv_heads=1, dim=16, vdim=32, conv=2, diff=0.3, window=13, rot_dims=8, softcap=25.0,
                                    mlp=plain.dense_mlp(32)),
              plain.latent_layer(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=16, window=19, mlp=None)]
    raw = plain.make_config(layers, width=32, vocab=64)

    def sharpen(t):
        for name in ("l0.mix.q", "l0.mix.k", "l1.mix.q", "l1.mix.uk"):
            t[name] = (t[name].float() * 3.0).to(t[name].dtype)

    folder, raw, tensors = folders("edges", raw, seed=7, edit=sharpen)
    toks = tokens_for(raw, 120, 3)
    want = plain.forward(tensors, raw, toks)
    for layer, delta in ((0, 1), (0, -1), (1, 1), (1, -1)):
        other = copy.deepcopy(raw)
        other["layers"][layer]["mixer"]["mask"]["size"] += delta
        moved = row_errors(plain.forward(tensors, other, toks), want)[20:]          # (rows that have a window's edge behind them)
        assert float(moved.mean()) > 0.03 and float(moved.max()) > 0.3, "the model does not show its windows"
    eng = make_engine(folder, dtype)
    check_request(eng, raw, tensors, toks, [120], dtype, "whole")
    check_request(eng, raw, tensors, toks, [11, 2, 13, 1, 1, 19, 2, 30] + [1] * 41, dtype, "portions and single tokens")


# --- generation through the engine's own entry points -----------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(graphs, folders):
    from edgerag_b200 import SamplingParams
    from edgerag_b200.engine.engine import Engine, EngineOptions

    folder, raw, tensors = folders("full", FULL, seed=1)
    prompts = [tokens_for(raw, n, 40 + i) for i, n in enumerate((37, 5, 21))]
    eng = Engine.from_pretrained(folder, EngineOptions(dtype="float32", block_size=16, num_blocks=24, max_batch_size=2,
                                                       max_step_tokens=64, chunk_size=8, cuda_graphs=graphs))
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12))
    for prompt, out in zip(prompts, outs):
        seq = list(prompt)
        for tok in out:                     # the engine's token is the plain argmax wherever the plain margin is clear
            logits = plain.forward(tensors, raw, seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(logits.abs().max()):
                assert tok == int(logits.argmax())
            seq.append(tok)
        assert len(out) == 12


@pytest.mark.gpu
def test_trace_replay_program(folders, tmp_path):
    import helpers

    folder, raw, tensors = folders("full", FULL, seed=1)
    trace = helpers.Trace()
    for i, n in enumerate((70, 33, 90, 18, 47)):
        trace.sequences[f"r{i}"] = tokens_for(raw, n, 60 + i)
    helpers.cut_mixed(trace, list(trace.sequences), seed=3)
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "out"),
           "--max-tokens", str(trace.max_tokens), "--poison-freed-pages"]
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [int(l.split()[1]) for l in proc.stdout.splitlines() if l.startswith("done ")] == [s["step"] for s in trace.steps]
    want = {rid: plain.forward(tensors, raw, seq) for rid, seq in trace.sequences.items()}
    got_rows, want_rows = [], []
    files = {}
    for step, row, rid, pos in trace.expect:
        if step not in files:
            files[step] = np.fromfile(tmp_path / "out" / f"{step}.f32", dtype="<f4").reshape(-1, raw["vocab"])
        got_rows.append(torch.from_numpy(files[step][row].copy()))
        want_rows.append(want[rid][pos])
    assert_close(torch.stack(got_rows), torch.stack(want_rows), "float32", "trace")


@pytest.mark.gpu
def test_command_line_generates_from_a_saved_model(folders):
    folder, raw, tensors = folders("full", FULL, seed=1)
    prompt = tokens_for(raw, 9, 77)
    proc = subprocess.run([sys.executable, "-m", "edgerag_b200", "--help"], capture_output=True, text=True, cwd=ROOT)
    assert proc.returncode == 0
    from edgerag_b200 import Engine, SamplingParams

    eng = Engine.from_pretrained(folder, dtype="bfloat16", block_size=16, num_blocks=16)
    out = eng.generate([prompt], SamplingParams(max_new_tokens=5))[0]
    assert len(out) == 5 and all(0 <= t < raw["vocab"] for t in out)
