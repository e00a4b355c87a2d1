"""The Naforax decoder in the engine against the plain implementation of ``plain_naforax.py``: each mechanism's kernel
alone, then whole models of several small configurations through the step function (whole prompts, token by token,
portions down to two tokens, unequal batches, pages and slots used again, long decoding), the replay program, and greedy
generation through ``LLMEngine`` and its scheduler.  Where random weights would hide a fault (one key among hundreds, a
chunk's edge, a page border) the weights are made so that one score stands out."""
import json
import math
import random

import numpy as np
import pytest
import torch

import plain_naforax as P
from trace_tools import TraceBuilder, mixed_trace, peak_tokens, run_trace

gpu = pytest.mark.gpu


def _attn(heads, kv_heads, dim, vdim, diff, scale, chunk=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def _moe(experts, top, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": {"ff": shared[0], "limit": shared[1]} if shared is not None else None}


# Five configurations that differ in every size and option.  a: every kind of layer and of feed-forward, a loop over the
# two recurrent layers, two norm groups, grouped key/value heads, a chunk that is no multiple of a page.  b: the loop starts
# at layer 0, runs three times and holds the attention layer (a cache of its own for every pass), one norm group, two taps,
# a multiplier of one, no logit cap, one key/value head, a chunk shorter than a page, a rotation over the whole map, one
# expert a token and no shared expert, a layer without a feed-forward, a width that is no multiple of 16.  c: no loop and
# no input convolution, sizes that the tensor-core products and attention take, a value wider than both maps' keys,
# sixteen experts of which four, 64 states a channel.  d: recurrent layers only (no pages at all), a loop of one pass,
# four taps, four norm groups, five states a channel.  e: attention without a mask and without a rotation, more than
# sixteen query heads, a value narrower than a map, every expert chosen, a loop that ends with the last layer.
NX = {
    "a": dict(seed=21, config={
        "architecture": "Naforax", "vocab": 211, "width": 64, "norm": {"eps": 1e-5, "groups": 2}, "canon": {"taps": 3}, "residual_mult": 0.5,
        "logit_softcap": 12.0, "loop": {"start": 1, "stop": 3, "times": 2},
        "layers": [
            {"type": "attention", "mixer": _attn(4, 2, 16, 24, 0.4, 0.3, chunk=20, rot=(500.0, 8)), "mlp": {"kind": "dense", "ff": 96}},
            {"type": "mingru", "mixer": {"width": 80}, "mlp": _moe(6, 2, 24, 2.0, shared=(40, 1.5))},
            {"type": "mamba1", "mixer": {"inner": 72, "state": 8, "dt_rank": 6, "conv": 4}, "mlp": _moe(6, 2, 24, 2.0, shared=(40, 1.5))},
            {"type": "attention", "mixer": _attn(2, 2, 8, 16, 0.6, 0.4, chunk=33, rot=(100.0, 4)), "mlp": {"kind": "dense", "ff": 80}},
        ]}),
    "b": dict(seed=22, config={
        "architecture": "Naforax", "vocab": 157, "width": 40, "norm": {"eps": 1e-6, "groups": 1}, "canon": {"taps": 2}, "residual_mult": 1.0,
        "loop": {"start": 0, "stop": 2, "times": 3},
        "layers": [
            {"type": "attention", "mixer": _attn(3, 1, 12, 20, 0.25, 0.35, chunk=7, rot=(1000.0, 12)), "mlp": None},
            {"type": "mingru", "mixer": {"width": 24}, "mlp": _moe(5, 1, 16, 3.0)},
            {"type": "mamba1", "mixer": {"inner": 48, "state": 16, "dt_rank": 3, "conv": 2}, "mlp": {"kind": "dense", "ff": 56}},
        ]}),
    "c": dict(seed=23, config={
        "architecture": "Naforax", "vocab": 509, "width": 128, "norm": {"eps": 1e-6, "groups": 4}, "residual_mult": 0.7, "logit_softcap": 30.0,
        "layers": [
            {"type": "attention", "mixer": _attn(8, 4, 32, 64, 0.5, 0.18, chunk=64, rot=(50000.0, 16)), "mlp": _moe(16, 4, 32, 1.0, shared=(64, 2.5))},
            {"type": "mamba1", "mixer": {"inner": 256, "state": 64, "dt_rank": 8, "conv": 3}, "mlp": {"kind": "dense", "ff": 192}},
            {"type": "attention", "mixer": _attn(4, 4, 16, 128, 0.3, 0.25, chunk=48, rot=(10000.0, 8)), "mlp": {"kind": "dense", "ff": 160}},
            {"type": "mingru", "mixer": {"width": 192}, "mlp": None},
        ]}),
    "d": dict(seed=24, config={
        "architecture": "Naforax", "vocab": 97, "width": 48, "norm": {"eps": 1e-5, "groups": 4}, "canon": {"taps": 4}, "residual_mult": 0.8,
        "logit_softcap": 8.0, "loop": {"start": 1, "stop": 2, "times": 1},
        "layers": [
            {"type": "mamba1", "mixer": {"inner": 24, "state": 5, "dt_rank": 2, "conv": 1}, "mlp": None},
            {"type": "mingru", "mixer": {"width": 56}, "mlp": {"kind": "dense", "ff": 72}},
            {"type": "mingru", "mixer": {"width": 32}, "mlp": _moe(3, 2, 8, 1.2, shared=(16, 0.9))},
        ]}),
    "e": dict(seed=25, config={
        "architecture": "Naforax", "vocab": 131, "width": 80, "norm": {"eps": 1e-6, "groups": 5}, "canon": {"taps": 3}, "residual_mult": 0.6,
        "logit_softcap": 20.0, "loop": {"start": 1, "stop": 2, "times": 2},
        "layers": [
            {"type": "attention", "mixer": _attn(20, 5, 8, 4, 0.2, 0.5), "mlp": {"kind": "dense", "ff": 64}},
            {"type": "attention", "mixer": _attn(2, 1, 24, 8, 0.7, 0.2, chunk=25), "mlp": _moe(4, 4, 12, 2.0, shared=(8, 2.0))},
        ]}),
}
TOL = {"float32": 2e-4, "bfloat16": 6e-2}      # largest difference over the largest logit


def agrees(got, want, dtype, what=""):
    """32-bit: every position within the tolerance.  bfloat16: a router's close call may fall the other way for a token, which
    swaps a whole expert there (and colours what a recurrence or a later query carries on from it), so the criterion is one
    of counts: nine positions in ten are within the tolerance and the median within half of it (of a handful of positions,
    at least half are within the tolerance)."""
    err = np.abs(got - want).max(axis=-1) / np.abs(want).max()
    if dtype == "float32":
        assert err.max() < TOL[dtype], f"{what}: position {int(err.argmax())} differs by {float(err.max()):.2e}"
    elif len(err) < 20:
        assert (err < TOL[dtype]).mean() >= 0.5, f"{what}: {err}"
    else:
        assert np.median(err) < TOL[dtype] / 2 and (err > TOL[dtype]).mean() <= 0.1, \
            f"{what}: median {float(np.median(err)):.2e}, {float((err > TOL[dtype]).mean()):.2f} over, worst {float(err.max()):.2e} at {int(err.argmax())}"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (model folder, config, weights); written with the safetensors library, not with the package's writer."""
    from safetensors.torch import save_file

    out = {}
    for name, case in NX.items():
        d = tmp_path_factory.mktemp(f"nx_{name}")
        cfg = case["config"]
        w = P.random_weights(cfg, case["seed"])
        with open(d / "config.json", "w") as f:
            json.dump(cfg, f)
        save_file({k: v.contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
        out[name] = (str(d), cfg, w)
    return out


_PLAIN = {}


def plain_logits(name, models, tokens):
    key = (name, tuple(tokens))
    if key not in _PLAIN:
        _, cfg, w = models[name]
        _PLAIN[key] = P.forward(w, cfg, list(tokens)).numpy()
    return _PLAIN[key]


def tokens_of(name, n, salt=0):
    rng = random.Random(NX[name]["seed"] * 1000 + n + salt)
    return [rng.randrange(NX[name]["config"]["vocab"]) for _ in range(n)]


def make_runner(model_dir, dtype, page_size=16, num_pages=64, max_num_seqs=4, graphs=True):
    from spyinfer_b200.config import EngineConfig, load_model_config
    from spyinfer_b200.engine.model import Model
    from spyinfer_b200.engine.runner import ModelRunner

    spec = load_model_config(model_dir).to_spec()
    config = EngineConfig(dtype=dtype, kvcache_block_size=page_size, num_kvcache_blocks=num_pages, max_num_seqs=max_num_seqs,
                          max_model_len=num_pages * page_size, max_num_batched_tokens=num_pages * page_size, use_cuda_graphs=graphs)
    model = Model(spec, torch.bfloat16 if dtype == "bfloat16" else torch.float32, config.device, config.max_model_len)
    model.load(model_dir)
    return ModelRunner(model, config)


def run_cuts(runner, rid, tokens, cuts, finish=True):
    """The logits of every position of one request fed in portions of the given sizes."""
    from spyinfer_b200.engine.batch import StepEntry

    rows, at = [], 0
    for c in cuts:
        rows.append(runner.step([StepEntry(rid, tokens[at:at + c], list(range(c)))]).float().cpu().numpy().copy())
        at += c
    assert at == len(tokens)
    runner.check_status()
    if finish:
        runner.finish(rid)
    return np.concatenate(rows)


def cycle_cuts(n, sizes):
    cuts, left = [], n
    while left:
        cuts.append(min(left, sizes[len(cuts) % len(sizes)]))
        left -= cuts[-1]
    return cuts


# ---- configuration, run order and cache bookkeeping (no GPU) --------------------------------------------

def test_config_is_found_by_its_architecture_key_and_declares_the_checkpoints_tensors():
    from spyinfer_b200.config import ConfigError, NaforaxConfig, config_from_json
    from spyinfer_b200.engine.model import declared_weights

    for name, case in NX.items():
        cfg = config_from_json(case["config"])
        assert isinstance(cfg, NaforaxConfig)
        spec = cfg.to_spec()
        declared = {d.name: tuple(d.shape) for d in declared_weights(spec)}
        assert declared == P.tensor_shapes(case["config"]), name
        assert [e.layer for e in spec.run_order] == [i for i, _, _ in P.run_order(case["config"])], name
        assert [e.before is not None for e in spec.run_order] == [first for _, _, first in P.run_order(case["config"])], name
        assert config_from_json(cfg.to_json()).to_json() == cfg.to_json()
    base = NX["a"]["config"]

    def broken(change):
        c = json.loads(json.dumps(base))
        change(c)
        with pytest.raises(ConfigError):
            config_from_json(c).to_spec()

    broken(lambda c: c["layers"][0].update(type="latent_attention"))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="experts"))
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))                   # 4 heads do not group over 3
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18))               # wider than a map
    broken(lambda c: c["layers"][0]["mixer"]["mask"].update(size=0))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=7))                # more than there are experts
    broken(lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"))
    broken(lambda c: c["layers"][2]["mixer"].pop("state"))
    broken(lambda c: c["loop"].update(stop=5))
    broken(lambda c: c["norm"].update(groups=3))                                   # does not divide the width
    broken(lambda c: c.pop("norm"))


def test_the_run_order_repeats_the_looped_layers_and_says_what_goes_in_ahead_of_each_pass():
    from spyinfer_b200.config import config_from_json

    order = config_from_json(NX["b"]["config"]).to_spec().run_order
    assert [e.layer for e in order] == [0, 1, 0, 1, 0, 1, 2]
    ahead = [(e.before.embedding, e.before.tensor, e.before.row) if e.before is not None else None for e in order]
    assert ahead == [(False, "loop.step", 0), None, (True, "loop.step", 1), None, (True, "loop.step", 2), None, None]
    assert all(e.cache_of is None for e in order)                                  # every pass keeps a cache of its own
    plain = P.run_order(NX["d"]["config"])
    assert [i for i, _, _ in plain] == [0, 1, 2] and [t for _, t, _ in plain] == [None, 0, None]
    none = json.loads(json.dumps(NX["c"]["config"]))
    assert all(e.before is None for e in config_from_json(none).to_spec().run_order)
    assert "loop.step" not in P.tensor_shapes(none)


def test_every_pass_of_a_layer_has_its_own_pages_and_states_and_the_convolutions_keep_their_inputs():
    from spyinfer_b200.cache import CacheManager
    from spyinfer_b200.config import CompositeCacheNeed, PagedCacheNeed, StateCacheNeed, config_from_json
    from spyinfer_b200.engine.model import Model

    model = Model(config_from_json(NX["b"]["config"]).to_spec(), torch.float32, None, 256)
    needs, cache_of = model.cache_needs()
    assert len(needs) == 7 and cache_of == [None] * 7
    # layer 0 (attention, no feed-forward): its input convolution's one past input, then the pages; rows of max(2 dim, vdim)
    assert needs[0] == CompositeCacheNeed((StateCacheNeed((40,), "float32"), PagedCacheNeed(1, 24, None)))
    assert needs[2] == needs[0] and needs[4] == needs[0]
    # layer 1 (minGRU and a mixture): both convolutions' inputs, then the recurrence's vector
    assert needs[1] == CompositeCacheNeed((StateCacheNeed((40,), "float32"), StateCacheNeed((40,), "float32"), StateCacheNeed((24,), "float32")))
    # layer 2 (selective scan): the block's convolutions, then the scan's states with its own convolution's input
    assert needs[6].flat() == [StateCacheNeed((40,), "float32"), StateCacheNeed((40,), "float32"), StateCacheNeed((48 * 16,), "float32"),
                               StateCacheNeed((48,), "float32")]
    cache = CacheManager(needs, 8, 12, 2, 96, device=None, cache_of=cache_of, max_step_tokens=16)
    assert cache.num_groups() == 1                               # three passes over one kind of pages: one group, three caches
    views = [cache.view(i).paged_views()[0] for i in (0, 2, 4)]
    assert len({id(v) for v in views}) == 3 and all(v.writes for v in views)
    # recurrent layers only: no pages at all; one tap: no state of the convolution
    model = Model(config_from_json(NX["d"]["config"]).to_spec(), torch.float32, None, 256)
    needs, _ = model.cache_needs()
    assert all(isinstance(n, StateCacheNeed) for need in needs for n in (need.flat() if isinstance(need, CompositeCacheNeed) else [need]))
    assert needs[0].flat() == [StateCacheNeed((3 * 48,), "float32"), StateCacheNeed((24 * 5,), "float32")]


def test_which_keys_the_plain_attention_sees_and_what_the_plain_mechanisms_do():
    v = P.chunk_visible(7, 3)
    assert v[5].tolist() == [False, False, False, True, True, True, False] and v[3].tolist() == [False, False, False, True, False, False, False]
    assert v[2].tolist() == [True, True, True, False, False, False, False] and int(P.chunk_visible(5, 1).sum()) == 5
    assert bool((P.chunk_visible(4, 9) == torch.tril(torch.ones(4, 4, dtype=torch.bool))).all())
    # the rotation turns pair i by position * base^(-2i/dims) and leaves the rest alone
    x = torch.arange(1.0, 7.0, dtype=P.F).repeat(2, 1)
    r = P.rotate_pairs(x, torch.tensor([0, 3]), 100.0, 4)
    assert torch.equal(r[0], x[0]) and torch.equal(r[1, 4:], x[1, 4:])
    a = 3 * 100.0 ** -0.5
    assert torch.allclose(r[1, 2:4], torch.tensor([3 * math.cos(a) - 4 * math.sin(a), 4 * math.cos(a) + 3 * math.sin(a)], dtype=P.F))
    # the convolution's last column meets the current token, zeros stand before the start
    h = torch.tensor([[1.0], [10.0], [100.0]], dtype=P.F)
    assert P.time_conv(h, torch.tensor([[3.0, 2.0]], dtype=P.F)).flatten().tolist() == [2.0, 23.0, 230.0]
    # group norm: each group on its own
    g = P.group_norm(torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=P.F), torch.ones(4, dtype=P.F), 2, 0.0)
    assert torch.allclose(g, torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=P.F) / torch.tensor([[12.5 ** 0.5] * 2 + [2.0 ** 0.5] * 2], dtype=P.F))
    # the recurrence's candidate is continuous at zero, and a gate of one replaces the state
    w = {"z": torch.zeros(1, 1, dtype=P.F), "z.b": torch.tensor([50.0], dtype=P.F), "x": torch.ones(1, 1, dtype=P.F), "x.b": torch.zeros(1, dtype=P.F),
         "g": torch.zeros(1, 1, dtype=P.F), "o": torch.ones(1, 1, dtype=P.F)}
    assert P.mingru(torch.tensor([[2.0], [-1e-9], [1e-9]], dtype=P.F), w, "").abs().max() == 0.0          # silu(0) = 0 closes the output
    w["g"] = torch.full((1, 1), 1e3, dtype=P.F)
    h = torch.tensor([[2.0], [-1e-9], [1e-9]], dtype=P.F)
    out = P.mingru(h, w, "") / torch.nn.functional.silu(1e3 * h)
    assert torch.allclose(out.flatten(), torch.tensor([2.5, 0.5, 0.5], dtype=P.F), atol=1e-6)


# ---- kernels alone ---------------------------------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_group_norm_adds_a_normed_output_and_norms_the_stream_for_the_next_sublayer(dtype):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(4)
    for rows, n, groups, splits in ((5, 40, 1, 1), (3, 200, 2, 3), (9, 1000, 5, 2), (4, 4096, 4, 1), (600, 256, 2, 2), (2, 50, 50, 1), (7, 6144, 3, 1)):
        h = torch.randn(rows, n, generator=g)
        y = torch.randn(splits, rows, n, generator=g) * 3
        wy, w = ((1.0 + 0.3 * torch.randn(n, generator=g)).to(torch.bfloat16) for _ in range(2))
        ys = y.double().sum(0) if splits > 1 else y[0].to(dtype).double()
        want_h = h.double() + 0.6 * P.group_norm(ys, wy.double(), groups, 1e-5)
        want_x = P.group_norm(want_h, w.double(), groups, 1e-5)
        hd = h.cuda()
        out = torch.empty((rows, n), dtype=dtype, device="cuda")
        kernels.group_norm(hd, groups, 1e-5, y=y.cuda() if splits > 1 else y[0].to(dtype).cuda(), y_weight=wy.cuda(), y_scale=0.6, weight=w.cuda(), out=out)
        assert torch.allclose(hd.cpu().double(), want_h, atol=3e-5, rtol=3e-6), (rows, n, groups)
        assert torch.allclose(out.cpu().double(), want_x, atol=2e-5 if dtype == torch.float32 else 3e-2, rtol=1e-5 if dtype == torch.float32 else 1e-2)
        # the norm alone, of gathered rows; the stream stays as it is
        pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device="cuda")
        few = torch.empty((2, n), dtype=dtype, device="cuda")
        before = hd.clone()
        kernels.group_norm(hd, groups, 1e-5, weight=w.cuda(), out=few, rows=pick)
        assert torch.equal(few, out[[rows - 1, 0]]) and torch.equal(hd, before)
    with pytest.raises(kernels.KernelError):
        kernels.group_norm(torch.zeros(2, 10, device="cuda"), 3, 1e-5, weight=torch.ones(10, device="cuda"), out=torch.empty(2, 10, device="cuda"))


# two requests' lengths and how they are cut into five steps: runs that stay short, and runs that are long in some steps (one of
# 100 tokens beside one of 4, then one token each, then 46 beside 11) with single tokens and pairs in between
RUNS = {"short": ({0: 20, 1: 9}, {0: [2, 1, 9, 1, 7], 1: [1, 2, 4, 1, 1]}),
        "long": ({0: 150, 1: 37}, {0: [2, 1, 100, 1, 46], 1: [1, 20, 4, 1, 11]})}


def _two_requests_in_portions(lens, cuts, feed):
    """Runs ``feed(parts, q_start, slots, one_each)`` for every step of two requests (in slots 0 and 2 of three) cut into
    portions; ``parts`` is [(request, first token, count)]."""
    at = {0: 0, 1: 0}
    for step in range(len(cuts[0])):
        parts = [(s, at[s], cuts[s][step]) for s in (0, 1)]
        q_start = torch.tensor([0, parts[0][2], parts[0][2] + parts[1][2]], dtype=torch.int32, device="cuda")
        slots = torch.tensor([0, 2], dtype=torch.int32, device="cuda")
        feed(parts, q_start, slots, all(c == 1 for _, _, c in parts))
        for s, a, c in parts:
            at[s] = a + c
    assert at == lens


@gpu
@pytest.mark.parametrize("channels,taps,extra,bias,residual,act", [(40, 3, 0, False, True, None), (24, 4, 9, True, False, "silu"), (7, 2, 1, True, True, None),
                                                                   (300, 1, 0, True, False, "silu"), (64, 8, 64, False, False, None)])
def test_convolution_over_time_keeps_its_last_inputs_through_portions_and_slots(channels, taps, extra, bias, residual, act):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(channels + taps)
    lens, cuts = {0: 23, 1: 11}, {0: [2, 1, 9, 1, 10], 1: [1, 2, 5, 1, 2]}
    x = {s: torch.randn(t, channels + extra, generator=g) for s, t in lens.items()}
    k = torch.randn(channels, taps, generator=g).to(torch.bfloat16)
    b = torch.randn(channels, generator=g).to(torch.bfloat16) if bias else None
    want = {}
    for s in lens:
        xs = x[s][:, :channels].double()
        r = P.time_conv(xs, k.double(), b.double() if bias else None) + (xs if residual else 0.0)
        want[s] = torch.nn.functional.silu(r) if act else r
    state = torch.zeros((3, max(taps - 1, 1) * channels), dtype=torch.float32, device="cuda")
    got = {0: [], 1: []}

    def feed(parts, q_start, slots, one_each):
        xin = torch.cat([x[s][a:a + c] for s, a, c in parts]).cuda()
        out = torch.empty((xin.shape[0], channels), dtype=torch.float32, device="cuda")
        kernels.time_conv(xin, channels, k.cuda(), b.cuda() if bias else None, state if taps > 1 else None, q_start, slots, 2,
                          1 if one_each else max(c for _, _, c in parts), out, residual=residual, activation=act)
        got[0].append(out[:parts[0][2]].cpu())
        got[1].append(out[parts[0][2]:].cpu())

    _two_requests_in_portions(lens, cuts, feed)
    for s in lens:
        assert torch.allclose(torch.cat(got[s]).double(), want[s], atol=2e-5, rtol=2e-5)
    assert bool((state[1] == 0.0).all())
    if taps > 1:                                                 # what a request leaves: its last taps - 1 inputs, oldest first or last
        kept = state[0].cpu().view(-1).sort().values
        assert torch.allclose(kept, x[0][-(taps - 1):, :channels].reshape(-1).sort().values)


@gpu
@pytest.mark.parametrize("runs", ["short", "long"])
@pytest.mark.parametrize("width,extra", [(24, 0), (80, 5), (320, 0), (1, 2)])
def test_mingru_scan_carries_its_state_through_portions_and_slots(width, extra, runs):
    """Short runs take the kernel that walks a run in order, long ones the kernel that scans slices of a run side by side."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(width)
    lens, cuts = RUNS[runs]
    ld = 3 * width + extra
    cols = (extra, extra + 2 * width, extra + width)              # z, the candidate, the output gate: in no particular order
    proj = {s: torch.randn(t, ld, generator=g) * 2 for s, t in lens.items()}
    bz, bx = torch.randn(width, generator=g), torch.randn(width, generator=g)
    want = {}
    for s, p in proj.items():
        p = p.double()
        z = torch.sigmoid(p[:, cols[0]:cols[0] + width] + bz.double())
        u = p[:, cols[1]:cols[1] + width] + bx.double()
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        S, rows = torch.zeros(width, dtype=P.F), []
        for t in range(p.shape[0]):
            S = (1 - z[t]) * S + z[t] * cand[t]
            rows.append(S * torch.nn.functional.silu(p[t, cols[2]:cols[2] + width]))
        want[s] = torch.stack(rows)
    state = torch.zeros((3, width), dtype=torch.float32, device="cuda")
    got = {0: [], 1: []}

    def feed(parts, q_start, slots, one_each):
        pin = torch.cat([proj[s][a:a + c] for s, a, c in parts]).cuda()
        out = torch.empty((pin.shape[0], width), dtype=torch.float32, device="cuda")
        kernels.mingru_scan(pin, cols[0], cols[1], cols[2], bz.cuda(), bx.cuda(), state, q_start, slots, 2, out, width)
        got[0].append(out[:parts[0][2]].cpu())
        got[1].append(out[parts[0][2]:].cpu())

    _two_requests_in_portions(lens, cuts, feed)
    for s in lens:
        assert torch.allclose(torch.cat(got[s]).double(), want[s], atol=2e-5, rtol=2e-5)
    assert bool((state[1] == 0.0).all()) and bool((state[0] != 0.0).any())


@gpu
@pytest.mark.parametrize("runs", ["short", "long"])
@pytest.mark.parametrize("inner,n,rank", [(24, 5, 2), (72, 8, 6), (48, 16, 3), (256, 64, 8), (40, 33, 4), (8, 1, 1)])
def test_selective_scan_carries_its_states_through_portions_and_slots(inner, n, rank, runs):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(inner + n)
    lens, cuts = RUNS[runs]
    x = {s: torch.randn(t, inner, generator=g) for s, t in lens.items()}
    dt_pre = {s: torch.randn(t, inner, generator=g) * 2 for s, t in lens.items()}
    proj = {s: torch.randn(t, rank + 2 * n, generator=g) for s, t in lens.items()}
    xz = {s: torch.randn(t, 2 * inner, generator=g) for s, t in lens.items()}
    a_log = torch.randn(inner, n, generator=g) * 0.5
    dt_b, D = torch.randn(inner, generator=g), torch.randn(inner, generator=g)
    dt_b[0] = 30.0                                                # softplus of a large number is the number
    want = {}
    for s in lens:
        dt = torch.nn.functional.softplus(dt_pre[s].double() + dt_b.double())
        A = -torch.exp(a_log.double())
        B, C = proj[s][:, rank:rank + n].double(), proj[s][:, rank + n:].double()
        S, rows = torch.zeros(inner, n, dtype=P.F), []
        for t in range(lens[s]):
            S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[s][t].double())[:, None] * B[t][None]
            rows.append(S @ C[t] + D.double() * x[s][t].double())
        z = xz[s][:, inner:].double()
        want[s] = torch.stack(rows) * torch.nn.functional.silu(z)
    state = torch.zeros((3, inner * n), dtype=torch.float32, device="cuda")
    got = {0: [], 1: []}

    def feed(parts, q_start, slots, one_each):
        cat = lambda d: torch.cat([d[s][a:a + c] for s, a, c in parts]).cuda()
        out = torch.empty((sum(c for _, _, c in parts), inner), dtype=torch.float32, device="cuda")
        kernels.selective_scan(cat(x), cat(dt_pre), dt_b.cuda(), cat(proj), rank, rank + n, cat(xz), inner, a_log.cuda(), D.cuda(), state, q_start, slots, 2, out)
        got[0].append(out[:parts[0][2]].cpu())
        got[1].append(out[parts[0][2]:].cpu())

    _two_requests_in_portions(lens, cuts, feed)
    for s in lens:
        assert torch.allclose(torch.cat(got[s]).double(), want[s], atol=1e-4, rtol=1e-4)
    assert bool((state[1] == 0.0).all()) and bool((state[2] != 0.0).any())


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,ff,shared", [(6, 2, 24, 40), (5, 1, 16, 0), (16, 4, 32, 64), (4, 4, 12, 8), (3, 2, 7, 3), (64, 6, 8, 0)])
def test_routing_weights_and_expert_activations(dtype, experts, top, ff, shared):
    """The chosen experts carry their softmax score over ALL experts (not renormalised), the others exactly zero; the
    shared expert carries the sigmoid of its own logit; both clamps, and the ``u + 1``."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(experts * 10 + top)
    T, limit, shared_limit = 37, 1.3, 0.8
    cols = experts * ff + shared
    gu = (torch.randn(T, 2 * cols, generator=g) * 2).to(dtype)
    logits = torch.randn(T, experts + (1 if shared else 0) + 2, generator=g) * 2
    scores = torch.softmax(logits[:, :experts].double(), -1)
    best = torch.topk(scores, top, dim=-1).indices
    weight = torch.zeros(T, experts, dtype=P.F).scatter(1, best, scores.gather(1, best))
    want = torch.zeros(T, cols, dtype=P.F)
    x = gu.double()
    for e in range(experts + (1 if shared else 0)):
        lo, n, lim = (2 * e * ff, ff, limit) if e < experts else (2 * experts * ff, shared, shared_limit)
        gate, up = torch.clamp(x[:, lo:lo + n], max=lim), torch.clamp(x[:, lo + n:lo + 2 * n], -lim, lim)
        wt = weight[:, e:e + 1] if e < experts else torch.sigmoid(logits[:, experts:experts + 1].double())
        want[:, (e * ff if e < experts else experts * ff):][:, :n] = wt * gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
    out = torch.empty((T, cols), dtype=dtype, device="cuda")
    w_out = torch.empty((T, experts + 1), dtype=torch.float32, device="cuda")
    kernels.moe_activation(gu.cuda(), logits.cuda(), out, experts, top, ff, limit, shared, shared_limit, 1.702, weights_out=w_out)
    assert torch.allclose(w_out[:, :experts].cpu().double(), weight, atol=1e-6)
    assert int((w_out[:, :experts] != 0).sum()) == T * top
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(out.cpu().double(), want, **tol)
    unchosen = (weight == 0).repeat_interleave(ff, dim=1)
    assert bool((out.cpu()[:, :experts * ff][unchosen] == 0).all())


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot,page_size", [(4, 2, 16, 24, 8, 8), (3, 1, 12, 20, 12, 4), (8, 4, 32, 64, 16, 16), (4, 4, 16, 128, 8, 16),
                                                                    (20, 5, 8, 4, 0, 8), (2, 1, 5, 3, 4, 2)])
def test_differential_queries_and_cache_rows(dtype, heads, kv_heads, dim, vdim, rot, page_size):
    """Bias, the norm of every map with the shared weight, the rotation of neighbouring pairs of each map's first elements;
    a query per map with zeros in the other map's columns, a key row ``[map 1 | map 2]``, the value row beside it."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(heads * 100 + dim)
    hd = (max(2 * dim, vdim) + 7) // 8 * 8
    lens = [11, 6]
    first = [3 * page_size + 1, 0]                                 # the first request is past its first pages already
    T = sum(lens)
    nq, nk, nv = 2 * heads * dim, 2 * kv_heads * dim, kv_heads * vdim
    ld = nq + nk + nv + heads * vdim
    proj = torch.randn(T, ld, generator=g)
    bias = torch.randn(ld, generator=g)
    qw, kw = 1.0 + 0.3 * torch.randn(dim, generator=g), 1.0 + 0.3 * torch.randn(dim, generator=g)
    positions = torch.tensor([first[0] + i for i in range(lens[0])] + [first[1] + i for i in range(lens[1])], dtype=torch.int32)
    seq_of = torch.tensor([0] * lens[0] + [1] * lens[1], dtype=torch.int32)
    base = 300.0
    table = None
    if rot:
        ang = torch.arange(64, dtype=P.F)[:, None] * torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=P.F)[None]
        table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().contiguous()
    pb = (proj + bias).double()
    q = P.unit_rms(pb[:, :nq].view(T, heads, 2, dim), 1e-5) * qw.double()
    k = P.unit_rms(pb[:, nq:nq + nk].view(T, kv_heads, 2, dim), 1e-5) * kw.double()
    if rot:
        q, k = P.rotate_pairs(q, positions, base, rot), P.rotate_pairs(k, positions, base, rot)
    v = pb[:, nq + nk:nq + nk + nv].view(T, kv_heads, vdim)
    width, num_pages = 12, 24
    perm = torch.randperm(num_pages, generator=g).to(torch.int32)
    block_table = torch.stack([perm[:width], perm[width:2 * width]]).contiguous()
    pages = torch.full((num_pages, 2, kv_heads, page_size, hd), 7.0, dtype=dtype, device="cuda")
    q_out = torch.full((T, 2 * heads * hd), 7.0, dtype=dtype, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    kernels.diff_qkv_store(proj.cuda(), 0, nq, nq + nk, bias.cuda(), qw.cuda(), kw.cuda(), 1e-5, table.cuda() if rot else None, positions.cuda(), seq_of.cuda(),
                           q_out, block_table.cuda(), pages, heads, kv_heads, dim, vdim, status=status)
    assert int(status[0]) == 0
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    got_q = q_out.cpu().double().view(T, heads, 2, hd)
    for m in (0, 1):
        assert torch.allclose(got_q[:, :, m, m * dim:(m + 1) * dim], q[:, :, m], **tol)
        other = torch.ones(hd, dtype=torch.bool)
        other[m * dim:(m + 1) * dim] = False
        assert bool((got_q[:, :, m][..., other] == 0).all())
    pg = pages.cpu().double()
    for t in range(T):
        s, p = int(seq_of[t]), int(positions[t])
        page, off = int(block_table[s, p // page_size]), p % page_size
        assert torch.allclose(pg[page, 0, :, off, :2 * dim], k[t].reshape(kv_heads, 2 * dim), **tol), t
        assert torch.allclose(pg[page, 1, :, off, :vdim], v[t], **tol), t
        assert bool((pg[page, 0, :, off, 2 * dim:] == 0).all()) and bool((pg[page, 1, :, off, vdim:] == 0).all())
    touched = {(int(block_table[int(seq_of[t]), int(positions[t]) // page_size]), int(positions[t]) % page_size) for t in range(T)}
    assert int((pg[:, 0, 0, :, 0] != 7.0).sum()) == len(touched)                # nothing else was written


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim,hd", [(4, 24, 32), (3, 20, 24), (4, 128, 128), (20, 4, 16), (1, 1, 8)])
def test_the_two_maps_are_subtracted_normed_and_gated(dtype, heads, vdim, hd):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(heads + vdim)
    T, lam, diff, eps = 13, 0.37, 0.4, 1e-5
    attn = torch.randn(T, 2 * heads * hd, generator=g).to(dtype)
    gate = torch.randn(T, 5 + heads * vdim, generator=g)
    a = attn.double().view(T, heads, 2, hd)[..., :vdim]
    o = P.unit_rms(a[:, :, 0] - lam * a[:, :, 1], eps) * (1 - diff)
    want = o.reshape(T, heads * vdim) * torch.sigmoid(gate[:, 5:].double())
    out = torch.empty((T, heads * vdim), dtype=dtype, device="cuda")
    kernels.diff_combine(attn.cuda(), hd, gate.cuda(), 5, out, heads, vdim, lam, 1 - diff, eps)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=1e-2, rtol=1e-2)
    assert torch.allclose(out.cpu().double(), want, **tol)
    kernels.diff_combine(attn.cuda(), hd, None, 0, out, heads, vdim, lam, 1 - diff, eps)
    assert torch.allclose(out.cpu().double(), o.reshape(T, heads * vdim), **tol)


@gpu
@pytest.mark.parametrize("M", [1, 8, 40, 100, 128, 200, 300, 640, 1200, 2048])
@pytest.mark.parametrize("N,K", [(320, 136), (4096, 1024), (6400, 2048)])
def test_product_with_the_gelu_gate_in_its_epilogue(M, N, K):
    """The tensor-core product over alternating gate and up rows hands out ``gelu_tanh(gate) * up``, on every kernel that the
    number of tokens selects."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (2.0 * torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    out = kernels.gemm_tcgen05(a.cuda(), w.cuda(), epilogue="geglu_tanh")
    prod = a.double() @ w.double().T
    want = P.gelu_tanh(prod[:, 0::2]) * prod[:, 1::2]
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (M, N // 2)
    assert torch.allclose(out.float().cpu().double(), want, atol=2e-2, rtol=2e-2)


@gpu
def test_gelu_gate_logit_cap_and_what_goes_into_the_stream_ahead_of_a_pass():
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(6)
    for dtype in (torch.float32, torch.bfloat16):
        gu = (torch.randn(9, 2 * 35, generator=g) * 3).to(dtype)
        out = torch.empty((9, 35), dtype=dtype, device="cuda")
        kernels.gated_activation(gu.cuda(), out, "gelu_tanh")
        want = P.gelu_tanh(gu[:, :35].double()) * gu[:, 35:].double()
        assert torch.allclose(out.cpu().double(), want, atol=1e-5, rtol=1e-5 if dtype == torch.float32 else 1e-2)
    x = torch.randn(6, 50, generator=g) * 40
    assert torch.allclose(kernels.softcap_(x.clone().cuda(), 11.0).cpu().double(), 11.0 * torch.tanh(x.double() / 11.0), atol=1e-5)
    stream = torch.randn(5, 48, generator=g)
    table = torch.randn(11, 48, generator=g).to(torch.bfloat16)
    row = torch.randn(48, generator=g).to(torch.bfloat16)
    ids = torch.tensor([3, 0, 10, 3, 7], dtype=torch.int32)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    both = kernels.stream_add(stream.clone().cuda(), table.cuda(), ids.cuda(), row.cuda(), status)
    assert torch.allclose(both.cpu(), stream + table.float()[ids.long()] + row.float(), atol=1e-6)
    only_row = kernels.stream_add(stream.clone().cuda(), None, None, row.cuda(), status)
    assert torch.allclose(only_row.cpu(), stream + row.float(), atol=1e-6)


# ---- whole models through the step function ----------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(NX))
def test_whole_prompts_token_by_token_and_portions_agree_with_the_plain_model(models, name, dtype):
    runner = make_runner(models[name][0], dtype)
    for n in (1, 2, 3, 47, 150):
        toks = tokens_of(name, n)
        want = plain_logits(name, models, toks)
        whole = run_cuts(runner, "w", toks, [n])
        agrees(whole, want, dtype, f"{n} tokens at once")
        if n >= 47:
            one_by_one = run_cuts(runner, "d", toks, [n - 40] + [1] * 40)
            agrees(one_by_one, want, dtype, f"{n} tokens, the last 40 one by one")
            portions = run_cuts(runner, "p", toks, cycle_cuts(n, [2, 3, 2, 17, 2, 5, 31, 2, 64]))
            agrees(portions, want, dtype, f"{n} tokens in portions")
            if dtype == "float32":                      # the cut must not show beyond rounding
                scale = np.abs(whole).max()
                assert np.abs(one_by_one - whole).max() / scale < 4e-6 and np.abs(portions - whole).max() / scale < 4e-6
    runner.cache.check_invariants()
    assert runner.cache.num_free_slots() == 4


@gpu
@pytest.mark.parametrize("name", sorted(NX))
def test_long_decoding_passes_chunks_and_pages(models, name):
    """260 tokens, all but the first three one by one (through the decode graphs): every chunk's edge and every page border
    is crossed by a decoded token, and the recurrences run 257 steps on their own state."""
    runner = make_runner(models[name][0], "float32", page_size=8, num_pages=40)
    toks = tokens_of(name, 260, salt=1)
    got = run_cuts(runner, "long", toks, [3] + [1] * 257)
    agrees(got, plain_logits(name, models, toks), "float32", "decoded")
    assert runner.graph_steps > 200


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(NX))
def test_unequal_batches_with_pages_and_slots_used_again(models, name, dtype):
    """Up to three live requests, portions of some beside decoded tokens of others, in a pool so small that every page
    and slot that is given back is needed again; each row equals the plain model's row for its request and position."""
    from spyinfer_b200.engine.batch import StepEntry

    rng = random.Random(9)
    reqs = {f"q{n}": tokens_of(name, n, salt=2) for n in (90, 5, 61, 2, 130, 33, 75)}
    b = TraceBuilder()
    mixed_trace(b, reqs, {r: max(1, len(t) - 25) for r, t in reqs.items()}, rng, max_live=3, portion_sizes=(7, 2, 19, 3, 40, 2))
    pages = -(-peak_tokens(b, round_to=8) // 8)
    runner = make_runner(models[name][0], dtype, page_size=8, num_pages=pages, max_num_seqs=3)
    got, want = [], []
    for st, rows in zip(b.steps, b.rows):
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]).float().cpu().numpy()
        for (rid, pos), row in zip(rows, logits):
            got.append(row)
            want.append(plain_logits(name, models, reqs[rid])[pos])
        for rid in st["end"]:
            runner.finish(rid)
    runner.check_status()
    agrees(np.stack(got), np.stack(want), dtype, "mixed steps")
    runner.cache.check_invariants()
    assert runner.cache.num_free_slots() == 3
    if any(l["type"] == "attention" for l in NX[name]["config"]["layers"]):
        assert runner.cache.min_free_pages() > 0


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "c", "e"])
def test_four_decoding_requests_beside_a_prompt_portion(models, name, dtype):
    """From four one-token requests on, a mixed step lays them out first and their attention takes the kernel made for
    decoding while the portion beside them takes the one for portions; every row still equals the plain model's."""
    from spyinfer_b200.engine.batch import StepEntry

    runner = make_runner(models[name][0], dtype, page_size=16, num_pages=60, max_num_seqs=5)
    olds = {f"o{n}": tokens_of(name, n, salt=5) for n in (70, 90, 33, 120)}
    new = tokens_of(name, 150, salt=6)
    for rid, toks in olds.items():                       # all but the last ten tokens of each
        runner.step([StepEntry(rid, toks[:-10], [])])
    got, want, at = [], [], 0
    for k, n in enumerate((37, 2, 41, 16, 3, 20, 5, 9, 11, 6)):
        entries = [StepEntry("new", new[at:at + n], list(range(n)))]
        entries[1:1] = [StepEntry(rid, [toks[len(toks) - 10 + k]], [0]) for rid, toks in olds.items()]     # the portion first, then the four
        logits = runner.step(entries).float().cpu().numpy()
        got += [logits[:n]] + [logits[n + j][None] for j in range(4)]
        want += [plain_logits(name, models, new)[at:at + n]] + [plain_logits(name, models, toks)[len(toks) - 10 + k][None] for toks in olds.values()]
        at += n
    runner.check_status()
    assert at == len(new)
    agrees(np.concatenate(got), np.concatenate(want), dtype, "four decoding beside a portion")


def _pointing_model(tmp_path, chunk):
    """A one-layer model (differential attention, chunked or not, no feed-forward, no input convolution) whose weights are
    made so that the token ``A`` as a query points at the token ``B`` as a key with a large score on the first map of its
    first head, wherever the two stand: the embedding of B is solved for so that its key is the direction that A's query
    likes best.  Every other map gets keys so small that the norm's eps swallows them: those maps weigh all visible keys
    alike, so their result moves when one key too many or too few is seen."""
    from safetensors.torch import save_file

    cfg = {"architecture": "Naforax", "vocab": 60, "width": 64, "norm": {"eps": 1e-5, "groups": 1}, "residual_mult": 1.0,
           "layers": [{"type": "attention", "mixer": _attn(2, 1, 32, 12, 0.3, 1.0, chunk=chunk, rot=(100.0, 2)), "mlp": None}]}
    w = {k: v.double() for k, v in P.random_weights(cfg, 77, gain=1.5).items()}
    A, B, d, eps = 58, 59, 32, 1e-5
    h_a = P.unit_rms(w["embed"][A][None], eps)[0] * w["l0.norm1"]
    q = P.unit_rms((w["l0.mix.q"] @ h_a + w["l0.mix.q.b"])[:d][None], eps)[0] * w["l0.mix.q.norm"]
    w["l0.mix.k.b"].zero_()
    w["l0.mix.k"][d:] *= 1e-4
    h_b = torch.linalg.pinv(w["l0.mix.k"][:d]) @ (q * w["l0.mix.k.norm"])
    w["embed"][B] = h_b / w["l0.norm1"]
    w["embed"][B] *= w["embed"][0].norm() / w["embed"][B].norm()
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    d_ = tmp_path / f"point_{chunk}"
    d_.mkdir()
    with open(d_ / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in w.items()}, str(d_ / "model.safetensors"))
    return str(d_), cfg, w, A, B


def _pointing_case(tmp_path, chunk):
    model_dir, cfg, w, A, B = _pointing_model(tmp_path, chunk)
    rng = random.Random(5)
    n = 400
    toks = [rng.randrange(50) for _ in range(n)]
    if chunk:
        # the key stands at a chunk's first place, at its last place, and in the sequence's first chunk; the query asks from
        # the chunk's last place (sees it), the next chunk's first (does not), right behind the key, and at the key's own chunk's start
        c = chunk
        keys = [4 * c, 7 * c - 1, 1]
        asks = [5 * c - 1, 5 * c, 4 * c + 1, 7 * c, 7 * c + 1, c - 1, c, 3]
        sees = [True, False, True, False, False, True, False, True]
    else:
        keys = [300, 1]
        asks = [301, 399, 300 + 16 - 300 % 16, 300 + 15 - 300 % 16, 350, 2, 17]
        sees = [True] * 7
    for k in keys:
        toks[k] = B
    for a in asks:
        toks[a] = A
    probs = []
    want = P.forward(w, cfg, toks, probs=probs).numpy()
    first_map = probs[0][0, 0]                                     # [query, key] of the first head's first map
    for a, s in zip(asks, sees):
        on_keys = float(first_map[a, keys].sum())
        assert (on_keys > 0.9) if s else (on_keys < 1e-9), (a, on_keys)
    return model_dir, toks, want, asks, keys


def test_the_plain_model_points_where_the_test_wants_it_to(tmp_path):
    for chunk in (None, 40):
        _pointing_case(tmp_path, chunk)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [None, 40])
def test_a_query_that_points_at_one_key_finds_it_far_back_and_at_every_edge(tmp_path, dtype, chunk):
    """The key token stands a few times in a sequence of 400 others; the query token is asked at places where the key is far
    back, at a page's first or last place, at the chunk's first place with the query at its last, one chunk over, and among
    the first tokens.  The plain model says how much weight the key gets (nearly all, or none); the engine's logits equal
    the plain model's, whole, in portions that cut chunks and pages anywhere, and decoded one by one."""
    model_dir, toks, want, asks, keys = _pointing_case(tmp_path, chunk)
    n = len(toks)
    runner = make_runner(model_dir, dtype, page_size=16, num_pages=30)
    tol = TOL[dtype]

    def check(got, what):
        worst = np.abs(got - want).max(axis=1) / np.abs(want).max()
        assert worst[asks].max() < tol, f"{what}: asked position {asks[int(worst[asks].argmax())]}"
        assert worst.max() < tol, f"{what}: position {int(worst.argmax())}"

    check(run_cuts(runner, "w", toks, [n]), "whole")
    start = min(keys[0], 150)
    check(run_cuts(runner, "d", toks, [start - 1, 2] + [1] * (n - start - 1)), "decoded")
    check(run_cuts(runner, "p", toks, cycle_cuts(n, [3, 61, 2, 16, 2, 45, 7])), "portions")
    if chunk:                                                      # portions that end and start exactly at the chunk's edges, and one token either side
        check(run_cuts(runner, "e", toks, [chunk, chunk - 1, 2, chunk - 1, chunk + 1, 2 * chunk - 1, n - 6 * chunk]), "portions at the edges")


@gpu
def test_the_replay_program_runs_the_model(models, tmp_path):
    name = "a"
    rng = random.Random(2)
    reqs = {f"r{n}": tokens_of(name, n, salt=3) for n in (40, 3, 77, 25)}
    b = TraceBuilder()
    b.whole("whole", reqs["r77"])
    mixed_trace(b, reqs, {r: max(1, len(t) - 10) for r, t in reqs.items()}, rng, max_live=4, portion_sizes=(5, 2, 16))
    for dtype in ("float32", "bfloat16"):
        out = run_trace(models[name][0], dtype, b, str(tmp_path / dtype), peak_tokens(b), NX[name]["config"]["vocab"])
        keys = sorted(out)
        got = np.stack([out[k] for k in keys])
        want = np.stack([plain_logits(name, models, reqs["r77" if rid == "whole" else rid])[pos] for rid, pos in keys])
        agrees(got, want, dtype, "replayed")


@gpu
@pytest.mark.parametrize("name", ["a", "b", "d"])
def test_greedy_generation_through_the_engine_and_its_scheduler(models, name):
    """Five prompts of unequal length, three slots, prompts cut by a small token budget, pages so few that requests wait
    and are preempted: the tokens equal the plain model's greedy continuation."""
    from spyinfer_b200 import LLMEngine, SamplingParams

    model_dir, cfg, w = models[name]
    prompts = [tokens_of(name, n, salt=4) for n in (30, 3, 55, 1, 18)]
    new = 12
    engine = LLMEngine(model_dir, dtype="float32", max_num_seqs=3, max_num_batched_tokens=24, kvcache_block_size=8, num_kvcache_blocks=20,
                       max_model_len=128)
    got = engine.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    for prompt, out in zip(prompts, got):
        toks = list(prompt)
        for i in range(new):
            logits = P.forward(w, cfg, toks)[-1]
            top = torch.topk(logits, 2).values
            if (top[0] - top[1]).item() < 1e-3:                    # the greedy choice must not hang on rounding: follow the engine from here
                assert out[i] in torch.topk(logits, 2).indices.tolist()
                toks.append(out[i])
                continue
            toks.append(int(logits.argmax()))
            assert out[i] == toks[-1], (i, out, toks[len(prompt):])
    assert engine.stats()["free_slots"] == 3


# ---- the routed form of the expert mixture ----------------------------------------------------------------

@gpu
@pytest.mark.parametrize("experts,top,shared", [(6, 2, True), (5, 1, False), (16, 4, True), (64, 6, False), (3, 2, True)])
def test_pairs_of_token_and_expert_sorted_by_expert(experts, top, shared):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(experts + top)
    T = 75
    logits = torch.randn(T, experts + (1 if shared else 0), generator=g) * 2
    scores = torch.softmax(logits[:, :experts].double(), -1)
    best = torch.topk(scores, top, dim=-1).indices.sort(dim=-1).values                # the chosen experts in ascending order
    offsets, slot, row_token, row_w, shared_w = kernels.moe_route(logits.cuda(), experts, top, shared)
    offsets, slot, row_token, row_w = offsets.cpu(), slot.cpu(), row_token.cpu(), row_w.cpu()
    counts = torch.bincount(best.flatten(), minlength=experts)
    assert offsets.tolist() == [0] + counts.cumsum(0).tolist()
    assert sorted(slot.flatten().tolist()) == list(range(T * top))                    # every row is used once
    for t in range(T):
        for k in range(top):
            r, e = int(slot[t, k]), int(best[t, k])
            assert offsets[e] <= r < offsets[e + 1] and int(row_token[r]) == t
            assert abs(float(row_w[r]) - float(scores[t, e])) < 1e-6
    for e in range(experts):                                                          # within an expert's run the tokens keep their order
        run = row_token[int(offsets[e]):int(offsets[e + 1])].tolist()
        assert run == sorted(run)
    if shared:
        assert torch.allclose(shared_w.cpu().double(), torch.sigmoid(logits[:, experts].double()), atol=1e-6)
    # gathered rows, activations with a weight a row, and the sum of each token's results
    x = torch.randn(T, 24, generator=g).to(torch.bfloat16)
    rows = kernels.gather_rows(x.cuda(), row_token.cuda(), torch.empty((T * top, 24), dtype=torch.bfloat16, device="cuda"))
    assert torch.equal(rows.cpu(), x[row_token.long()])
    gu = torch.randn(T * top, 2 * 10, generator=g) * 2
    y = kernels.expert_activation(gu.cuda(), row_w.cuda(), torch.empty((T * top, 10), dtype=torch.float32, device="cuda"), 1.3)
    ga, up = torch.clamp(gu[:, :10].double(), max=1.3), torch.clamp(gu[:, 10:].double(), -1.3, 1.3)
    assert torch.allclose(y.cpu().double(), row_w.double()[:, None] * ga * torch.sigmoid(1.702 * ga) * (up + 1), atol=1e-5)
    res, sh = torch.randn(T * top, 12, generator=g), torch.randn(T, 12, generator=g)
    out = kernels.moe_combine(res.cuda(), slot.cuda(), sh.cuda(), torch.empty((T, 12), dtype=torch.float32, device="cuda"))
    assert torch.allclose(out.cpu(), res[slot.long()].sum(1) + sh, atol=1e-5)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_the_routed_mixture_agrees_with_the_plain_model_and_with_the_dense_form(models, name, dtype, monkeypatch):
    """Steps of eight tokens or more take the routed form (each expert's products on its own rows), shorter ones and decoding the
    dense one; both agree with the plain model, and in float32 with each other to rounding."""
    toks = tokens_of(name, 150, salt=8)
    want = plain_logits(name, models, toks)
    dense = run_cuts(make_runner(models[name][0], dtype), "w", toks, [150])
    monkeypatch.setenv("SPYINFER_MOE_ROUTED_FROM", "8")
    runner = make_runner(models[name][0], dtype)
    mixtures = [l.feed_forward for l in runner.model.layers if getattr(l.feed_forward, "routed_from", None) is not None]
    assert mixtures and all(m.routed_from == 8 for m in mixtures)
    whole = run_cuts(runner, "w", toks, [150])
    agrees(whole, want, dtype, "routed, whole")
    portions = run_cuts(runner, "p", toks, cycle_cuts(150, [2, 31, 8, 3, 64, 9]))
    agrees(portions, want, dtype, "routed and dense portions")
    if dtype == "float32":
        scale = np.abs(dense).max()
        assert np.abs(whole - dense).max() / scale < 4e-6 and np.abs(portions - dense).max() / scale < 4e-6
