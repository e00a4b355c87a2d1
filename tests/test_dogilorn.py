"""The Dogilorn decoder in the engine against the plain implementation of ``plain_dogilorn.py``: each mechanism's kernel
alone, then whole models of several small configurations through the step function (whole prompts, token by token,
portions down to two tokens, unequal batches, pages and slots used again, long decoding), the replay program, and greedy
generation through ``LLMEngine`` and its scheduler.  Where random weights would hide a fault (one key among hundreds, a
window's edge, the kept first tokens, a page border, the sink) the weights are made so that one score stands out."""
import json
import math
import random

import numpy as np
import pytest
import torch

import plain_dogilorn as P
from trace_tools import TraceBuilder, mixed_trace, peak_tokens, run_trace

gpu = pytest.mark.gpu


def _attn(heads, kv_heads, dim, vdim, scale, mask=None, rot=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, identity, top, ff, groups=None, shared=None):
    r = {"experts": experts, "top": top, "identity": identity}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": r, "expert": {"ff": ff}, "shared": {"ff": shared} if shared is not None else None}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


# Five configurations that differ in every size and option.  a: two layers with keys and values of their own and two that
# read them with other masks (a wider window; more kept tokens), grouped key/value heads, a value wider than a key, windows
# that are no multiple of a page, grouped routing with identity experts.  b: a width that is no multiple of 16, two taps,
# an embedding scale of one, one key/value head, a window below a page without kept tokens, a rotation over the whole head,
# one expert a token and neither groups, identity experts nor a shared expert; a layer without a mask (every key, the sink
# alone) whose value is narrower than its key.  c: sizes that the tensor-core products and attention take, no input
# convolution, sixteen query heads on one key/value head, kept tokens that fill a page, a reader without kept tokens, a layer
# without a feed-forward.  d: more than sixteen query heads a key/value head and an odd head size (the plain attention
# kernel on both paths), more kept tokens than the window is wide, five taps, every expert chosen.  e: one tap (no state), a
# window of one token, a reader that sees every key of a layer whose own window is one.  f: a width that is no multiple of 8 (the
# CUDA-core products on both paths), sixteen taps, an odd number of rotated pairs, a reader with more query heads than the layer it
# reads, one group kept, a head wider than the tensor-core attention takes (values wider than keys).
DG = {
    "a": dict(seed=31, config={
        "architecture": "Dogilorn", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "canon": {"taps": 3}, "embedding": {"scale": 2.5},
        "layers": [
            {"type": "attention", "mixer": _attn(4, 2, 16, 24, 0.3, mask=(20, 3), rot=(500.0, 8)), "mlp": _dense(96, 1.5)},
            {"type": "attention", "mixer": _attn(4, 2, 16, 24, 0.25, mask=(33, 5), rot=(500.0, 8)), "mlp": _moe(6, 2, 3, 24, groups=(4, 2), shared=40)},
            {"type": "attention", "mixer": _attn(4, 2, 16, 24, 0.35, mask=(26, 1), rot=(500.0, 8), kv_from=0), "mlp": _dense(80, 0.8)},
            {"type": "attention", "mixer": _attn(8, 2, 16, 24, 0.2, mask=(9, 7), rot=(500.0, 8), kv_from=1), "mlp": None},
        ]}),
    "b": dict(seed=32, config={
        "architecture": "Dogilorn", "vocab": 157, "width": 40, "norm": {"eps": 1e-6}, "canon": {"taps": 2}, "embedding": {"scale": 1.0},
        "layers": [
            {"type": "attention", "mixer": _attn(3, 1, 12, 20, 0.35, mask=(7, 0), rot=(1000.0, 12)), "mlp": _moe(5, 0, 1, 16)},
            {"type": "attention", "mixer": _attn(3, 1, 12, 20, 0.3, mask=(7, 2), rot=(1000.0, 12), kv_from=0), "mlp": _dense(56, 0.7)},
            {"type": "attention", "mixer": _attn(2, 2, 10, 6, 0.4), "mlp": _moe(3, 1, 2, 8, groups=(2, 1), shared=16)},
        ]}),
    "c": dict(seed=33, config={
        "architecture": "Dogilorn", "vocab": 509, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
        "layers": [
            {"type": "attention", "mixer": _attn(8, 4, 32, 64, 0.18, mask=(64, 4), rot=(50000.0, 16)), "mlp": _moe(13, 3, 4, 32, groups=(4, 2), shared=64)},
            {"type": "attention", "mixer": _attn(4, 4, 64, 128, 0.125, mask=(48, 16), rot=(10000.0, 8)), "mlp": _dense(192, 2.0)},
            {"type": "attention", "mixer": _attn(8, 4, 32, 64, 0.2, mask=(100, 0), rot=(50000.0, 16), kv_from=0), "mlp": _dense(160, 1.0)},
            {"type": "attention", "mixer": _attn(16, 1, 128, 128, 0.09, mask=(40, 2), rot=(10000.0, 64)), "mlp": None},
        ]}),
    "d": dict(seed=34, config={
        "architecture": "Dogilorn", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "canon": {"taps": 5}, "embedding": {"scale": 0.5},
        "layers": [
            {"type": "attention", "mixer": _attn(20, 1, 7, 5, 0.4, mask=(25, 30), rot=(100.0, 4)), "mlp": _moe(4, 0, 4, 12, shared=8)},
        ]}),
    "f": dict(seed=36, config={
        "architecture": "Dogilorn", "vocab": 83, "width": 100, "norm": {"eps": 1e-5}, "canon": {"taps": 16}, "embedding": {"scale": 1.5},
        "layers": [
            {"type": "attention", "mixer": _attn(6, 3, 40, 36, 0.16, mask=(50, 12), rot=(2000.0, 10)), "mlp": _moe(7, 1, 2, 20, groups=(4, 1))},
            {"type": "attention", "mixer": _attn(12, 3, 40, 36, 0.2, mask=(18, 20), rot=(2000.0, 10), kv_from=0), "mlp": _dense(72, 1.2)},
            {"type": "attention", "mixer": _attn(2, 1, 160, 192, 0.08, mask=(31, 2), rot=(100.0, 160)), "mlp": None},
        ]}),
    "e": dict(seed=35, config={
        "architecture": "Dogilorn", "vocab": 131, "width": 80, "norm": {"eps": 1e-6}, "canon": {"taps": 1},
        "layers": [
            {"type": "attention", "mixer": _attn(2, 1, 24, 8, 0.2, mask=(1, 1)), "mlp": _dense(64, 3.0)},
            {"type": "attention", "mixer": _attn(2, 1, 24, 8, 0.25, kv_from=0), "mlp": _moe(2, 2, 2, 16, groups=(2, 2))},
        ]}),
}
TOL = {"float32": 2e-4, "bfloat16": 6e-2}      # largest difference over the largest logit


def agrees(got, want, dtype, what=""):
    """32-bit: every position within the tolerance.  bfloat16: a router's close call may fall the other way for a token, which
    swaps a whole expert there (and colours what a later query reads of it), so the criterion is one of counts: nine
    positions in ten are within the tolerance and the median within half of it."""
    err = np.abs(got - want).max(axis=-1) / np.abs(want).max()
    if dtype == "float32":
        assert err.max() < TOL[dtype], f"{what}: position {int(err.argmax())} differs by {float(err.max()):.2e}"
    elif len(err) < 20:
        assert (err < TOL[dtype]).mean() >= 0.5, f"{what}: {err}"
    else:
        assert np.median(err) < TOL[dtype] / 2 and (err > TOL[dtype]).mean() <= 0.1, \
            f"{what}: median {float(np.median(err)):.2e}, {float((err > TOL[dtype]).mean()):.2f} over, worst {float(err.max()):.2e} at {int(err.argmax())}"


def write_model(folder, cfg, w):
    from safetensors.torch import save_file

    with open(folder / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in w.items()}, str(folder / "model.safetensors"))
    return str(folder)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (model folder, config, weights in float64); written with the safetensors library, not with the package's writer."""
    out = {}
    for name, case in DG.items():
        w = P.random_weights(case["config"], case["seed"])
        out[name] = (write_model(tmp_path_factory.mktemp(f"dg_{name}"), case["config"], w), case["config"], P.as_float64(w))
    return out


_PLAIN = {}


def plain_logits(name, models, tokens):
    key = (name, tuple(tokens))
    if key not in _PLAIN:
        _, cfg, w = models[name]
        _PLAIN[key] = P.forward(cfg, w, list(tokens)).numpy()
    return _PLAIN[key]


def tokens_of(name, n, salt=0):
    rng = random.Random(DG[name]["seed"] * 1000 + n + salt)
    return [rng.randrange(DG[name]["config"]["vocab"]) for _ in range(n)]


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


# ---- configuration and cache bookkeeping (no GPU) ---------------------------------------------------------

def test_config_is_found_by_its_architecture_key_and_declares_the_checkpoints_tensors():
    from spyinfer_b200.config import ConfigError, DogilornConfig, config_from_json
    from spyinfer_b200.engine.model import declared_weights

    for name, case in DG.items():
        cfg = config_from_json(case["config"])
        assert isinstance(cfg, DogilornConfig)
        spec = cfg.to_spec()
        declared = {d.name: tuple(d.shape) for d in declared_weights(spec)}
        assert declared == P.tensor_shapes(case["config"]), name
        assert [e.cache_of for e in spec.run_order] == [l["mixer"].get("kv_from") for l in case["config"]["layers"]], name
        assert config_from_json(cfg.to_json()).to_json() == cfg.to_json()
    base = DG["a"]["config"]

    def broken(change):
        c = json.loads(json.dumps(base))
        change(c)
        with pytest.raises(ConfigError):
            config_from_json(c).to_spec()

    broken(lambda c: c["layers"][0].update(type="mamba1"))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="experts"))
    broken(lambda c: c["layers"][0]["mlp"].pop("limit"))
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))                   # 4 heads do not group over 3
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18))               # wider than a head
    broken(lambda c: c["layers"][0]["mixer"]["mask"].update(size=0))
    broken(lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=-1))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=9))                # more than there are router outputs
    broken(lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3))    # 8 outputs do not form 3 groups
    broken(lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=1))     # one group of two cannot give three experts
    broken(lambda c: c["layers"][2]["mixer"].update(kv_from=2))                    # not an earlier layer
    broken(lambda c: c["layers"][3]["mixer"].update(kv_from=2))                    # a layer that has no keys of its own
    broken(lambda c: c["layers"][2]["mixer"].update(dim=8))                        # differs from the layer it reads
    broken(lambda c: c.pop("norm"))


def test_a_layers_cache_keeps_what_its_readers_need_and_a_reader_keeps_its_own_convolution_state():
    from spyinfer_b200.cache import CacheManager
    from spyinfer_b200.config import CompositeCacheNeed, PagedCacheNeed, SharedCacheNeed, StateCacheNeed, config_from_json
    from spyinfer_b200.engine.model import Model

    model = Model(config_from_json(DG["a"]["config"]).to_spec(), torch.float32, None, 256)
    needs, cache_of = model.cache_needs()
    assert cache_of == [None, None, 0, 1]
    conv = StateCacheNeed((2 * 64,), "float32")
    # rows of max(dim, vdim) = 24; layer 0 keeps the wider window of its reader (26 against 20) and its own three kept tokens,
    # layer 1 its own window and its reader's seven kept tokens
    assert needs[0] == CompositeCacheNeed((conv, PagedCacheNeed(2, 24, 26, keep_first=3)))
    assert needs[1] == CompositeCacheNeed((conv, PagedCacheNeed(2, 24, 33, keep_first=7)))
    assert needs[2] == CompositeCacheNeed((conv, SharedCacheNeed())) and needs[3] == needs[2]
    cache = CacheManager(needs, 8, 40, 2, 320, device=None, cache_of=cache_of, max_step_tokens=16)
    assert cache.num_groups() == 2
    mine, theirs = cache.view(0), cache.view(2)
    assert theirs.parts[1].writes is False and theirs.parts[1].group == mine.parts[1].group and mine.parts[1].writes
    assert theirs.parts[0].kind == "state" and theirs.parts[0] is not mine.parts[0]
    # a reader that sees every key makes the layer it reads keep every key; one tap leaves no state
    model = Model(config_from_json(DG["e"]["config"]).to_spec(), torch.float32, None, 256)
    needs, cache_of = model.cache_needs()
    assert needs[0] == PagedCacheNeed(1, 24, None) and needs[1] is None and cache_of == [None, 0]


def test_the_pages_of_the_kept_first_tokens_are_never_given_back():
    from spyinfer_b200.cache import CacheManager
    from spyinfer_b200.config import PagedCacheNeed

    cache = CacheManager([PagedCacheNeed(1, 8, 10, keep_first=5), PagedCacheNeed(1, 8, 10)], 4, 64, 2, 256, device=None)
    assert cache.num_groups() == 2
    cache.add_request("r")
    cache.reserve("r", 60)
    cache.commit("r", 60)
    kept, plain = (cache.groups[g].tables[cache.slot("r")] for g in (0, 1))
    first_needed = (60 - 10 + 1) // 4
    assert all(kept[lp] >= 0 for lp in (0, 1)) and all(kept[lp] < 0 for lp in range(2, first_needed))          # 5 tokens: two pages of 4
    assert all(plain[lp] < 0 for lp in range(first_needed)) and all(t[lp] >= 0 for t in (kept, plain) for lp in range(first_needed, 15))
    cache.check_invariants()
    cache.free_request("r")
    assert cache.num_free_pages(0) == cache.num_free_pages(1)


def test_what_the_plain_mechanisms_do_on_inputs_known_by_hand():
    # visibility: the window counts the query's own position; kept tokens stay; nothing later is seen
    assert [P.visible(10, j, 3, 2) for j in range(12)] == [True, True, False, False, False, False, False, False, True, True, True, False]
    v = P.visibility(12, 3, 2)
    assert all(bool(v[i, j]) == P.visible(i, j, 3, 2) for i in range(12) for j in range(12))
    assert bool((P.visibility(5, None, 0) == torch.tril(torch.ones(5, 5, dtype=torch.bool))).all())
    # the sink: one key of score s weighs e^s / (1 + e^s)
    q, k, val = torch.tensor([[[2.0]]], dtype=P.F), torch.tensor([[[1.5]]], dtype=P.F), torch.tensor([[[4.0]]], dtype=P.F)
    o = P.sink_softmax_attention(q, k, val, 0.5, torch.tensor([2.0], dtype=P.F), None, 0)
    assert math.isclose(float(o), 4.0 * math.exp(3.0) / (1.0 + math.exp(3.0)), rel_tol=1e-12)
    # the rotation turns pair i by position * base^(-2i/dims) and leaves the rest alone
    x = torch.arange(1.0, 7.0, dtype=P.F).reshape(1, 1, 6).repeat(2, 1, 1)
    r = P.rotate_pairs(x, torch.tensor([0, 3]), 4, 100.0)
    a = 3 * 100.0 ** -0.5
    assert torch.equal(r[0], x[0]) and torch.equal(r[1, 0, 4:], x[1, 0, 4:])
    assert torch.allclose(r[1, 0, 2:4], torch.tensor([3 * math.cos(a) - 4 * math.sin(a), 4 * math.cos(a) + 3 * math.sin(a)], dtype=P.F))
    # the convolution's last column meets the current token
    h = torch.tensor([[1.0], [10.0], [100.0]], dtype=P.F)
    assert P.time_conv(h, torch.tensor([[3.0, 2.0]], dtype=P.F)).flatten().tolist() == [2.0, 23.0, 230.0]
    # the choice: scores .4 .3 .2 .1 in two groups; the correction lifts the second group over the first, whose experts then
    # cannot be chosen although their scores are larger; the weights are the scores without the correction
    mlp = {"router": {"experts": 3, "identity": 1, "top": 1, "groups": {"count": 2, "keep": 1}}}
    W = {"router": torch.log(torch.tensor([[0.4], [0.3], [0.2], [0.1]], dtype=P.F)), "correction": torch.tensor([0.0, 0.0, 0.0, 0.35], dtype=P.F)}
    idx, w = P.route(torch.ones(1, 1, dtype=P.F), mlp, W, "")
    assert idx.tolist() == [[3]] and torch.allclose(w, torch.tensor([[0.1]], dtype=P.F))
    W["correction"] = torch.tensor([-0.5, 0.0, 0.0, 0.0], dtype=P.F)         # choice scores may be negative: the first expert is still in a kept group
    idx, w = P.route(torch.ones(1, 1, dtype=P.F), mlp, W, "")
    assert idx.tolist() == [[1]] and torch.allclose(w, torch.tensor([[0.3]], dtype=P.F))


# ---- kernels alone ---------------------------------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_with_a_bias_adds_a_result_times_a_vector_along_the_row(dtype):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(4)
    for rows, n, splits in ((5, 40, 1), (3, 200, 3), (9, 1000, 2), (4, 4096, 1), (600, 256, 2), (2, 50, 1), (7, 6145, 1)):
        h = torch.randn(rows, n, generator=g)
        y = torch.randn(splits, rows, n, generator=g) * 3
        w, b, ls = ((0.3 * torch.randn(n, generator=g) + o).to(torch.bfloat16) for o in (1.0, 0.0, 0.6))
        ys = y.double().sum(0) if splits > 1 else y[0].to(dtype).double()
        db = 0.5 * torch.randn(n, generator=g) if rows % 2 else None          # the bias of the projection that made y, added ahead of the scale
        xr, rw = (torch.randn(rows, n, generator=g).to(dtype), torch.rand(rows, generator=g)) if rows % 3 else (None, None)    # a term with a weight a row
        want_h = h.double() + (ys + (db.double() if db is not None else 0.0) + (rw.double()[:, None] * xr.double() if xr is not None else 0.0)) * ls.double()
        want_x = P.layer_norm(want_h, w.double(), b.double(), 1e-5)
        hd = h.cuda()
        out = torch.empty((rows, n), dtype=dtype, device="cuda")
        kernels.layernorm(hd, w.cuda(), 1e-5, out, delta=y.cuda() if splits > 1 else y[0].to(dtype).cuda(), delta_weight=ls.cuda(), bias=b.cuda(), write_back=True,
                          delta_bias=db.cuda() if db is not None else None, delta_rows=(xr.cuda(), rw.cuda()) if xr is not None else None)
        assert torch.allclose(hd.cpu().double(), want_h, atol=3e-5, rtol=3e-6), (rows, n)
        assert torch.allclose(out.cpu().double(), want_x, atol=3e-5 if dtype == torch.float32 else 4e-2, rtol=1e-5 if dtype == torch.float32 else 1e-2)
        pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device="cuda")           # the norm alone, of gathered rows; the stream stays
        few = torch.empty((2, n), dtype=dtype, device="cuda")
        before = hd.clone()
        kernels.layernorm(hd, w.cuda(), 1e-5, few, rows=pick, bias=b.cuda())
        assert torch.equal(few, out[[rows - 1, 0]]) and torch.equal(hd, before)


def _paged_setup(lens, page_size, nkv, hd, dtype, seed=0):
    """Block tables of requests of the given lengths over shuffled pages, and an empty cache."""
    rng = random.Random(seed)
    per = [-(-n // page_size) for n in lens]
    ids = list(range(sum(per) + 3))
    rng.shuffle(ids)
    table = torch.full((len(lens), max(per) + 1), -1, dtype=torch.int32)
    at = 0
    for s, n in enumerate(per):
        table[s, :n] = torch.tensor(ids[at:at + n], dtype=torch.int32)
        at += n
    pages = torch.zeros((len(ids), 2, nkv, page_size, hd), dtype=dtype, device="cuda")
    return table.cuda(), pages


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot,page_size", [(4, 2, 16, 24, 8, 8), (3, 1, 12, 20, 12, 4), (8, 4, 32, 64, 16, 16), (16, 1, 128, 128, 64, 16),
                                                                   (20, 1, 7, 5, 4, 8), (2, 2, 10, 6, 0, 16)])
def test_queries_and_cache_rows_normed_over_the_whole_projection(dtype, heads, kv_heads, dim, vdim, rot, page_size):
    """Two requests' tokens in one batch, at positions that are not the batch's order: queries (normed over all heads at once,
    rotated, times the head's temperature) and the cache's key and value rows (values of unit root mean square) equal the
    plain functions'; a layer that reads another's cache gets its queries and writes nothing."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(heads * 100 + dim)
    hd = (max(dim, vdim) + 7) // 8 * 8
    nq, nk, nv = heads * dim, kv_heads * dim, kv_heads * vdim
    lens = [37, 21]
    pos = torch.tensor(list(range(30, 37)) + list(range(5, 21)), dtype=torch.int32)
    seq = torch.tensor([0] * 7 + [1] * 16, dtype=torch.int32)
    T = pos.shape[0]
    proj = torch.randn(T, nq + nk + nv + 5, generator=g) * 2
    qw, kw, temp = ((1.0 + 0.3 * torch.randn(n, generator=g)).to(torch.bfloat16) for n in (nq, nk, heads))
    table, pages = _paged_setup(lens, page_size, kv_heads, hd, dtype)
    rope = None
    if rot:
        inv = torch.tensor([300.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64)
        ang = torch.arange(64, dtype=torch.float64)[:, None] * inv[None]
        rope = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().cuda()
    q_out = torch.full((T, heads * hd), 7.0, dtype=dtype, device="cuda")
    eps = 1e-5
    kernels.sink_qkv_store(proj.cuda(), 0, nq, nq + nk, qw.cuda(), kw.cuda(), temp.cuda(), eps, rope, pos.cuda(), seq.cuda(), q_out, table, pages,
                           heads, kv_heads, dim, vdim, hd)
    pd = proj.double()
    q = (P.unit_rms(pd[:, :nq], eps) * qw.double()).reshape(T, heads, dim)
    k = (P.unit_rms(pd[:, nq:nq + nk], eps) * kw.double()).reshape(T, kv_heads, dim)
    q, k = P.rotate_pairs(q, pos, rot, 300.0) * temp.double()[None, :, None], P.rotate_pairs(k, pos, rot, 300.0)
    v = P.unit_rms(pd[:, nq + nk:nq + nk + nv].reshape(T, kv_heads, vdim), eps)
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=1e-2)
    got_q = q_out.cpu().double().reshape(T, heads, hd)
    assert torch.allclose(got_q[..., :dim], q, **tol) and float(got_q[..., dim:].abs().max() if hd > dim else 0.0) == 0.0
    table_h, pages_h = table.cpu(), pages.cpu().double()
    for t in range(T):
        page, slot = int(table_h[seq[t], pos[t] // page_size]), int(pos[t]) % page_size
        assert torch.allclose(pages_h[page, 0, :, slot, :dim], k[t], **tol) and torch.allclose(pages_h[page, 1, :, slot, :vdim], v[t], **tol)
        assert float(pages_h[page, 0, :, slot, dim:].abs().sum()) == 0.0 and float(pages_h[page, 1, :, slot, vdim:].abs().sum()) == 0.0
    written = {(int(table_h[seq[t], pos[t] // page_size]), int(pos[t]) % page_size) for t in range(T)}
    assert int((pages_h.abs().sum(dim=(1, 2, 4)) > 0).sum()) == len(written)                   # nothing else was touched
    # queries only
    q_only = torch.empty_like(q_out)
    kernels.sink_qkv_store(proj.cuda(), 0, nq, nq + nk, qw.cuda(), None, temp.cuda(), eps, rope, pos.cuda(), seq.cuda(), q_only, None, None,
                           heads, kv_heads, dim, vdim, hd)
    assert torch.equal(q_only, q_out)


def _plain_rows(q, keys, values, positions, seqs, scale, window, keep, sink):
    """q [T, H, d]; keys/values: per request [L, G, d]; the plain attention of every token at its position."""
    T, H = q.shape[0], q.shape[1]
    out = torch.zeros(T, H, values[0].shape[2], dtype=P.F)
    for t in range(T):
        k, v, pos = keys[int(seqs[t])], values[int(seqs[t])], int(positions[t])
        js = [j for j in range(pos + 1) if P.visible(pos, j, window, keep)]
        for h in range(H):
            g = h // (H // k.shape[1])
            e = torch.exp((k[js, g] @ q[t, h]) * scale)
            out[t, h] = (e / ((1.0 if sink else 0.0) + e.sum())) @ v[js, g]
    return out


@gpu
@pytest.mark.parametrize("path", ["plain32", "plain16", "tensor"])
@pytest.mark.parametrize("heads,kv_heads,hd,window,keep,page_size", [(4, 2, 24, 20, 3, 8), (8, 4, 64, 64, 4, 16), (16, 1, 128, 40, 16, 16), (2, 1, 32, 7, 0, 8),
                                                                     (4, 4, 128, None, 0, 32), (2, 2, 16, 25, 30, 16), (4, 1, 8, 1, 1, 8), (2, 1, 64, 130, 20, 16)])
def test_window_with_kept_first_keys_and_a_sink(path, heads, kv_heads, hd, window, keep, page_size):
    """Three requests (a portion of 150 tokens of a prompt of 300, a whole prompt of 40, one decoded token at position 260) over
    shuffled pages.  A few queries are scaled so that they point at one key with nearly all their weight: the oldest key of
    the window and the one before it, the last kept key and the one after it, a page's first and last place.  The plain
    kernel (both formats) does mask and sink itself; on the tensor-core path the window kernels (for portions, and for
    requests of one token) leave their logarithms of sums and ``sink_merge`` adds the kept keys and the sink."""
    from spyinfer_b200 import kernels

    dtype = torch.float32 if path == "plain32" else torch.bfloat16
    if path == "tensor" and not kernels.attention_tc_takes(heads, kv_heads, hd, dtype):
        pytest.skip("sizes the tensor-core kernels do not take")
    g = torch.Generator().manual_seed(hd + heads)
    lens = [300, 40, 261]
    keys = [torch.randn(n, kv_heads, hd, generator=g).to(dtype).double() for n in lens]
    values = [torch.randn(n, kv_heads, hd, generator=g).to(dtype).double() for n in lens]
    table, pages = _paged_setup(lens, page_size, kv_heads, hd, dtype, seed=3)
    pages_h = pages.cpu()
    for s, n in enumerate(lens):
        for j in range(n):
            page = int(table[s, j // page_size])
            pages_h[page, 0, :, j % page_size], pages_h[page, 1, :, j % page_size] = keys[s][j].to(dtype), values[s][j].to(dtype)
    pages.copy_(pages_h)
    pos = torch.tensor(list(range(150, 300)) + list(range(40)) + [260], dtype=torch.int32)
    seq = torch.tensor([0] * 150 + [1] * 40 + [2], dtype=torch.int32)
    T = pos.shape[0]
    q = torch.randn(T, heads, hd, generator=g) * 0.5
    # pointing queries: token t of request 0 looks for the key at position target
    w = window if window is not None else 10 ** 6
    targets = {}
    for t, target in ((20, 170 - w + 1), (21, 171 - w), (30, keep - 1), (31, keep), (40, (190 // page_size) * page_size), (41, (190 // page_size) * page_size - 1),
                      (60, 0), (149, 299)):
        if 0 <= target <= int(pos[t]):
            targets[t] = target
            q[t, 0] = keys[0][target, 0].float() * (12.0 / hd ** 0.5)
    q = q.to(dtype)
    scale = 1.0 / hd ** 0.5
    want = _plain_rows(q.double(), keys, values, pos, seq, scale, window, keep if window is not None else 0, True)
    qd, out = q.reshape(T, heads * hd).cuda(), torch.empty((T, heads * hd), dtype=dtype, device="cuda")
    if path != "tensor":
        kernels.attention_generic(qd, heads, hd, out, pages, table, pos.cuda(), seq.cuda(), scale, window=window, keep_first=keep if window else 0, sink=True)
    else:
        # the decoded token first (as the step function lays a mixed batch out), then the portions
        order = [T - 1] + list(range(T - 1))
        qd, pos_d, seq_d = qd[order].contiguous(), pos[order].cuda(), torch.tensor([0] + [1] * 150 + [2] * 40, dtype=torch.int32).cuda()
        table_d = table[[2, 0, 1]].contiguous()
        q_start = torch.tensor([0, 1, 151, 191], dtype=torch.int32).cuda()
        lse = torch.empty((T, heads), dtype=torch.float32, device="cuda")
        kernels.attention_decode(qd, heads, hd, out, pages, table_d[:1], pos_d, q_start[:2], 1, scale, window=window, lse=lse)
        kernels.attention_tc(qd, heads, hd, out, pages, table_d[1:], pos_d, q_start[1:], 2, scale, window=window, lse=lse)
        kernels.sink_merge(qd, heads, hd, out, lse, pages, table_d, pos_d, seq_d, scale, window, keep if window else 0, True)
        out = out[[order.index(t) for t in range(T)]]
    got = out.cpu().double().reshape(T, heads, hd)
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    worst = (got - want).abs().amax(dim=(1, 2))
    assert float(worst.max()) < tol, f"token {int(worst.argmax())} (position {int(pos[int(worst.argmax())])}) differs by {float(worst.max()):.3e}"
    # the pointing queries did point: where the key is visible the head's result is (nearly) its value, else it is not
    for t, target in targets.items():
        seen = P.visible(int(pos[t]), target, window, keep)
        near = float((want[t, 0] - values[0][target, 0]).abs().max()) < 0.2
        assert not (near and not seen) and (near or not seen or hd < 64), (t, target, seen)     # narrow heads point less sharply


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gate_with_the_biases_folded_in(dtype):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(8)
    for T, ff, limit in ((5, 96, 1.5), (300, 320, 1.0), (2, 7, 0.7), (33, 4096, 2.0)):
        gu = torch.randn(T, 2 * ff, generator=g) * 2
        b = torch.randn(2 * ff, generator=g) * 0.3
        for src in (gu, gu.to(dtype)):
            x = src.double() + b.double()
            gate, up = torch.clamp(x[:, :ff], max=limit), torch.clamp(x[:, ff:], -limit, limit)
            want = gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
            out = torch.empty((T, ff), dtype=dtype, device="cuda")
            kernels.clamped_glu(src.cuda(), b.cuda(), out, limit)
            assert torch.allclose(out.cpu().double(), want, atol=1e-5 if dtype == torch.float32 else 2e-2, rtol=1e-5 if dtype == torch.float32 else 1e-2)


@gpu
@pytest.mark.parametrize("M", [1, 8, 40, 100, 128, 200, 300, 640, 1200, 2048])
@pytest.mark.parametrize("N,K,bias", [(320, 136, True), (4096, 1024, True), (6400, 2048, False), (3364, 512, True)])
def test_product_with_the_clamped_gate_and_the_biases_in_its_epilogue(M, N, K, bias):
    """The tensor-core product over alternating gate and up rows adds the rows' biases and hands out the clamped gated
    activation, on every kernel that the number of tokens selects (and with a last tile of rows that is not full)."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (2.0 * torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = (0.5 * torch.randn(N, generator=g)) if bias else None
    limit = 1.3
    out = kernels.gemm_tcgen05(a.cuda(), w.cuda(), epilogue="clamped_swish", glu=(b.cuda() if bias else None, limit, 1.702))
    prod = a.double() @ w.double().T + (b.double() if bias else 0.0)
    gate, up = torch.clamp(prod[:, 0::2], max=limit), torch.clamp(prod[:, 1::2], -limit, limit)
    want = gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (M, N // 2)
    assert torch.allclose(out.float().cpu().double(), want, atol=2e-2, rtol=2e-2)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,identity,top,ff,groups,shared", [(6, 2, 3, 24, (4, 2), 40), (5, 0, 1, 16, None, 0), (13, 3, 4, 32, (4, 2), 64), (4, 0, 4, 12, None, 8),
                                                                   (3, 1, 2, 8, (2, 1), 16), (2, 2, 2, 16, (2, 2), 0), (60, 4, 6, 8, (8, 3), 0)])
def test_corrected_grouped_choice_identity_experts_and_silu_activations(dtype, experts, identity, top, ff, groups, shared):
    """The kernel's weights equal the plain choice's (an output that is not chosen weighs exactly zero; the identity experts'
    chosen weights are summed), its activations are weight * silu(gate) * up, and the identity share is added in 32-bit."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(experts * 10 + top)
    T, total = 50, experts + identity
    logits = torch.randn(T, total + (1 if shared else 0), generator=g) * 1.5
    corr = torch.randn(total, generator=g) * 0.1
    mlp = {"router": {"experts": experts, "identity": identity, "top": top}}
    if groups:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    W = {"router": torch.eye(total, dtype=P.F), "correction": corr.double()}
    idx, w = P.route(logits[:, :total].double(), mlp, W, "")
    want_w = torch.zeros(T, total, dtype=P.F).scatter_(1, idx, w)
    cols = experts * ff + shared
    gu = torch.randn(T, 2 * cols, generator=g).to(dtype)
    y = torch.empty((T, cols), dtype=dtype, device="cuda")
    weights = torch.empty((T, total + 1), dtype=torch.float32, device="cuda")
    idw = torch.empty((T,), dtype=torch.float32, device="cuda") if identity else None
    kernels.moe_activation(gu.cuda(), logits.cuda(), y, experts, top, ff, 0.0, shared, 0.0, weights_out=weights, identity=identity, correction=corr.cuda(),
                           groups=groups, activation="silu", id_weight=idw)
    got_w = weights.cpu().double()
    assert torch.equal(got_w[:, :total] != 0, want_w != 0) and torch.allclose(got_w[:, :total], want_w, atol=1e-6)
    if shared:
        assert torch.allclose(got_w[:, total], torch.sigmoid(logits[:, total].double()), atol=1e-6)
    if identity:
        assert torch.allclose(idw.cpu().double(), want_w[:, experts:].sum(1), atol=1e-6)
    gud = gu.double()
    want = torch.zeros(T, cols, dtype=P.F)
    for e in range(experts):
        a, b = gud[:, 2 * ff * e:2 * ff * e + ff], gud[:, 2 * ff * e + ff:2 * ff * (e + 1)]
        want[:, ff * e:ff * (e + 1)] = want_w[:, e:e + 1] * a * torch.sigmoid(a) * b
    if shared:
        a, b = gud[:, 2 * ff * experts:2 * ff * experts + shared], gud[:, 2 * ff * experts + shared:]
        want[:, ff * experts:] = torch.sigmoid(logits[:, total:].double()) * a * torch.sigmoid(a) * b
    assert torch.allclose(y.cpu().double(), want, atol=1e-5 if dtype == torch.float32 else 2e-2, rtol=1e-5 if dtype == torch.float32 else 1e-2)
    if identity:
        out, x = torch.randn(T, 40, generator=g), torch.randn(T, 40, generator=g).to(dtype)
        od = out.cuda()
        kernels.add_scaled_rows(od, x.cuda(), idw)
        assert torch.allclose(od.cpu().double(), out.double() + idw.cpu().double()[:, None] * x.double(), atol=1e-5)


# ---- whole models through the step function ---------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(DG))
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
@pytest.mark.parametrize("name", sorted(DG))
def test_long_decoding_passes_windows_and_pages(models, name):
    """260 tokens, all but the first three one by one (through the decode graphs): every window passes over decoded tokens,
    every page border is crossed by a decoded token, and the windowed groups give their pages back but for the first ones."""
    runner = make_runner(models[name][0], "float32", page_size=8, num_pages=40)
    toks = tokens_of(name, 260, salt=1)
    got = run_cuts(runner, "long", toks, [3] + [1] * 257)
    agrees(got, plain_logits(name, models, toks), "float32", "decoded")
    assert runner.graph_steps > 200


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(DG))
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


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "c", "d"])
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


def _pointing_model(tmp_path, window, keep, dim=32):
    """A one-layer model (no feed-forward, no input convolution) whose weights are made so that the token ``A`` as a query
    points at the token ``B`` as a key with a large score on its first head, wherever the two stand (no rotation): the
    embedding of B is solved for so that its key is the direction that A's query likes best.  The second head's queries are
    so small that it weighs all visible keys nearly alike, so its result moves when one key too many or too few is seen."""
    cfg = {"architecture": "Dogilorn", "vocab": 60, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
           "layers": [{"type": "attention", "mixer": _attn(2, 1, dim, 12, 1.0, mask=(window, keep) if window else None), "mlp": None}]}
    w = P.as_float64(P.random_weights(cfg, 77, gain=1.5))
    A, B, eps = 58, 59, 1e-5
    w["l0.norm1.b"].zero_()
    w["l0.mix.q.norm"][dim:] *= 1e-3
    w["l0.mix.temp"][:] = torch.tensor([3.0, 1.0], dtype=P.F)
    h_a = P.layer_norm(w["embed"][A][None], w["l0.norm1"], w["l0.norm1.b"], eps)[0]
    q = (P.unit_rms((w["l0.mix.q"] @ h_a)[None], eps)[0] * w["l0.mix.q.norm"])[:dim]
    h_b = torch.linalg.pinv(w["l0.mix.k"]) @ (q / w["l0.mix.k.norm"])
    h_b = h_b - h_b.mean()                                                           # a layer norm's output has no mean
    w["embed"][B] = h_b / w["l0.norm1"] * (w["embed"][0].norm() / (h_b / w["l0.norm1"]).norm())
    w["embed"][B] -= w["embed"][B].mean()
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    d_ = tmp_path / f"point_{window}_{keep}"
    d_.mkdir()
    return write_model(d_, cfg, w), cfg, P.as_float64(w), A, B


def _pointing_case(tmp_path, window, keep):
    model_dir, cfg, w, A, B = _pointing_model(tmp_path, window, keep)
    rng = random.Random(5)
    n = 400
    toks = [rng.randrange(50) for _ in range(n)]
    if window:
        # keys among the kept first tokens (the last kept place) and right behind them; far back; at a page's first and last place.
        # queries: the key is the window's oldest place, one before it, just kept, just not kept
        keys = [keep - 1, keep, 200, 303, 304]
        asks = [200 + window - 1, 200 + window, 150, 390, 305, 304 + window, 10]
        sees = [[200, keep - 1], [keep - 1], [keep - 1], [keep - 1], [303, 304, keep - 1], [keep - 1], [keep - 1, keep]]
    else:
        keys = [300, 1]
        asks = [301, 399, 304, 303, 350, 2, 17]
        sees = [[300, 1], [300, 1], [300, 1], [300, 1], [300, 1], [1], [1]]
    for k in keys:
        toks[k] = B
    for a in asks:
        toks[a] = A
    probs = []
    want = P.forward(cfg, w, toks, probs=probs).numpy()
    first_head = probs[0][0]                                       # [query, key] of the first head
    for a, seen in zip(asks, sees):
        seen = [k for k in seen if k <= a]
        unseen = [k for k in keys if k not in seen]
        on_seen = float(first_head[a, seen].sum()) if seen else 1.0
        assert on_seen > 0.8 and float(first_head[a, unseen].sum() if unseen else 0.0) < 1e-9, (a, on_seen)
    return model_dir, toks, want, asks, keys


def test_the_plain_model_points_where_the_test_wants_it_to(tmp_path):
    for window, keep in ((None, 0), (40, 6), (24, 17)):
        _pointing_case(tmp_path, window, keep)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,keep", [(None, 0), (40, 6), (24, 17)])
def test_a_query_that_points_at_one_key_finds_it_far_back_and_at_every_edge(tmp_path, dtype, window, keep):
    """The key token stands a few times in a sequence of 400 others; the query token is asked at places where the key is far
    back, at a page's first or last place, at the window's oldest place and one beyond it, and among the kept first tokens
    or right behind them.  The engine's logits equal the plain model's, whole, in portions that cut windows and pages
    anywhere, and decoded one by one."""
    model_dir, toks, want, asks, keys = _pointing_case(tmp_path, window, keep)
    n = len(toks)
    runner = make_runner(model_dir, dtype, page_size=16, num_pages=30)
    tol = TOL[dtype]

    def check(got, what):
        worst = np.abs(got - want).max(axis=1) / np.abs(want).max()
        assert worst[asks].max() < tol, f"{what}: asked position {asks[int(worst[asks].argmax())]}"
        assert worst.max() < tol, f"{what}: position {int(worst.argmax())}"

    check(run_cuts(runner, "w", toks, [n]), "whole")
    check(run_cuts(runner, "d", toks, [99, 2] + [1] * (n - 101)), "decoded")
    check(run_cuts(runner, "p", toks, cycle_cuts(n, [3, 61, 2, 16, 2, 45, 7])), "portions")
    if window:                                                     # portions that end and start exactly where the window's edge passes a key
        check(run_cuts(runner, "e", toks, [keep, 200 - keep, window - 1, 1, 1, n - 200 - window - 1]), "portions at the edges")


@gpu
def test_the_replay_program_runs_the_model(models, tmp_path):
    name = "a"
    rng = random.Random(2)
    reqs = {f"r{n}": tokens_of(name, n, salt=3) for n in (40, 3, 77, 25)}
    b = TraceBuilder()
    b.whole("whole", reqs["r77"])
    mixed_trace(b, reqs, {r: max(1, len(t) - 10) for r, t in reqs.items()}, rng, max_live=4, portion_sizes=(5, 2, 16))
    for dtype in ("float32", "bfloat16"):
        out = run_trace(models[name][0], dtype, b, str(tmp_path / dtype), peak_tokens(b), DG[name]["config"]["vocab"])
        keys = sorted(out)
        got = np.stack([out[k] for k in keys])
        want = np.stack([plain_logits(name, models, reqs["r77" if rid == "whole" else rid])[pos] for rid, pos in keys])
        agrees(got, want, dtype, "replayed")


@gpu
@pytest.mark.parametrize("name", ["a", "b", "e"])
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
            logits = P.forward(cfg, w, toks)[-1]
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
@pytest.mark.parametrize("experts,identity,top,groups,shared", [(6, 2, 3, (4, 2), True), (5, 0, 1, None, False), (13, 3, 4, (4, 2), True), (2, 2, 2, (2, 2), False),
                                                                (60, 4, 6, (8, 3), False)])
def test_pairs_of_token_and_chosen_real_expert_sorted_by_expert(experts, identity, top, groups, shared):
    """The sorted pairs of the general choice: every real expert's run of rows holds exactly the tokens that chose it, in their
    order, with the plain scores as weights; identity experts take no rows (their weights are summed a token); a token that
    chose fewer real experts than ``top`` has pairs without a row."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(experts + top)
    T, total = 300, experts + identity
    logits = torch.randn(T, total + (1 if shared else 0), generator=g) * 1.5
    corr = torch.randn(total, generator=g) * 0.1
    mlp = {"router": {"experts": experts, "identity": identity, "top": top}}
    if groups:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    idx, w = P.route(logits[:, :total].double(), mlp, {"router": torch.eye(total, dtype=P.F), "correction": corr.double()}, "")
    offsets, slot, row_token, row_w, shared_w, idw = kernels.moe_route_general(logits.cuda(), experts, top, identity, corr.cuda(), groups, shared)
    offsets, slot, row_token, row_w = offsets.cpu().tolist(), slot.cpu(), row_token.cpu(), row_w.cpu()
    want_rows = {e: [] for e in range(experts)}
    for t in range(T):
        for e, wt in sorted(zip(idx[t].tolist(), w[t].tolist())):
            if e < experts:
                want_rows[e].append((t, wt))
    assert offsets[0] == 0 and [offsets[e + 1] - offsets[e] for e in range(experts)] == [len(want_rows[e]) for e in range(experts)]
    for e in range(experts):
        got = [(int(row_token[r]), float(row_w[r])) for r in range(offsets[e], offsets[e + 1])]
        assert [t for t, _ in got] == [t for t, _ in want_rows[e]]
        assert np.allclose([x for _, x in got], [x for _, x in want_rows[e]], atol=1e-6)
    n = offsets[experts]
    for t in range(T):
        real = sorted(e for e in idx[t].tolist() if e < experts)
        rows = slot[t].tolist()
        assert all(r >= 0 for r in rows[:len(real)]) and all(r < 0 for r in rows[len(real):])
        assert [next(e for e in range(experts) if offsets[e] <= r < offsets[e + 1]) for r in rows[:len(real)]] == real and all(r < n for r in rows)
    if identity:
        want_id = torch.zeros(T, total, dtype=P.F).scatter_(1, idx, w)[:, experts:].sum(1)
        assert torch.allclose(idw.cpu().double(), want_id, atol=1e-6)
    if shared:
        assert torch.allclose(shared_w.cpu().double(), torch.sigmoid(logits[:, total].double()), atol=1e-6)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e", "f"])
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


# ---- configurations drawn at random -------------------------------------------------------------------------

def random_config(rng):
    """A configuration with every size, option and layer order drawn at random (tensor-core sizes and others, readers of earlier
    layers' keys, masks from one token to longer than the sequence, every kind of feed-forward and choice)."""
    cfg = {"architecture": "Dogilorn", "vocab": rng.randrange(50, 600), "width": rng.choice([64, 96, 128, 160, 192, 256, 320]),
           "norm": {"eps": rng.choice([1e-5, 1e-6])}}
    if rng.random() < 0.85:
        cfg["canon"] = {"taps": rng.choice([1, 2, 3, 4, 4, 6, 8])}
    if rng.random() < 0.85:
        cfg["embedding"] = {"scale": rng.choice([1.0, 2.0, 3.0, 0.5, 7.5])}
    layers, owners = [], []
    for i in range(rng.randrange(2, 9)):
        if owners and rng.random() < 0.4:                        # a reader of an earlier layer's keys and values, with a scale of its own
            j = rng.choice(owners)
            m = dict(layers[j]["mixer"], kv_from=j, scale=rng.choice([0.1, 0.2, layers[j]["mixer"]["dim"] ** -0.5]))
        else:
            heads = rng.choice([1, 2, 4, 8, 16, 3, 6, 20, 32])
            dim = rng.choice([8, 16, 32, 64, 128, 24, 48, 192, 10, 256])
            m = {"heads": heads, "kv_heads": rng.choice([d for d in range(1, heads + 1) if heads % d == 0]), "dim": dim,
                 "vdim": rng.choice([8, 16, 32, 64, 128, 40, dim, dim]), "scale": rng.choice([dim ** -0.5, 0.13, 0.3])}
            if rng.random() < 0.85:
                m["rot"] = {"base": rng.choice([10000.0, 500000.0, 100.0]), "dims": rng.choice(range(2, dim + 1, 2))}
            owners.append(i)
        m["mask"] = {"size": rng.choice([1, 5, 16, 17, 33, 64, 100, 200, 1000]), "keep_first": rng.choice([0, 1, 2, 4, 4, 8, 16, 17, 40])}
        kind = rng.random()
        if kind < 0.1:
            mlp = None
        elif kind < 0.55:
            mlp = _dense(rng.choice([32, 64, 96, 320, 100, 52]), rng.choice([1.0, 0.5, 2.0, 7.0]))
        else:
            while True:
                experts, identity = rng.randrange(1, 17), rng.randrange(0, 5)
                total = experts + identity
                top, groups = rng.randrange(1, min(total, 6) + 1), None
                if rng.random() < 0.7:
                    count = rng.choice([c for c in range(1, total + 1) if total % c == 0])
                    keeps = [k for k in range(1, count + 1) if k * (total // count) >= top]
                    if not keeps:
                        continue
                    groups = (count, rng.choice(keeps))
                break
            mlp = _moe(experts, identity, top, rng.choice([16, 32, 64, 24, 12]), groups=groups, shared=rng.choice([32, 96, 40]) if rng.random() < 0.7 else None)
        layers.append({"type": "attention", "mixer": m, "mlp": mlp})
    cfg["layers"] = layers
    return cfg


@gpu
@pytest.mark.parametrize("seed", [3, 11, 19, 27, 42, 58, 77, 91])
def test_configurations_drawn_at_random_agree_with_the_plain_model_in_every_cut(tmp_path, seed):
    """Whole, the last 60 tokens one by one, and portions down to two tokens, in both formats; in float32 the cuts agree with each
    other to rounding."""
    rng = random.Random(seed)
    cfg = random_config(rng)
    w = P.random_weights(cfg, seed)
    model_dir = write_model(tmp_path, cfg, w)
    n = 330
    toks = [rng.randrange(cfg["vocab"]) for _ in range(n)]
    want = P.forward(cfg, P.as_float64(w), toks).numpy()
    for dtype in ("float32", "bfloat16"):
        runner = make_runner(model_dir, dtype, page_size=16, num_pages=64)
        whole = run_cuts(runner, "w", toks, [n])
        one_by_one = run_cuts(runner, "d", toks, [n - 60] + [1] * 60)
        portions = run_cuts(runner, "p", toks, cycle_cuts(n, [2, 3, 2, 17, 2, 5, 31, 2, 64, 129]))
        for what, got in (("whole", whole), ("decoded", one_by_one), ("portions", portions)):
            agrees(got, want, dtype, f"{json.dumps(cfg)}: {what}")
        if dtype == "float32":
            scale = np.abs(whole).max()
            assert np.abs(one_by_one - whole).max() / scale < 4e-6 and np.abs(portions - whole).max() / scale < 4e-6
