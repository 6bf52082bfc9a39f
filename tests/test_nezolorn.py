"""The Nezolorn decoder in the engine against the plain implementation of ``plain_nezolorn.py``: each mechanism's
kernel alone, then whole models of several small configurations through the step function (whole prompts, token by
token, portions down to two tokens, unequal batches, pages and slots used again, long decoding), the replay program,
and greedy generation through ``LLMEngine`` and its scheduler.  Where random weights would hide a fault (one key among
many, a window's or a pooled block's edge) the inputs are made so that one score stands out."""
import json
import math
import random

import numpy as np
import pytest
import torch

import plain_nezolorn as P
from trace_tools import TraceBuilder, mixed_trace, peak_tokens, run_trace

gpu = pytest.mark.gpu

# Three configurations that differ in every size and option: a has one key/value head, a rotation of half the head, no
# band scaling, values wider than keys in the memory, a layer without feed-forward; b has no pair table, as many
# key/value heads as heads, band scaling with a short original length (all three bands occur), a pool of one token and a
# pool longer than its window, a decay rank that is no multiple of 8; c has head sizes that the tensor-core products
# take, two column tiles in the memory's state, and grouped heads; d has delta-rule layers only (no pages at all), one of
# them without a feed-forward, and a width that is no multiple of 16; e has attention without rotation and without
# pooled blocks, and a head size that is no multiple of 8.
NZ = {
    "a": dict(seed=5, config={
        "architecture": "Nezolorn", "vocab": 211, "width": 64, "residual_mult": 0.5, "norm": {"eps": 1e-5},
        "embedding": {"scale": 1.5, "bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 3}},
        "layers": [
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 96},
             "mixer": {"left_scale": 1.3, "right_scale": 0.6,
                       "left": {"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.3, "mask": {"size": 20, "pool": 5},
                                "rot": {"base": 500.0, "dims": 8}},
                       "right": {"heads": 2, "dim": 16, "vdim": 24, "gate_cap": 8.0}}},
            {"type": "general_delta", "mlp": {"kind": "dense", "ff": 80}, "mixer": {"heads": 2, "dim": 16, "decay_rank": 8}},
            {"type": "parallel", "mlp": None,
             "mixer": {"left_scale": 0.7, "right_scale": 1.0,
                       "left": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.2, "mask": {"size": 9, "pool": 4},
                                "rot": {"base": 10000.0, "dims": 32}},
                       "right": {"heads": 1, "dim": 24, "vdim": 40, "gate_cap": 20.0}}},
        ]}),
    "b": dict(seed=6, config={
        "architecture": "Nezolorn", "vocab": 331, "width": 96, "residual_mult": 1.0, "norm": {"eps": 1e-6},
        "embedding": {"scale": 1.0},
        "layers": [
            {"type": "general_delta", "mlp": {"kind": "dense", "ff": 128}, "mixer": {"heads": 3, "dim": 32, "decay_rank": 4}},
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 64},
             "mixer": {"left_scale": 1.0, "right_scale": 1.0,
                       "left": {"heads": 6, "kv_heads": 6, "dim": 16, "vdim": 16, "scale": 0.25, "mask": {"size": 33, "pool": 1},
                                "rot": {"base": 1000.0, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 64}}},
                       "right": {"heads": 3, "dim": 8, "vdim": 8, "gate_cap": 15.0}}},
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 64},
             "mixer": {"left_scale": 0.9, "right_scale": 1.2,
                       "left": {"heads": 2, "kv_heads": 1, "dim": 48, "vdim": 48, "scale": 0.15, "mask": {"size": 16, "pool": 40},
                                "rot": {"base": 300.0, "dims": 24, "scaling": {"factor": 2.0, "low": 2.0, "high": 8.0, "original": 128}}},
                       "right": {"heads": 2, "dim": 16, "vdim": 16, "gate_cap": 5.0}}},
        ]}),
    "c": dict(seed=7, config={
        "architecture": "Nezolorn", "vocab": 509, "width": 128, "residual_mult": 0.4, "norm": {"eps": 1e-6},
        "embedding": {"scale": 0.7, "bigram": {"buckets": 383, "mul_prev": 5, "mul_cur": 11}},
        "layers": [
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 192},
             "mixer": {"left_scale": 1.0, "right_scale": 0.9,
                       "left": {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.11, "mask": {"size": 64, "pool": 16},
                                "rot": {"base": 50000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 512}}},
                       "right": {"heads": 4, "dim": 32, "vdim": 64, "gate_cap": 12.0}}},
            {"type": "general_delta", "mlp": {"kind": "dense", "ff": 160}, "mixer": {"heads": 2, "dim": 64, "decay_rank": 16}},
        ]}),
    "d": dict(seed=8, config={
        "architecture": "Nezolorn", "vocab": 157, "width": 40, "residual_mult": 0.8, "norm": {"eps": 1e-5},
        "embedding": {"scale": 2.0, "bigram": {"buckets": 31, "mul_prev": 1, "mul_cur": 1}},
        "layers": [
            {"type": "general_delta", "mlp": None, "mixer": {"heads": 1, "dim": 24, "decay_rank": 3}},
            {"type": "general_delta", "mlp": {"kind": "dense", "ff": 56}, "mixer": {"heads": 5, "dim": 8, "decay_rank": 8}},
        ]}),
    "e": dict(seed=9, config={
        "architecture": "Nezolorn", "vocab": 97, "width": 48, "residual_mult": 1.0, "norm": {"eps": 1e-6},
        "embedding": {"scale": 1.0},
        "layers": [
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 72},
             "mixer": {"left_scale": 1.0, "right_scale": 1.0,
                       "left": {"heads": 3, "kv_heads": 3, "dim": 12, "vdim": 12, "scale": 0.4, "mask": {"size": 25}},
                       "right": {"heads": 1, "dim": 12, "vdim": 20, "gate_cap": 10.0}}},
        ]}),
}
TOL = {"float32": 2e-4, "bfloat16": 6e-2}      # largest difference over the largest logit


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (model folder, config, weights); written with the safetensors library, not with the package's writer.  The
    stored config.json of ``b`` leaves the decay rank out: the loader takes it from the tensor's shape."""
    from safetensors.torch import save_file

    out = {}
    for name, case in NZ.items():
        d = tmp_path_factory.mktemp(f"nz_{name}")
        cfg = case["config"]
        w = P.random_weights(cfg, case["seed"])
        stored = json.loads(json.dumps(cfg))
        if name == "b":
            for layer in stored["layers"]:
                layer["mixer"].pop("decay_rank", None)
        with open(d / "config.json", "w") as f:
            json.dump(stored, f)
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
    rng = random.Random(NZ[name]["seed"] * 1000 + n + salt)
    return [rng.randrange(NZ[name]["config"]["vocab"]) for _ in range(n)]


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


def rel(got, want):
    return float(np.abs(got - want).max() / np.abs(want).max())


# ---- configuration and cache bookkeeping (no GPU) -------------------------------------------------------

def test_config_is_found_by_its_architecture_key_and_declares_the_checkpoints_tensors():
    from spyinfer_b200.config import ConfigError, NezolornConfig, config_from_json
    from spyinfer_b200.engine.model import declared_weights

    for name, case in NZ.items():
        cfg = config_from_json(case["config"])
        assert isinstance(cfg, NezolornConfig)
        decls = {d.name: tuple(d.shape) for d in declared_weights(cfg.to_spec())}
        want = {k: tuple(v.shape) for k, v in P.random_weights(case["config"], 1).items()}
        assert decls == want
        again = config_from_json(cfg.to_json())
        assert again.to_json() == cfg.to_json()
    bad = json.loads(json.dumps(NZ["a"]["config"]))
    bad["layers"][0]["mixer"]["left"]["vdim"] = 8
    with pytest.raises(ConfigError, match="vdim"):
        config_from_json(bad)
    bad = json.loads(json.dumps(NZ["a"]["config"]))
    bad["layers"][1]["type"] = "something_else"
    with pytest.raises(ConfigError, match="not a known layer type"):
        config_from_json(bad)
    bad = json.loads(json.dumps(NZ["a"]["config"]))
    del bad["layers"][1]["mixer"]["decay_rank"]
    with pytest.raises(ConfigError, match="decay_rank"):
        config_from_json(bad).to_spec()


def test_a_size_that_config_json_leaves_out_comes_from_the_tensors_shape(models):
    from spyinfer_b200.config import load_model_config

    cfg = load_model_config(models["b"][0])
    assert cfg.layers[0]["mixer"]["decay_rank"] == 4
    cfg.to_spec()


def test_cache_groups_with_a_stride_and_mixers_with_several_needs():
    from spyinfer_b200.cache import CacheManager
    from spyinfer_b200.config.spec import CompositeCacheNeed, PagedCacheNeed, StateCacheNeed

    need = CompositeCacheNeed((CompositeCacheNeed((PagedCacheNeed(2, 8, window=12), PagedCacheNeed(2, 8, None, stride=5))), StateCacheNeed((3,))))
    cm = CacheManager([need, None, StateCacheNeed((1,), "int32")], page_size=4, num_pages=20, max_num_seqs=3, max_model_len=80, device=None)
    view = cm.view(0)
    assert view.kind == "composite" and [p.kind for p in view.parts] == ["composite", "state"]
    tokens, pooled = view.parts[0].parts
    assert (tokens.group, tokens.window, tokens.stride) == (0, 12, 1) and (pooled.group, pooled.window, pooled.stride) == (1, None, 5)
    assert [v.group for v in view.paged_views()] == [0, 1]
    assert cm.spare_slot == 3
    cm.add_request("r")
    cm.reserve("r", 23)                      # 23 tokens: 6 token pages, 4 whole blocks of 5 -> 1 pooled page
    assert cm.num_free_pages(0) == cm.group_pages[0] - 6 and cm.num_free_pages(1) == cm.group_pages[1] - 1
    cm.commit("r", 23)
    assert list(cm.block_table("r", 0)[:3]) == [-1, -1, -1] and cm.block_table("r", 0)[3] >= 0      # the window of 12 passed three pages
    assert cm.block_table("r", 1)[0] >= 0 and cm.block_table("r", 1)[1] == -1
    cm.reserve("r", 41)                      # 8 blocks -> 2 pooled pages
    assert cm.num_free_pages(1) == cm.group_pages[1] - 2
    cm.check_invariants()
    cm.free_request("r")
    assert cm.num_free_pages(0) == cm.group_pages[0] and cm.num_free_pages(1) == cm.group_pages[1]
    cm.check_invariants()
    with pytest.raises(ValueError):
        PagedCacheNeed(2, 8, window=4, stride=2)


def test_which_keys_the_plain_attention_sees():
    """The oracle itself on a case worked out by hand: window 4, pool 3, query 9 sees tokens 6..9 and the blocks 0 and 1
    (block 1 ends at 5 = 9 - 4); query 8 sees 5..8 and block 0 only (token 3 and 4 are seen by nobody)."""
    T, d = 10, 4
    k = torch.zeros(T, 1, d, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64)[:, None, None].repeat(1, 1, d)
    q = torch.zeros(T, 1, d, dtype=torch.float64)           # all scores equal: the output is the mean of what is seen
    o = P.windowed_pooled_attention(q, k, v, window=4, pool=3, scale=1.0)
    assert o[9, 0, 0].item() == pytest.approx((6 + 7 + 8 + 9 + 1 + 4) / 6)
    assert o[8, 0, 0].item() == pytest.approx((5 + 6 + 7 + 8 + 1) / 5)
    assert o[3, 0, 0].item() == pytest.approx((0 + 1 + 2 + 3) / 4)


# ---- kernels alone ---------------------------------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_kernel_with_scaled_sums_stacks_and_gathered_rows(dtype):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(3)
    n, size = 37, 200
    x = (torch.randn(n, size, generator=g) * 2 + 0.7)
    d1 = torch.randn(3, n, size, generator=g)
    d2 = torch.randn(n, size, generator=g)
    w = (1 + 0.1 * torch.randn(size, generator=g)).to(dtype)
    xs = x.cuda()
    out = torch.empty((n, size), dtype=dtype, device="cuda")
    kernels.layernorm(xs, w.cuda(), 1e-5, out, delta=d1.cuda(), delta_scale=0.3, delta2=d2.cuda(), delta2_scale=-1.1, write_back=True)
    total = x.double() + 0.3 * d1.double().sum(0) + (-1.1) * d2.double()
    want = P.layer_norm(total, w.double(), 1e-5)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(xs.cpu().double(), total, atol=1e-5)
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device="cuda")
    out2 = torch.empty((4, size), dtype=dtype, device="cuda")
    kernels.layernorm(xs, w.cuda(), 1e-5, out2, rows=rows)
    assert torch.allclose(out2.cpu().double(), want[[5, 0, 36, 5]], atol=tol, rtol=tol)
    out3 = torch.empty((n, size), dtype=dtype, device="cuda")
    kernels.layernorm(xs, w.cuda(), 1e-5, out3, center=False)
    assert torch.allclose(out3.cpu().double(), P.unit_rms(total, 1e-5) * w.double(), atol=tol, rtol=tol)


@gpu
def test_embedding_with_a_pair_table_keeps_the_last_token_between_portions():
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(4)
    V, H, B = 50, 24, 13
    table, pairs = torch.randn(V, H, generator=g).to(torch.bfloat16), torch.randn(B + 1, H, generator=g).to(torch.bfloat16)
    cfg = {"embedding": {"scale": 0.25, "bigram": {"buckets": B, "mul_prev": 7, "mul_cur": 3}}}
    seqs = {0: [4, 9, 9, 49, 0, 17, 3], 2: [11, 12, 13, 14, 15]}
    want = {s: P.embed({"embed": table, "bigram": pairs}, cfg, t, torch.float64) for s, t in seqs.items()}
    state = torch.zeros((4, 1), dtype=torch.int32, device="cuda")
    got = {0: [], 2: []}
    # portions of unequal sizes, two requests in one batch, slot 2 before slot 0
    for (a0, a1), (b0, b1) in (((0, 3), (0, 1)), ((3, 4), (1, 4)), ((4, 5), (4, 7))):
        ids = seqs[2][a0:a1] + seqs[0][b0:b1]
        pos = list(range(a0, a1)) + list(range(b0, b1))
        seq_of = [0] * (a1 - a0) + [1] * (b1 - b0)
        dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
        out = torch.empty((len(ids), H), dtype=torch.float32, device="cuda")
        kernels.embedding_scaled(table.cuda(), dev(ids), out, 0.25, None, pairs=pairs.cuda(), mul_prev=7, mul_cur=3, positions=dev(pos),
                                 seq_of_token=dev(seq_of), q_start=dev([0, a1 - a0, len(ids)]), state_slot=dev([2, 0]), prev_state=state)
        got[2].append(out[:a1 - a0].cpu())
        got[0].append(out[a1 - a0:].cpu())
    for s in seqs:
        assert torch.allclose(torch.cat(got[s]).double(), want[s][:sum(len(x) for x in got[s])], atol=1e-6)
    assert state[:, 0].tolist() == [seqs[0][6], 0, seqs[2][4], 0]


@gpu
def test_rotary_frequencies_by_wavelength_bands():
    from spyinfer_b200.parts import BuildContext, build_part
    from spyinfer_b200.config.spec import PartSpec

    rot = {"base": 1000.0, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 64}}
    want = P.rotary_frequencies(rot, torch.float64)
    plain = P.rotary_frequencies({"base": 1000.0, "dims": 16}, torch.float64)
    kept, slowed = (want == plain), torch.isclose(want, plain / 4.0)
    assert kept.any() and slowed.any() and (~kept & ~slowed).any(), "the test's constants must reach all three bands"
    ctx = BuildContext(dtype=torch.float32, device=torch.device("cuda"), max_model_len=300)
    part = build_part(PartSpec("rotary_half", {"theta": 1000.0, "rotary_dim": 16, "wavelength_scaling": rot["scaling"]}), ctx)
    table = part.rotation_table().cpu().double()
    ang = torch.arange(300, dtype=torch.float64)[:, None] * want[None, :]
    assert torch.allclose(table[..., 0], torch.cos(ang), atol=3e-5) and torch.allclose(table[..., 1], torch.sin(ang), atol=3e-5)


def _paged(kv, page_size, page_ids, dtype):
    """``kv [T, 2, G, d]`` laid into pages ``[pages, 2, G, page_size, d]`` at the given page ids (scattered on purpose)."""
    T, _, G, d = kv.shape
    pages = torch.full((max(page_ids) + 2, 2, G, page_size, d), 7.0, dtype=dtype)
    for t in range(T):
        pages[page_ids[t // page_size], :, :, t % page_size] = kv[t].to(dtype)
    return pages


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,pool,page_size", [(20, 5, 8), (7, 16, 4), (33, 1, 16), (16, 40, 16), (12, 0, 8)])
def test_pooled_window_attention_sees_exactly_its_keys(dtype, window, pool, page_size):
    """For many (query, target) pairs the query is made to point at one token's key with a large score.  If that token is
    inside the window the output is its value; if its block is pooled, the block's mean value (the query then points at
    the pooled key); if it is seen by nobody the output is far from it.  Compared with the plain attention, row by row."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(window * 100 + pool)
    T, H, G, d = 150, 4, 2, 16
    k = torch.randn(T, G, d, generator=g)
    k = (k / k.norm(dim=-1, keepdim=True)).to(dtype).float()          # unit keys, as the cache will hold them
    v = torch.randn(T, G, d, generator=g).to(dtype).float()
    # queries: position i, head h points (scale 60) at the key of a target that sits at an edge of what i sees
    q = torch.zeros(T, H, d)
    for i in range(T):
        edges = [i - window + 1, i - window, i, max(0, i - window + 1 - (pool or 1)), ((i - window + 1) // pool) * pool - 1 if pool else 0, 0]
        for h in range(H):
            j = min(max(edges[(i + h) % len(edges)], 0), i)
            q[i, h] = 60.0 * k[j, h // (H // G)]
    q = q.to(dtype).float()
    want = P.windowed_pooled_attention(q.double(), k.double(), v.double(), window, pool or 10 ** 9, 1.0)
    n_pages = -(-T // page_size)
    ids = list(reversed(range(3, 3 + n_pages)))
    pages = _paged(torch.stack([k, v], dim=1), page_size, ids, dtype).cuda()
    width = n_pages + 1
    bt = torch.full((2, width), -1, dtype=torch.int32)
    bt[1, :n_pages] = torch.tensor(ids, dtype=torch.int32)
    pooled = pt = None
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    seq_of = torch.ones(T, dtype=torch.int32, device="cuda")
    if pool:
        n_pool_pages = -(-(T // pool) // page_size) + 1
        pool_ids = list(range(n_pool_pages, 0, -1))
        pooled = torch.full((n_pool_pages + 2, 2, G, page_size, d), 9.0, dtype=dtype, device="cuda")
        pt = torch.full((2, width), -1, dtype=torch.int32)
        pt[1, :n_pool_pages] = torch.tensor(pool_ids, dtype=torch.int32)
        pt = pt.cuda()
        kernels.pool_store(pages, bt.cuda(), pooled, pt, pool, positions, seq_of)
        b = (T // pool) - 1                                     # the last whole block's entry is the mean of its rows
        got_mean = pooled[pool_ids[b // page_size], 0, 1, b % page_size].float().cpu()
        assert torch.allclose(got_mean, k[b * pool:(b + 1) * pool, 1].mean(0), atol=1e-2 if dtype == torch.bfloat16 else 1e-6)
    out = torch.empty((T, H * d), dtype=dtype, device="cuda")
    q_dev = q.to(dtype).reshape(T, H * d).cuda()
    kernels.attention_pool(q_dev, H, d, out, pages, bt.cuda(), pooled, pt, positions, seq_of, 1.0, window, pool)
    got = out.float().cpu().view(T, H, d).double()
    tol = 3e-2 if dtype == torch.bfloat16 else 2e-5
    worst = (got - want).abs().amax(dim=(1, 2))
    assert worst.max().item() < tol, f"query {int(worst.argmax())} differs by {worst.max().item()}"
    if dtype != torch.bfloat16 or page_size not in kernels.ATTENTION_TMA_PAGE_SIZES:
        return
    # The same queries on the paths that serving takes in bfloat16: the window on the tensor-core kernels, which hand out
    # every row's log-sum-exp, and the pooled entries merged into that softmax afterwards; as one prompt ...
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    out2, lse = torch.full((T, H * d), 3.0, dtype=dtype, device="cuda"), torch.empty((T, H), dtype=torch.float32, device="cuda")
    kernels.attention_tc(q_dev, H, d, out2, pages, bt[1:2].contiguous().cuda(), positions, i32([0, T]), 1, 1.0, window=window, lse=lse)
    kernels.attention_pool(q_dev, H, d, out2, pages, bt.cuda(), pooled, pt, positions, seq_of, 1.0, window, pool, lse=lse)
    worst = (out2.float().cpu().view(T, H, d).double() - want).abs().amax(dim=(1, 2))
    assert worst.max().item() < 6e-2, f"prompt path: query {int(worst.argmax())} differs by {worst.max().item()}"
    # ... and as T requests that each decode one token at their own position over the same pages
    out3, lse3 = torch.full((T, H * d), 3.0, dtype=dtype, device="cuda"), torch.empty((T, H), dtype=torch.float32, device="cuda")
    each = lambda table: table[1:2].expand(T, table.shape[1]).contiguous().cuda()
    kernels.attention_decode(q_dev, H, d, out3, pages, each(bt), positions, i32(list(range(T + 1))), T, 1.0, window=window, lse=lse3)
    kernels.attention_pool(q_dev, H, d, out3, pages, each(bt), pooled, each(pt.cpu()) if pool else None, positions, i32(list(range(T))), 1.0, window, pool, lse=lse3)
    worst = (out3.float().cpu().view(T, H, d).double() - want).abs().amax(dim=(1, 2))
    assert worst.max().item() < 6e-2, f"decode path: query {int(worst.argmax())} differs by {worst.max().item()}"


def _state_rows(heads, record, slots):
    return torch.zeros((slots, heads * record), dtype=torch.float32, device="cuda")


@gpu
@pytest.mark.parametrize("heads,dk,dv", [(2, 16, 24), (1, 48, 72), (3, 8, 8)])
def test_matrix_memory_scan_carries_its_state_through_portions_and_slots(heads, dk, dv):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(dk + dv)
    cap, lens, cuts = 6.0, {0: 23, 1: 9}, {0: [1, 7, 2, 13], 1: [4, 1, 1, 3]}
    ld = 2 * heads * dk + 2 * heads * dv + 2 * heads + 3
    offs = (3, 3 + heads * dk, 3 + 2 * heads * dk + heads * dv, ld - 2 * heads, ld - heads)       # v after g: columns in another order than the part's
    proj = {s: torch.randn(n, ld, generator=g) for s, n in lens.items()}
    for s in proj:
        proj[s][:, offs[3]:] *= 4.0                                 # gates beyond the cap's linear range
    bi, bf = torch.randn(heads, generator=g), torch.randn(heads, generator=g) + 1.0
    want = {}
    for s, x in proj.items():
        x = x.double()
        q = (x[:, offs[0]:offs[0] + heads * dk] * dk ** -0.5).view(-1, heads, dk)
        k = x[:, offs[1]:offs[1] + heads * dk].view(-1, heads, dk)
        v = x[:, offs[2]:offs[2] + heads * dv].view(-1, heads, dv)
        ig = cap * torch.tanh((x[:, offs[3]:offs[3] + heads] + bi.double()) / cap)
        fg = torch.nn.functional.logsigmoid(cap * torch.tanh((x[:, offs[4]:offs[4] + heads] + bf.double()) / cap))
        want[s] = torch.stack([P.matrix_memory(q[:, h], k[:, h], v[:, h], ig[:, h], fg[:, h]) for h in range(heads)], dim=1).reshape(-1, heads * dv)
    record = kernels.mlstm_record(dk, dv)
    state = _state_rows(heads, record, 4)
    state[3] = 5.0                                                  # a slot nobody uses keeps what it holds
    slot = {0: 2, 1: 0}
    got, at = {0: [], 1: []}, {0: 0, 1: 0}
    for step in range(4):
        parts = [(s, at[s], cuts[s][step]) for s in (1, 0)]
        x = torch.cat([proj[s][a:a + n] for s, a, n in parts]).cuda()
        q_start = torch.tensor([0, parts[0][2], parts[0][2] + parts[1][2]], dtype=torch.int32, device="cuda")
        slots = torch.tensor([slot[1], slot[0]], dtype=torch.int32, device="cuda")
        out = torch.empty((x.shape[0], heads * dv), dtype=torch.float32, device="cuda")
        kernels.mlstm_scan(x, offs, bi.cuda(), bf.cuda(), state, q_start, slots, 2, out, heads, dk, dv, dk ** -0.5, cap)
        got[1].append(out[:parts[0][2]].cpu())
        got[0].append(out[parts[0][2]:].cpu())
        for s, a, n in parts:
            at[s] = a + n
    for s in lens:
        assert torch.allclose(torch.cat(got[s]).double(), want[s], atol=2e-5, rtol=2e-5)
    assert bool((state[3] == 5.0).all()) and bool((state[1] == 0.0).all())


@gpu
@pytest.mark.parametrize("heads,d", [(2, 16), (1, 72), (3, 40)])
def test_delta_rule_scan_carries_its_state_through_portions_and_slots(heads, d):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(d)
    n = heads * d
    lens, cuts = {0: 19, 1: 8}, {0: [2, 1, 9, 7], 1: [1, 2, 4, 1]}
    ld = 4 * n + 5
    offs = (5, 5 + n, 5 + 2 * n, 5 + 3 * n)
    proj = {s: torch.randn(t, ld, generator=g) for s, t in lens.items()}
    pre = {s: torch.randn(t, n, generator=g) * 2 for s, t in lens.items()}
    ba, w0 = torch.randn(n, generator=g), torch.randn(n, generator=g)
    want = {}
    for s, x in proj.items():
        x = x.double()
        r, k, v = (x[:, o:o + n].view(-1, heads, d) for o in offs[:3])
        rate = torch.sigmoid(x[:, offs[3]:offs[3] + n] + ba.double()).view(-1, heads, d)
        decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(pre[s].double() + w0.double())).view(-1, heads, d)
        want[s] = torch.stack([P.delta_memory(r[:, h], k[:, h], v[:, h], decay[:, h], rate[:, h]) for h in range(heads)], dim=1).reshape(-1, n)
    state = _state_rows(heads, d * d, 3)
    slot = {0: 0, 1: 2}
    got, at = {0: [], 1: []}, {0: 0, 1: 0}
    for step in range(4):
        parts = [(s, at[s], cuts[s][step]) for s in (0, 1)]
        x = torch.cat([proj[s][a:a + c] for s, a, c in parts]).cuda()
        p = torch.cat([pre[s][a:a + c] for s, a, c in parts]).cuda()
        q_start = torch.tensor([0, parts[0][2], parts[0][2] + parts[1][2]], dtype=torch.int32, device="cuda")
        slots = torch.tensor([slot[0], slot[1]], dtype=torch.int32, device="cuda")
        out = torch.empty((x.shape[0], n), dtype=torch.float32, device="cuda")
        kernels.delta_scan(x, offs, p, ba.cuda(), w0.cuda(), state, q_start, slots, 2, out, heads, d)
        got[0].append(out[:parts[0][2]].cpu())
        got[1].append(out[parts[0][2]:].cpu())
        for s, a, c in parts:
            at[s] = a + c
    for s in lens:
        assert torch.allclose(torch.cat(got[s]).double(), want[s], atol=3e-5, rtol=3e-5)
    assert bool((state[1] == 0.0).all())


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_head_norm_and_the_weighted_sum_of_two_results(dtype):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(8)
    T, H, dv, off = 11, 3, 20, 7
    o, proj, w = torch.randn(T, H * dv, generator=g) * 3, torch.randn(T, off + H * dv + 2, generator=g), 1 + 0.2 * torch.randn(H * dv, generator=g)
    out = torch.empty((T, H * dv), dtype=dtype, device="cuda")
    kernels.gated_head_norm(o.cuda(), proj.cuda(), off, w.cuda(), out, H, dv, 1e-5)
    want = P.unit_rms(o.double().view(T, H, dv), 1e-5).reshape(T, -1) * w.double() * torch.sigmoid(proj.double()[:, off:off + H * dv])
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
    a, b = torch.randn(2, T, 16, generator=g), torch.randn(T, 16, generator=g)
    s = torch.empty((T, 16), dtype=torch.float32, device="cuda")
    kernels.scaled_sum(s, a.cuda(), 0.8, b.cuda(), -1.5)
    assert torch.allclose(s.cpu(), 0.8 * a.sum(0) + (-1.5) * b, atol=1e-5)


# ---- whole models through the step function --------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(NZ))
def test_whole_prompts_token_by_token_and_portions_agree_with_the_plain_model(models, name, dtype):
    runner = make_runner(models[name][0], dtype)
    for n in (1, 2, 3, 47, 150):
        toks = tokens_of(name, n)
        want = plain_logits(name, models, toks)
        whole = run_cuts(runner, "w", toks, [n])
        assert rel(whole, want) < TOL[dtype], f"{n} tokens at once"
        if n >= 47:
            head = n - 40
            one_by_one = run_cuts(runner, "d", toks, [head] + [1] * 40)
            assert rel(one_by_one, want) < TOL[dtype], f"{n} tokens, the last 40 one by one"
            sizes, cuts, left = [2, 3, 2, 17, 2, 5, 31, 2, 64], [], n
            while left:
                cuts.append(min(left, sizes[len(cuts) % len(sizes)]))
                left -= cuts[-1]
            portions = run_cuts(runner, "p", toks, cuts)
            assert rel(portions, want) < TOL[dtype], f"{n} tokens in portions"
            if dtype == "float32":                      # the cut must not show beyond rounding
                assert rel(one_by_one, whole) < 2e-6 and rel(portions, whole) < 2e-6
    runner.cache.check_invariants()
    assert runner.cache.num_free_slots() == 4


@gpu
@pytest.mark.parametrize("name", sorted(NZ))
def test_long_decoding_passes_windows_pooled_blocks_and_pages(models, name):
    """260 tokens, all but the first three one by one (through the decode graphs): every window, every pooled block's
    first appearance and every page border is crossed by a decoded token."""
    runner = make_runner(models[name][0], "float32", page_size=8, num_pages=40)
    toks = tokens_of(name, 260, salt=1)
    got = run_cuts(runner, "long", toks, [3] + [1] * 257)
    want = plain_logits(name, models, toks)
    worst = np.abs(got - want).max(axis=1) / np.abs(want).max()
    assert worst.max() < TOL["float32"], f"position {int(worst.argmax())}"
    assert runner.graph_steps > 200


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(NZ))
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
    worst = 0.0
    for st, rows in zip(b.steps, b.rows):
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]).float().cpu().numpy()
        for (rid, pos), row in zip(rows, logits):
            want = plain_logits(name, models, reqs[rid])
            worst = max(worst, float(np.abs(row - want[pos]).max() / np.abs(want).max()))
        for rid in st["end"]:
            runner.finish(rid)
    runner.check_status()
    assert worst < TOL[dtype]
    runner.cache.check_invariants()
    assert runner.cache.num_free_slots() == 3 and runner.cache.min_free_pages() > 0


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "c"])
def test_four_decoding_requests_beside_a_prompt_portion(models, name, dtype):
    """From four one-token requests on, a mixed step lays them out first and their attention takes the kernel made for
    decoding while the portion beside them takes the one for portions; every row still equals the plain model's."""
    from spyinfer_b200.engine.batch import StepEntry

    runner = make_runner(models[name][0], dtype, page_size=16, num_pages=60, max_num_seqs=5)
    olds = {f"o{n}": tokens_of(name, n, salt=5) for n in (70, 90, 33, 120)}
    new = tokens_of(name, 150, salt=6)
    for rid, toks in olds.items():                       # all but the last ten tokens of each
        runner.step([StepEntry(rid, toks[:-10], [])])
    worst, at = 0.0, 0
    for k, n in enumerate((37, 2, 41, 16, 3, 20, 5, 9, 11, 6)):
        entries = [StepEntry("new", new[at:at + n], list(range(n)))]
        entries[1:1] = [StepEntry(rid, [toks[len(toks) - 10 + k]], [0]) for rid, toks in olds.items()]     # the portion first, then the four
        logits = runner.step(entries).float().cpu().numpy()
        want_new = plain_logits(name, models, new)
        scale = np.abs(want_new).max()
        worst = max(worst, float(np.abs(logits[:n] - want_new[at:at + n]).max() / scale))
        for j, (rid, toks) in enumerate(olds.items()):
            want = plain_logits(name, models, toks)
            worst = max(worst, float(np.abs(logits[n + j] - want[len(toks) - 10 + k]).max() / np.abs(want).max()))
        at += n
    runner.check_status()
    assert at == len(new) and worst < TOL[dtype]


@gpu
def test_the_replay_program_runs_the_model(models, tmp_path):
    name = "a"
    rng = random.Random(2)
    reqs = {f"r{n}": tokens_of(name, n, salt=3) for n in (40, 3, 77, 25)}
    b = TraceBuilder()
    b.whole("whole", reqs["r77"])
    mixed_trace(b, reqs, {r: max(1, len(t) - 10) for r, t in reqs.items()}, rng, max_live=4, portion_sizes=(5, 2, 16))
    for dtype in ("float32", "bfloat16"):
        out = run_trace(models[name][0], dtype, b, str(tmp_path / dtype), peak_tokens(b), NZ[name]["config"]["vocab"])
        for (rid, pos), row in out.items():
            want = plain_logits(name, models, reqs["r77" if rid == "whole" else rid])
            assert np.abs(row - want[pos]).max() / np.abs(want).max() < TOL[dtype], (dtype, rid, pos)


@gpu
@pytest.mark.parametrize("name", ["a", "c"])
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
        for _ in range(new):
            logits = P.forward(w, cfg, toks)[-1]
            top = torch.topk(logits, 2).values
            assert (top[0] - top[1]).item() > 1e-3, "the test's greedy choice must not hang on rounding"
            toks.append(int(logits.argmax()))
        assert out == toks[len(prompt):]
    assert engine.stats()["free_slots"] == 3
