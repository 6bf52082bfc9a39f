"""The Daronex decoder in the engine against the plain implementation of ``plain_daronex.py``: each mechanism's kernel
alone, then whole models of several small configurations through the step function (whole prompts, token by token,
portions down to two tokens, unequal batches, pages and slots used again, long decoding), the replay program, and
greedy generation through ``LLMEngine`` and its scheduler.  Where random weights would hide a fault (one key among
hundreds, a window's edge, a page border) the inputs or the weights are made so that one score stands out."""
import json
import math
import random

import numpy as np
import pytest
import torch

import plain_daronex as P
from trace_tools import TraceBuilder, mixed_trace, peak_tokens, run_trace

gpu = pytest.mark.gpu


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims=None, window=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": dims if dims is not None else rot_dim}}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


# Five configurations that differ in every size and option.  a: every layer kind, a layer that reads another's cache and
# has no feed-forward, a rotation narrower than the rotated part, cache rows that the tensor-core attention takes.
# b: the recurrence first, one head, ranks that are no multiple of 8, a cache row that is no multiple of 4, a window
# shorter than a page, tau = 1, no logit multiplier, two layers reading one layer's cache.  c: sizes that the tensor-core
# products and attention take (a cache row of 128 and of 64), sixteen heads, a long window, two column tiles in the
# recurrence's state.  d: recurrent layers only (no pages at all), one without a feed-forward, a width that is no multiple
# of 16.  e: windowed layers only, one reading the other's cache, more than sixteen heads (the plain attention kernel
# in both formats), a window of one.
DX = {
    "a": dict(seed=11, config={
        "architecture": "Daronex", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 1.7,
        "layers": [
            {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 96}, "mixer": _latent(4, 16, 8, 24, 24, 24, 0.3, 500.0)},
            {"type": "gla", "mlp": {"kind": "dense", "ff": 80}, "mixer": {"heads": 2, "dim": 16, "vdim": 24, "tau": 4.0, "decay_rank": 8}},
            {"type": "latent_attention", "mlp": None, "mixer": _latent(2, 8, 8, 16, 16, 24, 0.5, 500.0, kv_from=0)},
            {"type": "latent_attention_2", "mlp": {"kind": "dense", "ff": 72}, "mixer": _latent(3, 16, 16, 8, 32, 32, 0.25, 10000.0, dims=8, window=20)},
        ]}),
    "b": dict(seed=12, config={
        "architecture": "Daronex", "vocab": 331, "width": 96, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
        "layers": [
            {"type": "gla", "mlp": {"kind": "dense", "ff": 128}, "mixer": {"heads": 3, "dim": 32, "vdim": 32, "tau": 1.0, "decay_rank": 4}},
            {"type": "latent_attention_2", "mlp": {"kind": "dense", "ff": 64}, "mixer": _latent(1, 24, 8, 40, 12, 40, 0.2, 1000.0, window=7)},
            {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 64}, "mixer": _latent(6, 8, 4, 8, 20, 18, 0.4, 300.0)},
            {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 48}, "mixer": _latent(2, 12, 4, 20, 10, 18, 0.3, 300.0, kv_from=2)},
            {"type": "latent_attention", "mlp": None, "mixer": _latent(3, 4, 4, 4, 36, 18, 0.6, 300.0, kv_from=2)},
        ]}),
    "c": dict(seed=13, config={
        "architecture": "Daronex", "vocab": 509, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 0.5,
        "layers": [
            {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 192}, "mixer": _latent(8, 32, 32, 32, 64, 96, 0.12, 50000.0)},
            {"type": "latent_attention_2", "mlp": {"kind": "dense", "ff": 160}, "mixer": _latent(16, 16, 16, 16, 48, 48, 0.17, 10000.0, window=64)},
            {"type": "gla", "mlp": {"kind": "dense", "ff": 160}, "mixer": {"heads": 4, "dim": 32, "vdim": 64, "tau": 16.0, "decay_rank": 16}},
        ]}),
    "d": dict(seed=14, config={
        "architecture": "Daronex", "vocab": 157, "width": 40, "norm": {"eps": 1e-5}, "logit_scale": 3.0,
        "layers": [
            {"type": "gla", "mlp": None, "mixer": {"heads": 1, "dim": 24, "vdim": 40, "tau": 2.0, "decay_rank": 3}},
            {"type": "gla", "mlp": {"kind": "dense", "ff": 56}, "mixer": {"heads": 5, "dim": 8, "vdim": 8, "tau": 8.0, "decay_rank": 8}},
        ]}),
    "e": dict(seed=15, config={
        "architecture": "Daronex", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "logit_scale": 1.2,
        "layers": [
            {"type": "latent_attention_2", "mlp": {"kind": "dense", "ff": 72}, "mixer": _latent(20, 8, 8, 4, 16, 16, 0.4, 100.0, window=25)},
            {"type": "latent_attention_2", "mlp": {"kind": "dense", "ff": 40}, "mixer": _latent(2, 16, 8, 16, 8, 16, 0.3, 100.0, window=25, kv_from=0)},
            {"type": "latent_attention_2", "mlp": None, "mixer": _latent(2, 8, 2, 8, 8, 6, 0.5, 10.0, window=1)},
        ]}),
}
TOL = {"float32": 2e-4, "bfloat16": 6e-2}      # largest difference over the largest logit


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (model folder, config, weights); written with the safetensors library, not with the package's writer.  The
    stored config.json of ``b`` leaves the decay rank out: the loader takes it from the tensor's shape."""
    from safetensors.torch import save_file

    out = {}
    for name, case in DX.items():
        d = tmp_path_factory.mktemp(f"dx_{name}")
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
    rng = random.Random(DX[name]["seed"] * 1000 + n + salt)
    return [rng.randrange(DX[name]["config"]["vocab"]) for _ in range(n)]


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
    from spyinfer_b200.config import ConfigError, DaronexConfig, config_from_json
    from spyinfer_b200.engine.model import declared_weights

    for name, case in DX.items():
        cfg = config_from_json(case["config"])
        assert isinstance(cfg, DaronexConfig)
        spec = cfg.to_spec()
        declared = {d.name: tuple(d.shape) for d in declared_weights(spec)}
        assert declared == P.tensor_shapes(case["config"]), name
        assert [e.cache_of for e in spec.run_order] == [l["mixer"].get("kv_from") for l in case["config"]["layers"]]
        assert config_from_json(cfg.to_json()).to_json() == cfg.to_json()
    base = DX["a"]["config"]

    def broken(change):
        c = json.loads(json.dumps(base))
        change(c)
        with pytest.raises(ConfigError):
            config_from_json(c).to_spec()

    broken(lambda c: c["layers"][0].update(type="attention"))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="experts"))
    broken(lambda c: c["layers"][2]["mixer"].update(kv_from=3))                    # a later layer
    broken(lambda c: c["layers"][2]["mixer"].update(kv_from=1))                    # no latent layer
    broken(lambda c: c["layers"][2]["mixer"].update(kv_rank=16))                   # another latent size than the layer it reads
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=16))               # wider than the rotated part
    broken(lambda c: c["layers"][3]["mixer"].pop("mask"))
    broken(lambda c: c["layers"][1]["mixer"].update(tau=0.0))
    broken(lambda c: c["layers"][1]["mixer"].pop("decay_rank"))                    # and no checkpoint to take it from
    broken(lambda c: c.pop("norm"))


def test_a_size_that_config_json_leaves_out_comes_from_the_tensors_shape(models):
    from spyinfer_b200.config import load_model_config

    cfg = load_model_config(models["b"][0])
    assert cfg.layers[0]["mixer"]["decay_rank"] == DX["b"]["config"]["layers"][0]["mixer"]["decay_rank"]


def test_latent_layers_keep_one_plane_and_a_reading_layer_keeps_nothing():
    from spyinfer_b200.cache import CacheManager
    from spyinfer_b200.config import PagedCacheNeed, StateCacheNeed, config_from_json
    from spyinfer_b200.engine.model import Model

    spec = config_from_json(DX["b"]["config"]).to_spec()
    model = Model(spec, torch.float32, None, 256)
    needs, cache_of = model.cache_needs()
    assert isinstance(needs[0], StateCacheNeed) and needs[0].shape == (3 * 32 * 32,)
    assert needs[1] == PagedCacheNeed(1, 48, 7, planes=1) and needs[2] == PagedCacheNeed(1, 22, None, planes=1)
    assert cache_of == [None, None, None, 2, 2] and needs[3] is None and needs[4] is None
    cache = CacheManager(needs, 8, 12, 2, 96, device=None, cache_of=cache_of, max_step_tokens=16)
    assert cache.num_groups() == 2                               # the window's and the full one; the readers add none
    assert cache.view(3).group == cache.view(2).group and not cache.view(3).writes and cache.view(2).writes
    assert CacheManager.bytes_per_page(needs, 8, torch.bfloat16) == 22 * 8 * 2      # one plane of the group that keeps every key
    with pytest.raises(ValueError):
        PagedCacheNeed(1, 8, planes=3)


def test_which_keys_the_plain_attention_sees():
    v = P.visible(6, 3)
    assert v[5].tolist() == [False, False, False, True, True, True] and v[1].tolist() == [True, True, False, False, False, False]
    assert P.visible(4, None)[2].tolist() == [True, True, True, False] and P.visible(3, 1).diagonal().all() and int(P.visible(3, 1).sum()) == 3


# ---- kernels alone ---------------------------------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_residual_norm_adds_the_normed_result_and_hands_out_a_copy(dtype):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(3)
    for rows, n, splits in ((5, 40, 1), (3, 200, 3), (9, 1000, 2), (4, 4096, 5), (2, 6144, 2), (600, 256, 2), (2, 50, 2)):
        h = torch.randn(rows, n, generator=g)
        y = torch.randn(splits, rows, n, generator=g) * 3
        w = (0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)
        want = h.double() + P.offset_norm(y.double().sum(0), w.double(), 1e-5)
        hd = h.cuda()
        copy = torch.empty((rows, n), dtype=dtype, device="cuda")
        stack = y.cuda() if splits > 1 else y[0].to(dtype).cuda()
        if splits == 1:
            want = h.double() + P.offset_norm(y[0].to(dtype).double(), w.double(), 1e-5)
        kernels.residual_norm(hd, stack, w.cuda(), 1e-5, weight_offset=1.0, copy=copy)
        assert torch.allclose(hd.cpu().double(), want, atol=2e-5, rtol=2e-6)
        assert torch.equal(copy.cpu(), hd.cpu().to(dtype))
        only = torch.empty((rows, n), dtype=dtype, device="cuda")
        kernels.residual_norm(hd, None, None, 0.0, copy=only)
        assert torch.equal(only, copy)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations_and_the_logit_multiplier(dtype):
    from spyinfer_b200 import kernels

    x = (torch.randn(7, 33, generator=torch.Generator().manual_seed(1)) * 3).to(dtype)
    xd = x.double()
    want = {"relu2": torch.relu(xd) ** 2, "relu": torch.relu(xd), "silu": xd * torch.sigmoid(xd),
            "gelu_tanh": 0.5 * xd * (1 + torch.tanh(math.sqrt(2 / math.pi) * (xd + 0.044715 * xd ** 3)))}
    for kind, w in want.items():
        out = torch.empty_like(x, device="cuda")
        kernels.activation(x.cuda(), out, kind)
        assert torch.allclose(out.cpu().double(), w, atol=1e-5, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5), kind
    z = torch.randn(5, 9).cuda()
    assert torch.allclose(kernels.scale_(z.clone(), 1.7), z * 1.7)
    with pytest.raises(kernels.KernelError):
        kernels.activation(x.cuda(), torch.empty_like(x, device="cuda"), "swish2")


@gpu
@pytest.mark.parametrize("M", [1, 8, 40, 100, 128, 200, 300, 640, 1200, 2048])
@pytest.mark.parametrize("N,K", [(320, 136), (4096, 1024), (6400, 2048)])
def test_product_with_the_relu_squared_epilogue(M, N, K):
    """The tensor-core product's epilogue squares relu of the result, on every kernel that the number of tokens selects
    (few-token tiles of each width, single blocks with shared K blocks, pairs of blocks with a shared last round)."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    out = kernels.gemm_tcgen05(a.cuda(), w.cuda(), epilogue="relu2")
    want = torch.relu(a.double() @ w.double().T) ** 2
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (M, N)
    assert torch.allclose(out.float().cpu().double(), want, atol=2e-2, rtol=2e-2)
    with pytest.raises(kernels.KernelError):
        kernels.gemm_tcgen05(a.cuda(), w.cuda(), epilogue="relu2", out_dtype=torch.float32)


def _pages_of(rows, page_size, page_ids, dtype, planes=1):
    """``rows [T, d]`` laid into pages ``[pages, planes, 1, page_size, d]`` (plane 0) at the given page ids, scattered on purpose."""
    T, d = rows.shape
    pages = torch.full((max(page_ids) + 2, planes, 1, page_size, d), 7.0, dtype=dtype)
    for t in range(T):
        pages[page_ids[t // page_size], 0, 0, t % page_size] = rows[t].to(dtype)
    return pages


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("q_rank,kv_rank,rot_dim,dims,page_size", [(24, 32, 16, 16, 8), (10, 18, 4, 4, 4), (72, 96, 32, 8, 16), (16, 6, 2, 2, 16)])
def test_latent_norms_rotation_and_cache_rows(dtype, interleaved, q_rank, kv_rank, rot_dim, dims, page_size):
    """The query latent's norm, the key/value latent's norm, the rotation of the shared key part and the row's place in
    the pages, for two requests whose tokens are mixed in one batch at positions of their own."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(q_rank + rot_dim)
    T, eps, base = 37, 1e-5, 300.0
    ld = 3 + q_rank + 5 + kv_rank + rot_dim
    off_q, off_c = 3, 3 + q_rank + 5
    fused = torch.randn(T, ld, generator=g) * 2
    wq, wc = 1 + 0.1 * torch.randn(q_rank, generator=g), 1 + 0.1 * torch.randn(kv_rank, generator=g)
    seq = torch.tensor([t % 2 for t in range(T)], dtype=torch.int32)
    pos = torch.tensor([40 + t // 2 if t % 2 == 0 else t // 2 for t in range(T)], dtype=torch.int32)
    inv = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32)
    table = kernels.build_rope_table(inv.cuda(), 128)
    width = kv_rank + rot_dim
    n_pages = -(-64 // page_size)
    ids = [list(range(2, 2 + n_pages)), list(range(2 + 2 * n_pages, 2 + n_pages, -1))]
    bt = torch.tensor(ids, dtype=torch.int32)
    pages = torch.full((3 + 2 * n_pages, 1, 1, page_size, width), 5.0, dtype=dtype, device="cuda")
    cq = torch.empty((T, q_rank), dtype=dtype, device="cuda")
    kernels.latent_prep(fused.cuda(), off_q, q_rank, wq.cuda(), cq, off_c, kv_rank, wc.cuda(), rot_dim, table, interleaved, pos.cuda(), seq.cuda(),
                        bt.cuda(), pages, eps)
    f = fused.double()
    want_q = P.rms(f[:, off_q:off_q + q_rank], eps) * wq.double()
    want_c = P.rms(f[:, off_c:off_c + kv_rank], eps) * wc.double()
    want_r = P.rotate(f[:, off_c + kv_rank:off_c + width], pos, base, dims, interleaved)
    tol = dict(atol=3e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=3e-5, rtol=1e-5)
    assert torch.allclose(cq.cpu().double(), want_q, **tol)
    host = pages.cpu()
    for t in range(T):
        row = host[ids[int(seq[t])][int(pos[t]) // page_size], 0, 0, int(pos[t]) % page_size].double()
        assert torch.allclose(row[:kv_rank], want_c[t], **tol) and torch.allclose(row[kv_rank:], want_r[t], **tol), t
    assert int((host == 5.0).all(dim=-1).sum()) == host.shape[0] * page_size - T          # every other row is untouched
    # a layer that reads another's cache norms its query latent and stores nothing
    before = pages.clone()
    kernels.latent_prep(fused.cuda(), off_q, q_rank, wq.cuda(), cq, -1, kv_rank, None, rot_dim, None, interleaved, pos.cuda(), seq.cuda(), None, None, eps)
    assert torch.equal(before, pages) and torch.allclose(cq.cpu().double(), want_q, **tol)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_per_head_products_with_a_rotated_tail_and_with_a_gate(dtype):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(8)
    for T, H, K, N, tail, dims, inter in ((19, 3, 16, 24, 8, 8, True), (9, 1, 24, 40, 8, 4, False), (33, 20, 8, 16, 8, 8, False), (5, 2, 12, 18, 0, 0, False)):
        x = torch.randn(T, H * (K + tail) + 3, generator=g).to(dtype)
        w = (torch.randn(H, K, N, generator=g) / math.sqrt(K)).to(torch.bfloat16)
        pos = torch.randint(0, 90, (T,), generator=g, dtype=torch.int32)
        table = kernels.build_rope_table(torch.tensor([50.0 ** (-2.0 * i / dims) for i in range(dims // 2)]).cuda(), 96) if dims else None
        out = torch.full((T, H * (N + tail) + 5), 3.0, dtype=dtype, device="cuda")
        kernels.head_product(x.cuda(), K + tail, w.cuda(), out, N + tail, tail=tail, rope_table=table, interleaved=inter, positions=pos.cuda())
        xin = x[:, :H * (K + tail)].double().view(T, H, K + tail)
        want = torch.einsum("thk,hkn->thn", xin[..., :K], w.double())
        if tail:
            want = torch.cat([want, P.rotate(xin[..., K:], pos, 50.0, dims, inter)], dim=-1)
        got = out.cpu().double()
        tol = dict(atol=4e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=2e-5, rtol=1e-5)
        assert torch.allclose(got[:, :H * (N + tail)].view(T, H, N + tail), want, **tol)
        assert bool((got[:, H * (N + tail):] == 3.0).all())
        gate = torch.randn(T, 7 + H * N, generator=g)
        out2 = torch.empty((T, H * N), dtype=dtype, device="cuda")
        kernels.head_product(x.cuda(), K + tail, w.cuda(), out2, N, gate=gate.cuda(), gate_offset=7)
        want2 = torch.einsum("thk,hkn->thn", xin[..., :K], w.double()) * torch.sigmoid(gate[:, 7:].double().view(T, H, N))
        assert torch.allclose(out2.cpu().double().view(T, H, N), want2, **tol)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,page_size,heads,rank,rot", [(None, 8, 4, 24, 8), (20, 8, 4, 24, 8), (7, 16, 2, 18, 4), (64, 16, 16, 48, 16), (None, 16, 8, 96, 32),
                                                              (1, 8, 3, 16, 8), (40, 16, 2, 512, 64)])
def test_attention_over_a_cache_of_one_plane_sees_exactly_its_keys(dtype, window, page_size, heads, rank, rot):
    """The cache holds rows ``[latent | rotated part]`` and the values are the rows' first ``rank`` elements.  For many
    (query, target) pairs the query is made to point at one row with a large score: a target far back, at a page's first
    or last place, at the window's oldest place, one before that (seen by nobody), the query's own and the sequence's first
    tokens.  Compared with the plain softmax row by row, on the plain kernel and, in bfloat16 where they take the sizes,
    on the tensor-core kernels for portions and for decoding."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed((window or 0) * 100 + rank)
    T, d = 300, rank + rot
    rows = torch.randn(T, d, generator=g)
    rows = (rows / rows.norm(dim=-1, keepdim=True)).to(dtype).float()
    q = torch.zeros(T, heads, d)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        edges = [lo, lo - 1, i, 0, 1, (i // page_size) * page_size, (i // page_size) * page_size - 1, i // 3, lo + 1]
        for h in range(heads):
            j = min(max(edges[(i + h) % len(edges)], 0), i)
            q[i, h] = 50.0 * rows[j]
    q = q.to(dtype).float()
    s = torch.einsum("ihd,jd->hij", q.double(), rows.double()).masked_fill(~P.visible(T, window)[None], -math.inf)
    want = torch.einsum("hij,jd->ihd", torch.softmax(s, dim=-1), rows.double())[..., :rank]
    n_pages = -(-T // page_size)
    ids = list(reversed(range(3, 3 + n_pages)))
    pages = _pages_of(rows, page_size, ids, dtype).cuda()
    bt = torch.full((2, n_pages + 1), -1, dtype=torch.int32)
    bt[1, :n_pages] = torch.tensor(ids, dtype=torch.int32)
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    q_dev = q.to(dtype).reshape(T, heads * d).cuda()
    out = torch.empty((T, heads * d), dtype=dtype, device="cuda")
    kernels.attention_generic(q_dev, heads, d, out, pages, bt.cuda(), positions, torch.ones(T, dtype=torch.int32, device="cuda"), 1.0, window=window)
    tol = 3e-2 if dtype == torch.bfloat16 else 2e-5
    worst = (out.float().cpu().view(T, heads, d)[..., :rank].double() - want).abs().amax(dim=(1, 2))
    assert worst.max().item() < tol, f"query {int(worst.argmax())} differs by {worst.max().item()}"
    if dtype != torch.bfloat16 or not kernels.attention_decode_takes(heads, 1, d, page_size, dtype):
        assert dtype != torch.bfloat16 or d % 8 != 0 or heads > 16 or d > 128      # why the tensor-core kernels do not take these sizes
        return
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    out2 = torch.full((T, heads * d), 3.0, dtype=dtype, device="cuda")                  # one prompt of T tokens ...
    kernels.attention_tc(q_dev, heads, d, out2, pages, bt[1:2].contiguous().cuda(), positions, i32([0, T]), 1, 1.0, window=window)
    worst = (out2.float().cpu().view(T, heads, d)[..., :rank].double() - want).abs().amax(dim=(1, 2))
    assert worst.max().item() < 6e-2, f"prompt path: query {int(worst.argmax())} differs by {worst.max().item()}"
    out3 = torch.full((T, heads * d), 3.0, dtype=dtype, device="cuda")                  # ... and T requests that decode one token each
    kernels.attention_decode(q_dev, heads, d, out3, pages, bt[1:2].expand(T, bt.shape[1]).contiguous().cuda(), positions, i32(list(range(T + 1))), T, 1.0,
                             window=window)
    worst = (out3.float().cpu().view(T, heads, d)[..., :rank].double() - want).abs().amax(dim=(1, 2))
    assert worst.max().item() < 6e-2, f"decode path: query {int(worst.argmax())} differs by {worst.max().item()}"


@gpu
@pytest.mark.parametrize("heads,dk,dv,tau", [(2, 16, 24, 4.0), (1, 48, 72, 1.0), (3, 8, 8, 16.0), (2, 32, 40, 2.0)])
def test_gated_linear_attention_scan_carries_its_state_through_portions_and_slots(heads, dk, dv, tau):
    """Two requests in slots 0 and 2, fed in portions of unequal sizes (single tokens among them, and one step in which
    both bring one token: the kernel made for decoding); slot 1 stays untouched."""
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(dk + dv)
    n, nv = heads * dk, heads * dv
    lens, cuts = {0: 20, 1: 9}, {0: [2, 1, 9, 1, 7], 1: [1, 2, 4, 1, 1]}
    ld = 2 * n + nv + 5
    offs = (5, 5 + n, 5 + 2 * n)
    proj = {s: torch.randn(t, ld, generator=g) for s, t in lens.items()}
    pre = {s: torch.randn(t, n, generator=g) * 2 for s, t in lens.items()}
    bias = torch.randn(n, generator=g) + 1.0
    want = {}
    for s, x in proj.items():
        x = x.double()
        q, k = (x[:, o:o + n].view(-1, heads, dk) for o in offs[:2])
        v = x[:, offs[2]:offs[2] + nv].view(-1, heads, dv)
        alpha = torch.sigmoid(pre[s].double() + bias.double()).pow(1.0 / tau).view(-1, heads, dk)
        want[s] = P.gla_recurrence(q * dk ** -0.5, k, v, alpha)[0].reshape(-1, nv)
    state = torch.zeros((3, heads * dk * dv), dtype=torch.float32, device="cuda")
    slot = {0: 0, 1: 2}
    got, at = {0: [], 1: []}, {0: 0, 1: 0}
    for step in range(5):
        parts = [(s, at[s], cuts[s][step]) for s in (0, 1)]
        x = torch.cat([proj[s][a:a + c] for s, a, c in parts]).cuda()
        p = torch.cat([pre[s][a:a + c] for s, a, c in parts]).cuda()
        q_start = torch.tensor([0, parts[0][2], parts[0][2] + parts[1][2]], dtype=torch.int32, device="cuda")
        slots = torch.tensor([slot[0], slot[1]], dtype=torch.int32, device="cuda")
        out = torch.empty((x.shape[0], nv), dtype=torch.float32, device="cuda")
        one_each = all(c == 1 for _, _, c in parts)
        kernels.gla_scan(x, offs, p, bias.cuda(), tau, state, q_start, slots, 2, out, heads, dk, dv, dk ** -0.5, longest=1 if one_each else None)
        got[0].append(out[:parts[0][2]].cpu())
        got[1].append(out[parts[0][2]:].cpu())
        for s, a, c in parts:
            at[s] = a + c
    for s in lens:
        assert torch.allclose(torch.cat(got[s]).double(), want[s], atol=3e-5, rtol=3e-5)
    assert bool((state[1] == 0.0).all())


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_with_a_silu_gate_and_columns_taken_as_they_are(dtype):
    from spyinfer_b200 import kernels

    g = torch.Generator().manual_seed(4)
    T, H, dv = 11, 3, 20
    o, proj, w = torch.randn(T, H * dv, generator=g) * 5, torch.randn(T, 7 + H * dv, generator=g), 1 + 0.1 * torch.randn(dv, generator=g)
    y = torch.empty((T, H * dv), dtype=dtype, device="cuda")
    kernels.gated_head_norm(o.cuda(), proj.cuda(), 7, w.repeat(H).cuda(), y, H, dv, 1e-5, gate="silu")
    gate = proj[:, 7:].double()
    want = (P.rms(o.double().view(T, H, dv), 1e-5) * w.double()).reshape(T, H * dv) * (gate * torch.sigmoid(gate))
    assert torch.allclose(y.float().cpu().double(), want, atol=3e-2 if dtype == torch.bfloat16 else 1e-5, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5)
    cols = torch.empty((T, 9), dtype=dtype, device="cuda")
    kernels.tanh_cols(proj.cuda(), 4, 9, cols, activation="none")
    assert torch.equal(cols.cpu(), proj[:, 4:13].to(dtype))


# ---- whole models through the step function --------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(DX))
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
                assert rel(one_by_one, whole) < 4e-6 and rel(portions, whole) < 4e-6
    runner.cache.check_invariants()
    assert runner.cache.num_free_slots() == 4


@gpu
@pytest.mark.parametrize("name", sorted(DX))
def test_long_decoding_passes_windows_and_pages(models, name):
    """260 tokens, all but the first three one by one (through the decode graphs): every window and every page border is
    crossed by a decoded token, and the recurrence runs 257 steps on its own state."""
    runner = make_runner(models[name][0], "float32", page_size=8, num_pages=40)
    toks = tokens_of(name, 260, salt=1)
    got = run_cuts(runner, "long", toks, [3] + [1] * 257)
    want = plain_logits(name, models, toks)
    worst = np.abs(got - want).max(axis=1) / np.abs(want).max()
    assert worst.max() < TOL["float32"], f"position {int(worst.argmax())}"
    assert runner.graph_steps > 200


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(DX))
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


def _pointing_model(tmp_path, window):
    """A one-layer model (latent attention, windowed or not, no feed-forward) whose weights are made so that the token
    ``A`` as a query points at the token ``B`` as a key with a large score on its first head, wherever the two stand: the
    embedding of B is solved for so that its latent is the direction that A's absorbed query likes best."""
    from safetensors.torch import save_file

    kind = "latent_attention_2" if window else "latent_attention"
    cfg = {"architecture": "Daronex", "vocab": 60, "width": 48, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
           "layers": [{"type": kind, "mlp": None, "mixer": _latent(2, 16, 4, 12, 16, 24, 1.0, 100.0, window=window)}]}
    w = {k: v.double() for k, v in P.random_weights(cfg, 77, gain=1.5).items()}
    A, B, r, eps = 58, 59, 24, 1e-5
    cq = P.rms(w["embed"][A] @ w["l0.mix.dq"].T, eps) * w["l0.mix.dq.norm"]
    q = (cq @ w["l0.mix.uq"].T).view(2, 20)[:, :16]
    liked = w["l0.mix.uk"].view(2, 16, r)[0].T @ q[0]                               # the latent direction that the first head's query scores highest
    target = liked / w["l0.mix.dkv.norm"]
    w["embed"][B] = torch.linalg.pinv(w["l0.mix.dkv"][:r]) @ target
    w["embed"][B] *= w["embed"][0].norm() / w["embed"][B].norm()
    w["l0.mix.dkv"][r:] *= 0.05                                                     # the shared rotated part carries little: the score is the latent's
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    d = tmp_path / f"point_{window}"
    d.mkdir()
    with open(d / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
    return str(d), cfg, w, A, B


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 40])
def test_a_query_that_points_at_one_key_finds_it_far_back_and_at_every_edge(tmp_path, dtype, window):
    """The key token stands once in a sequence of 400 others; the query token is asked at places where the key is far
    back, at a page's first or last place, the window's oldest place or one before it, and among the first tokens.  The
    plain model says how much of the weight the key gets (nearly all, or none); the engine's logits there equal the plain
    model's, whole, in portions and decoded one by one."""
    model_dir, cfg, w, A, B = _pointing_model(tmp_path, window)
    rng = random.Random(5)
    n, key_at = 400, 150 if window else 300
    toks = [rng.randrange(50) for _ in range(n)]
    toks[key_at] = B
    toks[1] = B
    if window:
        asks = [key_at + window - 1, key_at + window, key_at + 1, key_at + window - 2, 1 + window - 1, 1 + window, 3]
    else:
        asks = [key_at + 1, 399, key_at + 16 - key_at % 16, key_at + 15 - key_at % 16, 350, 2, 17]
    for a in asks:
        toks[a] = A
    probs = []
    want = P.forward(w, cfg, toks, probs_out=probs).numpy()
    seen = [float(probs[0][0, a, [1, key_at]].sum()) for a in asks]
    if window:
        assert seen[0] > 0.9 and seen[1] == 0.0 and seen[2] > 0.9 and seen[4] > 0.9 and seen[5] == 0.0 and seen[6] > 0.9
    else:
        assert min(seen) > 0.9
    runner = make_runner(model_dir, dtype, page_size=16, num_pages=30)
    whole = run_cuts(runner, "w", toks, [n])
    worst = np.abs(whole - want).max(axis=1) / np.abs(want).max()
    assert worst[asks].max() < TOL[dtype] and worst.max() < TOL[dtype], f"whole: position {int(worst.argmax())}"
    cuts = [key_at - 1, 2] + [1] * (n - key_at - 1)
    decoded = run_cuts(runner, "d", toks, cuts)
    worst = np.abs(decoded - want).max(axis=1) / np.abs(want).max()
    assert worst.max() < TOL[dtype], f"decoded: position {int(worst.argmax())}"
    sizes, cuts, left = [3, 61, 2, 16, 2, 45, 7], [], n
    while left:
        cuts.append(min(left, sizes[len(cuts) % len(sizes)]))
        left -= cuts[-1]
    portions = run_cuts(runner, "p", toks, cuts)
    worst = np.abs(portions - want).max(axis=1) / np.abs(want).max()
    assert worst.max() < TOL[dtype], f"portions: position {int(worst.argmax())}"


@gpu
def test_the_replay_program_runs_the_model(models, tmp_path):
    name = "a"
    rng = random.Random(2)
    reqs = {f"r{n}": tokens_of(name, n, salt=3) for n in (40, 3, 77, 25)}
    b = TraceBuilder()
    b.whole("whole", reqs["r77"])
    mixed_trace(b, reqs, {r: max(1, len(t) - 10) for r, t in reqs.items()}, rng, max_live=4, portion_sizes=(5, 2, 16))
    for dtype in ("float32", "bfloat16"):
        out = run_trace(models[name][0], dtype, b, str(tmp_path / dtype), peak_tokens(b), DX[name]["config"]["vocab"])
        for (rid, pos), row in out.items():
            want = plain_logits(name, models, reqs["r77" if rid == "whole" else rid])
            assert np.abs(row - want[pos]).max() / np.abs(want).max() < TOL[dtype], (dtype, rid, pos)


@gpu
@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_through_the_engine_and_its_scheduler(models, name):
    """Five prompts of unequal length, three slots, prompts cut by a small token budget, pages so few that requests wait
    and are preempted: the tokens equal the plain model's greedy continuation."""
    from spyinfer_b200 import LLMEngine, SamplingParams

    model_dir, cfg, w = models[name]
    prompts = [tokens_of(name, n, salt=4 if name == "a" else 7) for n in (30, 3, 55, 1, 18)]
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
