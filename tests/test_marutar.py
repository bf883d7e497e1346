"""Marutar through the framework against the plain implementation (plain_marutar.py): configuration and names, each mechanism
alone, and the engine's step function under every way of cutting the work.  The CPU tests run the engine's host logic with the
plain kernels standing in; the ``gpu`` tests run the kernels."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import plain_marutar
import plain_ops
import trace_tools
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.config import load_model_config
from tinyllama_inference_engine_b200.engine.batch import StepEntry
from tinyllama_inference_engine_b200.engine.runner import ModelRunner
from tinyllama_inference_engine_b200.errors import ConfigError
from tinyllama_inference_engine_b200.models import expected_tensors
from tinyllama_inference_engine_b200.models.marutar_config import MarutarConfig
from tinyllama_inference_engine_b200.weights import SafetensorsFile, write_random_model, write_safetensors


def _attention(heads, kv_heads, dim, vdim, window, mlp=None, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer, "mlp": None if mlp is None else {"kind": "dense", "ff": mlp}}


def _mingru(width, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": None if mlp is None else {"kind": "dense", "ff": mlp}}


def _config(width, vocab, positions, layers, eps=1e-5):
    return {"architecture": "Marutar", "vocab": vocab, "width": width, "max_positions": positions, "norm": {"eps": eps}, "layers": layers}


# Sizes that agree nowhere: key and value widths differ or not, one key/value head or as many as query heads, windows of one token, of
# exactly a page and of none, widths that are no multiple of a warp or of eight, layers with and without a feed-forward.
CONFIGS = {
    "mixed": (_config(48, 101, 224, [_mingru(40, 56), _attention(4, 2, 16, 24, 20), _mingru(33), _attention(3, 3, 8, 8, 7, mlp=64)]), 3),
    "wide_heads": (_config(64, 77, 400, [_attention(6, 1, 32, 16, 0, mlp=40), _mingru(64, 96), _attention(2, 2, 40, 48, 16)], eps=1e-6), 5),
    "ones": (_config(40, 53, 160, [_attention(1, 1, 16, 16, 1), _mingru(1), _attention(5, 1, 12, 20, 33, mlp=24, scale=0.3), _mingru(72, 8)]), 9),
    "recurrent_only": (_config(56, 64, 700, [_mingru(48), _mingru(80, 32)]), 4),
}
LENGTHS = {"mixed": [1, 9, 70, 150, 33, 64, 17], "wide_heads": [2, 130, 65, 16, 300], "ones": [3, 40, 100, 64, 7], "recurrent_only": [600, 5, 130]}
TOLERANCE = {"float32": 3e-5, "bfloat16": 2.5e-2}


def load_plain(folder):
    config = json.loads((folder / "config.json").read_text())
    file = SafetensorsFile(folder / "model.safetensors")
    tensors = {name: file.tensor(name).clone() for name in file.names()}
    file.close()
    return config, tensors


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("marutar")
    return {key: write_random_model(base / key, config, seed) for key, (config, seed) in CONFIGS.items()}


@pytest.fixture(scope="module")
def cases(folders):
    out = {}
    for key, folder in folders.items():
        config, tensors = load_plain(folder)
        requests = trace_tools.make_requests(config["vocab"], LENGTHS[key], seed=21)
        full = {rid: plain_marutar.forward(config, tensors, tokens) for rid, tokens in requests.items()}
        out[key] = (folder, requests, full, max(float(v.abs().max()) for v in full.values()))
    return out


def _runner(folder, dtype, device="cuda:0", max_tokens=1024, page_size=16, requests=4):
    return ModelRunner(folder, EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=max_tokens, max_requests=requests, max_batch_tokens=1024,
                                            device=device, poison_freed_pages=True, use_cuda_graphs=False))


def _schedules(requests, seed=3, page_size=16):
    mixed, peak = trace_tools.mixed(requests, seed=seed, page_size=page_size)
    return {"whole": (trace_tools.whole(requests), 1024), "decode": (trace_tools.tail_decode(requests), 1024), "portions": (trace_tools.portions(requests), 1024),
            "mixed": (mixed, peak)}   # a pool of exactly the peak: pages are used again, and with four slots so are the state slots


# --- configuration, registry, names ----------------------------------------------------------------------------------------------
def test_configuration_round_trip_and_registry(folders):
    architecture, config = load_model_config(folders["mixed"])
    assert architecture.name == "Marutar" and isinstance(config, MarutarConfig)
    assert MarutarConfig.from_dict(config.to_dict()) == config
    assert config.layers[1]["mixer"]["mask"] == {"size": 20} and config.layers[0]["mlp"] == {"kind": "dense", "ff": 56} and config.layers[2]["mlp"] is None
    spec = architecture.build_spec(config)
    names = {t.name: tuple(t.shape) for t in expected_tensors(spec)}
    assert names["embed"] == (101, 48) and names["pos"] == (224, 48) and names["embed.norm"] == (48,) and names["final.norm"] == (48,) and names["head"] == (101, 48)
    assert names["l0.mix.z"] == (40, 48) and names["l0.mix.z.b"] == (40,) and names["l0.mix.o"] == (48, 40) and names["l0.mlp.up"] == (56, 48)
    assert names["l1.mix.q"] == (64, 48) and names["l1.mix.k"] == (32, 48) and names["l1.mix.v"] == (48, 48) and names["l1.mix.g"] == (96, 48)
    assert names["l1.mix.talk"] == (4, 4) and names["l1.mix.o"] == (48, 96) and "l1.norm2" not in names and "l2.mlp.up" not in names and "l3.norm2" in names


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="lstm"), "type"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "dense"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][1]["mixer"].update(mask={"size": 0}), "mask.size"),
])
def test_configuration_refuses_what_the_design_lacks(change, message):
    data = json.loads(json.dumps(CONFIGS["mixed"][0]))
    change(data)
    with pytest.raises(ConfigError, match=message):
        MarutarConfig.from_dict(data)


def test_cache_groups_follow_the_mixers(folders, monkeypatch):
    plain_ops.install(monkeypatch)
    runner = _runner(folders["mixed"], "float32", device="cpu")
    pages = [(g.need.window, g.need.page_planes(), g.streams) for g in runner.cache.page_groups]
    assert pages == [(20, ((2, 16), (2, 24)), [1]), (7, ((3, 8), (3, 8)), [3])]
    assert [(g.need.state_shape, g.streams) for g in runner.cache.state_groups] == [((40,), [0]), ((33,), [2])]
    assert runner.cache.page_groups[0].tensor is None and len(runner.cache.page_groups[0].plane_tensors) == 2     # unequal planes: a tensor each
    assert runner.cache.page_groups[1].tensor is not None
    assert runner.model.capturable


# --- the plain implementation's own mechanisms ------------------------------------------------------------------------------------
def test_plain_mingru_carries_its_state():
    g = torch.Generator().manual_seed(1)
    t = {f"m.{n}": torch.randn(12, 20, generator=g) * 0.3 for n in ("z", "x", "g")}
    t.update({"m.z.b": torch.randn(12, generator=g), "m.x.b": torch.randn(12, generator=g), "m.o": torch.randn(20, 12, generator=g)})
    h = torch.randn(30, 20, generator=g)
    whole, last = plain_marutar.mingru_mixer(h, t, "m")
    first, state = plain_marutar.mingru_mixer(h[:11], t, "m")
    second, end = plain_marutar.mingru_mixer(h[11:], t, "m", state)
    assert torch.allclose(torch.cat([first, second]), whole, atol=1e-6) and torch.allclose(end, last, atol=1e-6)
    u = torch.tensor([-2.0, -1e-9, 0.0, 3.0])
    assert torch.allclose(plain_marutar.mingru_candidate(u), torch.tensor([float(torch.sigmoid(torch.tensor(-2.0))), 0.5, 0.5, 3.5]))


def test_plain_attention_window_and_bias():
    """A key one step outside the window changes nothing, the last one inside does; the bias grows with distance by each head's slope."""
    g = torch.Generator().manual_seed(2)
    mixer = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.5, "mask": {"size": 5}}
    t = {"a.q": torch.randn(32, 16, generator=g), "a.k": torch.randn(16, 16, generator=g), "a.v": torch.randn(12, 16, generator=g),
         "a.g": torch.randn(24, 16, generator=g), "a.o": torch.randn(16, 24, generator=g), "a.talk": torch.randn(4, 4, generator=g)}
    h = torch.randn(12, 16, generator=g)
    base = plain_marutar.attention_mixer(h, t, "a", mixer)
    outside, inside = h.clone(), h.clone()
    outside[6] += 1.0     # row 11 sees 7..11
    inside[7] += 1.0
    assert torch.equal(plain_marutar.attention_mixer(outside, t, "a", mixer)[11], base[11])
    assert not torch.allclose(plain_marutar.attention_mixer(inside, t, "a", mixer)[11], base[11])
    assert torch.allclose(plain_marutar.head_slopes(4), torch.tensor([0.25, 0.0625, 2.0 ** -6, 2.0 ** -8]))
    no_window = plain_marutar.attention_mixer(outside, t, "a", {k: v for k, v in mixer.items() if k != "mask"})
    assert not torch.allclose(no_window[11], plain_marutar.attention_mixer(h, t, "a", {k: v for k, v in mixer.items() if k != "mask"})[11])


# --- the engine's host logic on the CPU, the plain kernels standing in -----------------------------------------------------------------
@pytest.mark.parametrize("key", ["mixed", "ones"])
def test_engine_logic_on_cpu(cases, key, monkeypatch):
    plain_ops.install(monkeypatch)
    folder, requests, full, scale = cases[key]
    short = {rid: tokens for rid, tokens in requests.items() if len(tokens) <= 70}
    for name, (steps, pool) in _schedules(short).items():
        runner = _runner(folder, "float32", device="cpu", max_tokens=pool)
        trace_tools.run_and_compare(runner, steps, full, atol=TOLERANCE["float32"] * scale)
        runner.cache.check()
        assert not runner.cache.records


# --- kernels alone --------------------------------------------------------------------------------------------------------------------
def _cuda(t):
    return None if t is None else t.cuda()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,atol", [(torch.float32, 2e-6), (torch.bfloat16, 1.6e-2)])
@pytest.mark.parametrize("width,lens", [(33, [1, 1, 1]), (64, [70, 1, 2, 31]), (40, [600]), (1, [5, 1]), (200, [17, 16, 33, 1])])
def test_mingru_scan_kernel(dtype, atol, width, lens):
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(width + len(lens))
    tokens = sum(lens)
    zxg = (torch.randn(tokens, 3 * width, generator=g) * 1.5).to(dtype)
    bias_z, bias_x = torch.randn(width, generator=g) - 2.0, torch.randn(width, generator=g)
    state = torch.randn(7, width, generator=g)
    starts = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    slots = torch.tensor([5, 0, 3, 6][: len(lens)], dtype=torch.int32)
    want_state, want = state.clone(), torch.zeros(tokens, width, dtype=dtype)
    plain_ops.mingru_scan(zxg, bias_z, bias_x, want_state, starts, slots, want, max(lens))
    got_state, got = state.cuda(), torch.zeros(tokens, width, dtype=dtype, device="cuda")
    ops.mingru_scan(zxg.cuda(), bias_z.cuda(), bias_x.cuda(), got_state, starts.cuda(), slots.cuda(), got, max(lens))
    assert torch.allclose(got_state.cpu(), want_state, atol=2e-5, rtol=1e-5)
    assert float((got.cpu().float() - want.float()).abs().max()) <= atol * max(1.0, float(want.float().abs().max()))
    untouched = [s for s in range(7) if s not in slots.tolist()]
    assert torch.equal(got_state.cpu()[untouched], state[untouched])


def _attention_case(dtype, heads, kv, key_dim, value_dim, lens, firsts, gate, page_size=16):
    """Rows of some requests at given positions over pages handed out in a scrambled order; returns what both implementations take."""
    from types import SimpleNamespace

    from tinyllama_inference_engine_b200.parts.base import CacheNeed, LayerCache

    g = torch.Generator().manual_seed(heads * 100 + key_dim + len(lens))
    width = max(-(-(f + n) // page_size) for n, f in zip(lens, firsts))
    count = sum(-(-(f + n) // page_size) for n, f in zip(lens, firsts)) + 3
    order = torch.randperm(count, generator=g).tolist()
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    for r, (n, f) in enumerate(zip(lens, firsts)):
        for p in range(-(-(f + n) // page_size)):
            table[r, p] = order.pop()
    columns = heads * key_dim + kv * key_dim + kv * value_dim + (heads * value_dim if gate else 0)
    if key_dim == value_dim:
        pages = torch.randn(count, 2, kv, page_size, key_dim, generator=g).to(dtype)
        cpu_cache = LayerCache(CacheNeed("pages"), True, pages, table, page_size)
        gpu_cache = LayerCache(CacheNeed("pages"), True, pages.cuda(), table.cuda(), page_size)
    else:
        planes = (torch.randn(count, kv, page_size, key_dim, generator=g).to(dtype), torch.randn(count, kv, page_size, value_dim, generator=g).to(dtype))
        cpu_cache = LayerCache(CacheNeed("pages"), True, None, table, page_size, None, planes)
        gpu_cache = LayerCache(CacheNeed("pages"), True, None, table.cuda(), page_size, None, tuple(p.cuda() for p in planes))
    rows = torch.randn(sum(lens), columns, generator=g).to(dtype)
    positions = torch.tensor([f + i for n, f in zip(lens, firsts) for i in range(n)], dtype=torch.int32)
    token_seq = torch.tensor([r for r, n in enumerate(lens) for _ in range(n)], dtype=torch.int32)
    starts = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    batch = SimpleNamespace(max_q_len=max(lens), num_seqs=len(lens), max_seq_len=max(f + n for n, f in zip(lens, firsts)), seq_starts=starts.cuda(),
                            first_positions=torch.tensor(firsts, dtype=torch.int32).cuda(), num_tokens=sum(lens))
    mixing = torch.randn(heads, heads, generator=g) * 1.2 * heads ** -0.5      # mixed scores of the same size whatever the number of heads
    return rows, positions, token_seq, cpu_cache, gpu_cache, batch, mixing


def _compare_attention(dtype, atol, heads, kv, key_dim, value_dim, window, bias, mix, gate, lens, firsts, with_batch):
    from tinyllama_inference_engine_b200 import ops

    rows, positions, token_seq, cpu_cache, gpu_cache, batch, mixing = _attention_case(dtype, heads, kv, key_dim, value_dim, lens, firsts, gate)
    slopes = torch.tensor(plain_marutar.head_slopes(heads).tolist(), dtype=torch.float32) if bias else None
    mixing = mixing if mix else None
    k_offset, v_offset = heads * key_dim, heads * key_dim + kv * key_dim
    gate_offset = v_offset + kv * value_dim if gate else -1
    want = torch.zeros(sum(lens), heads * value_dim, dtype=dtype)
    plain_ops.store_kv_planes(rows, k_offset, v_offset, positions, token_seq, cpu_cache, kv, key_dim, value_dim)
    plain_ops.mixed_heads_attention(rows, gate_offset, positions, token_seq, cpu_cache, slopes, mixing, want, heads, kv, key_dim, value_dim, window, 0.3)
    got = torch.zeros(sum(lens), heads * value_dim, dtype=dtype, device="cuda")
    before = ops.launch_count
    ops.store_kv_planes(rows.cuda(), k_offset, v_offset, positions.cuda(), token_seq.cuda(), gpu_cache, kv, key_dim, value_dim)
    ops.mixed_heads_attention(rows.cuda(), gate_offset, positions.cuda(), token_seq.cuda(), gpu_cache, _cuda(slopes), _cuda(mixing), got, heads, kv, key_dim,
                              value_dim, window, 0.3, batch=batch if with_batch else None)
    for mine, theirs in zip([gpu_cache.pages] if key_dim == value_dim else gpu_cache.plane_pages, [cpu_cache.pages] if key_dim == value_dim else cpu_cache.plane_pages):
        assert torch.equal(mine.cpu(), theirs)
    assert float((got.cpu().float() - want.float()).abs().max()) <= atol * max(1.0, float(want.float().abs().max()))
    return ops.launch_count - before


ATTENTION_SHAPES = [
    (4, 2, 16, 16, 20, True, True, True), (4, 2, 16, 24, 0, True, True, True), (3, 3, 8, 8, 7, False, True, False), (6, 1, 32, 16, 33, True, False, True),
    (1, 1, 12, 20, 1, True, True, True), (8, 4, 112, 80, 16, True, True, True), (5, 5, 10, 6, 17, False, False, False),
    (8, 8, 128, 128, 40, True, True, True),     # a tile of all its key/value heads does not fit shared memory in 32-bit: rows come from global memory
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,atol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("heads,kv,key_dim,value_dim,window,bias,mix,gate", ATTENTION_SHAPES)
def test_mixed_heads_attention_kernel(dtype, atol, heads, kv, key_dim, value_dim, window, bias, mix, gate):
    """The general kernel: a portion from position 0, a decoded token, and a portion that starts inside a page; every option on and off."""
    _compare_attention(dtype, atol, heads, kv, key_dim, value_dim, window, bias, mix, gate, [37, 1, 18], [0, 52, 30], with_batch=False)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,kv,key_dim,value_dim,window,bias,mix,gate", [
    (4, 2, 16, 16, 20, True, True, True), (8, 4, 112, 80, 16, True, True, True), (6, 1, 32, 16, 33, True, False, True), (4, 2, 16, 32, 0, True, True, False),
    (2, 2, 48, 48, 70, False, True, True), (3, 1, 64, 64, 64, True, True, True), (6, 3, 32, 48, 1, True, True, True), (4, 4, 64, 16, 129, False, False, False),
])
def test_mixed_heads_attention_on_tensor_cores(heads, kv, key_dim, value_dim, window, bias, mix, gate):
    """The prompt kernel (mix folded into the queries, flash attention over the concatenated key heads): portions that start at 0, inside
    a page and far into a request, of 1 to 150 rows, against the plain function; the step's shape makes the wrapper choose it."""
    launches = _compare_attention(torch.bfloat16, 1.6e-2, heads, kv, key_dim, value_dim, window, bias, mix, gate, [1, 150, 18, 70, 1], [77, 0, 30, 215, 3], with_batch=True)
    assert launches == 3      # the store, the fold and the attention: not the general kernel


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,atol", [(torch.float32, 4e-5), (torch.bfloat16, 1.6e-2)])     # a thousand keys under a sharp softmax: 32-bit sums in another order differ by 2e-5 of the largest output
@pytest.mark.parametrize("heads,kv,key_dim,value_dim,window,bias,mix,gate", [
    (4, 2, 16, 16, 300, True, True, True), (8, 4, 112, 80, 0, True, True, True), (3, 1, 24, 40, 0, True, True, True), (16, 8, 32, 32, 5, True, True, False),
    (6, 3, 32, 48, 1, False, True, True), (16, 1, 64, 16, 0, True, False, True), (32, 4, 64, 64, 500, True, True, True), (10, 5, 16, 16, 33, True, True, True),
])
def test_mixed_heads_attention_of_few_rows(dtype, atol, heads, kv, key_dim, value_dim, window, bias, mix, gate):
    """Steps of few rows: each row's key tiles are dealt to several CTAs and merged (rows at 3 and 40 keys leave CTAs empty); in bfloat16
    with widths that are multiples of 16 the two products of a tile run on the tensor cores, the heads of a key/value head as the MMA's
    rows (groups of 1 to 16 heads).  Decoded tokens over long contexts, then short portions beside them."""
    _compare_attention(dtype, atol, heads, kv, key_dim, value_dim, window, bias, mix, gate, [1, 1, 1, 1], [700, 3, 1029, 40], with_batch=True)
    _compare_attention(dtype, atol, heads, kv, key_dim, value_dim, window, bias, mix, gate, [3, 1, 2, 1, 5], [10, 300, 77, 0, 31], with_batch=True)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_positioned_embedding_and_activation_kernels(dtype):
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(6)
    table, places, weight = torch.randn(50, 72, generator=g).to(dtype), torch.randn(30, 72, generator=g).to(dtype), 1 + 0.1 * torch.randn(72, generator=g)
    ids, positions = torch.tensor([3, 49, 0, 7], dtype=torch.int32), torch.tensor([0, 29, 11, 1], dtype=torch.int32)
    for place_table, norm in ((places, weight), (None, weight), (places, None)):
        want, got = torch.zeros(4, 72), torch.zeros(4, 72, device="cuda")
        plain_ops.embedding_positions(table, place_table, ids, positions, norm, 1e-5, want, 1.5)
        ops.embedding_positions(table.cuda(), _cuda(place_table), ids.cuda(), positions.cuda(), _cuda(norm), 1e-5, got, 1.5)
        assert torch.allclose(got.cpu(), want, atol=2e-6, rtol=1e-6)
    ops.embedding_positions(table.cuda(), places.cuda(), ids.cuda(), torch.tensor([0, 30, 1, 2], dtype=torch.int32).cuda(), None, 0.0, got)
    assert int(ops.error_flag(got.device).item()) & 4          # a position beyond the table is reported, not read
    ops.error_flag(got.device).zero_()
    x = (torch.randn(5, 37, generator=g) * 3).to(dtype)
    for kind in ops.ACTIVATIONS:
        want, got = torch.zeros_like(x), torch.zeros_like(x, device="cuda")
        plain_ops.activation(kind, x, want)
        ops.activation(kind, x.cuda(), got)
        assert torch.allclose(got.cpu().float(), want.float(), atol=1e-5 if dtype == torch.float32 else 0.07, rtol=1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 5, 16, 40])
@pytest.mark.parametrize("kind", ["relu_squared", "gelu_tanh", "silu"])
def test_product_with_activation_behind(rows, kind):
    """Up to 16 rows the activation is applied in the product's epilogue, beyond by a kernel of its own: the same numbers either way."""
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(rows)
    x, weight = torch.randn(rows, 72, generator=g).bfloat16(), (torch.randn(200, 72, generator=g) * 0.2).bfloat16()
    want = torch.zeros(rows, 200, dtype=torch.bfloat16)
    plain_ops.linear_activated(x, weight, want, kind)
    got = torch.zeros(rows, 200, dtype=torch.bfloat16, device="cuda")
    before = ops.launch_count
    ops.linear_activated(x.cuda(), weight.cuda(), got, kind)
    assert rows > 16 or ops.launch_count - before == 1
    assert torch.allclose(got.cpu().float(), want.float(), atol=2e-2, rtol=2e-2)
    residual, norm_weight = torch.randn(rows, 72, generator=g), 1 + 0.1 * torch.randn(72, generator=g)
    normed = torch.zeros(rows, 72, dtype=torch.bfloat16)
    plain_ops.add_rmsnorm(residual.clone(), None, norm_weight, 1e-5, normed)
    plain_ops.linear_activated(normed, weight, want, kind)
    lazy = ops.LazyNorm(residual.cuda(), norm_weight.cuda(), 1e-5, None, lambda: None)
    if rows <= 16:
        ops.linear_activated(lazy, weight.cuda(), got, kind)
        assert torch.allclose(got.cpu().float(), want.float(), atol=3e-2, rtol=3e-2)


# --- the engine on the GPU under every way of cutting the work -------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", list(CONFIGS))
def test_engine_matches_plain_under_every_schedule(cases, key, dtype):
    """Whole prompts, a tail decoded token by token, portions down to two tokens, and four live requests mixed in a pool that makes
    pages and state slots come round again (freed pages are poisoned with NaN)."""
    folder, requests, full, scale = cases[key]
    for name, (steps, pool) in _schedules(requests).items():
        runner = _runner(folder, dtype, max_tokens=pool)
        trace_tools.run_and_compare(runner, steps, full, atol=TOLERANCE[dtype] * scale)
        runner.cache.check()
        assert not runner.cache.records, name
        if name == "mixed":
            assert all(g.pool.reuses > 0 for g in runner.cache.page_groups)


def _sharpened(folder, name, edit):
    """A copy of a model folder with some tensors changed, so that one mechanism decides the logits."""
    target = folder.parent / f"{folder.name}_{name}"
    if not (target / "model.safetensors").exists():
        target.mkdir(exist_ok=True)
        (target / "config.json").write_text((folder / "config.json").read_text())
        config, tensors = load_plain(folder)
        edit(tensors)
        write_safetensors(target / "model.safetensors", tensors)
    return target


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tokens_hundreds_back_decide_through_the_state(folders, dtype):
    """Gates that hardly open keep what they took in for hundreds of steps: the last logits of a 600-token request then depend on
    its first tokens (by a hundred times the 32-bit tolerance), through every portion's hand-over of the state and through 150
    tokens decoded one by one."""
    def slow_gates(tensors):
        for name in tensors:
            if name.endswith(".z.b"):
                tensors[name] = torch.full_like(tensors[name], -7.0)

    folder = _sharpened(folders["recurrent_only"], "slow", slow_gates)
    config, tensors = load_plain(folder)
    requests = trace_tools.make_requests(config["vocab"], [600, 450], seed=8)
    full = {rid: plain_marutar.forward(config, tensors, tokens) for rid, tokens in requests.items()}
    other = [(t + 1) % config["vocab"] if i < 40 else t for i, t in enumerate(requests["r0"])]
    scale = max(float(v.abs().max()) for v in full.values())
    assert float((plain_marutar.forward(config, tensors, other)[-1] - full["r0"][-1]).abs().max()) > 50 * TOLERANCE["float32"] * scale   # the far tokens show
    for steps in (trace_tools.tail_decode(requests, tail=150), trace_tools.portions(requests), trace_tools.mixed(requests, seed=4, max_portion=90)[0]):
        trace_tools.run_and_compare(_runner(folder, dtype, max_tokens=2048, page_size=64), steps, full, atol=TOLERANCE[dtype] * scale)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_edges_decide(folders, dtype):
    """Queries and keys scaled up make single keys dominate a row: a key one place too many or too few at a window's edge (windows
    of 16 = one page, and none) then moves the logits far beyond the tolerance, in prompts and in decoded tokens."""
    def sharp(tensors):
        for name in tensors:
            if name.endswith(".mix.q") or name.endswith(".mix.k"):
                tensors[name] = (tensors[name].float() * 3.0).bfloat16()

    folder = _sharpened(folders["wide_heads"], "sharp", sharp)
    config, tensors = load_plain(folder)
    requests = trace_tools.make_requests(config["vocab"], [130, 48, 65, 33], seed=13)
    full = {rid: plain_marutar.forward(config, tensors, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    shifted = json.loads(json.dumps(config))
    shifted["layers"][2]["mixer"]["mask"]["size"] = 15
    moved = plain_marutar.forward(shifted, tensors, requests["r0"])
    assert float((moved - full["r0"]).abs().max()) > 3 * TOLERANCE[dtype] * scale           # one key less is seen in the logits, in bfloat16 too
    for steps in (trace_tools.tail_decode(requests, tail=40), trace_tools.portions(requests), trace_tools.mixed(requests, seed=6)[0]):
        trace_tools.run_and_compare(_runner(folder, dtype), steps, full, atol=TOLERANCE[dtype] * scale)


@pytest.mark.gpu
def test_rows_do_not_depend_on_the_batch(cases):
    """32-bit attention rows are bit-identical however the step is cut; the recurrence agrees to rounding."""
    folder, requests, full, scale = cases["mixed"]
    alone, together = _runner(folder, "float32"), _runner(folder, "float32")
    tokens = requests["r3"]
    whole = alone.step([StepEntry("x", tokens, [len(tokens) - 1])]).cpu()
    together.step([StepEntry("y", requests["r2"][:40], []), StepEntry("x", tokens[:77], [])])
    cut = together.step([StepEntry("x", tokens[77:], [len(tokens) - 78]), StepEntry("y", requests["r2"][40:41], [0])]).cpu()
    assert float((cut[0] - whole[0]).abs().max()) <= 1e-5 * scale


# --- generation through the engine's own entry point ------------------------------------------------------------------------------------------
def _plain_greedy(config, tensors, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(plain_marutar.forward(config, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(folders, graphs):
    """Prompts of unequal length through ``Engine.generate``: scheduler, portions under a small token budget, decode sessions
    (captured as graphs or not), state slots and windowed pages.  32-bit, so that the plain implementation's choice is the engine's."""
    from tinyllama_inference_engine_b200 import Engine, SamplingParams

    folder = folders["mixed"]
    config, tensors = load_plain(folder)
    rng = np.random.default_rng(31)
    prompts = [[int(t) for t in rng.integers(0, config["vocab"], size=n)] for n in (50, 3, 21, 34, 8)]
    engine = Engine(folder, EngineConfig(dtype="float32", page_size=16, max_cache_tokens=512, max_requests=3, max_batch_tokens=24, use_cuda_graphs=graphs))
    results = engine.generate(prompts, SamplingParams(max_tokens=20))
    for prompt, result in zip(prompts, results):
        assert result.generated_tokens == _plain_greedy(config, tensors, prompt, 20)
    again = engine.generate(prompts[:3], SamplingParams(max_tokens=20))       # slots and pages come round again; shapes repeat, so graphs replay
    assert [r.generated_tokens for r in again] == [r.generated_tokens for r in results[:3]]
    if graphs:
        assert any(s.graph is not None for s in engine._sessions.values())
    engine.runner.cache.check()


@pytest.mark.gpu
def test_generation_in_bfloat16_runs_and_repeats(folders):
    from tinyllama_inference_engine_b200 import generate

    rng = np.random.default_rng(2)
    prompts = [[int(t) for t in rng.integers(0, 77, size=n)] for n in (90, 12, 40)]
    first = generate(folders["wide_heads"], prompts, max_tokens=24, dtype="bfloat16", page_size=16, max_cache_tokens=1024, max_requests=4, max_batch_tokens=64)
    second = generate(folders["wide_heads"], prompts, max_tokens=24, dtype="bfloat16", page_size=16, max_cache_tokens=1024, max_requests=4, max_batch_tokens=64)
    assert first == second and all(len(tokens) == 24 for tokens in first)


@pytest.mark.gpu
def test_command_line_and_trace_program(folders, tmp_path, capsys):
    """The framework's command line generates, prints logits and builds a model from a config.json with seeded weights; `bin/trace_run`
    as a child process answers step by step and dumps every layer's output, which matches the plain implementation's trace."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    from tinyllama_inference_engine_b200.cli import main

    folder = folders["mixed"]
    config, tensors = load_plain(folder)
    prompt = [int(t) for t in np.random.default_rng(12).integers(0, config["vocab"], size=11)]
    text = ",".join(map(str, prompt))
    assert main(["generate", str(folder), text, "6", "--dtype", "float32", "--page-size", "16"]) == 0
    result = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert result["generated_tokens"] == _plain_greedy(config, tensors, prompt, 6) and result["prompt_tokens"] == 11
    assert main(["logits", str(folder), text, "--dtype", "float32"]) == 0
    logits = torch.tensor(json.loads(capsys.readouterr().out)["logits"])
    assert torch.allclose(logits, plain_marutar.forward(config, tensors, prompt)[-1], atol=2e-5)
    assert main(["generate", "-", text, "6", "--dtype", "float32", "--random-config", str(folder / "config.json"), "--weights-seed", str(CONFIGS["mixed"][1])]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["generated_tokens"] == result["generated_tokens"]

    program = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    out = tmp_path / "out"
    tokens = prompt + prompt[::-1]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:13], "want": [12]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[13:], "want": []}, {"id": "b", "tokens": prompt[:2], "want": [1]}], "end": ["a", "b"]}]
    child = subprocess.run([sys.executable, str(program), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "128", "--dump-layers"],
                           input="".join(json.dumps(step) + "\n" for step in steps), capture_output=True, text=True, env=dict(os.environ, PYTHONUNBUFFERED="1"))
    assert child.returncode == 0 and [line for line in child.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1"]
    trace = []
    full = plain_marutar.forward(config, tensors, tokens, trace)
    got = np.fromfile(out / "0.f32", dtype="<f4")
    assert float(np.abs(got - full[12].numpy()).max()) <= 3e-5 * float(full.abs().max())
    layers = np.fromfile(out / "0.layers.f32", dtype="<f4").reshape(len(config["layers"]), 13, config["width"])
    for index, want in enumerate(trace):
        assert float(np.abs(layers[index] - want[:13].numpy()).max()) <= 3e-5 * float(want.abs().max()), index
    other = plain_marutar.forward(config, tensors, prompt[:2])
    assert float(np.abs(np.fromfile(out / "1.f32", dtype="<f4") - other[1].numpy()).max()) <= 3e-5 * float(other.abs().max())

